"""minGRU: a gated recurrence whose gates read only the current token, over a float32 state of ``width`` elements per
request.

    z_t = sigmoid(W_z h_t + b_z)         u_t = W_x h_t + b_x         c_t = u_t + 1/2 (u_t >= 0), sigmoid(u_t) (u_t < 0)
    S_t = (1 - z_t) S_(t-1) + z_t c_t    element by element, zero before the request's first token
    out = W_o (S_t * silu(W_g h_t))

Because neither gate reads S, the recurrence is linear in S.  The state, the gates and the candidate are float32 in
either mode of the engine: the projections' float32 accumulators go to the recurrence unrounded.  The state is a
``StateNeed``: the engine gives the mixer a [slots, width] tensor and the step's slot ids, and clears a slot when its
request's first token arrives."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..registry import register_part
from .base import SplitMixer, WeightSpec, MATRIX, VECTOR, StateNeed, LayerContext


@register_part("mixer", "min_gru")
class MinGRU(SplitMixer):
    def __init__(self, hidden_size: int, width: int, names: Optional[Dict[str, str]] = None, prefix: str = ""):
        super().__init__(prefix)
        self.hidden_size, self.width = int(hidden_size), int(width)
        if self.width <= 0:
            raise ValueError("width must be positive")
        self.names = {"z": "z", "z_bias": "z.b", "x": "x", "x_bias": "x.b", "gate": "g", "o": "o"}
        self.names.update(names or {})
        self.w_in = self.w_o = self.bz = self.bx = None

    def cache_need(self):
        return StateNeed((self.width,), "float32")

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n = self.names
        return {n["z"]: WeightSpec((self.width, self.hidden_size), MATRIX),
                n["z_bias"]: WeightSpec((self.width,), VECTOR, init="normal", init_scale=0.5),
                n["x"]: WeightSpec((self.width, self.hidden_size), MATRIX),
                n["x_bias"]: WeightSpec((self.width,), VECTOR, init="normal", init_scale=0.5),
                n["gate"]: WeightSpec((self.width, self.hidden_size), MATRIX),
                n["o"]: WeightSpec((self.hidden_size, self.width), MATRIX)}

    def load(self, tensors, ops, act_dtype) -> None:
        n = self.names
        rows = [tensors[n["z"]], tensors[n["x"]], tensors[n["gate"]]]
        dt = rows[0].dtype if all(r.dtype == rows[0].dtype for r in rows) else torch.float32
        self.w_in = torch.cat([r.to(dt) for r in rows], dim=0).contiguous()      # rows [z | x | g]
        self.w_o = tensors[n["o"]]
        self.bz, self.bx = tensors[n["z_bias"]].contiguous(), tensors[n["x_bias"]].contiguous()

    def input_rows(self):
        return self.w_in

    def mixed_width(self) -> int:
        return self.width

    def output_cols(self):
        return self.w_o

    def mix(self, proj, col, ctx: LayerContext, mixed, mixed_col, out_scale, last_reader) -> None:
        if ctx.state is None:
            raise ValueError("min_gru needs a state tensor (StateNeed)")
        ctx.ops.min_gru(proj, col, col + self.width, col + 2 * self.width, self.bz, self.bx, ctx.state, ctx.batch, mixed,
                        self.width, out_off=mixed_col, out_scale=out_scale, last_reader=last_reader)
