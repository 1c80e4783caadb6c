"""Retention: linear attention with a fixed decay per head, no softmax and no denominator, over a state of fixed
size per request.

For head h with decay g_h, queries and keys of ``head_dim`` and values of ``v_head_dim`` elements:

    q_t, k_t   rotated by the layer's position encoding; k_t then multiplied by head_dim^-1/2
    S_t = g_h S_(t-1) + k_t v_t^T              S [head_dim, v_head_dim], zero before the request's first token
    o_t = S_t^T q_t
    out = concat_h( o_t / rms(o_t) ) * silu(W_g h_t),   rms over the head's v_head_dim elements with ``eps``, no weight

followed by the output projection.  The state, and everything that enters it behind the projections, is float32
in either mode of the engine: the projection's float32 accumulators go to the rotation and the recurrence
unrounded.  The state is a ``StateNeed``: the engine gives the mixer a [slots, heads, head_dim, v_head_dim] tensor,
the step's slot ids, and clears a slot when its request's first token arrives."""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from ..registry import register_part
from .base import Mixer, WeightSpec, MATRIX, StateNeed, LayerContext


@register_part("mixer", "retention")
class Retention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int, decay: Sequence[float],
                 eps: float, names: Optional[Dict[str, str]] = None, prefix: str = ""):
        super().__init__(prefix)
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.head_dim, self.v_head_dim = int(head_dim), int(v_head_dim)
        self.decay = tuple(float(x) for x in decay)
        if len(self.decay) != self.num_heads:
            raise ValueError(f"decay lists {len(self.decay)} values for {self.num_heads} heads")
        self.eps = float(eps)
        self.names = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "gate": "g_proj.weight",
                      "o": "o_proj.weight"}
        self.names.update(names or {})
        self.qk_width = self.num_heads * self.head_dim
        self.v_width = self.num_heads * self.v_head_dim
        self.w_in = self.w_o = self.decay_dev = None

    def cache_need(self):
        return StateNeed((self.num_heads, self.head_dim, self.v_head_dim), "float32")

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n = self.names
        return {n["q"]: WeightSpec((self.qk_width, self.hidden_size), MATRIX),
                n["k"]: WeightSpec((self.qk_width, self.hidden_size), MATRIX),
                n["v"]: WeightSpec((self.v_width, self.hidden_size), MATRIX),
                n["gate"]: WeightSpec((self.v_width, self.hidden_size), MATRIX),
                n["o"]: WeightSpec((self.hidden_size, self.v_width), MATRIX)}

    def load(self, tensors, ops, act_dtype) -> None:
        n = self.names
        rows = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["gate"]]]
        dt = rows[0].dtype if all(r.dtype == rows[0].dtype for r in rows) else torch.float32
        w = torch.cat([r.to(dt) for r in rows], dim=0)
        pad = (-w.shape[0]) % 8
        if pad:
            w = torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=dt, device=w.device)], dim=0)
        self.w_in = w.contiguous()
        self.w_o = tensors[n["o"]]
        self.decay_dev = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(self.w_o.device)

    def forward(self, h, ctx: LayerContext, residual):
        ops = ctx.ops
        T = h.shape[0]
        freq = ctx.position.frequencies() if ctx.position is not None else None
        mixed = torch.empty((T, self.v_width), dtype=h.dtype, device=h.device)
        ops.retain(h, self.w_in, freq, ctx.batch, ctx.state, self.decay_dev, mixed, self.num_heads, self.head_dim,
                   self.v_head_dim, float(self.head_dim) ** -0.5, self.eps)
        if residual is None:
            out = ops.sublayer_output(T, self.hidden_size, h.device, h.dtype)
            ops.gemm(mixed, self.w_o, out)
            return out
        ops.gemm(mixed, self.w_o, residual, residual=residual)
        return residual
