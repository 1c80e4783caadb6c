"""Routed feed-forward (mixture of experts): ``num_experts`` small gated feed-forwards without biases, of which every
token uses ``top``.

    s = sigmoid(W_r h)                                  router, computed in float32
    chosen = the ``top`` experts of largest s (the lower index wins a tie)
    w_e = s_e, or s_e / sum over the chosen when ``renormalize``
    weight_on "input":   out = sum_e down_e( act(gate_e(w_e h)) * up_e(w_e h) )
    weight_on "output":  out = sum_e w_e down_e( act(gate_e(h)) * up_e(h) )

The experts' tensors are ``<prefix>.e<i>.{gate,up,down}`` and the router ``<prefix>.router`` unless ``names`` says
otherwise; they are stacked into [E, 2 ff, hidden] (gate and up) and [E, hidden, ff] when loaded, and the tokens of a step are sorted
by expert on the device (kernels/library.py ``routed_mlp``): nothing of it waits for the host."""
from __future__ import annotations

from typing import Dict

import torch

from ..registry import register_part
from .base import FeedForward, WeightSpec, MATRIX


@register_part("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    ACTIVATIONS = ("silu", "gelu_tanh")

    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, top: int, activation: str = "silu",
                 renormalize: bool = False, weight_on: str = "output", names=None, prefix: str = ""):
        super().__init__(prefix)
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.num_experts, self.top = int(num_experts), int(top)
        if not 0 < self.top <= self.num_experts:
            raise ValueError(f"top ({self.top}) must lie in 1 .. num_experts ({self.num_experts})")
        if activation not in self.ACTIVATIONS:
            raise ValueError(f"activation must be one of {self.ACTIVATIONS}, got '{activation}'")
        if weight_on not in ("input", "output"):
            raise ValueError(f"weight_on must be 'input' or 'output', got '{weight_on}'")
        self.activation, self.renormalize, self.weight_on = activation, bool(renormalize), weight_on
        self.names = {"router": "router", "expert": "e{}", "gate": "gate", "up": "up", "down": "down"}
        self.names.update(names or {})
        self.w_router = self.w_gate_up = self.w_down = None
        self.gate_up_layout = "blocked"

    def _expert(self, e: int, which: str) -> str:
        return f"{self.names['expert'].format(e)}.{self.names[which]}"

    def weight_specs(self) -> Dict[str, WeightSpec]:
        s = {self.names["router"]: WeightSpec((self.num_experts, self.hidden_size), MATRIX)}
        for e in range(self.num_experts):
            s[self._expert(e, "gate")] = WeightSpec((self.intermediate_size, self.hidden_size), MATRIX)
            s[self._expert(e, "up")] = WeightSpec((self.intermediate_size, self.hidden_size), MATRIX)
            s[self._expert(e, "down")] = WeightSpec((self.hidden_size, self.intermediate_size), MATRIX)
        return s

    def load(self, tensors, ops, act_dtype) -> None:
        def all_of(*which):
            ts = [[tensors[self._expert(e, w)] for e in range(self.num_experts)] for w in which]
            same = all(t.dtype == ts[0][0].dtype for l in ts for t in l)
            return [[t if same else t.to(torch.float32) for t in l] for l in ts]
        self.w_router = tensors[self.names["router"]]
        gates, ups = all_of("gate", "up")
        # one tensor for gate and up of all experts; the kernel library chooses how their rows are laid out
        self.w_gate_up, self.gate_up_layout = ops.stack_gate_up(gates, ups)
        self.w_down = torch.stack(all_of("down")[0], dim=0).contiguous()

    def forward(self, h, ctx, residual):
        out = None
        if residual is None:
            out = torch.empty((h.shape[0], self.hidden_size), dtype=torch.float32, device=h.device)
        ctx.ops.routed_mlp(h, self.w_router, self.w_gate_up, self.gate_up_layout, self.w_down, residual, self.top, self.renormalize,
                           self.weight_on, self.activation, out=out)
        return residual if residual is not None else out
