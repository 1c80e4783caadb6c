"""Dense gated feed-forward: ``down( silu(gate(h)) * up(h) )`` without biases, with
``silu(g) = g / (1 + exp(-g))`` as the reference computes it
(src/kernel/cuda/unary.cu:10-27; built by ModelCreatorBase::build_ffn,
src/core/model/base/ModelCreatorBase.cpp:51-94), followed by the residual add
(src/core/model/qwen3/QWen3Creator.cpp:148-151).  ``activation`` chooses the gate's function: "silu", or
"gelu_tanh", ``0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3)))``; ``names`` the tensor names of "gate", "up" and
"down" relative to the prefix."""
from __future__ import annotations

from typing import Dict

import torch

from ..registry import register_part
from .base import FeedForward, WeightSpec, MATRIX


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    takes_deferred_norm = True        # the input only feeds the gate/up product

    ACTIVATIONS = ("silu", "gelu_tanh")

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu", names=None,
                 prefix: str = ""):
        super().__init__(prefix)
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        if activation not in self.ACTIVATIONS:
            raise ValueError(f"activation must be one of {self.ACTIVATIONS}, got '{activation}'")
        self.activation = activation
        self.names = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}
        self.names.update(names or {})
        self.w_gate_up = self.w_down = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n = self.names
        return {
            n["gate"]: WeightSpec((self.intermediate_size, self.hidden_size), MATRIX),
            n["up"]: WeightSpec((self.intermediate_size, self.hidden_size), MATRIX),
            n["down"]: WeightSpec((self.hidden_size, self.intermediate_size), MATRIX),
        }

    def load(self, tensors, ops, act_dtype) -> None:
        g, u = tensors[self.names["gate"]], tensors[self.names["up"]]
        dt = g.dtype if g.dtype == u.dtype else torch.float32
        # one projection instead of two; the kernel library chooses how gate and up rows are laid out
        self.w_gate_up = ops.merge_gate_up(g.to(dt), u.to(dt))
        self.w_down = tensors[self.names["down"]]

    def forward(self, h, ctx, residual):
        if residual is None:              # f(h) alone, for arrangements that do more with it than add it
            out = ctx.ops.sublayer_output(h.shape[0], self.hidden_size, h.device, h.dtype)
            ctx.ops.gated_mlp(h, self.w_gate_up, self.w_down, None, self.intermediate_size,
                              activation=self.activation, out=out)
            return out
        if self.activation == "silu":
            ctx.ops.gated_mlp(h, self.w_gate_up, self.w_down, residual, self.intermediate_size)
        else:
            ctx.ops.gated_mlp(h, self.w_gate_up, self.w_down, residual, self.intermediate_size,
                              activation=self.activation)
        return residual
