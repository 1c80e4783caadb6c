"""Several mixers side by side: all read the same input rows, and the result is the sum of their outputs, each times
a constant:  out = sum_b scale_b * mixer_b(h).

The branches are :class:`SplitMixer` parts (input projection -> token mixing -> output projection); here their input
projections are ONE product ([rows of branch 0 | rows of branch 1 | ...]), every branch mixes its columns of the
float32 accumulators into its columns of one activation (times its constant), and ONE output product over the
concatenated activation adds the sum to the residual.  A branch's tensors are named ``<prefix>.<branch name>.<its
own names>``.  At most one branch may keep pages and at most one a state: the layer's cache need is the pair."""
from __future__ import annotations

from typing import Any, Dict, List

import torch

from ..registry import register_part, get_part
from .base import Mixer, SplitMixer, WeightSpec, KVNeed, StateNeed, LayerContext


@register_part("mixer", "parallel")
class ParallelMixers(Mixer):
    def __init__(self, hidden_size: int, branches: List[Dict[str, Any]], prefix: str = ""):
        """branches: [{"name": tensor-name part, "kind": registry kind of a mixer, "params": {...}, "scale": constant}]"""
        super().__init__(prefix)
        self.hidden_size = int(hidden_size)
        if not branches:
            raise ValueError("parallel: at least one branch")
        self.branch_names, self.scales, self.branches = [], [], []
        for b in branches:
            part = get_part("mixer", b["kind"])(prefix="", **b.get("params", {}))
            if not isinstance(part, SplitMixer):
                raise ValueError(f"parallel: mixer '{b['kind']}' does not let its projections be shared (SplitMixer)")
            self.branch_names.append(str(b["name"]))
            self.scales.append(float(b.get("scale", 1.0)))
            self.branches.append(part)
        if len(set(self.branch_names)) != len(self.branch_names):
            raise ValueError("parallel: branch names must differ")
        needs = [m.cache_need() for m in self.branches]
        if sum(isinstance(n, KVNeed) for n in needs) > 1 or sum(isinstance(n, StateNeed) for n in needs) > 1:
            raise ValueError("parallel: at most one branch with pages and one with a state")
        self._needs = tuple(n for n in needs if n is not None)
        self.w_in = self.w_out = None

    def cache_need(self):
        if not self._needs:
            return None
        return self._needs[0] if len(self._needs) == 1 else self._needs

    def weight_specs(self) -> Dict[str, WeightSpec]:
        out = {}
        for name, m in zip(self.branch_names, self.branches):
            for rel, spec in m.weight_specs().items():
                out[f"{name}.{rel}"] = spec
        return out

    def load(self, tensors, ops, act_dtype) -> None:
        for name, m in zip(self.branch_names, self.branches):
            pre = name + "."
            m.load({k[len(pre):]: v for k, v in tensors.items() if k.startswith(pre)}, ops, act_dtype)
        ins = [m.input_rows() for m in self.branches]
        outs = [m.output_cols() for m in self.branches]
        dt_in = ins[0].dtype if all(w.dtype == ins[0].dtype for w in ins) else torch.float32
        dt_out = outs[0].dtype if all(w.dtype == outs[0].dtype for w in outs) else torch.float32
        self.in_cols, self.mixed_cols, c, mc = [], [], 0, 0
        for m, w in zip(self.branches, ins):
            self.in_cols.append(c)
            self.mixed_cols.append(mc)
            c += w.shape[0]
            mc += m.mixed_width()
        self.mixed_total = mc
        self.w_in = SplitMixer.padded_rows(torch.cat([w.to(dt_in) for w in ins], dim=0))
        self.w_out = torch.cat([w.to(dt_out) for w in outs], dim=1).contiguous()

    def forward(self, h, ctx: LayerContext, residual):
        ops = ctx.ops
        T = h.shape[0]
        proj = ops.projection_buffer(T, self.w_in.shape[0], h.device, h.dtype)
        ops.gemm(h, self.w_in, proj)
        mixed = torch.empty((T, self.mixed_total), dtype=h.dtype, device=h.device)
        last = len(self.branches) - 1
        for i, m in enumerate(self.branches):
            m.mix(proj, self.in_cols[i], ctx, mixed, self.mixed_cols[i], self.scales[i], i == last)
        if residual is None:
            out = ops.sublayer_output(T, self.hidden_size, h.device, h.dtype)
            ops.gemm(mixed, self.w_out, out)
            return out
        ops.gemm(mixed, self.w_out, residual, residual=residual)
        return residual
