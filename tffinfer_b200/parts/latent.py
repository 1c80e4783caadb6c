"""Latent attention: queries, keys and values are made from small vectors per token, and only those are cached.

For a token with mixer input h at position p (all norms x * rsqrt(mean(x^2) + eps) * w with a plain weight):

    cq = norm(W_dq h)                       q = W_uq cq, per head [dim unrotated | rot_dim rotated]
    [c' | r'] = W_dkv h                     c = norm(c') (kv_rank elements), r = rot(r', p) (rot_dim, one for all heads)
    k_h = [W_uk,h c | r]                    v_h = W_uv,h c
    out = W_o concat_h softmax_j<=p( (q_h . k_h,j) * scale ) v_h,j

The rotation is the layer's position encoding (``frequencies()``: interleaved pairs).  The cache need is one plane
with a slot of kv_rank + rot_dim elements per token, [c | r].  A layer built with ``shared_kv`` has no W_dkv and reads
the slots another layer wrote (its schedule entry names that layer's entry in ``cache_of``); it has its own W_uk,
W_uv and queries.  Per-head keys and values of cached tokens are never materialised; a step of whole prompts makes
those of its own tokens (kernels/library.py ``latent_attend``)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..registry import register_part
from .base import Mixer, WeightSpec, MATRIX, VECTOR, KVNeed, LayerContext


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, v_head_dim: int, q_rank: int,
                 kv_rank: int, eps: float, softmax_scale: Optional[float] = None, shared_kv: bool = False,
                 names: Optional[Dict[str, str]] = None, prefix: str = ""):
        super().__init__(prefix)
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.head_dim, self.rot_dim, self.v_head_dim = int(head_dim), int(rot_dim), int(v_head_dim)
        self.q_rank, self.kv_rank, self.eps = int(q_rank), int(kv_rank), float(eps)
        self.scale = float(softmax_scale) if softmax_scale is not None else float(self.head_dim + self.rot_dim) ** -0.5
        self.shared_kv = bool(shared_kv)
        if min(self.num_heads, self.head_dim, self.v_head_dim, self.q_rank, self.kv_rank) <= 0 or self.rot_dim < 0:
            raise ValueError("latent attention: sizes must be positive (rot_dim may be 0)")
        self.names = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk",
                      "uv": "uv", "o": "o"}
        self.names.update(names or {})
        self.w_down = self.w_uq = self.w_uk_t = self.w_uk = self.w_uv = self.w_o = self.q_norm_w = self.kv_norm_w = None

    def cache_need(self):
        return KVNeed(1, self.kv_rank + self.rot_dim, 0, planes=1)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n, H = self.names, self.num_heads
        s = {n["dq"]: WeightSpec((self.q_rank, self.hidden_size), MATRIX),
             n["dq_norm"]: WeightSpec((self.q_rank,), VECTOR, init="one_plus_normal"),
             n["uq"]: WeightSpec((H * (self.head_dim + self.rot_dim), self.q_rank), MATRIX),
             n["uk"]: WeightSpec((H * self.head_dim, self.kv_rank), MATRIX),
             n["uv"]: WeightSpec((H * self.v_head_dim, self.kv_rank), MATRIX),
             n["o"]: WeightSpec((self.hidden_size, H * self.v_head_dim), MATRIX)}
        if not self.shared_kv:
            s[n["dkv"]] = WeightSpec((self.kv_rank + self.rot_dim, self.hidden_size), MATRIX)
            s[n["dkv_norm"]] = WeightSpec((self.kv_rank,), VECTOR, init="one_plus_normal")
        return s

    def load(self, tensors, ops, act_dtype) -> None:
        n, H = self.names, self.num_heads
        rows = [tensors[n["dq"]]] + ([] if self.shared_kv else [tensors[n["dkv"]]])
        dt = rows[0].dtype if all(r.dtype == rows[0].dtype for r in rows) else torch.float32
        w = torch.cat([r.to(dt) for r in rows], dim=0)
        pad = (-w.shape[0]) % 8               # the product's output rows are stored 16 bytes at a time
        if pad:
            w = torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=dt, device=w.device)], dim=0)
        self.w_down = w.contiguous()
        self.w_uq = tensors[n["uq"]]
        # [heads, dim, kv_rank] -> [heads, kv_rank, dim]: the query's unrotated part goes through W_uk^T
        self.w_uk_t = tensors[n["uk"]].view(H, self.head_dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uk = tensors[n["uk"]]          # as stored, for steps of whole prompts (per-head keys of the step's tokens)
        self.w_uv = tensors[n["uv"]]
        self.w_o = tensors[n["o"]]
        self.q_norm_w = tensors[n["dq_norm"]]
        self.kv_norm_w = None if self.shared_kv else tensors[n["dkv_norm"]]

    def forward(self, h, ctx: LayerContext, residual):
        ops = ctx.ops
        T = h.shape[0]
        if self.shared_kv == ctx.write_cache:
            raise ValueError("a latent attention with shared_kv reads another layer's cache (cache_of), and only then")
        freq = ctx.position.frequencies() if (ctx.position is not None and self.rot_dim) else None
        if freq is not None and freq[1] > self.rot_dim:
            raise ValueError(f"the rotation covers {freq[1]} dimensions, the rotated key part has {self.rot_dim}")
        mixed = torch.empty((T, self.num_heads * self.v_head_dim), dtype=h.dtype, device=h.device)
        ops.latent_attend(h, self.w_down, self.q_norm_w, self.kv_norm_w, self.eps, self.w_uq, self.w_uk_t, self.w_uv,
                          freq, ctx.batch, ctx.block_table, ctx.kv_cache, ctx.kv_layer, ctx.page_size, mixed,
                          self.num_heads, self.head_dim, self.rot_dim, self.v_head_dim, self.q_rank, self.kv_rank,
                          self.scale, ctx.write_cache, w_uk=self.w_uk, shared=ctx.shared)
        if residual is None:
            out = ops.sublayer_output(T, self.hidden_size, h.device, h.dtype)
            ops.gemm(mixed, self.w_o, out)
            return out
        ops.gemm(mixed, self.w_o, residual, residual=residual)
        return residual
