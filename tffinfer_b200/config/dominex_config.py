"""Typed configuration of the Dominex design: a decoder-only model whose config.json lists its layers one by one.
A layer's mixer is ``latent_attention`` (queries, keys and values made from small cached vectors) or ``parallel``
(a chunked attention with distance-biased scores beside a minGRU recurrence); its feed-forward is a mixture of
experts, or absent.

    {"architecture": "Dominex", "vocab": V, "width": W, "embedding": {"scale": s}, "norm": {"eps": e},
     "logit_softcap": c,
     "layers": [{"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale",
                           "rot": {"base", "dims"}, "kv_from": j (optional)},
                 "mlp": {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}} | null},
                {"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"}},
                           "right": {"width"}, "left_scale", "right_scale"},
                 "mlp": ...}, ...]}

Every size and constant of a checkpoint comes from there.  Optional keys: ``embedding.scale`` (absent: 1),
``logit_softcap`` (absent or 0: none), ``kv_heads`` (absent: heads), ``mask`` (absent: all earlier keys), ``kv_from``,
``left_scale`` / ``right_scale`` (absent: 1), ``rot.dims`` (absent: rot_dim), ``max_position`` (absent:
MAX_POSITION_DEFAULT; the design itself has no limit, the engine's block tables need one)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .model_config import ModelConfig, ConfigError
from .tipezen_config import _need, _int, _float, MAX_POSITION_DEFAULT


@dataclass(frozen=True)
class DominexExperts:
    ff: int
    experts: int
    top: int


@dataclass(frozen=True)
class DominexLayer:
    type: str                          # "latent_attention" | "parallel"
    # latent_attention
    heads: int = 0
    dim: int = 0
    rot_dim: int = 0
    vdim: int = 0
    q_rank: int = 0
    kv_rank: int = 0
    scale: float = 0.0
    rot_base: float = 0.0
    rot_dims: int = 0
    kv_from: Optional[int] = None      # the layer whose cached vectors this one reads
    # parallel: the attention on the left, the recurrence on the right
    left_heads: int = 0
    left_kv_heads: int = 0
    left_dim: int = 0
    left_vdim: int = 0
    left_scale_qk: float = 0.0         # multiplier of q . k
    left_chunk: int = 0                # 0 = all earlier keys
    right_width: int = 0
    left_scale: float = 1.0            # multipliers of the two outputs
    right_scale: float = 1.0
    mlp: Optional[DominexExperts] = None


@dataclass(frozen=True)
class DominexConfig(ModelConfig):
    vocab_size: int = 0
    hidden_size: int = 0
    embed_scale: float = 1.0
    norm_eps: float = 0.0
    logit_softcap: float = 0.0
    layers: Tuple[DominexLayer, ...] = ()
    max_position: int = MAX_POSITION_DEFAULT

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    @staticmethod
    def from_json_dict(d: Dict[str, Any]) -> "DominexConfig":
        from .model_config import architecture_name
        raw = _need(d, "layers", "the top level")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, l in enumerate(raw):
            where = f"layers[{i}]"
            kind = _need(l, "type", where)
            m = _need(l, "mixer", where)
            mw = where + ".mixer"
            mlp = l.get("mlp")
            ex = None
            if mlp is not None:
                if mlp.get("kind", "moe") != "moe":
                    raise ConfigError(f"config.json: {where}.mlp.kind '{mlp.get('kind')}' is not supported (moe only)")
                ex = DominexExperts(ff=_int(_need(mlp, "expert", where + ".mlp"), "ff", where + ".mlp.expert"),
                                    experts=_int(_need(mlp, "router", where + ".mlp"), "experts", where + ".mlp.router"),
                                    top=_int(mlp["router"], "top", where + ".mlp.router"))
                if ex.ff <= 0 or not 0 < ex.top <= ex.experts:
                    raise ConfigError(f"config.json: {where}.mlp: ff must be positive and 1 <= top <= experts")
            if kind == "latent_attention":
                rot = _need(m, "rot", mw)
                rot_dim = _int(m, "rot_dim", mw)
                layer = DominexLayer(
                    type=kind, heads=_int(m, "heads", mw), dim=_int(m, "dim", mw), rot_dim=rot_dim, vdim=_int(m, "vdim", mw),
                    q_rank=_int(m, "q_rank", mw), kv_rank=_int(m, "kv_rank", mw), scale=_float(m, "scale", mw),
                    rot_base=_float(rot, "base", mw + ".rot"), rot_dims=_int(rot, "dims", mw + ".rot", rot_dim),
                    kv_from=_int(m, "kv_from", mw) if m.get("kv_from") is not None else None, mlp=ex)
                if min(layer.heads, layer.dim, layer.rot_dim, layer.vdim, layer.q_rank, layer.kv_rank) <= 0:
                    raise ConfigError(f"config.json: {mw}: heads, dim, rot_dim, vdim, q_rank and kv_rank must be positive")
                if layer.rot_dims <= 0 or layer.rot_dims % 2 or layer.rot_dims > rot_dim or not layer.rot_base > 0:
                    raise ConfigError(f"config.json: {mw}.rot: 'dims' must be even, positive and at most rot_dim, 'base' positive")
                if layer.kv_from is not None:
                    j = layer.kv_from
                    src = layers[j] if 0 <= j < i else None
                    if src is None or src.type != kind or src.kv_from is not None:
                        raise ConfigError(f"config.json: {mw}.kv_from must name an earlier latent_attention layer that "
                                          f"keeps a cache of its own, got {j}")
                    if (src.kv_rank, src.rot_dim, src.rot_base, src.rot_dims) != (layer.kv_rank, layer.rot_dim,
                                                                                 layer.rot_base, layer.rot_dims):
                        raise ConfigError(f"config.json: {mw}: kv_rank, rot_dim and rot must equal those of layer {j}")
            elif kind == "parallel":
                L, R = _need(m, "left", mw), _need(m, "right", mw)
                lw = mw + ".left"
                heads = _int(L, "heads", lw)
                kv = _int(L, "kv_heads", lw, heads)
                mask = L.get("mask")
                layer = DominexLayer(
                    type=kind, left_heads=heads, left_kv_heads=kv, left_dim=_int(L, "dim", lw), left_vdim=_int(L, "vdim", lw),
                    left_scale_qk=_float(L, "scale", lw), left_chunk=_int(mask, "size", lw + ".mask") if mask is not None else 0,
                    right_width=_int(R, "width", mw + ".right"), left_scale=_float(m, "left_scale", mw, 1.0),
                    right_scale=_float(m, "right_scale", mw, 1.0), mlp=ex)
                if kv <= 0 or heads <= 0 or heads % kv:
                    raise ConfigError(f"config.json: {lw}: heads ({heads}) must be a multiple of kv_heads ({kv})")
                if min(layer.left_dim, layer.left_vdim, layer.right_width) <= 0 or layer.left_chunk < 0:
                    raise ConfigError(f"config.json: {mw}: dim, vdim and width must be positive")
            else:
                raise ConfigError(f"config.json: {where}.type '{kind}' is not a mixer of this design "
                                  f"(latent_attention, parallel)")
            layers.append(layer)
        emb = d.get("embedding") or {}
        cfg = DominexConfig(
            architecture=architecture_name(d), vocab_size=_int(d, "vocab", "the top level"),
            hidden_size=_int(d, "width", "the top level"), embed_scale=_float(emb, "scale", "embedding", 1.0),
            norm_eps=_float(_need(d, "norm", "the top level"), "eps", "norm"),
            logit_softcap=_float(d, "logit_softcap", "the top level", 0.0), layers=tuple(layers),
            max_position=_int(d, "max_position", "the top level", MAX_POSITION_DEFAULT))
        if cfg.vocab_size <= 0 or cfg.hidden_size <= 0 or not cfg.norm_eps > 0 or cfg.logit_softcap < 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive, norm.eps > 0, logit_softcap >= 0")
        return cfg

    def to_json_dict(self) -> Dict[str, Any]:
        out = []
        for l in self.layers:
            if l.type == "latent_attention":
                m: Dict[str, Any] = {"heads": l.heads, "dim": l.dim, "rot_dim": l.rot_dim, "vdim": l.vdim,
                                     "q_rank": l.q_rank, "kv_rank": l.kv_rank, "scale": l.scale,
                                     "rot": {"base": l.rot_base, "dims": l.rot_dims}}
                if l.kv_from is not None:
                    m["kv_from"] = l.kv_from
            else:
                left: Dict[str, Any] = {"heads": l.left_heads, "kv_heads": l.left_kv_heads, "dim": l.left_dim,
                                        "vdim": l.left_vdim, "scale": l.left_scale_qk}
                if l.left_chunk > 0:
                    left["mask"] = {"size": l.left_chunk}
                m = {"left": left, "right": {"width": l.right_width}, "left_scale": l.left_scale,
                     "right_scale": l.right_scale}
            mlp = None
            if l.mlp is not None:
                mlp = {"kind": "moe", "expert": {"ff": l.mlp.ff}, "router": {"experts": l.mlp.experts, "top": l.mlp.top}}
            out.append({"type": l.type, "mixer": m, "mlp": mlp})
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "embedding": {"scale": self.embed_scale}, "norm": {"eps": self.norm_eps},
             "logit_softcap": self.logit_softcap, "layers": out}
        if self.max_position != MAX_POSITION_DEFAULT:
            d["max_position"] = self.max_position
        return d
