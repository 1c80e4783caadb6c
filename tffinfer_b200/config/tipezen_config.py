"""Typed configuration of the Tipezen design: a decoder-only model whose config.json lists its layers one by
one, each with the kind of its mixer ('attention' or 'retention'), the mixer's sizes and constants, and its
feed-forward (or none).

    {"architecture": "Tipezen", "vocab": V, "width": W, "streams": S, "norm": {"eps": e},
     "layers": [{"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap",
                                                "mask": {"size"}, "v_mix", "rot": {"base", "dims",
                                                "scaling": {"factor", "original", "fast", "slow"}}},
                 "mlp": {"kind": "dense", "ff": F} | null},
                {"type": "retention", "mixer": {"heads", "dim", "vdim", "decay": [...], "rot": {"base", "dims"}},
                 "mlp": ...}, ...]}

Every size and constant of a checkpoint comes from there.  Optional keys: ``streams`` (absent or 0: one plain
residual), ``rot`` and ``rot.scaling`` (absent: no rotation / plain frequencies), ``mask`` (absent: all earlier
keys), ``softcap`` (absent: none), ``scale`` (absent: dim^-1/2), ``v_mix`` (absent: false), ``max_position``
(absent: MAX_POSITION_DEFAULT; the design itself has no limit, the engine's block tables need one).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .model_config import ModelConfig, ConfigError

MAX_POSITION_DEFAULT = 1 << 17


def _need(d: Dict[str, Any], key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key '{key}' is missing in {where}")
    return d[key]


def _int(d, key, where, default=None) -> int:
    v = d.get(key) if isinstance(d, dict) else None
    if v is None:
        if default is None:
            raise ConfigError(f"config.json: required key '{key}' is missing in {where}")
        return default
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: key '{key}' in {where} has value {v!r}, expected int")
    return int(v)


def _float(d, key, where, default=None) -> float:
    v = d.get(key) if isinstance(d, dict) else None
    if v is None:
        if default is None:
            raise ConfigError(f"config.json: required key '{key}' is missing in {where}")
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: key '{key}' in {where} has value {v!r}, expected a number")
    return float(v)


@dataclass(frozen=True)
class RotaryConfig:
    """A rotation of the first ``dims`` dimensions of a head; ``scaling`` (factor, original, fast, slow) or None."""
    base: float
    dims: int
    scaling: Optional[Tuple[float, float, float, float]] = None

    @staticmethod
    def read(d, where: str) -> Optional["RotaryConfig"]:
        if d is None:
            return None
        sc = d.get("scaling")
        scaling = None
        if sc is not None:
            w = where + ".scaling"
            scaling = (_float(sc, "factor", w), _float(sc, "original", w), _float(sc, "fast", w), _float(sc, "slow", w))
        r = RotaryConfig(_float(d, "base", where), _int(d, "dims", where), scaling)
        if r.dims <= 0 or r.dims % 2 or not r.base > 0:
            raise ConfigError(f"config.json: {where}: 'dims' must be even and positive, 'base' positive")
        return r

    def to_json(self):
        d: Dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            d["scaling"] = dict(zip(("factor", "original", "fast", "slow"), self.scaling))
        return d


@dataclass(frozen=True)
class TipezenLayer:
    type: str                         # "attention" | "retention"
    heads: int
    dim: int
    vdim: int
    kv_heads: int = 0                 # attention
    scale: float = 0.0                # attention: multiplier of q . k
    softcap: float = 0.0              # attention: 0 = no cap
    window: int = 0                   # attention: 0 = all earlier keys
    v_mix: bool = False               # attention
    decay: Tuple[float, ...] = ()     # retention: one per head
    rot: Optional[RotaryConfig] = None
    ff: int = 0                       # 0 = the layer has no feed-forward
    ff_kind: str = "dense"


@dataclass(frozen=True)
class TipezenConfig(ModelConfig):
    vocab_size: int = 0
    hidden_size: int = 0
    streams: int = 0                  # 0 = one plain residual; S >= 1 = hyper-connections over S streams
    norm_eps: float = 0.0
    layers: Tuple[TipezenLayer, ...] = ()
    max_position: int = MAX_POSITION_DEFAULT

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    @staticmethod
    def from_json_dict(d: Dict[str, Any]) -> "TipezenConfig":
        from .model_config import architecture_name
        layers = []
        raw = _need(d, "layers", "the top level")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        for i, l in enumerate(raw):
            where = f"layers[{i}]"
            kind = _need(l, "type", where)
            m = _need(l, "mixer", where)
            mw = where + ".mixer"
            mlp = l.get("mlp")
            ff, ff_kind = 0, "dense"
            if mlp is not None:
                ff_kind = mlp.get("kind", "dense")
                if ff_kind != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind '{ff_kind}' is not supported (dense only)")
                ff = _int(mlp, "ff", where + ".mlp")
            rot = RotaryConfig.read(m.get("rot"), mw + ".rot")
            heads, dim, vdim = _int(m, "heads", mw), _int(m, "dim", mw), _int(m, "vdim", mw)
            if rot is not None and rot.dims > dim:
                raise ConfigError(f"config.json: {mw}.rot.dims ({rot.dims}) exceeds dim ({dim})")
            if kind == "attention":
                kv = _int(m, "kv_heads", mw, heads)
                if kv <= 0 or heads % kv:
                    raise ConfigError(f"config.json: {mw}: heads ({heads}) must be a multiple of kv_heads ({kv})")
                mask = m.get("mask")
                layers.append(TipezenLayer(
                    type=kind, heads=heads, dim=dim, vdim=vdim, kv_heads=kv,
                    scale=_float(m, "scale", mw, float(dim) ** -0.5), softcap=_float(m, "softcap", mw, 0.0),
                    window=_int(mask, "size", mw + ".mask") if mask is not None else 0,
                    v_mix=bool(m.get("v_mix", False)), rot=rot, ff=ff, ff_kind=ff_kind))
            elif kind == "retention":
                decay = _need(m, "decay", mw)
                if not isinstance(decay, list) or len(decay) != heads:
                    raise ConfigError(f"config.json: {mw}.decay must list one number per head ({heads})")
                layers.append(TipezenLayer(type=kind, heads=heads, dim=dim, vdim=vdim,
                                           decay=tuple(float(x) for x in decay), rot=rot, ff=ff, ff_kind=ff_kind))
            else:
                raise ConfigError(f"config.json: {where}.type '{kind}' is not a mixer of this design "
                                  f"(attention, retention)")
        cfg = TipezenConfig(
            architecture=architecture_name(d), vocab_size=_int(d, "vocab", "the top level"),
            hidden_size=_int(d, "width", "the top level"), streams=_int(d, "streams", "the top level", 0),
            norm_eps=_float(_need(d, "norm", "the top level"), "eps", "norm"), layers=tuple(layers),
            max_position=_int(d, "max_position", "the top level", MAX_POSITION_DEFAULT))
        if cfg.vocab_size <= 0 or cfg.hidden_size <= 0 or cfg.streams < 0 or not cfg.norm_eps > 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive, 'streams' >= 0, norm.eps > 0")
        return cfg

    def to_json_dict(self) -> Dict[str, Any]:
        out = []
        for l in self.layers:
            m: Dict[str, Any] = {"heads": l.heads, "dim": l.dim, "vdim": l.vdim}
            if l.rot is not None:
                m["rot"] = l.rot.to_json()
            if l.type == "attention":
                m.update(kv_heads=l.kv_heads, scale=l.scale, v_mix=l.v_mix)
                if l.softcap > 0:
                    m["softcap"] = l.softcap
                if l.window > 0:
                    m["mask"] = {"size": l.window}
            else:
                m["decay"] = list(l.decay)
            out.append({"type": l.type, "mixer": m, "mlp": {"kind": l.ff_kind, "ff": l.ff} if l.ff else None})
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "norm": {"eps": self.norm_eps}, "layers": out}
        if self.streams:
            d["streams"] = self.streams
        if self.max_position != MAX_POSITION_DEFAULT:
            d["max_position"] = self.max_position
        return d
