"""Tipezen as a model description: a decoder-only design whose layers are listed one by one in config.json, each
a windowed, capped, gated attention with a sink and value mixing, or a retention (linear attention with a fixed
decay per head over a float32 state), with an optional gated feed-forward (tanh-gelu), all of them reading and
writing a residual of several streams through hyper-connections with layer scale.

Tensor names: ``embed``, ``head``, ``final.norm``; layer i: ``l<i>.norm1/2``, ``l<i>.mix.{q,k,v,g,o}`` (and
``.vmix`` in attention layers that say ``v_mix``), ``l<i>.mlp.{gate,up,down}``, ``l<i>.ls1/2`` (layer scale),
``l<i>.hc1/2.{in,out,mix}`` (hyper-connections; 1 = mixer, 2 = feed-forward).
"""
from __future__ import annotations

from ..config.tipezen_config import TipezenConfig
from ..parts.description import ModelDescription, LayerSpec, PartSpec, ScheduleEntry
from ..registry import register_architecture

ARCHITECTURE = "Tipezen"


def describe_tipezen(cfg: TipezenConfig) -> ModelDescription:
    W, S = cfg.hidden_size, cfg.streams
    positions, layers = {}, []
    mix_source_seen = False

    def position_of(rot, pairing):
        if rot is None:
            return None
        name = f"{pairing}:{rot.dims}:{rot.base!r}:{rot.scaling!r}"
        if name not in positions:
            positions[name] = PartSpec("scaled_rotary", dict(rotary_dim=rot.dims, theta=rot.base, pairing=pairing,
                                                             scaling=rot.scaling))
        return name

    def connector(p, q):
        return PartSpec("hyper_connection", dict(
            streams=max(S, 1), hidden_size=W, learned=S > 0, layer_scale=True,
            names={"read": f"hc{q}.in", "write": f"hc{q}.out", "mix": f"hc{q}.mix", "scale": f"ls{q}"}), prefix=p)

    for i, l in enumerate(cfg.layers):
        p = f"l{i}"
        if l.type == "attention":
            if l.v_mix:
                mode = "mix" if mix_source_seen else "source"
                mix_source_seen = True
            else:
                mode = "none"
            mixer = PartSpec("gated_sink_attention", dict(
                hidden_size=W, num_heads=l.heads, num_kv_heads=l.kv_heads, head_dim=l.dim, v_head_dim=l.vdim,
                softmax_scale=l.scale, softcap=l.softcap, window=l.window, sink=True, value_mix=mode,
                value_key="first_values", head_gate=True, lambda_tensor=l.v_mix,
                names={"q": "q", "k": "k", "v": "v", "o": "o", "gate": "g", "lambda": "vmix"}), prefix=f"{p}.mix")
            position = position_of(l.rot, "interleaved")
        else:
            mixer = PartSpec("retention", dict(
                hidden_size=W, num_heads=l.heads, head_dim=l.dim, v_head_dim=l.vdim, decay=l.decay, eps=cfg.norm_eps,
                names={"q": "q", "k": "k", "v": "v", "gate": "g", "o": "o"}), prefix=f"{p}.mix")
            position = position_of(l.rot, "halves")
        ff = None
        if l.ff:
            ff = PartSpec("swiglu", dict(hidden_size=W, intermediate_size=l.ff, activation="gelu_tanh",
                                         names={"gate": "gate", "up": "up", "down": "down"}), prefix=f"{p}.mlp")
        norm = lambda q: PartSpec("rms_norm", dict(dim=W, eps=cfg.norm_eps, name=f"norm{q}"), prefix=p)
        layers.append(LayerSpec(
            mixer=mixer, feed_forward=ff, mixer_norm=norm(1), ffn_norm=norm(2) if ff is not None else None,
            block="stream_pre_norm", position=position,
            connectors={"mixer": connector(p, 1), **({"ffn": connector(p, 2)} if ff is not None else {})}))
    return ModelDescription(
        hidden_size=W, vocab_size=cfg.vocab_size, max_position=cfg.max_position,
        embed_name="embed", lm_head_name="head",
        final_norm=PartSpec("rms_norm", dict(dim=W, eps=cfg.norm_eps, name="norm"), prefix="final"),
        layers=layers, schedule=[ScheduleEntry(layer=i) for i in range(len(layers))],
        positions=positions, streams=max(S, 1))


register_architecture(ARCHITECTURE, TipezenConfig.from_json_dict, describe_tipezen, replace=True)
