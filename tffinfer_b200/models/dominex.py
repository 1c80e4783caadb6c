"""Dominex as a model description: a decoder-only design whose layers are listed one by one in config.json.  A layer
is pre-norm (``x + mixer(norm1 x)``, then ``x + moe(norm2 x)`` where it has a feed-forward) with RMS norms whose
weights are stored around zero (multiplier 1 + w).  Its mixer is a latent attention (parts/latent.py; a layer with
``kv_from`` reads the cached vectors of an earlier layer) or two mixers side by side (parts/parallel.py): a chunked
attention without rotation whose scores carry a per-head temperature and a logarithmic distance term, and a minGRU
recurrence.  The feed-forward is a mixture of experts whose sigmoid scores multiply the experts' inputs.  The
embedding is scaled, the output matrix is the embedding table, and the logits are capped by a tanh.

Tensor names: ``embed``, ``final.norm``; layer i: ``l<i>.norm1/2``; latent attention ``l<i>.mix.{dq,dq.norm,uq,dkv,
dkv.norm,uk,uv,o}``; parallel ``l<i>.mix.left.{q,k,v,o,temp,r1,r2}`` and ``l<i>.mix.right.{z,z.b,x,x.b,g,o}``;
experts ``l<i>.mlp.router`` and ``l<i>.mlp.e<j>.{gate,up,down}``."""
from __future__ import annotations

from ..config.dominex_config import DominexConfig
from ..parts.description import ModelDescription, LayerSpec, PartSpec, ScheduleEntry
from ..registry import register_architecture

ARCHITECTURE = "Dominex"


def describe_dominex(cfg: DominexConfig) -> ModelDescription:
    W = cfg.hidden_size
    positions, layers, schedule = {}, [], []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}"
        position = None
        if l.type == "latent_attention":
            position = f"interleaved:{l.rot_dims}:{l.rot_base!r}"
            if position not in positions:
                positions[position] = PartSpec("scaled_rotary", dict(rotary_dim=l.rot_dims, theta=l.rot_base,
                                                                     pairing="interleaved"))
            mixer = PartSpec("latent_attention", dict(
                hidden_size=W, num_heads=l.heads, head_dim=l.dim, rot_dim=l.rot_dim, v_head_dim=l.vdim, q_rank=l.q_rank,
                kv_rank=l.kv_rank, eps=cfg.norm_eps, softmax_scale=l.scale, shared_kv=l.kv_from is not None),
                prefix=f"{p}.mix")
        else:
            mixer = PartSpec("parallel", dict(hidden_size=W, branches=[
                dict(name="left", kind="biased_chunk_attention", scale=l.left_scale, params=dict(
                    hidden_size=W, num_heads=l.left_heads, num_kv_heads=l.left_kv_heads, head_dim=l.left_dim,
                    v_head_dim=l.left_vdim, softmax_scale=l.left_scale_qk, chunk=l.left_chunk, head_temperature=True,
                    distance_bias=True)),
                dict(name="right", kind="min_gru", scale=l.right_scale, params=dict(hidden_size=W, width=l.right_width)),
            ]), prefix=f"{p}.mix")
        ff = None
        if l.mlp is not None:
            ff = PartSpec("routed_experts", dict(hidden_size=W, intermediate_size=l.mlp.ff, num_experts=l.mlp.experts,
                                                 top=l.mlp.top, activation="silu", renormalize=False, weight_on="input"),
                          prefix=f"{p}.mlp")
        norm = lambda q: PartSpec("rms_norm", dict(dim=W, eps=cfg.norm_eps, name=f"norm{q}", weight_offset=1.0), prefix=p)
        layers.append(LayerSpec(mixer=mixer, feed_forward=ff, mixer_norm=norm(1),
                                ffn_norm=norm(2) if ff is not None else None, block="pre_norm", position=position))
        schedule.append(ScheduleEntry(layer=i, cache_of=l.kv_from))      # one run per layer: entry j is layer j
    return ModelDescription(
        hidden_size=W, vocab_size=cfg.vocab_size, max_position=cfg.max_position, embed_name="embed", lm_head_name=None,
        final_norm=PartSpec("rms_norm", dict(dim=W, eps=cfg.norm_eps, name="norm", weight_offset=1.0), prefix="final"),
        layers=layers, schedule=schedule, positions=positions, embed_scale=cfg.embed_scale,
        logit_softcap=cfg.logit_softcap)


register_architecture(ARCHITECTURE, DominexConfig.from_json_dict, describe_dominex, replace=True)
