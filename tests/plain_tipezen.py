"""A plain, slow, whole-sequence implementation of the Tipezen design in float64, one function per
mechanism.  It shares no code with the package: it reads the nested configuration (the dict that
config.json holds) and a dict of tensors by name, and runs one sequence at a time on the CPU.

Notation: T tokens at positions 0 .. T-1, rows are tokens.  ``w`` maps tensor names to float64 tensors.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

D = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x over the root of (its mean square + eps), along the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_frequencies(rot: dict):
    """(frequencies [dims/2], magnitude) of a rotation: base^(-2i/dims), with the YaRN change of the
    frequencies and of the magnitude of cos and sin when the entry has 'scaling'."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def dim_of(turns):
            return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
        hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
        out = []
        for i, fi in enumerate(f):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(fi / factor * ramp + fi * (1.0 - ramp))
        f = out
        mag = 0.1 * math.log(factor) + 1.0
    return torch.tensor(f, dtype=D), mag


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: Optional[dict], interleaved: bool) -> torch.Tensor:
    """x [T, heads, dim]: the first rot['dims'] dimensions of every head are rotated by position, the rest
    pass.  interleaved: (2i, 2i+1) are a pair; else (i, i + dims/2)."""
    if not rot:
        return x
    dims = int(rot["dims"])
    f, mag = rotary_frequencies(rot)
    ang = positions.to(x.dtype)[:, None] * f.to(x.dtype)[None, :]          # [T, dims/2]
    c, s = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    out = x.clone()
    if interleaved:
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    else:
        a, b = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2] = a * c - b * s
        out[..., dims // 2:dims] = b * c + a * s
    return out


def windowed_sink_attention(q, k, v, scale: float, softcap: float, window: int):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv].  Query i sees keys j with 0 <= i - j < window
    (all j <= i when window is 0); scores are scaled, then capped by softcap * tanh(. / softcap) when softcap
    > 0; the weights are exp(s_j) / (1 + sum_j exp(s_j))."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1) if window > 0 else 0
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            if softcap > 0:
                s = softcap * torch.tanh(s / softcap)
            e = torch.exp(s)
            out[i, h] = (e / (1.0 + e.sum())) @ v[lo:i + 1, g]
    return out


def _same(x):
    return x


def attention_mixer(h, positions, w: Dict[str, torch.Tensor], p: str, m: dict, v_first: Optional[torch.Tensor], r=_same):
    """The attention mixer on its input rows h [T, width].  Returns (output [T, width], the values this layer
    would hand on as v_first [T, G, dv]).  ``r`` is applied to what a 16-bit engine stores in 16 bits (queries,
    cached keys and values, the heads' outputs): the identity here, a rounding where conditioning is looked at."""
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q = (h @ w[p + ".q"].t()).view(T, H, d)
    k = (h @ w[p + ".k"].t()).view(T, G, d)
    v = (h @ w[p + ".v"].t()).view(T, G, dv)
    q = rotate(q, positions, m.get("rot"), interleaved=True)
    k = rotate(k, positions, m.get("rot"), interleaved=True)
    v_own = v
    if m.get("v_mix") and v_first is not None:
        lam = w[p + ".vmix"]
        v = (1.0 - lam) * v + lam * v_first
    window = int(m["mask"]["size"]) if m.get("mask") else 0
    o = windowed_sink_attention(r(q), r(k), r(v), float(m["scale"]), float(m.get("softcap") or 0.0), window)
    gate = torch.sigmoid(h @ w[p + ".g"].t())                   # [T, H]
    o = r(o * gate[:, :, None])
    return o.reshape(T, H * dv) @ w[p + ".o"].t(), v_own


def retention_recurrence(q, k, v, decay: List[float]):
    """S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, token by token; q, k [T, H, d], v [T, H, dv]."""
    T, H, d = q.shape
    dv = v.shape[-1]
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for hh in range(H):
        S = torch.zeros(d, dv, dtype=q.dtype)
        for t in range(T):
            S = decay[hh] * S + torch.outer(k[t, hh], v[t, hh])
            out[t, hh] = S.t() @ q[t, hh]
    return out


def retention_mixer(h, positions, w, p: str, m: dict, eps: float, r=_same):
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q = (h @ w[p + ".q"].t()).view(T, H, d)
    k = (h @ w[p + ".k"].t()).view(T, H, d)
    v = (h @ w[p + ".v"].t()).view(T, H, dv)
    q = rotate(q, positions, m.get("rot"), interleaved=False)
    k = rotate(k, positions, m.get("rot"), interleaved=False) * (d ** -0.5)
    o = rms(retention_recurrence(q, k, v, [float(x) for x in m["decay"]]), eps)
    g = h @ w[p + ".g"].t()
    g = g / (1.0 + torch.exp(-g))
    return r(o.reshape(T, H * dv) * g) @ w[p + ".o"].t()


def dense_ff(h, w, p: str, r=_same):
    return r(gelu_tanh(h @ w[p + ".gate"].t()) * (h @ w[p + ".up"].t())) @ w[p + ".down"].t()


def hyper_read(streams: torch.Tensor, w_in: torch.Tensor) -> torch.Tensor:
    """streams [S, T, width], w_in [S] -> the sublayer's input [T, width]."""
    return torch.einsum("s,stw->tw", w_in, streams)


def hyper_write(streams, y, w_mix, w_out):
    """new_t = sum_s mix[s, t] old_s + out[t] y, all streams at once from the old ones."""
    return torch.einsum("st,sxw->txw", w_mix, streams) + w_out[:, None, None] * y[None]


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, return_layers: bool = False, dtype=D,
            round_inputs: bool = False):
    """Logits [T, vocab] of one sequence (and, if asked, the sum of the streams after every layer).  ``dtype``
    float32 runs everything in 32 bits; ``round_inputs`` rounds every input of a matrix product and the attention's
    queries, keys and values to bfloat16 and nothing else: the two show how far rounding alone moves a position's
    logits (the conditioning of a set of weights at that position)."""
    r = (lambda t: t.to(torch.bfloat16).to(dtype)) if round_inputs else _same
    w = {n: t.to(dtype) for n, t in w.items()}
    eps = float(cfg["norm"]["eps"])
    S = int(cfg.get("streams") or 0)
    T = len(tokens)
    pos = torch.arange(T)
    x = w["embed"][torch.tensor(list(tokens), dtype=torch.long)]
    streams = x[None].repeat(max(S, 1), 1, 1)
    v_first = None
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        for q in (1, 2):
            if q == 2 and layer.get("mlp") is None:
                continue
            u = hyper_read(streams, w[f"{p}.hc{q}.in"]) if S else streams[0]
            hn = rms(u, eps) * w[f"{p}.norm{q}"]
            hn = r(hn)
            if q == 2:
                y = dense_ff(hn, w, p + ".mlp", r)
            elif layer["type"] == "attention":
                m = layer["mixer"]
                y, v_own = attention_mixer(hn, pos, w, p + ".mix", m, v_first if m.get("v_mix") else None, r)
                if m.get("v_mix") and v_first is None:
                    v_first = v_own
            elif layer["type"] == "retention":
                y = retention_mixer(hn, pos, w, p + ".mix", layer["mixer"], eps, r)
            else:
                raise ValueError(layer["type"])
            y = y * w[f"{p}.ls{q}"]
            streams = hyper_write(streams, y, w[f"{p}.hc{q}.mix"], w[f"{p}.hc{q}.out"]) if S else streams + y[None]
        after.append(streams.sum(0))
    x = streams.sum(0)
    logits = r(rms(x, eps) * w["final.norm"]) @ w["head"].t()
    return (logits, torch.stack(after)) if return_layers else logits
