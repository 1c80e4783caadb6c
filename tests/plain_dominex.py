"""A plain, slow implementation of the Dominex design in float64 (or float32), one function per mechanism, written
from the design's equations and sharing no code with the package.  It runs whole sequences at once on the CPU and
is what the framework's kernels, cache, state slots and batching are compared with.

Notation: T tokens at positions 0..T-1, W the model width, x the residual [T, W].

    layer:       x <- x + mixer(norm(x));  x <- x + moe(norm(x))         norm(x) = x / sqrt(mean(x^2) + eps) * (1 + w)
    parallel:    a * biased_chunk_attention(h) + b * min_gru(h)
    latent:      attention whose keys and values are made from a small vector per token
    output:      cap * tanh(E norm(x) / cap), E the embedding table
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_norm(x, w, eps: float, unit_offset: bool):
    """x / sqrt(mean(x^2) + eps) times (1 + w) or w; no weight when w is None."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    if w is None:
        return y
    return y * ((1.0 + w) if unit_offset else w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rotate_pairs(x, positions, base: float, dims: int):
    """x [T, ..., D]: the first ``dims`` elements are turned, element 2i with 2i+1, by positions * base^(-2i/dims)."""
    out = x.clone()
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    ang = positions.to(x.dtype)[:, None] * f[None, :]                    # [T, half]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def softmax_rows(scores, visible):
    """Softmax over the visible keys of every row; scores [.., T, T], visible bool [T, T]."""
    s = scores.masked_fill(~visible, float("-inf"))
    s = s - s.max(dim=-1, keepdim=True).values
    e = torch.exp(s)
    return e / e.sum(dim=-1, keepdim=True)


def biased_chunk_attention(h, wq, wk, wv, wo, temp, r1, r2, heads: int, kv_heads: int, dim: int, vdim: int,
                           scale: float, chunk: int, window: int = 0):
    """Grouped heads without rotation.  score(i, j) = q_i.k_j * scale * temp_h - r1_h * ln(1 + r2_h * (i - j)) for
    j <= i in the same block of ``chunk`` positions (blocks counted from position 0); chunk 0 = all j <= i."""
    T = h.shape[0]
    q = (h @ wq.T).reshape(T, heads, dim)
    k = (h @ wk.T).reshape(T, kv_heads, dim)
    v = (h @ wv.T).reshape(T, kv_heads, vdim)
    pos = torch.arange(T)
    dist = (pos[:, None] - pos[None, :]).clamp(min=0).to(h.dtype)
    visible = pos[None, :] <= pos[:, None]
    if chunk > 0:
        visible = visible & ((pos[:, None] // chunk) == (pos[None, :] // chunk))
    if window > 0:
        visible = visible & (pos[None, :] > pos[:, None] - window)
    outs = []
    for hd in range(heads):
        g = hd // (heads // kv_heads)
        s = (q[:, hd] @ k[:, g].T) * scale * (temp[hd] if temp is not None else 1.0)
        if r1 is not None:
            s = s - r1[hd] * torch.log1p(r2[hd] * dist)
        outs.append(softmax_rows(s, visible) @ v[:, g])
    return torch.cat(outs, dim=-1) @ wo.T


def min_gru(h, wz, bz, wx, bx, wg, wo, state=None):
    """z = sigmoid(Wz h + bz); u = Wx h + bx; c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0);
    S_t = (1 - z_t) S_(t-1) + z_t c_t, S_(-1) = state or 0; out = Wo (S_t * silu(Wg h)).  Returns (out, last S)."""
    z = torch.sigmoid(h @ wz.T + bz)
    u = h @ wx.T + bx
    c = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    S = torch.zeros(wz.shape[0], dtype=h.dtype) if state is None else state.clone()
    rows = []
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * c[t]
        rows.append(S)
    mixed = torch.stack(rows) * silu(h @ wg.T)
    return mixed @ wo.T, S


def latent_of(h, wdkv, dkv_norm, eps: float, kv_rank: int, rot_base: float, rot_dim: int, rot_dims: int = 0):
    """What a latent attention layer keeps of every token: (c [T, kv_rank] normed, r [T, rot_dim] with its first
    ``rot_dims`` (0: all) elements rotated)."""
    T = h.shape[0]
    d = h @ wdkv.T
    c = rms_norm(d[:, :kv_rank], dkv_norm, eps, unit_offset=False)
    r = rotate_pairs(d[:, kv_rank:kv_rank + rot_dim], torch.arange(T), rot_base, rot_dims or rot_dim)
    return c, r


def latent_attention(h, c, r, wdq, dq_norm, wuq, wuk, wuv, wo, eps: float, heads: int, dim: int, rot_dim: int,
                     vdim: int, scale: float, rot_base: float, rot_dims: int = 0):
    """Queries through a normed latent; per head [dim plain | rot_dim rotated]; keys W_uk c beside the shared r;
    values W_uv c; causal softmax of (q_plain.k_plain + q_rot.r) * scale."""
    T = h.shape[0]
    cq = rms_norm(h @ wdq.T, dq_norm, eps, unit_offset=False)
    q = (cq @ wuq.T).reshape(T, heads, dim + rot_dim)
    q_plain = q[..., :dim]
    q_rot = rotate_pairs(q[..., dim:].contiguous(), torch.arange(T), rot_base, rot_dims or rot_dim)
    k_plain = (c @ wuk.T).reshape(T, heads, dim)
    v = (c @ wuv.T).reshape(T, heads, vdim)
    pos = torch.arange(T)
    visible = pos[None, :] <= pos[:, None]
    outs = []
    for hd in range(heads):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ r.T) * scale
        outs.append(softmax_rows(s, visible) @ v[:, hd])
    return torch.cat(outs, dim=-1) @ wo.T


def routed_experts(h, w_router, experts: List[Dict[str, torch.Tensor]], top: int, weight_on: str = "input",
                   renormalize: bool = False):
    """s = sigmoid(W_r h); the ``top`` experts of largest s; out = sum_e down_e(silu(gate_e(s_e h)) * up_e(s_e h)):
    the score scales the expert's input, and the scores are used as they are.  (``weight_on`` "output": the score
    scales the expert's output instead; ``renormalize``: the chosen scores are divided by their sum.)"""
    s = torch.sigmoid(h @ w_router.T)
    out = torch.zeros(h.shape[0], experts[0]["down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        order = sorted(range(len(experts)), key=lambda e: (-float(s[t, e]), e))[:top]
        total = sum(s[t, e] for e in order) if renormalize else 1.0
        for e in order:
            wt = s[t, e] / total
            xin = wt * h[t] if weight_on == "input" else h[t]
            w = experts[e]
            y = w["down"] @ (silu(w["gate"] @ xin) * (w["up"] @ xin))
            out[t] += y if weight_on == "input" else wt * y
    return out


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens, dtype=torch.float64, layers_out: Optional[list] = None):
    """Logits [T, vocab] of a whole sequence.  ``config`` is the dict of config.json; ``weights`` by tensor name.
    ``layers_out``, a list, receives the residual after every layer."""
    Wt = {n: (t.to(dtype) if t.is_floating_point() else t) for n, t in weights.items()}
    eps = float(config["norm"]["eps"])
    T = len(tokens)
    x = Wt["embed"][torch.tensor(list(tokens), dtype=torch.long)] * float((config.get("embedding") or {}).get("scale", 1.0))
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}", layer["mixer"]
        h = rms_norm(x, Wt[f"{p}.norm1"], eps, unit_offset=True)
        if layer["type"] == "parallel":
            L, R = m["left"], m["right"]
            left = biased_chunk_attention(
                h, Wt[f"{p}.mix.left.q"], Wt[f"{p}.mix.left.k"], Wt[f"{p}.mix.left.v"], Wt[f"{p}.mix.left.o"],
                Wt[f"{p}.mix.left.temp"], Wt[f"{p}.mix.left.r1"], Wt[f"{p}.mix.left.r2"], L["heads"],
                L.get("kv_heads", L["heads"]), L["dim"], L["vdim"], float(L["scale"]),
                int(L["mask"]["size"]) if L.get("mask") else 0)
            right, _ = min_gru(h, Wt[f"{p}.mix.right.z"], Wt[f"{p}.mix.right.z.b"], Wt[f"{p}.mix.right.x"],
                               Wt[f"{p}.mix.right.x.b"], Wt[f"{p}.mix.right.g"], Wt[f"{p}.mix.right.o"])
            y = float(m.get("left_scale", 1.0)) * left + float(m.get("right_scale", 1.0)) * right
        elif layer["type"] == "latent_attention":
            base, rdim = float(m["rot"]["base"]), int(m["rot_dim"])
            rdims = int(m["rot"].get("dims", rdim))
            if m.get("kv_from") is None:
                kept[i] = latent_of(h, Wt[f"{p}.mix.dkv"], Wt[f"{p}.mix.dkv.norm"], eps, int(m["kv_rank"]), base, rdim, rdims)
                c, r = kept[i]
            else:
                c, r = kept[int(m["kv_from"])]
            y = latent_attention(h, c, r, Wt[f"{p}.mix.dq"], Wt[f"{p}.mix.dq.norm"], Wt[f"{p}.mix.uq"],
                                 Wt[f"{p}.mix.uk"], Wt[f"{p}.mix.uv"], Wt[f"{p}.mix.o"], eps, int(m["heads"]),
                                 int(m["dim"]), rdim, int(m["vdim"]), float(m["scale"]), base, rdims)
        else:
            raise ValueError(layer["type"])
        x = x + y
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, Wt[f"{p}.norm2"], eps, unit_offset=True)
            n = int(mlp["router"]["experts"])
            ex = [{k: Wt[f"{p}.mlp.e{e}.{k}"] for k in ("gate", "up", "down")} for e in range(n)]
            x = x + routed_experts(h, Wt[f"{p}.mlp.router"], ex, int(mlp["router"]["top"]))
        if layers_out is not None:
            layers_out.append(x.clone())
    hn = rms_norm(x, Wt["final.norm"], eps, unit_offset=True)
    logits = hn @ Wt["embed"].T
    cap = float(config.get("logit_softcap") or 0.0)
    if cap > 0:
        logits = cap * torch.tanh(logits / cap)
    return logits


def greedy(config: dict, weights, prompt, new_tokens: int, dtype=torch.float64):
    """Greedy continuation by recomputing the whole sequence for every token (first maximum)."""
    seq = list(prompt)
    for _ in range(new_tokens):
        seq.append(int(torch.argmax(forward(config, weights, seq, dtype)[-1])))
    return seq[len(prompt):]
