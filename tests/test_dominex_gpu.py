"""The Dominex design in the engine against its plain implementation (plain_dominex.py): every mechanism alone
through the kernel library, and whole models of several small configurations in every cut of the steps.  The
configurations differ in every size and option, with values that are unequal where a model might have them equal
(key and value sizes, heads and key/value heads, rotated dimensions and rotated part) and 1 where it might have more
(heads, experts, chosen experts, block size)."""
import random

import pytest
import torch

import plain_dominex as P
from helpers import trace_whole, trace_tail_decode, trace_portions, trace_mixed, run_trace, first_bad
from test_tipezen_gpu import fake_batch
from tffinfer_b200.config import EngineConfig, DominexConfig, DominexLayer, DominexExperts
from tffinfer_b200.engine import ModelRunner
from tffinfer_b200.weights.random_init import random_state_dict

pytestmark = pytest.mark.gpu
TOL = {"float32": 3e-5, "bfloat16": 5e-2}


def lat(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale=None, base=1e4, rot_dims=0, kv_from=None, mlp=None):
    return DominexLayer(type="latent_attention", heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank,
                        kv_rank=kv_rank, scale=scale if scale is not None else (dim + rot_dim) ** -0.5, rot_base=base,
                        rot_dims=rot_dims or rot_dim, kv_from=kv_from, mlp=mlp)


def par(heads, kv, dim, vdim, chunk, width, scale=None, ls=1.0, rs=1.0, mlp=None):
    return DominexLayer(type="parallel", left_heads=heads, left_kv_heads=kv, left_dim=dim, left_vdim=vdim,
                        left_scale_qk=scale if scale is not None else dim ** -0.5, left_chunk=chunk, right_width=width,
                        left_scale=ls, right_scale=rs, mlp=mlp)


def config(name: str) -> DominexConfig:
    if name == "a":      # sizes that take the tensor-core products; two layers that read an earlier layer's vectors
        m = DominexExperts(ff=64, experts=6, top=2)
        layers = (lat(4, 32, 16, 32, 48, 64, mlp=m), par(8, 2, 64, 64, 24, 96, ls=0.7, rs=1.2, mlp=m),
                  lat(4, 32, 16, 32, 48, 64, kv_from=0, mlp=m), lat(4, 32, 16, 32, 48, 64, kv_from=0),
                  par(8, 2, 64, 64, 24, 96, ls=0.7, rs=1.2, mlp=m))
        return DominexConfig("Dominex", vocab_size=320, hidden_size=128, embed_scale=8.0, norm_eps=1e-5,
                             logit_softcap=20.0, layers=layers)
    if name == "b":      # odd sizes everywhere: FMA products, three query heads a key/value head, a block of 7 positions
        m = DominexExperts(ff=22, experts=5, top=5)                      # that no page size divides, every expert chosen,
        layers = (par(6, 2, 24, 40, 7, 30, scale=0.3, rs=0.5),           # part of the rotated part not rotated, a layer
                  lat(3, 20, 6, 12, 10, 18, scale=0.2, base=1e3, rot_dims=4, mlp=m),      # without a feed-forward
                  par(6, 2, 24, 40, 7, 30, scale=0.3, rs=0.5, mlp=m),
                  lat(3, 20, 6, 12, 10, 18, scale=0.2, base=1e3, rot_dims=4, kv_from=1, mlp=m))
        return DominexConfig("Dominex", vocab_size=97, hidden_size=52, embed_scale=1.0, norm_eps=3e-6,
                             logit_softcap=0.0, layers=layers)
    if name == "c":      # one head, one expert, blocks of one position and no blocks at all, values wider than keys
        m1, m2 = DominexExperts(ff=48, experts=1, top=1), DominexExperts(ff=16, experts=9, top=1)
        layers = (lat(1, 16, 8, 72, 24, 160, base=5e5, mlp=m1), par(1, 1, 16, 32, 1, 64, mlp=m2),
                  par(2, 1, 32, 16, 0, 8, ls=1.5, mlp=m2), lat(2, 8, 32, 8, 16, 40, scale=0.4, mlp=m2))
        return DominexConfig("Dominex", vocab_size=264, hidden_size=64, embed_scale=3.0, norm_eps=1e-6,
                             logit_softcap=8.0, layers=layers)
    if name == "d":      # blocks of 64 over pages of 32, chains of borrowed vectors, a parallel layer first and last
        m = DominexExperts(ff=32, experts=12, top=3)
        layers = (par(8, 8, 16, 16, 64, 40, mlp=m), lat(2, 24, 8, 40, 32, 56, mlp=m), lat(2, 24, 8, 40, 32, 56, kv_from=1, mlp=m),
                  lat(4, 8, 8, 8, 8, 56, mlp=m), lat(2, 24, 8, 40, 32, 56, kv_from=1, mlp=m),
                  lat(4, 8, 8, 8, 8, 56, kv_from=3), par(8, 8, 16, 16, 64, 40, mlp=m))
        return DominexConfig("Dominex", vocab_size=150, hidden_size=96, embed_scale=9.8, norm_eps=1e-6,
                             logit_softcap=30.0, layers=layers)
    raise KeyError(name)


PAGE = {"a": 16, "b": 4, "c": 8, "d": 32}
PROMPTS = {"a": [5, 90, 37, 300], "b": [1, 13, 40, 64], "c": [3, 29, 150, 101], "d": [2, 70, 133]}


def weights(cfg, seed=11, sharp=4.0):
    """Random weights; the query projections are scaled up so that attention is far from uniform and a key that is
    wrongly seen or missed moves the logits; the distance term's numbers are kept positive."""
    sd = random_state_dict(cfg, seed, "bfloat16", norm_noise=0.2)
    for n in sd:
        if n.endswith(".left.q") or n.endswith(".left.k") or n.endswith(".mix.uq"):
            sd[n] = (sd[n].float() * sharp).to(torch.bfloat16)
        elif n.endswith(".left.r1") or n.endswith(".left.r2"):
            sd[n] = sd[n].float().abs().clamp_min(0.1).to(torch.bfloat16)
        elif n.endswith(".router"):
            sd[n] = (sd[n].float() * 8.0).to(torch.bfloat16)         # scores that differ between experts
    return sd


def runner_of(cfg, sd, dtype, page, tokens, live=4, graphs=False):
    return ModelRunner(config=cfg, tensors=dict(sd), engine_config=EngineConfig(
        dtype=dtype, page_size=page, max_cache_tokens=tokens, max_live_requests=live, use_cuda_graphs=graphs))


def requests_of(cfg, name, decoded, seed=5):
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(cfg.vocab_size) for _ in range(n + decoded)] for i, n in enumerate(PROMPTS[name])}


@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cut_matches_plain(name, dtype):
    """Whole prompts, a tail decoded token by token, portions down to two tokens, and mixed batches in a pool
    small enough that pages and slots are used again (released pages are poisoned)."""
    cfg = config(name)
    sd = weights(cfg)
    reqs = requests_of(cfg, name, decoded=12)
    cj = cfg.to_json_dict()
    want = {r: P.forward(cj, sd, t) for r, t in reqs.items()}
    page = PAGE[name]
    most = max(-(-len(t) // page) * page for t in reqs.values())
    cuts = {"whole": (trace_whole(reqs), most), "tail": (trace_tail_decode(reqs, tail=12), most),
            "portions": (trace_portions(reqs), most),
            "mixed": (trace_mixed(reqs, PROMPTS[name], max_live=3, page_size=page, pool_tokens=most + most // 2,
                                  chunk=48), most + most // 2)}
    for cut, (steps, pool) in cuts.items():
        r = runner_of(cfg, sd, dtype, page, pool, live=3)
        stats = {}
        got = run_trace(r, reqs, steps, poison=True, stats=stats)
        for q in reqs:
            bad = first_bad(got[q], want[q], TOL[dtype])
            assert bad is None, f"{name} {dtype} {cut}: request {q} token {bad[0]} off by {bad[1]:.3g}"
        if cut == "mixed":
            assert stats["pages_reused"] > 0


def test_cuts_agree_in_float32():
    """The logits of a position do not depend on how the prompt was cut beyond rounding: far tighter than the
    distance to the plain implementation allows."""
    cfg = config("a")
    sd = weights(cfg)
    reqs = requests_of(cfg, "a", decoded=8)
    most = max(-(-len(t) // 16) * 16 for t in reqs.values())
    ref = run_trace(runner_of(cfg, sd, "float32", 16, most), reqs, trace_whole(reqs))
    for steps in (trace_portions(reqs, sizes=(2, 31, 3, 16, 2, 33)), trace_tail_decode(reqs, tail=40)):
        got = run_trace(runner_of(cfg, sd, "float32", 16, most), reqs, steps)
        for q in reqs:
            assert first_bad(got[q], ref[q], 5e-6) is None


# ------------------------------------------------------------------------------ mechanisms alone
@pytest.fixture(scope="module")
def ops():
    from tffinfer_b200.kernels.library import CudaKernels
    return CudaKernels()


def _select(rows, cols, at):
    """A 0/1 matrix [rows, cols] that picks columns at .. at + rows."""
    w = torch.zeros(rows, cols, dtype=torch.float64)
    w[torch.arange(rows), at + torch.arange(rows)] = 1.0
    return w


def _chunk_case(ops, dtype, H, G, d, dv, chunk, window, lens, starts, aim, biased, page=8, splits=None):
    """Requests whose step brings lens[b] tokens after starts[b] cached ones; in every request a key is planted at
    distance aim[b] behind the LAST query (its query and that key are scaled so that their score stands out among all
    others) with a value of its own: whether it is seen decides the output."""
    dev, dt = "cuda", getattr(torch, dtype)
    g = torch.Generator().manual_seed(1)
    tol = 2e-5 if dtype == "float32" else 2e-2
    nq = H * G
    temp = r1 = r2 = None
    if biased:
        temp = 0.5 + torch.rand(nq, generator=g, dtype=torch.float64)
        r1 = 0.2 + torch.rand(nq, generator=g, dtype=torch.float64)
        r2 = 0.2 + torch.rand(nq, generator=g, dtype=torch.float64)
    dc = max(d, dv)
    full = fake_batch([s + n for n, s in zip(lens, starts)], [0] * len(lens), dev, page)
    cache = torch.full((full.pages + 1, 1, 2, H, page, dc), float("nan"), dtype=dt, device=dev)
    step = fake_batch(lens, starts, dev, page)
    step.block_table = full.block_table
    qs, want = [], []
    for b, (n, s) in enumerate(zip(lens, starts)):
        T = s + n
        q = torch.randn(T, nq, d, generator=g, dtype=torch.float64)
        k = torch.randn(T, H, d, generator=g, dtype=torch.float64)
        v = torch.randn(T, H, dv, generator=g, dtype=torch.float64)
        if 0 <= T - 1 - aim[b]:
            at = T - 1 - aim[b]
            k[at] = 3.0 * q[T - 1].reshape(H, G, d)[:, 0] / q[T - 1].reshape(H, G, d)[:, 0].norm(dim=-1, keepdim=True)
            q[T - 1] *= 3.0
            v[at] = 10.0
        q, k, v = (t.to(dt).double() for t in (q, k, v))          # what the kernel is given, exactly
        ts = torch.arange(T, device=dev)
        pg, sl = full.block_table[b].long()[ts // page], ts % page
        cache[pg, 0, 0, :, sl, :d] = k.to(dt).to(dev)
        cache[pg, 0, 1, :, sl, :dv] = v.to(dt).to(dev)
        hcat = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1)
        Wd = hcat.shape[1]
        ref = P.biased_chunk_attention(hcat, _select(nq * d, Wd, 0), _select(H * d, Wd, nq * d),
                                       _select(H * dv, Wd, nq * d + H * d), torch.eye(nq * dv, dtype=torch.float64),
                                       temp, r1, r2, nq, H, d, dv, 0.25, chunk, window)
        qs.append(q[s:].reshape(n, nq * d))
        want.append(ref[s:])
    qd = torch.cat(qs).to(dt).to(dev).contiguous()
    out = torch.full((qd.shape[0], nq * dv + 3), float("nan"), dtype=dt, device=dev)
    f32 = lambda t: None if t is None else t.float().to(dev)
    ops.attention_tile(qd, step, step.block_table, cache, 0, page, out, nq, H, d, dv, 0.25, window=window, chunk=chunk,
                       temp=f32(temp), r1=f32(r1), r2=f32(r2), out_scale=0.5, out_off=3, num_splits=splits)
    torch.cuda.synchronize()
    got = out[:, 3:].double().cpu() * 2.0
    want = torch.cat(want)
    err = float((got - want).abs().max() / want.abs().max())
    assert err < tol, f"off by {err:.3g}"
    assert torch.isnan(out[:, :3]).all()                        # columns ahead of out_off are nobody's


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("lens,starts", [([40, 1, 1, 1, 1], [0, 39, 40, 47, 300]), ([3, 2, 64, 9], [21, 46, 100, 0])])
def test_chunk_attention_edges_and_far_keys(ops, dtype, lens, starts):
    """Blocks of 24 positions over pages of 8: a key planted at the block's first position (just inside), one position
    ahead of it (just outside), and far away, for decoded tokens and for the last token of a portion; unseen pages are
    NaN.  With and without the distance term, grouped heads (three a key/value head) and unequal key and value sizes."""
    chunk = 24
    ends = [s + n - 1 for n, s in zip(lens, starts)]
    inside = [e % chunk for e in ends]                          # distance to the first position of the block
    for aim in (inside, [a + 1 for a in inside], [max(a - 1, 0) for a in inside], [200] * len(lens)):
        _chunk_case(ops, dtype, 2, 3, 24, 40, chunk, 0, lens, starts, aim, biased=True)
    _chunk_case(ops, dtype, 1, 1, 64, 64, 64, 0, lens, starts, [e % 64 for e in ends], biased=False, page=16)
    _chunk_case(ops, dtype, 1, 4, 16, 16, 0, 0, lens, starts, [e for e in ends], biased=True)        # the very first key, no blocks
    _chunk_case(ops, dtype, 2, 1, 32, 8, 0, 10, lens, starts, [9] * len(lens), biased=False)         # a window's last key
    _chunk_case(ops, dtype, 2, 1, 32, 8, 0, 10, lens, starts, [10] * len(lens), biased=False)        # ... and the one beyond
    _chunk_case(ops, dtype, 2, 2, 8, 8, 5, 3, lens, starts, [2] * len(lens), biased=True)            # both at once
    # the key range in shares (more shares than some rows have key blocks), merged afterwards
    for splits in (2, 8):
        _chunk_case(ops, dtype, 1, 4, 16, 16, 0, 0, lens, starts, [e for e in ends], biased=True, splits=splits)
        _chunk_case(ops, dtype, 2, 3, 24, 40, 64, 0, lens, starts, [e % 64 for e in ends], biased=True, splits=splits)


@pytest.mark.parametrize("width", [8, 100, 300])
def test_min_gru_steps_and_slots(ops, width):
    """The recurrence through two steps (portions, then one token each), slots out of order, other slots poisoned,
    against the plain recurrence over the whole sequences; output columns and scale as the caller says."""
    dev = "cuda"
    g = torch.Generator().manual_seed(2)
    lens1, lens2 = [5, 1, 200], [1, 1, 1]          # 200: the chunked passes, with a last chunk that is not full
    slots = [3, 0, 2]
    state = torch.full((5, width), float("nan"), device=dev)
    bz, bx = torch.randn(width, generator=g), torch.randn(width, generator=g)
    seqs = [torch.randn(a + b, 3 * width + 5, generator=g) * 2.0 for a, b in zip(lens1, lens2)]
    W = 3 * width + 5
    sel = lambda at: _select(width, W, at)
    want = [P.min_gru(s.double(), sel(2), bz.double(), sel(2 + width), bx.double(), sel(2 + 2 * width),
                      torch.eye(width, dtype=torch.float64))[0] for s in seqs]
    got = [[] for _ in seqs]
    for lens, starts in ((lens1, [0, 0, 0]), (lens2, lens1)):
        b = fake_batch(lens, starts, dev, 8, slots=slots)
        ops.reset_state_slots(state, b.slots, b.pos_start)
        proj = torch.cat([s[st:st + n] for s, n, st in zip(seqs, lens, starts)]).to(dev).contiguous()
        out = torch.full((proj.shape[0], width + 4), float("nan"), device=dev)
        ops.min_gru(proj, 2, 2 + width, 2 + 2 * width, bz.to(dev), bx.to(dev), state, b, out, width, out_off=4, out_scale=2.0)
        torch.cuda.synchronize()
        row = 0
        for i, n in enumerate(lens):
            got[i].append(out[row:row + n, 4:].double().cpu() / 2.0)
            row += n
    for i in range(len(seqs)):
        err = float((torch.cat(got[i]) - want[i]).abs().max())
        assert err < 1e-5, f"request {i} off by {err:.3g}"
    assert torch.isnan(state[1]).all() and torch.isnan(state[4]).all()          # nobody's slots were left alone


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,top,ff,W,T", [(5, 1, 24, 40, 70), (7, 3, 64, 128, 130), (3, 3, 10, 52, 9), (1, 1, 16, 64, 3),
                                           (64, 6, 64, 64, 200), (6, 2, 192, 136, 700), (5, 2, 128, 256, 1500)])
def test_routed_experts(ops, dtype, E, top, ff, W, T):
    """Route, sort by expert, the two grouped products and the sum, against the plain loop over tokens; the weight on
    the experts' input (as they are) and on their output (renormalised)."""
    dev, dt = "cuda", getattr(torch, dtype)
    g = torch.Generator().manual_seed(3)
    h = torch.randn(T, W, generator=g).to(dt)
    wr = (torch.randn(E, W, generator=g) * 0.5).to(dt)
    ex = [{"gate": (torch.randn(ff, W, generator=g) * W ** -0.5).to(dt), "up": (torch.randn(ff, W, generator=g) * W ** -0.5).to(dt),
           "down": (torch.randn(W, ff, generator=g) * ff ** -0.5).to(dt)} for _ in range(E)]
    gate_up, layout = ops.stack_gate_up([e["gate"].to(dev) for e in ex], [e["up"].to(dev) for e in ex])
    down = torch.stack([e["down"] for e in ex]).to(dev).contiguous()
    res = torch.randn(T, W, generator=g)
    for weight_on, renorm in (("input", False), ("output", True)):
        want = res.double() + P.routed_experts(h.double(), wr.double(), [{k: v.double() for k, v in e.items()} for e in ex],
                                               top, weight_on, renorm)
        out = res.clone().to(dev)
        ops.routed_mlp(h.to(dev), wr.to(dev), gate_up, layout, down, out, top, renorm, weight_on, "silu")
        torch.cuda.synchronize()
        err = float((out.double().cpu() - want).abs().max() / want.abs().max())
        assert err < (2e-5 if dtype == "float32" else 3e-2), f"{weight_on}: off by {err:.3g}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim,rot,rdims,vd", [(24, 12, 8, 20), (24, 8, 4, 16)])
def test_latent_attention_far_keys_and_borrowed_cache(ops, dtype, dim, rot, rdims, vd):
    """A latent attention layer alone: 700 tokens in portions that end inside pages, then single tokens, with sharp
    queries (a missed key among hundreds shows), part of the rotated part left unrotated; then a second layer with its
    own queries and up-projections reading the first one's cached vectors.  At the end the whole prompt as one step that
    starts at position 0: with sizes that are multiples of 8, in bfloat16, that is the form with per-head keys, the
    second layer taking the step's latents from the first."""
    from tffinfer_b200.parts.latent import LatentAttention
    from tffinfer_b200.parts.position import ScaledRotary
    from tffinfer_b200.parts.base import LayerContext
    dev, dt = "cuda", getattr(torch, dtype)
    g = torch.Generator().manual_seed(4)
    W, H, qr, kr, page, eps = 64, 3, 16, 40, 16, 1e-5
    T = 700
    h = torch.randn(T, W, generator=g).to(dt)
    names = {"dq": (qr, W), "dq.norm": (qr,), "uq": (H * (dim + rot), qr), "dkv": (kr + rot, W), "dkv.norm": (kr,),
             "uk": (H * dim, kr), "uv": (H * vd, kr), "o": (W, H * vd)}
    def make(shared):
        t = {}
        for n, shp in names.items():
            if shared and n.startswith("dkv"):
                continue
            x = torch.randn(*shp, generator=g)
            x = 1.0 + 0.2 * x if len(shp) == 1 else x * shp[-1] ** -0.5 * (4.0 if n == "uq" else 1.0)
            t[n] = x.to(torch.bfloat16)
        return t
    w1, w2 = make(False), make(True)
    pos = ScaledRotary(rdims, 1e4, "interleaved")
    pos.prepare(ops, dev, 0)
    cache = torch.full((T // page + 2, 1, 1, 1, page, kr + rot), float("nan"), dtype=dt, device=dev)
    layers = []
    for w, shared in ((w1, False), (w2, True)):
        m = LatentAttention(W, H, dim, rot, vd, qr, kr, eps, softmax_scale=0.3, shared_kv=shared)
        held = {n: (v.float() if len(v.shape) == 1 else v.to(dt)).to(dev).contiguous() for n, v in w.items()}
        m.load(held, ops, dt)
        layers.append(m)
    d64 = lambda w: {n: v.double() for n, v in w.items()}
    a, b = d64(w1), d64(w2)
    c, r = P.latent_of(h.double(), a["dkv"], a["dkv.norm"], eps, kr, 1e4, rot, rdims)
    want = [P.latent_attention(h.double(), c, r, w["dq"], w["dq.norm"], w["uq"], w["uk"], w["uv"], w["o"], eps, H, dim,
                               rot, vd, 0.3, 1e4, rdims) for w in (a, b)]
    got = [[], []]
    at = 0
    for n in (37, 300, 2, 345, 1, 1, 1, 1) + (1,) * 12:
        batch = fake_batch([n], [at], dev, page)
        table = torch.arange(T // page + 1, dtype=torch.int32, device=dev).reshape(1, -1)
        for i, m in enumerate(layers):
            ctx = LayerContext(batch=batch, ops=ops, kv_cache=cache, kv_layer=0, block_table=table, page_size=page,
                               write_cache=(i == 0), position=pos, shared={})
            got[i].append(m.forward(h[at:at + n].to(dev).contiguous(), ctx, None).double().cpu().clone())
            ops.reset_accumulators()
        at += n
    assert at == T
    for i in range(2):
        err = float((torch.cat(got[i]) - want[i]).abs().max() / want[i].abs().max())
        assert err < (3e-5 if dtype == "float32" else 3e-2), f"layer {i} off by {err:.3g}"
    import numpy as np
    cache.fill_(float("nan"))
    batch = fake_batch([T], [0], dev, page)
    batch.h_pos_start = np.array([0])
    table = torch.arange(T // page + 1, dtype=torch.int32, device=dev).reshape(1, -1)
    shared = {}
    for i, m in enumerate(layers):
        ctx = LayerContext(batch=batch, ops=ops, kv_cache=cache, kv_layer=0, block_table=table, page_size=page,
                           write_cache=(i == 0), position=pos, shared=shared)
        whole = m.forward(h.to(dev).contiguous(), ctx, None).double().cpu().clone()
        ops.reset_accumulators()
        err = float((whole - want[i]).abs().max() / want[i].abs().max())
        assert err < (3e-5 if dtype == "float32" else 3e-2), f"whole prompt, layer {i} off by {err:.3g}"
    assert (dtype == "bfloat16" and (dim + rot) % 8 == 0) == bool(shared), "which form ran is not the one expected"


def test_norm_with_a_weight_around_zero(ops):
    from tffinfer_b200.parts.norm import RMSNorm
    g = torch.Generator().manual_seed(5)
    x = torch.randn(9, 52, generator=g) * 3.0
    w = (torch.randn(52, generator=g) * 0.3).to(torch.bfloat16)
    n = RMSNorm(52, 1e-5, name="w", weight_offset=1.0)
    n.load({"w": w.float().cuda()}, ops, torch.float32)
    got = n.forward(x.cuda(), ops, torch.float32).double().cpu()
    want = P.rms_norm(x.double(), w.double(), 1e-5, unit_offset=True)
    assert float((got - want).abs().max()) < 1e-5


def test_grouped_product_of_column_blocks(ops):
    """Per-group products on column blocks of wider rows, against torch: sizes that fill no tile."""
    g = torch.Generator().manual_seed(6)
    G, M, N, K = 3, 70, 37, 21
    a = torch.randn(M, G * K + 5, generator=g).cuda()
    b = torch.randn(G, N, K, generator=g).to(torch.bfloat16).cuda()
    c = torch.full((M, G * N + 2), float("nan")).cuda()
    ops.gemm_grouped(a, b, c, G, M, N, K, a.shape[1], K, K, N * K, c.shape[1], N)
    torch.cuda.synchronize()
    for i in range(G):
        want = a[:, i * K:(i + 1) * K].double() @ b[i].double().T
        assert float((c[:, i * N:(i + 1) * N].double() - want).abs().max()) < 1e-4
    assert torch.isnan(c[:, G * N:]).all()


@pytest.mark.parametrize("M,N,K,G", [(300, 72, 40, 3), (5, 256, 512, 2), (129, 8, 8, 1)])
def test_grouped_product_on_tensor_cores(ops, M, N, K, G):
    """bfloat16 operands of aligned sizes take the tensor-core kernel: against torch on the same bfloat16 values, for
    tiles that are full, ragged in rows, in columns and in K."""
    g = torch.Generator().manual_seed(7)
    a = torch.randn(M, G * K + 8, generator=g).to(torch.bfloat16).cuda()
    b = torch.randn(G, N, K, generator=g).to(torch.bfloat16).cuda()
    assert ops.grouped_on_tensor_cores(a, b, K, a.shape[1], K, K, N * K, "", N)
    for dt in (torch.float32, torch.bfloat16):
        c = torch.full((M, G * N + 2), float("nan"), dtype=dt).cuda()
        ops.gemm_grouped(a, b, c, G, M, N, K, a.shape[1], K, K, N * K, c.shape[1], N)
        torch.cuda.synchronize()
        for i in range(G):
            want = a[:, i * K:(i + 1) * K].double() @ b[i].double().T
            err = float((c[:, i * N:(i + 1) * N].double() - want).abs().max() / want.abs().max())
            assert err < (1e-5 if dt == torch.float32 else 1e-2), err
        assert torch.isnan(c[:, G * N:]).all()


# ------------------------------------------------------------------------------ generation through the engine
@pytest.mark.parametrize("dtype,name", [("float32", "a"), ("float32", "b"), ("bfloat16", "a")])
def test_greedy_generation_through_the_engine(dtype, name):
    """Six requests on three state slots and a pool that holds two of them at a time, decode steps replayed as CUDA
    graphs, 60 new tokens each: the scheduler admits, preempts and frees; in 32-bit every request's tokens are those
    of the plain implementation decoding greedily (a token whose two best logits are closer than rounding may
    differ: from there on the rest is not compared)."""
    import tffinfer_b200 as tff
    cfg = config(name)
    sd = weights(cfg, sharp=2.0)
    rng = random.Random(2)
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(n)] for n in (3, 40, 17, 64, 9, 25)]
    new = 60
    runner = ModelRunner(config=cfg, tensors=dict(sd), engine_config=EngineConfig(
        dtype=dtype, page_size=PAGE[name], max_cache_tokens=256, max_live_requests=3, use_cuda_graphs=True,
        max_tokens_per_step=48))
    eng = tff.Engine(runner=runner)
    outs = eng.generate(prompts, max_new_tokens=new)
    assert all(len(o) == new for o in outs)
    if dtype != "float32":
        return
    cj = cfg.to_json_dict()
    for p, o in zip(prompts[:3], outs[:3]):
        seq = list(p)
        for i in range(new):
            logits = P.forward(cj, sd, seq)[-1]
            top = torch.topk(logits, 2).values
            if float(top[0] - top[1]) < 1e-3 * float(logits.abs().max()):
                break
            assert int(logits.argmax()) == o[i], f"token {i} differs"
            seq.append(o[i])


# ------------------------------------------------------------------------------ the replay tool and the command line
def test_trace_replay_tool_on_a_model_folder(tmp_path):
    """bin/trace_run on a Dominex folder written by the random-weights mode: a mixed schedule (portions beside single
    tokens, four live requests, a pool that makes later requests reuse pages and slots) in both number formats."""
    import numpy as np
    from test_trace_run_gpu import _replay, _max_tokens
    from helpers import steps_to_jsonl
    from tffinfer_b200.weights import write_random_model
    from tffinfer_b200.weights.safetensors_io import SafetensorsFile
    cfg = config("d")
    d = write_random_model(str(tmp_path / "model"), cfg, seed=5)
    f = SafetensorsFile(str(tmp_path / "model" / "model.safetensors"))
    sd = {n: f.tensor(n).clone() for n in f.names()}
    rng = random.Random(9)
    prompts = [70, 3, 130, 41, 18]
    reqs = {f"q{i}": [rng.randrange(cfg.vocab_size) for _ in range(n + 10)] for i, n in enumerate(prompts)}
    want = {r: P.forward(cfg.to_json_dict(), sd, t) for r, t in reqs.items()}
    steps = trace_mixed(reqs, prompts, max_live=4, page_size=64, pool_tokens=384, chunk=33)
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        out.mkdir()
        assert _replay(d, dtype, _max_tokens(reqs, steps), steps_to_jsonl(reqs, steps), str(out)) == 0
        got = {r: [None] * len(t) for r, t in reqs.items()}
        for i, (entries, _) in enumerate(steps):
            rows = sum(n for _, _, n in entries)
            arr = torch.from_numpy(np.fromfile(str(out / f"{i}.f32"), dtype="<f4").reshape(rows, cfg.vocab_size))
            row = 0
            for r, start, n in entries:
                for k in range(n):
                    got[r][start + k] = arr[row]
                    row += 1
        for r in reqs:
            assert first_bad(torch.stack(got[r]), want[r], TOL[dtype]) is None, (dtype, r)


def test_command_line_generates(tmp_path):
    import json
    import subprocess
    import sys
    import os
    from tffinfer_b200.weights import write_random_model
    d = write_random_model(str(tmp_path / "model"), config("b"), seed=1)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, "-m", "tffinfer_b200", d, "--prompt-ids", "1,2,3,4,5", "--prompt-ids", "7,8",
                        "--n-predict", "12", "--max-live", "2", "--max-cache-tokens", "128", "--json"],
                       cwd=root, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    out = json.loads(p.stdout.strip().splitlines()[-1])
    assert [len(o) for o in out["outputs"]] == [12, 12]


# ------------------------------------------------------------------------------ configurations drawn at random
def draw(seed: int):
    """Layer orders, sizes and constants drawn at random: which products run (tensor-core or FMA) follows from the sizes."""
    rng = random.Random(seed)
    W = rng.choice([64, 96, 128, 192]) if rng.random() < 0.75 else rng.choice([36, 100, 150])
    n_layers = rng.choice([2, 3, 4, 6])
    heads = rng.choice([1, 2, 4, 8])
    dim, rot = rng.choice([8, 16, 32, 24]), rng.choice([4, 8, 16, 32])
    latent = dict(heads=heads, dim=dim, rot_dim=rot, vdim=rng.choice([8, 16, 40, 64]), q_rank=rng.choice([8, 24, 48, 13]),
                  kv_rank=rng.choice([16, 32, 72, 128, 27]), scale=rng.choice([None, 0.11, 0.3]),
                  base=rng.choice([1e4, 5e5]), rot_dims=rng.choice([0, 0, rot // 2 // 2 * 2 or rot]))
    a_heads = rng.choice([1, 2, 4, 6])
    a_kv = rng.choice([h for h in (1, 2, 3, 4, 6) if a_heads % h == 0])
    a_dim = rng.choice([16, 32, 64, 48])
    parallel = dict(heads=a_heads, kv=a_kv, dim=a_dim, vdim=a_dim if rng.random() < 0.5 else rng.choice([16, 32, 96]),
                    chunk=rng.choice([0, 1, 5, 16, 33, 64, 100]), width=rng.choice([8, 64, 100, 224]),
                    scale=rng.choice([None, 0.2]), ls=rng.choice([1.0, 0.6]), rs=rng.choice([1.0, 1.3]))
    E = rng.choice([1, 4, 8, 12])
    mlp = DominexExperts(ff=rng.choice([16, 64, 40]), experts=E, top=rng.randint(1, min(E, 4)))
    layers, own = [], []
    for i in range(n_layers):
        m = mlp if rng.random() < 0.85 else None
        if rng.random() < 0.6:
            src = rng.choice(own) if own and rng.random() < 0.4 else None
            if src is None:
                own.append(i)
            layers.append(lat(kv_from=src, mlp=m, **latent))
        else:
            layers.append(par(mlp=m, **parallel))
    cfg = DominexConfig("Dominex", vocab_size=rng.choice([97, 256, 311, 1000]), hidden_size=W,
                        embed_scale=rng.choice([1.0, W ** 0.5]), norm_eps=rng.choice([1e-6, 1e-5]),
                        logit_softcap=rng.choice([0.0, 15.0, 40.0]), layers=tuple(layers))
    return cfg, rng.choice([8, 16, 32]), [rng.randint(1, 40), rng.randint(60, 200), rng.randint(2, 330), rng.randint(20, 90)]


@pytest.mark.parametrize("seed", list(range(1, 17)))
def test_random_configuration_matches_plain(seed):
    cfg, page, prompts = draw(seed)
    sd = weights(cfg, seed=seed, sharp=3.0)
    rng = random.Random(50 + seed)
    reqs = {f"r{i}": [rng.randrange(cfg.vocab_size) for _ in range(n + 5)] for i, n in enumerate(prompts)}
    cj = cfg.to_json_dict()
    want = {r: P.forward(cj, sd, t) for r, t in reqs.items()}
    most = max(-(-len(t) // page) * page for t in reqs.values())
    pool = most + most // 2
    for dtype in ("float32", "bfloat16"):
        for steps, tokens in ((trace_mixed(reqs, prompts, max_live=3, page_size=page, pool_tokens=pool, chunk=48), pool),
                              (trace_portions(reqs, sizes=(64, 2, 17, 130, 3)), most)):
            got = run_trace(runner_of(cfg, sd, dtype, page, tokens, live=3), reqs, steps, poison=True)
            for q in reqs:
                bad = first_bad(got[q], want[q], TOL[dtype])
                assert bad is None, f"draw {seed} {dtype}: request {q} token {bad[0]} off by {bad[1]:.3g}: {cj}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_graph_replay(dtype):
    """Two requests decoded for 300 tokens, one token a step, the steps replayed as CUDA graphs: the blocks of the
    chunked attention pass over decoded tokens many times, pages are given back behind them, and the recurrent state
    is carried all the way."""
    cfg = config("a")
    sd = weights(cfg)
    rng = random.Random(4)
    reqs = {r: [rng.randrange(cfg.vocab_size) for _ in range(n + 300)] for r, n in (("r0", 21), ("r1", 3))}
    want = {r: P.forward(cfg.to_json_dict(), sd, t) for r, t in reqs.items()}
    steps = [([("r0", 0, 21), ("r1", 0, 3)], [])]
    steps += [([("r0", 21 + i, 1), ("r1", 3 + i, 1)], ["r0", "r1"] if i == 299 else []) for i in range(300)]
    r = runner_of(cfg, sd, dtype, 16, 2 * 336, live=2, graphs=True)
    got = run_trace(r, reqs, steps, poison=True)
    assert any(st["graphs"] for st in r._graphs.values()), "the decode steps were not replayed as graphs"
    for q in reqs:
        bad = first_bad(got[q], want[q], TOL[dtype])
        assert bad is None, f"{dtype}: request {q} token {bad[0]} off by {bad[1]:.3g}"
