"""The Tipezen design in the engine against its plain implementation (plain_tipezen.py): every mechanism alone
through the kernel library, and whole models of several small configurations in every cut of the steps.  The
configurations differ in every size and option, with values that are unequal where a model might have them
equal (key and value sizes, heads and key/value heads, rotated part and head size) and 1 where it might have more
(streams, heads, window)."""
import math
import random
from types import SimpleNamespace

import pytest
import torch

import plain_tipezen as P
from helpers import trace_whole, trace_tail_decode, trace_portions, trace_mixed, run_trace, first_bad
from tffinfer_b200.config import EngineConfig, TipezenConfig, TipezenLayer, RotaryConfig
from tffinfer_b200.engine import ModelRunner
from tffinfer_b200.weights.random_init import random_state_dict

pytestmark = pytest.mark.gpu
TOL = {"float32": 3e-5, "bfloat16": 5e-2}
YARN = (4.0, 64.0, 8.0, 1.0)


def att(heads, kv, dim, vdim, window, rot=None, v_mix=False, softcap=20.0, scale=None, ff=0):
    return TipezenLayer(type="attention", heads=heads, kv_heads=kv, dim=dim, vdim=vdim, window=window, rot=rot,
                        v_mix=v_mix, softcap=softcap, scale=scale if scale is not None else dim ** -0.5, ff=ff)


def ret(heads, dim, vdim, decay, rot=None, ff=0):
    return TipezenLayer(type="retention", heads=heads, dim=dim, vdim=vdim, decay=tuple(decay), rot=rot, ff=ff)


def config(name: str) -> TipezenConfig:
    if name == "a":      # every mechanism, sizes that take the tensor-core products and the head-64 attention kernels
        r1, r2 = RotaryConfig(1e4, 32, YARN), RotaryConfig(5e5, 16)
        layers = (att(4, 2, 64, 64, 24, r1, v_mix=True, ff=128), ret(2, 32, 64, [0.96, 0.995], r2),
                  att(4, 2, 64, 64, 24, r1, v_mix=True), ret(2, 32, 64, [0.9, 0.999], r2, ff=192),
                  att(4, 2, 64, 64, 9, r1, v_mix=True, ff=128))
        return TipezenConfig("Tipezen", vocab_size=320, hidden_size=128, streams=3, norm_eps=1e-5, layers=layers)
    if name == "b":      # odd sizes everywhere: FMA products, the general attention kernel, one stream, one head
        r1, r2 = RotaryConfig(1e3, 20), RotaryConfig(2e4, 12, (8.0, 32.0, 4.0, 0.5))
        layers = (ret(1, 20, 12, [0.97], r1, ff=70), att(3, 3, 24, 40, 1, r2, softcap=0.0, scale=0.3),
                  att(6, 2, 40, 24, 200, None, v_mix=False, ff=52), ret(3, 12, 28, [0.5, 0.9, 1.0], None))
        return TipezenConfig("Tipezen", vocab_size=97, hidden_size=52, streams=1, norm_eps=3e-6, layers=layers)
    if name == "c":      # a plain residual (no streams key), five streams in "d"; whole-head rotation; wide values
        r = RotaryConfig(1e6, 64)
        layers = (att(2, 1, 64, 128, 33, r, v_mix=True, ff=64), att(2, 1, 64, 128, 70, r, v_mix=True),
                  ret(2, 64, 64, [0.99, 0.9], r))
        return TipezenConfig("Tipezen", vocab_size=264, hidden_size=64, streams=0, norm_eps=1e-6, layers=layers)
    if name == "d":
        c = config("c")
        return TipezenConfig("Tipezen", vocab_size=c.vocab_size, hidden_size=c.hidden_size, streams=5,
                             norm_eps=c.norm_eps, layers=c.layers)
    raise KeyError(name)


PAGE = {"a": 16, "b": 4, "c": 8, "d": 32}
PROMPTS = {"a": [5, 90, 37, 300], "b": [1, 13, 40, 64], "c": [3, 29, 150, 101], "d": [2, 70, 33]}


def weights(cfg, seed=11, sharp=4.0):
    """Random weights; the query and key projections are scaled up so that attention is far from uniform and a
    key that is wrongly seen or missed moves the logits."""
    sd = random_state_dict(cfg, seed, "bfloat16", norm_noise=0.2)
    tame = min(1.0, 3.0 / max(cfg.streams, 1))      # many streams of independent noise nearly cancel in a read
    for n in sd:
        if n.endswith(".mix.q") or n.endswith(".mix.k"):
            sd[n] = (sd[n].float() * sharp).to(torch.bfloat16)
        elif ".hc" in n and n.endswith(".mix"):
            eye = torch.eye(sd[n].shape[0])
            sd[n] = (eye + (sd[n].float() - eye) * tame).to(torch.bfloat16)
        elif ".hc" in n:
            sd[n] = (1.0 + (sd[n].float() - 1.0) * tame).to(torch.bfloat16)
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
def fake_batch(lens, starts, dev, page, slots=None):
    """The arrays of a step in which request b brings lens[b] tokens from position starts[b]; pages in order."""
    pos, req, qs = [], [], [0]
    for b, (n, s) in enumerate(zip(lens, starts)):
        pos += list(range(s, s + n))
        req += [b] * n
        qs.append(qs[-1] + n)
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    width = max(-(-(s + n) // page) for n, s in zip(lens, starts))
    table, nxt = [], 0
    for n, s in zip(lens, starts):
        k = -(-(s + n) // page)
        table.append(list(range(nxt, nxt + k)) + [-1] * (width - k))
        nxt += k
    import numpy as np
    order = sorted(range(len(lens)), key=lambda b: (lens[b], -(starts[b] + lens[b])))   # as the engine packs a step
    return SimpleNamespace(positions=t(pos), tok_req=t(req), q_start=t(qs), pos_start=t(starts),
                           slots=t(slots if slots is not None else list(range(len(lens)))), num_requests=len(lens),
                           max_q_len=max(lens), num_tokens=len(pos), block_table=t(table), pages=nxt,
                           max_kv_len=max(s + n for n, s in zip(lens, starts)), req_order=t(order),
                           h_sorted_q_lens=np.array([lens[b] for b in order]),
                           h_sorted_kv_lens=np.array([starts[b] + lens[b] for b in order]), key_split_class=None)


@pytest.fixture(scope="module")
def ops():
    from tffinfer_b200.kernels.library import CudaKernels
    return CudaKernels()


@pytest.mark.parametrize("S,W", [(1, 40), (4, 256), (7, 1030)])
def test_stream_step(ops, S, W):
    g = torch.Generator().manual_seed(S)
    T = 9
    x = torch.randn(T, S, W, generator=g)
    y, scale, w = torch.randn(T, W, generator=g), 1 + 0.3 * torch.randn(W, generator=g), 1 + 0.3 * torch.randn(W, generator=g)
    mix, out, rd = torch.randn(S, S, generator=g), torch.randn(S, generator=g), torch.randn(S, generator=g)
    new = P.hyper_write(x.transpose(0, 1).double(), (y * scale).double(), mix.double(), out.double())
    want_h = P.rms(P.hyper_read(new, rd.double()), 1e-5) * w.double()
    xd = x.cuda()
    h = torch.empty(T, W, device="cuda")
    ops.stream_step(xd, y=y.cuda(), scale=scale.cuda(), mix=mix.cuda(), out=out.cuda(), read=rd.cuda(),
                    norm_weight=w.cuda(), eps=1e-5, h=h)
    assert torch.allclose(xd.cpu().double(), new.transpose(0, 1), rtol=1e-5, atol=1e-5)
    assert torch.allclose(h.cpu().double(), want_h, rtol=1e-4, atol=1e-5)
    # the write alone, then the read alone at some rows, give the same
    xd2 = x.cuda()
    ops.stream_step(xd2, y=y.cuda(), scale=scale.cuda(), mix=mix.cuda(), out=out.cuda())
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device="cuda")
    h2 = torch.empty(3, W, device="cuda", dtype=torch.bfloat16)
    ops.stream_step(xd2, read=rd.cuda(), norm_weight=w.cuda(), eps=1e-5, h=h2, row_index=rows)
    assert torch.equal(xd2, xd)
    assert torch.allclose(h2.float().cpu().double(), want_h[[7, 0, 3]], rtol=1e-2, atol=1e-2)
    # write and read at chosen rows, one of them twice: the streams stay as they were, the rows' h is that of the write
    xd3 = x.cuda()
    rows = torch.tensor([5, 2, 5], dtype=torch.int32, device="cuda")
    h3 = torch.empty(3, W, device="cuda")
    ops.stream_step(xd3, y=y.cuda(), scale=scale.cuda(), mix=mix.cuda(), out=out.cuda(), read=rd.cuda(),
                    norm_weight=w.cuda(), eps=1e-5, h=h3, row_index=rows)
    assert torch.equal(xd3.cpu(), x)
    assert torch.allclose(h3.cpu().double(), want_h[[5, 2, 5]], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("pairing", ["interleaved", "halves"])
@pytest.mark.parametrize("rot", [{"base": 1e4, "dims": 8}, {"base": 5e5, "dims": 24},
                                 {"base": 1e4, "dims": 16, "scaling": {"factor": 8.0, "original": 64, "fast": 4.0, "slow": 0.5}}])
def test_rotation_and_cache_write(ops, pairing, rot):
    """Rotation of part of a head in either pairing, with rescaled frequencies; keys land in their page slots."""
    from tffinfer_b200.parts.position import ScaledRotary
    nq, nkv, d, dv, page = 3, 1, 24, 10, 4
    b = fake_batch([5, 1, 7], [0, 1203, 30], "cuda", page)
    T = b.num_tokens
    g = torch.Generator().manual_seed(3)
    proj = torch.randn(T, (nq + nkv) * d + nkv * dv + nq + 3, generator=g)
    part = ScaledRotary(rot["dims"], rot["base"], pairing, tuple(rot["scaling"][k] for k in ("factor", "original", "fast", "slow"))
                        if "scaling" in rot else None)
    part.prepare(ops, "cuda", 0)
    cache = torch.full((b.pages, 1, 2, nkv, page, d), float("nan"), device="cuda")
    q = torch.empty(T, nq * d, device="cuda")
    gates = torch.empty(T, nq, device="cuda")
    ops.qkv_finish(proj.cuda(), q, None, part.frequencies(), b, b.block_table, cache, 0, page, nq, nkv, d, dv,
                   gate_off=(nq + nkv) * d + nkv * dv, gate_out=gates)
    pos = b.positions.cpu()
    wq = P.rotate(proj[:, :nq * d].double().view(T, nq, d), pos, rot, pairing == "interleaved")
    wk = P.rotate(proj[:, nq * d:(nq + nkv) * d].double().view(T, nkv, d), pos, rot, pairing == "interleaved")
    assert torch.allclose(q.cpu().double().view(T, nq, d), wq, rtol=1e-4, atol=2e-4)     # float32 angles near 1200 rad
    table = b.block_table.cpu()
    for t in range(T):
        pg = int(table[int(b.tok_req[t]), int(pos[t]) // page])
        assert torch.allclose(cache[pg, 0, 0, :, int(pos[t]) % page].cpu().double(), wk[t], rtol=1e-4, atol=2e-4)
        assert torch.allclose(cache[pg, 0, 1, 0, int(pos[t]) % page, :dv].cpu(), proj[t, (nq + nkv) * d:(nq + nkv) * d + dv])
    assert torch.allclose(gates.cpu(), torch.sigmoid(proj[:, (nq + nkv) * d + nkv * dv:][:, :nq]), atol=1e-6)


def _attention_case(ops, dtype, window, softcap, lens, starts, aim):
    """One kv head; the query of the last token of request 0 is aimed at the key ``aim`` positions back with a
    score that dwarfs all others, so its output is that key's value if the key is seen, and far from it if not."""
    nq, nkv, d, dv, page = 2, 1, 64, 64, 16
    total = [s + n for n, s in zip(lens, starts)]
    g = torch.Generator().manual_seed(window + (aim or 0))
    keys = [torch.randn(n, nkv, d, generator=g) for n in total]
    vals = [torch.randn(n, nkv, dv, generator=g) for n in total]
    qs = [torch.randn(n, nq, d, generator=g) for n in total]
    if aim is not None:
        qs[0][-1] = 6.0 * keys[0][total[0] - 1 - aim, 0] / keys[0][total[0] - 1 - aim, 0].norm()
        keys[0][total[0] - 1 - aim, 0] *= 6.0 / keys[0][total[0] - 1 - aim, 0].norm()
    b = fake_batch(lens, starts, "cuda", page)
    cache = torch.full((b.pages + 1, 1, 2, nkv, page, d), float("nan"), dtype=dtype, device="cuda")
    table = b.block_table.cpu()
    for r, n in enumerate(total):
        for p in range(n):
            pg = int(table[r, p // page])
            cache[pg, 0, 0, :, p % page] = keys[r][p].to(dtype)
            cache[pg, 0, 1, :, p % page] = vals[r][p].to(dtype)
    q = torch.cat([qs[r][starts[r]:] for r in range(len(lens))]).reshape(-1, nq * d).to(dtype).cuda()
    gates = torch.rand(q.shape[0], nq, generator=g)
    out = torch.empty(q.shape[0], nq * dv, dtype=dtype, device="cuda")
    ops.attention_ext(q, b, b.block_table, cache, 0, page, out, nq, nkv, d, dv, 1.0, window, softcap, True, gates.cuda())
    want = []
    for r in range(len(lens)):
        rd = lambda t: t.to(dtype).double()
        o = P.windowed_sink_attention(rd(qs[r]), rd(keys[r]), rd(vals[r]), 1.0, softcap, window)
        want.append(o[starts[r]:])
    want = torch.cat(want) * gates.double()[:, :, None]
    return out.float().cpu().double().view(-1, nq, dv), want


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("lens,starts", [([40, 3], [60, 0]), ([1, 1], [99, 17]), ([300, 2], [0, 500])])
def test_attention_window_edges_cap_and_sink(ops, dtype, lens, starts):
    """A key just inside the window and a key just outside it, in a prompt's portion and for a decoded token, also
    with the window's edge on a page border; the cap flattens the aimed score, the sink takes its share."""
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for window in (16, 23, 64):
        for aim in (window - 1, window, 0):
            for softcap in (0.0, 5.0):
                got, want = _attention_case(ops, dtype, window, softcap, lens, starts, aim)
                assert torch.allclose(got, want, rtol=tol, atol=tol), (window, aim, softcap, float((got - want).abs().max()))
    # the first tokens of a sequence: the sink is most of the denominator there
    got, want = _attention_case(ops, dtype, 8, 0.0, [3, 1], [0, 0], None)
    assert torch.allclose(got, want, rtol=tol, atol=tol)


@pytest.mark.parametrize("H,d,dv", [(2, 64, 32), (1, 12, 28), (3, 128, 128), (1, 256, 64), (1, 16, 320), (1, 256, 256)])
def test_retention_steps_chunks_and_far_keys(ops, H, d, dv):
    """The recurrence token by token and chunk by chunk against the plain loop: requests at different places of
    their sequences, states in slots out of order, one far key that a slow decay must still carry."""
    g = torch.Generator().manual_seed(d)
    decay = [0.999, 0.9, 0.97][:H]
    n0, n1 = 170, 45
    q = [torch.randn(n, H, d, generator=g) for n in (n0, n1)]
    k = [torch.randn(n, H, d, generator=g) * d ** -0.5 for n in (n0, n1)]
    v = [torch.randn(n, H, dv, generator=g) for n in (n0, n1)]
    k[0][3, 0] *= 40.0                                    # a far key that dominates head 0's state
    q[0][-1, 0] = k[0][3, 0] / k[0][3, 0].norm() * 3
    gate = [torch.randn(n, H * dv, generator=g) for n in (n0, n1)]
    want = [P.rms(P.retention_recurrence(q[r].double(), k[r].double(), v[r].double(), decay), 1e-6).reshape(-1, H * dv)
            * (gate[r].double() / (1 + torch.exp(-gate[r].double()))) for r in range(2)]
    dec = torch.tensor(decay, dtype=torch.float32, device="cuda")
    state = torch.full((5, H, d, dv), float("nan"), device="cuda")
    slots = [3, 1]
    got = [torch.empty(n, H * dv) for n in (n0, n1)]
    done = [0, 0]
    for lens in ([70, 2], [1, 1], [1, 1], [33, 40], [45, 1], [0, 0]):
        lens = [min(l, n - c) for l, n, c in zip(lens, (n0, n1), done)]
        if lens == [0, 0]:
            lens = [n0 - done[0], n1 - done[1]]
        live = [r for r in range(2) if lens[r] > 0]
        b = fake_batch([lens[r] for r in live], [done[r] for r in live], "cuda", 16, slots=[slots[r] for r in live])
        ops.reset_state_slots(state, b.slots, b.pos_start)
        cat = lambda xs: torch.cat([xs[r][done[r]:done[r] + lens[r]] for r in live])
        qq, kk = cat(q).reshape(-1, H * d).cuda(), cat(k).reshape(-1, H * d).cuda()
        vg = torch.cat([cat(v).reshape(-1, H * dv), cat(gate)], dim=1).cuda()
        out = torch.empty(qq.shape[0], H * dv, device="cuda")
        ops.retention(qq, kk, vg, 0, H * dv, state, b, dec, out, H, d, dv, 1e-6)
        row = 0
        for r in live:
            got[r][done[r]:done[r] + lens[r]] = out[row:row + lens[r]].cpu()
            row += lens[r]
            done[r] += lens[r]
    for r in range(2):
        assert torch.allclose(got[r].double(), want[r], rtol=2e-4, atol=2e-4), float((got[r].double() - want[r]).abs().max())


def test_gelu_gate(ops):
    g = torch.Generator().manual_seed(1)
    gu = torch.randn(5, 2 * 70, generator=g) * 3
    out = torch.empty(5, 70, device="cuda")
    ops.gated_act(gu.cuda(), out, 0, "gelu_tanh")
    want = P.gelu_tanh(gu[:, :70].double()) * gu[:, 70:].double()
    assert torch.allclose(out.cpu().double(), want, rtol=1e-5, atol=1e-6)


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
    """bin/trace_run on a Tipezen folder written by the random-weights mode: a mixed schedule (portions beside single
    tokens, four live requests, a pool that makes later requests reuse pages and slots) in both number formats."""
    import numpy as np
    from test_trace_run_gpu import _replay, _max_tokens
    from helpers import steps_to_jsonl
    from tffinfer_b200.weights import write_random_model
    from tffinfer_b200.weights.safetensors_io import SafetensorsFile
    cfg = config("a")
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
    """Layer orders, sizes and constants drawn at random: which kernels run (tensor-core or FMA products, the head-64/128
    attention kernels or the general one, the chunked retention or the token-by-token one) follows from the sizes."""
    rng = random.Random(seed)
    W = rng.choice([64, 96, 128, 192, 256]) if rng.random() < 0.75 else rng.choice([36, 100, 150])
    S = rng.choice([0, 1, 2, 4, 4, 6, 9])
    n_layers = rng.choice([2, 3, 4, 6])
    a_heads = rng.choice([1, 2, 4, 8])
    a_kv = rng.choice([h for h in (1, 2, 4, 8) if a_heads % h == 0])
    a_dim = rng.choice([16, 32, 64, 64, 128, 48])
    a_vdim = a_dim if rng.random() < 0.6 else rng.choice([16, 32, 64, 96])
    rot_a = RotaryConfig(rng.choice([1e4, 5e5]), rng.choice([d for d in (8, 16, 32, 64, 128) if d <= a_dim]),
                         rng.choice([None, (rng.choice([2.0, 6.0, 32.0]), rng.choice([64.0, 1024.0, 4096.0]),
                                            rng.choice([16.0, 24.0]), rng.choice([1.0, 2.0]))]))
    window = rng.choice([5, 16, 33, 64, 100])
    softcap = rng.choice([0.0, 10.0, 25.0, 50.0])
    scale = rng.choice([a_dim ** -0.5, 0.11, 0.2])
    r_heads = rng.choice([1, 2, 3, 4])
    r_dim = rng.choice([16, 32, 64, 128, 24])
    r_vdim = rng.choice([16, 32, 64, 128, 40])
    rot_r = rng.choice([None, RotaryConfig(rng.choice([1e4, 1e6]), rng.choice([d for d in (8, 16, 24, 32, 64, 128) if d <= r_dim]))])
    layers = []
    for i in range(n_layers):
        ff = rng.choice([0, 64, 128, 192, 100])
        if rng.random() < 0.5:
            layers.append(att(a_heads, a_kv, a_dim, a_vdim, window, rot_a, v_mix=rng.random() < 0.7, softcap=softcap,
                              scale=scale, ff=ff))
        else:
            layers.append(ret(r_heads, r_dim, r_vdim, [1.0 - 2.0 ** -rng.uniform(2, 10) for _ in range(r_heads)], rot_r, ff=ff))
    cfg = TipezenConfig("Tipezen", vocab_size=rng.choice([97, 256, 311, 1000]), hidden_size=W, streams=S,
                        norm_eps=rng.choice([1e-6, 1e-5]), layers=tuple(layers))
    return cfg, rng.choice([8, 16, 32]), [rng.randint(1, 40), rng.randint(60, 200), rng.randint(2, 330), rng.randint(20, 90)]


@pytest.mark.parametrize("seed", list(range(1, 25)))
def test_random_configuration_matches_plain(seed):
    cfg, page, prompts = draw(seed)
    sd = weights(cfg, seed=seed, sharp=3.0)
    rng = random.Random(50 + seed)
    reqs = {f"r{i}": [rng.randrange(cfg.vocab_size) for _ in range(n + 5)] for i, n in enumerate(prompts)}
    cj = cfg.to_json_dict()
    want = {r: P.forward(cj, sd, t) for r, t in reqs.items()}
    # Random hyper-connections can make a position ill-conditioned (streams that nearly cancel in a read).  The bar of a
    # position is therefore the usual one or, where that is larger, four times what rounding alone does to the plain
    # implementation there: run in float32 throughout, or with every sublayer's input rounded to bfloat16.
    rel = lambda a, b: ((a.double() - b).abs() / b.abs().amax(-1, keepdim=True)).amax(-1)
    bar = {"float32": {r: (4 * rel(P.forward(cj, sd, t, dtype=torch.float32), want[r])).clamp_min(TOL["float32"])
                       for r, t in reqs.items()},
           "bfloat16": {r: (4 * rel(P.forward(cj, sd, t, round_inputs=True), want[r])).clamp_min(TOL["bfloat16"])
                        for r, t in reqs.items()}}
    most = max(-(-len(t) // page) * page for t in reqs.values())
    pool = most + most // 2
    for dtype in ("float32", "bfloat16"):
        for steps, tokens in ((trace_mixed(reqs, prompts, max_live=3, page_size=page, pool_tokens=pool, chunk=48), pool),
                              (trace_portions(reqs, sizes=(64, 2, 17, 130, 3)), most)):
            got = run_trace(runner_of(cfg, sd, dtype, page, tokens, live=3), reqs, steps, poison=True)
            for q in reqs:
                err = torch.nan_to_num(rel(got[q], want[q]), nan=float("inf"))
                bad = (err > bar[dtype][q]).nonzero()
                assert bad.numel() == 0, (f"draw {seed} {dtype}: request {q} token {int(bad[0])} off by "
                                          f"{float(err[int(bad[0])]):.3g} (bar {float(bar[dtype][q][int(bad[0])]):.3g}): {cj}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_graph_replay(dtype):
    """Two requests decoded for 300 tokens, one token a step, the steps replayed as CUDA graphs: the windows pass over
    decoded tokens many times, pages are given back behind them, and the retention state is carried all the way."""
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
