"""Host side of the Dominex design (no GPU): configuration round trip, defaults and errors; the description's tensor
names, cache needs and schedule; and the plain implementation against itself (a recurrence run in two halves, the
per-head keys against the absorbed form, a routed feed-forward with every expert chosen against a dense sum)."""
import copy

import pytest
import torch

import plain_dominex as P
from tffinfer_b200.config import DominexConfig, ConfigError
from tffinfer_b200.parts import Model, KVNeed, StateNeed
from tffinfer_b200.registry import get_architecture
import tffinfer_b200.models  # noqa: F401


def sample_json():
    moe = {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 5, "top": 2}}
    latent = {"heads": 3, "dim": 20, "rot_dim": 6, "vdim": 12, "q_rank": 10, "kv_rank": 18, "scale": 0.2,
              "rot": {"base": 1000.0, "dims": 4}}
    par = {"left": {"heads": 6, "kv_heads": 2, "dim": 24, "vdim": 40, "scale": 0.3, "mask": {"size": 7}},
           "right": {"width": 30}, "left_scale": 0.75, "right_scale": 0.5}
    return {"architecture": "Dominex", "vocab": 97, "width": 52, "embedding": {"scale": 2.5}, "norm": {"eps": 3e-6},
            "logit_softcap": 12.0,
            "layers": [{"type": "parallel", "mixer": par, "mlp": None},
                       {"type": "latent_attention", "mixer": latent, "mlp": moe},
                       {"type": "latent_attention", "mixer": dict(latent, kv_from=1), "mlp": moe}]}


def test_round_trip_and_defaults():
    cj = sample_json()
    cfg = DominexConfig.from_json_dict(cj)
    assert cfg.to_json_dict() == cj
    assert cfg.layers[2].kv_from == 1 and cfg.layers[0].left_chunk == 7 and cfg.layers[1].rot_dims == 4
    d = copy.deepcopy(cj)
    del d["embedding"], d["logit_softcap"], d["layers"][0]["mixer"]["left"]["mask"], d["layers"][0]["mixer"]["left_scale"]
    del d["layers"][0]["mixer"]["left"]["kv_heads"], d["layers"][1]["mixer"]["rot"]["dims"]
    d["layers"][2]["mixer"]["rot"] = {"base": 1000.0}
    c2 = DominexConfig.from_json_dict(d)
    assert c2.embed_scale == 1.0 and c2.logit_softcap == 0.0 and c2.layers[0].left_chunk == 0
    assert c2.layers[0].left_scale == 1.0 and c2.layers[0].left_kv_heads == 6 and c2.layers[1].rot_dims == 6


@pytest.mark.parametrize("edit,word", [
    (lambda d: d["layers"][1].__setitem__("type", "convolution"), "type"),
    (lambda d: d["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][2]["mixer"].__setitem__("kv_from", 0), "kv_from"),
    (lambda d: d["layers"][2]["mixer"].__setitem__("kv_from", 2), "kv_from"),
    (lambda d: d["layers"][2]["mixer"].__setitem__("kv_rank", 20), "equal"),
    (lambda d: d["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 4), "kv_heads"),
    (lambda d: d["layers"][1]["mlp"]["router"].__setitem__("top", 6), "top"),
    (lambda d: d["layers"][1]["mlp"].__setitem__("kind", "dense"), "kind"),
    (lambda d: d["layers"][1]["mixer"]["rot"].__setitem__("dims", 5), "dims"),
    (lambda d: d.pop("norm"), "norm"),
])
def test_errors_name_the_key(edit, word):
    d = sample_json()
    edit(d)
    with pytest.raises(ConfigError) as e:
        DominexConfig.from_json_dict(d)
    assert word in str(e.value)


def test_description_names_needs_and_schedule():
    cfg = DominexConfig.from_json_dict(sample_json())
    desc = get_architecture("Dominex").describe(cfg)
    m = Model(desc)
    names = set(m.expected_tensors())
    for n in ("embed", "final.norm", "l0.norm1", "l0.mix.left.q", "l0.mix.left.temp", "l0.mix.left.r1", "l0.mix.left.r2",
              "l0.mix.right.z", "l0.mix.right.z.b", "l0.mix.right.x.b", "l0.mix.right.g", "l0.mix.right.o",
              "l1.mix.dq", "l1.mix.dq.norm", "l1.mix.uq", "l1.mix.dkv", "l1.mix.dkv.norm", "l1.mix.uk", "l1.mix.uv",
              "l1.mix.o", "l1.norm2", "l1.mlp.router", "l1.mlp.e4.down", "l2.mix.uk"):
        assert n in names, n
    assert "l2.mix.dkv" not in names and "l0.norm2" not in names and "l1.mlp.e5.gate" not in names
    needs = m.cache_needs()
    assert needs[0] == (KVNeed(2, 40, 7), StateNeed((30,), "float32"))
    assert needs[1] == KVNeed(1, 24, 0, planes=1) and needs[2] is None
    assert [e.cache_of for e in desc.schedule] == [None, None, 1]
    assert desc.lm_head_name is None and desc.embed_scale == 2.5 and desc.logit_softcap == 12.0


def test_recurrence_in_two_halves():
    g = torch.Generator().manual_seed(1)
    w, W = 9, 14
    h = torch.randn(20, W, generator=g, dtype=torch.float64)
    m = [torch.randn(w, W, generator=g, dtype=torch.float64) for _ in range(3)]
    b = [torch.randn(w, generator=g, dtype=torch.float64) for _ in range(2)]
    wo = torch.randn(W, w, generator=g, dtype=torch.float64)
    whole, S = P.min_gru(h, m[0], b[0], m[1], b[1], m[2], wo)
    first, S1 = P.min_gru(h[:7], m[0], b[0], m[1], b[1], m[2], wo)
    second, S2 = P.min_gru(h[7:], m[0], b[0], m[1], b[1], m[2], wo, state=S1)
    assert torch.allclose(torch.cat([first, second]), whole, atol=1e-12) and torch.allclose(S2, S, atol=1e-12)
    # the candidate is continuous at zero and positive
    u = torch.tensor([-1e-9, 0.0, 1e-9], dtype=torch.float64)
    c = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    assert float((c - 0.5).abs().max()) < 1e-8


def test_absorbed_keys_equal_per_head_keys():
    """(W_uk c) . q = c . (W_uk^T q): the form the engine computes gives the scores of the per-head keys."""
    g = torch.Generator().manual_seed(2)
    H, dim, kr = 3, 5, 7
    wuk = torch.randn(H * dim, kr, generator=g, dtype=torch.float64)
    c = torch.randn(11, kr, generator=g, dtype=torch.float64)
    q = torch.randn(4, H, dim, generator=g, dtype=torch.float64)
    k = (c @ wuk.T).reshape(11, H, dim)
    direct = torch.einsum("thd,nhd->thn", q, k)
    absorbed = torch.einsum("thr,nr->thn", torch.einsum("thd,hdr->thr", q, wuk.reshape(H, dim, kr)), c)
    assert torch.allclose(direct, absorbed, atol=1e-12)


def test_every_expert_chosen_is_a_dense_sum():
    g = torch.Generator().manual_seed(3)
    E, W, ff = 4, 6, 5
    h = torch.randn(8, W, generator=g, dtype=torch.float64)
    wr = torch.randn(E, W, generator=g, dtype=torch.float64)
    ex = [{"gate": torch.randn(ff, W, generator=g, dtype=torch.float64), "up": torch.randn(ff, W, generator=g, dtype=torch.float64),
           "down": torch.randn(W, ff, generator=g, dtype=torch.float64)} for _ in range(E)]
    got = P.routed_experts(h, wr, ex, E)
    s = torch.sigmoid(h @ wr.T)
    want = sum((P.silu((s[:, e:e + 1] * h) @ ex[e]["gate"].T) * ((s[:, e:e + 1] * h) @ ex[e]["up"].T)) @ ex[e]["down"].T
               for e in range(E))
    assert torch.allclose(got, want, atol=1e-12)
    one = P.routed_experts(h, wr, ex, 1)
    best = s.argmax(dim=1)
    for t in range(8):
        x = s[t, best[t]] * h[t]
        e = ex[int(best[t])]
        assert torch.allclose(one[t], e["down"] @ (P.silu(e["gate"] @ x) * (e["up"] @ x)), atol=1e-12)
