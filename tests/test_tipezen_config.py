"""Host-side tests of the Tipezen design: its configuration reader, its model description (tensor names, cache
and state needs), the rotation frequencies against the plain implementation's, and properties of the plain
implementation itself that the kernels' restatements rest on."""
import json
import math

import pytest
import torch

import plain_tipezen as P
import tffinfer_b200 as tff
from tffinfer_b200.config import (TipezenConfig, TipezenLayer, RotaryConfig, ConfigError, architecture_name,
                                  read_config_json)
from tffinfer_b200.parts import Model, KVNeed, StateNeed
from tffinfer_b200.parts.position import scaled_frequencies
from tffinfer_b200.weights import write_random_model
from tffinfer_b200.weights.safetensors_io import SafetensorsFile


def small_config():
    r = RotaryConfig(1e4, 8, (4.0, 64.0, 8.0, 1.0))
    layers = (TipezenLayer(type="retention", heads=2, dim=8, vdim=4, decay=(0.9, 0.99), rot=RotaryConfig(1e5, 4)),
              TipezenLayer(type="attention", heads=4, kv_heads=2, dim=8, vdim=12, scale=0.25, softcap=15.0, window=7,
                           v_mix=True, rot=r, ff=24),
              TipezenLayer(type="attention", heads=4, kv_heads=2, dim=8, vdim=12, scale=0.25, window=0, v_mix=True, rot=r),
              TipezenLayer(type="attention", heads=2, kv_heads=1, dim=16, vdim=8, scale=0.3, softcap=5.0, window=3, ff=16))
    return TipezenConfig("Tipezen", vocab_size=50, hidden_size=24, streams=3, norm_eps=1e-5, layers=layers)


def test_config_round_trip_and_defaults():
    cfg = small_config()
    d = cfg.to_json_dict()
    assert architecture_name(d) == "Tipezen" and architecture_name({"architectures": ["X"]}) == "X"
    assert TipezenConfig.from_json_dict(json.loads(json.dumps(d))) == cfg
    # optional keys: no streams, no rotation, no mask, no cap, no scale, no kv_heads
    bare = {"architecture": "Tipezen", "vocab": 9, "width": 8, "norm": {"eps": 1e-6},
            "layers": [{"type": "attention", "mixer": {"heads": 2, "dim": 4, "vdim": 4}, "mlp": None}]}
    c = TipezenConfig.from_json_dict(bare)
    l = c.layers[0]
    assert c.streams == 0 and l.kv_heads == 2 and l.window == 0 and l.softcap == 0.0 and l.rot is None
    assert l.scale == pytest.approx(0.5) and l.ff == 0 and not l.v_mix


@pytest.mark.parametrize("change,key", [
    (lambda d: d["layers"][0].update(type="convolution"), "type"),
    (lambda d: d["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
    (lambda d: d["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=10), "dims"),
    (lambda d: d.pop("width"), "width"),
    (lambda d: d["layers"][1]["mlp"].update(kind="routed"), "kind"),
])
def test_config_errors_name_the_key(change, key):
    d = small_config().to_json_dict()
    change(d)
    with pytest.raises(ConfigError) as e:
        TipezenConfig.from_json_dict(d)
    assert key in str(e.value)


def test_description_names_needs_and_groups():
    cfg = small_config()
    arch = tff.get_architecture("Tipezen")
    model = Model(arch.describe(cfg))
    names = model.expected_tensors()
    for n, shape in {"embed": (50, 24), "head": (50, 24), "final.norm": (24,), "l0.mix.g": (8, 24), "l0.mix.o": (24, 8),
                     "l0.hc1.mix": (3, 3), "l0.ls1": (24,), "l1.mix.g": (4, 24), "l1.mix.vmix": (), "l2.mix.vmix": (),
                     "l1.mix.v": (24, 24), "l1.mlp.gate": (24, 24), "l1.hc2.in": (3,), "l3.mix.q": (32, 24)}.items():
        assert tuple(names[n].shape) == shape, n
    assert "l0.norm2" not in names and "l0.hc2.in" not in names and "l2.mlp.up" not in names
    # a layer that mixes no values may carry the scalar or not; a layer that does must
    assert names["l3.mix.vmix"].optional and not names["l1.mix.vmix"].optional and not names["l2.mix.vmix"].optional
    needs = model.cache_needs()
    assert needs[0] == StateNeed((2, 8, 4), "float32")
    assert needs[1] == KVNeed(2, 12, 7) and needs[2] == KVNeed(2, 12, 0) and needs[3] == KVNeed(1, 16, 3)
    modes = [b.mixer.value_mix for b in model.blocks[1:]]
    assert modes == ["source", "mix", "none"]
    # one plain residual: a single stream without learned connections, layer scale kept
    flat = TipezenConfig("Tipezen", vocab_size=50, hidden_size=24, streams=0, norm_eps=1e-5, layers=cfg.layers)
    names = Model(arch.describe(flat)).expected_tensors()
    assert "l0.hc1.in" not in names and "l0.ls1" in names


def test_random_model_folder(tmp_path):
    cfg = small_config()
    d = write_random_model(str(tmp_path / "m"), cfg, seed=3)
    assert TipezenConfig.from_json_dict(read_config_json(d)) == cfg
    f = SafetensorsFile(str(tmp_path / "m" / "model.safetensors"))
    w = {n: f.tensor(n).clone() for n in f.names()}
    assert "l3.mix.vmix" not in w and "l1.mix.vmix" in w
    # the loader's checks: an optional tensor may be there or not, a required one must
    from tffinfer_b200.weights.loader import check_tensors, WeightError
    expected = Model(tff.get_architecture("Tipezen").describe(cfg)).expected_tensors()
    assert "l3.mix.vmix" not in check_tensors(w, expected, torch.float32, "cpu")
    assert "l3.mix.vmix" in check_tensors({**w, "l3.mix.vmix": torch.zeros(())}, expected, torch.float32, "cpu")
    with pytest.raises(WeightError) as e:
        check_tensors({n: t for n, t in w.items() if n != "l2.mix.vmix"}, expected, torch.float32, "cpu")
    assert "l2.mix.vmix" in str(e.value)
    logits, layers = P.forward(cfg.to_json_dict(), w, [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5], return_layers=True)
    assert logits.shape == (11, 50) and layers.shape == (4, 11, 24) and torch.isfinite(logits).all()


@pytest.mark.parametrize("rot", [RotaryConfig(1e4, 64), RotaryConfig(1e6, 32, (16.0, 1024.0, 24.0, 1.0)),
                                 RotaryConfig(500.0, 6, (2.5, 40.0, 3.0, 0.7))])
def test_frequencies_match_the_plain_ones(rot):
    f, mag = scaled_frequencies(rot.dims, rot.base, rot.scaling)
    pf, pmag = P.rotary_frequencies(rot.to_json())
    assert mag == pytest.approx(pmag, rel=1e-15)
    assert torch.allclose(torch.tensor(f, dtype=torch.float64), pf, rtol=1e-14, atol=0)
    if rot.scaling:                       # slow dimensions are divided by the factor, fast ones untouched
        assert f[0] == pytest.approx(1.0) or f[0] == pytest.approx(1.0 / rot.scaling[0])
        assert f[-1] == pytest.approx(rot.base ** (-(rot.dims - 2) / rot.dims) / rot.scaling[0])


def test_chunked_retention_equals_the_recurrence():
    """The chunk form the prompt kernels use, in float64 against the token-by-token loop."""
    g = torch.Generator().manual_seed(0)
    T, d, dv, decay, C = 37, 6, 5, 0.93, 8
    q, k, v = (torch.randn(T, 1, n, generator=g, dtype=torch.float64) for n in (d, d, dv))
    want = P.retention_recurrence(q, k, v, [decay])[:, 0]
    S = torch.zeros(d, dv, dtype=torch.float64)
    got = []
    for t0 in range(0, T, C):
        n = min(C, T - t0)
        qq, kk, vv = q[t0:t0 + n, 0], k[t0:t0 + n, 0], v[t0:t0 + n, 0]
        i = torch.arange(n)
        A = (qq @ kk.t()) * torch.where(i[:, None] >= i[None, :], decay ** (i[:, None] - i[None, :]).double(), 0.0)
        got.append(A @ vv + (decay ** (i + 1).double())[:, None] * (qq @ S))
        S = decay ** n * S + (kk * (decay ** (n - 1 - i).double())[:, None]).t() @ vv
    assert torch.allclose(torch.cat(got), want, rtol=1e-12, atol=1e-12)


def test_sink_and_window_of_the_plain_attention():
    g = torch.Generator().manual_seed(1)
    T = 9
    q, k = torch.randn(T, 2, 4, generator=g, dtype=torch.float64), torch.randn(T, 1, 4, generator=g, dtype=torch.float64)
    ones = torch.ones(T, 1, 1, dtype=torch.float64)
    # with values of one, the output is the weights' sum: below one by the sink's share
    o = P.windowed_sink_attention(q, k, ones, 1.0, 0.0, 3)
    s = (q[5, 0] @ k[3:6, 0].t())
    assert o[5, 0, 0] == pytest.approx(float(torch.exp(s).sum() / (1 + torch.exp(s).sum())))
    capped = P.windowed_sink_attention(q * 50, k, ones, 1.0, 2.0, 0)
    assert float(capped.max()) <= T * math.e ** 2 / (1 + T * math.e ** 2) + 1e-12


def test_one_stream_of_identity_connections_is_the_plain_residual():
    g = torch.Generator().manual_seed(2)
    x, y = torch.randn(1, 5, 7, generator=g, dtype=torch.float64), torch.randn(5, 7, generator=g, dtype=torch.float64)
    one = torch.ones(1, dtype=torch.float64)
    assert torch.equal(P.hyper_read(x, one), x[0])
    assert torch.allclose(P.hyper_write(x, y, torch.ones(1, 1, dtype=torch.float64), one)[0], x[0] + y)
