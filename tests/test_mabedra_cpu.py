"""CPU suite of the Mabedra family: the config reader, the registry, and the NumPy statement of the design against
hand-made cases (frequency scaling, rotation, convolution, router, PolyNorm, window, depth average)."""
import json

import numpy as np
import pytest

from llama3_np_b200.mabedra import stack_config
from llama3_np_b200.stack import DIFF, FF_POLYNORM, ROUTE_SIGMOID_IN
from oracle import ref_mabedra as R

CFG = {
    "architecture": "Mabedra", "vocab": 53, "width": 40, "norm": {"eps": 1e-4}, "canon": {"taps": 3},
    "layers": [
        {"type": "attention",
         "mixer": {"heads": 6, "kv_heads": 3, "dim": 8, "vdim": 12, "diff": 0.4, "scale": 0.25, "mask": {"size": 11},
                   "rot": {"base": 777.0, "dims": 6, "scaling": {"factor": 3.0, "low": 1.5, "high": 5.0, "original": 96}}},
         "mlp": {"kind": "moe", "expert": {"ff": 10}, "router": {"experts": 5, "top": 2}, "shared": {"ff": 14}}},
        {"type": "attention",
         "mixer": {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 16, "diff": 0.1, "scale": 0.5, "rot": {"base": 100.0, "dims": 16}},
         "mlp": {"kind": "dense", "ff": 28}},
        {"type": "attention",
         "mixer": {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 4, "diff": 0.2, "scale": 0.5, "mask": {"size": 2}, "rot": {"base": 100.0, "dims": 2}},
         "mlp": None},
    ],
}


def test_config_reader_takes_every_size_from_the_config():
    sc = stack_config(CFG, max_seq_len=77, max_batch_size=3, dtype="bfloat16")
    assert (sc.width, sc.vocab, sc.max_seq_len, sc.max_batch_size, sc.dtype) == (40, 53, 77, 3, "bfloat16")
    assert sc.parallel and sc.norm_input and sc.norm_center and sc.layer_scale and sc.depth_avg and sc.canon_taps == 3
    assert not sc.norm_one_plus and not sc.norm_scalar and not sc.token_shift and sc.loop is None
    assert sc.norm_eps == pytest.approx(1e-4)
    a, b, c = sc.layers
    assert (a.mixer, a.heads, a.kv_heads, a.dim, a.vdim, a.window, a.rot_dims) == (DIFF, 6, 3, 8, 12, 11, 6)
    assert a.diff == pytest.approx(0.4) and a.scale == pytest.approx(0.25) and a.rot_base == pytest.approx(777.0)
    assert a.rot_scaling == (3.0, 1.5, 5.0, 96)
    assert (a.ff, a.experts, a.top, a.router_kind, a.shared_ff) == (10, 5, 2, ROUTE_SIGMOID_IN, 14)
    assert (b.window, b.rot_scaling, b.ff, b.ff_kind, b.experts) == (0, None, 28, FF_POLYNORM, 0)
    assert (c.ff, c.experts, c.window, c.kv_heads) == (0, 0, 2, 1)
    plain = json.loads(json.dumps(CFG))
    del plain["canon"]
    del plain["layers"][0]["mlp"]["shared"]
    sc = stack_config(plain)
    assert sc.canon_taps == 0 and sc.layers[0].shared_ff == 0
    bad = json.loads(json.dumps(CFG))
    bad["layers"][1]["type"] = "hyena"
    with pytest.raises(ValueError):
        stack_config(bad)
    bad = json.loads(json.dumps(CFG))
    bad["layers"][1]["mlp"]["kind"] = "glu"
    with pytest.raises(ValueError):
        stack_config(bad)


def test_registry_knows_the_architecture():
    from llama3_np_b200.models import ARCHITECTURES
    assert "Mabedra" in ARCHITECTURES


def test_frequency_scaling_bands():
    rot = {"base": 10000.0, "dims": 32, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 1024}}
    plain = R.rotary_frequencies({"base": 10000.0, "dims": 32})
    f = R.rotary_frequencies(rot)
    wave = 2 * np.pi / plain
    short, long_ = wave < 1024 / 4.0, wave > 1024 / 1.0
    assert short.any() and long_.any() and (~short & ~long_).any()
    assert np.array_equal(f[short], plain[short])
    assert np.allclose(f[long_], plain[long_] / 8.0)
    mid = ~short & ~long_
    assert np.all(f[mid] < plain[mid]) and np.all(f[mid] > plain[mid] / 8.0)
    # continuous at both ends of the band
    lo = {"base": 1.0, "dims": 2, "scaling": dict(rot["scaling"])}
    for wl, want in ((1024 / 4.0, 1.0), (1024 / 1.0, 1 / 8.0)):
        lo["base"] = 1.0
        fi = 2 * np.pi / wl
        t = (1024 / wl - 1.0) / 3.0
        assert (1 - t) * fi / 8.0 + t * fi == pytest.approx(fi * want)


def test_rotate_half_pairs_entry_i_with_i_plus_half():
    v = np.arange(1.0, 9.0)
    out = R.rotate_half(v, 3, {"base": 100.0, "dims": 4})
    f = np.power(100.0, -2.0 * np.arange(2) / 4)
    for i in range(2):
        c, s = np.cos(3 * f[i]), np.sin(3 * f[i])
        assert out[i] == pytest.approx(v[i] * c - v[i + 2] * s)
        assert out[i + 2] == pytest.approx(v[i + 2] * c + v[i] * s)
    assert np.array_equal(out[4:], v[4:])
    assert np.array_equal(R.rotate_half(v, 0, {"base": 100.0, "dims": 8}), v)


def test_convolution_reads_zeros_ahead_of_the_sequence():
    w = np.array([[1.0, 10.0, 100.0], [2.0, 20.0, 200.0]])
    st = {}
    hs = [np.array([1.0, 1.0]), np.array([2.0, 3.0]), np.array([4.0, 5.0]), np.array([6.0, 7.0])]
    outs = [R.canon(h, w, st, "c") for h in hs]
    assert np.allclose(outs[0], hs[0] + w[:, 2] * hs[0])
    assert np.allclose(outs[1], hs[1] + w[:, 2] * hs[1] + w[:, 1] * hs[0])
    assert np.allclose(outs[3], hs[3] + w[:, 2] * hs[3] + w[:, 1] * hs[2] + w[:, 0] * hs[1])
    one = {}
    assert np.allclose(R.canon(hs[1], w[:, :1], one, "c"), hs[1] * (1 + w[:, 0]))


def test_router_takes_the_largest_scores_ties_to_the_lower_index():
    P = {"mlp.router": np.array([[1.0, 0.0], [3.0, 0.0], [3.0, 0.0], [-2.0, 0.0]])}
    chosen, weights = R.route(np.array([1.0, 5.0]), P, {"top": 2})
    assert chosen == [1, 2] and weights[0] == pytest.approx(1 / (1 + np.exp(-3.0)))
    chosen, weights = R.route(np.array([-1.0, 5.0]), P, {"top": 3})
    assert chosen == [3, 0, 1] and weights[0] == pytest.approx(1 / (1 + np.exp(-2.0)))
    assert sum(weights) != pytest.approx(1.0)  # not renormalised


def test_polynorm():
    z = np.array([1.0, -2.0, 3.0])
    got = R.polynorm(z, (2.0, 3.0, 5.0, 7.0), 0.0)
    n = lambda v: v / np.sqrt(np.mean(v * v))
    assert np.allclose(got, 2 * n(z) + 3 * n(z ** 2) + 5 * n(z ** 3) + 7)


def test_oracle_window_and_depth_average():
    """The oracle against itself: a token beyond every layer's reach does not move the logits; and with the depth average
    set to pass layer results straight on the model is a plain stack of residual layers."""
    cfg = json.loads(json.dumps(CFG))
    del cfg["canon"]
    cfg["layers"] = cfg["layers"][2:]  # one layer, window 2, no feed-forward
    t = R.random_model(cfg, 1)
    o = R.OracleMabedra(cfg, t)
    ids = np.array([3, 9, 4, 7, 1])
    a = o.run(ids)[-1]
    alt = ids.copy(); alt[2] = 8
    o.reset()
    assert np.allclose(o.run(alt)[-1], a)
    alt = ids.copy(); alt[3] = 8
    o.reset()
    assert not np.allclose(o.run(alt)[-1], a)
    t["l0.dwa"] = np.array([0.0, 1.0])
    o = R.OracleMabedra(cfg, t)
    lg, res = o.run(ids, want_residual=True)
    x = t["embed"][ids[0]]
    h = R.layer_norm(x, t["l0.norm1"], 1e-4)
    y = x + t["l0.ls1"] * R.diff_attention_step(h, 0, o.layers[0], cfg["layers"][0]["mixer"], 1e-4, {})
    assert np.allclose(res[0, 0], y)


def test_random_model_names_match_the_config():
    t = R.random_model(CFG, 0)
    assert {"embed", "head", "final.norm", "l0.mlp.shared.down", "l0.mlp.e4.gate", "l1.mlp.act", "l2.dwa", "l0.canon2"} <= set(t)
    assert "l2.ls2" not in t and "l2.canon2" not in t and "l1.mlp.router" not in t
    assert t["l2.dwa"].shape == (4,) and t["l0.mix.q"].shape == (2 * 6 * 8, 40) and t["l0.mix.v.b"].shape == (36,)
