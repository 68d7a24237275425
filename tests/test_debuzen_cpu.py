"""CPU suite of the Debuzen family: the config reader, the registry, and the NumPy statement of the design against
hand-made cases (grouped norm, rotation layouts, window and kept tokens, sink, sigmoid weights, convolution, the three
recurrences) and against itself (carried state against closed forms)."""
import json

import numpy as np
import pytest

from llama3_np_b200.debuzen import DEFAULT_RANK, stack_config
from llama3_np_b200.stack import ATTN_SIGMOID, ATTN_SINK, GATED_DELTA, GLA, SSD, WINDOW
from oracle import ref_debuzen as R

CFG = {
    "architecture": "Debuzen", "vocab": 53, "width": 40, "norm": {"eps": 1e-4, "groups": 5}, "logit_softcap": 9.0,
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        {"type": "gla", "mixer": {"heads": 2, "dim": 8, "vdim": 12, "tau": 4.0}, "mlp": None},
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 24},
         "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.3, "mask": {"size": 7, "keep_first": 2},
                            "rot": {"base": 777.0, "dims": 4}},
                   "left_scale": 0.75, "right_scale": 1.5,
                   "right": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "conv": 3}}},
        {"type": "parallel_2", "mlp": {"kind": "dense", "ff": 16},
         "mixer": {"left": {"heads": 3, "kv_heads": 3, "dim": 16, "vdim": 4, "scale": 0.2, "mask": {"size": 5},
                            "rot": {"base": 100.0, "dims": 16}},
                   "left_scale": 1.25, "right_scale": 0.5,
                   "right": {"heads": 4, "groups": 2, "state": 8, "vdim": 6, "conv": 2, "norm_groups": 3}}},
    ],
}


def test_config_reader_takes_every_size_from_the_config_or_the_tensors():
    shapes = {k: np.shape(v) for k, v in R.random_tensors(CFG, 1).items()}
    shapes["l0.mix.a1"] = (5, 40)
    shapes["l1.mix.right.a1"], shapes["l1.mix.right.g1"] = (7, 40), (3, 40)
    sc = stack_config(CFG, shapes, max_seq_len=77, max_batch_size=3, dtype="bfloat16")
    assert (sc.width, sc.vocab, sc.max_seq_len, sc.max_batch_size, sc.dtype) == (40, 53, 77, 3, "bfloat16")
    assert sc.norm_input and sc.token_shift and sc.embed_norm and sc.loop_in and not sc.norm_one_plus and not sc.norm_scalar
    assert sc.norm_eps == pytest.approx(1e-4) and sc.norm_groups == 5 and sc.loop == (1, 3, 3) and sc.glu_act == "silu"
    assert sc.logit_softcap == pytest.approx(9.0)
    g, p1, p2 = sc.layers
    assert (g.mixer, g.heads, g.dim, g.vdim, g.rank_decay, g.ff, g.pair) == (GLA, 2, 8, 12, 5, 0, None) and g.tau == pytest.approx(4.0)
    assert (p1.mixer, p1.heads, p1.kv_heads, p1.dim, p1.vdim, p1.window, p1.keep_first, p1.rot_dims, p1.rot_layout) == (WINDOW, 4, 2, 8, 12, 7, 2, 4, 0)
    assert p1.attn_kind == ATTN_SIGMOID and p1.qk_unit and p1.ff == 24 and p1.rot_base == pytest.approx(777.0) and p1.scale == pytest.approx(0.3)
    assert (p1.mix_scale, p1.pair_scale) == (pytest.approx(0.75), pytest.approx(1.5))
    r = p1.pair
    assert (r.mixer, r.heads, r.kv_heads, r.dim, r.vdim, r.conv_taps, r.rank_decay, r.rank_gate) == (GATED_DELTA, 4, 2, 8, 6, 3, 7, 3)
    assert (p2.mixer, p2.heads, p2.kv_heads, p2.dim, p2.vdim, p2.window, p2.keep_first, p2.rot_dims, p2.rot_layout) == (WINDOW, 3, 3, 16, 4, 5, 0, 16, 1)
    assert p2.attn_kind == ATTN_SINK and not p2.qk_unit and p2.ff == 16
    r = p2.pair
    assert (r.mixer, r.heads, r.kv_heads, r.dim, r.vdim, r.conv_taps, r.out_norm_groups) == (SSD, 4, 2, 8, 6, 2, 3)
    # no tensors at hand (random weights): the inner widths fall back to the configuration or the default
    sc = stack_config(CFG)
    assert sc.layers[0].rank_decay == DEFAULT_RANK and sc.layers[1].pair.rank_gate == DEFAULT_RANK
    plain = json.loads(json.dumps(CFG))
    del plain["loop"]
    del plain["logit_softcap"]
    del plain["norm"]["groups"]
    sc = stack_config(plain)
    assert sc.loop is None and not sc.loop_in and sc.logit_softcap == 0.0 and sc.norm_groups == 1
    bad = json.loads(json.dumps(CFG))
    bad["layers"][1]["type"] = "hyena"
    with pytest.raises(ValueError):
        stack_config(bad)
    bad = json.loads(json.dumps(CFG))
    bad["layers"][1]["mlp"]["kind"] = "moe"
    with pytest.raises(ValueError):
        stack_config(bad)


def test_registry_knows_the_architecture():
    from llama3_np_b200.models import ARCHITECTURES
    assert "Debuzen" in ARCHITECTURES


def test_grouped_norm():
    x = np.array([3.0, 4.0, 0.0, 0.0, 1.0, 1.0])
    w = np.array([1.0, 2.0, 1.0, 1.0, 1.0, -1.0])
    y = R.group_rms_norm(x, w, 3, 0.0 + 1e-12)
    assert np.allclose(y[:2], [3 / np.sqrt(12.5), 2 * 4 / np.sqrt(12.5)])
    assert np.allclose(y[2:4], 0.0) and np.allclose(y[4:], [1.0, -1.0])
    assert np.allclose(R.group_rms_norm(x, w, 1, 0.0), x / np.sqrt((x * x).mean()) * w)


def test_rotation_layouts_and_partial_rotation():
    x = np.arange(1.0, 9.0)[None]
    for layout, pairs in (("pairs", [(0, 1), (2, 3)]), ("halves", [(0, 2), (1, 3)])):
        y = R.rotate(x, 3, 4, 100.0, layout)
        assert np.array_equal(y[0, 4:], x[0, 4:])  # entries past `dims` pass unchanged
        for i, (a, b) in enumerate(pairs):
            ang = 3 * 100.0 ** (-2.0 * i / 4)
            assert y[0, a] == pytest.approx(x[0, a] * np.cos(ang) - x[0, b] * np.sin(ang))
            assert y[0, b] == pytest.approx(x[0, b] * np.cos(ang) + x[0, a] * np.sin(ang))
    assert np.array_equal(R.rotate(x, 5, 0, 10.0, "pairs"), x)
    # scores depend on the distance only
    q, k = np.random.default_rng(0).standard_normal((2, 1, 8))
    for layout in ("pairs", "halves"):
        a = R.rotate(q, 17, 8, 50.0, layout)[0] @ R.rotate(k, 11, 8, 50.0, layout)[0]
        b = R.rotate(q, 106, 8, 50.0, layout)[0] @ R.rotate(k, 100, 8, 50.0, layout)[0]
        assert a == pytest.approx(b)


def test_window_and_kept_tokens():
    vis = [j for j in range(21) if R.visible(20, j, 5, 3)]
    assert vis == [0, 1, 2, 16, 17, 18, 19, 20]
    assert [j for j in range(4) if R.visible(3, j, 5, 3)] == [0, 1, 2, 3]
    assert [j for j in range(11) if R.visible(10, j, 1, 0)] == [10]


def test_sink_takes_its_share_and_sigmoid_weights_do_not_sum_to_one():
    keys = [np.zeros((1, 2)) for _ in range(4)]           # all scores 0
    vals = [np.full((1, 1), float(j + 1)) for j in range(4)]
    q = np.ones((1, 2))
    o = R.window_attention(q, keys, vals, 3, scale=1.0, size=4, keep_first=0, kind="sink", extra=np.array([np.log(4.0)]))
    assert o[0, 0] == pytest.approx((1 + 2 + 3 + 4) / 8.0)   # the sink holds half of the mass and has no value
    o = R.window_attention(q, keys, vals, 3, scale=1.0, size=2, keep_first=1, kind="sigmoid", extra=np.array([0.0]))
    assert o[0, 0] == pytest.approx(0.5 * (1 + 3 + 4))       # keys 0 (kept), 2, 3; each weighs sigmoid(0)


def test_convolution_step_carries_its_tail():
    w = np.array([[1.0, 10.0, 100.0]])
    tail = np.zeros((1, 2))
    outs = []
    for x in (1.0, 2.0, 3.0, 4.0):
        y, tail = R.causal_conv(np.array([x]), tail, w, np.array([0.5]))
        outs.append(y[0])
    assert outs == [100.5, 210.5, 321.5, 432.5]


def test_recurrences_against_closed_forms():
    rng = np.random.default_rng(1)
    q, k = rng.standard_normal((2, 6, 4))
    v = rng.standard_normal((6, 3))
    g = rng.uniform(0.5, 1.0, (6, 4))
    S = np.zeros((4, 3))
    for t in range(6):
        S, o = R.decay_outer_step(S, q[t], k[t], v[t], g[t])
    want = sum(np.outer(np.prod(g[j + 1:], axis=0) * k[j], v[j]) for j in range(6))
    assert np.allclose(S, want) and np.allclose(o, want.T @ q[5])
    S2 = np.zeros((4, 3))
    for t in range(6):
        S2, _ = R.decay_outer_step(S2, q[t], k[t], v[t], 0.9)
    assert np.allclose(S2, sum(0.9 ** (5 - j) * np.outer(k[j], v[j]) for j in range(6)))
    # delta rule: with beta = 1 and a unit key the state returns exactly v for that key right after the write
    kk = R.unit(k[0], 0.0)
    S3, _ = R.delta_step(rng.standard_normal((4, 3)), q[0], kk, v[0], np.ones(4), 1.0)
    assert np.allclose(S3.T @ kk, v[0])


def test_whole_run_equals_steps_and_the_loop_order():
    t = R.random_tensors(CFG, 2)
    o = R.Debuzen(CFG, t)
    assert [i for i, _ in o.runs] == [0, 1, 2, 1, 2, 1, 2] and [f for _, f in o.runs] == [False, True, False, True, False, True, False]
    ids = np.random.default_rng(3).integers(0, 53, 15)
    lg, res = o.run(ids, want_residual=True)
    assert lg.shape == (15, 53) and res.shape == (7, 15, 40) and np.isfinite(lg).all()
    assert np.abs(lg).max() < 9.0   # the cap
    o.reset()
    again = np.stack([o.step(int(x)) for x in ids])
    assert np.array_equal(lg, again)
    for k, a in t.items():           # a bfloat16 checkpoint holds these values exactly
        assert not (a.view(np.uint32) & 0xFFFF).any(), k
