"""Mabedra on the GPU against the plain NumPy statement of the design (oracle/ref_mabedra.py): every mechanism alone,
whole prompts against token-by-token decoding and against portions down to two tokens, batches against single
sequences, reused slots, keys far away and on both sides of a window's edge, the first tokens of a sequence, long
decoding, sizes that make the usual coincidences false (vdim != dim, kv_heads = heads, top > 1, shared width != expert
width, taps 1 .. 5), and greedy generation through the library's own loop and scheduler.  Small random models; fp32
mode is held to 1e-4 of the logit scale, bf16 to 6e-2 (see `close`)."""
import json

import numpy as np
import pytest

from oracle.ref_mabedra import OracleMabedra, random_model

pytestmark = pytest.mark.gpu

FP32_BAR, BF16_BAR = 1e-4, 6e-2


def dense(ff=48):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=24, shared=40):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def attn(heads=4, kv_heads=2, dim=16, vdim=24, window=9, diff=0.25, scale=0.3, base=5000.0, dims=None, scaling=(8.0, 1.0, 4.0, 64),
         mlp=None):
    rot = {"base": base, "dims": dim if dims is None else dims}
    if scaling:
        rot["scaling"] = {"factor": scaling[0], "low": scaling[1], "high": scaling[2], "original": scaling[3]}
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "scale": scale, "rot": rot}
    if window:
        mixer["mask"] = {"size": window}
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def config(layers, width=64, vocab=97, taps=3, eps=1e-5):
    c = {"architecture": "Mabedra", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if taps:
        c["canon"] = {"taps": taps}
    return c


def build(cfg, seed=0, dtype="float32", max_seq_len=128, max_batch_size=1, tensors=None):
    from llama3_np_b200.mabedra import Mabedra
    t = random_model(cfg, seed) if tensors is None else tensors
    return Mabedra(cfg, t, dtype=dtype, max_seq_len=max_seq_len, max_batch_size=max_batch_size), OracleMabedra(cfg, t)


def row_errs(got, want):
    """per row: rms of the mean-free difference over the rms of the mean-free logits"""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return np.sqrt((d * d).mean(-1)) / np.sqrt((w * w).mean())


def err(got, want):
    return float(row_errs(got, want).max())


def close(got, want, dtype):
    """fp32: every row within the bar.  bf16: a router's choice between two nearly equal scores may fall the other
    way for a token once its inputs are rounded, and that token's row then differs by far more than rounding; so
    nine rows in ten are held to the bar and the typical row to a third of it."""
    e = row_errs(got, want)
    if dtype == "float32":
        return bool(e.max() < FP32_BAR)
    return bool(np.quantile(e, 0.9) < BF16_BAR and np.median(e) < BF16_BAR / 3)


def toks(n, vocab, seed=1):
    return np.random.default_rng(seed).integers(0, vocab, n)


def fresh(o):
    o.reset()
    return o


ALONE = {
    "attention_only": dict(layers=[attn()]),
    "attention_no_window_no_scaling": dict(layers=[attn(window=0, scaling=None)]),
    "attention_partial_rotation": dict(layers=[attn(heads=2, kv_heads=2, dim=24, vdim=8, dims=10, base=300.0)]),
    "attention_no_rotation": dict(layers=[attn(dims=0)]),
    "no_convolution": dict(layers=[attn(mlp=dense())], taps=0),
    "one_tap": dict(layers=[attn(mlp=dense())], taps=1),
    "five_taps": dict(layers=[attn(mlp=dense(ff=40))], taps=5),
    "dense_polynorm": dict(layers=[attn(mlp=dense(ff=72))]),
    "experts_top1_no_shared": dict(layers=[attn(mlp=moe(experts=5, top=1, shared=0))]),
    "experts_top3_shared": dict(layers=[attn(mlp=moe(experts=7, top=3, ff=16, shared=56))]),
    "depth_average_over_three": dict(layers=[attn(mlp=dense()), attn(heads=2, kv_heads=1, dim=32, vdim=32), attn(mlp=moe())]),
}


@pytest.mark.parametrize("name", sorted(ALONE))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_each_mechanism_alone(name, dtype):
    cfg = config(**ALONE[name])
    m, o = build(cfg, seed=3, dtype=dtype)
    ids = toks(40, cfg["vocab"])
    got, resid = m.forward_rows(ids[None], 0, list(range(40)), want_residual=True)
    want, wres = o.run(ids, want_residual=True)
    assert resid.shape == (len(cfg["layers"]), 40, cfg["width"])
    assert close(got, want, dtype)
    if dtype == "float32":
        assert np.allclose(resid, wres, rtol=1e-4, atol=1e-4)
    m.close()


MIXED = [attn(mlp=dense()), attn(heads=2, kv_heads=1, dim=32, vdim=16, window=13, mlp=moe()), attn(window=6),
         attn(heads=3, kv_heads=3, dim=8, vdim=40, window=30, dims=4, mlp=moe(experts=4, top=2, ff=32, shared=16))]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_then_token_by_token_and_portions(dtype):
    """The same 70 tokens as one prompt, token by token, and in portions of many sizes (two tokens included, cuts in the
    middle of every window and of the convolutions' reach): the logits of a position do not depend on the cut."""
    cfg = config(MIXED)
    m, o = build(cfg, seed=7, dtype=dtype)
    ids = toks(70, cfg["vocab"], seed=8)
    want = o.run(ids)
    whole = m.forward_rows(ids[None], 0, list(range(70)))
    assert close(whole, want, dtype)
    single = np.stack([m.forward(ids[None, i:i + 1], i)[0] for i in range(70)])
    assert close(single, want, dtype)
    for cuts in ([2, 2, 3, 17, 1, 2, 20, 16, 2, 5], [33, 2, 35], [1, 69], [9] * 7 + [7]):
        assert sum(cuts) == 70
        rows, pos = [], 0
        for c in cuts:
            rows.append(m.forward_rows(ids[None, pos:pos + c], pos, list(range(c))))
            pos += c
        got = np.concatenate(rows)
        assert close(got, want, dtype)
        if dtype == "float32":
            assert err(got, whole) < 2e-5
    m.close()


def test_long_decoding_matches_the_oracle():
    cfg = config(MIXED[:3], width=48)
    m, o = build(cfg, seed=9, max_seq_len=400)
    ids = toks(330, cfg["vocab"], seed=10)
    want = o.run(ids)
    m.forward(ids[None, :5], 0)
    got = np.stack([m.forward(ids[None, i:i + 1], i)[0] for i in range(5, 330)])
    assert err(got, want[5:]) < FP32_BAR
    m.close()


def test_batch_rows_equal_single_sequences_and_slots_are_reused():
    """Three different sequences in one batch against each alone; then the slots start new sequences (position 0) on top
    of what the old ones left - caches, convolution tails - and a shorter batch reuses the first slots."""
    cfg = config(MIXED)
    m, o = build(cfg, seed=11, max_seq_len=64, max_batch_size=3)
    seqs = np.stack([toks(40, cfg["vocab"], seed=s) for s in (12, 13, 14)])
    want = [fresh(o).run(s) for s in seqs]
    last = m.forward(seqs[:, :30], 0)
    for b in range(3):
        assert err(last[b:b + 1], want[b][29:30]) < FP32_BAR
    for i in range(30, 40):
        step = m.forward(seqs[:, i:i + 1], i)
        for b in range(3):
            assert err(step[b:b + 1], want[b][i:i + 1]) < FP32_BAR
    other = np.stack([toks(25, cfg["vocab"], seed=s) for s in (15, 16)])
    wo = [fresh(o).run(s) for s in other]
    got = m.forward_rows(other[:, :11], 0, list(range(22)))
    assert err(got[:11], wo[0][:11]) < FP32_BAR and err(got[11:], wo[1][:11]) < FP32_BAR
    got = m.forward_rows(other[:, 11:], 11, list(range(28)))
    assert err(got[:14], wo[0][11:]) < FP32_BAR and err(got[14:], wo[1][11:]) < FP32_BAR
    m.close()


def _sharp(t, n_layers, gain):
    """Scale the query norm so that the softmax of every map is sharp: single keys carry the output, and a key that is
    wrongly seen or missed changes the logits by far more than rounding."""
    t = dict(t)
    for i in range(n_layers):
        t[f"l{i}.mix.q.norm"] = t[f"l{i}.mix.q.norm"] * gain
    return t


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [0, 64, 65, 200])
def test_sharp_attention_over_long_contexts(window, dtype):
    """300 tokens with sharp attention: far keys (no window), windows that end on and beside a tile border of the prompt
    kernel, prompts and decoded tokens alike."""
    cfg = config([attn(window=window, heads=2, kv_heads=1, dim=32, vdim=64, scale=0.4, mlp=dense()), attn(window=window, dim=16, vdim=24)], taps=2)
    t = _sharp(random_model(cfg, 17), 2, 4.0)
    m, o = build(cfg, dtype=dtype, max_seq_len=320, tensors=t)
    ids = toks(300, cfg["vocab"], seed=18)
    want = o.run(ids)
    got = np.concatenate([m.forward_rows(ids[None, :230], 0, list(range(230))),
                          m.forward_rows(ids[None, 230:260], 230, list(range(30))),
                          np.stack([m.forward(ids[None, i:i + 1], i)[0] for i in range(260, 300)])])
    assert close(got, want, dtype)
    m.close()


@pytest.mark.parametrize("window", [1, 2, 7, 64, 100])
def test_window_edge_exactly(window):
    """One layer without convolutions: the logits at position i depend on token i - window + 1 and not on token
    i - window, in a prompt (tiled kernel and short-portion kernel) and for a decoded token."""
    cfg = config([attn(window=window, dim=32, vdim=32, dims=16)], taps=0, width=32, vocab=50)
    t = _sharp(random_model(cfg, 19), 1, 3.0)
    m, o = build(cfg, max_seq_len=160, tensors=t)
    n = 150
    ids = toks(n, 50, seed=20)
    i = n - 1
    base = m.forward_rows(ids[None], 0, [i])[0]
    assert err(base[None], o.run(ids)[i:i + 1]) < FP32_BAR
    for portion in (n, 8, 1):  # the last `portion` tokens form the call that holds position i
        for back, seen in ((window, False), (window - 1, True)):
            if i - back < 0:
                continue
            alt = ids.copy()
            alt[i - back] = (alt[i - back] + 1) % 50
            if portion < n:
                m.forward(alt[None, :n - portion], 0)
            got = m.forward_rows(alt[None, n - portion:], n - portion, [portion - 1])[0]
            moved = float(np.abs(got - base).max())
            if seen:
                assert moved > 1e-3, (portion, back)
            else:
                assert moved < 1e-5, (portion, back)
    m.close()


@pytest.mark.parametrize("planted", [0, 1, 63, 64, 190])
def test_one_planted_key_is_found_from_everywhere(planted):
    """No window: one token whose keys dominate (a token used nowhere else, queries and that key scaled up) must reach
    every later position; the oracle agrees and the logits differ clearly from the same run without the plant."""
    cfg = config([attn(window=0, dim=16, vdim=16, scaling=None, dims=0)], taps=0, width=32, vocab=60)
    t = _sharp(random_model(cfg, 21), 1, 5.0)
    m, o = build(cfg, max_seq_len=260, tensors=t)
    ids = toks(250, 59, seed=22)
    with_plant = ids.copy()
    with_plant[planted] = 59
    want = o.run(with_plant)
    got = np.concatenate([m.forward_rows(with_plant[None, :200], 0, list(range(200))),
                          np.stack([m.forward(with_plant[None, i:i + 1], i)[0] for i in range(200, 250)])])
    assert err(got, want) < FP32_BAR
    m.close()


def test_first_tokens_of_a_sequence():
    """Positions 0 .. taps: the convolutions read zeros ahead of the sequence, the first token attends to itself alone."""
    cfg = config(MIXED, taps=4)
    m, o = build(cfg, seed=23, max_seq_len=16)
    ids = toks(6, cfg["vocab"], seed=24)
    want = o.run(ids)
    assert err(m.forward_rows(ids[None], 0, list(range(6))), want) < FP32_BAR
    assert err(m.forward_rows(ids[None, :1], 0, [0]), want[:1]) < FP32_BAR
    assert err(m.forward_rows(ids[None, 1:3], 1, [0, 1]), want[1:3]) < FP32_BAR
    assert err(m.forward_rows(ids[None, 3:6], 3, [0, 1, 2]), want[3:6]) < FP32_BAR
    m.close()


def test_router_weight_scales_the_input_not_the_output():
    """A gated unit is not homogeneous of degree one: scaling its input by w differs from scaling its output.  With large
    expert inputs the two readings are far apart; the product must follow the oracle's."""
    cfg = config([attn(mlp=moe(experts=4, top=2, ff=32, shared=0))], width=32, vocab=40)
    t = random_model(cfg, 25)
    for e in range(4):
        t[f"l0.mlp.e{e}.gate"] = t[f"l0.mlp.e{e}.gate"] * 3.0
    m, o = build(cfg, tensors=t)
    ids = toks(30, 40, seed=26)
    want = o.run(ids)
    assert err(m.forward_rows(ids[None], 0, list(range(30))), want) < FP32_BAR
    assert err(np.stack([m.forward(ids[None, i:i + 1], i)[0] for i in range(30)]), want) < FP32_BAR
    m.close()


ODD = {
    "width_36_heads_3": config([attn(heads=3, kv_heads=1, dim=12, vdim=20, mlp=dense(ff=44)), attn(heads=6, kv_heads=2, dim=4, vdim=4, mlp=moe(experts=3, top=3, ff=12, shared=8))],
                               width=36, vocab=31, taps=2),
    "one_head_one_expert": config([attn(heads=1, kv_heads=1, dim=40, vdim=72, window=1, mlp=moe(experts=1, top=1, ff=8, shared=8))], width=40, vocab=19, taps=1),
    "wide_heads": config([attn(heads=2, kv_heads=1, dim=128, vdim=128, window=50, scale=0.09, mlp=dense(ff=200))], width=72, vocab=64, eps=1e-3),
    "tiled_64_128": config([attn(heads=2, kv_heads=2, dim=64, vdim=128, window=40, scale=0.12), attn(heads=4, kv_heads=1, dim=64, vdim=64, window=0, scale=0.12)], width=48, vocab=64),
}


@pytest.mark.parametrize("name", sorted(ODD))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_odd_sizes(name, dtype):
    cfg = ODD[name]
    m, o = build(cfg, seed=27, dtype=dtype)
    ids = toks(60, cfg["vocab"], seed=28)
    want = o.run(ids)
    got = np.concatenate([m.forward_rows(ids[None, :45], 0, list(range(45))), m.forward_rows(ids[None, 45:47], 45, [0, 1]),
                          np.stack([m.forward(ids[None, i:i + 1], i)[0] for i in range(47, 60)])])
    assert close(got, want, dtype)
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_library_loop(dtype):
    cfg = config(MIXED)
    m, o = build(cfg, seed=29, dtype=dtype, max_seq_len=96, max_batch_size=2)
    prompts = np.stack([toks(12, cfg["vocab"], seed=s) for s in (30, 31)])
    lazy = np.concatenate(list(m.generate(prompts, 40)), axis=1)
    bulk = m.generate_all(prompts, 40)
    assert np.array_equal(lazy, bulk)
    # teacher-forced check: every emitted token is the oracle's argmax for the same prefix, unless the oracle's
    # top two are closer than the mode's error bar
    margin = 1e-3 if dtype == "float32" else 0.2
    for b in range(2):
        seq = np.concatenate([prompts[b], bulk[b]])
        lg = fresh(o).run(seq[:-1])
        for i in range(40):
            row = lg[11 + i]
            top = np.sort(row)[-2:]
            if top[1] - top[0] > margin * np.std(row):
                assert int(np.argmax(row)) == int(bulk[b, i]), f"sequence {b}, new token {i}"
    m.close()


def test_scheduler_runs_unequal_prompts_as_each_alone():
    cfg = config(MIXED[:3])
    m, _ = build(cfg, seed=32, max_seq_len=64, max_batch_size=2)
    prompts = [toks(n, cfg["vocab"], seed=33 + n) for n in (5, 9, 5, 2, 9)]
    outs = m.generate_ragged(prompts, 10)
    for p, got in zip(prompts, outs):
        assert np.array_equal(got, m.generate_all(p[None], 10)[0])
    m.close()


def _write_folder(tmp_path, cfg, t):
    from test_risalix_cpu import write_safetensors
    write_safetensors(tmp_path / "model.safetensors", t)
    (tmp_path / "config.json").write_text(json.dumps(cfg))


def test_registry_and_checkpoint_folder(tmp_path):
    from llama3_np_b200.models import load_model
    cfg = config([attn(mlp=moe()), attn(mlp=dense())], width=32, vocab=41)
    t = random_model(cfg, 34)
    _write_folder(tmp_path, cfg, t)
    m = load_model(str(tmp_path), dtype="float32", max_seq_len=32)
    assert type(m).__name__ == "Mabedra"
    ids = toks(16, 41, seed=35)
    assert err(m.forward_rows(ids[None], 0, list(range(16))), OracleMabedra(cfg, t).run(ids)) < FP32_BAR
    m.close()


def test_trace_runner_replays_a_trace(tmp_path):
    """bin/trace_run as a user runs it: two requests after one another through the same slot, portions cut in odd
    places and longer than one forward call."""
    import os
    import subprocess
    import sys
    from conftest import ROOT
    cfg = config([attn(window=5, mlp=moe()), attn(mlp=dense())], width=32, vocab=41)
    t = random_model(cfg, 36)
    _write_folder(tmp_path, cfg, t)
    o = OracleMabedra(cfg, t)
    reqs = {"a": toks(23, 41, seed=37), "b": toks(9, 41, seed=38)}
    want = {k: fresh(o).run(v) for k, v in reqs.items()}
    steps, expect, n = [], {}, 0
    for rid, cuts in (("a", [11, 1, 2, 9]), ("b", [9])):
        pos = 0
        for c in cuts:
            w = [0, c - 1] if c > 1 else [0]
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [int(x) for x in reqs[rid][pos:pos + c]], "want": w}],
                          "end": [rid] if pos + c == len(reqs[rid]) else []})
            expect[n] = want[rid][[pos + i for i in w]]
            pos += c
            n += 1
    steps.append({"step": n, "entries": [], "end": []})
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(tmp_path), "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "64", "--piece", "5"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(n + 1)]
    for i, e in expect.items():
        got = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, 41)
        assert err(got, e) < FP32_BAR, i


def test_larger_shapes_take_the_tensor_core_projections():
    """Width 256 and 150 rows: in bf16 mode the projections of a portion run as tcgen05 GEMMs, the experts as one
    masked GEMM over all of them; decode rows read only the chosen experts."""
    cfg = config([attn(heads=4, kv_heads=2, dim=64, vdim=64, window=100, scale=0.12, mlp=moe(experts=8, top=2, ff=64, shared=128)),
                  attn(heads=8, kv_heads=4, dim=32, vdim=32, window=0, scale=0.18, mlp=dense(ff=512))], width=256, vocab=300, taps=4)
    for dtype in ("bfloat16", "float32"):
        m, o = build(cfg, seed=39, dtype=dtype, max_seq_len=192)
        ids = toks(160, 300, seed=40)
        want = o.run(ids)
        got = np.concatenate([m.forward_rows(ids[None, :150], 0, list(range(150))),
                              np.stack([m.forward(ids[None, i:i + 1], i)[0] for i in range(150, 160)])])
        assert close(got, want, dtype)
        m.close()


@pytest.mark.parametrize("seed", [101, 102, 103, 104])
def test_random_configurations(seed):
    """Configurations drawn at random - widths, vocabularies, taps, layer counts and orders, head counts and sizes, rotated
    parts, windows, constants, feed-forward kinds - each as a whole prompt, as a prompt with decoded tokens and in random
    portions, in both modes."""
    rng = np.random.default_rng(seed)
    for _ in range(5):
        layers = []
        for _ in range(int(rng.integers(1, 5))):
            G, rep = int(rng.choice([1, 2, 3])), int(rng.choice([1, 2, 4]))
            dim, vdim = int(rng.choice([8, 16, 24, 32, 64])), int(rng.choice([8, 16, 32, 40, 64, 128]))
            k = rng.random()
            if k < 0.2:
                mlp = None
            elif k < 0.5:
                mlp = dense(int(rng.choice([40, 64, 100])))
            else:
                E = int(rng.choice([1, 3, 4, 9]))
                mlp = moe(experts=E, top=int(rng.integers(1, min(E, 3) + 1)), ff=int(rng.choice([8, 24, 48])), shared=int(rng.choice([0, 16, 40])))
            layers.append(attn(heads=G * rep, kv_heads=G, dim=dim, vdim=vdim, window=int(rng.choice([0, 1, 5, 31, 64, 90])),
                               diff=float(rng.choice([0.1, 0.4, 0.7])), scale=float(dim ** -0.5 * rng.choice([0.5, 1.0, 2.0])),
                               base=float(rng.choice([50.0, 10000.0, 300000.0])), dims=int(rng.choice([dim, dim // 2, dim // 4 * 2, 0])),
                               scaling=None if rng.random() < 0.3 else (float(rng.choice([2.0, 8.0])), 1.0, float(rng.choice([2.0, 4.0])), int(rng.choice([16, 128]))),
                               mlp=mlp))
        cfg = config(layers, width=int(rng.choice([24, 40, 64, 100, 128])), vocab=int(rng.choice([50, 97, 300])),
                     taps=int(rng.choice([0, 1, 2, 4, 7])), eps=float(rng.choice([1e-6, 1e-5, 1e-3])))
        n = int(rng.choice([30, 75, 140]))
        t = random_model(cfg, int(rng.integers(1 << 30)))
        ids = rng.integers(0, cfg["vocab"], n)
        want = OracleMabedra(cfg, t).run(ids)
        for dtype in ("float32", "bfloat16"):
            m, _ = build(cfg, dtype=dtype, max_seq_len=n + 4, tensors=t)
            assert close(m.forward_rows(ids[None], 0, list(range(n))), want, dtype), (dtype, cfg)
            nd = min(n - 1, 20)
            got = np.concatenate([m.forward_rows(ids[None, :n - nd], 0, list(range(n - nd)))] + [m.forward(ids[None, i:i + 1], i) for i in range(n - nd, n)])
            assert close(got, want, dtype), (dtype, cfg)
            rows, pos = [], 0
            while pos < n:
                c = int(min(n - pos, rng.choice([1, 2, 2, 3, 7, 16, 33, 64])))
                rows.append(m.forward_rows(ids[None, pos:pos + c], pos, list(range(c))))
                pos += c
            assert close(np.concatenate(rows), want, dtype), (dtype, cfg)
            m.close()
