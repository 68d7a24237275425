"""Debuzen on the GPU against the plain NumPy statement of the design (oracle/ref_debuzen.py): every mechanism alone,
whole prompts against token-by-token decoding and against portions down to two tokens, batches against single
sequences, reused slots, keys far away and just inside / outside the window and the kept first tokens (planted so
that one key decides the output), sinks that matter, looped blocks, long decoding, odd sizes, and greedy generation
through the library's own loop and scheduler.  Small random models; fp32 mode is held to 1e-4 of the logit scale,
bf16 to 6e-2."""
import json

import numpy as np
import pytest

from oracle.ref_debuzen import Debuzen as Oracle
from oracle.ref_debuzen import random_tensors

pytestmark = pytest.mark.gpu

FP32_BAR, BF16_BAR = 1e-4, 6e-2
DENSE = {"kind": "dense", "ff": 80}


def attn(heads=4, kv_heads=2, dim=24, vdim=40, size=9, keep_first=None, dims=8, base=10000.0, scale=0.25):
    mask = {"size": size}
    if keep_first is not None:
        mask["keep_first"] = keep_first
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": mask, "rot": {"base": base, "dims": dims},
            "scale": scale}


def par(left=None, heads=3, kv_heads=3, dim=16, vdim=24, conv=3, ls=0.7, rs=1.3, mlp=DENSE):
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": left or attn(keep_first=3), "left_scale": ls, "right_scale": rs,
                      "right": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}}


def par2(left=None, heads=6, groups=3, state=16, vdim=8, conv=4, norm_groups=2, ls=1.1, rs=0.6, mlp=DENSE):
    return {"type": "parallel_2", "mlp": mlp,
            "mixer": {"left": left or attn(heads=6, kv_heads=1, dim=32, vdim=16, size=11, dims=16, base=5000.0), "left_scale": ls,
                      "right_scale": rs,
                      "right": {"heads": heads, "groups": groups, "state": state, "vdim": vdim, "conv": conv, "norm_groups": norm_groups}}}


def gla(heads=3, dim=16, vdim=24, tau=8.0, mlp=DENSE):
    return {"type": "gla", "mlp": mlp, "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}}


def config(layers, width=96, vocab=101, loop=None, eps=1e-5, groups=3, cap=12.0):
    c = {"architecture": "Debuzen", "layers": layers, "norm": {"eps": eps, "groups": groups}, "vocab": vocab, "width": width,
         "logit_softcap": cap}
    if loop:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


def build(cfg, seed=0, dtype="float32", max_seq_len=128, max_batch_size=1, tensors=None):
    from llama3_np_b200.debuzen import Debuzen
    t = random_tensors(cfg, seed) if tensors is None else tensors
    return Debuzen(cfg, t, dtype=dtype, max_seq_len=max_seq_len, max_batch_size=max_batch_size), Oracle(cfg, t)


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
    e = row_errs(got, want)
    return bool(e.max() < (FP32_BAR if dtype == "float32" else BF16_BAR))


def toks(n, vocab, seed=1):
    return np.random.default_rng(seed).integers(0, vocab, n)


def fresh(o):
    o.reset()
    return o


def portions(m, ids, cuts, start=0):
    """the logits of every token, the sequence fed in portions of the given sizes (the last size repeats)"""
    out, pos, k = [], 0, 0
    while pos < len(ids):
        c = min(cuts[min(k, len(cuts) - 1)], len(ids) - pos)
        out.append(m.forward_rows(ids[None, pos:pos + c], start + pos, list(range(c))))
        pos += c
        k += 1
    return np.concatenate(out)


ALONE = {
    "sigmoid_window_and_delta": [par()],
    "sink_window_and_state_space": [par2()],
    "gated_linear": [gla()],
    "no_feed_forward": [par(mlp=None), par2(mlp=None), gla(mlp=None)],
}


@pytest.mark.parametrize("name", sorted(ALONE))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_each_mechanism_alone(name, dtype):
    cfg = config(ALONE[name])
    m, o = build(cfg, seed=3, dtype=dtype)
    ids = toks(40, cfg["vocab"])
    got, resid = m.forward_rows(ids[None], 0, list(range(40)), want_residual=True)
    want, wres = o.run(ids, want_residual=True)
    assert resid.shape == (len(cfg["layers"]), 40, cfg["width"])
    assert close(got, want, dtype)
    if dtype == "float32":
        assert np.allclose(resid, wres, rtol=1e-4, atol=1e-4)
    m.close()


MIXED = [par(), par2(), gla(), par(left=attn(heads=2, kv_heads=1, dim=40, vdim=8, size=6, keep_first=1, dims=40), conv=2), gla(heads=1, dim=8, vdim=72)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_then_token_by_token_and_portions(dtype):
    cfg = config(MIXED, loop=(1, 4, 2))
    m, o = build(cfg, seed=5, dtype=dtype)
    ids = toks(70, cfg["vocab"], seed=6)
    want = o.run(ids)
    whole = m.forward_rows(ids[None], 0, list(range(70)))
    assert close(whole, want, dtype)
    one = portions(m, ids, [1])
    assert close(one, want, dtype)
    for cuts in ([2], [3, 2, 7, 2, 17, 5, 2], [33, 2, 4], [64, 1]):
        got = portions(m, ids, cuts)
        assert close(got, want, dtype), cuts
        if dtype == "float32":  # the paths differ by the order of a few sums only
            assert err(got, whole) < 2e-5, cuts
    m.close()


def test_token_shift_reads_the_previous_token_and_zeros_at_the_start():
    cfg = config([gla(), par()], width=48, vocab=40, groups=2)
    t = random_tensors(cfg, 4)
    for i in range(2):
        t[f"l{i}.shift"] = np.ones(48, np.float32)
    m, o = build(cfg, tensors=t)
    ids = toks(12, 40, seed=5)
    want = o.run(ids)
    assert err(m.forward_rows(ids[None], 0, list(range(12))), want) < FP32_BAR
    assert err(portions(m, ids, [5, 1, 2, 4]), want) < FP32_BAR
    m.close()


def test_looped_block_keeps_one_state_per_pass():
    cfg = config([gla(), par(), par2()], loop=(0, 2, 3))
    m, o = build(cfg, seed=7)
    assert m.n_runs == 7
    ids = toks(30, cfg["vocab"], seed=8)
    want, wres = o.run(ids, want_residual=True)
    got, resid = m.forward_rows(ids[None], 0, list(range(30)), want_residual=True)
    assert err(got, want) < FP32_BAR
    assert np.allclose(resid, wres, rtol=1e-4, atol=1e-4)
    assert err(portions(m, ids, [7, 2, 9]), want) < FP32_BAR
    m.close()


@pytest.mark.parametrize("loop", [None, (0, 3, 1), (0, 3, 2), (2, 3, 4), (1, 2, 2)])
def test_loop_bounds(loop):
    cfg = config([gla(mlp=None), par(mlp=None), par2()], width=48, groups=1, loop=loop)
    m, o = build(cfg, seed=9)
    ids = toks(14, cfg["vocab"], seed=10)
    assert err(m.forward_rows(ids[None], 0, list(range(14))), o.run(ids)) < FP32_BAR
    m.close()


def test_long_decoding_matches_the_oracle():
    """160 tokens one by one behind a short prompt: the windows (6, 9, 11 keys) pass over decoded tokens many times."""
    cfg = config(MIXED)
    m, o = build(cfg, seed=11, max_seq_len=192)
    ids = toks(165, cfg["vocab"], seed=12)
    want = o.run(ids)
    got = portions(m, ids, [5, 1])
    assert err(got, want) < FP32_BAR
    m.close()


def test_batch_rows_equal_single_sequences_and_slots_are_reused():
    cfg = config(MIXED[:3], loop=(0, 2, 2))
    m, o = build(cfg, seed=13, max_batch_size=3)
    seqs = np.stack([toks(26, cfg["vocab"], seed=s) for s in (14, 15, 16)])
    want = np.stack([fresh(o).run(s) for s in seqs])
    # the batch as a whole, then continued in portions of unequal sizes
    got = m.forward_rows(seqs[:, :17], 0, list(range(3 * 17))).reshape(3, 17, -1)
    assert err(got, want[:, :17]) < FP32_BAR
    got = m.forward_rows(seqs[:, 17:19], 17, list(range(3 * 2))).reshape(3, 2, -1)
    assert err(got, want[:, 17:19]) < FP32_BAR
    got = m.forward_rows(seqs[:, 19:], 19, list(range(3 * 7))).reshape(3, 7, -1)
    assert err(got, want[:, 19:]) < FP32_BAR
    # slot 0 starts another sequence at position 0: nothing of the old one is left
    other = toks(20, cfg["vocab"], seed=17)
    assert err(m.forward_rows(other[None], 0, list(range(20))), fresh(o).run(other)) < FP32_BAR
    # and a shorter one after a longer one, fed token by token (cache rows past its position hold the old sequence)
    short = toks(6, cfg["vocab"], seed=18)
    assert err(portions(m, short, [1]), fresh(o).run(short)) < FP32_BAR
    m.close()


def planted(cfg, t, key_tok, query_tok, amp):
    """Rewrites layer 0's left attention so that the key of token `key_tok` stands out for the query of `query_tok`:
    no token shift and no rotation in the way, q and k point along one direction for these two tokens.  Returns the
    tensors; the value of the planted key is made large so that seeing it or not decides the output."""
    o = Oracle(cfg, t)
    W = cfg["width"]
    mc = cfg["layers"][0]["mixer"]["left"]
    H, G, dk, dv = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
    t = dict(t)
    t["l0.shift"] = np.zeros(W, np.float32)

    def h_of(tok):
        x0 = o.norm(o.t["embed"][tok], "embed.norm")
        x = o.t["loop.in"] @ np.concatenate([x0, x0]) if cfg.get("loop") and cfg["loop"]["start"] == 0 else x0
        return o.norm(x, "l0.norm1")

    hk, hq = h_of(key_tok), h_of(query_tok)
    u = np.zeros(dk)
    u[mc["rot"]["dims"]:] = 1.0  # only entries that do not rotate
    rng = np.random.default_rng(0)
    t["l0.mix.left.q"] = (0.02 * rng.standard_normal((H * dk, W)) + amp * np.outer(np.tile(u, H), hq) / (hq @ hq)).astype(np.float32)
    t["l0.mix.left.k"] = (0.02 * rng.standard_normal((G * dk, W)) + amp * np.outer(np.tile(u, G), hk) / (hk @ hk)).astype(np.float32)
    t["l0.mix.left.v"] = (t["l0.mix.left.v"] + 12.0 * np.outer(np.ones(G * dv), hk) / (hk @ hk)).astype(np.float32)
    return t


@pytest.mark.parametrize("kind", ["parallel", "parallel_2"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_planted_key_at_the_windows_edges_and_among_the_kept_tokens(kind, dtype):
    """One key decides the attention's output.  It sits just inside the window, just outside it, far behind it, and
    (sigmoid kind) among the kept first tokens or right behind them; the query is the last token of a prompt, of a
    portion of two tokens, or a token decoded alone."""
    size, keep = 37, 3
    left = attn(heads=4, kv_heads=2, dim=24, vdim=40, size=size, keep_first=keep if kind == "parallel" else None, dims=8, scale=0.5)
    layer = par(left=left, ls=2.0, mlp=None) if kind == "parallel" else par2(left=left, ls=2.0, mlp=None)
    cfg = config([layer], vocab=60, cap=0.0)
    base = random_tensors(cfg, 19)
    if kind == "parallel":
        base["l0.mix.left.pb"] = np.full(4, -6.0, np.float32)  # every other key weighs next to nothing
    KEY, QUERY, n = 58, 59, 150
    t = planted(cfg, base, KEY, QUERY, amp=6.0 if kind == "parallel" else 9.0)
    m, o = build(cfg, dtype=dtype, tensors=t, max_seq_len=160)
    places = [n - size, n - size - 1, n - size + 1, 40, n - 2]
    if kind == "parallel":
        places += [0, keep - 1, keep, keep + 1]
    outs = {}
    for at in places:
        ids = toks(n, 58, seed=20)  # ids below the two special tokens
        ids[at], ids[n - 1] = KEY, QUERY
        want = fresh(o).run(ids)
        outs[at] = want[-1]
        assert close(m.forward_rows(ids[None], 0, [n - 1]), want[-1:], dtype), ("prompt", at)
        got = portions(m, ids, [n - 30, 13, 15, 2])
        assert close(got[-2:], want[-2:], dtype), ("portion of two", at)
        got = portions(m, ids, [n - 1, 1])
        assert close(got[-1:], want[-1:], dtype), ("decoded", at)
    # the planted key is worth seeing: inside and outside differ by far more than the error bar
    assert err(outs[n - size], outs[n - size - 1]) > 0.1
    if kind == "parallel":
        assert err(outs[keep - 1], outs[keep]) > 0.1
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sinks_and_biases_matter(dtype):
    """A large sink takes most of the softmax's mass; a large bias opens every sigmoid: dropping either shows."""
    cfg = config([par2(), par()], vocab=50)
    t = random_tensors(cfg, 21)
    t["l0.mix.left.sink"] = np.array([6.0, -3.0, 2.0, 0.0, 4.0, -1.0], np.float32)
    t["l1.mix.left.pb"] = np.array([2.0, -1.0, 0.5, -4.0], np.float32)
    m, o = build(cfg, dtype=dtype, tensors=t)
    ids = toks(30, 50, seed=22)
    want = o.run(ids)
    assert close(m.forward_rows(ids[None], 0, list(range(30))), want, dtype)
    assert close(portions(m, ids, [9, 2, 1]), want, dtype)
    t2 = dict(t)
    t2["l0.mix.left.sink"] = np.full(6, -30.0, np.float32)
    assert err(Oracle(cfg, t2).run(ids), want) > 0.05
    m.close()


def test_keys_far_away_through_the_recurrent_states():
    """Windows of 4 keys: what a token 200 places back said can only arrive through the recurrent states."""
    small = attn(heads=2, kv_heads=1, dim=8, vdim=8, size=4, dims=8)
    cfg = config([par(left=dict(small, mask={"size": 4, "keep_first": 0})), par2(left=small), gla(tau=64.0)], width=48, vocab=50, groups=2)
    t = random_tensors(cfg, 23)
    t["l2.mix.a2.b"] = np.full_like(t["l2.mix.a2.b"], 6.0)   # slow decays: the state remembers
    m, o = build(cfg, tensors=t, max_seq_len=256)
    ids = toks(230, 50, seed=24)
    ids2 = ids.copy()
    ids2[10] = (ids[10] + 7) % 50
    want, want2 = o.run(ids), fresh(o).run(ids2)
    assert err(want[-1:], want2[-1:]) > 1e-3   # the far token is felt at the end
    for seq, w in ((ids, want), (ids2, want2)):
        assert err(m.forward_rows(seq[None], 0, [229]), w[-1:]) < FP32_BAR
        assert err(portions(m, seq, [100, 2, 97, 1])[-1:], w[-1:]) < FP32_BAR
    m.close()


def test_states_after_a_prompt_and_after_a_slot_is_used_again():
    """The recurrent state matrices and the convolutions' tails a prompt leaves, read back from the slot; then the same
    slot runs another sequence in portions and must hold that sequence's state only."""
    cfg = config([par(mlp=None), par2(mlp=None), gla(mlp=None)], width=48, vocab=50, groups=2, loop=(0, 2, 2))
    m, o = build(cfg, seed=38)

    def check(ids):
        for run, (layer, _) in enumerate(o.runs):
            S, tail = m.read_state(run)
            st = o.state[run]
            kind = cfg["layers"][layer]["type"]
            want_S = st["S"] if kind == "gla" else st["right"]["S"]
            assert np.allclose(S, want_S, rtol=1e-4, atol=1e-5), (run, kind)
            if kind == "parallel":
                r = st["right"]
                assert np.allclose(tail, np.concatenate([r["tail_q"], r["tail_k"], r["tail_v"]]), rtol=1e-4, atol=1e-5), run
            elif kind == "parallel_2":
                assert np.allclose(tail, st["right"]["tail"], rtol=1e-4, atol=1e-5), run

    ids = toks(21, 50, seed=39)
    m.forward(ids[None], 0)
    fresh(o).run(ids)
    check(ids)
    other = toks(9, 50, seed=40)
    portions(m, other, [4, 1, 2, 1, 1])
    fresh(o).run(other)
    check(other)
    m.close()


ODD = {
    "one_head_one_group": [par(left=attn(heads=1, kv_heads=1, dim=8, vdim=8, size=1, keep_first=1, dims=0), heads=1, kv_heads=1, dim=8, vdim=8, conv=1),
                           par2(left=attn(heads=1, kv_heads=1, dim=16, vdim=8, size=3, dims=16), heads=1, groups=1, state=8, vdim=8, conv=1, norm_groups=1),
                           gla(heads=1, dim=8, vdim=8, tau=1.0)],
    "sizes_off_the_grid": [par(left=attn(heads=6, kv_heads=2, dim=10, vdim=36, size=5, keep_first=7, dims=6), heads=4, kv_heads=2, dim=12, vdim=20, conv=5),
                           par2(left=attn(heads=3, kv_heads=3, dim=12, vdim=68, size=200, dims=4), heads=4, groups=2, state=12, vdim=20, conv=2, norm_groups=5),
                           gla(heads=5, dim=12, vdim=20, tau=3.0)],
    "wide_heads": [par(left=attn(heads=2, kv_heads=1, dim=128, vdim=128, size=17, keep_first=2, dims=64, scale=0.09), heads=2, kv_heads=1, dim=64, vdim=128),
                   par2(left=attn(heads=2, kv_heads=2, dim=64, vdim=256, size=8, dims=32, scale=0.12), heads=2, groups=1, state=128, vdim=64)],
}


@pytest.mark.parametrize("name", sorted(ODD))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_odd_sizes(name, dtype):
    cfg = config(ODD[name], width=120 if name != "one_head_one_group" else 40, vocab=77, groups=5 if name != "one_head_one_group" else 1,
                 loop=(0, len(ODD[name]), 2), cap=0.0 if name == "sizes_off_the_grid" else 20.0)
    m, o = build(cfg, seed=25, dtype=dtype)
    ids = toks(45, 77, seed=26)
    want = o.run(ids)
    assert close(m.forward_rows(ids[None], 0, list(range(45))), want, dtype)
    assert close(portions(m, ids, [11, 2, 1, 1, 20, 3]), want, dtype)
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_library_loop(dtype):
    cfg = config(MIXED, loop=(0, 2, 2))
    m, o = build(cfg, seed=27, dtype=dtype, max_seq_len=96, max_batch_size=2)
    prompts = np.stack([toks(12, cfg["vocab"], seed=s) for s in (28, 29)])
    lazy = np.concatenate(list(m.generate(prompts, 40)), axis=1)
    bulk = m.generate_all(prompts, 40)
    assert np.array_equal(lazy, bulk)
    # teacher-forced: every emitted token is the oracle's argmax for the same prefix, unless the oracle's top two
    # are closer than the mode's error bar
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
    cfg = config(MIXED[:3], loop=(1, 2, 2))
    m, _ = build(cfg, seed=30, max_seq_len=64, max_batch_size=2)
    prompts = [toks(n, cfg["vocab"], seed=31 + n) for n in (5, 9, 5, 2, 9)]
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
    cfg = config([par(), gla()], width=48, vocab=41, groups=2, loop=(0, 1, 2))
    t = random_tensors(cfg, 32)
    _write_folder(tmp_path, cfg, t)
    m = load_model(str(tmp_path), dtype="float32", max_seq_len=32)
    assert type(m).__name__ == "Debuzen"
    ids = toks(16, 41, seed=33)
    assert err(m.forward_rows(ids[None], 0, list(range(16))), Oracle(cfg, t).run(ids)) < FP32_BAR
    m.close()


def test_trace_runner_replays_a_trace(tmp_path):
    """bin/trace_run as a user runs it: two requests after one another through the same slot, portions cut in odd
    places and longer than one forward call."""
    import os
    import subprocess
    import sys
    from conftest import ROOT
    cfg = config([par2(), par(), gla()], width=48, vocab=41, groups=2, loop=(0, 2, 2))
    t = random_tensors(cfg, 34)
    _write_folder(tmp_path, cfg, t)
    o = Oracle(cfg, t)
    reqs = {"a": toks(23, 41, seed=35), "b": toks(9, 41, seed=36)}
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


def test_generate_command_prints_the_loop_s_tokens(tmp_path):
    import os
    import subprocess
    import sys
    from conftest import ROOT
    from llama3_np_b200.models import load_model
    cfg = config([gla(), par2(), par()], width=48, vocab=47, groups=2, loop=(1, 3, 2))
    _write_folder(tmp_path, cfg, random_tensors(cfg, 41))
    prompts = np.stack([toks(7, 47, seed=s) for s in (42, 43)])
    (tmp_path / "prompts.txt").write_text("\n".join(" ".join(str(int(x)) for x in p) for p in prompts) + "\n")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "generate"), "--model", str(tmp_path), "--dtype", "float32",
                        "--batch-file", str(tmp_path / "prompts.txt"), "--new", "12"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    printed = np.array([[int(x) for x in line.split()] for line in r.stdout.strip().splitlines()[-2:]])
    m = load_model(str(tmp_path), dtype="float32", max_seq_len=19, max_batch_size=2)
    assert np.array_equal(printed, m.generate_all(prompts, 12))
    m.close()


def test_wide_windows_and_many_kept_tokens_over_several_key_tiles():
    """Windows of 150 and 70 keys with 9 kept tokens over a prompt of 400: a query's keys span several 64-key tiles, the
    kept tokens sit in a tile of their own ahead of the window, and short portions split the tiles over CTAs."""
    a1 = attn(heads=4, kv_heads=2, dim=32, vdim=16, size=150, keep_first=9, dims=16, scale=0.2)
    a2 = attn(heads=2, kv_heads=2, dim=16, vdim=48, size=70, dims=8, scale=0.3)
    cfg = config([par(left=a1, mlp=None), par2(left=a2, mlp=None)], width=64, vocab=90, groups=2)
    m, o = build(cfg, seed=44, max_seq_len=420)
    ids = toks(400, 90, seed=45)
    want = o.run(ids)
    assert err(m.forward_rows(ids[None], 0, list(range(400))), want) < FP32_BAR
    got = portions(m, ids, [130, 2, 64, 3, 100, 8, 1, 1, 50, 5, 1])
    assert err(got, want) < FP32_BAR
    m.close()


@pytest.mark.parametrize("fast_decay", [False, True])
def test_long_prompts_of_state_space_layers_run_chunk_parallel(fast_decay):
    """States of 64 x 64 and prompts of 128 tokens and more take the chunk-parallel form of the recurrence (sums in another
    order than the token-by-token chain): both must agree with the oracle and with each other, also where the decays are so
    small that a chunk's product of them underflows."""
    a2 = attn(heads=2, kv_heads=1, dim=16, vdim=16, size=20, dims=8)
    cfg = config([par2(left=a2, heads=4, groups=2, state=64, vdim=64, conv=4, norm_groups=2, mlp=None), gla(mlp=None)], width=64, vocab=80, groups=2)
    t = random_tensors(cfg, 46)
    if fast_decay:
        t["l0.mix.right.dt_bias"] = np.full(4, 4.0, np.float32)
        t["l0.mix.right.A_log"] = np.array([1.0, 0.5, 2.0, -1.0], np.float32)
    m, o = build(cfg, tensors=t, max_seq_len=400)
    ids = toks(390, 80, seed=47)
    want = o.run(ids)
    whole = m.forward_rows(ids[None], 0, list(range(390)))
    assert err(whole, want) < FP32_BAR
    mixed = portions(m, ids, [130, 3, 192, 1, 1, 40, 23])
    assert err(mixed, want) < FP32_BAR
    assert err(mixed, whole) < 2e-5
    m.close()


def test_random_configurations():
    """Sizes, layer order, windows, kept tokens and loops drawn at random; whole prompts, portions, decoded tokens."""
    rng = np.random.default_rng(37)
    for case in range(6):
        layers = []
        for _ in range(int(rng.integers(2, 5))):
            kind = int(rng.integers(0, 3))
            g = int(rng.choice([1, 2, 3]))
            left = attn(heads=g * int(rng.choice([1, 2])), kv_heads=g, dim=int(rng.choice([8, 16, 20, 32])), vdim=int(rng.choice([8, 24, 40])),
                        size=int(rng.integers(1, 30)), keep_first=int(rng.integers(0, 5)) if kind == 0 else None,
                        dims=int(rng.choice([0, 4, 8])), scale=float(rng.uniform(0.1, 0.4)))
            mlp = DENSE if rng.integers(0, 2) else None
            if kind == 0:
                layers.append(par(left=left, heads=g * 2, kv_heads=g, dim=int(rng.choice([8, 16])), vdim=int(rng.choice([8, 16, 24])),
                                  conv=int(rng.integers(1, 5)), mlp=mlp))
            elif kind == 1:
                layers.append(par2(left=left, heads=g * 2, groups=g, state=int(rng.choice([8, 16, 24])), vdim=8, conv=int(rng.integers(1, 5)),
                                   norm_groups=int(rng.choice([1, 2])), mlp=mlp))
            else:
                layers.append(gla(heads=g, dim=int(rng.choice([8, 16])), vdim=int(rng.choice([8, 24])), tau=float(rng.uniform(1, 20)), mlp=mlp))
        a = int(rng.integers(0, len(layers)))
        b = int(rng.integers(a + 1, len(layers) + 1))
        loop = (a, b, int(rng.integers(1, 4))) if rng.integers(0, 3) else None
        cfg = config(layers, width=int(rng.choice([48, 72, 96])), vocab=int(rng.integers(20, 90)), groups=int(rng.choice([1, 2, 3])), loop=loop)
        m, o = build(cfg, seed=40 + case)
        n = int(rng.integers(20, 60))
        ids = toks(n, cfg["vocab"], seed=50 + case)
        want = o.run(ids)
        assert err(m.forward_rows(ids[None], 0, list(range(n))), want) < FP32_BAR, case
        cuts = [int(x) for x in rng.integers(1, 9, 6)] + [1]
        assert err(portions(m, ids, cuts), want) < FP32_BAR, (case, cuts)
        m.close()


def test_larger_shapes_take_the_tensor_core_projections():
    """Width 256 and 64 rows: bf16 mode runs the tcgen05 projections; the logits stay inside the bf16 bar."""
    left1 = attn(heads=4, kv_heads=2, dim=64, vdim=64, size=40, keep_first=4, dims=32, scale=0.15)
    left2 = attn(heads=8, kv_heads=2, dim=32, vdim=32, size=48, dims=32, scale=0.18)
    cfg = config([par(left=left1, heads=4, kv_heads=2, dim=32, vdim=64, conv=4, mlp={"kind": "dense", "ff": 512}),
                  par2(left=left2, heads=8, groups=2, state=32, vdim=32, mlp={"kind": "dense", "ff": 512}),
                  gla(heads=4, dim=32, vdim=64, mlp={"kind": "dense", "ff": 512})], width=256, vocab=300, groups=2, loop=(0, 2, 2))
    m, o = build(cfg, seed=60, dtype="bfloat16", max_seq_len=160)
    ids = toks(100, 300, seed=61)
    want = o.run(ids)
    m.launch_count(reset=True)
    assert close(m.forward_rows(ids[None], 0, list(range(100))), want, "bfloat16")
    assert m.launch_count() > 0
    assert close(portions(m, ids, [64, 20, 2, 1]), want, "bfloat16")
    m.close()
