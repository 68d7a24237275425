"""Plain NumPy float64 oracle of the Debuzen decoder: one function per mechanism, token by token with explicit
state, written from the equations and sharing no code with the library.

Debuzen is a pre-norm decoder.  Every norm is an RMS norm in groups (the vector is cut into `norm.groups` equal
parts, each divided by its own root mean square).  The embedding output passes such a norm.  A block of layers
runs `loop.times` times with one set of weights; ahead of every pass the stream becomes `W_in [x ; x0]` with x0
the embedding output.  The mixer of a layer reads its normed input mixed with the previous token's (token
shift).  Mixers:

* `parallel`: two mixers side by side on the same input, summed with fixed weights - sliding-window attention
  that also keeps the first tokens, with rotary pairs (2i, 2i + 1), unit-RMS queries and keys and un-normalised
  sigmoid weights; and a gated delta rule behind short convolutions.
* `parallel_2`: sliding-window softmax attention with a sink in the denominator and rotary pairs (i, i + dims / 2);
  and a Mamba-2 state-space mixer.
* `gla`: gated linear attention with a decay per key channel.

The feed-forward is a gated unit with silu; the logits pass a tanh soft cap.
"""
from __future__ import annotations

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.maximum(z, 0.0) + np.log1p(np.exp(-np.abs(z)))


def group_rms_norm(x, w, groups, eps):
    """x [..., n] cut into `groups` equal parts, each over its own root mean square, then times w."""
    parts = x.reshape(x.shape[:-1] + (groups, -1))
    parts = parts / np.sqrt((parts * parts).mean(-1, keepdims=True) + eps)
    return parts.reshape(x.shape) * w


def token_shift(h, prev, mu):
    """What the mixer reads, and the row the next token will see as `prev` (the un-mixed h)."""
    return h + (prev - h) * mu, h


def rotate(x, pos, dims, base, layout):
    """x [heads, dim]; the first `dims` entries of every head turn by pos * base^(-2 i / dims).
    layout "pairs": entry 2i with 2i + 1; "halves": entry i with i + dims / 2."""
    out = x.copy()
    if dims == 0:
        return out
    i = np.arange(dims // 2)
    ang = pos * base ** (-2.0 * i / dims)
    c, s = np.cos(ang), np.sin(ang)
    if layout == "pairs":
        u, v = x[:, 0:dims:2], x[:, 1:dims:2]
        out[:, 0:dims:2] = u * c - v * s
        out[:, 1:dims:2] = v * c + u * s
    else:
        u, v = x[:, :dims // 2], x[:, dims // 2:dims]
        out[:, :dims // 2] = u * c - v * s
        out[:, dims // 2:dims] = v * c + u * s
    return out


def visible(i, j, size, keep_first):
    return j <= i and (i - j < size or j < keep_first)


def window_attention(q, keys, vals, pos, *, scale, size, keep_first, kind, extra):
    """q [H, dk] of the token at `pos`; keys / vals: lists over positions 0..pos of [G, dk] / [G, dv].
    kind "sigmoid": weight = sigmoid(score + extra[h]), no normalisation;
    kind "sink": softmax whose denominator also holds exp(extra[h])."""
    H, G = q.shape[0], keys[0].shape[0]
    out = np.zeros((H, vals[0].shape[1]))
    js = [j for j in range(pos + 1) if visible(pos, j, size, keep_first)]
    for h in range(H):
        g = h // (H // G)
        sc = np.array([q[h] @ keys[j][g] for j in js]) * scale
        if kind == "sigmoid":
            wts = sigmoid(sc + extra[h])
        else:
            m = max(sc.max(), extra[h])
            e = np.exp(sc - m)
            wts = e / (e.sum() + np.exp(extra[h] - m))
        for wj, j in zip(wts, js):
            out[h] += wj * vals[j][g]
    return out


def causal_conv(x_new, tail, w, bias=None):
    """One step of a causal convolution per channel: tail [C, taps - 1] (oldest first), w [C, taps] (last column =
    the current token).  Returns (output [C], new tail)."""
    full = np.concatenate([tail, x_new[:, None]], axis=1)
    y = (full * w).sum(-1)
    if bias is not None:
        y = y + bias
    return y, full[:, 1:]


def unit(x, eps=1e-6):
    return x / np.sqrt((x * x).sum(-1, keepdims=True) + eps)


def delta_step(S, q, k, v, g, beta):
    """Per head: S [dk, dv].  S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    S = g[:, None] * S
    u = beta * (v - S.T @ k)
    S = S + np.outer(k, u)
    return S, S.T @ q


def decay_outer_step(S, q, k, v, g):
    """S <- diag(g) S + k v^T; o = S^T q (g a vector over key channels, or a number)."""
    S = (g[:, None] if np.ndim(g) else g) * S + np.outer(k, v)
    return S, S.T @ q


class Debuzen:
    def __init__(self, config, tensors):
        self.c = config
        self.t = {k: np.asarray(v, dtype=np.float64) for k, v in tensors.items()}
        self.eps = float(config["norm"]["eps"])
        self.groups = int(config["norm"].get("groups", 1))
        lp = config.get("loop")
        n = len(config["layers"])
        if lp and int(lp["times"]) > 0:
            a, b, times = int(lp["start"]), int(lp["stop"]), int(lp["times"])
            self.runs = [(i, False) for i in range(a)]
            for _ in range(times):
                self.runs += [(i, i == a) for i in range(a, b)]
            self.runs += [(i, False) for i in range(b, n)]
        else:
            self.runs = [(i, False) for i in range(n)]
        self.reset()

    def reset(self):
        self.pos = 0
        self.state = [dict() for _ in self.runs]

    def norm(self, x, name):
        return group_rms_norm(x, self.t[name], self.groups, self.eps)

    # ------------------------------------------------------------------ mixers
    def _attention(self, p, mc, h, st, layout, kind):
        t = self.t
        H, G, dk, dv = int(mc["heads"]), int(mc["kv_heads"]), int(mc["dim"]), int(mc["vdim"])
        q = (t[p + "q"] @ h).reshape(H, dk)
        k = (t[p + "k"] @ h).reshape(G, dk)
        v = (t[p + "v"] @ h).reshape(G, dv)
        rot = mc.get("rot") or {}
        dims, base = int(rot.get("dims", 0)), float(rot.get("base", 10000.0))
        q = rotate(q, self.pos, dims, base, layout)
        k = rotate(k, self.pos, dims, base, layout)
        if kind == "sigmoid":  # unit RMS per head, no weight
            q = q / np.sqrt((q * q).mean(-1, keepdims=True) + self.eps)
            k = k / np.sqrt((k * k).mean(-1, keepdims=True) + self.eps)
        st.setdefault("k", []).append(k)
        st.setdefault("v", []).append(v)
        mask = mc["mask"]
        o = window_attention(q, st["k"], st["v"], self.pos, scale=float(mc["scale"]), size=int(mask["size"]),
                             keep_first=int(mask.get("keep_first", 0)), kind=kind,
                             extra=t[p + ("pb" if kind == "sigmoid" else "sink")])
        return t[p + "o"] @ o.reshape(-1)

    def _gated_delta(self, p, mc, h, st):
        t = self.t
        H, G, dk, dv, taps = int(mc["heads"]), int(mc["kv_heads"]), int(mc["dim"]), int(mc["vdim"]), int(mc["conv"])
        outs = []
        for nm in ("q", "k", "v"):
            x = t[p + nm] @ h
            tail = st.get("tail_" + nm)
            if tail is None:
                tail = np.zeros((x.shape[0], taps - 1))
            y, st["tail_" + nm] = causal_conv(x, tail, t[p + nm + ".conv"])
            outs.append(silu(y))
        q = unit(outs[0].reshape(G, dk)) * dk ** -0.5
        k = unit(outs[1].reshape(G, dk))
        v = outs[2].reshape(H, dv)
        beta = sigmoid(t[p + "b"] @ h)
        dt = softplus(t[p + "a2"] @ (t[p + "a1"] @ h) + t[p + "dt_bias"]).reshape(H, dk)
        g = np.exp(-np.exp(t[p + "A_log"])[:, None] * dt)
        S = st.get("S")
        if S is None:
            S = np.zeros((H, dk, dv))
        o = np.zeros((H, dv))
        for hh in range(H):
            kh = hh // (H // G)
            S[hh], o[hh] = delta_step(S[hh], q[kh], k[kh], v[hh], g[hh], beta[hh])
        st["S"] = S
        o = o / np.sqrt((o * o).mean(-1, keepdims=True) + self.eps) * t[p + "norm"]
        gate = sigmoid(t[p + "g2"] @ (t[p + "g1"] @ h)).reshape(H, dv)
        return t[p + "o"] @ (o * gate).reshape(-1)

    def _ssd(self, p, mc, h, st):
        t = self.t
        H, dv, N, G, taps = int(mc["heads"]), int(mc["vdim"]), int(mc["state"]), int(mc["groups"]), int(mc["conv"])
        inner = H * dv
        u = t[p + "in"] @ h
        z, xbc, dt = u[:inner], u[inner:2 * inner + 2 * G * N], u[2 * inner + 2 * G * N:]
        tail = st.get("tail")
        if tail is None:
            tail = np.zeros((xbc.shape[0], taps - 1))
        y, st["tail"] = causal_conv(xbc, tail, t[p + "conv"], t[p + "conv.b"])
        y = silu(y)
        x = y[:inner].reshape(H, dv)
        Bm = y[inner:inner + G * N].reshape(G, N)
        Cm = y[inner + G * N:].reshape(G, N)
        dt = softplus(dt + t[p + "dt_bias"])
        a = np.exp(-np.exp(t[p + "A_log"]) * dt)
        S = st.get("S")
        if S is None:
            S = np.zeros((H, N, dv))
        out = np.zeros((H, dv))
        for hh in range(H):
            g = hh // (H // G)
            S[hh], o = decay_outer_step(S[hh], Cm[g], Bm[g], dt[hh] * x[hh], a[hh])
            out[hh] = o + t[p + "D"][hh] * x[hh]
        st["S"] = S
        yv = out.reshape(-1) * silu(z)
        yv = group_rms_norm(yv, t[p + "norm"], int(mc["norm_groups"]), self.eps)
        return t[p + "o"] @ yv

    def _gla(self, p, mc, h, st):
        t = self.t
        H, dk, dv, tau = int(mc["heads"]), int(mc["dim"]), int(mc["vdim"]), float(mc["tau"])
        q = (t[p + "q"] @ h).reshape(H, dk) * dk ** -0.5
        k = (t[p + "k"] @ h).reshape(H, dk)
        v = (t[p + "v"] @ h).reshape(H, dv)
        zz = t[p + "a2"] @ (t[p + "a1"] @ h) + t[p + "a2.b"]
        alpha = (sigmoid(zz) ** (1.0 / tau)).reshape(H, dk)
        S = st.get("S")
        if S is None:
            S = np.zeros((H, dk, dv))
        o = np.zeros((H, dv))
        for hh in range(H):
            S[hh], o[hh] = decay_outer_step(S[hh], q[hh], k[hh], v[hh], alpha[hh])
        st["S"] = S
        o = o / np.sqrt((o * o).mean(-1, keepdims=True) + self.eps) * t[p + "norm"]
        return t[p + "o"] @ (o.reshape(-1) * silu(t[p + "g"] @ h))

    def mixer(self, i, h, st):
        lc = self.c["layers"][i]
        kind, mc, p = lc["type"], lc["mixer"], f"l{i}.mix."
        if kind == "parallel":
            left = self._attention(p + "left.", mc["left"], h, st.setdefault("left", {}), "pairs", "sigmoid")
            right = self._gated_delta(p + "right.", mc["right"], h, st.setdefault("right", {}))
            return float(mc["left_scale"]) * left + float(mc["right_scale"]) * right
        if kind == "parallel_2":
            left = self._attention(p + "left.", mc["left"], h, st.setdefault("left", {}), "halves", "sink")
            right = self._ssd(p + "right.", mc["right"], h, st.setdefault("right", {}))
            return float(mc["left_scale"]) * left + float(mc["right_scale"]) * right
        if kind == "gla":
            return self._gla(p, mc, h, st)
        raise ValueError(kind)

    def feed_forward(self, i, h):
        t, p = self.t, f"l{i}.mlp."
        return t[p + "down"] @ (silu(t[p + "gate"] @ h) * (t[p + "up"] @ h))

    # ------------------------------------------------------------------ one token
    def step(self, token, want_residual=False):
        """Feed one token at the sequence's next position; returns the logits (and the stream after every layer run)."""
        t, W = self.t, int(self.c["width"])
        x0 = self.norm(t["embed"][token], "embed.norm")
        x = x0
        trace = []
        for ri, (i, first_of_pass) in enumerate(self.runs):
            st = self.state[ri]
            if first_of_pass:
                x = t["loop.in"] @ np.concatenate([x, x0])
            h = self.norm(x, f"l{i}.norm1")
            h, st["prev"] = token_shift(h, st.get("prev", np.zeros(W)), t[f"l{i}.shift"])
            x = x + self.mixer(i, h, st)
            if self.c["layers"][i].get("mlp") is not None:
                x = x + self.feed_forward(i, self.norm(x, f"l{i}.norm2"))
            trace.append(x)
        y = t["head"] @ self.norm(x, "final.norm")
        cap = float(self.c.get("logit_softcap") or 0.0)
        if cap > 0:
            y = cap * np.tanh(y / cap)
        self.pos += 1
        return (y, np.stack(trace)) if want_residual else y

    def run(self, tokens, want_residual=False):
        outs = [self.step(int(tk), want_residual) for tk in tokens]
        if want_residual:
            return np.stack([o[0] for o in outs]), np.stack([o[1] for o in outs], axis=1)
        return np.stack(outs)


def random_tensors(config, seed=0, scale=1.0):
    """Random float32 tensors of every name a Debuzen configuration needs (tests)."""
    rng = np.random.default_rng(seed)
    W, V = int(config["width"]), int(config["vocab"])
    t = {}

    def mat(n, k, s=1.0):
        return (rng.standard_normal((n, k)) * s * scale / np.sqrt(k)).astype(np.float32)

    def vec(n, mean=0.0, s=0.2):
        return (mean + rng.standard_normal(n) * s).astype(np.float32)

    t["embed"] = rng.standard_normal((V, W)).astype(np.float32)
    t["embed.norm"] = vec(W, 1.0, 0.1)
    t["final.norm"] = vec(W, 1.0, 0.1)
    t["head"] = mat(V, W, 2.0)
    if config.get("loop"):
        t["loop.in"] = mat(W, 2 * W, 1.4)

    def attention(p, mc, kind):
        H, G, dk, dv = int(mc["heads"]), int(mc["kv_heads"]), int(mc["dim"]), int(mc["vdim"])
        t[p + "q"], t[p + "k"], t[p + "v"], t[p + "o"] = mat(H * dk, W, 2.0), mat(G * dk, W, 2.0), mat(G * dv, W), mat(W, H * dv)
        t[p + ("pb" if kind == "sigmoid" else "sink")] = vec(H, -1.0 if kind == "sigmoid" else 0.5, 0.5)

    for i, lc in enumerate(config["layers"]):
        p, mc = f"l{i}.", lc["mixer"]
        t[p + "norm1"], t[p + "shift"] = vec(W, 1.0, 0.1), rng.uniform(0, 1, W).astype(np.float32)
        if lc.get("mlp") is not None:
            ff = int(lc["mlp"]["ff"])
            t[p + "norm2"] = vec(W, 1.0, 0.1)
            t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = mat(ff, W), mat(ff, W), mat(W, ff)
        if lc["type"] == "parallel":
            attention(p + "mix.left.", mc["left"], "sigmoid")
            r, q = mc["right"], p + "mix.right."
            H, G, dk, dv, taps = int(r["heads"]), int(r["kv_heads"]), int(r["dim"]), int(r["vdim"]), int(r["conv"])
            ra, rg = int(r.get("rank_decay", 8)), int(r.get("rank_gate", 8))
            t[q + "q"], t[q + "k"], t[q + "v"] = mat(G * dk, W, 2.0), mat(G * dk, W, 2.0), mat(H * dv, W, 2.0)
            for nm, n in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                t[q + nm + ".conv"] = (rng.standard_normal((n, taps)) / np.sqrt(taps)).astype(np.float32)
            t[q + "b"], t[q + "A_log"], t[q + "norm"] = mat(H, W), vec(H, 0.0, 0.5), vec(dv, 1.0, 0.1)
            t[q + "a1"], t[q + "a2"], t[q + "dt_bias"] = mat(ra, W), mat(H * dk, ra), vec(H * dk, -1.0, 0.5)
            t[q + "g1"], t[q + "g2"], t[q + "o"] = mat(rg, W), mat(H * dv, rg), mat(W, H * dv)
        elif lc["type"] == "parallel_2":
            attention(p + "mix.left.", mc["left"], "sink")
            r, q = mc["right"], p + "mix.right."
            H, dv, N, G, taps = int(r["heads"]), int(r["vdim"]), int(r["state"]), int(r["groups"]), int(r["conv"])
            inner, ch = H * dv, H * dv + 2 * G * N
            t[q + "in"] = mat(2 * inner + 2 * G * N + H, W, 1.5)
            t[q + "conv"] = (rng.standard_normal((ch, taps)) / np.sqrt(taps)).astype(np.float32)
            t[q + "conv.b"], t[q + "dt_bias"], t[q + "A_log"] = vec(ch, 0.0, 0.2), vec(H, -0.5, 0.5), vec(H, 0.0, 0.5)
            t[q + "D"], t[q + "norm"], t[q + "o"] = vec(H, 1.0, 0.3), vec(inner, 1.0, 0.1), mat(W, inner)
        else:
            q = p + "mix."
            H, dk, dv, ra = int(mc["heads"]), int(mc["dim"]), int(mc["vdim"]), int(mc.get("rank_decay", 8))
            t[q + "q"], t[q + "k"], t[q + "v"], t[q + "g"] = mat(H * dk, W, 2.0), mat(H * dk, W, 2.0), mat(H * dv, W), mat(H * dv, W)
            t[q + "a1"], t[q + "a2"], t[q + "a2.b"] = mat(ra, W), mat(H * dk, ra, 2.0), vec(H * dk, 2.0, 1.0)
            t[q + "norm"], t[q + "o"] = vec(dv, 1.0, 0.1), mat(W, H * dv)
    # values a bfloat16 checkpoint can hold exactly
    for k in t:
        t[k] = (np.ascontiguousarray(t[k], np.float32).view(np.uint32) & np.uint32(0xFFFF0000)).view(np.float32)
    return t
