"""Plain NumPy (float64) statement of the Mabedra decoder, one function per mechanism.

The oracle of `llama3_np_b200.mabedra`: it shares no code with the product path, runs token by token with
explicit per-sequence state, and keeps every intermediate in float64.  Nothing here is fast.

Notation: `x` the stream row a layer receives (width W), `P` a dict of one layer's tensors with the `l<i>.` prefix
removed, `st` the mutable per-sequence state of one layer (cached keys / values, the last inputs of the
convolutions).  With X_0 = E[token] and LN(v) = (v - mean v) / sqrt(var v + eps) * w:

    layer i:  h = LN_i(x)
              u_s = h + sum_j c_s[:, j] * h_(t - T + 1 + j)          s = 1 (mixer), 2 (feed-forward); h_(<0) = 0
              X_(i+1) = x + g1 * mixer(u_1) + g2 * ff(u_2)            g1, g2 per channel
              x <- sum_(j <= i+1) a_i[j] * X_j                        the stream layer i + 1 receives
    logits = head LN_f(x)
"""
from __future__ import annotations

import numpy as np


# ------------------------------------------------------------------ scalar functions
def layer_norm(x, w, eps):
    d = x - x.mean()
    return d / np.sqrt(np.mean(d * d) + eps) * w


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softmax(z):
    e = np.exp(z - np.max(z))
    return e / e.sum()


# ------------------------------------------------------------------ rotary positions
def rotary_frequencies(rot):
    """f_i = base^(-2i / dims), then rescaled by wavelength l = 2 pi / f: short waves (l < original / high) stay, long ones
    (l > original / low) are divided by `factor`, the band between is blended linearly in original / l."""
    dims = int(rot["dims"])
    f = np.power(float(rot["base"]), -2.0 * np.arange(dims // 2) / dims)
    sc = rot.get("scaling")
    if not sc:
        return f
    out = f.copy()
    for i, fi in enumerate(f):
        wave = 2.0 * np.pi / fi
        if wave < sc["original"] / sc["high"]:
            continue
        if wave > sc["original"] / sc["low"]:
            out[i] = fi / sc["factor"]
        else:
            t = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
            out[i] = (1.0 - t) * fi / sc["factor"] + t * fi
    return out


def rotate_half(v, pos, rot):
    """Entry i of the first `dims` entries turns together with entry i + dims / 2; the rest passes unchanged."""
    dims = int(rot.get("dims", 0)) if rot else 0
    out = np.array(v, dtype=np.float64)
    if dims == 0:
        return out
    ang = pos * rotary_frequencies(rot)
    c, s = np.cos(ang), np.sin(ang)
    a, b = out[: dims // 2].copy(), out[dims // 2: dims].copy()
    out[: dims // 2] = a * c - b * s
    out[dims // 2: dims] = b * c + a * s
    return out


# ------------------------------------------------------------------ input convolution
def canon(h, w, st, key):
    """h + sum_j w[:, j] * (input T - 1 - j tokens back); `st[key]` holds the last T - 1 inputs, oldest first."""
    taps = w.shape[1]
    past = st.setdefault(key, [np.zeros_like(h) for _ in range(taps - 1)])
    seq = past + [h]
    out = h + sum(w[:, j] * seq[j] for j in range(taps))
    st[key] = seq[1:]
    return out


# ------------------------------------------------------------------ differential attention
def diff_lambda(P, mc):
    return np.exp(np.dot(P["mix.lq1"], P["mix.lk1"])) - np.exp(np.dot(P["mix.lq2"], P["mix.lk2"])) + mc["diff"]


def diff_attention_step(u, pos, P, mc, eps, st):
    H, G, dk = int(mc["heads"]), int(mc.get("kv_heads", mc["heads"])), int(mc["dim"])
    dv = int(mc.get("vdim", dk))
    rot = mc.get("rot")
    window = int((mc.get("mask") or {}).get("size", 0))
    q = (P["mix.q"] @ u + P["mix.q.b"]).reshape(H, 2, dk)
    k = (P["mix.k"] @ u + P["mix.k.b"]).reshape(G, 2, dk)
    v = (P["mix.v"] @ u + P["mix.v.b"]).reshape(G, dv)
    q = rms_unit(q, eps) * P["mix.q.norm"]
    k = rms_unit(k, eps) * P["mix.k.norm"]
    for a in range(H):
        for mp in range(2):
            q[a, mp] = rotate_half(q[a, mp], pos, rot)
    for g in range(G):
        for mp in range(2):
            k[g, mp] = rotate_half(k[g, mp], pos, rot)
    st.setdefault("k", []).append(k)
    st.setdefault("v", []).append(v)
    first = max(0, pos - window + 1) if window > 0 else 0
    K = np.stack(st["k"][first: pos + 1])   # [n, G, 2, dk]
    V = np.stack(st["v"][first: pos + 1])   # [n, G, dv]
    lam = diff_lambda(P, mc)
    out = np.zeros((H, dv))
    for a in range(H):
        g = a // (H // G)
        a1 = softmax(K[:, g, 0] @ q[a, 0] * mc["scale"]) @ V[:, g]
        a2 = softmax(K[:, g, 1] @ q[a, 1] * mc["scale"]) @ V[:, g]
        out[a] = rms_unit(a1 - lam * a2, eps) * (1.0 - mc["diff"])
    return P["mix.o"] @ out.reshape(-1)


# ------------------------------------------------------------------ feed-forwards
def polynorm(z, coef, eps):
    a, b, c, e = coef
    return a * rms_unit(z, eps) + b * rms_unit(z ** 2, eps) + c * rms_unit(z ** 3, eps) + e


def dense_ff(u, P, eps):
    return P["mlp.down"] @ polynorm(P["mlp.up"] @ u, P["mlp.act"], eps)


def gated_unit(u, P, prefix):
    return P[prefix + "down"] @ (silu(P[prefix + "gate"] @ u) * (P[prefix + "up"] @ u))


def route(u, P, rc):
    """(chosen experts, their weights): the `top` largest sigmoid scores, ties to the lower index, weights = scores."""
    s = sigmoid(P["mlp.router"] @ u)
    order = sorted(range(len(s)), key=lambda e: (-s[e], e))[: int(rc["top"])]
    return order, [s[e] for e in order]


def moe_ff(u, P, mlp):
    """The routing weight scales the expert's INPUT; the shared expert sees the input as it is."""
    chosen, weights = route(u, P, mlp["router"])
    out = np.zeros(P["mlp.e0.down"].shape[0])
    for e, w in zip(chosen, weights):
        out += gated_unit(w * u, P, f"mlp.e{e}.")
    if mlp.get("shared"):
        out += gated_unit(u, P, "mlp.shared.")
    return out


# ------------------------------------------------------------------ the model
class OracleMabedra:
    def __init__(self, config, tensors):
        self.cfg = config
        self.eps = float(config["norm"]["eps"])
        self.T = {k: np.asarray(v, dtype=np.float64) for k, v in tensors.items()}
        self.layers = []
        for i in range(len(config["layers"])):
            pre = f"l{i}."
            self.layers.append({k[len(pre):]: v for k, v in self.T.items() if k.startswith(pre)})
        self.reset()

    def reset(self):
        self.pos = 0
        self.state = [dict() for _ in self.cfg["layers"]]

    def step(self, token, want_residual=False):
        X = [self.T["embed"][int(token)].copy()]
        x = X[0]
        resid = []
        for i, (lc, P, st) in enumerate(zip(self.cfg["layers"], self.layers, self.state)):
            h = layer_norm(x, P["norm1"], self.eps)
            u1 = canon(h, P["canon1"], st, "c1") if "canon1" in P else h
            y = x + P["ls1"] * diff_attention_step(u1, self.pos, P, lc["mixer"], self.eps, st)
            mlp = lc.get("mlp")
            if mlp:
                u2 = canon(h, P["canon2"], st, "c2") if "canon2" in P else h
                y = y + P["ls2"] * (dense_ff(u2, P, self.eps) if mlp["kind"] == "dense" else moe_ff(u2, P, mlp))
            X.append(y)
            x = sum(P["dwa"][j] * X[j] for j in range(i + 2))
            resid.append(x.copy())
        self.pos += 1
        logits = self.T["head"] @ layer_norm(x, self.T["final.norm"], self.eps)
        return (logits, np.stack(resid)) if want_residual else logits

    def run(self, tokens, want_residual=False):
        outs = [self.step(t, want_residual) for t in tokens]
        if want_residual:
            return np.stack([o[0] for o in outs]), np.stack([o[1] for o in outs], axis=1)
        return np.stack(outs)


def random_model(config, seed, bf16_round=True):
    """Random tensors of every name the config implies; values rounded to bf16 so that both dtypes load them exactly."""
    rng = np.random.default_rng(seed)
    W, V = int(config["width"]), int(config["vocab"])
    taps = int((config.get("canon") or {}).get("taps", 0))

    def mat(o, i, gain=1.0):
        return rng.standard_normal((o, i)) * gain / np.sqrt(i)

    t = {"embed": rng.standard_normal((V, W)), "head": mat(V, W), "final.norm": 1.0 + 0.1 * rng.standard_normal(W)}
    for i, lc in enumerate(config["layers"]):
        p, mc = f"l{i}.", lc["mixer"]
        H, G, dk = int(mc["heads"]), int(mc.get("kv_heads", mc["heads"])), int(mc["dim"])
        dv = int(mc.get("vdim", dk))
        t[p + "norm1"] = 1.0 + 0.1 * rng.standard_normal(W)
        for nm, rows in (("q", 2 * H * dk), ("k", 2 * G * dk), ("v", G * dv)):
            t[p + "mix." + nm] = mat(rows, W, 2.0)
            t[p + "mix." + nm + ".b"] = 0.3 * rng.standard_normal(rows)
        t[p + "mix.q.norm"] = 1.0 + 0.2 * rng.standard_normal(dk)
        t[p + "mix.k.norm"] = 1.0 + 0.2 * rng.standard_normal(dk)
        for nm in ("lq1", "lk1", "lq2", "lk2"):
            t[p + "mix." + nm] = 0.3 * rng.standard_normal(dk)
        t[p + "mix.o"] = mat(W, H * dv)
        t[p + "ls1"] = 0.5 + 0.2 * rng.standard_normal(W)
        if taps:
            t[p + "canon1"] = 0.4 * rng.standard_normal((W, taps))
        t[p + "dwa"] = rng.standard_normal(i + 2) * 0.3 + np.where(np.arange(i + 2) == i + 1, 1.0, 0.2)
        mlp = lc.get("mlp")
        if not mlp:
            continue
        t[p + "ls2"] = 0.5 + 0.2 * rng.standard_normal(W)
        if taps:
            t[p + "canon2"] = 0.4 * rng.standard_normal((W, taps))
        if mlp["kind"] == "dense":
            ff = int(mlp["ff"])
            t[p + "mlp.up"] = mat(ff, W)
            t[p + "mlp.down"] = mat(W, ff)
            t[p + "mlp.act"] = np.array([0.6, 0.3, 0.2, 0.1]) + 0.1 * rng.standard_normal(4)
        else:
            ff = int(mlp["expert"]["ff"])
            t[p + "mlp.router"] = mat(int(mlp["router"]["experts"]), W, 3.0)
            names = [f"e{e}" for e in range(int(mlp["router"]["experts"]))]
            widths = [ff] * len(names)
            if mlp.get("shared"):
                names.append("shared")
                widths.append(int(mlp["shared"]["ff"]))
            for nm, wd in zip(names, widths):
                t[p + f"mlp.{nm}.gate"] = mat(wd, W, 1.5)
                t[p + f"mlp.{nm}.up"] = mat(wd, W, 1.5)
                t[p + f"mlp.{nm}.down"] = mat(W, wd)
    if bf16_round:
        for k, v in t.items():
            u = np.ascontiguousarray(v, dtype=np.float32).view(np.uint32)
            u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
            t[k] = u.view(np.float32).astype(np.float64)
    return t
