"""Plain float64 restatement of the Savidra design, one function per mechanism, numpy only.

Test infrastructure: nothing under ntransformer_b200/ imports it and it shares no code with the product path.  It keeps no
cache and no state: every function sees the whole sequence (recurrences and convolutions are loops over time from position 0),
so the product's cache, state hand-over and schedules are checked against something that cannot have the same fault.

Notation.  X is [T, width]; weights are [out, in] and applied as x @ W.T.  `cfg` is the parsed config.json, `P` maps tensor
names to float64 arrays.  A layer is  x <- n(alpha x + mixer(shift(x)), g1),  x <- n(alpha x + ff(x), g2)  with
n(y, g) = y / sqrt(mean(y^2) + eps) (1 + g).
"""
from __future__ import annotations

import math

import numpy as np


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_zero_centred(x, w, eps):
    return rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms(x, eps) * w


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def token_shift(X, mu):
    """h_t = x_t + (x_{t-1} - x_t) mu, x_{-1} = 0."""
    prev = np.zeros_like(X)
    prev[1:] = X[:-1]
    return X + (prev - X) * mu


def causal_conv(U, w):
    """U [T, C], w [C, taps]: y_t = sum_j w[:, j] u_{t - taps + 1 + j}; the last column multiplies the current token."""
    T, C = U.shape
    taps = w.shape[1]
    pad = np.concatenate([np.zeros((taps - 1, C)), U], axis=0)
    Y = np.zeros_like(U)
    for j in range(taps):
        Y += pad[j:j + T] * w[:, j]
    return Y


def rotate_half(v, pos, dims, base, divide=1.0):
    """v [T, heads, d]: the first `dims` channels rotate, channel i with channel i + dims/2, angle pos * base^(-2i/dims) / divide."""
    if not dims:
        return v
    out = v.copy()
    half = dims // 2
    f = base ** (-2.0 * np.arange(half) / dims) / divide
    a = np.asarray(pos, dtype=np.float64).reshape(-1, 1, 1) * f
    c, s = np.cos(a), np.sin(a)
    u, w = v[..., :half], v[..., half:dims]
    out[..., :half] = u * c - w * s
    out[..., half:dims] = w * c + u * s
    return out


def rotate_for(v, pos, m):
    r = m.get("rot")
    if not r:
        return v
    sc = r.get("scaling")
    return rotate_half(v, pos, r["dims"], r["base"], sc["factor"] if sc else 1.0)


def causal_weights(q, k, scale, group, sink=None, temp=None):
    """q [T, H, D], k [T, G, D] -> softmax weights [H, T, T] over the visible keys j <= i.  sink [H]: exp(sink_h) joins the
    denominator.  temp [H]: the scores of head h are multiplied by temp[h]."""
    T, H, _ = q.shape
    Wt = np.zeros((H, T, T))
    mask = np.tril(np.ones((T, T), dtype=bool))
    for h in range(H):
        s = (q[:, h] @ k[:, h // group].T) * scale
        if temp is not None:
            s = s * temp[h]
        s = np.where(mask, s, -np.inf)
        m = s.max(axis=1, keepdims=True)
        if sink is not None:
            m = np.maximum(m, sink[h])
        e = np.exp(s - m)
        den = e.sum(axis=1, keepdims=True)
        if sink is not None:
            den = den + np.exp(sink[h] - m)
        Wt[h] = e / den
    return Wt


def apply_weights(Wt, v, group):
    """Wt [H, T, T], v [T, G, V] -> [T, H * V]; head h reads value head h // group."""
    H, T, _ = Wt.shape
    return np.stack([Wt[h] @ v[:, h // group] for h in range(H)], axis=1).reshape(T, -1)


def sink_attention(Hx, P, p, m, eps, pos, v_first=None):
    """The 'attention' mixer.  Returns (output [T, width], the values it attended over [T, G, V])."""
    T = Hx.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (Hx @ P[p + "q"].T).reshape(T, H, D)
    k = (Hx @ P[p + "k"].T).reshape(T, G, D)
    v = (Hx @ P[p + "v"].T).reshape(T, G, V)
    q = rotate_for(norm_plain(q, P[p + "q.norm"], eps), pos, m)
    k = rotate_for(norm_plain(k, P[p + "k.norm"], eps), pos, m)
    if v_first is not None:
        lam = float(np.asarray(P[p + "vmix"]).reshape(-1)[0])
        v = (1.0 - lam) * v + lam * v_first
    Wt = causal_weights(q, k, m["scale"], H // G, sink=P[p + "sink"])
    return apply_weights(Wt, v, H // G) @ P[p + "o"].T, v


def talking_attention(Hx, P, p, m, eps, pos):
    """The left half of the 'parallel' mixer: biased projections, a short convolution on q, k, v, per-head q/k norm, scaled rotary
    positions, per-head temperature, softmax, weights mixed across heads, biased output projection."""
    T = Hx.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    conv = (lambda u, n: causal_conv(u, P[p + n + ".conv"])) if m.get("conv") else (lambda u, n: u)
    q = conv(Hx @ P[p + "q"].T + P[p + "q.b"], "q").reshape(T, H, D)
    k = conv(Hx @ P[p + "k"].T + P[p + "k.b"], "k").reshape(T, G, D)
    v = conv(Hx @ P[p + "v"].T + P[p + "v.b"], "v").reshape(T, G, V)
    q = rotate_for(norm_plain(q, P[p + "q.norm"], eps), pos, m)
    k = rotate_for(norm_plain(k, P[p + "k.norm"], eps), pos, m)
    Wt = causal_weights(q, k, m["scale"], H // G, temp=P[p + "temp"])
    Wt = np.einsum("hg,gij->hij", P[p + "talk"], Wt)
    return apply_weights(Wt, v, H // G) @ P[p + "o"].T + P[p + "o.b"]


def delta_rule(q, k, v, beta, g):
    """q, k [T, H, D] (already per value head), v [T, H, V], beta [T, H], g [T, H, D] -> o [T, H, V].
    S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q."""
    T, H, D = q.shape
    V = v.shape[2]
    S = np.zeros((H, D, V))
    O = np.zeros((T, H, V))
    for t in range(T):
        for h in range(H):
            S[h] *= g[t, h][:, None]
            u = beta[t, h] * (v[t, h] - S[h].T @ k[t, h])
            S[h] += np.outer(k[t, h], u)
            O[t, h] = S[h].T @ q[t, h]
    return O


def gated_delta(Hx, P, p, m, eps):
    """The right half of the 'parallel' mixer."""
    T = Hx.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(Hx @ P[p + "q"].T, P[p + "q.conv"])).reshape(T, G, D)
    k = silu(causal_conv(Hx @ P[p + "k"].T, P[p + "k.conv"])).reshape(T, G, D)
    v = silu(causal_conv(Hx @ P[p + "v"].T, P[p + "v.conv"])).reshape(T, H, V)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * D ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    rep = H // G
    q = np.repeat(q, rep, axis=1)
    k = np.repeat(k, rep, axis=1)
    beta = sigmoid(Hx @ P[p + "b"].T)
    a = (Hx @ P[p + "a1"].T) @ P[p + "a2"].T + P[p + "dt_bias"]
    g = np.exp(-np.exp(P[p + "A_log"])[None, :, None] * softplus(a).reshape(T, H, D))
    o = delta_rule(q, k, v, beta, g)
    o = norm_plain(o, P[p + "norm"], eps)
    gate = sigmoid((Hx @ P[p + "g1"].T) @ P[p + "g2"].T).reshape(T, H, V)
    return (o * gate).reshape(T, H * V) @ P[p + "o"].T


def feed_forward(X, P, p):
    return (np.maximum(X @ P[p + "gate"].T, 0.0) * (X @ P[p + "up"].T)) @ P[p + "down"].T


def forward(cfg, P, tokens, layers_out=None):
    """Logits [T, vocab] of a whole sequence from position 0.  layers_out: a list that receives the residual after every layer."""
    eps = cfg["norm"]["eps"]
    alpha = cfg["postln_alpha"]
    X = P["embed"][np.asarray(tokens)]
    pos = np.arange(len(tokens))
    v_first = None
    for i, L in enumerate(cfg["layers"]):
        p = "l%d." % i
        m = L["mixer"]
        Hx = token_shift(X, P[p + "shift"])
        if L["type"] == "parallel":
            y = m["left_scale"] * talking_attention(Hx, P, p + "mix.left.", m["left"], eps, pos) + \
                m["right_scale"] * gated_delta(Hx, P, p + "mix.right.", m["right"], eps)
        elif L["type"] == "attention":
            mixing = bool(m.get("v_mix"))
            y, v = sink_attention(Hx, P, p + "mix.", m, eps, pos, v_first if mixing else None)
            if mixing and v_first is None:
                v_first = v
        else:
            raise ValueError(L["type"])
        X = norm_zero_centred(alpha * X + y, P[p + "norm1"], eps)
        if L.get("mlp"):
            X = norm_zero_centred(alpha * X + feed_forward(X, P, p + "mlp."), P[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(X.copy())
    return norm_zero_centred(X, P["final.norm"], eps) @ P["head"].T


# ---------------------------------------------------------------- random configurations and weights for the tests
def bf16_grid(a):
    """Values a bfloat16 holds exactly (round to nearest even), so that 16-bit and 32-bit weight storage describe the same model."""
    b = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = ((b + 0x7FFF + ((b >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return r.view(np.float32).astype(np.float64).reshape(np.shape(a))


def make_config(pattern=("parallel", "attention", "parallel", "attention"), vocab=53, width=48, ff=40, mlp=None, alpha=1.7, eps=1e-5,
                left=None, right=None, attn=None, v_mix=(1, 3), left_scale=1.3, right_scale=0.8):
    """The family's config.json as a dict.  left / right / attn override the mixers' sizes; mlp: per layer True / False; v_mix: the
    attention layers that blend their values with the first of them."""
    lf = dict(heads=4, kv_heads=2, dim=12, vdim=10, conv=3, rot_dims=8, base=10000.0, factor=4.0)
    lf.update(left or {})
    rt = dict(heads=4, kv_heads=2, dim=10, vdim=6, conv=2, decay_rank=5, gate_rank=7)
    rt.update(right or {})
    at = dict(heads=4, kv_heads=2, dim=8, vdim=12, rot_dims=4, base=500.0)
    at.update(attn or {})

    def rot_of(d, with_factor):
        if not d["rot_dims"]:
            return None
        r = {"base": d["base"], "dims": d["rot_dims"]}
        if with_factor and d.get("factor"):
            r["scaling"] = {"factor": d["factor"]}
        return r

    layers = []
    for i, typ in enumerate(pattern):
        if typ == "parallel":
            L = {"heads": lf["heads"], "kv_heads": lf["kv_heads"], "dim": lf["dim"], "vdim": lf["vdim"], "scale": lf["dim"] ** -0.5}
            if lf["conv"]:
                L["conv"] = lf["conv"]
            if rot_of(lf, True):
                L["rot"] = rot_of(lf, True)
            R = {k: rt[k] for k in ("heads", "kv_heads", "dim", "vdim", "conv", "decay_rank", "gate_rank")}
            m = {"left": L, "right": R, "left_scale": left_scale, "right_scale": right_scale}
        else:
            m = {"heads": at["heads"], "kv_heads": at["kv_heads"], "dim": at["dim"], "vdim": at["vdim"], "scale": at["dim"] ** -0.5}
            if rot_of(at, False):
                m["rot"] = rot_of(at, False)
            if i in v_mix:
                m["v_mix"] = True
        has_mlp = True if mlp is None else bool(mlp[i % len(mlp)])
        layers.append({"type": typ, "mixer": m, "mlp": {"kind": "dense", "ff": ff} if has_mlp else None})
    return {"architecture": "Savidra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "postln_alpha": alpha, "layers": layers}


def random_weights(rng, cfg):
    W = cfg["width"]
    P = {}

    def mat(rows, cols, gain=1.0):
        return bf16_grid(rng.standard_normal((rows, cols)) * gain * cols ** -0.5)

    def vec(n, mean=0.0, std=0.2):
        return bf16_grid(mean + std * rng.standard_normal(n))

    P["embed"] = mat(cfg["vocab"], W, W ** 0.5)
    P["final.norm"] = vec(W)
    P["head"] = mat(cfg["vocab"], W)
    first_mix = None
    for i, L in enumerate(cfg["layers"]):
        p = "l%d." % i
        P[p + "norm1"] = vec(W)
        P[p + "shift"] = bf16_grid(rng.uniform(0.0, 0.9, W))
        if L["type"] == "parallel":
            m = L["mixer"]["left"]
            q = p + "mix.left."
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, rows in (("q", H * D), ("k", G * D), ("v", G * V)):
                P[q + n] = mat(rows, W, 1.5)
                P[q + n + ".b"] = vec(rows, 0.0, 0.3)
                if m.get("conv"):
                    P[q + n + ".conv"] = bf16_grid(rng.standard_normal((rows, m["conv"])) * 0.6 + 0.2)
            P[q + "q.norm"] = vec(D, 1.0, 0.3)
            P[q + "k.norm"] = vec(D, 1.0, 0.3)
            P[q + "talk"] = bf16_grid(np.eye(H) * 0.7 + rng.standard_normal((H, H)) * 0.3)
            P[q + "temp"] = bf16_grid(rng.uniform(0.5, 2.0, H))
            P[q + "o"] = mat(W, H * V)
            P[q + "o.b"] = vec(W, 0.0, 0.2)
            m = L["mixer"]["right"]
            q = p + "mix.right."
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, rows in (("q", G * D), ("k", G * D), ("v", H * V)):
                P[q + n] = mat(rows, W, 1.5)
                P[q + n + ".conv"] = bf16_grid(rng.standard_normal((rows, m["conv"])) * 0.6 + 0.2)
            P[q + "b"] = mat(H, W)
            P[q + "A_log"] = bf16_grid(rng.uniform(-3.0, 0.5, H))
            P[q + "norm"] = vec(V, 1.0, 0.2)
            P[q + "a1"] = mat(m["decay_rank"], W)
            P[q + "a2"] = mat(H * D, m["decay_rank"])
            P[q + "dt_bias"] = bf16_grid(rng.uniform(-4.0, -1.0, H * D))
            P[q + "g1"] = mat(m["gate_rank"], W)
            P[q + "g2"] = mat(H * V, m["gate_rank"], 2.0)
            P[q + "o"] = mat(W, H * V)
        else:
            m = L["mixer"]
            q = p + "mix."
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            P[q + "q"] = mat(H * D, W, 1.5)
            P[q + "k"] = mat(G * D, W, 1.5)
            P[q + "v"] = mat(G * V, W)
            P[q + "q.norm"] = vec(D, 1.0, 0.3)
            P[q + "k.norm"] = vec(D, 1.0, 0.3)
            P[q + "sink"] = bf16_grid(rng.uniform(-1.0, 4.0, H))
            if m.get("v_mix"):
                P[q + "vmix"] = bf16_grid(np.array(rng.uniform(0.2, 0.6)))
            P[q + "o"] = mat(W, H * V)
        if L.get("mlp"):
            f = L["mlp"]["ff"]
            P[p + "norm2"] = vec(W)
            P[p + "mlp.gate"] = mat(f, W)
            P[p + "mlp.up"] = mat(f, W)
            P[p + "mlp.down"] = mat(W, f)
    return P


def random_model(rng, **kw):
    cfg = make_config(**kw)
    return cfg, random_weights(rng, cfg)
