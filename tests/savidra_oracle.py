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
        lam = float(P[p + "vmix"])
        v = (1.0 - lam) * v + lam * v_first
    Wt = causal_weights(q, k, m["scale"], H // G, sink=P[p + "sink"])
    return apply_weights(Wt, v, H // G) @ P[p + "o"].T, v


def talking_attention(Hx, P, p, m, eps, pos):
    """The left half of the 'parallel' mixer: biased projections, a short convolution on q, k, v, per-head q/k norm, scaled rotary
    positions, per-head temperature, softmax, weights mixed across heads, biased output projection."""
    T = Hx.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv(Hx @ P[p + "q"].T + P[p + "q.b"], P[p + "q.conv"]).reshape(T, H, D)
    k = causal_conv(Hx @ P[p + "k"].T + P[p + "k.b"], P[p + "k.conv"]).reshape(T, G, D)
    v = causal_conv(Hx @ P[p + "v"].T + P[p + "v.b"], P[p + "v.conv"]).reshape(T, G, V)
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
