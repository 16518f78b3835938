"""Plain float64 restatement of the Tanolorn design, one function per mechanism, numpy only.

Test infrastructure: nothing under ntransformer_b200/ imports it and it shares no code with the product path.  It keeps no
cache and no state: every function sees the whole sequence (the recurrences are written as loops over time), so the product's
cache, state hand-over and schedules are checked against something that cannot have the same fault.

Notation.  X is [T, width]; weights are [out, in] and applied as x @ W.T.  `cfg` is the parsed config.json, `P` maps tensor names
to float64 arrays.
"""
from __future__ import annotations

import math

import numpy as np


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_zero_centred(x, w, eps):
    """The model's norm: weight stored around zero."""
    return rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms(x, eps) * w


def silu(z):
    return z / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_half(v, pos, dims, base):
    """v [T, ..., d]: the first `dims` channels rotate, channel i with channel i + dims/2, angle pos * base^(-2i/dims)."""
    out = v.copy()
    half = dims // 2
    f = base ** (-2.0 * np.arange(half) / dims)
    a = np.asarray(pos, dtype=np.float64).reshape((-1,) + (1,) * (v.ndim - 1)) * f
    c, s = np.cos(a), np.sin(a)
    u, w = v[..., :half], v[..., half:dims]
    out[..., :half] = u * c - w * s
    out[..., half:dims] = w * c + u * s
    return out


def rotate_for(v, pos, m):
    """The mixer's rotation, or none when its configuration has no \"rot\"."""
    r = m.get("rot")
    return rotate_half(v, pos, r["dims"], r["base"]) if r and r["dims"] else v


def latent_kv(X, P, p, m, eps, pos):
    """What a latent-attention layer caches: the normed latent [T, kv_rank] and the shared rotated key part [T, rot_dim]."""
    r = m["kv_rank"]
    d = X @ P[p + "mix.dkv"].T
    c = norm_plain(d[:, :r], P[p + "mix.dkv.norm"], eps)
    kr = rotate_for(d[:, r:], pos, m)
    return c, kr


def latent_attention(X, P, p, m, eps, pos, kv):
    """kv = (c, kr) of this layer or of the layer named by kv_from; queries, W_uk, W_uv and W_o are this layer's own."""
    T = X.shape[0]
    H, D, R, V = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = kv
    cq = norm_plain(X @ P[p + "mix.dq"].T, P[p + "mix.dq.norm"], eps)
    q = (cq @ P[p + "mix.uq"].T).reshape(T, H, D + R)
    qn = q[:, :, :D]
    qr = rotate_for(q[:, :, D:], pos, m)
    kn = (c @ P[p + "mix.uk"].T).reshape(-1, H, D)
    v = (c @ P[p + "mix.uv"].T).reshape(-1, H, V)
    out = np.zeros((T, H, V))
    for h in range(H):
        s = (qn[:, h] @ kn[:, h].T + qr[:, h] @ kr.T) * m["scale"]
        s = np.where(np.tril(np.ones((T, s.shape[1]), dtype=bool)), s, -np.inf)
        s = s - s.max(axis=1, keepdims=True)
        w = np.exp(s)
        w /= w.sum(axis=1, keepdims=True)
        out[:, h] = w @ v[:, h]
    return out.reshape(T, H * V) @ P[p + "mix.o"].T


def causal_conv(u, w, b):
    """u [T, C], w [C, taps] (last column is the current token's), zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    pad = np.concatenate([np.zeros((taps - 1, C)), u], axis=0)
    out = np.tile(b, (T, 1)).astype(np.float64)
    for k in range(taps):
        out += pad[k:k + T] * w[:, k]
    return out


def mamba2(X, P, p, m, eps):
    T = X.shape[0]
    H, V, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * V
    u = X @ P[p + "mix.in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, P[p + "mix.conv"], P[p + "mix.conv.b"]))
    x = xbc[:, :inner].reshape(T, H, V)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + P[p + "mix.dt_bias"])
    A = -np.exp(P[p + "mix.A_log"])
    Dk = P[p + "mix.D"]
    y = np.zeros((T, H, V))
    S = np.zeros((H, N, V))
    per = H // G
    for t in range(T):
        for h in range(H):
            g = h // per
            S[h] = math.exp(A[h] * dt[t, h]) * S[h] + dt[t, h] * np.outer(B[t, g], x[t, h])
            y[t, h] = S[h].T @ C[t, g] + Dk[h] * x[t, h]
    y = y.reshape(T, inner) * silu(z)
    ng = m["norm_groups"]
    y = rms(y.reshape(T, ng, inner // ng), eps).reshape(T, inner) * P[p + "mix.norm"]
    return y @ P[p + "mix.o"].T


def dense_ff(X, P, p):
    g = X @ P[p + "mlp.gate"].T + P[p + "mlp.gate.b"]
    u = X @ P[p + "mlp.up"].T + P[p + "mlp.up.b"]
    return (silu(g) * u) @ P[p + "mlp.down"].T + P[p + "mlp.down.b"]


def route(X, P, p, mlp):
    """Chosen experts [T, top] and their weights.  Sigmoid scores; the choice adds the correction; only the best `keep` groups
    (a group scores the sum of its two largest choice scores) can be chosen; weights are the plain scores of the chosen."""
    r = mlp["router"]
    E, top = r["experts"], r["top"]
    s = 1.0 / (1.0 + np.exp(-(X @ P[p + "mlp.router"].T)))
    ch = s + P[p + "mlp.correction"]
    grp = r.get("groups")
    if grp:
        n, keep = grp["count"], grp["keep"]
        per = E // n
        gs = np.sort(ch.reshape(-1, n, per), axis=2)[:, :, -2:].sum(axis=2) if per >= 2 else ch.reshape(-1, n, per).sum(axis=2)
        best = np.argsort(-gs, axis=1, kind="stable")[:, :keep]
        allowed = np.zeros((X.shape[0], n), dtype=bool)
        np.put_along_axis(allowed, best, True, axis=1)
        ch = np.where(np.repeat(allowed, per, axis=1), ch, -np.inf)
    sel = np.argsort(-ch, axis=1, kind="stable")[:, :top]
    return sel, np.take_along_axis(s, sel, axis=1)


def moe_ff(X, P, p, mlp):
    sel, wt = route(X, P, p, mlp)
    out = np.zeros_like(X)
    for t in range(X.shape[0]):
        for k in range(sel.shape[1]):
            q = p + "mlp.e%d." % sel[t, k]
            h = silu(X[t] @ P[q + "gate"].T) * (X[t] @ P[q + "up"].T)
            out[t] += wt[t, k] * (h @ P[q + "down"].T)
    return out


def token_side(X, tokens, P, p, i, dim, eps):
    e = P["side.embed"][tokens][:, i * dim:(i + 1) * dim]
    g = gelu_tanh(X @ P[p + "side.gate"].T) * e
    y = g @ P[p + "side.proj"].T
    return norm_plain(y, P[p + "side.norm"], eps)


def forward(cfg, P, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence from position 0.  layers_out (a list) receives the residual stream after every layer."""
    tokens = np.asarray(tokens)
    eps = cfg["norm"]["eps"]
    pos = np.arange(len(tokens))
    X = P["embed"][tokens].astype(np.float64)
    side = cfg.get("token_side")
    kvs = {}
    for i, L in enumerate(cfg["layers"]):
        p = "l%d." % i
        m = L["mixer"]
        if L["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                kvs[i] = latent_kv(X, P, p, m, eps, pos)
                src = i
            y = latent_attention(X, P, p, m, eps, pos, kvs[src])
        elif L["type"] == "mamba2":
            y = mamba2(X, P, p, m, eps)
        else:
            raise ValueError(L["type"])
        X = X + norm_zero_centred(y, P[p + "norm1"], eps)
        mlp = L.get("mlp")
        if mlp:
            y = dense_ff(X, P, p) if mlp["kind"] == "dense" else moe_ff(X, P, p, mlp)
            X = X + norm_zero_centred(y, P[p + "norm2"], eps)
        if side:
            X = X + token_side(X, tokens, P, p, i, side["dim"], eps)
        if layers_out is not None:
            layers_out.append(X.copy())
    return norm_zero_centred(X, P["final.norm"], eps) @ P["head"].T


# ---------------------------------------------------------------- random models for the tests
def _bf16(a):
    """Round to values bfloat16 holds exactly, so that a 16-bit checkpoint and the float64 oracle see the same weights."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).astype(np.float64)


def random_model(rng, vocab=41, width=40, pattern=("scan", "latent", "scan", "latent"), kv_from=None, mlp=("dense", "moe", "moe", None),
                 heads=3, dim=8, rot_dim=6, vdim=10, q_rank=12, kv_rank=20, rot_dims=None, base=50.0, scale=None,
                 s_heads=4, s_vdim=6, state=12, groups=2, conv=4, norm_groups=2,
                 ff=24, experts=6, top=2, eff=10, route_groups=(3, 2), side=5, eps=1e-5, corr_shift=0.0):
    """(config dict, weights dict).  pattern: mixer per layer; mlp: feed-forward kind per layer (None: none); kv_from: {layer: earlier
    latent layer whose cache rows it reads}; route_groups: (count, keep) or None; side: width of the per-layer token input (0: none)."""
    kv_from = kv_from or {}
    layers = []
    for i, kind in enumerate(pattern):
        if kind == "latent":
            m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                 "scale": float(scale if scale is not None else (dim + rot_dim) ** -0.5)}
            if rot_dim:
                m["rot"] = {"dims": rot_dim if rot_dims is None else rot_dims, "base": base}
            if i in kv_from:
                m["kv_from"] = kv_from[i]
            typ = "latent_attention"
        else:
            m = {"heads": s_heads, "vdim": s_vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}
            typ = "mamba2"
        k = mlp[i % len(mlp)]
        if k == "dense":
            f = {"kind": "dense", "ff": ff}
        elif k == "moe":
            r = {"experts": experts, "top": top}
            if route_groups:
                r["groups"] = {"count": route_groups[0], "keep": route_groups[1]}
            f = {"kind": "moe", "expert": {"ff": eff}, "router": r}
        else:
            f = None
        layers.append({"type": typ, "mixer": m, "mlp": f})
    cfg = {"architecture": "Tanolorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if side:
        cfg["token_side"] = {"dim": side}
    mat = lambda r, c, s=1.0: _bf16(rng.standard_normal((r, c)) * s * c ** -0.5)
    gain0 = lambda n: _bf16(0.2 * rng.standard_normal(n))          # stored around zero
    gain1 = lambda n: _bf16(1.0 + 0.2 * rng.standard_normal(n))
    W = {"embed": _bf16(rng.standard_normal((vocab, width))), "final.norm": gain0(width), "head": mat(vocab, width)}
    if side:
        W["side.embed"] = _bf16(rng.standard_normal((vocab, len(layers) * side)))
    for i, e in enumerate(layers):
        p, m = "l%d." % i, e["mixer"]
        W[p + "norm1"] = gain0(width)
        if e["type"] == "latent_attention":
            W[p + "mix.dq"] = mat(q_rank, width)
            W[p + "mix.dq.norm"] = gain1(q_rank)
            W[p + "mix.uq"] = mat(heads * (dim + rot_dim), q_rank, 1.5)
            if "kv_from" not in m:
                W[p + "mix.dkv"] = mat(kv_rank + rot_dim, width)
                W[p + "mix.dkv.norm"] = gain1(kv_rank)
            W[p + "mix.uk"] = mat(heads * dim, kv_rank, 1.5)
            W[p + "mix.uv"] = mat(heads * vdim, kv_rank)
            W[p + "mix.o"] = mat(width, heads * vdim)
        else:
            inner, ch = s_heads * s_vdim, s_heads * s_vdim + 2 * groups * state
            W[p + "mix.in"] = mat(inner + ch + s_heads, width)
            W[p + "mix.conv"] = _bf16(rng.standard_normal((ch, conv)) * conv ** -0.5)
            W[p + "mix.conv.b"] = _bf16(0.1 * rng.standard_normal(ch))
            W[p + "mix.dt_bias"] = _bf16(rng.uniform(-3.0, 0.5, s_heads))
            W[p + "mix.A_log"] = _bf16(np.log(rng.uniform(0.5, 4.0, s_heads)))
            W[p + "mix.D"] = _bf16(1.0 + 0.3 * rng.standard_normal(s_heads))
            W[p + "mix.norm"] = gain1(inner)
            W[p + "mix.o"] = mat(width, inner)
        f = e["mlp"]
        if f:
            W[p + "norm2"] = gain0(width)
            if f["kind"] == "dense":
                for n, (r, c) in (("gate", (ff, width)), ("up", (ff, width)), ("down", (width, ff))):
                    W[p + "mlp." + n] = mat(r, c)
                    W[p + "mlp." + n + ".b"] = _bf16(0.2 * rng.standard_normal(r))
            else:
                W[p + "mlp.router"] = mat(experts, width, 2.0)
                W[p + "mlp.correction"] = _bf16(0.3 * rng.standard_normal(experts) + corr_shift)
                for x in range(experts):
                    W[p + "mlp.e%d.gate" % x] = mat(eff, width)
                    W[p + "mlp.e%d.up" % x] = mat(eff, width)
                    W[p + "mlp.e%d.down" % x] = mat(width, eff)
        if side:
            W[p + "side.gate"] = mat(side, width)
            W[p + "side.proj"] = mat(width, side)
            W[p + "side.norm"] = gain1(width)
    return cfg, W
