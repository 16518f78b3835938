"""Savidra on the GPU against the plain float64 oracle (tests/savidra_oracle.py): each mechanism's kernel alone, then whole models
through the engine's step function — prompt pass vs token-by-token decoding, portions down to two tokens, cache rows and every carried
state reused by a second request, keys far away and at the borders of the kernels' key groups, the first tokens, sizes that are odd, 1
or equal where the usual ones differ, long decoding with and without graph replay, and greedy generation through the engine's entry
point."""
import ctypes as C

import numpy as np
import pytest
import torch

import savidra_oracle as O
from savidra_util import device_tensors
from zelunex_util import rel_rms, write_model_dir

from ntransformer_b200._lib import lib
from ntransformer_b200.dtypes import DType
from ntransformer_b200.engine import Engine, Model

pytestmark = pytest.mark.gpu


def dev(a, dt=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda().to(dt).contiguous()


def stream():
    return torch.cuda.current_stream().cuda_stream


def host(t):
    return t.double().cpu().numpy()


def ptr(t):
    return t.data_ptr() if t is not None else None


_KEPT = []


def dp(a):
    """Device pointer of a fresh copy of `a`; the copy lives until the test ends (the launches are asynchronous)."""
    t = dev(a)
    _KEPT.append(t)
    return t.data_ptr()


@pytest.fixture(autouse=True)
def _release_kept():
    yield
    torch.cuda.synchronize()
    _KEPT.clear()


def ptr_array(ts):
    return (C.c_void_p * len(ts))(*[ptr(t) for t in ts])


def int_array(v):
    return (C.c_int * len(v))(*v)


# ---------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("width", [1, 7, 300])
def test_token_shift_carries_the_previous_row(width):
    rng = np.random.default_rng(width)
    T = 23
    X, mu = rng.standard_normal((T, width)), rng.uniform(0, 1, width)
    ref = O.token_shift(X, mu)
    for sizes in ([T], [1] * T, [2, 1, 9, 11]):
        carried = dev(rng.standard_normal(width))                  # stale numbers of an earlier sequence: position 0 must not read them
        got, pos = [], 0
        for n in sizes:
            h = torch.empty(n, width, device="cuda")
            lib().nt_b200_token_shift_rows(h.data_ptr(), dp(X[pos:pos + n]), dp(mu), carried.data_ptr(), n, width, pos, stream())
            got.append(host(h)); pos += n
        np.testing.assert_allclose(np.concatenate(got), ref, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_short_convolutions_carry_their_last_inputs(taps):
    """Three projections in one launch, each with its own width, bias and activation; portions shorter than the taps too."""
    rng = np.random.default_rng(taps)
    T, chs, acts = 29, [5, 300, 64], [0, 1, 0]
    U = [rng.standard_normal((T, c)) for c in chs]
    Wt = [rng.standard_normal((c, taps)) for c in chs]
    B = [rng.standard_normal(chs[0]), None, rng.standard_normal(chs[2])]
    ref = []
    for u, w, b, a in zip(U, Wt, B, acts):
        y = O.causal_conv(u + (b if b is not None else 0.0), w)
        ref.append(O.silu(y) if a else y)
    for sizes in ([T], [1] * T, [2, 1, 3, 1, 22]):
        state = [dev(rng.standard_normal((max(taps - 1, 1), c))) for c in chs]
        outs, pos = [[] for _ in chs], 0
        for n in sizes:
            u = [dev(x[pos:pos + n]) for x in U]
            o = [torch.empty(n, c, device="cuda") for c in chs]
            w = [dev(x) for x in Wt]
            b = [dev(x) if x is not None else None for x in B]
            lib().nt_b200_short_conv(ptr_array(u), ptr_array(o), ptr_array(w), ptr_array(b), ptr_array(state), int_array(chs), int_array([taps] * 3), int_array(acts),
                                     3, n, pos, stream())
            for i in range(3):
                outs[i].append(host(o[i]))
            pos += n
        for i in range(3):
            np.testing.assert_allclose(np.concatenate(outs[i]), ref[i], rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("cache", [DType.F32, DType.BF16])
@pytest.mark.parametrize("H,G,D,V,dims,divide", [(4, 2, 12, 10, 8, 4.0), (3, 3, 7, 5, 6, 1.0), (2, 1, 64, 64, 64, 8.0), (1, 1, 2, 1, 0, 1.0)])
def test_head_norm_rotation_multiplier_blend_and_cache_write(cache, H, G, D, V, dims, divide):
    rng = np.random.default_rng(H * 100 + D)
    T, p0, n, eps = 9, 37, 64, 1e-5
    Q, K, Vv = rng.standard_normal((T, H, D)), rng.standard_normal((T, G, D)), rng.standard_normal((T, G, V))
    qg, kg, temp = rng.uniform(0.5, 1.5, D), rng.uniform(0.5, 1.5, D), rng.uniform(0.5, 2.0, H)
    first, lam = rng.standard_normal((T, G, V)), 0.37
    pos = np.arange(p0, p0 + T)
    rot = {"rot": {"dims": dims, "base": 1000.0, "scaling": {"factor": divide}}} if dims else {}
    q_ref = O.rotate_for(O.norm_plain(Q, qg, eps), pos, rot) * temp[None, :, None]
    k_ref = O.rotate_for(O.norm_plain(K, kg, eps), pos, rot)
    v_ref = (1 - lam) * Vv + lam * first
    freq = dev(1000.0 ** (-2.0 * np.arange(dims // 2) / max(dims, 1)) / divide) if dims else None
    tdt = torch.float32 if cache == DType.F32 else torch.bfloat16
    kc, vc = torch.zeros(n, G * D, device="cuda", dtype=tdt), torch.zeros(n, G * V, device="cuda", dtype=tdt)
    q, pub = dev(Q), torch.zeros(T, G * V, device="cuda")
    lib().nt_b200_head_prep(q.data_ptr(), dp(K), dp(Vv), H, G, D, V, dp(qg), dp(kg), eps, dims, 0, ptr(freq),
                            dp(temp), dp(np.array([lam])), dp(first), None, kc.data_ptr(), vc.data_ptr(), int(cache), T, p0, stream())
    tol = 2e-5 if cache == DType.F32 else 1e-2
    np.testing.assert_allclose(host(q).reshape(T, H, D), q_ref, rtol=2e-5, atol=2e-5)
    np.testing.assert_allclose(host(kc[p0:p0 + T]).reshape(T, G, D), k_ref, rtol=tol, atol=tol)
    np.testing.assert_allclose(host(vc[p0:p0 + T]).reshape(T, G, V), v_ref, rtol=tol, atol=tol)
    assert float(kc[:p0].abs().sum()) == 0 and float(kc[p0 + T:].abs().sum()) == 0                # only the step's rows are written
    # publishing: the values as projected go out, the cache holds them unblended
    lib().nt_b200_head_prep(q.data_ptr(), dp(K), dp(Vv), H, G, D, V, None, None, eps, 0, 0, None, None, None, None, pub.data_ptr(),
                            kc.data_ptr(), vc.data_ptr(), int(cache), T, p0, stream())
    np.testing.assert_allclose(host(pub).reshape(T, G, V), Vv, rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(host(vc[p0:p0 + T]).reshape(T, G, V), Vv, rtol=tol, atol=tol)
    np.testing.assert_allclose(host(kc[p0:p0 + T]).reshape(T, G, D), K, rtol=tol, atol=tol)    # no gains, no rotation: keys as they came


def attention_ref(Q, K, Vv, scale, sink=None, talk=None):
    H, G = Q.shape[1], K.shape[1]
    Wt = O.causal_weights(Q, K, scale, H // G, sink=sink)
    if talk is not None:
        Wt = np.einsum("hg,gij->hij", talk, Wt)
    return O.apply_weights(Wt, Vv, H // G)


def run_attention(Q, K, Vv, scale, sink, talk, cache, sizes, one_pass=1):
    """Cache rows written up front (positions = rows); queries run in portions, each over the rows up to its own position."""
    S, H, D = Q.shape
    G, V = K.shape[1], Vv.shape[2]
    tdt = torch.float32 if cache == DType.F32 else torch.bfloat16
    kc, vc = dev(K.reshape(S, -1), tdt), dev(Vv.reshape(S, -1), tdt)
    out, pos = [], 0
    for n in sizes:
        o = torch.empty(n, H * V, device="cuda")
        scratch = torch.empty(n * H * G * V, device="cuda") if talk is not None else None
        lib().nt_b200_attention_heads(o.data_ptr(), dp(Q[pos:pos + n]), kc.data_ptr(), vc.data_ptr(), int(cache), n, pos, S, H, G, D, V, scale,
                                      dp(sink) if sink is not None else None, dp(talk) if talk is not None else None, ptr(scratch), one_pass, stream())
        torch.cuda.synchronize()
        out.append(host(o)); pos += n
    return np.concatenate(out)


@pytest.mark.parametrize("H,G,D,V", [(4, 2, 12, 10), (3, 3, 5, 7), (8, 2, 64, 32), (2, 1, 33, 1), (6, 6, 16, 100)])
def test_sink_and_head_mixed_attention(H, G, D, V):
    rng = np.random.default_rng(H + D)
    S = 75
    Q, K, Vv = rng.standard_normal((S, H, D)), rng.standard_normal((S, G, D)), rng.standard_normal((S, G, V))
    sink, talk = rng.uniform(-1, 3, H), np.eye(H) * 0.6 + rng.standard_normal((H, H)) * 0.4
    scale = D ** -0.5
    for sizes in ([S], [40] + [1] * 35, [2, 3, 17, 53]):
        np.testing.assert_allclose(run_attention(Q, K, Vv, scale, sink, None, DType.F32, sizes), attention_ref(Q, K, Vv, scale, sink=sink), rtol=2e-5, atol=2e-5)
        for one_pass in ((1, 0) if G * V <= 512 else (0,)):     # every value head in one pass (up to 512 numbers) / one pass per value head: the same numbers
            got = run_attention(Q, K, Vv, scale, None, talk, DType.F32, sizes, one_pass)
            np.testing.assert_allclose(got, attention_ref(Q, K, Vv, scale, talk=talk), rtol=3e-5, atol=3e-5)
    b = lambda a: O.bf16_grid(a)
    got = run_attention(Q, b(K), b(Vv), scale, sink, None, DType.BF16, [S])
    np.testing.assert_allclose(got, attention_ref(Q, b(K), b(Vv), scale, sink=sink), rtol=2e-5, atol=2e-5)


def test_a_sink_takes_its_share_and_nothing_else():
    """All keys equal: every weight is 1 / (n + e^sink / e^score); with a huge sink the output vanishes, with a tiny one it is the plain mean."""
    S, H, D, V = 40, 2, 8, 4
    Q, K, Vv = np.ones((S, H, D)), np.zeros((S, 1, D)), np.ones((S, 1, V))
    for sink, share in ((np.log(3.0), lambda n: n / (n + 3.0)), (-80.0, lambda n: 1.0), (80.0, lambda n: 0.0)):
        got = run_attention(Q, K, Vv, 1.0, np.full(H, sink), None, DType.F32, [30] + [1] * 10)
        want = np.array([share(i + 1.0) for i in range(S)])
        np.testing.assert_allclose(got, np.repeat(want[:, None], H * V, 1), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("far", [0, 1, 31, 32, 255, 256, 257, 1023])
@pytest.mark.parametrize("talking", [False, True])
def test_one_loud_key_among_a_thousand(far, talking):
    """One key far back matches the queries, a thousand others do not: its value must come through, wherever it lies against the kernels'
    groups of 32 keys, the tiles of 64 and the slices of a decoded token's cluster — in a prompt, in portions and when decoding."""
    rng = np.random.default_rng(far)
    S, H, G, D, V = 1100, 4, 2, 16, 8
    Q, K, Vv = rng.standard_normal((S, H, D)) * 0.1, rng.standard_normal((S, G, D)) * 0.1, rng.standard_normal((S, G, V))
    Q[:, :, 0] = 6.0
    K[far, :, 0] = 6.0
    Vv[far] = 50.0
    talk = np.eye(H) * 0.5 + 0.1 if talking else None
    sink = None if talking else np.zeros(H)
    ref = attention_ref(Q, K, Vv, 1.0, sink=sink, talk=talk)
    assert np.abs(ref[-1]).min() > 20.0                                      # the far value dominates the last rows
    for sizes in ([S], [1040] + [1] * 60, [far + 1, S - far - 1] if far + 1 < S else [S]):
        got = run_attention(Q, K, Vv, 1.0, sink, talk, DType.F32, sizes)
        np.testing.assert_allclose(got[far:], ref[far:], rtol=1e-4, atol=1e-4)
        if far > 0:
            assert np.abs(got[far - 1]).max() < 10.0                          # and nobody sees it before its position


def delta_inputs(rng, T, H, G, D, V):
    q, k = rng.standard_normal((T, G, D)), rng.standard_normal((T, G, D))
    v = rng.standard_normal((T, H, V))
    a_raw, b_raw = rng.standard_normal((T, H, D)), rng.standard_normal((T, H))
    dt_bias, A_log = rng.uniform(-4, -1, H * D), rng.uniform(-3, 0.5, H)
    return q, k, v, a_raw, b_raw, dt_bias, A_log


def delta_ref(q, k, v, a_raw, b_raw, dt_bias, A_log):
    T, G, D = q.shape
    H = v.shape[1]
    qn = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * D ** -0.5
    kn = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    g = np.exp(-np.exp(A_log)[None, :, None] * O.softplus(a_raw + dt_bias.reshape(H, D)))
    return O.delta_rule(np.repeat(qn, H // G, 1), np.repeat(kn, H // G, 1), v, O.sigmoid(b_raw), g), g


@pytest.mark.parametrize("H,G,D,V", [(4, 2, 10, 6), (6, 6, 32, 64), (2, 1, 1, 1), (3, 1, 17, 5), (2, 2, 64, 20), (2, 1, 128, 33), (1, 1, 256, 9), (2, 2, 200, 40)])
def test_delta_rule_and_state_hand_over(H, G, D, V):
    rng = np.random.default_rng(H * 1000 + D)
    T = 45
    q, k, v, a_raw, b_raw, dt_bias, A_log = delta_inputs(rng, T, H, G, D, V)
    ref, _ = delta_ref(q, k, v, a_raw, b_raw, dt_bias, A_log)
    for sizes in ([T], [1] * T, [2, 16, 1, 17, 9]):
        state = dev(rng.standard_normal((H, V, D)))                           # stale: a step at position 0 starts from zeros
        got, pos = [], 0
        for n in sizes:
            sl = slice(pos, pos + n)
            dq, dk, da, db = dev(q[sl]), dev(k[sl]), dev(a_raw[sl]), dev(b_raw[sl])
            qk, out = torch.empty(n, G, device="cuda"), torch.empty(n, H, V, device="cuda")
            lib().nt_b200_delta_prep(dq.data_ptr(), dk.data_ptr(), da.data_ptr(), db.data_ptr(), qk.data_ptr(), dp(dt_bias), dp(A_log), n, H, G, D,
                                     stream())
            lib().nt_b200_delta_rule_rows(out.data_ptr(), dq.data_ptr(), dk.data_ptr(), dp(v[sl]), da.data_ptr(), db.data_ptr(), qk.data_ptr(),
                                          state.data_ptr(), n, H, G, D, V, pos, stream())
            got.append(host(out)); pos += n
        np.testing.assert_allclose(np.concatenate(got), ref, rtol=2e-4, atol=2e-5)


def test_delta_rule_keeps_a_far_write_under_slow_decay_and_loses_it_under_fast():
    rng = np.random.default_rng(5)
    T, H, G, D, V = 700, 2, 1, 8, 4
    q, k, v, a_raw, b_raw, dt_bias, _ = delta_inputs(rng, T, H, G, D, V)
    # token 3 writes along key channel 0, which no later key touches (a later key along it would overwrite the entry: that is the
    # rule's own forgetting); every query reads that channel, so only the decay stands between the write and the last row
    k[:, :, 0] = 0.0; k[3] = 0.0; k[3, :, 0] = 1.0
    q[:, :, 0] = 2.0
    v[3] = 40.0
    for A_log, alive in ((np.full(H, -9.0), True), (np.full(H, 3.0), False)):
        ref, g = delta_ref(q, k, v, a_raw, b_raw, dt_bias, A_log)
        dq, dk, da, db = dev(q), dev(k), dev(a_raw), dev(b_raw)
        qk, out, state = torch.empty(T, G, device="cuda"), torch.empty(T, H, V, device="cuda"), torch.zeros(H, V, D, device="cuda")
        lib().nt_b200_delta_prep(dq.data_ptr(), dk.data_ptr(), da.data_ptr(), db.data_ptr(), qk.data_ptr(), dp(dt_bias), dp(A_log), T, H, G, D, stream())
        np.testing.assert_allclose(host(da).reshape(T, H, D), g, rtol=1e-5, atol=1e-7)
        lib().nt_b200_delta_rule_rows(out.data_ptr(), dq.data_ptr(), dk.data_ptr(), dp(v), da.data_ptr(), db.data_ptr(), qk.data_ptr(), state.data_ptr(), T, H, G,
                                      D, V, 0, stream())
        np.testing.assert_allclose(host(out), ref, rtol=5e-4, atol=5e-5)
        v2 = v.copy(); v2[3] = 0.0
        moved = np.abs(ref[-1] - delta_ref(q, k, v2, a_raw, b_raw, dt_bias, A_log)[0][-1]).max()
        assert (moved > 1e-2) == alive


@pytest.mark.parametrize("H,V", [(4, 6), (1, 1), (3, 200)])
def test_delta_output_norm_and_gate(H, V):
    rng = np.random.default_rng(V)
    T, eps = 11, 1e-5
    o, graw, gain = rng.standard_normal((T, H, V)), rng.standard_normal((T, H, V)), rng.uniform(0.5, 1.5, V)
    out = torch.empty(T, H, V, device="cuda")
    lib().nt_b200_delta_gate_norm(out.data_ptr(), dp(o), dp(graw), dp(gain), eps, T, H, V, stream())
    np.testing.assert_allclose(host(out), O.norm_plain(o, gain, eps) * O.sigmoid(graw), rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("width", [1, 48, 1000])
def test_norm_of_the_residual_sum_with_the_next_shift(width):
    rng = np.random.default_rng(width)
    T, eps, a, s1, s2 = 7, 1e-5, 1.7, 1.3, 0.8
    X, Y1, Y2 = (rng.standard_normal((T, width)) for _ in range(3))
    b1, g = rng.standard_normal(width), 1.0 + 0.2 * rng.standard_normal(width)
    for two, bias in ((True, True), (False, False), (True, False)):
        ref = O.rms(a * X + s1 * (Y1 + (b1 if bias else 0.0)) + (s2 * Y2 if two else 0.0), eps) * g
        x = dev(X)
        lib().nt_b200_sum_rmsnorm_rows(x.data_ptr(), a, dp(Y1), s1, dp(b1) if bias else None, dp(Y2) if two else None, s2, dp(g), T, width,
                                       eps, None, None, None, 0, stream())
        np.testing.assert_allclose(host(x), ref, rtol=2e-5, atol=2e-6)
    # one row at a time with the shift riding along: the same as shifting the normed rows afterwards
    ref = O.rms(a * X + s1 * Y1, eps) * g
    mu = rng.uniform(0, 1, width)
    carried, hs = dev(rng.standard_normal(width)), []
    for t in range(T):
        x, h = dev(X[t:t + 1]), torch.empty(1, width, device="cuda")
        lib().nt_b200_sum_rmsnorm_rows(x.data_ptr(), a, dp(Y1[t:t + 1]), s1, None, None, 0.0, dp(g), 1, width, eps, h.data_ptr(), dp(mu),
                                       carried.data_ptr(), t, stream())
        hs.append(host(h))
    np.testing.assert_allclose(np.concatenate(hs), O.token_shift(ref, mu), rtol=3e-5, atol=3e-6)


# ---------------------------------------------------------------- whole models through the engine
def build(cfg, W, exact, max_context=256):
    return Model.from_config_json(cfg, device_tensors(W, exact), max_context=max_context, exact_f32=exact)


def run_portions(model, toks, sizes):
    rows, pos = [], 0
    for n in sizes:
        rows.append(model.forward_logits(toks[pos:pos + n], pos, list(range(n))))
        pos += n
    assert pos == len(toks)
    return np.concatenate(rows)


CONFIGS = {
    "base": dict(),
    "attention_only": dict(pattern=("attention", "attention", "attention"), v_mix=(0, 2), mlp=(True, False, True)),
    "pairs_only_no_feed_forward": dict(pattern=("parallel", "parallel"), mlp=(False, True)),
    "attention_first_single_blend": dict(pattern=("attention", "parallel", "attention"), v_mix=(2,)),
    "every_size_one": dict(width=3, vocab=5, ff=1, left=dict(heads=1, kv_heads=1, dim=2, vdim=1, conv=1, rot_dims=2, factor=1.0),
                           right=dict(heads=1, kv_heads=1, dim=1, vdim=1, conv=1, decay_rank=1, gate_rank=1), attn=dict(heads=1, kv_heads=1, dim=2, vdim=1, rot_dims=2)),
    "all_heads_their_own_wide_values": dict(left=dict(heads=6, kv_heads=6, dim=6, vdim=90, conv=5, rot_dims=6, factor=None), right=dict(heads=6, kv_heads=6, dim=7, vdim=3, conv=4),
                                            attn=dict(heads=3, kv_heads=3, dim=9, vdim=9, rot_dims=8), alpha=1.0, left_scale=1.0, right_scale=1.0),
    "no_rotation_no_convolution_on_the_left": dict(left=dict(rot_dims=0, conv=0, heads=6, kv_heads=1), attn=dict(rot_dims=0, heads=2, kv_heads=1), right=dict(heads=6, kv_heads=1, dim=40, vdim=5)),
    # tile-aligned matrices: with BF16 weights the projections run on the tensor cores and the attentions on the tiled kernel
    "tensor_core_tiles": dict(pattern=("parallel", "attention"), v_mix=(), width=128, vocab=128, ff=128, left=dict(heads=4, kv_heads=2, dim=64, vdim=64, rot_dims=64),
                              right=dict(heads=4, kv_heads=2, dim=32, vdim=32, decay_rank=8, gate_rank=8), attn=dict(heads=2, kv_heads=2, dim=64, vdim=64, rot_dims=32)),
}


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("exact", [True, False])
def test_model_schedules_agree_with_oracle(name, exact):
    rng = np.random.default_rng(len(name))
    cfg, W = O.random_model(rng, **CONFIGS[name])
    S = 61
    toks = rng.integers(0, cfg["vocab"], S).astype(np.int32)
    ref = O.forward(cfg, W, toks)
    m = build(cfg, W, exact)
    tol = 3e-4 if exact else 3e-2                                        # 16-bit cache rows in the second mode; everything else is F32 there too
    whole = run_portions(m, toks, [S])
    assert rel_rms(whole, ref) < tol
    single = run_portions(m, toks, [1] * S)
    assert rel_rms(single, ref) < tol
    mixed = run_portions(m, toks, [2, 17, 3, 2, 20, 5, 1, 1, 8, 2])      # portions cut anywhere, shorter than the convolutions too
    assert rel_rms(mixed, ref) < tol
    assert rel_rms(run_portions(m, toks, [40] + [1] * 21), ref) < tol
    if exact:                                                            # how a prompt is cut changes rounding only
        assert rel_rms(single, whole) < 1e-4 and rel_rms(mixed, whole) < 1e-4
    m.close()


def test_residual_after_every_mechanism_matches():
    """Models of one layer each, so that a fault names its mechanism."""
    for k, kw in enumerate((dict(pattern=("attention",), mlp=(False,), v_mix=()), dict(pattern=("attention",), mlp=(True,), v_mix=(0,)),
                            dict(pattern=("parallel",), mlp=(False,), right_scale=0.0), dict(pattern=("parallel",), mlp=(False,), left_scale=0.0),
                            dict(pattern=("parallel",), mlp=(True,)))):
        rng = np.random.default_rng(k)
        cfg, W = O.random_model(rng, **kw)
        toks = rng.integers(0, cfg["vocab"], 30).astype(np.int32)
        m = build(cfg, W, True)
        assert rel_rms(run_portions(m, toks, [30]), O.forward(cfg, W, toks)) < 1e-4, kw
        assert rel_rms(run_portions(m, toks, [1] * 30), O.forward(cfg, W, toks)) < 1e-4, kw
        m.close()


def test_first_tokens_and_single_token_request():
    rng = np.random.default_rng(2)
    cfg, W = O.random_model(rng)
    toks = rng.integers(0, cfg["vocab"], 5).astype(np.int32)
    ref = O.forward(cfg, W, toks)
    m = build(cfg, W, True)
    assert rel_rms(run_portions(m, toks[:1], [1]), ref[:1]) < 2e-4
    assert rel_rms(run_portions(m, toks, [2, 3]), ref) < 2e-4
    assert rel_rms(run_portions(m, toks, [1, 1, 1, 2]), ref) < 2e-4
    m.close()


def test_rows_and_states_are_reused_between_requests():
    """A second request starts at position 0 over the first one's cache rows, shifted rows, convolution inputs and matrix states:
    bit-equal to running alone."""
    rng = np.random.default_rng(21)
    cfg, W = O.random_model(rng)
    a = rng.integers(0, cfg["vocab"], 50).astype(np.int32)
    b = rng.integers(0, cfg["vocab"], 30).astype(np.int32)
    for first in ([50], [20] + [1] * 30):
        m = build(cfg, W, True)
        run_portions(m, a, first)
        after_a = run_portions(m, b, [18] + [1] * 12)
        m2 = build(cfg, W, True)
        alone = run_portions(m2, b, [18] + [1] * 12)
        np.testing.assert_array_equal(after_a, alone)
        assert rel_rms(alone, O.forward(cfg, W, b)) < 2e-4
        after_a = run_portions(m, b[:3], [1, 1, 1])                      # and again, decoding from the very first token
        np.testing.assert_array_equal(after_a, run_portions(m2, b[:3], [1, 1, 1]))
        m.close(); m2.close()


def test_prompt_longer_than_one_portion_of_the_engine():
    """2100 tokens: the engine cuts the prompt at 2048, so every state crosses that cut; tile-aligned sizes, both modes."""
    rng = np.random.default_rng(3)
    cfg, W = O.random_model(rng, **CONFIGS["tensor_core_tiles"])
    S = 2100
    toks = rng.integers(0, cfg["vocab"], S).astype(np.int32)
    ref = O.forward(cfg, W, toks)
    want = [0, 1, 63, 64, 2047, 2048, 2049, S - 1]
    for exact in (True, False):
        m = build(cfg, W, exact, max_context=2304)
        got = m.forward_logits(toks, 0, want)
        assert rel_rms(got, ref[want]) < (5e-4 if exact else 3e-2)
        m.close()


def test_long_decode_and_graph_replay():
    rng = np.random.default_rng(8)
    cfg, W = O.random_model(rng, pattern=("parallel", "attention"), v_mix=(1,), width=32, vocab=50)
    S = 300
    toks = rng.integers(0, cfg["vocab"], S).astype(np.int32)
    ref = O.forward(cfg, W, toks)
    m = build(cfg, W, True, max_context=512)
    assert rel_rms(run_portions(m, toks, [3] + [1] * (S - 3)), ref) < 3e-4
    m.use_graph(False)
    m.clear_kv()
    assert rel_rms(run_portions(m, toks, [3] + [1] * (S - 3)), ref) < 3e-4
    m.close()


@pytest.mark.parametrize("pattern", [("attention",), ("parallel",)])
def test_a_far_token_reaches_the_last_position(pattern):
    """One layer, so the mixer is the only path between positions.  A token that occurs nowhere else sits far back (rows 0 and 2 of 600)
    and writes a loud key that every later query looks for: the last logits must follow the oracle in a prompt, across portions and when
    decoding, and the oracle itself must move."""
    rng = np.random.default_rng(13)
    cfg, W = O.random_model(rng, pattern=pattern, mlp=(False,), v_mix=(), right_scale=0.3, left=dict(conv=1, rot_dims=0), attn=dict(rot_dims=0))
    p = "l0.mix.left." if pattern == ("parallel",) else "l0.mix."
    m0 = cfg["layers"][0]["mixer"]
    D = (m0["left"] if pattern == ("parallel",) else m0)["dim"]
    W["l0.shift"][:] = 0.0
    W["embed"][:, :2] = 0.0; W["embed"][0, 0] = 6.0; W["embed"][1:, 1] = 2.0
    for r in range(0, W[p + "k"].shape[0], D):                                # channel 0 of every key head hears the special token only
        W[p + "k"][r, :] = 0.0; W[p + "k"][r, 0] = 3.0
    for r in range(0, W[p + "q"].shape[0], D):                                # channel 0 of every query head is loud for every other token
        W[p + "q"][r, :] = 0.0; W[p + "q"][r, 1] = 3.0
    W[p + "q.norm"][:] = 1.0; W[p + "k.norm"][:] = 1.0
    if pattern == ("parallel",):
        W[p + "q.b"][:] = 0.0; W[p + "k.b"][:] = 0.0
        W[p + "q.conv"][:] = 1.0; W[p + "k.conv"][:] = 1.0
    (m0["left"] if pattern == ("parallel",) else m0)["scale"] = 3.0
    S = 600
    toks = rng.integers(1, cfg["vocab"], S).astype(np.int32)
    base = O.forward(cfg, W, toks)
    m = build(cfg, W, True, max_context=1024)
    for special_at in (0, 2):
        t = toks.copy(); t[special_at] = 0
        ref = O.forward(cfg, W, t)
        assert rel_rms(ref[-1:], base[-1:]) > 1e-2
        for sizes in ([S], [256, 300] + [1] * 44, [3, 597]):
            got = run_portions(m, t, sizes)
            assert rel_rms(got[-40:], ref[-40:]) < 3e-4
    m.close()


def test_greedy_generation_through_the_engine(tmp_path):
    rng = np.random.default_rng(4)
    cfg, W = O.random_model(rng)
    for L in cfg["layers"]:                                                   # the folder states no ranks: the tensors' shapes give them
        if L["type"] == "parallel":
            del L["mixer"]["right"]["decay_rank"], L["mixer"]["right"]["gate_rank"]
    d = write_model_dir(tmp_path / "m", cfg, W)
    prompt = rng.integers(0, cfg["vocab"], 19).astype(np.int32)
    for exact in (True, False):
        e = Engine()
        assert e.load_path(d, max_context=128, exact_f32=exact)
        assert e.vocab_size == cfg["vocab"] and e.n_layers == 4
        new = e.generate_ids(prompt, max_tokens=24, temperature=0.0)
        assert len(new) == 24
        assert e.generate_ids(prompt, max_tokens=24, temperature=0.0) == new       # rows and states are taken over from position 0
        logits = O.forward(cfg, W, np.concatenate([prompt, np.asarray(new, dtype=np.int32)]))
        for i, tok in enumerate(new):                                         # every generated id is the oracle's greedy choice
            row = logits[len(prompt) - 1 + i]
            assert row[tok] >= row.max() - (1e-3 if exact else 0.1), (exact, i)
        sampled = e.generate_ids(prompt, max_tokens=8, temperature=0.8, top_k=10, top_p=0.9, repeat_penalty=1.1, seed=7)
        assert len(sampled) == 8 and all(0 <= s < cfg["vocab"] for s in sampled)
        e.close()


def test_model_folder_loads_like_device_tensors(tmp_path):
    rng = np.random.default_rng(6)
    cfg, W = O.random_model(rng)
    toks = rng.integers(0, cfg["vocab"], 33).astype(np.int32)
    a = Model.load_dir(write_model_dir(tmp_path / "m", cfg, W), max_context=64, exact_f32=True)
    b = build(cfg, W, True, max_context=64)
    np.testing.assert_array_equal(a.forward_logits(toks, 0, [0, 5, 32]), b.forward_logits(toks, 0, [0, 5, 32]))
