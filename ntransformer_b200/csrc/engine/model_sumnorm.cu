// model_sumnorm.cu — layers of BlockForm::SUM_NORM for the resident layer-spec model (engine/model_spec.cu):
//       h = shift(x);   x <- n(a x + mixer(h), g1);   x <- n(a x + ff(x), g2)
// with the mixer an attention (per-head q / k norm, optional biases, short convolutions on q, k, v, rotary positions from a frequency
// table, per-head score multiplier, sink, weights mixed across heads, values blended with an earlier layer's), the gated delta rule, or
// several of them side by side (MixerKind::BRANCHES).  One function serves a decoded token (T = 1, position read on the device, inside
// the captured graph) and the rows of a prompt portion; what a sequence carries between steps — cache rows, the shift's previous row,
// the convolutions' last inputs, the delta rule's matrix state — is written by the step that owns the tokens and read by later steps
// only from there, and every state reads as zeros when a step starts at position 0, so a new request needs no clearing.
//
// Launches per decoded token: all projections of the layer's mixers in one GEMV launch, all their convolutions in one launch, then per
// attention [norm / rotation / cache write] [attention] ([head mix]) [o GEMV], per delta rule [decay GEMV] [gate GEMV] [prep] [recurrence]
// [gate + norm] [o GEMV], then [sum + norm (+ the next layer's shift)] [gate / up GEMV with the ReLU gate] [down GEMV] [sum + norm + shift]:
// 16 for a layer of two mixers, 8 for an attention layer.  Prompt rows take the tensor-core GEMMs (short matrices through their
// zero-padded copies, the gated pair fused with its activation), the tiled attention kernel where the head widths fit it, and the
// tiled recurrence.
#include "model.h"

#include <algorithm>
#include <cmath>

namespace nt { namespace b200 {

namespace {
template <typename T> T* dmalloc0(size_t n) {
    T* p = nullptr;
    NT_CUDA_CHECK(cudaMalloc(&p, std::max<size_t>(n, 1) * sizeof(T)));
    NT_CUDA_CHECK(cudaMemset(p, 0, std::max<size_t>(n, 1) * sizeof(T)));
    return p;
}
constexpr size_t kScratchSlack = 256;       // floats behind RowBufs::wide for the 16-byte alignment of the buffers carved from it
GemvMat mat_of(const Weight& w, float* y) { GemvMat m; m.W = w.ptr; m.y = y; m.out = w.rows; m.dtype = w.dtype; m.row_pitch = w.pitch; return m; }

// floats per row that one mixer's intermediates take in RowBufs::wide (the buffers layer_sumnorm carves for it)
size_t mixer_floats(const LayerSpec& S) {
    const size_t H = (size_t)S.heads, G = (size_t)S.kv_heads, D = (size_t)S.dim, V = (size_t)S.vdim;
    if (S.mixer == MixerKind::DELTA_RULE)
        return 2 * (2 * G * D + H * V) + H + (size_t)S.delta.decay_rank + H * D + (size_t)S.delta.gate_rank + H * V + G + 2 * H * V;
    return 2 * (H * D + G * D + G * V) + (S.talking ? H * G * V : 0) + H * V;
}
}  // namespace

// The rows of one mixer inside RowBufs::wide, [T, width] each.
struct Model::MixerBufs {
    float *q = nullptr, *k = nullptr, *v = nullptr;        // projected rows
    float *qc = nullptr, *kc = nullptr, *vc = nullptr;     // behind the convolutions (== q, k, v when there is none)
    float *tmp = nullptr, *o = nullptr;                    // attention: per-head results over every value head; joined heads
    float *b = nullptr, *a1 = nullptr, *a = nullptr, *g1 = nullptr, *g = nullptr, *qk = nullptr, *og = nullptr;   // delta rule
    float *pub = nullptr;                                  // the step's published values [T, kv_heads * vdim] (LayerSpec::v_first)
};

size_t Model::sumnorm_scratch_width() const {
    size_t m = 1, vf = 0;
    for (const LayerSpec& S : cfg_.layers) {
        size_t w = 0;
        if (S.mixer == MixerKind::BRANCHES) for (const LayerSpec& b : S.branches) w += mixer_floats(b);
        else w = mixer_floats(S);
        m = std::max(m, w);
        if (S.v_first >= 0) vf = std::max(vf, (size_t)S.kv_heads * S.vdim);
    }
    return m + vf + 2 * (size_t)cfg_.hidden_size + kScratchSlack;          // + the published values of the step + the two branch outputs + alignment gaps
}

bool Model::finalize_mixer_state(LayerSpec& S, LayerWeights& M, int layer) {
    const bool delta = S.mixer == MixerKind::DELTA_RULE;
    const size_t qw = (size_t)(delta ? S.kv_heads : S.heads) * S.dim, kw = (size_t)S.kv_heads * S.dim, vw = (size_t)(delta ? S.heads : S.kv_heads) * S.vdim;
    bool ok = M.wq.ptr && M.wk.ptr && M.wv.ptr && M.wo.ptr;
    if (S.conv > 0) ok = ok && M.q_conv && M.k_conv && M.v_conv;
    if (delta) {
        ok = ok && S.conv > 0 && M.d_beta.ptr && M.d_a1.ptr && M.d_a2.ptr && M.d_g1.ptr && M.d_g2.ptr && M.d_dt_bias && M.d_a_log && M.d_norm;
        if (ok && (M.d_a2.cols != M.d_a1.rows || M.d_g2.cols != M.d_g1.rows)) { fprintf(stderr, "model: layer %d: the low-rank pairs of the delta rule do not fit together\n", layer); return false; }
        if (S.dim > DELTA_MAX_DIM) { fprintf(stderr, "model: layer %d: delta-rule key heads wider than %d are not covered\n", layer, DELTA_MAX_DIM); return false; }
    } else {
        ok = ok && (S.qk_norm != QKNorm::PER_HEAD || (M.q_norm && M.k_norm)) && (!S.qkv_bias || (M.q_bias && M.k_bias && M.v_bias && M.o_bias)) &&
             (!S.head_temp || M.head_temp) && (!S.talking || M.talk) && (!S.sink || M.sink) && (S.v_first < 0 || S.v_first == layer || M.v_mix);
        if (S.mixer != MixerKind::ATTN_WINDOW || S.maps != 1 || S.kv_from >= 0 || S.softcap != 0.f) { fprintf(stderr, "model: layer %d: this mixer has no kernels in the sum-norm block\n", layer); return false; }
        if (S.dim > 1024 || S.vdim > 512) { fprintf(stderr, "model: layer %d: heads wider than 1024 (keys) / 512 (values) are not covered\n", layer); return false; }
    }
    if (!ok) { fprintf(stderr, "model: layer %d is missing tensors\n", layer); return false; }
    if (S.conv > 1) {
        M.q_conv_state = dmalloc0<float>((size_t)(S.conv - 1) * qw);
        M.k_conv_state = dmalloc0<float>((size_t)(S.conv - 1) * kw);
        M.v_conv_state = dmalloc0<float>((size_t)(S.conv - 1) * vw);
    }
    if (delta) M.delta_state = dmalloc0<float>((size_t)S.heads * S.vdim * S.dim);
    for (Weight* w : {&M.wq, &M.wk, &M.wv, &M.d_beta, &M.d_a1, &M.d_g1}) pad_for_tensor_cores(*w);
    if (!delta && S.rot.dims > 0) {
        const RotarySpec& R = S.rot;
        std::vector<float> f((size_t)R.dims / 2);
        for (int i = 0; i < R.dims / 2; i++) f[(size_t)i] = (float)(std::pow((double)R.base, -2.0 * i / R.dims) / (double)R.divide);
        M.rot_freq = dmalloc0<float>(f.size());
        NT_CUDA_CHECK(cudaMemcpy(M.rot_freq, f.data(), sizeof(float) * f.size(), cudaMemcpyHostToDevice));
    }
    return true;
}

bool Model::finalize_sumnorm_layer(int i) {
    LayerSpec& S = cfg_.layers[(size_t)i];
    LayerWeights& M = layers_[(size_t)i];
    if (S.weights_of >= 0) { fprintf(stderr, "model: layer %d: shared tensors are not covered in the sum-norm block\n", i); return false; }
    bool ok = M.attn_norm && (!S.token_shift || M.shift_mu);
    if (S.ff > 0) ok = ok && S.ff_kind == FfKind::GLU && !S.ff_bias && M.ffn_norm && M.gate.ptr && M.up.ptr && M.down.ptr;
    if (!ok) { fprintf(stderr, "model: layer %d is missing tensors\n", i); return false; }
    if (S.token_shift) M.shift_state = dmalloc0<float>((size_t)cfg_.hidden_size);
    if (S.mixer == MixerKind::BRANCHES) {
        if (S.branches.size() != 2 || S.branch_scale.size() != 2 || M.branch.size() != 2) { fprintf(stderr, "model: layer %d: two mixers side by side are covered, no other count\n", i); return false; }
        if (S.branches[1].qkv_bias) { fprintf(stderr, "model: layer %d: only the first of two mixers may have a biased output\n", i); return false; }
        for (size_t b = 0; b < 2; b++)
            if (!finalize_mixer_state(S.branches[b], M.branch[b], i)) return false;
        return true;
    }
    if (S.v_first >= 0 && S.v_first != i) {
        const LayerSpec& F = cfg_.layers[(size_t)S.v_first];
        if (S.v_first > i || F.v_first != S.v_first || F.kv_heads * F.vdim != S.kv_heads * S.vdim) { fprintf(stderr, "model: layer %d: the layer its values blend with does not fit\n", i); return false; }
    }
    return finalize_mixer_state(S, M, i);
}

void Model::mixer_attention_rows(int layer, const LayerSpec& S, const LayerWeights& L, const MixerBufs& b, float* y, int T, const int* pos_dev, int p0, cudaStream_t s) {
    const int H = S.heads, G = S.kv_heads, D = S.dim, V = S.vdim;
    void* kc = kcs_[(size_t)S.cache_slot];
    void* vc = vcs_[(size_t)S.cache_slot];
    HeadPrep p;
    p.heads = H; p.kv_heads = G; p.dim = D; p.vdim = V; p.eps = cfg_.norm_eps;
    if (S.qk_norm == QKNorm::PER_HEAD) { p.q_gain = L.q_norm; p.k_gain = L.k_norm; }
    p.rot_dims = S.rot.dims; p.interleaved = S.rot.interleaved ? 1 : 0; p.freq = L.rot_freq;
    p.temp = S.head_temp ? L.head_temp : nullptr;
    if (S.v_first >= 0 && S.v_first == layer) p.v_publish = b.pub;
    else if (S.v_first >= 0) { p.v_first = b.pub; p.v_lambda = L.v_mix; }
    head_prep(b.qc, b.kc, b.vc, p, kc, vc, cache_dt_, T, pos_dev, p0, s);
    WindowAttn a;
    a.heads = H; a.kv_heads = G; a.dim = D; a.vdim = V; a.window = S.window; a.keep = S.keep_first; a.scale = S.scale; a.chunk = S.chunk;
    a.sink = S.sink ? L.sink : nullptr;
    if (!S.talking) attention_window(b.o, b.qc, kc, vc, cache_dt_, T, pos_dev, p0, cfg_.max_seq_len, a, s);
    else if (G * V <= 512) {
        // every query head over the values of all value heads at once, then the heads' results mixed (attention_heads.cu)
        a.vdim = G * V; a.joint_v = 1; a.v_stride = G * V;
        attention_window(b.tmp, b.qc, kc, vc, cache_dt_, T, pos_dev, p0, cfg_.max_seq_len, a, s);
        talk_mix(b.o, b.tmp, L.talk, T, H, G, V, (size_t)H * G * V, (size_t)G * V, (size_t)V, s);
    } else {
        // wide value rows: one pass per value head, each over a slice of the value rows
        a.joint_v = 1; a.v_stride = G * V;
        for (int c = 0; c < G; c++)
            attention_window(b.tmp + (size_t)c * T * H * V, b.qc, kc, static_cast<const uint8_t*>(vc) + (size_t)c * V * dtype_size(cache_dt_), cache_dt_, T, pos_dev, p0,
                             cfg_.max_seq_len, a, s);
        talk_mix(b.o, b.tmp, L.talk, T, H, G, V, (size_t)H * V, (size_t)V, (size_t)T * H * V, s);
    }
    rows_matmul(y, b.o, L.wo, T, s);
}

void Model::mixer_delta_rows(const LayerSpec& S, const LayerWeights& L, const MixerBufs& b, float* y, int T, const int* pos_dev, int p0, cudaStream_t s) {
    const int H = S.heads, G = S.kv_heads, D = S.dim, V = S.vdim;
    rows_matmul(b.a, b.a1, L.d_a2, T, s);
    rows_matmul(b.g, b.g1, L.d_g2, T, s);
    delta_prep(b.qc, b.kc, b.a, b.b, b.qk, L.d_dt_bias, L.d_a_log, T, H, G, D, s);
    delta_rule_rows(b.o, b.qc, b.kc, b.vc, b.a, b.b, b.qk, L.delta_state, T, H, G, D, V, pos_dev, p0, s);
    delta_gate_norm(b.og, b.o, b.g, L.d_norm, cfg_.norm_eps, T, H, V, s);
    rows_matmul(y, b.og, L.wo, T, s);
}

void Model::layer_sumnorm(int i, int T, const int* pos_dev, int p0, const RowBufs& B, cudaStream_t s) {
    const LayerSpec& S = cfg_.layers[(size_t)i];
    LayerWeights& L = layers_[(size_t)i];
    const int hidden = cfg_.hidden_size;
    const float eps = cfg_.norm_eps, alpha = cfg_.skip_scale;
    // ---- the mixer's input: a decoded token gets it from the sum-norm launch that produced x (see the end of this function) ----
    float* h = S.token_shift ? B.t[0] : B.x;
    if (S.token_shift && (T > 1 || i == 0)) token_shift_rows(h, B.x, L.shift_mu, L.shift_state, T, hidden, pos_dev, p0, s);
    // ---- carve the mixers' rows: [published values | branch outputs y1, y2 | per mixer ...] ----
    // every buffer starts on 16 bytes (vector loads of the tiled kernels), whatever T is: at most 3 floats are skipped per buffer
    size_t off = 0, cur = 0;
    auto take = [&](size_t w) { cur = (cur + 3) & ~(size_t)3; float* p = B.wide + cur; cur += w * (size_t)T; off += w; return p; };
    size_t vf = 0;
    for (const LayerSpec& Z : cfg_.layers) if (Z.v_first >= 0) vf = std::max(vf, (size_t)Z.kv_heads * Z.vdim);
    float* published = take(vf);
    float* y1 = take((size_t)hidden);
    float* y2 = take((size_t)hidden);
    const bool pair = S.mixer == MixerKind::BRANCHES;
    const int n_mix = pair ? (int)S.branches.size() : 1;
    MixerBufs bufs[2];
    const LayerSpec* specs[2] = {pair ? &S.branches[0] : &S, pair ? &S.branches[1] : nullptr};
    const LayerWeights* weights[2] = {pair ? &L.branch[0] : &L, pair ? &L.branch[1] : nullptr};
    GemvMat mats[DENSE_MAX_MATS];
    const Weight* mat_w[DENSE_MAX_MATS];
    int n_mats = 0;
    ConvSeg segs[SHORT_CONV_MAX_SEGS];
    int n_segs = 0;
    auto project = [&](const Weight& w, float* out) { mat_w[n_mats] = &w; mats[n_mats++] = mat_of(w, out); };
    auto convolve = [&](const LayerSpec& Z, float* u, float* out, int ch, const float* w, const float* bias, float* state, int act) {
        ConvSeg c;
        c.u = u; c.ld = ch; c.col0 = 0; c.out = out; c.out_ld = ch; c.ch = ch; c.taps = std::max(1, Z.conv); c.w = Z.conv > 0 ? w : nullptr; c.in_bias = bias; c.state = state; c.act = act;
        segs[n_segs++] = c;
    };
    for (int m = 0; m < n_mix; m++) {
        const LayerSpec& Z = *specs[m];
        const LayerWeights& W = *weights[m];
        MixerBufs& b = bufs[m];
        const bool delta = Z.mixer == MixerKind::DELTA_RULE;
        const int qw = (delta ? Z.kv_heads : Z.heads) * Z.dim, kw = Z.kv_heads * Z.dim, vw = (delta ? Z.heads : Z.kv_heads) * Z.vdim;
        b.q = take((size_t)qw); b.k = take((size_t)kw); b.v = take((size_t)vw);
        project(W.wq, b.q); project(W.wk, b.k); project(W.wv, b.v);
        const bool conv = Z.conv > 0 || Z.qkv_bias;
        if (conv) {
            b.qc = take((size_t)qw); b.kc = take((size_t)kw); b.vc = take((size_t)vw);
            const int act = delta ? 1 : 0;
            convolve(Z, b.q, b.qc, qw, W.q_conv, Z.qkv_bias ? W.q_bias : nullptr, W.q_conv_state, act);
            convolve(Z, b.k, b.kc, kw, W.k_conv, Z.qkv_bias ? W.k_bias : nullptr, W.k_conv_state, act);
            convolve(Z, b.v, b.vc, vw, W.v_conv, Z.qkv_bias ? W.v_bias : nullptr, W.v_conv_state, act);
        } else { b.qc = b.q; b.kc = b.k; b.vc = b.v; }
        if (delta) {
            b.b = take((size_t)Z.heads); b.a1 = take((size_t)W.d_a1.rows); b.a = take((size_t)Z.heads * Z.dim);
            b.g1 = take((size_t)W.d_g1.rows); b.g = take((size_t)vw); b.qk = take((size_t)Z.kv_heads); b.o = take((size_t)vw); b.og = take((size_t)vw);
            project(W.d_beta, b.b); project(W.d_a1, b.a1); project(W.d_g1, b.g1);
        } else {
            if (Z.talking) b.tmp = take((size_t)Z.heads * Z.kv_heads * Z.vdim);
            b.o = take((size_t)Z.heads * Z.vdim);
            b.pub = published;
        }
    }
    NT_CHECK(off <= sumnorm_scratch_width() && cur <= sumnorm_scratch_width() * (size_t)T, "layer_sumnorm: scratch rows overrun");
    // ---- projections (one launch for a decoded token), convolutions (one launch), then each mixer ----
    if (T == 1) gemv_dense(mats, n_mats, hidden, h, DENSE_STORE, nullptr, 1.f, s);
    else {
        bool split_done = false;                       // every projection reads h: its 16-bit split is made once
        for (int m = 0; m < n_mats; m++) rows_matmul(mats[m].y, h, *mat_w[m], T, s, &split_done);
    }
    if (n_segs > 0) short_conv(segs, n_segs, T, pos_dev, p0, s);
    for (int m = 0; m < n_mix; m++) {
        float* y = m == 0 ? y1 : y2;
        if (specs[m]->mixer == MixerKind::DELTA_RULE) mixer_delta_rows(*specs[m], *weights[m], bufs[m], y, T, pos_dev, p0, s);
        else mixer_attention_rows(i, *specs[m], *weights[m], bufs[m], y, T, pos_dev, p0, s);
    }
    // ---- x <- n(a x + sum of the mixers); the next shifted input rides along when this is the layer's last norm of a decoded token ----
    const bool next_shift = T == 1 && i + 1 < cfg_.n_layers && cfg_.layers[(size_t)i + 1].token_shift;
    LayerWeights* N = next_shift ? &layers_[(size_t)i + 1] : nullptr;
    const float s1 = pair ? S.branch_scale[0] : 1.f, s2 = pair ? S.branch_scale[1] : 0.f;
    const bool last1 = S.ff == 0;
    sum_rmsnorm_rows(B.x, alpha, y1, s1, weights[0]->o_bias, pair ? y2 : nullptr, s2, L.attn_norm, T, hidden, eps, s, (N && last1) ? B.t[0] : nullptr,
                     N ? N->shift_mu : nullptr, N ? N->shift_state : nullptr, pos_dev, p0);
    if (S.ff > 0) {
        float *g = B.t[1], *up = B.t[2];
        if (T == 1) {
            GemvMat gu[2] = {mat_of(L.gate, g), mat_of(L.up, nullptr)};
            gemv_dense(gu, 2, hidden, B.x, S.act == GluAct::RELU ? DENSE_REGLU : (S.act == GluAct::GELU_TANH ? DENSE_GEGLU : DENSE_SWIGLU), nullptr, 1.f, s);
            rows_matmul(B.y, g, L.down, T, s);
        } else if (pf_.ws && pf_.ws2 && spec_tc_ok(L.gate) && spec_tc_ok(L.up) && spec_tc_ok(L.down) && S.ff % 128 == 0) {
            // gate / up GEMMs with the gated activation and the split for the down projection in the epilogue: the [T, ff]
            // activations never reach HBM in FP32
            TcOpts o; o.bf16 = true; o.gelu = S.act == GluAct::GELU_TANH; o.relu = S.act == GluAct::RELU;
            split_activations(pf_.ws, B.x, T, hidden, s, true);
            NT_CHECK(gemm_f16_tc_swiglu_ws(pf_.ws2, pf_.ws, L.gate.ptr, L.up.ptr, T, S.ff, hidden, s, o), "prefill GEMM (gate/up) rejected");
            spec_gemm(B.y, nullptr, pf_.ws2, L.down, T, DENSE_STORE, nullptr, 1.f, s);
        } else {
            bool split_done = false;
            rows_matmul(g, B.x, L.gate, T, s, &split_done);
            rows_matmul(up, B.x, L.up, T, s, &split_done);
            glu_mul(g, g, up, (size_t)T * S.ff, S.act == GluAct::GELU_TANH, s, S.act == GluAct::RELU);
            rows_matmul(B.y, g, L.down, T, s);
        }
        sum_rmsnorm_rows(B.x, alpha, B.y, 1.f, nullptr, nullptr, 0.f, L.ffn_norm, T, hidden, eps, s, N ? B.t[0] : nullptr, N ? N->shift_mu : nullptr,
                         N ? N->shift_state : nullptr, pos_dev, p0);
    }
}

}}  // namespace nt::b200
