// attention_prefill_mma.cu — causal GQA attention over a whole prompt chunk (prefill), sm_100a.
//
// Same contract as the reference's attention_prefill_kernel (src/cuda/attention.cu:216-311): F32 queries
// [seq][n_heads][hd], F16 KV cache [max_seq][n_kv][hd], query i attends keys 0..start_pos+i, softmax(q.k*scale).v.
// The reference (and csrc/attention.cu's prefill_kernel) re-reads the whole key range once per query; here a CTA owns
// 64 queries of one head and streams 64-key K/V tiles through shared memory (cp.async, double buffered), with the two
// contractions on the warp-level tensor-core path (mma.sync m16n8k16, F32 accumulate) and an online softmax in
// registers (flash-attention-2 data flow).  F32 operands are split into two F16 terms (q = hi + lo, p = hi + lo) so
// the result keeps ~22 mantissa bits and stays within the 2e-5 tolerance of the oracle.
//
// The same kernel serves windowed attention (csrc/attention_window.cu's rule: key j visible from position p iff j <= p and
// (p - j < window or j < keep)), optionally with soft-capped scores cap * tanh(s / cap) and a BF16 cache (BF: both MMAs take
// BF16 operands, the splits are BF16 pairs): a query block then walks only the key tiles of the kept prefix and of its window.
#include "kernels_internal.h"
#include <cuda_fp16.h>
#include <cuda_bf16.h>

namespace nt { namespace b200 {

namespace {

constexpr int BQ = 64, BKV = 64, PAD = 8;      // PAD halfs: row stride 272 B (hd 128) keeps LDS.32 / ldmatrix conflict-free

template <bool BF>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if (BF)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
// (x, y) -> packed F16 hi pair and lo pair with x = hi + lo to ~2^-22
template <bool BF>
__device__ __forceinline__ void split2(float x, float y, uint32_t& hi, uint32_t& lo) {
    if (BF) {
        const __nv_bfloat162 b = __floats2bfloat162_rn(x, y);
        const float2 fb = __bfloat1622float2(b);
        const __nv_bfloat162 l = __floats2bfloat162_rn(x - fb.x, y - fb.y);
        hi = *reinterpret_cast<const uint32_t*>(&b);
        lo = *reinterpret_cast<const uint32_t*>(&l);
        return;
    }
    const __half2 h = __floats2half2_rn(x, y);
    const float2 f = __half22float2(h);
    hi = h2_bits(h);
    lo = h2_bits(__floats2half2_rn(x - f.x, y - f.y));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// HD: query / key head width, HDV: value head width.  maps > 1: blockIdx.y walks (head, map) pairs — map m of head h scores against
// map m of key head kvh (key rows [n_kv][maps][HD]) and sums kvh's one value row (value rows [n_kv][HDV]); n_heads counts the
// (head, map) pairs.  chunk > 0 replaces the window rule: key j visible from p iff j <= p and j / chunk == p / chunk.
template <int HD, int HDV, bool BF>
__global__ void __launch_bounds__(128, 2) prefill_mma_kernel(float* __restrict__ out, const float* __restrict__ Q,
                                                             const __half* __restrict__ kc, const __half* __restrict__ vc,
                                                             int seq_len, int start_pos, int n_heads, int n_kv, int max_seq,
                                                             float scale, int window, int keep, float softcap, int maps, int chunk,
                                                             const float* __restrict__ sink, int joint_v) {
    constexpr int LD = HD + PAD, LDV = HDV + PAD, KS = HD / 16, NT = HDV / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half* sK = reinterpret_cast<__half*>(smem_raw);                 // [2][BKV][LD]
    __half* sV = sK + 2 * BKV * LD;                                   // [2][BKV][LDV]
    const int qb = gridDim.x - 1 - blockIdx.x;                        // heaviest (latest) query blocks first
    const int head = blockIdx.y, vh = (head / maps) / ((n_heads / maps) / n_kv), kvh = vh * maps + head % maps, n_k = n_kv * maps;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int r0 = qb * BQ + warp * 16 + g, r1 = r0 + 8;              // this thread's two query rows (chunk-relative)
    const int p0 = start_pos + r0, p1 = start_pos + r1;               // their absolute positions == last visible key

    // ---- Q fragments (A operand, 16 x HD per warp), split into F16 hi + lo ----
    uint32_t qhi[KS][4], qlo[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int r = (i & 1) ? r1 : r0, c = ks * 16 + 2 * t + ((i & 2) ? 8 : 0);
            float2 v = make_float2(0.f, 0.f);
            if (r < seq_len) v = *reinterpret_cast<const float2*>(Q + ((size_t)r * n_heads + head) * HD + c);
            split2<BF>(v.x, v.y, qhi[ks][i], qlo[ks][i]);
        }
    }
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; n++) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    const int last_q = min(qb * BQ + BQ, seq_len) - 1;                // last valid query of the block
    // key tiles: those of the kept prefix that lie before the block's window, then the window's (full causal: all from tile 0)
    // (chunk: from the tile holding the first row of the first query's block of positions; later queries' blocks start no earlier)
    const int first_win = chunk > 0 ? ((start_pos + qb * BQ) / chunk * chunk) / BKV : (window > 0 ? max(0, start_pos + qb * BQ - window + 1) / BKV : 0);
    const int n_keep = (window > 0 && chunk <= 0) ? min((keep + BKV - 1) / BKV, first_win) : 0;
    const int n_tiles = n_keep + (start_pos + last_q) / BKV + 1 - first_win;
    auto tile_of = [&](int j) { return j < n_keep ? j : first_win + (j - n_keep); };

    auto load_tile = [&](int j, int st) {
        constexpr int CH = HD / 8, CHV = HDV / 8;                     // 16-byte chunks per row
        for (int c = threadIdx.x; c < BKV * CH; c += 128) {
            const int row = c / CH, ch = c % CH;
            const int key = min(tile_of(j) * BKV + row, max_seq - 1); // rows past the cache are masked by causality anyway
            cp_async16(sK + ((size_t)st * BKV + row) * LD + ch * 8, kc + ((size_t)key * n_k + kvh) * HD + ch * 8);
        }
        for (int c = threadIdx.x; c < BKV * CHV; c += 128) {
            const int row = c / CHV, ch = c % CHV;
            const int key = min(tile_of(j) * BKV + row, max_seq - 1);
            cp_async16(sV + ((size_t)st * BKV + row) * LDV + ch * 8, vc + (joint_v ? (size_t)key : (size_t)key * n_kv + vh) * HDV + ch * 8);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    load_tile(0, 0);
    for (int j = 0; j < n_tiles; j++) {
        const int st = j & 1;
        if (j + 1 < n_tiles) {
            load_tile(j + 1, st ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const __half* tK = sK + (size_t)st * BKV * LD;
        const __half* tV = sV + (size_t)st * BKV * LDV;

        // ---- S = Q K^T (16 x 64 per warp) ----
        float s[8][4];
#pragma unroll
        for (int n = 0; n < 8; n++) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
#pragma unroll
            for (int n = 0; n < 8; n++) {
                const __half* kp = tK + (size_t)(n * 8 + g) * LD + ks * 16 + 2 * t;
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(kp), b1 = *reinterpret_cast<const uint32_t*>(kp + 8);
                mma16816<BF>(s[n], qhi[ks], b0, b1);
                mma16816<BF>(s[n], qlo[ks], b0, b1);
            }
        }
        // ---- scale, causal mask, online softmax ----
        const int key0 = tile_of(j) * BKV;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int n = 0; n < 8; n++) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int key = key0 + n * 8 + 2 * t + (i & 1);
                const int p = (i & 2) ? p1 : p0;
                const bool seen = key <= p && (chunk > 0 ? key >= p / chunk * chunk : (window <= 0 || p - key < window || key < keep));
                float v = s[n][i] * scale;
                if (softcap > 0.f) v = softcap * (1.0f - 2.0f / (__expf(2.0f * v / softcap) + 1.0f));     // cap * tanh(v / cap)
                v = seen ? v : -INFINITY;
                s[n][i] = v;
                if (i & 2) mx1 = fmaxf(mx1, v); else mx0 = fmaxf(mx0, v);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, 2));
        // full causal: finite from tile 0 on (key 0 is visible to every row); with a window a row can find a whole tile masked
        // before its first visible key: subtract 0 instead of -inf so every exponential is exp(-inf) = 0, not NaN
        const float mr0 = fmaxf(m0, mx0), mr1 = fmaxf(m1, mx1);
        const float mn0 = mr0 == -INFINITY ? 0.f : mr0, mn1 = mr1 == -INFINITY ? 0.f : mr1;
        const float a0 = __expf(m0 - mn0), a1 = __expf(m1 - mn1);
        m0 = mr0; m1 = mr1;
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int n = 0; n < 8; n++) {
            s[n][0] = __expf(s[n][0] - mn0); s[n][1] = __expf(s[n][1] - mn0);
            s[n][2] = __expf(s[n][2] - mn1); s[n][3] = __expf(s[n][3] - mn1);
            sum0 += s[n][0] + s[n][1]; sum1 += s[n][2] + s[n][3];
        }
        l0 = l0 * a0 + sum0; l1 = l1 * a1 + sum1;                    // per-thread partial row sums (reduced at the end)
#pragma unroll
        for (int n = 0; n < NT; n++) { o[n][0] *= a0; o[n][1] *= a0; o[n][2] *= a1; o[n][3] *= a1; }

        // ---- O += P V : the accumulator layout of S is the A-operand layout of the second MMA ----
#pragma unroll
        for (int kt = 0; kt < BKV / 16; kt++) {
            uint32_t phi[4], plo[4];
            split2<BF>(s[2 * kt][0], s[2 * kt][1], phi[0], plo[0]);
            split2<BF>(s[2 * kt][2], s[2 * kt][3], phi[1], plo[1]);
            split2<BF>(s[2 * kt + 1][0], s[2 * kt + 1][1], phi[2], plo[2]);
            split2<BF>(s[2 * kt + 1][2], s[2 * kt + 1][3], phi[3], plo[3]);
#pragma unroll
            for (int np = 0; np < HDV / 16; np++) {
                // four 8x8 blocks of V^T: (keys +0..7 | +8..15) x (hd +0..7 | +8..15)
                const __half* vp = tV + (size_t)(kt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDV + np * 16 + (lane >> 4) * 8;
                uint32_t v0, v1, v2, v3;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                             : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3) : "r"((uint32_t)__cvta_generic_to_shared(vp)));
                mma16816<BF>(o[2 * np], phi, v0, v1);
                mma16816<BF>(o[2 * np], plo, v0, v1);
                mma16816<BF>(o[2 * np + 1], phi, v2, v3);
                mma16816<BF>(o[2 * np + 1], plo, v2, v3);
            }
        }
        __syncthreads();                                             // this stage is overwritten by the prefetch of tile j + 2
    }
    l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, 1); l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, 2);
    l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, 1); l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, 2);
    if (sink) {                     // exp(sink) joins the denominator; the maximum is raised to the sink first so nothing overflows
        const float sk = sink[head / maps];
        const float n0 = fmaxf(m0, sk), n1 = fmaxf(m1, sk);
        const float f0 = __expf(m0 - n0), f1 = __expf(m1 - n1);
        l0 = l0 * f0 + __expf(sk - n0); l1 = l1 * f1 + __expf(sk - n1);
#pragma unroll
        for (int n = 0; n < NT; n++) { o[n][0] *= f0; o[n][1] *= f0; o[n][2] *= f1; o[n][3] *= f1; }
    }
    const float i0 = 1.0f / l0, i1 = 1.0f / l1;
#pragma unroll
    for (int n = 0; n < NT; n++) {
        const int c = n * 8 + 2 * t;
        if (r0 < seq_len) *reinterpret_cast<float2*>(out + ((size_t)r0 * n_heads + head) * HDV + c) = make_float2(o[n][0] * i0, o[n][1] * i0);
        if (r1 < seq_len) *reinterpret_cast<float2*>(out + ((size_t)r1 * n_heads + head) * HDV + c) = make_float2(o[n][2] * i1, o[n][3] * i1);
    }
}

template <int HD, int HDV, bool BF>
void launch(float* out, const float* Q, const __half* kc, const __half* vc, int seq_len, int start_pos, int n_heads, int n_kv,
            int max_seq, float scale, int window, int keep, float softcap, cudaStream_t s, int maps = 1, int chunk = 0, const float* sink = nullptr,
            int joint_v = 0) {
    const int smem = 2 * BKV * (HD + PAD + HDV + PAD) * (int)sizeof(__half);
    static unsigned long long configured = 0;      // bit per device id
    opt_in_dynamic_smem(prefill_mma_kernel<HD, HDV, BF>, (int)(smem), configured);
    prefill_mma_kernel<HD, HDV, BF><<<dim3((seq_len + BQ - 1) / BQ, n_heads * maps), 128, smem, s>>>(out, Q, kc, vc, seq_len, start_pos, n_heads * maps, n_kv,
                                                                                                    max_seq, scale, window, keep, softcap, maps, chunk, sink, joint_v);
    NT_LAUNCH_CHECK();
    count_launch();
}

}  // namespace

bool attention_prefill_mma_supported(int seq_len, int n_heads, int n_kv, int hd) {
    return seq_len >= 16 && (hd == 64 || hd == 128) && n_kv > 0 && n_heads % n_kv == 0;
}

void attention_prefill_mma(float* out, const float* Q, const void* kc, const void* vc, int seq_len, int start_pos, int n_heads,
                           int n_kv, int hd, int max_seq, float scale, cudaStream_t s) {
    const __half* k = static_cast<const __half*>(kc);
    const __half* v = static_cast<const __half*>(vc);
    if (hd == 128) launch<128, 128, false>(out, Q, k, v, seq_len, start_pos, n_heads, n_kv, max_seq, scale, 0, 0, 0.f, s);
    else launch<64, 64, false>(out, Q, k, v, seq_len, start_pos, n_heads, n_kv, max_seq, scale, 0, 0, 0.f, s);
}

// Windowed / block-masked / soft-capped form over a BF16 cache: (dim, vdim) in {(64, 64), (128, 128), (32, 64), (64, 128)}, one or
// two score maps per head, at least 16 queries.
bool attention_window_mma_supported(int tokens, const WindowAttn& a, DType cache_dt) {
    const bool shape = (a.dim == a.vdim && (a.dim == 64 || a.dim == 128)) || (a.vdim == 2 * a.dim && (a.dim == 32 || a.dim == 64));
    // joint values: one value row of width vdim per key, packed (the stride equals the width)
    const bool strides = a.k_stride == 0 && (a.joint_v ? (a.v_stride == a.vdim && a.maps == 1) : a.v_stride == 0);
    return cache_dt == DType::BF16 && shape && strides && a.maps >= 1 && a.maps <= 2 && tokens >= 16 && a.kv_heads > 0 && a.heads % a.kv_heads == 0;
}
void attention_window_mma(float* out, const float* Q, const void* kc, const void* vc, int tokens, int p0, int max_seq, const WindowAttn& a,
                          cudaStream_t s) {
    const __half* k = static_cast<const __half*>(kc);       // 16-bit words either way; the BF instantiation reads them as BF16
    const __half* v = static_cast<const __half*>(vc);
#define NT_AW(D, V) launch<D, V, true>(out, Q, k, v, tokens, p0, a.heads, a.kv_heads, max_seq, a.scale, a.window, a.keep, a.softcap, s, a.maps, a.chunk, a.sink, a.joint_v)
    if (a.dim == 128) NT_AW(128, 128);
    else if (a.dim == 64 && a.vdim == 64) NT_AW(64, 64);
    else if (a.dim == 64) NT_AW(64, 128);
    else NT_AW(32, 64);
#undef NT_AW
}

// Per-head 16-bit operands built for the call (latent attention's expanded keys / values): key width 64, 128 or 192, value width 64
// or 128, every head its own key / value head, full causal mask.
bool attention_heads_mma_widths(int key_dim, int value_dim, int* kw, int* vw) {
    if (key_dim <= 0 || value_dim <= 0 || key_dim > 192 || value_dim > 128) return false;
    *kw = key_dim <= 64 ? 64 : key_dim <= 128 ? 128 : 192;
    *vw = value_dim <= 64 ? 64 : 128;
    return true;
}
void attention_heads_mma(float* out, const float* Q, const void* kc, const void* vc, int tokens, int p0, int rows, int heads, int kw, int vw, float scale,
                         cudaStream_t s) {
    const __half* k = static_cast<const __half*>(kc);
    const __half* v = static_cast<const __half*>(vc);
#define NT_AH(D, V) launch<D, V, true>(out, Q, k, v, tokens, p0, heads, heads, rows, scale, 0, 0, 0.f, s)
    if (kw == 64 && vw == 64) NT_AH(64, 64);
    else if (kw == 64 && vw == 128) NT_AH(64, 128);
    else if (kw == 128 && vw == 64) NT_AH(128, 64);
    else if (kw == 128 && vw == 128) NT_AH(128, 128);
    else if (kw == 192 && vw == 64) NT_AH(192, 64);
    else if (kw == 192 && vw == 128) NT_AH(192, 128);
    else NT_CHECK(false, "attention_heads_mma: widths from attention_heads_mma_widths");
#undef NT_AH
}

}}  // namespace nt::b200
