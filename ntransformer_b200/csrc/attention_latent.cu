// attention_latent.cu — low-rank ("latent") attention around its projections (engine/layer_spec.h LatentSpec).
// A position's cache row is [c : kv_rank | kr : rot_dim]: c the RMS-normed key / value latent, kr one rotated key part shared by all
// heads.  Head h's key is [W_uk,h c | kr] and its value W_uv,h c, so with qa_h = [W_uk,h^T q_h,unrotated | rot(q_h,rotated)]
//     score_ij = scale * <qa_h,i , row_j>        out_h,i = W_uv,h * sum_j softmax_j(score_ij) c_j ,
// i.e. one attention with a single key / value head of width kv_rank + rot_dim whose values are the first kv_rank numbers of the same
// rows (attention_window.cu with row strides).  Nothing per head is ever expanded per cached position: a prompt portion, a whole
// prompt and a decoded token read the same rows.
//   latent_prep      RMS norm (gain) of the query latent in place; RMS norm of the first kv_rank numbers of W_dkv h and rotation of the
//                    rest, both written to cache row pos (skipped for a layer that reads another layer's rows)
//   latent_q_absorb  qa = [W_uk,h^T q_unrotated | rot(q_rotated)] for every head, tiles of 8 tokens per CTA
//   latent_v_up      out = W_uv,h o_latent per head, tiles of 8 tokens per CTA
// A prompt portion of 16 tokens or more instead expands the rows it can see into per-head keys and values once (two tensor-core GEMMs
// over the latents: latent_rows_f32 feeds them, latent_expand_pack packs their results with the rotated key part into 16-bit
// [row, head, width] operands) and runs the tiled tensor-core attention kernel over them (attention_heads_mma): heads * (dim + rot_dim +
// vdim) multiply-adds per (query, key) instead of heads * (2 kv_rank + rot_dim).  latent_q_rot_pad rotates and pads the queries.
// Rotation: channel i of the rotated part pairs with channel i + dims/2 (or 2i with 2i+1), angle pos * base^(-2i/dims), computed
// in double and applied in F32; channels past `dims` pass unchanged.  Norms, angles and sums are F32 or better.
// Compiled WITHOUT --use_fast_math.
#include "kernels_internal.h"
#include "ring.cuh"
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <algorithm>
#include <cmath>
#include <cfloat>
#include <cstdint>
#include <cstdlib>

namespace nt { namespace b200 {

namespace {

__device__ __forceinline__ float wld(const float* p, size_t i) { return __ldg(p + i); }
__device__ __forceinline__ float wld(const __half* p, size_t i) { return __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(p) + i))); }
__device__ __forceinline__ float wld(const __nv_bfloat16* p, size_t i) { return __uint_as_float((unsigned)__ldg(reinterpret_cast<const unsigned short*>(p) + i) << 16); }
__device__ __forceinline__ void cst(float* p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void cst(__nv_bfloat16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// out[i] for channel i of a rot_dim-wide vector `src` at position pos
__device__ __forceinline__ float rotated(const float* src, int i, int dims, int interleaved, double log2_base, int pos) {
    if (i >= dims) return src[i];
    const int half = dims >> 1;
    int pair, mate;
    bool first;
    if (interleaved) { pair = i >> 1; first = (i & 1) == 0; mate = first ? i + 1 : i - 1; }
    else { first = i < half; pair = first ? i : i - half; mate = first ? i + half : i - half; }
    const double ang = (double)pos * exp2(-2.0 * (double)pair / (double)dims * log2_base);
    double sn, cs;
    sincos(ang, &sn, &cs);
    const float c = (float)cs, sv = (float)sn;
    // (u, v) -> (u cos - v sin, v cos + u sin)
    return first ? src[i] * c - src[mate] * sv : src[i] * c + src[mate] * sv;
}

__device__ __forceinline__ float block_sum_256(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) tot += red[w];
    return tot;
}

// grid (T, 2): y == 0 the query latent, y == 1 the key / value row
template <typename KT>
__global__ void __launch_bounds__(256) latent_prep_kernel(float* __restrict__ cq, int q_rank, const float* __restrict__ q_gain, const float* __restrict__ dkv,
                                                          int kv_rank, int rot_dim, const float* __restrict__ kv_gain, float eps, KT* __restrict__ cache,
                                                          int dims, int interleaved, double log2_base, const int* __restrict__ pos_dev, int p0) {
    __shared__ float red[8];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (blockIdx.y == 0) {
        float* r = cq + (size_t)t * q_rank;
        float ss = 0.f;
        for (int i = threadIdx.x; i < q_rank; i += 256) ss = fmaf(r[i], r[i], ss);
        const float inv = 1.0f / sqrtf(block_sum_256(ss, red) / (float)q_rank + eps);
        for (int i = threadIdx.x; i < q_rank; i += 256) r[i] = r[i] * inv * q_gain[i];
        return;
    }
    if (!dkv) return;
    const int pos = (pos_dev ? *pos_dev : p0) + t;
    const int row = kv_rank + rot_dim;
    const float* r = dkv + (size_t)t * row;
    float ss = 0.f;
    for (int i = threadIdx.x; i < kv_rank; i += 256) ss = fmaf(r[i], r[i], ss);
    const float inv = 1.0f / sqrtf(block_sum_256(ss, red) / (float)kv_rank + eps);
    for (int i = threadIdx.x; i < kv_rank; i += 256) cst(cache, (size_t)pos * row + i, r[i] * inv * kv_gain[i]);
    for (int i = threadIdx.x; i < rot_dim; i += 256) cst(cache, (size_t)pos * row + kv_rank + i, rotated(r + kv_rank, i, dims, interleaved, log2_base, pos));
}

constexpr int LT = 8;      // tokens per CTA in the two per-head products

// grid (ceil(T / LT), heads, ceil(kv_rank / 64)).  q [T, heads, dim + rot_dim]; qa [T, heads, kv_rank + rot_dim]; W_uk [heads * dim, kv_rank].
// A CTA owns 64 latent channels of a head: thread (r, part) sums every fourth row of W_uk,h for channel r, the four parts meet in
// shared memory.  One decoded token then has heads * kv_rank / 64 CTAs with short chains instead of `heads` CTAs with long ones.
template <typename WT>
__global__ void __launch_bounds__(256) latent_q_absorb_kernel(float* __restrict__ qa, const float* __restrict__ q, const WT* __restrict__ W_uk, int T, int heads,
                                                              int dim, int rot_dim, int kv_rank, int dims, int interleaved, double log2_base,
                                                              const int* __restrict__ pos_dev, int p0) {
    extern __shared__ __align__(16) float qs[];           // [LT][dim + rot_dim] | partial sums [4][64][LT]
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.x * LT, h = blockIdx.y, qd = dim + rot_dim, od = kv_rank + rot_dim;
    const int nt = min(LT, T - t0);
    float* red = qs + LT * qd;
    for (int e = threadIdx.x; e < LT * qd; e += 256) {
        const int tt = e / qd, i = e % qd;
        qs[e] = tt < nt ? q[((size_t)(t0 + tt) * heads + h) * qd + i] : 0.f;
    }
    __syncthreads();
    const WT* Wh = W_uk + (size_t)h * dim * kv_rank;
    const int rl = threadIdx.x & 63, part = threadIdx.x >> 6, r = blockIdx.z * 64 + rl;
    float acc[LT];
#pragma unroll
    for (int tt = 0; tt < LT; tt++) acc[tt] = 0.f;
    if (r < kv_rank) {
#pragma unroll 4
        for (int d = part; d < dim; d += 4) {
            const float w = wld(Wh, (size_t)d * kv_rank + r);
#pragma unroll
            for (int tt = 0; tt < LT; tt++) acc[tt] = fmaf(w, qs[tt * qd + d], acc[tt]);
        }
    }
#pragma unroll
    for (int tt = 0; tt < LT; tt++) red[(part * 64 + rl) * LT + tt] = acc[tt];
    __syncthreads();
    for (int e = threadIdx.x; e < 64 * LT; e += 256) {
        const int rr = e / LT, tt = e % LT, ro = blockIdx.z * 64 + rr;
        if (ro < kv_rank && tt < nt)
            qa[((size_t)(t0 + tt) * heads + h) * od + ro] = (red[rr * LT + tt] + red[(64 + rr) * LT + tt]) + (red[(128 + rr) * LT + tt] + red[(192 + rr) * LT + tt]);
    }
    if (blockIdx.z != 0) return;
    const int base = pos_dev ? *pos_dev : p0;
    for (int e = threadIdx.x; e < nt * rot_dim; e += 256) {
        const int tt = e / rot_dim, i = e % rot_dim;
        qa[((size_t)(t0 + tt) * heads + h) * od + kv_rank + i] = rotated(qs + tt * qd + dim, i, dims, interleaved, log2_base, base + t0 + tt);
    }
}

// grid (ceil(T / LT), heads, ceil(vdim / 32)).  ol [T, heads, kv_rank]; out [T, heads * vdim]; W_uv [heads * vdim, kv_rank].  A warp per output
// channel, 32 channels per CTA.
template <typename WT>
__global__ void __launch_bounds__(256) latent_v_up_kernel(float* __restrict__ out, const float* __restrict__ ol, const WT* __restrict__ W_uv, int T, int heads,
                                                          int vdim, int kv_rank) {
    extern __shared__ __align__(16) float os[];           // [LT][kv_rank]
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.x * LT, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nt = min(LT, T - t0);
    for (int e = threadIdx.x; e < LT * kv_rank; e += 256) {
        const int tt = e / kv_rank, i = e % kv_rank;
        os[e] = tt < nt ? ol[((size_t)(t0 + tt) * heads + h) * kv_rank + i] : 0.f;
    }
    __syncthreads();
    for (int v = blockIdx.z * 32 + warp; v < min(vdim, (int)blockIdx.z * 32 + 32); v += 8) {
        const WT* wr = W_uv + ((size_t)h * vdim + v) * kv_rank;
        float acc[LT];
#pragma unroll
        for (int tt = 0; tt < LT; tt++) acc[tt] = 0.f;
        for (int r = lane; r < kv_rank; r += 32) {
            const float w = wld(wr, r);
#pragma unroll
            for (int tt = 0; tt < LT; tt++) acc[tt] = fmaf(w, os[tt * kv_rank + r], acc[tt]);
        }
#pragma unroll
        for (int tt = 0; tt < LT; tt++) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc[tt] += __shfl_xor_sync(0xFFFFFFFFu, acc[tt], o);
        }
        if (lane == 0)
            for (int tt = 0; tt < nt; tt++) out[(size_t)(t0 + tt) * heads * vdim + (size_t)h * vdim + v] = acc[tt];
    }
}

// ---- per-head keys and values of a prompt portion (the tiled attention kernel reads 16-bit [row, head, width] operands) ----

// out [n, kv_rank] F32 <- the latents of cache rows r0 .. r0 + n - 1
__global__ void __launch_bounds__(256) latent_rows_f32_kernel(float* __restrict__ out, const __nv_bfloat16* __restrict__ cache, int row, int kv_rank, int r0, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t e = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (e >= total) return;
    const size_t r = e / kv_rank;
    const int i = (int)(e % kv_rank);
    out[e] = wld(cache, ((size_t)r0 + r) * row + i);
}

// kfull [r, h, kw] = [ku[r - r0, h, :dim] | rotated key part of row r | 0 ...]; vfull [r, h, vw] = [vu[r - r0, h, :vdim] | 0 ...]
__global__ void __launch_bounds__(256) latent_expand_pack_kernel(__nv_bfloat16* __restrict__ kfull, __nv_bfloat16* __restrict__ vfull, const float* __restrict__ ku,
                                                                 const float* __restrict__ vu, const __nv_bfloat16* __restrict__ cache, int row, int kv_rank,
                                                                 int r0, int heads, int dim, int rot_dim, int vdim, int kw, int vw) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x, h = blockIdx.y;
    const size_t ar = (size_t)r0 + r;
    for (int i = threadIdx.x; i < kw; i += 256) {
        __nv_bfloat16 v = __float2bfloat16_rn(0.f);
        if (i < dim) v = __float2bfloat16_rn(ku[((size_t)r * heads + h) * dim + i]);
        else if (i < dim + rot_dim) v = cache[ar * row + kv_rank + (i - dim)];
        kfull[(ar * heads + h) * kw + i] = v;
    }
    for (int i = threadIdx.x; i < vw; i += 256)
        vfull[(ar * heads + h) * vw + i] = __float2bfloat16_rn(i < vdim ? vu[((size_t)r * heads + h) * vdim + i] : 0.f);
}

// qp [t, h, kw] = [q[t, h, :dim] | rot(q[t, h, dim:]) | 0 ...]
__global__ void __launch_bounds__(256) latent_q_rot_pad_kernel(float* __restrict__ qp, const float* __restrict__ q, int heads, int dim, int rot_dim, int kw, int dims,
                                                               int interleaved, double log2_base, int p0) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y, qd = dim + rot_dim;
    const float* src = q + ((size_t)t * heads + h) * qd;
    float* dst = qp + ((size_t)t * heads + h) * kw;
    for (int i = threadIdx.x; i < kw; i += 256) {
        float v = 0.f;
        if (i < dim) v = src[i];
        else if (i < qd) v = rotated(src + dim, i - dim, dims, interleaved, log2_base, p0 + t);
        dst[i] = v;
    }
}

// out [t, h * vdim + i] = o [t, h, vw][i]
__global__ void __launch_bounds__(256) latent_unpad_kernel(float* __restrict__ out, const float* __restrict__ o, int vdim, int vw, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t e = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (e >= total) return;
    out[e] = o[e / vdim * vw + e % vdim];
}

// ---- attention of a few queries over ONE shared key / value head stored as rows (the absorbed form: every head scores the same rows) ----
// A CTA takes a (query, key slice) and serves ALL heads from one copy of the rows in shared memory: tiles of 16 rows are loaded once
// (16-byte copies) instead of once per head.  Warp w owns heads w, w + 8, ...: a tile's 16 scores of a head sit in 16 lanes x 2 halves
// of the row (combined by one shuffle), the online softmax state of a head is uniform in its warp, the probabilities go through a
// per-head line of shared memory that only the owning warp reads, and the weighted sum is lane-per-channel-pair with the four heads'
// accumulators in registers.  Every CTA writes (max, sum, unnormalised vector) per head; latent_shared_merge_kernel joins the slices.
constexpr int LS_KEYS = 16, LS_HB = 4, LS_CC = 8;      // rows per tile; heads per warp (heads <= 32); channel pairs per lane (vdim <= 512)

template <typename KT> struct RowVec;
template <> struct RowVec<float> {
    static constexpr int N = 4;
    __device__ static void load(const float* p, float (&v)[4]) { const float4 t = *reinterpret_cast<const float4*>(p); v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
    __device__ static float2 pair(const float* p) { return *reinterpret_cast<const float2*>(p); }
};
template <> struct RowVec<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static void load(const __nv_bfloat16* p, float (&v)[8]) {
        const uint4 t = *reinterpret_cast<const uint4*>(p);
        const unsigned u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int e = 0; e < 4; e++) { v[2 * e] = __uint_as_float(u[e] << 16); v[2 * e + 1] = __uint_as_float(u[e] & 0xFFFF0000u); }
    }
    __device__ static float2 pair(const __nv_bfloat16* p) { const unsigned u = *reinterpret_cast<const unsigned*>(p); return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xFFFF0000u)); }
};

// grid (tokens, slices).  Q [tokens, heads, dim]; rows [*, row] with keys = the first dim numbers, values = the first vdim numbers.
// part [tokens, slices, heads, vdim + 2].  dim, row multiples of RowVec::N; vdim even.
template <typename KT>
__global__ void __launch_bounds__(256) latent_shared_attn_kernel(float* __restrict__ part, const float* __restrict__ Q, const KT* __restrict__ rows,
                                                                 const int* __restrict__ pos_dev, int p0, int heads, int dim, int vdim, int row, float scale) {
    constexpr int VN = RowVec<KT>::N;
    extern __shared__ __align__(16) unsigned char ls_raw[];
    float* qs = reinterpret_cast<float*>(ls_raw);                              // [heads][dim]
    float* ps = qs + (size_t)heads * dim;                                       // [heads][LS_KEYS]
    KT* kt = reinterpret_cast<KT*>(ps + (size_t)heads * LS_KEYS);               // [LS_KEYS][dim + VN]: the pad keeps 16-byte reads of 8 rows on 8 bank groups
    const int ldk = dim + VN;
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, slice = blockIdx.y, n_slices = gridDim.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, key = lane & 15, half = lane >> 4;
    const int n_keys = (pos_dev ? *pos_dev : p0) + t + 1;
    const float* q = Q + (size_t)t * heads * dim;
    for (int e = threadIdx.x * 4; e < heads * dim; e += 1024) *reinterpret_cast<float4*>(qs + e) = *reinterpret_cast<const float4*>(q + e);
    float m[LS_HB], l[LS_HB], acc[LS_HB][LS_CC][2];
#pragma unroll
    for (int i = 0; i < LS_HB; i++) {
        m[i] = -FLT_MAX; l[i] = 0.f;
#pragma unroll
        for (int c = 0; c < LS_CC; c++) acc[i][c][0] = acc[i][c][1] = 0.f;
    }
    const int n_chunks = dim / VN;
    for (int k0 = slice * LS_KEYS; k0 < n_keys; k0 += n_slices * LS_KEYS) {
        __syncthreads();                                   // the previous tile is consumed (first pass: qs is written)
        for (int e = threadIdx.x; e < LS_KEYS * n_chunks; e += 256) {
            const int r = e / n_chunks, c = e - r * n_chunks;
            const int src = min(k0 + r, n_keys - 1);       // rows past the last visible one are masked below
            *reinterpret_cast<uint4*>(kt + (size_t)r * ldk + c * VN) = *reinterpret_cast<const uint4*>(rows + (size_t)src * row + c * VN);
        }
        __syncthreads();
        const bool valid = k0 + key < n_keys;
        // ---- scores: this lane's row, every second chunk of it, against the warp's heads ----
        float sc[LS_HB] = {0.f, 0.f, 0.f, 0.f};
        for (int c = half; c < n_chunks; c += 2) {
            float kv[VN];
            RowVec<KT>::load(kt + (size_t)key * ldk + c * VN, kv);
#pragma unroll
            for (int i = 0; i < LS_HB; i++) {
                const int h = warp + 8 * i;
                if (h < heads) {
                    const float* qh = qs + (size_t)h * dim + c * VN;
#pragma unroll
                    for (int e = 0; e < VN; e += 4) {
                        const float4 qv = *reinterpret_cast<const float4*>(qh + e);
                        sc[i] = fmaf(qv.x, kv[e], sc[i]); sc[i] = fmaf(qv.y, kv[e + 1], sc[i]); sc[i] = fmaf(qv.z, kv[e + 2], sc[i]); sc[i] = fmaf(qv.w, kv[e + 3], sc[i]);
                    }
                }
            }
        }
#pragma unroll
        for (int i = 0; i < LS_HB; i++) {
            const int h = warp + 8 * i;
            if (h >= heads) continue;                      // uniform in the warp
            float s = sc[i] + __shfl_xor_sync(0xFFFFFFFFu, sc[i], 16);
            s = valid ? s * scale : -FLT_MAX;
            float mt = s;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) mt = fmaxf(mt, __shfl_xor_sync(0xFFFFFFFFu, mt, o));
            const float mn = fmaxf(m[i], mt);
            const float corr = expf(m[i] - mn), pk = valid ? expf(s - mn) : 0.f;
            float sum = pk;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
            l[i] = l[i] * corr + sum;
            m[i] = mn;
            if (half == 0) ps[h * LS_KEYS + key] = pk;
#pragma unroll
            for (int c = 0; c < LS_CC; c++) { acc[i][c][0] *= corr; acc[i][c][1] *= corr; }
        }
        __syncwarp();                                       // a head's probabilities are read by its own warp only
        // ---- weighted sum: lane owns channel pairs 2 lane + 64 c ----
#pragma unroll 4
        for (int k = 0; k < LS_KEYS; k++) {
            float pk[LS_HB];
#pragma unroll
            for (int i = 0; i < LS_HB; i++) pk[i] = warp + 8 * i < heads ? ps[(warp + 8 * i) * LS_KEYS + k] : 0.f;
#pragma unroll
            for (int c = 0; c < LS_CC; c++) {
                const int ch = 2 * lane + 64 * c;
                if (ch < vdim) {
                    const float2 v = RowVec<KT>::pair(kt + (size_t)k * ldk + ch);
#pragma unroll
                    for (int i = 0; i < LS_HB; i++) { acc[i][c][0] = fmaf(pk[i], v.x, acc[i][c][0]); acc[i][c][1] = fmaf(pk[i], v.y, acc[i][c][1]); }
                }
            }
        }
        __syncwarp();
    }
#pragma unroll
    for (int i = 0; i < LS_HB; i++) {
        const int h = warp + 8 * i;
        if (h >= heads) continue;
        float* dst = part + (((size_t)t * n_slices + slice) * heads + h) * (vdim + 2);
        if (lane == 0) { dst[0] = m[i]; dst[1] = l[i]; }
#pragma unroll
        for (int c = 0; c < LS_CC; c++) {
            const int ch = 2 * lane + 64 * c;
            if (ch < vdim) { dst[2 + ch] = acc[i][c][0]; dst[3 + ch] = acc[i][c][1]; }
        }
    }
}

// grid (tokens, heads, ceil(vdim / 64)): out [t, h, :] = sum_s acc_s exp(m_s - M) / sum_s l_s exp(m_s - M).  Thread (channel, g) sums
// every fourth slice of its channel; the four partial sums meet in shared memory.
__global__ void __launch_bounds__(256) latent_shared_merge_kernel(float* __restrict__ out, const float* __restrict__ part, int n_slices, int heads, int vdim) {
    extern __shared__ __align__(16) float wsm[];           // [n_slices]
    __shared__ float red[8];
    __shared__ float sums[4][64];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y;
    const float* base = part + ((size_t)t * n_slices * heads + h) * (vdim + 2);
    const size_t step = (size_t)heads * (vdim + 2);
    float mx = -FLT_MAX;
    for (int s = threadIdx.x; s < n_slices; s += 256) mx = fmaxf(mx, base[s * step]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    float M = -FLT_MAX;
#pragma unroll
    for (int w = 0; w < 8; w++) M = fmaxf(M, red[w]);
    float ls = 0.f;
    for (int s = threadIdx.x; s < n_slices; s += 256) { const float w = expf(base[s * step] - M); wsm[s] = w; ls = fmaf(base[s * step + 1], w, ls); }
    const float L = block_sum_256(ls, red);                // its barriers also publish wsm
    const int cl = threadIdx.x & 63, g = threadIdx.x >> 6, c = blockIdx.z * 64 + cl;
    float v = 0.f;
    if (c < vdim) {
#pragma unroll 8
        for (int s = g; s < n_slices; s += 4) v = fmaf(base[s * step + 2 + c], wsm[s], v);
    }
    sums[g][cl] = v;
    __syncthreads();
    if (g == 0 && c < vdim) out[((size_t)t * heads + h) * vdim + c] = ((sums[0][cl] + sums[1][cl]) + (sums[2][cl] + sums[3][cl])) / L;
}

}  // namespace

void latent_prep(float* cq, int q_rank, const float* q_gain, const float* dkv, int kv_rank, int rot_dim, const float* kv_gain, float eps, void* cache,
                 DType cache_dt, int rot_dims, bool interleaved, float rot_base, int T, const int* pos_dev, int p0, cudaStream_t s) {
    if (T <= 0) return;
    NT_CHECK(cache_dt == DType::F32 || cache_dt == DType::BF16, "latent_prep: F32 or BF16 cache");
    const double l2b = std::log2((double)rot_base);
    if (cache_dt == DType::F32)
        launch_k(latent_prep_kernel<float>, dim3(T, 2), dim3(256), 0, s, cq, q_rank, q_gain, dkv, kv_rank, rot_dim, kv_gain, eps, static_cast<float*>(cache),
                 rot_dims, interleaved ? 1 : 0, l2b, pos_dev, p0);
    else
        launch_k(latent_prep_kernel<__nv_bfloat16>, dim3(T, 2), dim3(256), 0, s, cq, q_rank, q_gain, dkv, kv_rank, rot_dim, kv_gain, eps,
                 static_cast<__nv_bfloat16*>(cache), rot_dims, interleaved ? 1 : 0, l2b, pos_dev, p0);
    count_launch();
}

void latent_q_absorb(float* qa, const float* q, const void* W_uk, DType dt, int T, int heads, int dim, int rot_dim, int kv_rank, int rot_dims,
                     bool interleaved, float rot_base, const int* pos_dev, int p0, cudaStream_t s) {
    if (T <= 0) return;
    const size_t smem = sizeof(float) * (LT * (size_t)(dim + rot_dim) + 4 * 64 * LT);
    NT_CHECK(smem <= 48 * 1024, "latent_q_absorb: query heads wider than 1280 are not covered");
    const double l2b = std::log2((double)rot_base);
    const dim3 grid((T + LT - 1) / LT, heads, (kv_rank + 63) / 64);
#define NT_QA(TY) launch_k(latent_q_absorb_kernel<TY>, grid, dim3(256), smem, s, qa, q, static_cast<const TY*>(W_uk), T, heads, dim, rot_dim, kv_rank, rot_dims, \
                           interleaved ? 1 : 0, l2b, pos_dev, p0)
    if (dt == DType::F32) NT_QA(float); else if (dt == DType::F16) NT_QA(__half); else if (dt == DType::BF16) NT_QA(__nv_bfloat16);
    else NT_CHECK(false, "latent_q_absorb: dense dtypes only");
#undef NT_QA
    count_launch();
}

void latent_v_up(float* out, const float* ol, const void* W_uv, DType dt, int T, int heads, int vdim, int kv_rank, cudaStream_t s) {
    if (T <= 0) return;
    const size_t smem = sizeof(float) * LT * (size_t)kv_rank;
    NT_CHECK(smem <= 48 * 1024, "latent_v_up: latents wider than 1536 are not covered");
    const dim3 grid((T + LT - 1) / LT, heads, (vdim + 31) / 32);
#define NT_VU(TY) launch_k(latent_v_up_kernel<TY>, grid, dim3(256), smem, s, out, ol, static_cast<const TY*>(W_uv), T, heads, vdim, kv_rank)
    if (dt == DType::F32) NT_VU(float); else if (dt == DType::F16) NT_VU(__half); else if (dt == DType::BF16) NT_VU(__nv_bfloat16);
    else NT_CHECK(false, "latent_v_up: dense dtypes only");
#undef NT_VU
    count_launch();
}

void latent_rows_f32(float* out, const void* cache, DType cache_dt, int row, int kv_rank, int r0, int n, cudaStream_t s) {
    if (n <= 0) return;
    NT_CHECK(cache_dt == DType::BF16, "latent_rows_f32: BF16 cache rows");
    const size_t total = (size_t)n * kv_rank;
    launch_k(latent_rows_f32_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, s, out, static_cast<const __nv_bfloat16*>(cache), row, kv_rank, r0, total);
    count_launch();
}

void latent_expand_pack(void* kfull, void* vfull, const float* ku, const float* vu, const void* cache, DType cache_dt, int kv_rank, int r0, int n, int heads,
                        int dim, int rot_dim, int vdim, int kw, int vw, cudaStream_t s) {
    if (n <= 0) return;
    NT_CHECK(cache_dt == DType::BF16, "latent_expand_pack: BF16 cache rows");
    NT_CHECK(kw >= dim + rot_dim && vw >= vdim, "latent_expand_pack: padded widths below the head's");
    launch_k(latent_expand_pack_kernel, dim3(n, heads), dim3(256), 0, s, static_cast<__nv_bfloat16*>(kfull), static_cast<__nv_bfloat16*>(vfull), ku, vu,
             static_cast<const __nv_bfloat16*>(cache), kv_rank + rot_dim, kv_rank, r0, heads, dim, rot_dim, vdim, kw, vw);
    count_launch();
}

void latent_q_rot_pad(float* qp, const float* q, int T, int heads, int dim, int rot_dim, int kw, int rot_dims, bool interleaved, float rot_base, int p0,
                      cudaStream_t s) {
    if (T <= 0) return;
    launch_k(latent_q_rot_pad_kernel, dim3(T, heads), dim3(256), 0, s, qp, q, heads, dim, rot_dim, kw, rot_dims, interleaved ? 1 : 0, std::log2((double)rot_base), p0);
    count_launch();
}

void latent_unpad(float* out, const float* o, int T, int heads, int vdim, int vw, cudaStream_t s) {
    const size_t total = (size_t)T * heads * vdim;
    if (!total) return;
    launch_k(latent_unpad_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, s, out, o, vdim, vw, total);
    count_launch();
}

// ---- attention over one shared key / value head (see latent_shared_attn_kernel) ----
namespace { constexpr int LS_MAX_PARTS = 512; }           // (query, slice) pairs per launch: bounds the scratch

bool attention_shared_rows_supported(int heads, int dim, int vdim, int row, DType cache_dt, const void* cache) {
    static const bool off = getenv("NT_B200_NO_SHARED_ROWS") != nullptr;
    if (off || (cache_dt != DType::F32 && cache_dt != DType::BF16)) return false;
    const int vn = cache_dt == DType::F32 ? 4 : 8;
    const size_t smem = sizeof(float) * ((size_t)heads * dim + (size_t)heads * LS_KEYS) + (size_t)LS_KEYS * (dim + vn) * (cache_dt == DType::F32 ? 4 : 2);
    return heads >= 1 && heads <= 8 * LS_HB && dim % vn == 0 && row % vn == 0 && dim <= row && vdim <= row && vdim % 2 == 0 && vdim <= 64 * LS_CC &&
           (reinterpret_cast<uintptr_t>(cache) & 15) == 0 && smem <= 200 * 1024;
}
int attention_shared_rows_slices(int tokens, int max_seq) {
    return std::max(1, std::min({(max_seq + LS_KEYS - 1) / LS_KEYS, LS_MAX_PARTS / std::max(1, tokens), 128}));      // one query: up to 128 CTAs
}
size_t attention_shared_rows_scratch_floats(int heads, int vdim) { return (size_t)LS_MAX_PARTS * heads * ((size_t)vdim + 2); }

// out [tokens, heads, vdim]; Q [tokens, heads, dim]; scratch >= attention_shared_rows_scratch_floats.  The grid depends on tokens and
// max_seq only, never on the position: the captured decode step replays it unchanged.
void attention_shared_rows(float* out, const float* Q, const void* cache, DType cache_dt, int tokens, const int* pos_dev, int p0, int max_seq, int heads, int dim,
                           int vdim, int row, float scale, float* scratch, cudaStream_t s) {
    if (tokens <= 0) return;
    NT_CHECK(attention_shared_rows_supported(heads, dim, vdim, row, cache_dt, cache), "attention_shared_rows: shape not covered");
    const bool f32 = cache_dt == DType::F32;
    const int vn = f32 ? 4 : 8;
    const size_t smem = sizeof(float) * ((size_t)heads * dim + (size_t)heads * LS_KEYS) + (size_t)LS_KEYS * (dim + vn) * (f32 ? 4 : 2);
    for (int t0 = 0; t0 < tokens; t0 += LS_MAX_PARTS) {           // long portions (exact mode): blocks of queries with one slice each
        const int nt = std::min(LS_MAX_PARTS, tokens - t0);
        const int slices = attention_shared_rows_slices(nt, max_seq);
        static unsigned long long cfg_f = 0, cfg_b = 0;
        if (f32) {
            opt_in_dynamic_smem(latent_shared_attn_kernel<float>, 200 * 1024, cfg_f);
            launch_k(latent_shared_attn_kernel<float>, dim3(nt, slices), dim3(256), smem, s, scratch, Q + (size_t)t0 * heads * dim, static_cast<const float*>(cache), pos_dev,
                     p0 + t0, heads, dim, vdim, row, scale);
        } else {
            opt_in_dynamic_smem(latent_shared_attn_kernel<__nv_bfloat16>, 200 * 1024, cfg_b);
            launch_k(latent_shared_attn_kernel<__nv_bfloat16>, dim3(nt, slices), dim3(256), smem, s, scratch, Q + (size_t)t0 * heads * dim,
                     static_cast<const __nv_bfloat16*>(cache), pos_dev, p0 + t0, heads, dim, vdim, row, scale);
        }
        count_launch();
        launch_k(latent_shared_merge_kernel, dim3(nt, heads, (vdim + 63) / 64), dim3(256), sizeof(float) * slices, s, out + (size_t)t0 * heads * vdim, (const float*)scratch, slices, heads, vdim);
        count_launch();
    }
}

}}  // namespace nt::b200
