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

// grid (ceil(T / LT), heads).  q [T, heads, dim + rot_dim]; qa [T, heads, kv_rank + rot_dim]; W_uk [heads * dim, kv_rank]
template <typename WT>
__global__ void __launch_bounds__(256) latent_q_absorb_kernel(float* __restrict__ qa, const float* __restrict__ q, const WT* __restrict__ W_uk, int T, int heads,
                                                              int dim, int rot_dim, int kv_rank, int dims, int interleaved, double log2_base,
                                                              const int* __restrict__ pos_dev, int p0) {
    extern __shared__ __align__(16) float qs[];           // [LT][dim + rot_dim]
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.x * LT, h = blockIdx.y, qd = dim + rot_dim, od = kv_rank + rot_dim;
    const int nt = min(LT, T - t0);
    for (int e = threadIdx.x; e < LT * qd; e += 256) {
        const int tt = e / qd, i = e % qd;
        qs[e] = tt < nt ? q[((size_t)(t0 + tt) * heads + h) * qd + i] : 0.f;
    }
    __syncthreads();
    const WT* Wh = W_uk + (size_t)h * dim * kv_rank;
    for (int r = threadIdx.x; r < kv_rank; r += 256) {
        float acc[LT];
#pragma unroll
        for (int tt = 0; tt < LT; tt++) acc[tt] = 0.f;
        for (int d = 0; d < dim; d++) {
            const float w = wld(Wh, (size_t)d * kv_rank + r);
#pragma unroll
            for (int tt = 0; tt < LT; tt++) acc[tt] = fmaf(w, qs[tt * qd + d], acc[tt]);
        }
#pragma unroll
        for (int tt = 0; tt < LT; tt++) if (tt < nt) qa[((size_t)(t0 + tt) * heads + h) * od + r] = acc[tt];
    }
    const int base = pos_dev ? *pos_dev : p0;
    for (int e = threadIdx.x; e < nt * rot_dim; e += 256) {
        const int tt = e / rot_dim, i = e % rot_dim;
        qa[((size_t)(t0 + tt) * heads + h) * od + kv_rank + i] = rotated(qs + tt * qd + dim, i, dims, interleaved, log2_base, base + t0 + tt);
    }
}

// grid (ceil(T / LT), heads).  ol [T, heads, kv_rank]; out [T, heads * vdim]; W_uv [heads * vdim, kv_rank].  A warp per output channel.
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
    for (int v = warp; v < vdim; v += 8) {
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
    const size_t smem = sizeof(float) * LT * (size_t)(dim + rot_dim);
    NT_CHECK(smem <= 48 * 1024, "latent_q_absorb: query heads wider than 1536 are not covered");
    const double l2b = std::log2((double)rot_base);
    const dim3 grid((T + LT - 1) / LT, heads);
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
    const dim3 grid((T + LT - 1) / LT, heads);
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

}}  // namespace nt::b200
