// attention_heads.cu — what sits between the projections (and their short convolutions) and attention_window for attention with
// per-head query / key norm, and the mixing of softmax weights across heads behind it:
//   head_prep   per token: every dim-wide head of the query and key rows is RMS-normed on its own (x / sqrt(mean x^2 + eps) * gain, one
//               gain vector of the head's width shared by all heads; null: no norm); the first `dims` channels of every head are rotated
//               (channel i with i + dims/2 — or 2i with 2i+1 when interleaved — by angle = position * freq[i], F32, the table made on the
//               host with any frequency scaling folded in); query head h is then multiplied by temp[h] (a per-head score multiplier,
//               null: none); queries in place, keys into cache row base + t.  Values: v <- (1 - lambda) v + lambda v_first[t] when a
//               blend is given (v_first: the values another layer computed for the same tokens, F32, [T, vdim]); the values as the layer
//               computed them are published to v_publish when given; then into the cache row.
//   talk_mix    out[t, h, :] = sum_g M[h, g] A[t, g, kv(h), :] where A[t, g, c, :] = sum_j w_g(t, j) v_c(j) is what attention_window
//               yields when query head g is applied to the values of EVERY key / value head c (WindowAttn::joint_v): mixing the
//               normalised weights of the heads, w_h <- sum_g M[h, g] w_g, and then applying them to head h's own values is linear in the
//               weights, so it equals this sum of the per-head results; the softmax of each head stays an ordinary online softmax.
// A step's base position is *pos_dev when given (the captured decode step), else p0.  All F32; compiled WITHOUT --use_fast_math.
#include "kernels_internal.h"
#include "ring.cuh"
#include <cuda_bf16.h>
#include <algorithm>

namespace nt { namespace b200 {

namespace {

__device__ __forceinline__ void cst(float* p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void cst(__nv_bfloat16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// One head in shared memory: norm, rotate; `row` [dim] is overwritten with the result.  Called by one warp.
__device__ __forceinline__ void norm_rotate_head(float* row, int dim, const float* __restrict__ gain, float eps, int dims, bool interleaved,
                                                 const float* cs, const float* sn, int lane) {
    if (gain) {
        float ss = 0.f;
        for (int i = lane; i < dim; i += 32) ss = fmaf(row[i], row[i], ss);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
        const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
        for (int i = lane; i < dim; i += 32) row[i] = row[i] * inv * gain[i];
        __syncwarp();
    }
    const int half = dims >> 1;
    for (int i = lane; i < half; i += 32) {
        const int c0 = interleaved ? 2 * i : i, c1 = interleaved ? 2 * i + 1 : i + half;
        const float u = row[c0], v = row[c1];
        row[c0] = u * cs[i] - v * sn[i];
        row[c1] = v * cs[i] + u * sn[i];
    }
    __syncwarp();
}

// grid (T, y), 256 threads: the CTAs of a token share its heads (a warp per head) and value channels, each with its own cos / sin of the
// position; shared: cos[dims/2] | sin[dims/2] | one head per warp [8][dim]
template <typename KT>
__global__ void __launch_bounds__(256) head_prep_kernel(float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V, HeadPrep p,
                                                        KT* __restrict__ kc, KT* __restrict__ vc, const int* __restrict__ pos_dev, int p0) {
    extern __shared__ float sm[];
    const int half = p.rot_dims >> 1;
    float* cs = sm;
    float* sn = sm + half;
    float* rows = sn + half;
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();
    const int pos = (pos_dev ? *pos_dev : p0) + t;
    for (int i = threadIdx.x; i < half; i += 256) sincosf((float)pos * p.freq[i], &sn[i], &cs[i]);
    __syncthreads();
    float* row = rows + (size_t)warp * p.dim;
    const int n_heads = p.heads + p.kv_heads;
    for (int hh = blockIdx.y * 8 + warp; hh < n_heads; hh += 8 * gridDim.y) {
        const bool is_q = hh < p.heads;
        const int h = is_q ? hh : hh - p.heads;
        const float* src = is_q ? Q + ((size_t)t * p.heads + h) * p.dim : K + ((size_t)t * p.kv_heads + h) * p.dim;
        for (int i = lane; i < p.dim; i += 32) row[i] = src[i];
        __syncwarp();
        norm_rotate_head(row, p.dim, is_q ? p.q_gain : p.k_gain, p.eps, p.rot_dims, p.interleaved != 0, cs, sn, lane);
        if (is_q) {
            const float m = p.temp ? p.temp[h] : 1.f;
            float* dst = Q + ((size_t)t * p.heads + h) * p.dim;
            for (int i = lane; i < p.dim; i += 32) dst[i] = row[i] * m;
        } else {
            const size_t base = ((size_t)pos * p.kv_heads + h) * p.dim;
            for (int i = lane; i < p.dim; i += 32) cst(kc, base + i, row[i]);
        }
        __syncwarp();
    }
    const int vw = p.kv_heads * p.vdim;
    const float lam = p.v_lambda ? *p.v_lambda : 0.f;
    for (int i = blockIdx.y * 256 + threadIdx.x; i < vw; i += 256 * gridDim.y) {
        float v = V[(size_t)t * vw + i];
        if (p.v_publish) p.v_publish[(size_t)t * vw + i] = v;
        if (p.v_first) v = (1.0f - lam) * v + lam * p.v_first[(size_t)t * vw + i];
        cst(vc, (size_t)pos * vw + i, v);
    }
}

// grid (T, heads)
__global__ void __launch_bounds__(128) talk_mix_kernel(float* __restrict__ out, const float* __restrict__ A, const float* __restrict__ M, int heads, int kv_heads,
                                                       int vdim, size_t t_stride, size_t g_stride, size_t c_stride) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y, c = h / (heads / kv_heads);
    const float* a = A + (size_t)t * t_stride + (size_t)c * c_stride;
    for (int i = threadIdx.x; i < vdim; i += 128) {
        float acc = 0.f;
        for (int g = 0; g < heads; g++) acc = fmaf(M[h * heads + g], a[(size_t)g * g_stride + i], acc);
        out[((size_t)t * heads + h) * vdim + i] = acc;
    }
}

}  // namespace

void head_prep(float* Q, const float* K, const float* V, const HeadPrep& p, void* kc, void* vc, DType cache_dt, int tokens, const int* pos_dev, int p0,
               cudaStream_t s) {
    NT_CHECK(cache_dt == DType::F32 || cache_dt == DType::BF16, "head_prep: F32 or BF16 cache");
    NT_CHECK(p.rot_dims >= 0 && p.rot_dims <= p.dim && !(p.rot_dims & 1) && (p.rot_dims == 0 || p.freq), "head_prep: rot_dims must be even, at most dim, with a frequency table");
    if (tokens <= 0) return;
    const size_t smem = sizeof(float) * ((size_t)p.rot_dims + (size_t)8 * p.dim);
    NT_CHECK(smem <= 48 * 1024, "head_prep: heads wider than the kernel's shared memory");
    const int ny = std::max(1, std::min(8, (p.heads + p.kv_heads + 7) / 8));       // a decoded token has one row: spread its heads over a few CTAs
    if (cache_dt == DType::F32)
        launch_k(head_prep_kernel<float>, dim3(tokens, ny), dim3(256), smem, s, Q, K, V, p, static_cast<float*>(kc), static_cast<float*>(vc), pos_dev, p0);
    else
        launch_k(head_prep_kernel<__nv_bfloat16>, dim3(tokens, ny), dim3(256), smem, s, Q, K, V, p, static_cast<__nv_bfloat16*>(kc), static_cast<__nv_bfloat16*>(vc),
                 pos_dev, p0);
    count_launch();
}

void talk_mix(float* out, const float* A, const float* M, int tokens, int heads, int kv_heads, int vdim, size_t t_stride, size_t g_stride, size_t c_stride,
              cudaStream_t s) {
    if (tokens <= 0) return;
    launch_k(talk_mix_kernel, dim3(tokens, heads), dim3(128), 0, s, out, A, M, heads, kv_heads, vdim, t_stride, g_stride, c_stride);
    count_launch();
}

}}  // namespace nt::b200
