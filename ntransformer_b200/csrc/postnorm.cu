// postnorm.cu — row-wise pieces of the post-norm block form (engine/layer_spec.h BlockForm::POST_NORM) and of its per-layer token
// input, all F32:
//   add_rmsnorm_rows   x[t] += rms(y[t] + bias) * gain        (a sublayer's output is normed, then joins the residual)
//   glu_bias_mul       out = act(gate + b_g) * (up + b_u)      (biases may be null)
//   side_gate_rows     g[t, j] <- gelu_tanh(g[t, j]) * E[token_t, col0 + j]     (E: a second embedding table, any dense dtype)
// One CTA per row; a row is read twice (sum of squares, then the update), both times from L1/L2.
// Compiled WITHOUT --use_fast_math.
#include "kernels_internal.h"
#include "ring.cuh"
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace nt { namespace b200 {

namespace {

__device__ __forceinline__ float gelu_tanh_f(float z) { return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

__global__ void __launch_bounds__(256) add_rmsnorm_rows_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ gain,
                                                               const float* __restrict__ bias, int width, float eps) {
    __shared__ float red[8];
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    const float* yr = y + t * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += 256) { const float v = yr[i] + (bias ? bias[i] : 0.f); ss = fmaf(v, v, ss); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) tot += red[w];
    const float inv = 1.0f / sqrtf(tot / (float)width + eps);
    float* xr = x + t * width;
    for (int i = threadIdx.x; i < width; i += 256) { const float v = yr[i] + (bias ? bias[i] : 0.f); xr[i] += v * inv * gain[i]; }
}

__global__ void glu_bias_mul_kernel(float* __restrict__ out, const float* __restrict__ gate, const float* __restrict__ up, const float* __restrict__ bg,
                                    const float* __restrict__ bu, size_t n, int cols, int gelu) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int c = (int)(i % cols);
    const float g = gate[i] + (bg ? bg[c] : 0.f), u = up[i] + (bu ? bu[c] : 0.f);
    out[i] = (gelu ? gelu_tanh_f(g) : silu_f(g)) * u;
}

template <typename ET>
__device__ __forceinline__ float eld(const ET* p, size_t i);
template <> __device__ __forceinline__ float eld<float>(const float* p, size_t i) { return p[i]; }
template <> __device__ __forceinline__ float eld<__half>(const __half* p, size_t i) { return __half2float(p[i]); }
template <> __device__ __forceinline__ float eld<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }

template <typename ET>
__global__ void side_gate_rows_kernel(float* __restrict__ g, const ET* __restrict__ E, int e_cols, int col0, const int* __restrict__ tokens, size_t n, int dim) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t t = i / dim, j = i % dim;
    g[i] = gelu_tanh_f(g[i]) * eld<ET>(E, (size_t)tokens[t] * e_cols + col0 + j);
}

}  // namespace

void add_rmsnorm_rows(float* x, const float* y, const float* gain, const float* bias, int rows, int width, float eps, cudaStream_t s) {
    if (rows <= 0) return;
    launch_k(add_rmsnorm_rows_kernel, dim3(rows), dim3(256), 0, s, x, y, gain, bias, width, eps);
    count_launch();
}

void glu_bias_mul(float* out, const float* gate, const float* up, const float* gate_bias, const float* up_bias, int rows, int cols, bool gelu, cudaStream_t s) {
    const size_t n = (size_t)rows * cols;
    if (!n) return;
    launch_k(glu_bias_mul_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, out, gate, up, gate_bias, up_bias, n, cols, gelu ? 1 : 0);
    count_launch();
}

void side_gate_rows(float* g, const void* E, DType dt, int e_cols, int col0, const int* tokens_dev, int rows, int dim, cudaStream_t s) {
    const size_t n = (size_t)rows * dim;
    if (!n) return;
    const dim3 grid((unsigned)((n + 255) / 256));
    if (dt == DType::F32) launch_k(side_gate_rows_kernel<float>, grid, dim3(256), 0, s, g, static_cast<const float*>(E), e_cols, col0, tokens_dev, n, dim);
    else if (dt == DType::F16) launch_k(side_gate_rows_kernel<__half>, grid, dim3(256), 0, s, g, static_cast<const __half*>(E), e_cols, col0, tokens_dev, n, dim);
    else if (dt == DType::BF16) launch_k(side_gate_rows_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, g, static_cast<const __nv_bfloat16*>(E), e_cols, col0, tokens_dev, n, dim);
    else NT_CHECK(false, "side_gate_rows: dense dtypes only");
    count_launch();
}

}}  // namespace nt::b200
