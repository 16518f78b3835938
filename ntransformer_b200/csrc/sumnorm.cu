// sumnorm.cu — row-wise pieces of the block form that norms the residual sum itself (engine/layer_spec.h BlockForm::SUM_NORM) and of
// the token shift in front of a mixer (LayerSpec::token_shift), all F32:
//   sum_rmsnorm_rows   x[t] <- rms(a x[t] + s1 (y1[t] + b1) + s2 y2[t]) * gain      (y2, b1 may be null; gain already holds its offset)
//                      and, when a shift is given, the NEXT mixer's input in the same pass: h[t] = x'[t] + (x'[t-1] - x'[t]) mu with
//                      x'[-1] the carried row (zeros when the step starts at position 0); one row only (a decoded token): the carried
//                      row is then replaced by x'[t]
//   token_shift_rows   h[t] = x[t] + (x[t-1] - x[t]) mu for the rows of a step, x[-1] from the carried row; token_shift_keep stores the
//                      step's last row as the new carried row (a launch of its own for more than one row: every row must have read
//                      the old one first)
// One CTA per row; a row is read twice (sum of squares, then the result), both times from L1/L2.
// A step's base position is *pos_dev when given (the captured decode step), else p0.  Compiled WITHOUT --use_fast_math.
#include "kernels_internal.h"
#include "ring.cuh"

namespace nt { namespace b200 {

namespace {

__global__ void __launch_bounds__(256) sum_rmsnorm_rows_kernel(float* __restrict__ x, float a, const float* __restrict__ y1, float s1, const float* __restrict__ b1,
                                                               const float* __restrict__ y2, float s2, const float* __restrict__ gain, int width, float eps,
                                                               float* __restrict__ h_next, const float* __restrict__ mu, float* __restrict__ carried,
                                                               const int* __restrict__ pos_dev, int p0) {
    __shared__ float red[8];
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    float* xr = x + t * width;
    const float* r1 = y1 + t * width;
    const float* r2 = y2 ? y2 + t * width : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += 256) {
        float v = fmaf(a, xr[i], s1 * (r1[i] + (b1 ? b1[i] : 0.f)));
        if (r2) v = fmaf(s2, r2[i], v);
        ss = fmaf(v, v, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) tot += red[w];
    const float inv = 1.0f / sqrtf(tot / (float)width + eps);
    const bool fresh = (pos_dev ? *pos_dev : p0) == 0;
    for (int i = threadIdx.x; i < width; i += 256) {
        float v = fmaf(a, xr[i], s1 * (r1[i] + (b1 ? b1[i] : 0.f)));
        if (r2) v = fmaf(s2, r2[i], v);
        const float n = v * inv * gain[i];
        xr[i] = n;
        if (h_next) {                                   // one row: shift against the carried row, then carry this one
            const float prev = fresh ? 0.f : carried[i];
            h_next[i] = fmaf(prev - n, mu[i], n);
            carried[i] = n;
        }
    }
}

__global__ void __launch_bounds__(256) token_shift_rows_kernel(float* __restrict__ h, const float* __restrict__ x, const float* __restrict__ mu,
                                                               float* __restrict__ carried, int width, int keep, const int* __restrict__ pos_dev, int p0) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    const bool fresh = (pos_dev ? *pos_dev : p0) == 0;
    const float* xr = x + t * width;
    for (int i = threadIdx.x; i < width; i += 256) {
        const float cur = xr[i];
        const float prev = t > 0 ? xr[i - width] : (fresh ? 0.f : carried[i]);
        h[t * width + i] = fmaf(prev - cur, mu[i], cur);
        if (keep) carried[i] = cur;
    }
}

}  // namespace

void sum_rmsnorm_rows(float* x, float a, const float* y1, float s1, const float* b1, const float* y2, float s2, const float* gain, int rows, int width, float eps,
                      cudaStream_t s, float* h_next, const float* mu, float* carried, const int* pos_dev, int p0) {
    if (rows <= 0) return;
    NT_CHECK(!h_next || (rows == 1 && mu && carried), "sum_rmsnorm_rows: the fused shift takes one row, the blend vector and the carried row");
    launch_k(sum_rmsnorm_rows_kernel, dim3(rows), dim3(256), 0, s, x, a, y1, s1, b1, y2, s2, gain, width, eps, h_next, mu, carried, pos_dev, p0);
    count_launch();
}

void token_shift_rows(float* h, const float* x, const float* mu, float* carried, int rows, int width, const int* pos_dev, int p0, cudaStream_t s) {
    if (rows <= 0) return;
    launch_k(token_shift_rows_kernel, dim3(rows), dim3(256), 0, s, h, x, mu, carried, width, rows == 1 ? 1 : 0, pos_dev, p0);
    count_launch();
    if (rows > 1) copy(carried, x + (size_t)(rows - 1) * width, width, s);
}

}}  // namespace nt::b200
