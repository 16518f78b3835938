// ssm_scan.cu — the pieces of a selective state-space mixer around its projections (engine/layer_spec.h ScanSpec):
//   ssm_conv         causal per-channel convolution of `taps` taps + bias + SiLU over the rows of a step; the taps - 1 inputs before
//                    the step's first row come from the sequence's convolution state (zeros when the step starts at position 0)
//   ssm_conv_state   the state's update: the last taps - 1 inputs of [state ++ step rows]
//   ssm_scan         per head h (group g = h / (heads / groups)), state S [state, vdim] in F32:
//                        dt = softplus(dt_raw + dt_bias_h),  S <- exp(-exp(A_log_h) * dt) * S + dt * B_g x_h^T,  y_h = S^T C_g + D_h x_h
//                    sequential over the step's rows; the state is read at the start (zeros at position 0) and written back at the
//                    end, so a prompt cut anywhere continues exactly.  One decoded token: a warp per (head, value channel), lanes over
//                    the state dimension.  Prompt rows: ssm_scan_rows_kernel below
//   ssm_gate_norm    y * silu(z), RMS norm over each of `norm_groups` equal parts, times a gain
// A step's base position is *pos_dev when given (the captured decode step), else p0.  Everything is F32.
// Compiled WITHOUT --use_fast_math (expf / log1pf / division at full precision).
#include "kernels_internal.h"
#include "ring.cuh"
#include <algorithm>
#include <cstdint>

namespace nt { namespace b200 {

namespace {

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// grid (ceil(ch / 256), T)
__global__ void __launch_bounds__(256) ssm_conv_kernel(float* __restrict__ out, const float* __restrict__ u, int ld, int col0, const float* __restrict__ state,
                                                       const float* __restrict__ w, const float* __restrict__ b, int T, int ch, int taps,
                                                       const int* __restrict__ pos_dev, int p0) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x * 256 + threadIdx.x, t = blockIdx.y;
    if (c >= ch) return;
    const bool fresh = (pos_dev ? *pos_dev : p0) == 0;
    float acc = b ? b[c] : 0.f;
    for (int k = 0; k < taps; k++) {
        const int tt = t - (taps - 1) + k;
        float v;
        if (tt >= 0) v = u[(size_t)tt * ld + col0 + c];
        else v = fresh ? 0.f : state[(size_t)(taps - 1 + tt) * ch + c];
        acc = fmaf(w[(size_t)c * taps + k], v, acc);
    }
    out[(size_t)t * ch + c] = silu_f(acc);
}

// One thread per channel; slot j ascending: slot j takes element T + j of [state ++ rows], which lies behind every slot written so far.
__global__ void __launch_bounds__(256) ssm_conv_state_kernel(float* __restrict__ state, const float* __restrict__ u, int ld, int col0, int T, int ch, int taps,
                                                             const int* __restrict__ pos_dev, int p0) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= ch) return;
    const bool fresh = (pos_dev ? *pos_dev : p0) == 0;
    for (int j = 0; j < taps - 1; j++) {
        const int idx = T + j;
        const float v = idx < taps - 1 ? (fresh ? 0.f : state[(size_t)idx * ch + c]) : u[(size_t)(idx - (taps - 1)) * ld + col0 + c];
        state[(size_t)j * ch + c] = v;
    }
}

constexpr int SC_WARPS = 4;
constexpr int SC_NPL = 8;       // state elements per lane: state <= 256

// xbc [T, ch] = [x: heads * vdim | B: groups * N | C: groups * N] (after the convolution); dt_raw = u[t, dt_col0 + h].
// state [heads, vdim, N].  One warp per (h, v).
template <int NPL>
__global__ void __launch_bounds__(SC_WARPS * 32) ssm_scan_kernel(float* __restrict__ y, const float* __restrict__ xbc, int ch, const float* __restrict__ u, int ld,
                                                                 int dt_col0, float* __restrict__ state, const float* __restrict__ dt_bias,
                                                                 const float* __restrict__ A_log, const float* __restrict__ D, int T, int heads, int vdim,
                                                                 int N, int groups, const int* __restrict__ pos_dev, int p0) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hv = blockIdx.x * SC_WARPS + warp;
    if (hv >= heads * vdim) return;
    const int h = hv / vdim, v = hv % vdim, g = h / (heads / groups);
    const bool fresh = (pos_dev ? *pos_dev : p0) == 0;
    float* st = state + (size_t)hv * N;
    float S[NPL];
#pragma unroll
    for (int e = 0; e < NPL; e++) { const int n = lane + 32 * e; S[e] = (!fresh && n < N) ? st[n] : 0.f; }
    const float a_h = -expf(A_log[h]), bias = dt_bias[h], d_h = D[h];
    const int inner = heads * vdim;
    const float* Bp = xbc + inner + (size_t)g * N;
    const float* Cp = Bp + (size_t)groups * N;
    for (int t = 0; t < T; t++) {
        const float dt = softplus_f(u[(size_t)t * ld + dt_col0 + h] + bias);
        const float decay = expf(a_h * dt);
        const float x = xbc[(size_t)t * ch + hv];
        const float dx = dt * x;
        float part = 0.f;
#pragma unroll
        for (int e = 0; e < NPL; e++) {
            const int n = lane + 32 * e;
            if (n < N) {
                S[e] = fmaf(decay, S[e], dx * Bp[(size_t)t * ch + n]);
                part = fmaf(S[e], Cp[(size_t)t * ch + n], part);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xFFFFFFFFu, part, o);
        if (lane == 0) y[(size_t)t * inner + hv] = fmaf(d_h, x, part);
    }
#pragma unroll
    for (int e = 0; e < NPL; e++) { const int n = lane + 32 * e; if (n < N) st[n] = S[e]; }
}

// Prompt rows.  A CTA owns VB (32, or 16 when that is what fills the SMs) value channels of one head, LN (8 or 16) lanes per channel,
// NPT state elements per lane (lane l holds elements 4 (l + LN q) + j), so the channels of a warp share every B_t / C_t read as one
// broadcast 16-byte load.  The kernel is bound by instruction latency (one to two warps per scheduler), so states of 64 and more take
// 16 lanes per channel: twice the warps, half the chain per lane.  The step's rows come through
// shared memory in tiles of TT tokens (cp.async, two buffers): B and C of the head's group, the channels' x, the head's raw dt; softplus
// and the decay's exponential are computed once per (token, head) when a tile lands, outside the serial chain.  The chain itself is
// NPT multiply-adds for the state, NPT for y, and three shuffles per token.
__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
template <int NPT, int SR_VB, int LN>
__global__ void __launch_bounds__(SR_VB * LN) ssm_scan_rows_kernel(float* __restrict__ y, const float* __restrict__ xbc, int ch, const float* __restrict__ u, int ld,
                                                            int dt_col0, float* __restrict__ state, const float* __restrict__ dt_bias,
                                                            const float* __restrict__ A_log, const float* __restrict__ D, int T, int heads, int vdim,
                                                            int N, int groups, int p0) {
    constexpr int TT = LN * NPT > 128 ? 8 : 16, NS = LN * NPT, BUF = 2 * TT * NS + TT * SR_VB + TT;
    extern __shared__ __align__(16) float sm[];
    float* ysm = sm + 2 * BUF;             // [TT][SR_VB]
    float* dd = ysm + TT * SR_VB;          // [2][TT]: dt, decay
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.y, v0 = blockIdx.x * SR_VB, g = h / (heads / groups);
    const int pair = threadIdx.x / LN, l = threadIdx.x % LN, v = v0 + pair;
    const bool live = v < vdim;
    const int inner = heads * vdim;
    for (int e = threadIdx.x; e < 2 * BUF; e += SR_VB * LN) sm[e] = 0.f;          // the pad columns n >= N stay zero: cp.async never writes them
    __syncthreads();
    const float* Bp = xbc + inner + (size_t)g * N;
    const float* Cp = Bp + (size_t)groups * N;
    const bool vec = ((N | ch | inner) & 3) == 0 && (reinterpret_cast<uintptr_t>(xbc) & 15) == 0;
    auto stage = [&](int k, int b) {
        float* Bs = sm + b * BUF; float* Cs = Bs + TT * NS; float* xs = Cs + TT * NS; float* ds = xs + TT * SR_VB;
        const int t0 = k * TT, nt = min(TT, T - t0);
        if (vec) {                                          // 16-byte copies: N, the row stride and the B / C offsets are multiples of 4 floats
            const int n4 = N >> 2;
            for (int e = threadIdx.x; e < nt * n4; e += SR_VB * LN) {
                const int tt = e / n4, n = (e - tt * n4) << 2;
                cp_async16(Bs + tt * NS + n, Bp + (size_t)(t0 + tt) * ch + n);
                cp_async16(Cs + tt * NS + n, Cp + (size_t)(t0 + tt) * ch + n);
            }
        } else {
            for (int e = threadIdx.x; e < nt * N; e += SR_VB * LN) {
                const int tt = e / N, n = e % N;
                cp_async4(Bs + tt * NS + n, Bp + (size_t)(t0 + tt) * ch + n);
                cp_async4(Cs + tt * NS + n, Cp + (size_t)(t0 + tt) * ch + n);
            }
        }
        for (int e = threadIdx.x; e < nt * SR_VB; e += SR_VB * LN) {
            const int tt = e / SR_VB, vv = e % SR_VB;
            if (v0 + vv < vdim) cp_async4(xs + e, xbc + (size_t)(t0 + tt) * ch + (size_t)h * vdim + v0 + vv);
        }
        if (threadIdx.x < nt) cp_async4(ds + threadIdx.x, u + (size_t)(t0 + threadIdx.x) * ld + dt_col0 + h);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float S[NPT];
    float* st = state + ((size_t)h * vdim + (live ? v : 0)) * N;
#pragma unroll
    for (int q = 0; q < NPT / 4; q++)
#pragma unroll
        for (int j = 0; j < 4; j++) { const int n = 4 * (l + LN * q) + j; S[4 * q + j] = (p0 != 0 && live && n < N) ? st[n] : 0.f; }
    const float a_h = -expf(A_log[h]), bias = dt_bias[h], d_h = D[h];
    const int n_tiles = (T + TT - 1) / TT;
    stage(0, 0);
    for (int k = 0; k < n_tiles; k++) {
        const int b = k & 1, t0 = k * TT, nt = min(TT, T - t0);
        if (k + 1 < n_tiles) { stage(k + 1, b ^ 1); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const float* Bs = sm + b * BUF; const float* Cs = Bs + TT * NS; const float* xs = Cs + TT * NS; const float* ds = xs + TT * SR_VB;
        if (threadIdx.x < nt) {
            const float dt = softplus_f(ds[threadIdx.x] + bias);
            dd[threadIdx.x] = dt; dd[TT + threadIdx.x] = expf(a_h * dt);
        }
        __syncthreads();
        float yv[TT];                                       // this channel's outputs of the tile: stored behind the loop, so that no shared
                                                            // store stands between one token's loads and the next one's
        auto step = [&](int tt) {
            const float dt = dd[tt], decay = dd[TT + tt];
            const float x = live ? xs[tt * SR_VB + pair] : 0.f, dx = dt * x;
            float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int q = 0; q < NPT / 4; q++) {
                const float4 bv = *reinterpret_cast<const float4*>(Bs + tt * NS + 4 * (l + LN * q));
                const float4 cv = *reinterpret_cast<const float4*>(Cs + tt * NS + 4 * (l + LN * q));
                S[4 * q + 0] = fmaf(decay, S[4 * q + 0], dx * bv.x); part[0] = fmaf(S[4 * q + 0], cv.x, part[0]);
                S[4 * q + 1] = fmaf(decay, S[4 * q + 1], dx * bv.y); part[1] = fmaf(S[4 * q + 1], cv.y, part[1]);
                S[4 * q + 2] = fmaf(decay, S[4 * q + 2], dx * bv.z); part[2] = fmaf(S[4 * q + 2], cv.z, part[2]);
                S[4 * q + 3] = fmaf(decay, S[4 * q + 3], dx * bv.w); part[3] = fmaf(S[4 * q + 3], cv.w, part[3]);
            }
            float p = (part[0] + part[1]) + (part[2] + part[3]);
            #pragma unroll
            for (int o = 1; o < LN; o <<= 1) p += __shfl_xor_sync(0xFFFFFFFFu, p, o);
            return fmaf(d_h, x, p);
        };
        if (nt == TT) {
#pragma unroll
            for (int tt = 0; tt < TT; tt++) yv[tt] = step(tt);       // independent loads and reductions of neighbouring tokens overlap; only S is carried
        } else {
#pragma unroll
            for (int tt = 0; tt < TT; tt++) if (tt < nt) yv[tt] = step(tt);
        }
        if (l == 0) {
#pragma unroll
            for (int tt = 0; tt < TT; tt++) if (tt < nt) ysm[tt * SR_VB + pair] = yv[tt];
        }
        __syncthreads();
        for (int e = threadIdx.x; e < nt * SR_VB; e += SR_VB * LN) {
            const int tt = e / SR_VB, vv = e % SR_VB;
            if (v0 + vv < vdim) y[(size_t)(t0 + tt) * inner + (size_t)h * vdim + v0 + vv] = ysm[e];
        }
    }
    if (live) {
#pragma unroll
        for (int q = 0; q < NPT / 4; q++)
#pragma unroll
            for (int j = 0; j < 4; j++) { const int n = 4 * (l + LN * q) + j; if (n < N) st[n] = S[4 * q + j]; }
    }
}

// grid (T, norm_groups); z = u[t, z_col0 + i]
__global__ void __launch_bounds__(256) ssm_gate_norm_kernel(float* __restrict__ out, const float* __restrict__ y, const float* __restrict__ u, int ld, int z_col0,
                                                            const float* __restrict__ gain, float eps, int inner, int per) {
    __shared__ float red[8];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, i0 = blockIdx.y * per;
    float ss = 0.f;
    for (int i = threadIdx.x; i < per; i += 256) {
        const float v = y[(size_t)t * inner + i0 + i] * silu_f(u[(size_t)t * ld + z_col0 + i0 + i]);
        ss = fmaf(v, v, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) tot += red[w];
    const float inv = 1.0f / sqrtf(tot / (float)per + eps);
    for (int i = threadIdx.x; i < per; i += 256) {
        const float v = y[(size_t)t * inner + i0 + i] * silu_f(u[(size_t)t * ld + z_col0 + i0 + i]);
        out[(size_t)t * inner + i0 + i] = v * inv * gain[i0 + i];
    }
}

}  // namespace

void ssm_conv(float* out, const float* u, int ld, int col0, float* conv_state, const float* w, const float* b, int T, int ch, int taps,
              const int* pos_dev, int p0, cudaStream_t s) {
    if (T <= 0 || ch <= 0) return;
    NT_CHECK(taps >= 1, "ssm_conv: at least one tap");
    launch_k(ssm_conv_kernel, dim3((ch + 255) / 256, T), dim3(256), 0, s, out, u, ld, col0, (const float*)conv_state, w, b, T, ch, taps, pos_dev, p0);
    count_launch();
    if (taps > 1) {
        launch_k(ssm_conv_state_kernel, dim3((ch + 255) / 256), dim3(256), 0, s, conv_state, u, ld, col0, T, ch, taps, pos_dev, p0);
        count_launch();
    }
}

void ssm_scan(float* y, const float* xbc, const float* u, int ld, int dt_col0, float* state, const float* dt_bias, const float* A_log, const float* D,
              int T, int heads, int vdim, int N, int groups, const int* pos_dev, int p0, cudaStream_t s) {
    if (T <= 0) return;
    NT_CHECK(N >= 1 && N <= 32 * SC_NPL, "ssm_scan: state sizes up to 256 are covered");
    NT_CHECK(groups >= 1 && heads % groups == 0, "ssm_scan: heads must be a multiple of groups");
    const int ch = heads * vdim + 2 * groups * N;
    static const bool no_rows = getenv("NT_B200_NO_SCAN_ROWS") != nullptr;
    if (T > 1 && !pos_dev && !no_rows) {
        const bool narrow = vdim <= 16 || heads * ((vdim + 31) / 32) < 148;       // 16 channels per CTA: twice the CTAs
#define NT_SCAN_ROWS_V(NPT, VB, LN) do { constexpr int TT = LN * NPT > 128 ? 8 : 16; \
        launch_k(ssm_scan_rows_kernel<NPT, VB, LN>, dim3((vdim + VB - 1) / VB, heads), dim3(VB * LN), \
                 sizeof(float) * (2 * (2 * TT * LN * NPT + TT * VB + TT) + TT * VB + 2 * TT), \
                 s, y, xbc, ch, u, ld, dt_col0, state, dt_bias, A_log, D, T, heads, vdim, N, groups, p0); } while (0)
#define NT_SCAN_ROWS(NPT, LN) do { if (narrow) NT_SCAN_ROWS_V(NPT, 16, LN); else NT_SCAN_ROWS_V(NPT, 32, LN); } while (0)
        if (N <= 32) NT_SCAN_ROWS(4, 8); else if (N <= 64) NT_SCAN_ROWS(4, 16); else if (N <= 128) NT_SCAN_ROWS(8, 16); else NT_SCAN_ROWS(16, 16);
#undef NT_SCAN_ROWS
#undef NT_SCAN_ROWS_V
        count_launch();
        return;
    }
    const dim3 grid((heads * vdim + SC_WARPS - 1) / SC_WARPS);
#define NT_SCAN(NPL) launch_k(ssm_scan_kernel<NPL>, grid, dim3(SC_WARPS * 32), 0, s, y, xbc, ch, u, ld, dt_col0, state, dt_bias, A_log, D, T, heads, vdim, N, groups, pos_dev, p0)
    if (N <= 32) NT_SCAN(1); else if (N <= 64) NT_SCAN(2); else if (N <= 128) NT_SCAN(4); else NT_SCAN(8);
#undef NT_SCAN
    count_launch();
}

void ssm_gate_norm(float* out, const float* y, const float* u, int ld, int z_col0, const float* gain, float eps, int T, int inner, int norm_groups,
                   cudaStream_t s) {
    if (T <= 0) return;
    NT_CHECK(norm_groups >= 1 && inner % norm_groups == 0, "ssm_gate_norm: the parts must be equal");
    launch_k(ssm_gate_norm_kernel, dim3(T, norm_groups), dim3(256), 0, s, out, y, u, ld, z_col0, gain, eps, inner, inner / norm_groups);
    count_launch();
}

}}  // namespace nt::b200
