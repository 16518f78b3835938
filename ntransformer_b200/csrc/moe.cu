// moe.cu — routed mixture of squared-ReLU experts, y = sum_{k < top} p_k * W_down[e_k] relu(W_up[e_k] h)^2, plus an optional shared
// expert scaled by sigmoid(<w_sg, h>).  Router logits, the choice and the softmax over the chosen logits are F32.
//   moe_route                one CTA per token: a warp per router row, then the top-k (lowest index wins a tie) and its softmax.
//   decode (one token)       moe_expert_up_token / moe_expert_down_token: warp-per-row GEMVs that read the chosen experts' rows through
//                            a device pointer table (the choice never visits the host, so the step stays inside the CUDA graph);
//                            the shared expert rides in the same two launches as one more slot.
//   prompt rows              moe_group sorts the (token, k) assignments by expert (token order inside an expert), then two gathered
//                            GEMMs (64x64x16 tiles, FP32 FMA on CUDA cores) run every expert over its own rows only, and moe_combine
//                            sums a token's rows in k order.  Every output element is one dot product in a fixed order, so a token's
//                            result does not depend on which other tokens share its tile.
// Variants (MoeWeights): gated experts W_down (silu(W_gate h) * W_up h) through a third pointer table; a router that scores by
// sigmoid, adds a correction vector for the choice only, restricts the choice to the best runs of neighbouring experts and weights
// by the plain scores.
// Expert matrices: F32, F16 or BF16 rows.  Compiled WITHOUT --use_fast_math.
#include "kernels_internal.h"
#include "ring.cuh"
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cfloat>

namespace nt { namespace b200 {

namespace {

template <typename T> struct El;
template <> struct El<float> {
    static constexpr int P = 4;
    static __device__ __forceinline__ float one(const void* row, int i) { return __ldg(static_cast<const float*>(row) + i); }
    static __device__ __forceinline__ void unpack(const uint4& w, float* f) { f[0] = __uint_as_float(w.x); f[1] = __uint_as_float(w.y); f[2] = __uint_as_float(w.z); f[3] = __uint_as_float(w.w); }
};
template <> struct El<__half> {
    static constexpr int P = 8;
    static __device__ __forceinline__ float one(const void* row, int i) { return __half2float(__ushort_as_half(__ldg(static_cast<const unsigned short*>(row) + i))); }
    static __device__ __forceinline__ void unpack(const uint4& w, float* f) {
        const unsigned u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int k = 0; k < 4; k++) { float2 p = __half22float2(*reinterpret_cast<const __half2*>(&u[k])); f[2 * k] = p.x; f[2 * k + 1] = p.y; }
    }
};
template <> struct El<__nv_bfloat16> {
    static constexpr int P = 8;
    static __device__ __forceinline__ float one(const void* row, int i) { return __uint_as_float((unsigned)__ldg(static_cast<const unsigned short*>(row) + i) << 16); }
    static __device__ __forceinline__ void unpack(const uint4& w, float* f) {
        const unsigned u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int k = 0; k < 4; k++) { f[2 * k] = __uint_as_float(u[k] << 16); f[2 * k + 1] = __uint_as_float(u[k] & 0xFFFF0000u); }
    }
};

__device__ __forceinline__ uint4 ld_nc16(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// <row, xs> over K by one warp; vec: the row starts on 16 bytes and K is a multiple of the elements per 16 bytes
template <typename T>
__device__ __forceinline__ float warp_dot(const unsigned char* row, const float* xs, int K, int lane, bool vec) {
    float acc = 0.f;
    constexpr int P = El<T>::P;
    if (vec) {
        const int nv = K / P;
        int v = lane;
        for (; v + 96 < nv; v += 128) {          // four 16-byte loads in flight per lane
            uint4 w[4];
#pragma unroll
            for (int u = 0; u < 4; u++) w[u] = ld_nc16(reinterpret_cast<const uint4*>(row) + v + 32 * u);
#pragma unroll
            for (int u = 0; u < 4; u++) {
                float f[P];
                El<T>::unpack(w[u], f);
                const float* xp = xs + (size_t)(v + 32 * u) * P;
#pragma unroll
                for (int k = 0; k < P; k++) acc = fmaf(f[k], xp[k], acc);
            }
        }
        for (; v < nv; v += 32) {
            float f[P];
            El<T>::unpack(ld_nc16(reinterpret_cast<const uint4*>(row) + v), f);
            const float* xp = xs + (size_t)v * P;
#pragma unroll
            for (int k = 0; k < P; k++) acc = fmaf(f[k], xp[k], acc);
        }
    } else {
        for (int i = lane; i < K; i += 32) acc = fmaf(El<T>::one(row, i), xs[i], acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
    return acc;
}

constexpr int RT_WARPS = 8;
constexpr int MAX_EXPERTS = 256;

__global__ void __launch_bounds__(RT_WARPS * 32) moe_route_kernel(int* __restrict__ sel, float* __restrict__ wt, float* __restrict__ sgate,
                                                                  const float* __restrict__ h, const float* __restrict__ router,
                                                                  const float* __restrict__ shared_gate, int experts, int top, int width,
                                                                  int sigmoid, const float* __restrict__ correction, int groups, int keep, StreamsIO sio, const float* __restrict__ norm_w, float eps, float* __restrict__ h_out) {
    extern __shared__ __align__(16) float hs[];
    __shared__ float z[MAX_EXPERTS + 1];
    __shared__ float sc[MAX_EXPERTS];
    __shared__ float red[RT_WARPS];
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += RT_WARPS * 32) {
        float v;
        if (sio.X_in) {                   // the blend of the token's residual streams
            v = 0.f;
            for (int st = 0; st < sio.S; st++) { const float xv = sio.X_in[((size_t)t * sio.S + st) * width + i]; v = sio.a ? fmaf(sio.a[st], xv, v) : v + xv; }
        } else v = h[(size_t)t * width + i];
        hs[i] = v; ss = fmaf(v, v, ss);
    }
    if (norm_w) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < RT_WARPS; w++) tot += red[w];
        const float inv = 1.0f / sqrtf(tot / (float)width + eps);
        for (int i = threadIdx.x; i < width; i += RT_WARPS * 32) hs[i] = hs[i] * inv * norm_w[i];
    }
    __syncthreads();
    if (h_out) for (int i = threadIdx.x; i < width; i += RT_WARPS * 32) h_out[(size_t)t * width + i] = hs[i];
    const bool vec = width % 4 == 0 && (reinterpret_cast<uintptr_t>(router) & 15) == 0;
    const int rows = experts + (shared_gate ? 1 : 0);
    for (int e = warp; e < rows; e += RT_WARPS) {
        const float* row = e < experts ? router + (size_t)e * width : shared_gate;
        const bool v2 = vec && (reinterpret_cast<uintptr_t>(row) & 15) == 0;
        const float d = warp_dot<float>(reinterpret_cast<const unsigned char*>(row), hs, width, lane, v2);
        if (lane == 0) z[e] = d;
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    if (shared_gate) sgate[t] = 1.0f / (1.0f + expf(-z[experts]));
    if (sigmoid) {
        // scores sigmoid(logit); the choice looks at score + correction, the weight is the plain score of what was chosen
        for (int e = 0; e < experts; e++) { sc[e] = 1.0f / (1.0f + expf(-z[e])); z[e] = sc[e] + (correction ? correction[e] : 0.f); }
        if (groups > 0) {
            // a run of neighbours scores the sum of its two largest choice scores; runs outside the best `keep` drop out (-inf, not 0:
            // choice scores may be negative); the kept runs are a bit mask
            const int per = experts / groups;
            unsigned long long kept[4] = {0ull, 0ull, 0ull, 0ull};
            for (int k = 0; k < keep; k++) {
                int bg = -1;
                float bs = -INFINITY;
                for (int g = 0; g < groups; g++) {
                    if (kept[g >> 6] >> (g & 63) & 1ull) continue;
                    float m1 = -INFINITY, m2 = -INFINITY;
                    for (int e = g * per; e < (g + 1) * per; e++) { const float v = z[e]; if (v > m1) { m2 = m1; m1 = v; } else if (v > m2) m2 = v; }
                    const float gs = per >= 2 ? m1 + m2 : m1;
                    if (bg < 0 || gs > bs) { bs = gs; bg = g; }
                }
                kept[bg >> 6] |= 1ull << (bg & 63);
            }
            for (int g = 0; g < groups; g++)
                if (!(kept[g >> 6] >> (g & 63) & 1ull)) for (int e = g * per; e < (g + 1) * per; e++) z[e] = -INFINITY;
        }
        for (int k = 0; k < top; k++) {
            int best = -1;
            float bv = -INFINITY;
            for (int e = 0; e < experts; e++) if (z[e] > bv) { bv = z[e]; best = e; }      // strict: the lowest index wins a tie
            if (best < 0) best = 0;
            sel[(size_t)t * top + k] = best;
            wt[(size_t)t * top + k] = sc[best];
            z[best] = -INFINITY;
        }
        return;
    }
    // the `top` largest logits, largest first; an expert already taken is marked by -inf
    float zmax = 0.f, den = 0.f;
    for (int k = 0; k < top; k++) {
        int best = 0;
        float bv = -INFINITY;
        for (int e = 0; e < experts; e++) if (z[e] > bv) { bv = z[e]; best = e; }
        if (k == 0) zmax = bv;
        const float p = expf(bv - zmax);
        sel[(size_t)t * top + k] = best;
        wt[(size_t)t * top + k] = p;
        den += p;
        z[best] = -INFINITY;
    }
    for (int k = 0; k < top; k++) wt[(size_t)t * top + k] /= den;
}

struct MoeDev {
    const void* const* gate;       // null: squared-ReLU experts
    const void* const* up; const void* const* down;
    const void* shared_up; const void* shared_down;
    int top, ff, width, shared_ff;
};

constexpr int TK_WARPS = 8;
// act [top * ff + shared_ff]: slot k < top is expert sel[k], the last slot the shared expert
template <typename T>
__global__ void __launch_bounds__(TK_WARPS * 32) moe_up_token_kernel(float* __restrict__ act, const float* __restrict__ h, const int* __restrict__ sel, MoeDev m) {
    extern __shared__ __align__(16) float hs[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();
    for (int i = threadIdx.x; i < m.width; i += TK_WARPS * 32) hs[i] = h[i];
    __syncthreads();
    const int total = m.top * m.ff + m.shared_ff;
    const size_t pitch = (size_t)m.width * sizeof(T);
    const bool kvec = m.width % El<T>::P == 0;
    for (int r = blockIdx.x * TK_WARPS + warp; r < total; r += gridDim.x * TK_WARPS) {
        const unsigned char* base;
        int row;
        if (r < m.top * m.ff) { base = static_cast<const unsigned char*>(m.up[sel[r / m.ff]]); row = r % m.ff; }
        else { base = static_cast<const unsigned char*>(m.shared_up); row = r - m.top * m.ff; }
        const unsigned char* wr = base + (size_t)row * pitch;
        const float d = warp_dot<T>(wr, hs, m.width, lane, kvec && (reinterpret_cast<uintptr_t>(wr) & 15) == 0);
        if (m.gate && r < m.top * m.ff) {       // gated unit: silu(<gate row, h>) * <up row, h>
            const unsigned char* gr = static_cast<const unsigned char*>(m.gate[sel[r / m.ff]]) + (size_t)row * pitch;
            const float g = warp_dot<T>(gr, hs, m.width, lane, kvec && (reinterpret_cast<uintptr_t>(gr) & 15) == 0);
            if (lane == 0) act[r] = g / (1.0f + expf(-g)) * d;
            continue;
        }
        if (lane == 0) { const float z = fmaxf(d, 0.f); act[r] = z * z; }
    }
}
template <typename T>
__global__ void __launch_bounds__(TK_WARPS * 32) moe_down_token_kernel(float* __restrict__ y, const float* __restrict__ act, const int* __restrict__ sel,
                                                                       const float* __restrict__ wt, const float* __restrict__ sgate, MoeDev m, StreamsIO sio) {
    extern __shared__ __align__(16) float as[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();
    const int total = m.top * m.ff + m.shared_ff;
    for (int i = threadIdx.x; i < total; i += TK_WARPS * 32) as[i] = act[i];
    __syncthreads();
    const bool kvec = m.ff % El<T>::P == 0, svec = m.shared_ff % El<T>::P == 0;
    for (int r = blockIdx.x * TK_WARPS + warp; r < m.width; r += gridDim.x * TK_WARPS) {
        float acc = 0.f;
        for (int k = 0; k < m.top; k++) {
            const unsigned char* wr = static_cast<const unsigned char*>(m.down[sel[k]]) + (size_t)r * m.ff * sizeof(T);
            acc = fmaf(wt[k], warp_dot<T>(wr, as + (size_t)k * m.ff, m.ff, lane, kvec && (reinterpret_cast<uintptr_t>(wr) & 15) == 0 && (((size_t)k * m.ff) & 3) == 0), acc);
        }
        if (m.shared_ff > 0) {
            const unsigned char* wr = static_cast<const unsigned char*>(m.shared_down) + (size_t)r * m.shared_ff * sizeof(T);
            acc = fmaf(sgate[0], warp_dot<T>(wr, as + (size_t)m.top * m.ff, m.shared_ff, lane, svec && (reinterpret_cast<uintptr_t>(wr) & 15) == 0 && (((size_t)m.top * m.ff) & 3) == 0), acc);
        }
        if (lane == 0) {
            if (!sio.X_out) y[r] = acc;
            else {                        // X[t][r] <- sum_s M[s][t] X[s][r] + b[t] * acc, all t from the old values
                float xv[16], nv[16];
#pragma unroll
                for (int s = 0; s < 16; s++) xv[s] = s < sio.S ? sio.X_out[(size_t)s * m.width + r] : 0.f;
#pragma unroll
                for (int t = 0; t < 16; t++) {
                    float a2 = 0.f;
                    if (t < sio.S) {
#pragma unroll
                        for (int s = 0; s < 16; s++) if (s < sio.S) a2 = fmaf(sio.M[s * sio.S + t], xv[s], a2);
                        a2 = fmaf(sio.b[t], acc, a2);
                    }
                    nv[t] = a2;
                }
#pragma unroll
                for (int t = 0; t < 16; t++) if (t < sio.S) sio.X_out[(size_t)t * m.width + r] = nv[t];
            }
        }
    }
}

// ---- prompt rows ----
// work = [offsets: experts + 1][row_token: n][assign_row: n], n = tokens * top.  One warp per expert; two launches (count, place).
__global__ void moe_count_kernel(int* __restrict__ work, const int* __restrict__ sel, int n, int experts) {
    pdl_launch_dependents();
    pdl_wait();
    const int e = blockIdx.x, lane = threadIdx.x;
    int c = 0;
    for (int a = lane; a < n; a += 32) c += sel[a] == e ? 1 : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xFFFFFFFFu, c, o);
    if (lane == 0) work[experts + 1 + 2 * (size_t)n + e] = c;      // counts live behind the two tables
}
constexpr int PL_WARPS = 8;
// One CTA per expert; its warps take consecutive slices of the assignments: count per slice, prefix over the slices, then an
// ordered placement inside each slice (ballot + popc), so rows of an expert stay in assignment (= token) order.
__global__ void __launch_bounds__(PL_WARPS * 32) moe_place_kernel(int* __restrict__ work, const int* __restrict__ sel, int n, int experts, int top) {
    __shared__ int slice_count[PL_WARPS];
    pdl_launch_dependents();
    pdl_wait();
    const int e = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* counts = work + experts + 1 + 2 * (size_t)n;
    int off = 0;
    for (int x = 0; x < e; x++) off += counts[x];
    int* row_token = work + experts + 1;
    int* assign_row = row_token + n;
    if (threadIdx.x == 0) { work[e] = off; if (e == experts - 1) work[experts] = off + counts[e]; }
    const int per = ((n + PL_WARPS - 1) / PL_WARPS + 31) / 32 * 32;
    const int a_begin = min(n, warp * per), a_end = min(n, a_begin + per);
    int c = 0;
    for (int a = a_begin + lane; a < a_end; a += 32) c += sel[a] == e ? 1 : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xFFFFFFFFu, c, o);
    if (lane == 0) slice_count[warp] = c;
    __syncthreads();
    int placed = off;
    for (int w = 0; w < warp; w++) placed += slice_count[w];
    for (int a0 = a_begin; a0 < a_end; a0 += 32) {
        const int a = a0 + lane;
        const bool mine = a < a_end && sel[a] == e;
        const unsigned m = __ballot_sync(0xFFFFFFFFu, mine);
        if (mine) {
            const int row = placed + __popc(m & ((1u << lane) - 1u));
            row_token[row] = a / top;
            assign_row[a] = row;
        }
        placed += __popc(m);
    }
}

constexpr int GT = 64, GK = 16;
// C[row, :] = epilogue(A[src(row), :] . W_e^T) for the rows of expert e = blockIdx.z; src(row) = a_index ? a_index[row] : row
template <typename T>
__global__ void __launch_bounds__(256) moe_rows_gemm_kernel(float* __restrict__ C, const float* __restrict__ A, const int* __restrict__ a_index,
                                                            const void* const* __restrict__ Wt, const int* __restrict__ offsets, int N, int K, int relu2) {
    __shared__ float As[GK][GT + 4];
    __shared__ float Ws[GK][GT + 4];
    __shared__ int src[GT];
    pdl_launch_dependents();
    pdl_wait();
    const int e = blockIdx.z;
    const int r_begin = offsets[e], r_end = offsets[e + 1];
    const int t0 = r_begin + blockIdx.y * GT, n0 = blockIdx.x * GT;
    if (t0 >= r_end) return;
    const unsigned char* W = static_cast<const unsigned char*>(Wt[e]);
    const size_t pitch = (size_t)K * sizeof(T);
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    if (threadIdx.x < GT) { const int r = t0 + threadIdx.x; src[threadIdx.x] = r < r_end ? (a_index ? a_index[r] : r) : -1; }
    __syncthreads();
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += GK) {
        for (int x = threadIdx.x; x < GT * GK; x += 256) {
            const int r = x / GK, k = x % GK;
            const int n = n0 + r, kk = k0 + k;
            As[k][r] = (src[r] >= 0 && kk < K) ? A[(size_t)src[r] * K + kk] : 0.f;
            Ws[k][r] = (n < N && kk < K) ? El<T>::one(W + (size_t)n * pitch, kk) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GK; k++) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) { a[i] = As[k][ty * 4 + i]; w[i] = Ws[k][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int r = t0 + ty * 4 + i;
        if (r >= r_end) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (relu2) { v = fmaxf(v, 0.f); v *= v; }
            C[(size_t)r * N + n] = v;
        }
    }
}

// rows in expert order: out[row] = h[row_token[row]]
__global__ void moe_gather_rows_kernel(float* __restrict__ out, const float* __restrict__ h, const int* __restrict__ row_token, size_t n, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t r = i / width, c = i % width;
    out[i] = h[(size_t)row_token[r] * width + c];
}
__global__ void moe_combine_kernel(float* __restrict__ y, const float* __restrict__ y_rows, const int* __restrict__ assign_row, const float* __restrict__ wt,
                                   const float* __restrict__ sgate, const float* __restrict__ shared_y, size_t n, int top, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t t = i / width, c = i % width;
    float acc = 0.f;
    for (int k = 0; k < top; k++) acc = fmaf(wt[t * top + k], y_rows[(size_t)assign_row[t * top + k] * width + c], acc);
    if (shared_y) acc = fmaf(sgate[t], shared_y[i], acc);
    y[i] = acc;
}
__global__ void relu2_kernel(float* __restrict__ x, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) { const float z = fmaxf(x[i], 0.f); x[i] = z * z; }
}

MoeDev dev_of(const MoeWeights& w) { return MoeDev{w.gate, w.up, w.down, w.shared_up, w.shared_down, w.top, w.ff, w.width, w.shared_up ? w.shared_ff : 0}; }

}  // namespace

void moe_route(int* sel, float* wt, float* sgate, const float* h, const MoeWeights& w, int tokens, cudaStream_t s, const StreamsIO* sio_p,
               const float* norm_w, float eps, float* h_out) {
    const StreamsIO sio = sio_p ? *sio_p : StreamsIO();
    NT_CHECK(w.experts >= 1 && w.experts <= MAX_EXPERTS && w.top >= 1 && w.top <= w.experts, "moe_route: 1 <= top <= experts <= 256");
    NT_CHECK(w.groups == 0 || (w.sigmoid && w.experts % w.groups == 0 && w.keep >= 1 && w.keep <= w.groups && w.keep * (w.experts / w.groups) >= w.top),
             "moe_route: expert groups must be equal runs whose kept part holds at least top experts");
    if (tokens <= 0) return;
    const size_t smem = (size_t)w.width * sizeof(float);
    NT_CHECK(smem <= 160 * 1024, "moe_route: the activation row does not fit in shared memory");
    static unsigned long long done = 0;
    if (smem > 40 * 1024) opt_in_dynamic_smem(moe_route_kernel, 160 * 1024, done);
    launch_k(moe_route_kernel, dim3(tokens), dim3(RT_WARPS * 32), smem, s, sel, wt, sgate, h, w.router, w.shared_gate, w.experts, w.top, w.width,
             w.sigmoid ? 1 : 0, w.correction, w.groups, w.keep, sio, norm_w, eps, h_out);
    count_launch();
}

#define NT_MOE_DT(CALL) \
    if (w.dtype == DType::F32) { CALL(float) } else if (w.dtype == DType::F16) { CALL(__half) } else if (w.dtype == DType::BF16) { CALL(__nv_bfloat16) } \
    else NT_CHECK(false, "moe: dense expert dtypes only");

void moe_expert_up_token(float* act, const float* h, const int* sel, const MoeWeights& w, cudaStream_t s) {
    const MoeDev m = dev_of(w);
    const int total = m.top * m.ff + m.shared_ff;
    const size_t smem = (size_t)w.width * sizeof(float);
    NT_CHECK(smem <= 200 * 1024, "moe: the activation row does not fit in shared memory");
    const int grid = std::min((total + TK_WARPS - 1) / TK_WARPS, 148 * 8);
#define NT_CALL(TY) { static unsigned long long done = 0; if (smem > 48 * 1024) opt_in_dynamic_smem(moe_up_token_kernel<TY>, 200 * 1024, done); \
                      launch_k(moe_up_token_kernel<TY>, dim3(grid), dim3(TK_WARPS * 32), smem, s, act, h, sel, m); }
    NT_MOE_DT(NT_CALL)
#undef NT_CALL
    count_launch();
}

void moe_expert_down_token(float* y, const float* act, const int* sel, const float* wt, const float* sgate, const float* /*shared_y*/,
                           const MoeWeights& w, cudaStream_t s, const StreamsIO* sio_p) {
    const MoeDev m = dev_of(w);
    const StreamsIO sio = sio_p ? *sio_p : StreamsIO();
    const size_t smem = (size_t)(m.top * m.ff + m.shared_ff) * sizeof(float);
    NT_CHECK(smem <= 200 * 1024, "moe: the chosen experts' activations do not fit in shared memory");
    const int grid = std::min((w.width + TK_WARPS - 1) / TK_WARPS, 148 * 8);
#define NT_CALL(TY) { static unsigned long long done = 0; if (smem > 48 * 1024) opt_in_dynamic_smem(moe_down_token_kernel<TY>, 200 * 1024, done); \
                      launch_k(moe_down_token_kernel<TY>, dim3(grid), dim3(TK_WARPS * 32), smem, s, y, act, sel, wt, sgate, m, sio); }
    NT_MOE_DT(NT_CALL)
#undef NT_CALL
    count_launch();
}

size_t moe_work_ints(int tokens, int experts, int top) { return (size_t)experts + 1 + 2 * (size_t)tokens * top + (size_t)experts; }

void moe_group(int* work, const int* sel, int tokens, int experts, int top, cudaStream_t s) {
    if (tokens <= 0) return;
    launch_k(moe_count_kernel, dim3(experts), dim3(32), 0, s, work, sel, tokens * top, experts);
    launch_k(moe_place_kernel, dim3(experts), dim3(PL_WARPS * 32), 0, s, work, sel, tokens * top, experts, top);
    count_launch(2);
}

void moe_expert_up_rows(float* act_rows, const float* h, const int* work, const MoeWeights& w, int tokens, cudaStream_t s) {
    if (tokens <= 0) return;
    const dim3 grid((w.ff + GT - 1) / GT, (tokens + GT - 1) / GT, w.experts);
    const int relu2 = w.gate ? 0 : 1;
#define NT_CALL(TY) launch_k(moe_rows_gemm_kernel<TY>, grid, dim3(256), 0, s, act_rows, h, work + w.experts + 1, w.up, work, w.ff, w.width, relu2);
    NT_MOE_DT(NT_CALL)
#undef NT_CALL
    count_launch();
}
void moe_expert_gate_rows(float* gate_rows, const float* h, const int* work, const MoeWeights& w, int tokens, cudaStream_t s) {
    if (tokens <= 0) return;
    NT_CHECK(w.gate != nullptr, "moe_expert_gate_rows: the experts have no gate matrices");
    const dim3 grid((w.ff + GT - 1) / GT, (tokens + GT - 1) / GT, w.experts);
#define NT_CALL(TY) launch_k(moe_rows_gemm_kernel<TY>, grid, dim3(256), 0, s, gate_rows, h, work + w.experts + 1, w.gate, work, w.ff, w.width, 0);
    NT_MOE_DT(NT_CALL)
#undef NT_CALL
    count_launch();
}
void moe_expert_down_rows(float* y_rows, const float* act_rows, const int* work, const MoeWeights& w, int tokens, cudaStream_t s) {
    if (tokens <= 0) return;
    const dim3 grid((w.width + GT - 1) / GT, (tokens + GT - 1) / GT, w.experts);
#define NT_CALL(TY) launch_k(moe_rows_gemm_kernel<TY>, grid, dim3(256), 0, s, y_rows, act_rows, (const int*)nullptr, w.down, work, w.width, w.ff, 0);
    NT_MOE_DT(NT_CALL)
#undef NT_CALL
    count_launch();
}
void moe_combine(float* y, const float* y_rows, const int* work, const float* wt, const float* sgate, const float* shared_y, int tokens,
                 int experts, int top, int width, cudaStream_t s) {
    const size_t n = (size_t)tokens * width;
    if (!n) return;
    launch_k(moe_combine_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, y, y_rows, work + experts + 1 + (size_t)tokens * top, wt, sgate,
             shared_y, n, top, width);
    count_launch();
}
void moe_gather_rows(float* out, const float* h, const int* work, int tokens, int experts, int top, int width, cudaStream_t s) {
    const size_t n = (size_t)tokens * top * width;
    if (!n) return;
    launch_k(moe_gather_rows_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, out, h, work + experts + 1, n, width);
    count_launch();
}
void relu2(float* x, size_t n, cudaStream_t s) {
    if (!n) return;
    launch_k(relu2_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, x, n);
    count_launch();
}

}}  // namespace nt::b200
