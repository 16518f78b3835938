// delta_rule.cu — the gated delta-rule mixer around its projections and convolutions (engine/layer_spec.h DeltaSpec).  Per value head h,
// reading query / key head g = h / (heads / kv_heads), with a matrix state S [dim, vdim] in F32:
//       S <- diag(a_t) S;   u_t = beta_t (v_t - S^T k_t);   S <- S + k_t u_t^T;   o_t = S^T q_t        (in this order)
//   delta_prep        q, k [T, kv_heads, dim] scaled to unit length per head (x / sqrt(sum x^2 + 1e-6); q also by dim^-1/2), in place;
//                     a = exp(-exp(A_log_h) softplus(raw + dt_bias)) per (head, key channel), in place on raw [T, heads * dim];
//                     beta = sigmoid(raw) in place [T, heads];  qk [T, kv_heads] = <q, k> of the scaled vectors
//   delta_rule_rows   the recurrence.  Every column j of S (the dim numbers that produce value channel j) evolves on its own:
//                         s <- a * s;  d1 = <k, s>;  d2 = <q, s>;  u = beta (v_j - d1);  s <- s + k u;  o_j = d2 + <q, k> u,
//                     so one reduction per token serves both the correction and the read-out.  LN lanes share a column (dim / LN state
//                     numbers each, in registers); a CTA owns 128 / LN columns of one head and walks the step's rows in tiles staged
//                     through shared memory (q, k, a of the head, v and beta of its columns).  The state [heads, vdim, dim] is read at the
//                     start (zeros when the step starts at position 0) and written back at the end, so a prompt cut anywhere — and a
//                     decoded token, T = 1 — continues exactly.
//   delta_gate_norm   out = o / sqrt(mean_v(o^2) + eps) * gain[v] * sigmoid(gate_raw), per head
// A step's base position is *pos_dev when given (the captured decode step), else p0.  Everything is F32; compiled WITHOUT
// --use_fast_math (expf / log1pf / division at full precision).
#include "kernels_internal.h"
#include "ring.cuh"
#include <algorithm>

namespace nt { namespace b200 {

namespace {

__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }

// grid (T), 256 threads
__global__ void __launch_bounds__(256) delta_prep_kernel(float* __restrict__ q, float* __restrict__ k, float* __restrict__ a, float* __restrict__ beta,
                                                         float* __restrict__ qk, const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                                                         int heads, int kv_heads, int dim) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float qs = 1.0f / sqrtf((float)dim);
    for (int g = warp; g < kv_heads; g += 8) {
        float* qr = q + (t * kv_heads + g) * dim;
        float* kr = k + (t * kv_heads + g) * dim;
        float sq = 0.f, sk = 0.f;
        for (int i = lane; i < dim; i += 32) { sq = fmaf(qr[i], qr[i], sq); sk = fmaf(kr[i], kr[i], sk); }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) { sq += __shfl_xor_sync(0xFFFFFFFFu, sq, o); sk += __shfl_xor_sync(0xFFFFFFFFu, sk, o); }
        const float iq = qs / sqrtf(sq + 1e-6f), ik = 1.0f / sqrtf(sk + 1e-6f);
        float d = 0.f;
        for (int i = lane; i < dim; i += 32) {
            const float x = qr[i] * iq, y = kr[i] * ik;
            qr[i] = x; kr[i] = y;
            d = fmaf(x, y, d);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xFFFFFFFFu, d, o);
        if (lane == 0) qk[t * kv_heads + g] = d;
    }
    const int n = heads * dim;
    for (int i = threadIdx.x; i < n; i += 256) {
        const float rate = expf(A_log[i / dim]);
        a[t * n + i] = expf(-rate * softplus_f(a[t * n + i] + dt_bias[i]));
    }
    for (int h = threadIdx.x; h < heads; h += 256) beta[t * heads + h] = sigmoid_f(beta[t * heads + h]);
}

constexpr int DR_THREADS = 128;
constexpr int DR_TILE = 16;      // rows staged per tile

// grid (ceil(vdim / (128 / LN)), heads).  Lane l of a column holds state elements l + LN * e, e < NPT.
template <int LN, int NPT>
__global__ void __launch_bounds__(DR_THREADS) delta_rule_rows_kernel(float* __restrict__ out, const float* __restrict__ q, const float* __restrict__ k,
                                                                    const float* __restrict__ v, const float* __restrict__ a, const float* __restrict__ beta,
                                                                    const float* __restrict__ qk, float* __restrict__ state, int T, int heads, int kv_heads,
                                                                    int dim, int vdim, const int* __restrict__ pos_dev, int p0) {
    constexpr int COLS = DR_THREADS / LN;
    extern __shared__ __align__(16) float sm[];
    float* sq = sm;                           // [DR_TILE][dim]
    float* sk = sq + DR_TILE * dim;
    float* sa = sk + DR_TILE * dim;
    float* sv = sa + DR_TILE * dim;           // [DR_TILE][COLS]
    float* sb = sv + DR_TILE * COLS;          // [DR_TILE] beta, [DR_TILE] <q, k>
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.y, g = h / (heads / kv_heads);
    const int col_l = threadIdx.x / LN, l = threadIdx.x % LN;
    const int col = blockIdx.x * COLS + col_l;
    const bool live = col < vdim;
    const bool fresh = (pos_dev ? *pos_dev : p0) == 0;
    float* st = state + ((size_t)h * vdim + (live ? col : 0)) * dim;
    float S[NPT];
#pragma unroll
    for (int e = 0; e < NPT; e++) { const int d = l + LN * e; S[e] = (live && !fresh && d < dim) ? st[d] : 0.f; }
    for (int t0 = 0; t0 < T; t0 += DR_TILE) {
        const int nt = min(DR_TILE, T - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < nt * dim; i += DR_THREADS) {
            const int tt = i / dim, d = i % dim;
            const size_t t = (size_t)(t0 + tt);
            sq[i] = q[(t * kv_heads + g) * dim + d];
            sk[i] = k[(t * kv_heads + g) * dim + d];
            sa[i] = a[(t * heads + h) * dim + d];
        }
        for (int i = threadIdx.x; i < nt * COLS; i += DR_THREADS) {
            const int tt = i / COLS, c = blockIdx.x * COLS + i % COLS;
            sv[i] = c < vdim ? v[((size_t)(t0 + tt) * heads + h) * vdim + c] : 0.f;
        }
        for (int i = threadIdx.x; i < nt; i += DR_THREADS) {
            sb[i] = beta[(size_t)(t0 + i) * heads + h];
            sb[DR_TILE + i] = qk[(size_t)(t0 + i) * kv_heads + g];
        }
        __syncthreads();
        for (int tt = 0; tt < nt; tt++) {
            const float* kq = sk + tt * dim;
            const float* qq = sq + tt * dim;
            const float* aa = sa + tt * dim;
            float d1 = 0.f, d2 = 0.f;
#pragma unroll
            for (int e = 0; e < NPT; e++) {
                const int d = l + LN * e;
                if (d < dim) {
                    S[e] *= aa[d];
                    d1 = fmaf(kq[d], S[e], d1);
                    d2 = fmaf(qq[d], S[e], d2);
                }
            }
#pragma unroll
            for (int o = LN / 2; o > 0; o >>= 1) { d1 += __shfl_xor_sync(0xFFFFFFFFu, d1, o); d2 += __shfl_xor_sync(0xFFFFFFFFu, d2, o); }
            const float u = sb[tt] * (sv[tt * COLS + col_l] - d1);
#pragma unroll
            for (int e = 0; e < NPT; e++) { const int d = l + LN * e; if (d < dim) S[e] = fmaf(kq[d], u, S[e]); }
            if (l == 0 && live) out[((size_t)(t0 + tt) * heads + h) * vdim + col] = fmaf(sb[DR_TILE + tt], u, d2);
        }
    }
    if (live) {
#pragma unroll
        for (int e = 0; e < NPT; e++) { const int d = l + LN * e; if (d < dim) st[d] = S[e]; }
    }
}

// grid (T, heads), 128 threads
__global__ void __launch_bounds__(128) delta_gate_norm_kernel(float* __restrict__ out, const float* __restrict__ o, const float* __restrict__ gate_raw,
                                                              const float* __restrict__ gain, float eps, int heads, int vdim) {
    __shared__ float red[4];
    pdl_launch_dependents();
    pdl_wait();
    const size_t base = ((size_t)blockIdx.x * heads + blockIdx.y) * vdim;
    float ss = 0.f;
    for (int i = threadIdx.x; i < vdim; i += 128) ss = fmaf(o[base + i], o[base + i], ss);
#pragma unroll
    for (int w = 16; w > 0; w >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, w);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    const float inv = 1.0f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)vdim + eps);
    for (int i = threadIdx.x; i < vdim; i += 128) out[base + i] = o[base + i] * inv * gain[i] * sigmoid_f(gate_raw[base + i]);
}

template <int LN, int NPT>
void launch_rows(float* out, const float* q, const float* k, const float* v, const float* a, const float* beta, const float* qk, float* state, int T, int heads,
                 int kv_heads, int dim, int vdim, const int* pos_dev, int p0, cudaStream_t s) {
    constexpr int COLS = DR_THREADS / LN;
    const size_t smem = sizeof(float) * ((size_t)3 * DR_TILE * dim + (size_t)DR_TILE * COLS + 2 * DR_TILE);
    static unsigned long long done = 0;
    if (smem > 48 * 1024) opt_in_dynamic_smem(delta_rule_rows_kernel<LN, NPT>, (int)smem, done);
    launch_k(delta_rule_rows_kernel<LN, NPT>, dim3((vdim + COLS - 1) / COLS, heads), dim3(DR_THREADS), smem, s, out, q, k, v, a, beta, qk, state, T, heads,
             kv_heads, dim, vdim, pos_dev, p0);
}

}  // namespace

void delta_prep(float* q, float* k, float* a, float* beta, float* qk, const float* dt_bias, const float* A_log, int T, int heads, int kv_heads, int dim,
                cudaStream_t s) {
    if (T <= 0) return;
    launch_k(delta_prep_kernel, dim3(T), dim3(256), 0, s, q, k, a, beta, qk, dt_bias, A_log, heads, kv_heads, dim);
    count_launch();
}

void delta_rule_rows(float* out, const float* q, const float* k, const float* v, const float* a, const float* beta, const float* qk, float* state, int T,
                     int heads, int kv_heads, int dim, int vdim, const int* pos_dev, int p0, cudaStream_t s) {
    NT_CHECK(dim >= 1 && dim <= DELTA_MAX_DIM, "delta_rule_rows: key heads wider than 256 are not covered");
    NT_CHECK(kv_heads > 0 && heads % kv_heads == 0, "delta_rule_rows: heads must be a multiple of kv_heads");
    if (T <= 0) return;
#define NT_DR(LN, NPT) launch_rows<LN, NPT>(out, q, k, v, a, beta, qk, state, T, heads, kv_heads, dim, vdim, pos_dev, p0, s)
    if (dim <= 16) NT_DR(4, 4);
    else if (dim <= 32) NT_DR(8, 4);
    else if (dim <= 64) NT_DR(16, 4);
    else if (dim <= 128) NT_DR(32, 4);
    else NT_DR(32, 8);
#undef NT_DR
    count_launch();
}

void delta_gate_norm(float* out, const float* o, const float* gate_raw, const float* gain, float eps, int T, int heads, int vdim, cudaStream_t s) {
    if (T <= 0) return;
    launch_k(delta_gate_norm_kernel, dim3(T, heads), dim3(128), 0, s, out, o, gate_raw, gain, eps, heads, vdim);
    count_launch();
}

}}  // namespace nt::b200
