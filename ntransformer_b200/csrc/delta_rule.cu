// delta_rule.cu — the gated delta-rule mixer around its projections and convolutions (engine/layer_spec.h DeltaSpec).  Per value head h,
// reading query / key head g = h / (heads / kv_heads), with a matrix state S [dim, vdim] in F32:
//       S <- diag(a_t) S;   u_t = beta_t (v_t - S^T k_t);   S <- S + k_t u_t^T;   o_t = S^T q_t        (in this order)
//   delta_prep        q, k [T, kv_heads, dim] scaled to unit length per head (x / sqrt(sum x^2 + 1e-6); q also by dim^-1/2), in place;
//                     a = exp(-exp(A_log_h) softplus(raw + dt_bias)) per (head, key channel), in place on raw [T, heads * dim];
//                     beta = sigmoid(raw) in place [T, heads];  qk [T, kv_heads] = <q, k> of the scaled vectors
//   delta_rule_rows   the recurrence.  Every column j of S (the dim numbers that produce value channel j) evolves on its own:
//                         s <- a * s;  d1 = <k, s>;  d2 = <q, s>;  u = beta (v_j - d1);  s <- s + k u;  o_j = d2 + <q, k> u,
//                     so one reduction per token serves both the correction and the read-out.  LN lanes share a column (dim / LN state
//                     numbers each, in registers; LN is 2 to 16: the reduction over them is on the dependent chain); a CTA owns its
//                     threads / LN columns of one head and walks the step's rows in tiles of 16 staged through shared memory by cp.async
//                     into two buffers (q, k, a of the head, v and beta of its columns).  The state [heads, vdim, dim] is read at the
//                     start (zeros when the step starts at position 0) and written back at the end, so a prompt cut anywhere — and a
//                     decoded token, T = 1 — continues exactly.
//   delta_gate_norm   out = o / sqrt(mean_v(o^2) + eps) * gain[v] * sigmoid(gate_raw), per head
// A step's base position is *pos_dev when given (the captured decode step), else p0.  Everything is F32; compiled WITHOUT
// --use_fast_math (expf / log1pf / division at full precision).
#include "kernels_internal.h"
#include "ring.cuh"
#include <algorithm>
#include <cstdint>

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

constexpr int DR_TILE = 16;      // rows staged per tile

__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// grid (ceil(vdim / (THREADS / LN)), heads).  Lane l of a column holds state elements l + LN * e, e < NPT.  Two tile buffers: the next
// tile's rows arrive (cp.async) while the current one is walked.
template <int LN, int NPT, int THREADS>
__global__ void __launch_bounds__(THREADS) delta_rule_rows_kernel(float* __restrict__ out, const float* __restrict__ q, const float* __restrict__ k,
                                                                 const float* __restrict__ v, const float* __restrict__ a, const float* __restrict__ beta,
                                                                 const float* __restrict__ qk, float* __restrict__ state, int T, int heads, int kv_heads,
                                                                 int dim, int vdim, const int* __restrict__ pos_dev, int p0) {
    constexpr int COLS = THREADS / LN;
    extern __shared__ __align__(16) float sm[];
    const int tile_floats = 3 * DR_TILE * dim + DR_TILE * COLS + 2 * DR_TILE;     // q | k | a [DR_TILE][dim], v [DR_TILE][COLS], beta, <q, k> [DR_TILE]
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
    auto load_tile = [&](int t0, int buf) {
        float* sq = sm + (size_t)buf * tile_floats;
        float* sk = sq + DR_TILE * dim;
        float* sa = sk + DR_TILE * dim;
        float* sv = sa + DR_TILE * dim;
        float* sb = sv + DR_TILE * COLS;
        const int nt = min(DR_TILE, T - t0);
        for (int i = threadIdx.x; i < nt * dim; i += THREADS) {
            const int tt = i / dim, d = i % dim;
            const size_t t = (size_t)(t0 + tt);
            cp_async4(sq + i, q + (t * kv_heads + g) * dim + d);
            cp_async4(sk + i, k + (t * kv_heads + g) * dim + d);
            cp_async4(sa + i, a + (t * heads + h) * dim + d);
        }
        for (int i = threadIdx.x; i < nt * COLS; i += THREADS) {
            const int tt = i / COLS, c = blockIdx.x * COLS + i % COLS;
            if (c < vdim) cp_async4(sv + i, v + ((size_t)(t0 + tt) * heads + h) * vdim + c);
            else sv[i] = 0.f;
        }
        for (int i = threadIdx.x; i < nt; i += THREADS) {
            cp_async4(sb + i, beta + (size_t)(t0 + i) * heads + h);
            cp_async4(sb + DR_TILE + i, qk + (size_t)(t0 + i) * kv_heads + g);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int n_tiles = (T + DR_TILE - 1) / DR_TILE;
    load_tile(0, 0);
    for (int j = 0; j < n_tiles; j++) {
        const int t0 = j * DR_TILE, nt = min(DR_TILE, T - t0), buf = j & 1;
        if (j + 1 < n_tiles) {
            load_tile(t0 + DR_TILE, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const float* sq = sm + (size_t)buf * tile_floats;
        const float* sk = sq + DR_TILE * dim;
        const float* sa = sk + DR_TILE * dim;
        const float* sv = sa + DR_TILE * dim;
        const float* sb = sv + DR_TILE * COLS;
        for (int tt = 0; tt < nt; tt++) {
            const float* kq = sk + tt * dim;
            const float* qq = sq + tt * dim;
            const float* aa = sa + tt * dim;
            // two partial sums per dot product: half the dependent chain
            float d1a = 0.f, d1b = 0.f, d2a = 0.f, d2b = 0.f;
#pragma unroll
            for (int e = 0; e < NPT; e++) {
                const int d = l + LN * e;
                if (d < dim) {
                    S[e] *= aa[d];
                    if (e & 1) { d1b = fmaf(kq[d], S[e], d1b); d2b = fmaf(qq[d], S[e], d2b); }
                    else { d1a = fmaf(kq[d], S[e], d1a); d2a = fmaf(qq[d], S[e], d2a); }
                }
            }
            float d1 = d1a + d1b, d2 = d2a + d2b;
#pragma unroll
            for (int o = LN / 2; o > 0; o >>= 1) { d1 += __shfl_xor_sync(0xFFFFFFFFu, d1, o); d2 += __shfl_xor_sync(0xFFFFFFFFu, d2, o); }
            const float u = sb[tt] * (sv[tt * COLS + col_l] - d1);
#pragma unroll
            for (int e = 0; e < NPT; e++) { const int d = l + LN * e; if (d < dim) S[e] = fmaf(kq[d], u, S[e]); }
            if (l == 0 && live) out[((size_t)(t0 + tt) * heads + h) * vdim + col] = fmaf(sb[DR_TILE + tt], u, d2);
        }
        __syncthreads();                       // the buffer is refilled by the load of tile j + 2
    }
    if (live) {
#pragma unroll
        for (int e = 0; e < NPT; e++) { const int d = l + LN * e; if (d < dim) st[d] = S[e]; }
    }
}

// The same recurrence for key widths that are a multiple of 4: lane l of a column holds CH chunks of 4 consecutive state numbers
// (chunk c at d = 4 (c LN + l)), so q, k, a come from shared memory as 16-byte loads and the per-row instruction count drops to a
// third; LN is chosen as wide as the head allows (dim / 4 lanes), which keeps more warps in flight — the kernel issues one instruction
// every three to four cycles per warp, so warps per scheduler, not work per lane, set its speed.
template <int LN, int CH>
__global__ void __launch_bounds__(128) delta_rule_rows_vec_kernel(float* __restrict__ out, const float* __restrict__ q, const float* __restrict__ k,
                                                                 const float* __restrict__ v, const float* __restrict__ a, const float* __restrict__ beta,
                                                                 const float* __restrict__ qk, float* __restrict__ state, int T, int heads, int kv_heads,
                                                                 int dim, int vdim, const int* __restrict__ pos_dev, int p0) {
    constexpr int THREADS = 128, COLS = THREADS / LN;
    extern __shared__ __align__(16) float sm[];
    const int tile_floats = 3 * DR_TILE * dim + DR_TILE * COLS + 2 * DR_TILE;
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.y, g = h / (heads / kv_heads);
    const int col_l = threadIdx.x / LN, l = threadIdx.x % LN;
    const int col = blockIdx.x * COLS + col_l;
    const bool live = col < vdim;
    const bool fresh = (pos_dev ? *pos_dev : p0) == 0;
    float* st = state + ((size_t)h * vdim + (live ? col : 0)) * dim;
    int d0[CH];
    bool on[CH];
    float4 S[CH];
#pragma unroll
    for (int c = 0; c < CH; c++) {
        d0[c] = 4 * (c * LN + l);
        on[c] = d0[c] < dim;
        S[c] = (on[c] && live && !fresh) ? *reinterpret_cast<const float4*>(st + d0[c]) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (!on[c]) d0[c] = 0;                  // an idle chunk reads a valid address and keeps zeros
    }
    auto load_tile = [&](int t0, int buf) {
        float* sq = sm + (size_t)buf * tile_floats;
        float* sk = sq + DR_TILE * dim;
        float* sa = sk + DR_TILE * dim;
        float* sv = sa + DR_TILE * dim;
        float* sb = sv + DR_TILE * COLS;
        const int nt = min(DR_TILE, T - t0), d4 = dim / 4;
        for (int i = threadIdx.x; i < nt * d4; i += THREADS) {
            const int tt = i / d4, d = (i % d4) * 4;
            const size_t t = (size_t)(t0 + tt);
            cp_async16(sq + tt * dim + d, q + (t * kv_heads + g) * dim + d);
            cp_async16(sk + tt * dim + d, k + (t * kv_heads + g) * dim + d);
            cp_async16(sa + tt * dim + d, a + (t * heads + h) * dim + d);
        }
        for (int i = threadIdx.x; i < nt * COLS; i += THREADS) {
            const int tt = i / COLS, c = blockIdx.x * COLS + i % COLS;
            if (c < vdim) cp_async4(sv + i, v + ((size_t)(t0 + tt) * heads + h) * vdim + c);
            else sv[i] = 0.f;
        }
        for (int i = threadIdx.x; i < nt; i += THREADS) {
            cp_async4(sb + i, beta + (size_t)(t0 + i) * heads + h);
            cp_async4(sb + DR_TILE + i, qk + (size_t)(t0 + i) * kv_heads + g);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int n_tiles = (T + DR_TILE - 1) / DR_TILE;
    load_tile(0, 0);
    for (int j = 0; j < n_tiles; j++) {
        const int t0 = j * DR_TILE, nt = min(DR_TILE, T - t0), buf = j & 1;
        if (j + 1 < n_tiles) {
            load_tile(t0 + DR_TILE, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const float* sq = sm + (size_t)buf * tile_floats;
        const float* sk = sq + DR_TILE * dim;
        const float* sa = sk + DR_TILE * dim;
        const float* sv = sa + DR_TILE * dim;
        const float* sb = sv + DR_TILE * COLS;
#pragma unroll 4
        for (int tt = 0; tt < nt; tt++) {
            float4 kk[CH];
            float d1 = 0.f, d2 = 0.f;
#pragma unroll
            for (int c = 0; c < CH; c++) {
                const float4 aa = *reinterpret_cast<const float4*>(sa + tt * dim + d0[c]);
                const float4 qq = *reinterpret_cast<const float4*>(sq + tt * dim + d0[c]);
                kk[c] = *reinterpret_cast<const float4*>(sk + tt * dim + d0[c]);
                S[c].x *= aa.x; S[c].y *= aa.y; S[c].z *= aa.z; S[c].w *= aa.w;
                d1 = fmaf(kk[c].x, S[c].x, d1); d2 = fmaf(qq.x, S[c].x, d2);
                d1 = fmaf(kk[c].y, S[c].y, d1); d2 = fmaf(qq.y, S[c].y, d2);
                d1 = fmaf(kk[c].z, S[c].z, d1); d2 = fmaf(qq.z, S[c].z, d2);
                d1 = fmaf(kk[c].w, S[c].w, d1); d2 = fmaf(qq.w, S[c].w, d2);
            }
#pragma unroll
            for (int o = LN / 2; o > 0; o >>= 1) { d1 += __shfl_xor_sync(0xFFFFFFFFu, d1, o); d2 += __shfl_xor_sync(0xFFFFFFFFu, d2, o); }
            const float u = sb[tt] * (sv[tt * COLS + col_l] - d1);
#pragma unroll
            for (int c = 0; c < CH; c++) {
                if (on[c]) { S[c].x = fmaf(kk[c].x, u, S[c].x); S[c].y = fmaf(kk[c].y, u, S[c].y); S[c].z = fmaf(kk[c].z, u, S[c].z); S[c].w = fmaf(kk[c].w, u, S[c].w); }
            }
            if (l == 0 && live) out[((size_t)(t0 + tt) * heads + h) * vdim + col] = fmaf(sb[DR_TILE + tt], u, d2);
        }
        __syncthreads();
    }
    if (live) {
#pragma unroll
        for (int c = 0; c < CH; c++) if (on[c]) *reinterpret_cast<float4*>(st + 4 * (c * LN + l)) = S[c];
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

template <int LN, int NPT, int THREADS>
void launch_rows(float* out, const float* q, const float* k, const float* v, const float* a, const float* beta, const float* qk, float* state, int T, int heads,
                 int kv_heads, int dim, int vdim, const int* pos_dev, int p0, cudaStream_t s) {
    constexpr int COLS = THREADS / LN;
    const size_t smem = sizeof(float) * 2 * ((size_t)3 * DR_TILE * dim + (size_t)DR_TILE * COLS + 2 * DR_TILE);
    static unsigned long long done = 0;
    if (smem > 48 * 1024) opt_in_dynamic_smem(delta_rule_rows_kernel<LN, NPT, THREADS>, (int)smem, done);
    launch_k(delta_rule_rows_kernel<LN, NPT, THREADS>, dim3((vdim + COLS - 1) / COLS, heads), dim3(THREADS), smem, s, out, q, k, v, a, beta, qk, state, T, heads,
             kv_heads, dim, vdim, pos_dev, p0);
}

template <int LN, int CH>
void launch_rows_vec(float* out, const float* q, const float* k, const float* v, const float* a, const float* beta, const float* qk, float* state, int T, int heads,
                     int kv_heads, int dim, int vdim, const int* pos_dev, int p0, cudaStream_t s) {
    constexpr int COLS = 128 / LN;
    const size_t smem = sizeof(float) * 2 * ((size_t)3 * DR_TILE * dim + (size_t)DR_TILE * COLS + 2 * DR_TILE);
    static unsigned long long done = 0;
    if (smem > 48 * 1024) opt_in_dynamic_smem(delta_rule_rows_vec_kernel<LN, CH>, (int)smem, done);
    launch_k(delta_rule_rows_vec_kernel<LN, CH>, dim3((vdim + COLS - 1) / COLS, heads), dim3(128), smem, s, out, q, k, v, a, beta, qk, state, T, heads, kv_heads, dim,
             vdim, pos_dev, p0);
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
    const bool aligned = dim % 4 == 0 && ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(a) |
                                           reinterpret_cast<uintptr_t>(state)) & 15) == 0;
    if (aligned) {                  // 16-byte rows: the vector form, dim / 4 lanes per column
#define NT_DV(LN, CH) launch_rows_vec<LN, CH>(out, q, k, v, a, beta, qk, state, T, heads, kv_heads, dim, vdim, pos_dev, p0, s)
        // lanes per column: as many as the head allows while the grid stays within about four warps per scheduler (the reduction over
        // the lanes costs instructions; beyond that the kernel is bound by issue slots, not by latency), else half as many with two chunks each
        const auto crowded = [&](int ln) { return (long)heads * vdim * ln / 32 > 4L * 4 * 148; };
        if (dim <= 8) NT_DV(2, 1);
        else if (dim <= 16) NT_DV(4, 1);
        else if (dim <= 32) { if (crowded(8)) NT_DV(4, 2); else NT_DV(8, 1); }
        else if (dim <= 64) { if (crowded(16)) NT_DV(8, 2); else NT_DV(16, 1); }
        else if (dim <= 128) { if (crowded(32)) NT_DV(16, 2); else NT_DV(32, 1); }
        else NT_DV(32, 2);
#undef NT_DV
        count_launch();
        return;
    }
    // few lanes per column keep the per-row reduction short (it sits on the recurrence's dependent chain); CTAs of 64 threads when
    // CTAs of 128 would leave most SMs without one
#define NT_DR(LN, NPT) do { if ((long)((vdim + 128 / LN - 1) / (128 / LN)) * heads >= 148) launch_rows<LN, NPT, 128>(out, q, k, v, a, beta, qk, state, T, heads, kv_heads, dim, vdim, pos_dev, p0, s); \
                            else launch_rows<LN, NPT, 64>(out, q, k, v, a, beta, qk, state, T, heads, kv_heads, dim, vdim, pos_dev, p0, s); } while (0)
    if (dim <= 16) NT_DR(2, 8);
    else if (dim <= 32) NT_DR(4, 8);
    else if (dim <= 64) NT_DR(4, 16);
    else if (dim <= 128) NT_DR(8, 16);
    else NT_DR(16, 16);
#undef NT_DR
    count_launch();
}

void delta_gate_norm(float* out, const float* o, const float* gate_raw, const float* gain, float eps, int T, int heads, int vdim, cudaStream_t s) {
    if (T <= 0) return;
    launch_k(delta_gate_norm_kernel, dim3(T, heads), dim3(128), 0, s, out, o, gate_raw, gain, eps, heads, vdim);
    count_launch();
}

}}  // namespace nt::b200
