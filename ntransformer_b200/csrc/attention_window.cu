// attention_window.cu — attention over a sliding window plus the sequence's first `keep` tokens, scores soft-capped, no positional
// rotation:   s_ij = cap * tanh(scale * <q_i, k_j> / cap)   (cap == 0: s_ij = scale * <q_i, k_j>),
//             j visible from i  <=>  j <= i  and  (i - j < window  or  j < keep)        (window == 0: every j <= i),
//             out_i = sum_j softmax_j(s_ij) v_j.
// Query/key heads are `dim` wide, value heads `vdim` wide (they may differ); query head h reads key/value head h / (heads / kv_heads).
// Keys and values come from the per-layer cache ([max_seq, kv_heads * dim] and [max_seq, kv_heads * vdim], F32 or BF16 storage):
// the caller writes the step's rows first (qk_norm_kv_write), so a prompt portion, a whole prompt and a decoded token all take the
// same kernel and see the same stored values.  Softmax, score and the weighted sum are F32.
//   one CTA per (query token, head); its warps stride over the visible keys (the kept prefix, then the window) in groups of 32
//   with a running (max, sum, acc) each, merged through shared memory at the end; for a single decoded token the keys of a head
//   are further split over the CTAs of a thread-block cluster and merged through the leader's distributed shared memory.  Prompts over a BF16 cache with equal key and
//   value width go to the tiled tensor-core form in attention_prefill_mma.cu instead.
// WindowAttn::sink adds exp(sink_h) to head h's denominator (a learned term without key or value); WindowAttn::joint_v makes every query
// head sum one value row per key that spans all value heads, which attention_heads.cu's talk_mix turns into head-mixed softmax weights.
// Compiled WITHOUT --use_fast_math (tanhf / expf at full precision).
#include "kernels_internal.h"
#include "ring.cuh"
#include <cuda_bf16.h>
#include <cooperative_groups.h>
#include <cfloat>
#include <cstdlib>
#include <algorithm>

namespace nt { namespace b200 {

namespace {

constexpr int AW_WARPS = 8;
constexpr int AW_MAX_SPLITS = 8;   // CTAs of one cluster sharing a (token, head): portable cluster size

__device__ __forceinline__ float cache_ld(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float cache_ld(const __nv_bfloat16* p, size_t i) { return __uint_as_float((unsigned)reinterpret_cast<const unsigned short*>(p)[i] << 16); }
__device__ __forceinline__ void cache_st(float* p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void cache_st(__nv_bfloat16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// <q, row> for one cache row held by ONE lane (16-byte loads when the row is aligned)
__device__ __forceinline__ float dot_row(const float* row, const float* qs, int dim, bool vec) {
    float d = 0.f;
    if (vec) {
#pragma unroll 8
        for (int c = 0; c < dim; c += 4) {
            const float4 k = *reinterpret_cast<const float4*>(row + c);
            d = fmaf(qs[c], k.x, d); d = fmaf(qs[c + 1], k.y, d); d = fmaf(qs[c + 2], k.z, d); d = fmaf(qs[c + 3], k.w, d);
        }
    } else {
        for (int c = 0; c < dim; c++) d = fmaf(qs[c], row[c], d);
    }
    return d;
}
__device__ __forceinline__ float dot_row(const __nv_bfloat16* row, const float* qs, int dim, bool vec) {
    float d = 0.f;
    if (vec) {
#pragma unroll 8
        for (int c = 0; c < dim; c += 8) {
            const uint4 k = *reinterpret_cast<const uint4*>(row + c);
            const unsigned u[4] = {k.x, k.y, k.z, k.w};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                d = fmaf(qs[c + 2 * e], __uint_as_float(u[e] << 16), d);
                d = fmaf(qs[c + 2 * e + 1], __uint_as_float(u[e] & 0xFFFF0000u), d);
            }
        }
    } else {
        for (int c = 0; c < dim; c++) d = fmaf(qs[c], cache_ld(row, c), d);
    }
    return d;
}

// Warps take groups of 32 visible keys.  Scoring is lane-per-key (each lane walks one key row against q in shared memory: no
// cross-lane reduction per key); the group's maximum and the rescale are one warp reduction; the weighted value sum is
// lane-per-channel (the 32 probabilities are broadcast one by one, value rows are read coalesced).
template <typename KT, int AW_MAXV>       // AW_MAXV: value elements per lane (vdim <= 32 * AW_MAXV)
__global__ void __launch_bounds__(AW_WARPS * 32) attention_window_kernel(float* __restrict__ out, const float* __restrict__ Q, const KT* __restrict__ kc,
                                                                         const KT* __restrict__ vc, const int* __restrict__ pos_dev, int p0,
                                                                         WindowAttn a) {
    // q[dim rounded to 4] | per-warp acc[AW_WARPS][vdim] | m[AW_WARPS] | l[AW_WARPS] | per-CTA partials [splits][vdim + 2] (leader's copy is used)
    extern __shared__ __align__(16) float sm[];
    float* qs = sm;
    float* accs = sm + ((a.dim + 3) & ~3);
    float* ms = accs + AW_WARPS * a.vdim;
    float* ls = ms + AW_WARPS;
    float* part = ls + AW_WARPS;
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int splits = gridDim.z, rank = blockIdx.z;       // the cluster spans z: its CTAs share the (token, head) and split the keys
    // blockIdx.y walks (head, map): map mp of head h scores against map mp of key head g and sums the head's one value row
    const int t = blockIdx.x, hm = blockIdx.y, h = hm / a.maps, mp = hm % a.maps, g = h / (a.heads / a.kv_heads), gk = g * a.maps + mp;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();
    const int pos = (pos_dev ? *pos_dev : p0) + t;
    const float* q = Q + (size_t)t * a.heads * a.maps * a.dim + (size_t)hm * a.dim;
    for (int i = threadIdx.x; i < a.dim; i += AW_WARPS * 32) qs[i] = q[i];
    __syncthreads();
    if (splits > 1) cluster.sync();                          // every CTA of the cluster is resident before anyone writes into a peer's shared memory
    // visible keys: [0, n_first) and [lo, pos]
    const int lo = a.chunk > 0 ? (pos / a.chunk) * a.chunk : (a.window > 0 ? max(0, pos - a.window + 1) : 0);
    const int n_first = a.chunk > 0 ? 0 : min(a.keep, lo);
    const int n_keys = n_first + (pos - lo + 1);
    const size_t kstride = a.k_stride > 0 ? (size_t)a.k_stride : (size_t)a.kv_heads * a.maps * a.dim;
    const size_t vstride = a.v_stride > 0 ? (size_t)a.v_stride : (size_t)a.kv_heads * a.vdim;
    constexpr int PER16 = 16 / (int)sizeof(KT);
    const bool vec = a.dim % PER16 == 0 && kstride % PER16 == 0 && (reinterpret_cast<uintptr_t>(kc) & 15) == 0;      // every key row then starts on 16 bytes
    float m = -FLT_MAX, l = 0.f, acc[AW_MAXV];
#pragma unroll
    for (int e = 0; e < AW_MAXV; e++) acc[e] = 0.f;
    for (int n0 = (rank * AW_WARPS + warp) * 32; n0 < n_keys; n0 += splits * AW_WARPS * 32) {
        const int n = n0 + lane;
        const bool valid = n < n_keys;
        const int j = valid ? (n < n_first ? n : lo + (n - n_first)) : 0;
        float sc = -FLT_MAX;
        if (valid) {
            sc = dot_row(kc + (size_t)j * kstride + (size_t)gk * a.dim, qs, a.dim, vec) * a.scale;
            if (a.softcap > 0.f) sc = a.softcap * tanhf(sc / a.softcap);
        }
        float gmax = sc;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) gmax = fmaxf(gmax, __shfl_xor_sync(0xFFFFFFFFu, gmax, o));
        const float mn = fmaxf(m, gmax);
        const float corr = expf(m - mn), p = valid ? expf(sc - mn) : 0.f;
        l = l * corr + p;                                   // per-lane partial sums, reduced once at the end
        m = mn;
#pragma unroll
        for (int e = 0; e < AW_MAXV; e++) acc[e] *= corr;
        // all 32 slots: lanes past the last key carry p == 0 and row 0, so the trip count is fixed and the loads of several
        // keys are in flight together
#pragma unroll 8
        for (int kk = 0; kk < 32; kk++) {
            const float pk = __shfl_sync(0xFFFFFFFFu, p, kk);
            const int jk = __shfl_sync(0xFFFFFFFFu, j, kk);
            const KT* vr = vc + (size_t)jk * vstride + (a.joint_v ? 0 : (size_t)g * a.vdim);
#pragma unroll
            for (int e = 0; e < AW_MAXV; e++) {
                const int i = lane + 32 * e;
                if (i < a.vdim) acc[e] = fmaf(pk, cache_ld(vr, i), acc[e]);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xFFFFFFFFu, l, o);
    if (lane == 0) { ms[warp] = m; ls[warp] = l; }
#pragma unroll
    for (int e = 0; e < AW_MAXV; e++) { const int i = lane + 32 * e; if (i < a.vdim) accs[warp * a.vdim + i] = acc[e]; }
    __syncthreads();
    float M = -FLT_MAX;
    for (int w = 0; w < AW_WARPS; w++) M = fmaxf(M, ms[w]);
    float L = 0.f;
    for (int w = 0; w < AW_WARPS; w++) L += ls[w] * expf(ms[w] - M);
    float* o = out + (size_t)t * a.heads * a.maps * a.vdim + (size_t)hm * a.vdim;
    if (splits == 1) {
        // the sink joins the denominator as one more term exp(sink - max): the maximum is raised to it first so nothing overflows
        float fix = 1.f;
        if (a.sink) { const float sk = a.sink[h], M2 = fmaxf(M, sk); fix = expf(M - M2); L = L * fix + expf(sk - M2); }
        for (int i = threadIdx.x; i < a.vdim; i += AW_WARPS * 32) {
            float v = 0.f;
            for (int w = 0; w < AW_WARPS; w++) v += accs[w * a.vdim + i] * expf(ms[w] - M);
            o[i] = v * fix / L;
        }
        return;
    }
    // this CTA's (max, sum, unnormalised vector) goes into slot `rank` of the leader's shared memory (distributed shared memory),
    // the cluster barrier orders the writes before the leader's reads, the leader merges the slots
    float* dst = cluster.map_shared_rank(part, 0) + (size_t)rank * (a.vdim + 2);
    for (int i = threadIdx.x; i < a.vdim; i += AW_WARPS * 32) {
        float v = 0.f;
        for (int w = 0; w < AW_WARPS; w++) v += accs[w * a.vdim + i] * expf(ms[w] - M);
        dst[2 + i] = v;
    }
    if (threadIdx.x == 0) { dst[0] = M; dst[1] = L; }
    cluster.sync();
    if (rank != 0) return;
    float MM = -FLT_MAX;
    for (int r = 0; r < splits; r++) MM = fmaxf(MM, part[(size_t)r * (a.vdim + 2)]);
    if (a.sink) MM = fmaxf(MM, a.sink[h]);
    float LL = a.sink ? expf(a.sink[h] - MM) : 0.f;
    for (int r = 0; r < splits; r++) LL += part[(size_t)r * (a.vdim + 2) + 1] * expf(part[(size_t)r * (a.vdim + 2)] - MM);
    for (int i = threadIdx.x; i < a.vdim; i += AW_WARPS * 32) {
        float v = 0.f;
        for (int r = 0; r < splits; r++) v += part[(size_t)r * (a.vdim + 2) + 2 + i] * expf(part[(size_t)r * (a.vdim + 2)] - MM);
        o[i] = v / LL;
    }
}

// grid (tokens, 2).  y == 0: the query row, RMS-normalised over its whole length in place (or left alone);
// y == 1: the key row, normalised the same way, and the value row, both written to cache row pos.
template <typename KT>
__global__ void __launch_bounds__(256) qk_norm_kv_write_kernel(float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
                                                               const float* __restrict__ qn, const float* __restrict__ kn, float eps, KT* __restrict__ kc,
                                                               KT* __restrict__ vc, const int* __restrict__ pos_dev, int p0, int qdim, int kdim, int vdim) {
    __shared__ float red[8];
    __shared__ float inv_s;
    const int t = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const int pos = (pos_dev ? *pos_dev : p0) + t;
    const bool is_q = blockIdx.y == 0;
    const int n = is_q ? qdim : kdim;
    const float* src = is_q ? Q + (size_t)t * qdim : K + (size_t)t * kdim;
    const float* gain = is_q ? qn : kn;
    float inv = 1.f;
    if (gain) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < n; i += 256) ss = fmaf(src[i], src[i], ss);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        if (threadIdx.x == 0) {
            float tot = 0.f;
            for (int w = 0; w < 8; w++) tot += red[w];
            inv_s = 1.0f / sqrtf(tot / (float)n + eps);
        }
        __syncthreads();
        inv = inv_s;
    }
    if (is_q) {
        if (gain) { float* qr = Q + (size_t)t * qdim; for (int i = threadIdx.x; i < n; i += 256) qr[i] = qr[i] * inv * gain[i]; }
        return;
    }
    for (int i = threadIdx.x; i < kdim; i += 256) cache_st(kc, (size_t)pos * kdim + i, gain ? src[i] * inv * gain[i] : src[i]);
    const float* vr = V + (size_t)t * vdim;
    for (int i = threadIdx.x; i < vdim; i += 256) cache_st(vc, (size_t)pos * vdim + i, vr[i]);
}

}  // namespace

void attention_window(float* out, const float* Q, const void* kc, const void* vc, DType cache_dt, int tokens, const int* pos_dev, int p0,
                      int max_seq, const WindowAttn& a, cudaStream_t s) {
    static const bool no_mma = getenv("NT_B200_NO_WINDOW_MMA") != nullptr;
    if (!pos_dev && !no_mma && attention_window_mma_supported(tokens, a, cache_dt)) { attention_window_mma(out, Q, kc, vc, tokens, p0, max_seq, a, s); return; }
    NT_CHECK(a.vdim <= 512, "attention_window: value heads wider than 512 are not covered");
    NT_CHECK(a.heads % a.kv_heads == 0, "attention_window: heads must be a multiple of kv_heads");
    NT_CHECK(cache_dt == DType::F32 || cache_dt == DType::BF16, "attention_window: F32 or BF16 cache");
    if (tokens <= 0) return;
    // A single decoded token has only `heads` CTAs: split each head's keys over a thread-block cluster (one CTA per ~256 keys of
    // the longest visible range), merged through the leader's shared memory.  Prompt portions have CTAs enough without it.
    const int longest = a.chunk > 0 ? std::min(max_seq, a.chunk) : (a.window > 0 ? std::min(max_seq, a.window + a.keep) : max_seq);
    const int splits = tokens == 1 ? std::max(1, std::min(AW_MAX_SPLITS, (longest + 255) / 256)) : 1;
    const size_t smem = sizeof(float) * ((size_t)((a.dim + 3) & ~3) + (size_t)AW_WARPS * a.vdim + 2 * AW_WARPS + (size_t)splits * (a.vdim + 2));
    cudaLaunchConfig_t cfg{};
    NT_CHECK(a.maps >= 1, "attention_window: maps >= 1");
    NT_CHECK(!a.joint_v || (a.v_stride > 0 && a.maps == 1), "attention_window: joint values need the value row stride and one map");
    cfg.gridDim = dim3(tokens, a.heads * a.maps, splits); cfg.blockDim = dim3(AW_WARPS * 32); cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    at[1].id = cudaLaunchAttributeClusterDimension;
    at[1].val.clusterDim.x = 1; at[1].val.clusterDim.y = 1; at[1].val.clusterDim.z = (unsigned)splits;
    cfg.attrs = at; cfg.numAttrs = 2;
    NT_CHECK(smem <= 48 * 1024, "attention_window: the head does not fit in shared memory");
    const bool wide = a.vdim > 256;          // wide value rows (a latent as the value) keep 16 numbers per lane
    if (cache_dt == DType::F32) {
        auto* kern = wide ? attention_window_kernel<float, 16> : attention_window_kernel<float, 8>;
        NT_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, out, Q, static_cast<const float*>(kc), static_cast<const float*>(vc), pos_dev, p0, a));
    } else {
        auto* kern = wide ? attention_window_kernel<__nv_bfloat16, 16> : attention_window_kernel<__nv_bfloat16, 8>;
        NT_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, out, Q, static_cast<const __nv_bfloat16*>(kc), static_cast<const __nv_bfloat16*>(vc), pos_dev, p0, a));
    }
    count_launch();
}

void qk_norm_kv_write(float* Q, const float* K, const float* V, const float* q_gain, const float* k_gain, float eps, void* kc, void* vc,
                      DType cache_dt, int tokens, const int* pos_dev, int p0, int qdim, int kdim, int vdim, cudaStream_t s) {
    NT_CHECK(cache_dt == DType::F32 || cache_dt == DType::BF16, "qk_norm_kv_write: F32 or BF16 cache");
    if (tokens <= 0) return;
    if (cache_dt == DType::F32)
        launch_k(qk_norm_kv_write_kernel<float>, dim3(tokens, 2), dim3(256), 0, s, Q, K, V, q_gain, k_gain, eps, static_cast<float*>(kc),
                 static_cast<float*>(vc), pos_dev, p0, qdim, kdim, vdim);
    else
        launch_k(qk_norm_kv_write_kernel<__nv_bfloat16>, dim3(tokens, 2), dim3(256), 0, s, Q, K, V, q_gain, k_gain, eps,
                 static_cast<__nv_bfloat16*>(kc), static_cast<__nv_bfloat16*>(vc), pos_dev, p0, qdim, kdim, vdim);
    count_launch();
}

}}  // namespace nt::b200
