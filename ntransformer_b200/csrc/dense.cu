// dense.cu — GEMV / GEMM over dense weight rows (F32, F16, BF16) with F32 activations and F32 accumulation, plus the
// elementwise pieces of the layer-spec model families (engine/layer_spec.h).
//
//   gemv_dense   decode: up to 3 matrices share one activation vector staged once per CTA in shared memory; a warp streams one
//                output row with 16-byte loads; the prologue can RMS-normalise the staged vector; epilogues fuse the residual (+ per-channel gain) and the gated activations, so a
//                decode step needs no separate add / scale / activation launch.
//   gemm_dense   prompt tokens on CUDA cores: 64x64x16 tiles, 4x4 outputs per thread, true FP32 FMA.  It serves the exact
//                32-bit mode and shapes the tcgen05 tiles of prefill_gemm.cu do not cover (rows % 128, cols % 64).
// This file is compiled WITHOUT --use_fast_math (tanh / exp / division at full precision): the 32-bit mode depends on it.
#include "kernels_internal.h"
#include "ring.cuh"
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <algorithm>

namespace nt { namespace b200 {

namespace {

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

template <typename T> struct Elem;
template <> struct Elem<float> {
    static constexpr int PER16 = 4;
    static __device__ __forceinline__ float one(const void* row, int i) { return __ldg(static_cast<const float*>(row) + i); }
    static __device__ __forceinline__ void unpack(const uint4& w, float* f) { f[0] = __uint_as_float(w.x); f[1] = __uint_as_float(w.y); f[2] = __uint_as_float(w.z); f[3] = __uint_as_float(w.w); }
};
template <> struct Elem<__half> {
    static constexpr int PER16 = 8;
    static __device__ __forceinline__ float one(const void* row, int i) { return __half2float(__ushort_as_half(__ldg(static_cast<const unsigned short*>(row) + i))); }
    static __device__ __forceinline__ void unpack(const uint4& w, float* f) {
        const unsigned u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int k = 0; k < 4; k++) { float2 p = __half22float2(*reinterpret_cast<const __half2*>(&u[k])); f[2 * k] = p.x; f[2 * k + 1] = p.y; }
    }
};
template <> struct Elem<__nv_bfloat16> {
    static constexpr int PER16 = 8;
    static __device__ __forceinline__ float one(const void* row, int i) { return __uint_as_float((unsigned)__ldg(static_cast<const unsigned short*>(row) + i) << 16); }
    static __device__ __forceinline__ void unpack(const uint4& w, float* f) {
        const unsigned u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int k = 0; k < 4; k++) { f[2 * k] = __uint_as_float(u[k] << 16); f[2 * k + 1] = __uint_as_float(u[k] & 0xFFFF0000u); }
    }
};

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// element r of every stream of one token: X[t][r] <- sum_s M[s][t] X[s][r] + b[t] * v  (all t from the old values)
__device__ __forceinline__ void streams_update(const StreamsIO& sio, int N, int r, float v) {
    float xv[16], nv[16];
#pragma unroll
    for (int s = 0; s < 16; s++) xv[s] = s < sio.S ? sio.X_out[(size_t)s * N + r] : 0.f;
#pragma unroll
    for (int t = 0; t < 16; t++) {
        float acc = 0.f;
        if (t < sio.S) {
#pragma unroll
            for (int s = 0; s < 16; s++) if (s < sio.S) acc = fmaf(sio.M[s * sio.S + t], xv[s], acc);
            acc = fmaf(sio.b[t], v, acc);
        }
        nv[t] = acc;
    }
#pragma unroll
    for (int t = 0; t < 16; t++) if (t < sio.S) sio.X_out[(size_t)t * N + r] = nv[t];
}

struct DenseMats {
    const unsigned char* W[DENSE_MAX_MATS];
    float* y[DENSE_MAX_MATS];
    int out[DENSE_MAX_MATS];
    size_t pitch[DENSE_MAX_MATS];
    int n;
};

constexpr int DV_WARPS = 8;

// <row, xs> for one row; vec: row base and pitch 16-byte aligned and K a multiple of PER16
template <typename T>
__device__ __forceinline__ float dense_row_dot(const unsigned char* row, const float* xs, int K, int lane, bool vec) {
    float acc = 0.f;
    constexpr int P = Elem<T>::PER16;
    if (vec) {
        const int nv = K / P;
        int v = lane;
        for (; v + 96 < nv; v += 128) {
            uint4 w[4];
#pragma unroll
            for (int u = 0; u < 4; u++) w[u] = ld_stream16(row + (size_t)(v + 32 * u) * 16);
#pragma unroll
            for (int u = 0; u < 4; u++) {
                float f[P];
                Elem<T>::unpack(w[u], f);
                const float* xp = xs + (size_t)(v + 32 * u) * P;
#pragma unroll
                for (int k = 0; k < P; k++) acc = fmaf(f[k], xp[k], acc);
            }
        }
        for (; v < nv; v += 32) {
            float f[P];
            Elem<T>::unpack(ld_stream16(row + (size_t)v * 16), f);
            const float* xp = xs + (size_t)v * P;
#pragma unroll
            for (int k = 0; k < P; k++) acc = fmaf(f[k], xp[k], acc);
        }
    } else {
        for (int i = lane; i < K; i += 32) acc = fmaf(Elem<T>::one(row, i), xs[i], acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
    return acc;
}

template <typename T>
__global__ void __launch_bounds__(DV_WARPS * 32) gemv_dense_kernel(DenseMats m, const float* __restrict__ x, int K, int ep,
                                                                   const float* __restrict__ row_scale, float alpha, int vec,
                                                                   const float* __restrict__ norm_w, float eps, StreamsIO sio) {
    extern __shared__ __align__(16) float xs[];
    __shared__ float red[DV_WARPS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();
    float ss = 0.f;
    for (int i = threadIdx.x; i < K; i += DV_WARPS * 32) {
        float v;
        if (sio.X_in) {                   // the blend of the token's residual streams
            v = 0.f;
            for (int st = 0; st < sio.S; st++) { const float xv = sio.X_in[(size_t)st * K + i]; v = sio.a ? fmaf(sio.a[st], xv, v) : v + xv; }
        } else v = x[i];
        xs[i] = v; ss = fmaf(v, v, ss);
    }
    if (norm_w) {
        // RMS norm of the staged vector: every CTA sums the squares in the same order, so all CTAs (and every launch that reads the
        // same x) derive the bit-identical normalised vector
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < DV_WARPS; w++) tot += red[w];
        const float inv = 1.0f / sqrtf(tot / (float)K + eps);
        for (int i = threadIdx.x; i < K; i += DV_WARPS * 32) xs[i] = xs[i] * inv * norm_w[i];
    }
    __syncthreads();
    const bool glu = ep == DENSE_SWIGLU || ep == DENSE_GEGLU || ep == DENSE_REGLU;
    int total = m.out[0];
    if (!glu) for (int i = 1; i < m.n; i++) total += m.out[i];
    for (int r = blockIdx.x * DV_WARPS + warp; r < total; r += gridDim.x * DV_WARPS) {
        if (glu) {
            const float g = dense_row_dot<T>(m.W[0] + (size_t)r * m.pitch[0], xs, K, lane, vec);
            const float u = dense_row_dot<T>(m.W[1] + (size_t)r * m.pitch[1], xs, K, lane, vec);
            if (lane == 0) m.y[0][r] = (ep == DENSE_GEGLU ? gelu_tanh_f(g) : ep == DENSE_REGLU ? fmaxf(g, 0.f) : silu_f(g)) * u;
            continue;
        }
        int mi = 0, row = r;
        while (mi + 1 < m.n && row >= m.out[mi]) { row -= m.out[mi]; mi++; }
        const float v = dense_row_dot<T>(m.W[mi] + (size_t)row * m.pitch[mi], xs, K, lane, vec);
        if (lane == 0 && ep == DENSE_STREAMS) streams_update(sio, m.out[0], row, v);
        else if (lane == 0) {
            float* y = m.y[mi] + row;
            if (ep == DENSE_ADD) *y += v;
            else if (ep == DENSE_SCALED_ADD) *y = fmaf(alpha * (row_scale ? row_scale[row] : 1.f), v, *y);
            else *y = v;
        }
    }
}

// ---- C[T,N] (ep)= A[T,K] . W[N,K]^T on CUDA cores ----
constexpr int GT = 64, GK = 16;
template <typename T>
__global__ void __launch_bounds__(256) gemm_dense_kernel(float* __restrict__ C, const float* __restrict__ A, const unsigned char* __restrict__ W,
                                                         size_t pitch, int Tn, int N, int K, int ep, const float* __restrict__ row_scale, float alpha) {
    __shared__ float As[GK][GT + 4];
    __shared__ float Ws[GK][GT + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int t0 = blockIdx.y * GT, n0 = blockIdx.x * GT;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += GK) {
        for (int e = threadIdx.x; e < GT * GK; e += 256) {
            const int r = e / GK, k = e % GK;
            const int t = t0 + r, n = n0 + r, kk = k0 + k;
            As[k][r] = (t < Tn && kk < K) ? A[(size_t)t * K + kk] : 0.f;
            Ws[k][r] = (n < N && kk < K) ? Elem<T>::one(W + (size_t)n * pitch, kk) : 0.f;
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
        const int t = t0 + ty * 4 + i;
        if (t >= Tn) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float* c = C + (size_t)t * N + n;
            if (ep == DENSE_ADD) *c += acc[i][j];
            else if (ep == DENSE_SCALED_ADD) *c = fmaf(alpha * (row_scale ? row_scale[n] : 1.f), acc[i][j], *c);
            else *c = acc[i][j];
        }
    }
}

__global__ void glu_mul_kernel(float* __restrict__ out, const float* __restrict__ gate, const float* __restrict__ up, size_t n, int act) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = (act == 1 ? gelu_tanh_f(gate[i]) : act == 2 ? fmaxf(gate[i], 0.f) : silu_f(gate[i])) * up[i];
}
__global__ void scaled_add_rows_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ row_scale, float alpha,
                                       size_t n, int cols) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = fmaf(alpha * (row_scale ? row_scale[i % cols] : 1.f), y[i], x[i]);
}
__global__ void copy_cols_kernel(float* __restrict__ out, const float* __restrict__ in, size_t n, int cols, int ld) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = in[(i / cols) * ld + i % cols];
}
template <typename T>
__global__ void to_f32_kernel(float* __restrict__ out, const T* __restrict__ in, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = Elem<T>::one(in + i, 0);
}

}  // namespace

bool dense_dtype(DType dt) { return dt == DType::F32 || dt == DType::F16 || dt == DType::BF16; }

void gemv_dense(const GemvMat* mats, int n_mat, int K, const float* x, DenseEpilogue ep, const float* row_scale, float alpha, cudaStream_t s,
                const float* norm_w, float eps, const StreamsIO* sio_p) {
    NT_CHECK(n_mat >= 1 && n_mat <= DENSE_MAX_MATS, "gemv_dense: too many matrices for one launch");
    const StreamsIO sio = sio_p ? *sio_p : StreamsIO();
    NT_CHECK(ep != DENSE_STREAMS || (n_mat == 1 && sio.X_out && sio.M && sio.b && sio.S >= 1 && sio.S <= 16), "gemv_dense: the streams epilogue takes one matrix and the stream tables");
    NT_CHECK(!sio.X_in || (sio.S >= 1 && sio.S <= 16), "gemv_dense: 1..16 streams");
    const bool glu = ep == DENSE_SWIGLU || ep == DENSE_GEGLU || ep == DENSE_REGLU;
    NT_CHECK(!glu || (n_mat == 2 && mats[0].out == mats[1].out), "gemv_dense: a gated epilogue takes two matrices of equal height");
    const DType dt = mats[0].dtype;
    NT_CHECK(dense_dtype(dt), "gemv_dense: dense dtypes only");
    DenseMats m{};
    m.n = n_mat;
    const int per16 = dt == DType::F32 ? 4 : 8;
    int vec = (K % per16 == 0) ? 1 : 0, total = 0;
    for (int i = 0; i < n_mat; i++) {
        NT_CHECK(mats[i].dtype == dt, "gemv_dense: one dtype per launch");
        m.W[i] = static_cast<const unsigned char*>(mats[i].W); m.y[i] = mats[i].y; m.out[i] = mats[i].out;
        m.pitch[i] = mats[i].row_pitch ? mats[i].row_pitch : dtype_row_size(dt, (size_t)K);
        if ((reinterpret_cast<uintptr_t>(mats[i].W) & 15) || (m.pitch[i] & 15)) vec = 0;
        total += mats[i].out;
    }
    if (glu) total = mats[0].out;
    if (total <= 0) return;
    const size_t smem = (size_t)K * sizeof(float);
    NT_CHECK(smem <= 200 * 1024, "gemv_dense: the activation vector does not fit in shared memory");
    int grid = (total + DV_WARPS - 1) / DV_WARPS;
    const int resident = (int)std::max<size_t>(1, std::min<size_t>(8, (size_t)(220 * 1024) / (smem + 1024))) * 148;
    grid = std::min(grid, resident);
#define NT_DV(TY) { static unsigned long long done = 0; if (smem > 48 * 1024) opt_in_dynamic_smem(gemv_dense_kernel<TY>, 200 * 1024, done); \
                    launch_k(gemv_dense_kernel<TY>, dim3(grid), dim3(DV_WARPS * 32), smem, s, m, x, K, (int)ep, row_scale, alpha, vec, norm_w, eps, sio); }
    if (dt == DType::F32) NT_DV(float) else if (dt == DType::F16) NT_DV(__half) else NT_DV(__nv_bfloat16)
#undef NT_DV
    count_launch();
}

void gemm_dense(float* C, const float* A, const void* W, DType dt, size_t row_pitch, int T, int N, int K, DenseEpilogue ep,
                const float* row_scale, float alpha, cudaStream_t s) {
    NT_CHECK(dense_dtype(dt), "gemm_dense: dense dtypes only");
    NT_CHECK(ep == DENSE_STORE || ep == DENSE_ADD || ep == DENSE_SCALED_ADD, "gemm_dense: store / add / scaled-add epilogues");
    if (T <= 0 || N <= 0) return;
    const size_t pitch = row_pitch ? row_pitch : dtype_row_size(dt, (size_t)K);
    const dim3 grid((N + GT - 1) / GT, (T + GT - 1) / GT);
    const unsigned char* w = static_cast<const unsigned char*>(W);
    if (dt == DType::F32) gemm_dense_kernel<float><<<grid, 256, 0, s>>>(C, A, w, pitch, T, N, K, (int)ep, row_scale, alpha);
    else if (dt == DType::F16) gemm_dense_kernel<__half><<<grid, 256, 0, s>>>(C, A, w, pitch, T, N, K, (int)ep, row_scale, alpha);
    else gemm_dense_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(C, A, w, pitch, T, N, K, (int)ep, row_scale, alpha);
    NT_LAUNCH_CHECK();
    count_launch();
}

void glu_mul(float* out, const float* gate, const float* up, size_t n, bool gelu, cudaStream_t s, bool relu) {
    if (!n) return;
    glu_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(out, gate, up, n, relu ? 2 : (gelu ? 1 : 0));
    NT_LAUNCH_CHECK();
    count_launch();
}

void copy_cols(float* out, const float* in, int rows, int cols, int ld, cudaStream_t s) {
    const size_t n = (size_t)rows * cols;
    if (!n) return;
    copy_cols_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(out, in, n, cols, ld);
    NT_LAUNCH_CHECK();
    count_launch();
}

void scaled_add_rows(float* x, const float* y, const float* row_scale, float alpha, int rows, int cols, cudaStream_t s) {
    const size_t n = (size_t)rows * cols;
    if (!n) return;
    scaled_add_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(x, y, row_scale, alpha, n, cols);
    NT_LAUNCH_CHECK();
    count_launch();
}

void dense_to_f32(float* out, const void* in, DType dt, size_t n, cudaStream_t s) {
    if (!n) return;
    const unsigned g = (unsigned)((n + 255) / 256);
    if (dt == DType::F32) NT_CUDA_CHECK(cudaMemcpyAsync(out, in, n * 4, cudaMemcpyDeviceToDevice, s));
    else if (dt == DType::F16) to_f32_kernel<__half><<<g, 256, 0, s>>>(out, static_cast<const __half*>(in), n);
    else if (dt == DType::BF16) to_f32_kernel<__nv_bfloat16><<<g, 256, 0, s>>>(out, static_cast<const __nv_bfloat16*>(in), n);
    else NT_CHECK(false, "dense_to_f32: dense dtypes only");
    NT_LAUNCH_CHECK();
}

}}  // namespace nt::b200
