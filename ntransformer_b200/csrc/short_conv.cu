// short_conv.cu — short causal per-channel convolutions over time on projected rows (LayerSpec::conv), several projections per launch:
//       y_t[c] = act( sum_j w[c, j] * u_{t - taps + 1 + j}[c] ),   u_t = (W x_t)[c] (+ bias[c]),   u_t = 0 before the sequence's start,
// the last tap being the current token's.  Each projection ("segment") brings its own rows, taps, optional input bias (the bias of a biased
// projection: it belongs to u, so it is part of what the state keeps, and the zeros before the start stay zeros), activation (none or
// SiLU) and state [taps - 1, channels] holding the last taps - 1 inputs of the sequence (one tap without weights: only the bias and the
// activation are applied).  The state is read unless the step starts at position 0 and is rewritten with the step's last inputs, so a
// prompt cut anywhere continues exactly.
//   one decoded token: one launch, a thread per channel reads its state column, convolves and shifts the column;
//   prompt rows: a launch over (channels, rows), then a launch that rewrites the state (it must not run before every row has read it).
// A step's base position is *pos_dev when given (the captured decode step), else p0.  All F32; compiled WITHOUT --use_fast_math.
#include "kernels_internal.h"
#include "ring.cuh"

namespace nt { namespace b200 {

namespace {

struct ConvPack {
    ConvSeg s[SHORT_CONV_MAX_SEGS];
    int first_block[SHORT_CONV_MAX_SEGS + 1];      // blocks of 256 channels: segment i owns [first_block[i], first_block[i + 1])
    int n;
};

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

__device__ __forceinline__ int segment_of(const ConvPack& p, int block, int& c) {
    int i = 0;
    while (i + 1 < p.n && block >= p.first_block[i + 1]) i++;
    c = (block - p.first_block[i]) * 256 + threadIdx.x;
    return i;
}

// grid (blocks, T)
__global__ void __launch_bounds__(256) short_conv_rows_kernel(ConvPack p, int T, const int* __restrict__ pos_dev, int p0) {
    pdl_launch_dependents();
    pdl_wait();
    int c;
    const ConvSeg& g = p.s[segment_of(p, blockIdx.x, c)];
    if (c >= g.ch) return;
    const int t = blockIdx.y;
    const bool fresh = (pos_dev ? *pos_dev : p0) == 0;
    const float bias = g.in_bias ? g.in_bias[c] : 0.f;
    float acc = 0.f;
    for (int k = 0; k < g.taps; k++) {
        const int tt = t - (g.taps - 1) + k;
        float v;
        if (tt >= 0) v = g.u[(size_t)tt * g.ld + g.col0 + c] + bias;
        else v = fresh ? 0.f : g.state[(size_t)(g.taps - 1 + tt) * g.ch + c];
        acc = fmaf(g.w ? g.w[(size_t)c * g.taps + k] : 1.f, v, acc);
    }
    g.out[(size_t)t * g.out_ld + c] = g.act ? silu_f(acc) : acc;
}

// grid (blocks).  Slot j ascending takes element T + j of [state ++ rows], which lies behind every slot written so far.
__global__ void __launch_bounds__(256) short_conv_state_kernel(ConvPack p, int T, const int* __restrict__ pos_dev, int p0) {
    pdl_launch_dependents();
    pdl_wait();
    int c;
    const ConvSeg& g = p.s[segment_of(p, blockIdx.x, c)];
    if (c >= g.ch) return;
    const bool fresh = (pos_dev ? *pos_dev : p0) == 0;
    const float bias = g.in_bias ? g.in_bias[c] : 0.f;
    for (int j = 0; j < g.taps - 1; j++) {
        const int idx = T + j;
        g.state[(size_t)j * g.ch + c] = idx < g.taps - 1 ? (fresh ? 0.f : g.state[(size_t)idx * g.ch + c]) : g.u[(size_t)(idx - (g.taps - 1)) * g.ld + g.col0 + c] + bias;
    }
}

// One row: convolve and shift the state column in the same thread.
__global__ void __launch_bounds__(256) short_conv_step_kernel(ConvPack p, const int* __restrict__ pos_dev, int p0) {
    pdl_launch_dependents();
    pdl_wait();
    int c;
    const ConvSeg& g = p.s[segment_of(p, blockIdx.x, c)];
    if (c >= g.ch) return;
    const bool fresh = (pos_dev ? *pos_dev : p0) == 0;
    const float cur = g.u[g.col0 + c] + (g.in_bias ? g.in_bias[c] : 0.f);
    float acc = 0.f;
    for (int k = 0; k + 1 < g.taps; k++) {
        const float v = fresh ? 0.f : g.state[(size_t)k * g.ch + c];
        acc = fmaf(g.w[(size_t)c * g.taps + k], v, acc);
        if (k > 0) g.state[(size_t)(k - 1) * g.ch + c] = v;
    }
    acc = fmaf(g.w ? g.w[(size_t)c * g.taps + g.taps - 1] : 1.f, cur, acc);
    if (g.taps > 1) g.state[(size_t)(g.taps - 2) * g.ch + c] = cur;
    g.out[c] = g.act ? silu_f(acc) : acc;
}

}  // namespace

void short_conv(const ConvSeg* segs, int n, int T, const int* pos_dev, int p0, cudaStream_t s) {
    NT_CHECK(n >= 1 && n <= SHORT_CONV_MAX_SEGS, "short_conv: too many segments for one launch");
    if (T <= 0) return;
    ConvPack p{};
    p.n = n;
    int blocks = 0;
    bool any_state = false;
    for (int i = 0; i < n; i++) {
        NT_CHECK(segs[i].taps >= 1 && segs[i].ch > 0 && (segs[i].taps == 1 || (segs[i].state && segs[i].w)), "short_conv: a segment needs taps >= 1, channels, taps' weights and a state");
        p.s[i] = segs[i];
        p.first_block[i] = blocks;
        blocks += (segs[i].ch + 255) / 256;
        any_state = any_state || segs[i].taps > 1;
    }
    p.first_block[n] = blocks;
    if (T == 1) {
        launch_k(short_conv_step_kernel, dim3(blocks), dim3(256), 0, s, p, pos_dev, p0);
        count_launch();
        return;
    }
    launch_k(short_conv_rows_kernel, dim3(blocks, T), dim3(256), 0, s, p, T, pos_dev, p0);
    count_launch();
    if (any_state) {
        launch_k(short_conv_state_kernel, dim3(blocks), dim3(256), 0, s, p, T, pos_dev, p0);
        count_launch();
    }
}

}}  // namespace nt::b200
