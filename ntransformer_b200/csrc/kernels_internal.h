// kernels_internal.h — host-callable launch functions behind the C-ABI (include/nt_b200.h)
// and behind the nt::cuda::launch_* drop-in symbols. Everything here is sm_100a CUDA; there is
// deliberately no CPU path.
#pragma once
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>
#include "nt_types.h"

namespace nt { namespace b200 {

// ---------------------------------------------------------------------------------------------
// Block-scaled 3-term int8 activations ("xq").  x[e] ~= scale[e/32] * (q1*16384 + q2*128 + q3)
// with q1 in [-127,127], q2,q3 in [-64,64]: |error| <= 2^-22 of the 32-block absmax, i.e. F32-class.
// Integer dot products against the 4/5/6/8-bit weight codes are exact (IDP.4A), the float work is
// one scale per 16/32 weights instead of one convert + FMA per weight.
//   layout for K elements (K % 128 == 0): [q1: K][q2: K][q3: K][scale: K/32 f32][sum16: K/16 f32]; inside each plane
//   element e lives at byte e ^ (((e >> 7) & 7) << 4)  (the GEMV's bank-conflict-free shared-memory order)
// sum16 holds exact F32 sums of x over 16-element groups (for the dmin / -32 offset terms).
// ---------------------------------------------------------------------------------------------
inline size_t xq_bytes(int K) { return (size_t)3 * K + (size_t)(K / 32) * 4 + (size_t)(K / 16) * 4; }
void quantize_x(const float* x, void* xq, int K, cudaStream_t s);

// One weight matrix inside a (possibly fused) GEMV launch.
struct GemvMat {
    const void* W = nullptr;   // row-major GGUF blocks
    float* y = nullptr;        // output rows
    int out = 0;               // rows
    DType dtype = DType::F32;
    size_t row_pitch = 0;      // bytes between rows (0 = dense GGUF rows)
};
enum GemvEpilogue { GEMV_STORE = 0, GEMV_ADD = 1 /* y += W.x (residual) */, GEMV_SWIGLU = 2 /* y0 = silu(W0.x) * (W1.x) */,
                    GEMV_PEER = 3 /* tensor parallel: rows go to every rank's slot over NVLink (PeerOut), y is not written */ };


// Fused K-quant GEMV over up to 3 matrices sharing one activation vector (already in xq form).
// All matrices must be Q4_K / Q5_K / Q6_K with 16-byte aligned W and row pitch.
// Where the shared activation vector comes from: either pre-quantised `xq`, or an F32 vector `x` that the
// kernel quantises in its prologue (staged over the not-yet-primed part of its TMA ring), optionally as
// RMSNorm(x) * norm_w: the prologue quantises x * norm_w, sums x^2 in the same pass and the scalar
// rsqrt(mean(x^2) + eps) is applied to the results.
// Where a tensor-parallel GEMV (o-projection / down-projection shard) delivers its partial rows (engine/peer_xchg.h): the slot
// [parity][rank][hidden] of every rank.  A slot element is ONE 8-byte word {sequence number : value bits} written with a single
// 64-bit store (single-copy atomic), so the data is its own arrival flag: no fence, no separate flag hop — the receiver polls
// the element until it carries the sequence number it expects.  Pointers index ranks; entry `rank` is this GPU's own buffer.
struct PeerOut {
    static constexpr int kMaxTP = 8;
    unsigned long long* slots[kMaxTP];
    unsigned* seq;                 // exchanges completed on this rank; the exchange in flight carries *seq + 1
    unsigned* abort_word;
    int rank, size, hidden;
};
struct GemvInput {
    const void* xq = nullptr;
    const float* x = nullptr;
    const float* norm_w = nullptr;
    float eps = 0.f;
    const PeerOut* peer = nullptr;     // epilogue GEMV_PEER only
};
bool gemv_kq_supported(const GemvMat* mats, int n_mat, int K);
void gemv_kq(const GemvMat* mats, int n_mat, int K, const GemvInput& in, GemvEpilogue ep, cudaStream_t s);
void gemv_kq(const GemvMat* mats, int n_mat, int K, const void* xq, GemvEpilogue ep, cudaStream_t s);
// gemv_kquant_q.cu: the quarter-block kernel (lane <-> 64 weights, up to 16 warps); false = shape not covered, nothing launched
bool gemv_kq_quarter(const GemvMat* mats, int n_mat, int K, const GemvInput& in, GemvEpilogue ep, const PeerOut* peer, cudaStream_t s);
// epilogue GEMV_PEER: one matrix, rows == peer.hidden
void gemv_kq_peer(const GemvMat& mat, int K, const GemvInput& in, const PeerOut& peer, cudaStream_t s);

// Generic GEMV for every dtype / any alignment, F32 activations (Q8_0, Q4_0, F16, F32 and
// unaligned K-quant shards).
void gemv_generic(float* y, const void* W, const float* x, int out, int in, DType dt, size_t row_pitch,
                  GemvEpilogue ep, cudaStream_t s);


// ---- elementwise / norm / rope / kv / attention (reference kernels K10-K21) ----
void rmsnorm(float* y, const float* x, const float* w, int rows, int hidden, float eps, cudaStream_t s);
void rmsnorm_f16(void* y, const float* x, const float* w, int rows, int hidden, float eps, cudaStream_t s);
// fused: y = rmsnorm(x) (optional, may be null) and xq = quantise(rmsnorm(x)); rows == 1
void rmsnorm_xq(float* y, void* xq, const float* x, const float* w, int hidden, float eps, cudaStream_t s);
void rope(float* q, float* k, const int* positions, int seq_len, int n_heads, int n_kv_heads, int head_dim,
          float theta, float freq_scale, bool interleaved, cudaStream_t s);
void copy_to_kv_cache(void* kc, void* vc, const float* k, const float* v, int seq_len, int n_kv, int hd,
                      int start_pos, int max_seq, cudaStream_t s);
void silu_mul(float* out, const float* gate, const float* up, int n, cudaStream_t s);
void add_bias(float* y, const float* b, int n, cudaStream_t s);
void add(float* out, const float* a, const float* b, int n, cudaStream_t s);
void add_inplace(float* a, const float* b, int n, cudaStream_t s);
void copy(float* dst, const float* src, int n, cudaStream_t s);
void cosine_similarity(float* result, const float* a, const float* b, int n, cudaStream_t s);
void softmax(float* out, const float* in, int rows, int cols, cudaStream_t s);
void masked_softmax(float* out, const float* in, const bool* mask, int rows, int cols, cudaStream_t s);
void gemm_f32(float* C, const float* A, const float* B, int M, int N, int K, cudaStream_t s);
void attention_decode(float* out, const float* q, const void* kc, const void* vc, int seq_len, int n_heads,
                      int n_kv, int hd, int max_seq, float scale, cudaStream_t s);
void attention_prefill(float* out, const float* Q, const void* kc, const void* vc, int seq_len, int start_pos,
                       int n_heads, int n_kv, int hd, int max_seq, float scale, cudaStream_t s);
// attention_prefill_mma.cu: 64-query x 64-key tiles on mma.sync (used by attention_prefill for seq_len >= 16, hd 64/128)
bool attention_prefill_mma_supported(int seq_len, int n_heads, int n_kv, int hd);
void attention_prefill_mma(float* out, const float* Q, const void* kc, const void* vc, int seq_len, int start_pos, int n_heads,
                           int n_kv, int hd, int max_seq, float scale, cudaStream_t s);
// CUDA-graph friendly decode attention: context length = *pos_dev + 1 is read on the device.
int attention_decode_dyn_splits(int max_seq, int n_heads, int n_kv);
size_t attention_decode_dyn_scratch_floats(int max_seq, int n_heads, int n_kv, int hd);
// xq_out (optional): the merged output is also written in xq form for the o-projection GEMV.
void attention_decode_dyn(float* out, const float* q, const void* kc, const void* vc, const int* pos_dev, int max_seq,
                          int n_heads, int n_kv, int hd, float scale, float* scratch, void* xq_out, cudaStream_t s);
// The decode step's attention sub-block in one launch: RoPE (q and the new key; q, k are NOT modified in memory) + F16 KV-cache
// write at row *pos_dev + split-context attention + merge of the splits + optional xq of the result.  scratch as for
// attention_decode_dyn; tickets: attention_decode_fused_tickets() zeroed words (left zeroed).  hd 64 / 128 / 256.
int attention_decode_fused_tickets(int n_heads, int n_kv);
void attention_decode_fused(float* out, const float* q, const float* k, const float* v, void* kc, void* vc, const int* pos_dev,
                            int max_seq, int n_heads, int n_kv, int hd, float theta, float freq_scale, float scale, float* scratch,
                            unsigned* tickets, void* xq_out, cudaStream_t s);
// Two-launch form: RoPE + KV-cache write inside the split-context decode kernel (q, k not modified in memory), then the merge kernel.
void attention_decode_rope_dyn(float* out, const float* q, const float* k, const float* v, void* kc, void* vc, const int* pos_dev,
                               int max_seq, int n_heads, int n_kv, int hd, float theta, float freq_scale, float scale, float* scratch,
                               void* xq_out, cudaStream_t s);
// Fused RoPE (q, k in place; reference rotary.cu:16-62, non-interleaved pairs) + F16 KV-cache write at *pos_dev.
void rope_kv_decode(float* q, float* k, const float* v, void* kc, void* vc, const int* pos_dev, int n_heads, int n_kv,
                    int hd, float theta, float freq_scale, int max_seq, cudaStream_t s);
// Embedding-row gather + dequant on the GPU (reference does this on the CPU, transformer.cpp:419-599).
void embed_rows(float* out, const void* table, DType dt, const int* tokens_dev, int n_tokens, int hidden, cudaStream_t s);

// sample.cu: repeat penalty (in place on the logits) + temperature + top-k + top-p + inverse-CDF draw with the host-supplied
// uniform variate r; the sampled token id goes to out_dev[0].  Returns false (nothing launched) unless 0 < top_k <= 1024 < n
// and temperature > 0 — the caller then samples on the host like the reference (sampler.cpp:47-117).
bool sample_topk_supported(int n, float temperature, int top_k);
bool sample_topk(float* logits_dev, int n, float temperature, int top_k, float top_p, float repeat_penalty, const int* recent_dev,
                 int n_recent, float r, int* out_dev, cudaStream_t s);

// ---- dense.cu / attention_window.cu: kernels of the layer-spec model families (dense F32 / F16 / BF16 weights, F32 activations) ----
enum DenseEpilogue { DENSE_STORE = 0, DENSE_ADD = 1, DENSE_SCALED_ADD = 2 /* y[r] += alpha * row_scale[r] * (W.x)[r]; row_scale may be null */,
                     DENSE_SWIGLU = 3 /* y0 = silu(W0.x) * (W1.x) */, DENSE_GEGLU = 4 /* y0 = gelu_tanh(W0.x) * (W1.x) */,
                     DENSE_STREAMS = 5 /* one matrix; its output enters the residual streams: StreamsIO::X_out, y is not written */,
                     DENSE_REGLU = 6 /* y0 = relu(W0.x) * (W1.x) */ };
constexpr int DENSE_MAX_MATS = 12;      // matrices of one gemv_dense launch
// Residual streams [S, n] of ONE token folded into a GEMV (decode).  Prologue (X_in given): the activation vector is
// x[i] = sum_s a[s] * X_in[s * K + i] (a == null: the plain sum) instead of the x argument.  Epilogue DENSE_STREAMS: with v = (W.x)[r],
// X_out[t * N + r] <- sum_s M[s * S + t] * X_out[s * N + r] + b[t] * v for every t (row r is owned by one warp, so the update is race-free).
struct StreamsIO {
    const float* X_in = nullptr; const float* a = nullptr;
    float* X_out = nullptr; const float* M = nullptr; const float* b = nullptr;
    int S = 0;
};
bool dense_dtype(DType dt);
// Up to DENSE_MAX_MATS matrices of one dense dtype sharing the activation vector x[K] (GemvMat::y: each matrix's output rows).
// norm_w: the kernel's prologue first replaces x by x / sqrt(mean(x^2) + eps) * norm_w (the block's RMS norm, recomputed per CTA).
void gemv_dense(const GemvMat* mats, int n_mat, int K, const float* x, DenseEpilogue ep, const float* row_scale, float alpha, cudaStream_t s,
                const float* norm_w = nullptr, float eps = 0.f, const StreamsIO* sio = nullptr);
// C[T,N] (ep)= A[T,K] . W[N,K]^T in true FP32 on CUDA cores (store / add / scaled-add; row_scale indexes N).
void gemm_dense(float* C, const float* A, const void* W, DType dt, size_t row_pitch, int T, int N, int K, DenseEpilogue ep,
                const float* row_scale, float alpha, cudaStream_t s);
void glu_mul(float* out, const float* gate, const float* up, size_t n, bool gelu, cudaStream_t s, bool relu = false);      // out = act(gate) * up (SiLU, tanh-GELU or ReLU)
void scaled_add_rows(float* x, const float* y, const float* row_scale, float alpha, int rows, int cols, cudaStream_t s);   // x[r,c] += alpha * row_scale[c] * y[r,c]
void dense_to_f32(float* out, const void* in, DType dt, size_t n, cudaStream_t s);
void copy_cols(float* out, const float* in, int rows, int cols, int ld, cudaStream_t s);      // out [rows, cols] = the first cols columns of in [rows, ld]
struct WindowAttn {
    int heads = 0, kv_heads = 0, dim = 0, vdim = 0;
    int window = 0, keep = 0;          // window == 0: full causal
    float scale = 1.f, softcap = 0.f;  // softcap == 0: none
    int chunk = 0;                     // > 0 (instead of a window): key j visible from i iff j <= i and j / chunk == i / chunk
    int maps = 1;                      // score maps per head: Q rows are [heads][maps][dim], key rows [kv_heads][maps][dim], values [kv_heads][vdim];
                                       // every map is an attention of its own over the head's values; out [tokens, heads*maps*vdim]
    int k_stride = 0, v_stride = 0;    // elements between consecutive positions' key / value rows; 0: packed (kv_heads*maps*dim, kv_heads*vdim).
                                       // With strides the two caches may be one buffer (values = a slice of the key rows: latent attention)
    const float* sink = nullptr;       // [heads] (device): exp(sink[h]) joins head h's softmax denominator; it has no key and no value
    int joint_v = 0;                   // 1: every query head sums ONE value row per key, vdim wide, at the start of the key's value row (whatever its
                                       // key head): with vdim = kv_heads * (a head's width) each head's weights are applied to every value head at once
};
// Q [tokens, heads*dim] at positions base.. (base = *pos_dev when pos_dev is given, else p0); caches [max_seq, kv_heads*dim|vdim] of
// cache_dt (F32 or BF16) that already hold the rows of these tokens; out [tokens, heads*vdim].
// max_seq: rows of the cache (the tiled tensor-core form clamps its tile loads to it); prompts of >= 16 tokens over a BF16 cache
// with dim == vdim in {64, 128} take attention_prefill_mma.cu's tiles, everything else one CTA per (token, head).
void attention_window(float* out, const float* Q, const void* kc, const void* vc, DType cache_dt, int tokens, const int* pos_dev, int p0,
                      int max_seq, const WindowAttn& a, cudaStream_t s);
bool attention_window_mma_supported(int tokens, const WindowAttn& a, DType cache_dt);
void attention_window_mma(float* out, const float* Q, const void* kc, const void* vc, int tokens, int p0, int max_seq, const WindowAttn& a,
                          cudaStream_t s);
// Whole-projection RMS norm of the query rows (in place) and key rows (gains may be null: no norm), key/value rows -> cache rows base + t.
void qk_norm_kv_write(float* Q, const float* K, const float* V, const float* q_gain, const float* k_gain, float eps, void* kc, void* vc,
                      DType cache_dt, int tokens, const int* pos_dev, int p0, int qdim, int kdim, int vdim, cudaStream_t s);

// ---- rotary.cu / streams.cu / moe.cu: mechanisms of the layer-spec families beyond the first one ----
// Rotary positions on the first `dims` channels of every `dim`-wide head of the query rows (in place) and key rows, then key / value
// rows -> cache rows base + t.  freq: dims/2 angular frequencies (F32, device), mag multiplies cos and sin; pairs (2i, 2i+1) when
// interleaved, else (i, i + dims/2).  K == nullptr: only the queries are rotated (a layer that reads another layer's cache).
// Host: the dims/2 angular frequencies base^(-2i/dims) of a rotary layer, blended for long contexts when factor > 0 (see
// engine/layer_spec.h RotarySpec), computed in double; returns the multiplier of cos and sin.
float rotary_table(float* freq_host, int dims, float base, float factor, float original, float fast, float slow);
void rope_partial_kv_write(float* Q, const float* K, const float* V, const float* freq, float mag, int dims, bool interleaved, int dim,
                           void* kc, void* vc, DType cache_dt, int tokens, const int* pos_dev, int p0, int qdim, int kdim, int vdim, cudaStream_t s);
// Differential combination of two attention maps: A [tokens, heads, 2, vdim] -> out [tokens, heads * vdim],
// o = a1 - lambda * a2, out = o / sqrt(mean(o^2) + eps) * (1 - diff), lambda = exp(<lq1, lk1>) - exp(<lq2, lk2>) + diff (vectors of n_l).
void diff_combine(float* out, const float* A, const float* lq1, const float* lk1, const float* lq2, const float* lk2, int n_l, float diff,
                  float eps, int tokens, int heads, int vdim, cudaStream_t s);
// Residual streams X [tokens, S, width].  spread: every stream <- scale * e.  read: u = sum_s a[s] X[s] (a == null: all ones).
// write: X'[t] = sum_s M[s * S + t] X[s] + b[t] * y for all t at once.
void streams_spread(float* X, const float* e, float scale, int tokens, int S, int width, cudaStream_t s);
void streams_read(float* u, const float* X, const float* a, int tokens, int S, int width, cudaStream_t s);
void streams_write(float* X, const float* y, const float* M, const float* b, int tokens, int S, int width, cudaStream_t s);
void scale_rows(float* x, float scale, size_t n, cudaStream_t s);
// Mixture of experts.  h [tokens, width] F32 (already normed where the block norms).  Squared-ReLU experts W_down relu(W_up h)^2, or —
// `gate` given — gated experts W_down (silu(W_gate h) * W_up h).
struct MoeWeights {
    const float* router = nullptr;       // [experts, width] F32
    const float* shared_gate = nullptr;  // [width] F32 or null
    const void* const* up = nullptr;     // device table [experts] of [ff, width] rows
    const void* const* down = nullptr;   // device table [experts] of [width, ff] rows
    const void* shared_up = nullptr;     // [shared_ff, width] / [width, shared_ff] of the same dtype, or null: the decode kernels
    const void* shared_down = nullptr;   //   run the shared expert as one more slot
    DType dtype = DType::BF16;           // of the expert matrices
    int experts = 0, top = 0, ff = 0, width = 0, shared_ff = 0;
    const void* const* gate = nullptr;   // device table [experts] of [ff, width] rows: the experts are gated units
    // How the router chooses and weights (engine/layer_spec.h RouteSpec).  sigmoid: score = sigmoid(logit), weight = the chosen experts'
    // scores as they are; else softmax over the chosen logits.  correction [experts]: added to the scores for the choice only.
    // groups > 0: only experts of the `keep` runs of neighbours with the largest sum of their two largest choice scores can be chosen.
    bool sigmoid = false;
    const float* correction = nullptr;
    int groups = 0, keep = 0;
};
// Router: logits in F32, the `top` largest (lowest index on ties), softmax over the chosen -> sel [tokens, top], wt [tokens, top];
// sgate [tokens] = sigmoid(<shared_gate, h>) when shared_gate is given.
// sio->X_in: the token's input is the blend of its residual streams ([tokens, S, width]) instead of h; norm_w: it is RMS-normalised
// (times norm_w) first; h_out: the vector the router saw is written there for the expert kernels.
void moe_route(int* sel, float* wt, float* sgate, const float* h, const MoeWeights& w, int tokens, cudaStream_t s,
               const StreamsIO* sio = nullptr, const float* norm_w = nullptr, float eps = 0.f, float* h_out = nullptr);
// One token (decode): act [top * ff + shared_ff] = relu(W_up[sel] h)^2 ; y [width] = sum_k wt[k] * W_down[sel[k]] act[k] + sgate * shared part.
void moe_expert_up_token(float* act, const float* h, const int* sel, const MoeWeights& w, cudaStream_t s);
// sio->X_out: the result enters the residual streams (StreamsIO) instead of y.
void moe_expert_down_token(float* y, const float* act, const int* sel, const float* wt, const float* sgate, const float* shared_y,
                           const MoeWeights& w, cudaStream_t s, const StreamsIO* sio = nullptr);
// Prompt rows: assignments grouped per expert (order inside an expert = token order), gathered GEMMs on CUDA cores in F32.
//   work: ints [experts + 1 (offsets) + tokens*top (row -> token) + tokens*top (assignment -> row)]
size_t moe_work_ints(int tokens, int experts, int top);
void moe_group(int* work, const int* sel, int tokens, int experts, int top, cudaStream_t s);
// [tokens*top, ff]: relu(W_up h)^2, or for gated experts the plain W_up h; moe_expert_gate_rows: W_gate h (combine with glu_bias_mul)
void moe_expert_up_rows(float* act_rows, const float* h, const int* work, const MoeWeights& w, int tokens, cudaStream_t s);
void moe_expert_gate_rows(float* gate_rows, const float* h, const int* work, const MoeWeights& w, int tokens, cudaStream_t s);
void moe_expert_down_rows(float* y_rows, const float* act_rows, const int* work, const MoeWeights& w, int tokens, cudaStream_t s); // [tokens*top, width]
// y [tokens, width] = sum_k wt[t, k] * y_rows[row(t, k)] (+ sgate[t] * shared_y[t])
void moe_combine(float* y, const float* y_rows, const int* work, const float* wt, const float* sgate, const float* shared_y, int tokens,
                 int experts, int top, int width, cudaStream_t s);
// h rows in the grouped order (the tensor-core path splits them per expert): out [tokens*top, width]
void moe_gather_rows(float* out, const float* h, const int* work, int tokens, int experts, int top, int width, cudaStream_t s);
void relu2(float* x, size_t n, cudaStream_t s);

// ---- attention_latent.cu / ssm_scan.cu / postnorm.cu: mechanisms added with the third layer-spec family ----
// Latent attention (engine/layer_spec.h LatentSpec).  cq [T, q_rank]: RMS-normed in place (gain).  dkv [T, kv_rank + rot_dim] (null: the layer
// reads another layer's rows): [RMS-normed first part | rotated rest] -> cache row base + t of `cache` ([max_seq, kv_rank + rot_dim]).
void latent_prep(float* cq, int q_rank, const float* q_gain, const float* dkv, int kv_rank, int rot_dim, const float* kv_gain, float eps, void* cache,
                 DType cache_dt, int rot_dims, bool interleaved, float rot_base, int T, const int* pos_dev, int p0, cudaStream_t s);
// q [T, heads, dim + rot_dim] -> qa [T, heads, kv_rank + rot_dim] = [W_uk,h^T q_unrotated | rot(q_rotated)];  W_uk [heads * dim, kv_rank]
void latent_q_absorb(float* qa, const float* q, const void* W_uk, DType dt, int T, int heads, int dim, int rot_dim, int kv_rank, int rot_dims,
                     bool interleaved, float rot_base, const int* pos_dev, int p0, cudaStream_t s);
// ol [T, heads, kv_rank] -> out [T, heads * vdim] = W_uv,h ol_h;  W_uv [heads * vdim, kv_rank]
void latent_v_up(float* out, const float* ol, const void* W_uv, DType dt, int T, int heads, int vdim, int kv_rank, cudaStream_t s);
// Prompt portions: F32 latents of cache rows r0.. (input of the two up-projection GEMMs); their results packed with the rotated key part
// into 16-bit per-head operands kfull [row, heads, kw] / vfull [row, heads, vw] (zero padded); queries rotated and padded to kw; the
// padded outputs [T, heads, vw] back to [T, heads * vdim].
void latent_rows_f32(float* out, const void* cache, DType cache_dt, int row, int kv_rank, int r0, int n, cudaStream_t s);
void latent_expand_pack(void* kfull, void* vfull, const float* ku, const float* vu, const void* cache, DType cache_dt, int kv_rank, int r0, int n, int heads,
                        int dim, int rot_dim, int vdim, int kw, int vw, cudaStream_t s);
void latent_q_rot_pad(float* qp, const float* q, int T, int heads, int dim, int rot_dim, int kw, int rot_dims, bool interleaved, float rot_base, int p0,
                      cudaStream_t s);
void latent_unpad(float* out, const float* o, int T, int heads, int vdim, int vw, cudaStream_t s);
// Attention of a few queries over ONE key / value head stored as rows (keys: the first dim numbers of a row, values: the first vdim),
// every head served from one shared-memory copy of the rows; key slices merged by a second launch.  Full causal mask.
bool attention_shared_rows_supported(int heads, int dim, int vdim, int row, DType cache_dt, const void* cache);
size_t attention_shared_rows_scratch_floats(int heads, int vdim);
void attention_shared_rows(float* out, const float* Q, const void* cache, DType cache_dt, int tokens, const int* pos_dev, int p0, int max_seq, int heads, int dim,
                           int vdim, int row, float scale, float* scratch, cudaStream_t s);
// attention_prefill_mma.cu: full causal attention of `tokens` queries [tokens, heads, kw] at positions p0.. over BF16 per-head keys
// [rows, heads, kw] and values [rows, heads, vw]; (kw, vw) from attention_heads_mma_widths.  out [tokens, heads, vw].
bool attention_heads_mma_widths(int key_dim, int value_dim, int* kw, int* vw);
void attention_heads_mma(float* out, const float* Q, const void* k, const void* v, int tokens, int p0, int rows, int heads, int kw, int vw, float scale,
                         cudaStream_t s);
// State-space scan (ScanSpec).  u [T, ld]: the input projection's rows; channels of interest start at a column offset.
// conv_state [taps - 1, ch], state [heads, vdim, N]: the sequence's state, read unless the step starts at position 0, updated in place.
void ssm_conv(float* out, const float* u, int ld, int col0, float* conv_state, const float* w, const float* b, int T, int ch, int taps,
              const int* pos_dev, int p0, cudaStream_t s);
void ssm_scan(float* y, const float* xbc, const float* u, int ld, int dt_col0, float* state, const float* dt_bias, const float* A_log, const float* D,
              int T, int heads, int vdim, int N, int groups, const int* pos_dev, int p0, cudaStream_t s);
void ssm_gate_norm(float* out, const float* y, const float* u, int ld, int z_col0, const float* gain, float eps, int T, int inner, int norm_groups,
                   cudaStream_t s);
// Post-norm block form: x[t] += rms(y[t] + bias) * gain;  out = act(gate + b_g) * (up + b_u);  g[t, j] <- gelu_tanh(g[t, j]) * E[token_t, col0 + j]
void add_rmsnorm_rows(float* x, const float* y, const float* gain, const float* bias, int rows, int width, float eps, cudaStream_t s);
void glu_bias_mul(float* out, const float* gate, const float* up, const float* gate_bias, const float* up_bias, int rows, int cols, bool gelu, cudaStream_t s);
void side_gate_rows(float* g, const void* E, DType dt, int e_cols, int col0, const int* tokens_dev, int rows, int dim, cudaStream_t s);

// ---- short_conv.cu / delta_rule.cu / sumnorm.cu / attention_heads.cu: mechanisms added with the fourth layer-spec family ----
// Short causal convolutions on projected rows, several projections ("segments") per launch.  u [T, ld], channel c at column col0 + c;
// out [T, out_ld] (not the rows it reads); w [ch, taps], the last tap is the current token's; in_bias [ch] or null is added to every input
// row (zeros before the sequence's start stay zeros); state [taps - 1, ch]: the sequence's last inputs, read unless the step starts at
// position 0, rewritten with the step's last inputs; act: 0 none, 1 SiLU.
struct ConvSeg {
    const float* u = nullptr; int ld = 0, col0 = 0;
    float* out = nullptr; int out_ld = 0;
    int ch = 0, taps = 0;
    const float* w = nullptr; const float* in_bias = nullptr;
    float* state = nullptr;
    int act = 0;
};
constexpr int SHORT_CONV_MAX_SEGS = 6;
void short_conv(const ConvSeg* segs, int n, int T, const int* pos_dev, int p0, cudaStream_t s);
// Gated delta rule (engine/layer_spec.h DeltaSpec).  prep, in place: q, k [T, kv_heads, dim] to unit length per head (q also times dim^-1/2);
// a [T, heads, dim] <- exp(-exp(A_log_h) softplus(a + dt_bias)); beta [T, heads] <- sigmoid(beta); qk [T, kv_heads] = <q, k>.
// rows: out [T, heads, vdim] from the recurrence over the step's rows; state [heads, vdim, dim] is read unless the step starts at
// position 0 and written back.  gate_norm: out = o / sqrt(mean_v o^2 + eps) * gain[v] * sigmoid(gate_raw), per head.
constexpr int DELTA_MAX_DIM = 256;
void delta_prep(float* q, float* k, float* a, float* beta, float* qk, const float* dt_bias, const float* A_log, int T, int heads, int kv_heads, int dim,
                cudaStream_t s);
void delta_rule_rows(float* out, const float* q, const float* k, const float* v, const float* a, const float* beta, const float* qk, float* state, int T,
                     int heads, int kv_heads, int dim, int vdim, const int* pos_dev, int p0, cudaStream_t s);
void delta_gate_norm(float* out, const float* o, const float* gate_raw, const float* gain, float eps, int T, int heads, int vdim, cudaStream_t s);
// Block form that norms the residual sum: x[t] <- rms(a x[t] + s1 (y1[t] + b1) + s2 y2[t]) * gain (y2, b1 may be null).  h_next (one row
// only): also the next mixer's shifted input h = x' + (carried - x') mu, after which x' becomes the carried row.
void sum_rmsnorm_rows(float* x, float a, const float* y1, float s1, const float* b1, const float* y2, float s2, const float* gain, int rows, int width, float eps,
                      cudaStream_t s, float* h_next = nullptr, const float* mu = nullptr, float* carried = nullptr, const int* pos_dev = nullptr, int p0 = 0);
// Token shift: h[t] = x[t] + (x[t-1] - x[t]) mu; x[-1] is the carried row (zeros when the step starts at position 0), which then becomes the step's last row.
void token_shift_rows(float* h, const float* x, const float* mu, float* carried, int rows, int width, const int* pos_dev, int p0, cudaStream_t s);
// Per-head query / key norm, rotation from a frequency table, per-head query multiplier, value blend, cache write (attention_heads.cu).
struct HeadPrep {
    int heads = 0, kv_heads = 0, dim = 0, vdim = 0;
    const float* q_gain = nullptr; const float* k_gain = nullptr; float eps = 0.f;      // [dim] each; null: no norm
    int rot_dims = 0, interleaved = 0; const float* freq = nullptr;                      // [rot_dims / 2] angular frequencies (device)
    const float* temp = nullptr;            // [heads] or null
    const float* v_lambda = nullptr;        // one number (device); used with v_first
    const float* v_first = nullptr;         // [T, kv_heads * vdim] F32 or null
    float* v_publish = nullptr;             // [T, kv_heads * vdim] F32 or null: receives the values as projected
};
void head_prep(float* Q, const float* K, const float* V, const HeadPrep& p, void* kc, void* vc, DType cache_dt, int tokens, const int* pos_dev, int p0,
               cudaStream_t s);
// out [T, heads, vdim] = sum_g M[h, g] A(t, g, kv(h), :), A addressed as A + t * t_stride + g * g_stride + c * c_stride.
void talk_mix(float* out, const float* A, const float* M, int tokens, int heads, int kv_heads, int vdim, size_t t_stride, size_t g_stride, size_t c_stride,
              cudaStream_t s);

// Programmatic dependent launch (PDL): when enabled, kernels are launched with
// cudaLaunchAttributeProgrammaticStreamSerialization so that a kernel's prologue (barrier init, TMA weight
// prefetch) overlaps the tail of its predecessor; every kernel executes griddepcontrol.wait before it touches
// data produced upstream, so ordering is unchanged.  Off by default; the engine turns it on for decode graphs.
void set_pdl(bool on);
bool pdl_enabled();
template <typename... KArgs, typename... Args>
inline void launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = at; cfg.numAttrs = 1;
    NT_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
}

// prefill_gemm.cu: tcgen05/TMEM GEMM, C[M,N] = A[M,K] (F32, split hi+lo F16) . W[N,K]^T (F16)
size_t gemm_f16_tc_workspace_bytes(int M, int K);
bool gemm_f16_tc(float* C, const float* A, const void* W_f16, int M, int N, int K, void* workspace, cudaStream_t s);
bool gemm_f16_tc_supported(const void* W_f16, int N, int K, size_t row_pitch);
bool gemm_f16_tc_ragged_supported(const void* W_f16, int N, int K, size_t row_pitch);   // gemm_f16_tc_ws alone: N >= 128, N % 4 == 0
// Variants of the tensor-core GEMM: bf16 — weights and the activation split are BF16 (safetensors families; the same 16-bit
// layouts, only the MMA's operand format changes); gelu — the gated epilogue uses tanh-GELU instead of SiLU; col_scale / alpha —
// the store / add epilogue writes C (+)= alpha * col_scale[n] * (A.W^T) (per-channel layer scale and residual multiplier).
struct TcOpts { bool bf16 = false; bool gelu = false; const float* col_scale = nullptr; float alpha = 1.0f; bool relu = false; /* gated epilogue: ReLU gate */ };
void split_activations(void* workspace, const float* A, int M, int K, cudaStream_t s, bool bf16 = false);
bool gemm_f16_tc_ws(float* C, const void* workspace, const void* W_f16, int M, int N, int K, bool add, cudaStream_t s, const TcOpts& o = TcOpts());
// workspace_out <- split(silu(A.Wgate^T) * (A.Wup^T)): the FFN's gate/up GEMMs with the SwiGLU + split fused in the epilogue
bool gemm_f16_tc_swiglu_ws(void* workspace_out, const void* workspace_in, const void* Wgate_f16, const void* Wup_f16, int M, int N, int K,
                           cudaStream_t s, const TcOpts& o = TcOpts());
void rmsnorm_split(void* workspace, const float* x, const float* w, int rows, int hidden, float eps, cudaStream_t s, bool bf16 = false);
// prefill_dequant.cu: any GGUF weight matrix -> dense F16 pair with W = w_hi + w_lo (operands of two tensor-core GEMMs)
bool dequant_split_supported(DType dt);
void dequant_split(void* w_hi, void* w_lo, const void* W, DType dt, size_t row_pitch, int rows, int cols, cudaStream_t s);

// Opt-in to > 48 KB of dynamic shared memory.  The attribute is per DEVICE, so the "already done" state is a bit per device
// id (a process that drives a second GPU must opt in there too).  `done` is the call site's static mask.
template <typename K>
inline void opt_in_dynamic_smem(K* kernel, int bytes, unsigned long long& done) {
    int dev = 0;
    NT_CUDA_CHECK(cudaGetDevice(&dev));
    const unsigned long long bit = 1ull << (dev & 63);
    if (done & bit) return;
    NT_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    done |= bit;
}
// After a raw <<<>>> launch: a rejected configuration must not pass silently.
#define NT_LAUNCH_CHECK() NT_CUDA_CHECK(cudaPeekAtLastError())

// Number of kernels launched by this library since load (bench.py's gpu_launches claim).
unsigned long long launch_count();
void count_launch(int n = 1);

}}  // namespace nt::b200
