/*
 * nt_b200_engine.h — token-level C-ABI of the resident model (additions to include/ntransformer.h).
 *
 * Mirrors the reference's C++ surface nt::Transformer::{load,forward,config} (src/model/transformer.h:31-61,
 * forward = src/model/transformer.cpp:604-669): tokens in (HOST int32), logits out (HOST or DEVICE float32
 * [vocab]).  Weights come either from a GGUF file or from caller-owned device tensors in GGUF block layout
 * (synthetic benchmarks); tensor names are the reference's GGUF names (transformer.cpp:89-104, 286-322).
 * Tensor parallelism (new; the reference is single GPU): one process per GPU, ranks exchange a 128-byte
 * NCCL id through their own plumbing and call nt_tp_init before the first forward.
 */
#ifndef NT_B200_ENGINE_H
#define NT_B200_ENGINE_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
    int vocab_size, hidden_size, intermediate_size, n_layers, n_heads, n_kv_heads, head_dim, max_seq_len;
    float norm_eps, rope_theta;
    int bos_token_id, eos_token_id;
} nt_model_config;

typedef void* nt_model_t;

/* GGUF path: returns NULL on failure.  max_context caps llama.context_length like the CLI's -c. */
nt_model_t nt_model_load_gguf(const char* path, int max_context, int tp_rank, int tp_size);
/* Device-pointer path: create -> set_tensor (every tensor, shapes already sharded for the rank) -> finalize */
nt_model_t nt_model_create(const nt_model_config* cfg, int tp_rank, int tp_size);
int  nt_model_set_tensor(nt_model_t m, const char* gguf_name, const void* dev_ptr, int dtype, size_t row_pitch);
int  nt_model_finalize(nt_model_t m);
void nt_model_free(nt_model_t m);
int  nt_model_get_config(nt_model_t m, nt_model_config* out);

/* Model folders (config.json + model.safetensors) of a registered layer-spec family; exact_f32: everything in true 32-bit. */
nt_model_t nt_model_load_dir(const char* dir, int max_context, int exact_f32);
/* Host only: validates <dir>/config.json and model.safetensors against each other; text summary (or the reason, with -1) in out. */
int  nt_model_dir_describe(const char* dir, char* out, size_t cap);
/* The same family from a config.json TEXT and caller-owned device tensors: create_json -> set_tensor (checkpoint names; matrices
 * F32 / F16 / BF16 row-major, gain vectors F32) -> finalize. */
nt_model_t nt_model_create_json(const char* config_json, int max_context, int exact_f32);
/* forward + the logits at the wanted places (ascending indices into the tokens) -> logits_host [n_want, vocab] */
int  nt_model_forward_logits(nt_model_t m, const int* tokens_host, int seq_len, int start_pos, const int* want, int n_want, float* logits_host);
/* Engine: load a GGUF file or a model folder; generate over token ids (returns the number generated, ids in out_ids[0..cap)) */
int  nt_engine_load_path(void* engine, const char* path, int max_context, int exact_f32);
int  nt_engine_generate_ids(void* engine, const int* prompt_ids, int n_prompt, int max_tokens, float temperature, int top_k, float top_p,
                            float repeat_penalty, unsigned long long seed, int* out_ids, int cap);
/* Kernels of the layer-spec mechanisms (numerics tests): epilogue 0 store, 1 add, 2 y += alpha * row_scale * Wx, 3 SiLU gate, 4 GELU gate */
void nt_b200_gemv_dense(float* y0, float* y1, float* y2, const void* W0, const void* W1, const void* W2, int out0, int out1, int out2, int n_mat, int K,
                        const float* x, int dtype, int epilogue, const float* row_scale, float alpha, void* stream);
void nt_b200_gemm_dense(float* C, const float* A, const void* W, int dtype, int T, int N, int K, int epilogue, const float* row_scale, float alpha, void* stream);
void nt_b200_attention_window(float* out, const float* Q, const void* kc, const void* vc, int cache_dtype, int tokens, int p0, int heads, int kv_heads,
                              int dim, int vdim, int window, int keep, float scale, float softcap, int max_seq, void* stream);
void nt_b200_qk_norm_kv_write(float* Q, const float* K, const float* V, const float* q_gain, const float* k_gain, float eps, void* kc, void* vc,
                              int cache_dtype, int tokens, int p0, int qdim, int kdim, int vdim, void* stream);
void nt_b200_glu_mul(float* out, const float* gate, const float* up, long long n, int gelu, void* stream);
/* Attention with `maps` score maps per head (Q rows [heads][maps][dim], key rows [kv_heads][maps][dim], one value row per kv head) and a
 * block-local causal mask (chunk > 0: j visible from i iff j <= i and j / chunk == i / chunk); out [tokens, heads * maps * vdim] */
void nt_b200_attention_maps(float* out, const float* Q, const void* kc, const void* vc, int cache_dtype, int tokens, int p0, int heads, int kv_heads,
                            int dim, int vdim, int chunk, int maps, float scale, int max_seq, void* stream);
/* host: dims/2 angular frequencies (long-context blend when factor > 0); returns the multiplier of cos and sin */
float nt_b200_rotary_table(float* freq_host, int dims, float base, float factor, float original, float fast, float slow);
void nt_b200_rope_partial_kv_write(float* Q, const float* K, const float* V, const float* freq, float mag, int dims, int interleaved, int dim, void* kc,
                                   void* vc, int cache_dtype, int tokens, int p0, int qdim, int kdim, int vdim, void* stream);
void nt_b200_diff_combine(float* out, const float* A, const float* lq1, const float* lk1, const float* lq2, const float* lk2, int n_l, float diff, float eps,
                          int tokens, int heads, int vdim, void* stream);
/* residual streams X [tokens, S, width] */
void nt_b200_streams_spread(float* X, const float* e, float scale, int tokens, int S, int width, void* stream);
void nt_b200_streams_read(float* u, const float* X, const float* a, int tokens, int S, int width, void* stream);
void nt_b200_streams_write(float* X, const float* y, const float* M, const float* b, int tokens, int S, int width, void* stream);
/* mixture of squared-ReLU experts: router (F32 rows) -> sel / wt [tokens, top], sgate [tokens]; experts through device pointer tables */
void nt_b200_moe_route(int* sel, float* wt, float* sgate, const float* h, const float* router, const float* shared_gate, int experts, int top, int width,
                       int tokens, void* stream);
void nt_b200_moe_experts(float* y, const float* h, const int* sel, const float* wt, const float* sgate, const void* const* up_tab, const void* const* down_tab,
                         const void* shared_up, const void* shared_down, const float* shared_y, int dtype, int experts, int top, int ff, int width,
                         int shared_ff, int tokens, int mode, void* scratch, void* stream);

/* latent attention: cache rows [normed latent : kv_rank | rotated key part : rot_dim]; the query side absorbs the per-head key up-projection */
void nt_b200_latent_prep(float* cq, int q_rank, const float* q_gain, const float* dkv, int kv_rank, int rot_dim, const float* kv_gain, float eps, void* cache,
                         int cache_dtype, int rot_dims, int interleaved, float rot_base, int tokens, int p0, void* stream);
void nt_b200_latent_q_absorb(float* qa, const float* q, const void* W_uk, int dtype, int tokens, int heads, int dim, int rot_dim, int kv_rank, int rot_dims,
                             int interleaved, float rot_base, int p0, void* stream);
void nt_b200_latent_v_up(float* out, const float* ol, const void* W_uv, int dtype, int tokens, int heads, int vdim, int kv_rank, void* stream);
/* prompt portions (16 tokens or more, BF16 cache rows): per-head keys / values expanded once, then tiled tensor-core attention; -1: widths not covered */
int nt_b200_latent_attention_expanded(float* out, const float* q, const void* cache, const void* W_uk, const void* W_uv, int dtype, int tokens, int p0, int heads,
                                      int dim, int rot_dim, int vdim, int kv_rank, int rot_dims, int interleaved, float rot_base, float scale, void* stream);
/* full causal attention over ONE key / value head stored as rows of `row` numbers: keys the first dim, values the first vdim of a row */
void nt_b200_attention_rows(float* out, const float* Q, const void* cache, int cache_dtype, int tokens, int p0, int heads, int dim, int vdim, int row, float scale,
                            int max_seq, void* stream);
/* the same with all heads served from one shared-memory copy of the rows; -1: shape not covered (dim, row multiples of 16 bytes, heads <= 32, even vdim <= 512) */
int nt_b200_attention_rows_shared(float* out, const float* Q, const void* cache, int cache_dtype, int tokens, int p0, int heads, int dim, int vdim, int row, float scale,
                                  int max_seq, void* stream);
/* state-space scan: causal convolution + SiLU with a carried state, the recurrence with a carried state, gate + grouped RMS norm */
void nt_b200_ssm_conv(float* out, const float* u, int ld, int col0, float* conv_state, const float* w, const float* b, int tokens, int ch, int taps, int p0, void* stream);
void nt_b200_ssm_scan(float* y, const float* xbc, const float* u, int ld, int dt_col0, float* state, const float* dt_bias, const float* A_log, const float* D,
                      int tokens, int heads, int vdim, int N, int groups, int p0, void* stream);
void nt_b200_ssm_gate_norm(float* out, const float* y, const float* u, int ld, int z_col0, const float* gain, float eps, int tokens, int inner, int norm_groups,
                           void* stream);
/* post-norm block: x += rms(y + bias) * gain; out = act(gate + b_g) * (up + b_u); g <- gelu_tanh(g) * E[token, col0 + j] */
void nt_b200_add_rmsnorm_rows(float* x, const float* y, const float* gain, const float* bias, int rows, int width, float eps, void* stream);
void nt_b200_glu_bias_mul(float* out, const float* gate, const float* up, const float* gate_bias, const float* up_bias, int rows, int cols, int gelu, void* stream);
void nt_b200_side_gate_rows(float* g, const void* E, int dtype, int e_cols, int col0, const int* tokens_dev, int rows, int dim, void* stream);
/* Kernels of the block that norms the residual sum, short convolutions with carried inputs, the gated delta rule, attention with per-head
 * norm / sink / head-mixed weights (numerics tests).  Optional pointers may be null. */
void nt_b200_short_conv(const void* const* u, void* const* out, const void* const* w, const void* const* in_bias, void* const* state, const int* ch, const int* taps,
                        const int* act, int n_seg, int tokens, int p0, void* stream);
void nt_b200_delta_prep(float* q, float* k, float* a, float* beta, float* qk, const float* dt_bias, const float* A_log, int tokens, int heads, int kv_heads, int dim,
                        void* stream);
void nt_b200_delta_rule_rows(float* out, const float* q, const float* k, const float* v, const float* a, const float* beta, const float* qk, float* state, int tokens,
                             int heads, int kv_heads, int dim, int vdim, int p0, void* stream);
void nt_b200_delta_gate_norm(float* out, const float* o, const float* gate_raw, const float* gain, float eps, int tokens, int heads, int vdim, void* stream);
void nt_b200_sum_rmsnorm_rows(float* x, float a, const float* y1, float s1, const float* b1, const float* y2, float s2, const float* gain, int rows, int width, float eps,
                              float* h_next, const float* mu, float* carried, int p0, void* stream);
void nt_b200_token_shift_rows(float* h, const float* x, const float* mu, float* carried, int rows, int width, int p0, void* stream);
void nt_b200_head_prep(float* Q, const float* K, const float* V, int heads, int kv_heads, int dim, int vdim, const float* q_gain, const float* k_gain, float eps,
                       int rot_dims, int interleaved, const float* freq, const float* temp, const float* v_lambda, const float* v_first, float* v_publish, void* kc,
                       void* vc, int cache_dtype, int tokens, int p0, void* stream);
void nt_b200_attention_heads(float* out, const float* Q, const void* kc, const void* vc, int cache_dtype, int tokens, int p0, int max_seq, int heads, int kv_heads,
                             int dim, int vdim, float scale, const float* sink, const float* talk, float* scratch, int one_pass, void* stream);
/* router with sigmoid scores, a choice-only correction and a limit to the best runs of neighbouring experts; gated experts */
void nt_b200_moe_route_scored(int* sel, float* wt, const float* h, const float* router, const float* correction, int experts, int top, int groups, int keep,
                              int width, int tokens, void* stream);
void nt_b200_moe_glu_experts(float* y, const float* h, const int* sel, const float* wt, const void* const* gate_tab, const void* const* up_tab,
                             const void* const* down_tab, int dtype, int experts, int top, int ff, int width, int tokens, int mode, void* scratch, void* stream);

/* forward(tokens[seq_len], start_pos): logits of the last token. logits_host may be NULL.  Returns 0. */
int  nt_model_forward(nt_model_t m, const int* tokens_host, int seq_len, int start_pos, float* logits_host);
/* asynchronous launch only (no sync, no copy); nt_model_sync waits for the model's stream */
int  nt_model_forward_async(nt_model_t m, const int* tokens_host, int seq_len, int start_pos);
int  nt_model_sync(nt_model_t m);
float* nt_model_logits_device(nt_model_t m);
void*  nt_model_stream(nt_model_t m);
int  nt_model_argmax(nt_model_t m);                 /* greedy token of the last logits, computed on the GPU */
void nt_model_clear_kv(nt_model_t m);
void nt_model_use_graph(nt_model_t m, int on);
/* prompts of >= n tokens use the batched tcgen05 prefill when every layer matrix is F16 and tile-aligned
 * (default 16; 0 = always replay the per-token decode step like the reference's forward loop) */
void nt_model_set_prefill_min_tokens(nt_model_t m, int n);
/* algorithmic bytes read per decoded token by this rank at context length ctx */
unsigned long long nt_model_bytes_per_token(nt_model_t m, int ctx);

/* Samples the next token from the last logits ON THE GPU: repeat penalty over recent_window (host ids, oldest first; applied in
 * place to the device logits), temperature, top-k, top-p and the inverse-CDF draw with the uniform variate r — the steps of the
 * reference's Sampler::apply_repeat_penalty + Sampler::sample (src/inference/sampler.cpp:30-117) in the same order.  Returns the
 * token id, or -1 when the settings are not covered (temperature <= 0, top_k <= 0, top_k > 1024, top_k >= vocab): sample on the
 * host then (nt_sample_token).  nt_sampler_uniform(seed, i) is the (i+1)-th variate of the reference's mt19937 stream. */
int   nt_model_sample(nt_model_t m, float temperature, int top_k, float top_p, float repeat_penalty, const int* recent_window,
                      int n_window, float r);
float nt_sampler_uniform(uint64_t seed, int n_draws_before);

/* Opt-in: run each decoded token as ONE persistent kernel (all layers; grid barriers and, under tensor parallelism,
 * NVLink peer-memory exchanges inside the kernel) instead of the CUDA graph of fused launches.  Same maths, same KV
 * cache.  Models whose shapes/dtypes the kernel does not cover keep the graph path (a note goes to stderr).
 * Also enabled by the environment variable NT_B200_MEGAKERNEL=1.  Call before the first forward. */
void nt_model_use_megakernel(nt_model_t m, int on);
/* wall-clock seconds nt_model_load_gguf took for this model (header parse + shard plan + pipelined pread -> pinned staging ->
 * cudaMemcpyAsync upload + buffer allocation); 0 for models built from device tensors.  Reference behaviour it replaces: one
 * synchronous cudaMemcpy per tensor from the pageable mmap (src/model/transformer.cpp:286-328, src/core/tensor.cpp:224-225). */
double nt_model_load_seconds(nt_model_t m);
/* how a tensor-parallel model sums the o-projection / down-projection partials: 0 not tensor parallel (or no step run yet),
 * 1 ncclAllReduce, 2 NVLink peer-memory exchange fused into the GEMV epilogue (default; NT_B200_TP_NCCL=1 selects 1) */
int  nt_model_tp_exchange(nt_model_t m);
int  nt_model_megakernel_active(nt_model_t m);      /* 1 once the persistent kernel has been built and is in use */
/* phase kinds of the persistent kernel's per-token program (0 norm+quantise, 1 quantise, 2 GEMV, 3 attention,
 * 4 combine); returns the number of phases (may exceed cap), 0 when the kernel is not active */
int  nt_model_megakernel_plan(nt_model_t m, int* kinds, int cap);
/* tuning aid: record the SM clock at every phase boundary of the persistent kernel on its first 4 CTAs; _read returns the number of
 * values (per CTA: [phases][start, work done, barrier passed] ticks, then clock start/end and %globaltimer start/end for the
 * tick -> ns conversion) of the most recent launch and copies up to cap of them */
void nt_model_megakernel_trace(nt_model_t m, int on);
long long nt_model_megakernel_trace_read(nt_model_t m, unsigned long long* out_host, size_t cap);
/* debug: copies one of the persistent kernel's working vectors ("hid0", "hid1", "q", "attn", "act", "slots") to the host;
 * returns its length in floats, -1 when unknown / not active */
long long nt_model_debug_read(nt_model_t m, const char* name, float* out_host, size_t cap);

/* Host-only self-test of the persistent kernel's plan builder: builds the per-token program for one tensor-parallel rank
 * of a model of shape *cfg (layer_dtypes: n_layers x 7 nt::DType values in the order q,k,v,o,gate,up,down) on a grid of
 * `grid` CTAs (fuse: producer-side fusion bits, 1 = activation quantiser, 2 = split combine, 4 = residual add + next norm, single rank only) and replays the schedule of every GEMV phase on the CPU.  info (8 ints, optional): phases, body phases, GEMV
 * phases, min warps, min ring stages, exchanges, attention splits, keys per split.  Returns 0 ok, 1 shape not covered,
 * 2 inconsistent plan (a bug), -1 bad arguments; msg receives the reason. */
int  nt_mega_plan_selftest(const nt_model_config* cfg, int tp_rank, int tp_size, const int* layer_dtypes, int head_dtype,
                           int grid, int split_fixed, int fuse, int* info, char* msg, size_t cap);

/* ---- host-only helpers (no GPU needed): GGUF header, tokenizer and sampler of the CLI path ---- */
/* JSON description of a GGUF file as the engine parses it (config, vocab size, tensor table). Returns the
 * number of bytes written (excluding NUL) or -1. */
int  nt_gguf_describe(const char* path, char* out, size_t cap);
int  nt_tokenize(const char* gguf_path, const char* text, int add_bos, int* ids, int cap);      /* returns count or -1 */
int  nt_detokenize(const char* gguf_path, const int* ids, int n, char* out, size_t cap);       /* returns bytes or -1 */
/* One draw of the reference-compatible sampler (repeat penalty over `recent`, temperature, top-k, top-p, mt19937(seed)). */
int  nt_sample_token(const float* logits, int n, float temperature, int top_k, float top_p, float repeat_penalty,
                     int repeat_window, const int* recent, int n_recent, uint64_t seed);

/* tensor-parallel communicator */
int  nt_tp_unique_id(void* out128);                 /* rank 0; returns 0 on success */
int  nt_tp_init(nt_model_t m, const void* id128, int rank, int size);

#ifdef __cplusplus
}
#endif
#endif
