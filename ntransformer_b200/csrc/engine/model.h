// model.h — resident Llama-family forward on one GPU (or one tensor-parallel rank).
//
// Host-side counterpart of the reference's nt::Transformer resident branch
// (src/model/transformer.cpp:59-126 load, :286-391 layers/buffers, :604-669 forward) with the per-layer
// launch sequence of Attention::forward (src/model/attention.cpp:120-211) and FFN::forward
// (src/model/ffn.cpp:85-134) re-expressed as fused sm_100a launches captured in a CUDA graph:
//   reference: 15 launches / layer / token, CPU embedding dequant, 2 sync H2D + 1 sync D2H per token;
//   here:      10 launches / layer / token in one graph replay, embedding gathered on the GPU.
// The streaming / tiered / speculative branches of the reference are out of scope.
#pragma once
#include <cuda_runtime.h>
#include <string>
#include <vector>
#include <memory>
#include "../kernels_internal.h"
#include "gguf.h"
#include "decode_mega.h"
#include "peer_xchg.h"
#include "model_registry.h"

namespace nt { namespace b200 {

class TPComm;    // NCCL communicator (engine/tp_comm.cpp); null when tp_size == 1

struct Weight {
    const void* ptr = nullptr;   // device, GGUF block layout, this rank's shard
    DType dtype = DType::F32;
    int rows = 0, cols = 0;      // shard shape (out_features, in_features)
    size_t pitch = 0;            // bytes between rows
    bool owned = false;
    // Layer-spec families: a copy of a short matrix (fewer rows than a tensor-core tile) with zero rows appended up to tc_rows, so that
    // prompt rows can take the tensor-core GEMM; the first `rows` columns of its result are the product.  Null: none.
    const void* tc_ptr = nullptr;
    int tc_rows = 0;
    size_t bytes() const { return (size_t)rows * dtype_row_size(dtype, (size_t)cols); }   // algorithmic bytes
};

struct LayerWeights {
    const float* attn_norm = nullptr;
    const float* ffn_norm = nullptr;
    Weight wq, wk, wv, wo, gate, up, down;
    // layer-spec families (engine/layer_spec.h): whole-projection query / key norm gains, per-channel branch gains (F32, may be null)
    const float* q_norm = nullptr;
    const float* k_norm = nullptr;
    const float* ls1 = nullptr;
    const float* ls2 = nullptr;
    // differential attention: the four vectors of lambda; residual streams, sublayer 0 (mixer) and 1 (feed-forward): read blend [S],
    // write gains [S], stream mixing [S, S] (from, to); all F32, null when the mechanism is off
    const float *lq1 = nullptr, *lk1 = nullptr, *lq2 = nullptr, *lk2 = nullptr;
    const float *hc_in[2] = {nullptr, nullptr}, *hc_out[2] = {nullptr, nullptr}, *hc_mix[2] = {nullptr, nullptr};
    // mixture of experts: router rows and the shared expert's gate row (F32), expert matrices, the shared expert
    const float* router = nullptr;
    const float* shared_gate = nullptr;
    std::vector<Weight> e_up, e_down;
    Weight sh_up, sh_down;
    const void** e_up_tab = nullptr;       // device tables of the experts' row pointers (the chosen expert is looked up on the device)
    const void** e_down_tab = nullptr;
    float* rot_freq = nullptr;             // device, rot.dims / 2 angular frequencies (long-context blend applied), made at finalize
    float rot_mag = 1.f;
    // low-rank attention (LatentSpec): query latent down / up, key-value latent down, per-head key / value up; gains of the two latents
    Weight w_dq, w_uq, w_dkv, w_uk, w_uv;
    const float *dq_norm = nullptr, *dkv_norm = nullptr;
    // state-space scan (ScanSpec): input projection; convolution taps [channels, taps] and bias, step bias, log decay rate, skip gain per head,
    // gain of the grouped output norm (all F32); the sequence's state: last taps - 1 convolution inputs and S [heads, vdim, state] (owned)
    Weight ssm_in;
    const float *ssm_conv = nullptr, *ssm_conv_b = nullptr, *ssm_dt_bias = nullptr, *ssm_a_log = nullptr, *ssm_d = nullptr, *ssm_norm = nullptr;
    float *conv_state = nullptr, *ssm_state = nullptr;
    // feed-forward biases, the router's choice correction, gate matrices of gated experts (+ their device pointer table)
    const float *gate_b = nullptr, *up_b = nullptr, *down_b = nullptr, *route_corr = nullptr;
    std::vector<Weight> e_gate;
    const void** e_gate_tab = nullptr;
    // per-layer token input: gate [side_dim, width], projection [width, side_dim], gain [width]
    Weight side_gate, side_proj;
    const float* side_norm = nullptr;
    // token shift: per-channel blend (F32) and the sequence's carried row [width] (owned)
    const float* shift_mu = nullptr;
    float* shift_state = nullptr;
    // attention options: projection biases, short-convolution taps [channels, taps] of q, k, v and the sequence's last taps - 1 inputs of
    // each (owned), per-head score multiplier, head-mixing matrix [heads, heads], per-head sink, value-blend weight (all F32)
    const float *q_bias = nullptr, *k_bias = nullptr, *v_bias = nullptr, *o_bias = nullptr, *q_conv = nullptr, *k_conv = nullptr, *v_conv = nullptr;
    float *q_conv_state = nullptr, *k_conv_state = nullptr, *v_conv_state = nullptr;
    const float *head_temp = nullptr, *talk = nullptr, *sink = nullptr, *v_mix = nullptr;
    // gated delta rule (DeltaSpec): beta projection, the two low-rank pairs (decay, output gate), decay bias [heads * dim], log decay rate
    // [heads], output-norm gain [vdim]; the sequence's matrix state [heads, vdim, dim] in F32 (owned)
    Weight d_beta, d_a1, d_a2, d_g1, d_g2;
    const float *d_dt_bias = nullptr, *d_a_log = nullptr, *d_norm = nullptr;
    float* delta_state = nullptr;
    // MixerKind::BRANCHES: each branch's tensors and state
    std::vector<LayerWeights> branch;
};

class Model {
public:
    Model() = default;
    ~Model();
    Model(const Model&) = delete;
    Model& operator=(const Model&) = delete;

    // (a) from a GGUF file: parse, shard for (tp_rank, tp_size), upload, allocate, capture.
    bool load_gguf(const std::string& path, int max_context, int tp_rank = 0, int tp_size = 1);
    // (a') from a model folder (config.json + model.safetensors) of a registered layer-spec family (engine/model_registry.h).
    bool load_dir(const std::string& dir, int max_context);
    // Either of the two, by what the path is (a directory or a file).
    bool load(const std::string& path, int max_context);
    // Layer-spec families, before load / finalize: keep every tensor, the KV cache and all arithmetic in true 32-bit (weights are
    // widened once at load; prompt GEMMs run on CUDA cores).  Off: weights stay in their stored dtype (BF16), BF16 cache.
    void set_exact_f32(bool on) { exact32_ = on; }
    bool exact_f32() const { return exact32_; }
    // (b) from caller-owned device tensors (synthetic benchmarks): init -> set_tensor* -> finalize.
    void init(const ModelConfig& cfg, int tp_rank = 0, int tp_size = 1);
    bool set_tensor(const std::string& gguf_name, const void* dev_ptr, DType dtype, size_t row_pitch = 0);
    bool finalize();

    void set_comm(TPComm* comm) { comm_ = comm; }

    // Runs seq_len tokens at positions start_pos.. and returns DEVICE logits [vocab] of the last token
    // (same contract as Transformer::forward, transformer.cpp:604-669; synchronises the stream).
    float* forward(const int* tokens, int seq_len, int start_pos);
    // Like forward(), and also copies the logits at the wanted places (ascending indices into tokens) to out_host [n_want, vocab].
    void forward_logits(const int* tokens, int seq_len, int start_pos, const int* want, int n_want, float* out_host);
    // Asynchronous variant used by the benchmark: no host sync.
    void forward_async(const int* tokens, int seq_len, int start_pos);
    // Greedy next token computed on the GPU from the last logits (argmax, lowest index on ties like Sampler::argmax).
    int argmax_last();
    int sync();                            // waits for the model's stream: returns the cudaError_t; reports a persistent-kernel time-out
    // Samples the next token from the last logits on the GPU (csrc/sample.cu; penalty is applied in place to the device
    // logits).  recent_window: the ids the repeat penalty looks at, oldest first.  Returns -1 when the settings are not
    // covered (top_k <= 0, > 1024 or >= vocab, temperature <= 0): the caller samples on the host.
    int sample_last(float temperature, int top_k, float top_p, float repeat_penalty, const int* recent_window, int n_window, float r);

    const ModelConfig& config() const { return cfg_; }
    const GGUFVocab& vocab() const { return vocab_; }
    cudaStream_t stream() const { return stream_; }
    float* logits_device() const { return logits_; }
    int tp_rank() const { return tp_rank_; }
    int tp_size() const { return tp_size_; }
    // Algorithmic bytes this rank reads per decoded token at context length ctx (SURVEY §8d B_tok).
    size_t bytes_per_token(int ctx) const;
    size_t weight_bytes() const;
    double load_seconds() const { return load_seconds_; }     // wall time of load_gguf (parse + plan + pipelined upload + buffers)
    void set_use_graph(bool on) { use_graph_ = on; }
    void set_use_pdl(bool on) { use_pdl_ = on; }
    // Prompts of at least n tokens go through the batched tensor-core prefill when the weights allow it (0 = never).
    void set_prefill_min_tokens(int n) { prefill_min_tokens_ = n; }
    bool batched_prefill_ok(int seq_len, int start_pos) const;
    void clear_kv();
    // Opt-in (also NT_B200_MEGAKERNEL=1): run the decode step as one persistent kernel (engine/decode_mega.h) instead of
    // the graph of fused launches.  Falls back to the graph path, with a note on stderr, when a shape is not covered.
    void set_use_megakernel(bool on) { use_mega_ = on; }
    int tp_exchange_kind() const { return tp_size_ == 1 || !xchg_tried_ ? 0 : (xchg_ ? 2 : 1); }
    bool megakernel_active();                 // true once the persistent kernel has been built for this model
    // Debug read-back of the persistent kernel's working buffers ("hid0", "hid1", "q", "attn", "act", "slots"): device pointer.
    const float* mega_debug_buffer(const char* name, size_t* count);
    void mega_trace(bool on);                  // record the persistent kernel's phase timeline (debug/tuning)
    size_t mega_trace_read(unsigned long long* out_host, size_t cap);   // [4 CTAs][phases][start, work done, barrier passed] ns
    int mega_plan_kinds(int* kinds, int cap);  // phase kinds of the per-token program; returns their number (0 when inactive)

private:
    // ---- layer-spec families (engine/model_spec.cu) ----
    const LayerWeights& layer_weights(int i) const { const int j = cfg_.layer_spec() ? cfg_.layers[(size_t)i].weights_of : -1; return layers_[(size_t)(j >= 0 ? j : i)]; }
    bool bind_slot(TensorSlot slot, int layer, const void* ptr, DType dt, int rows, int cols, size_t pitch, int index = 0, int branch = -1);
    // STREAMS block form: one decoded token / a chunk of prompt rows
    void layer_streams_token(int i, cudaStream_t s);
    void layer_streams_rows(int i, int T, int p0, cudaStream_t s);
    MoeWeights moe_of(int i, bool with_shared) const;
    // POST_NORM block form (latent attention / state-space scan mixers, biased or routed gated feed-forward, per-layer token input):
    // T rows at positions base.. (base = *pos_dev when given, else p0); T == 1 with pos_dev is the captured decode step.
    struct RowBufs { float *x = nullptr, *y = nullptr, *t[5] = {nullptr, nullptr, nullptr, nullptr, nullptr}; float* wide = nullptr; };
    // SUM_NORM block form (token shift, attention with per-head norm / convolutions / sink / mixed heads / blended values, the gated
    // delta rule, mixers side by side): engine/model_sumnorm.cu.  Same conventions as layer_postnorm.
    void layer_sumnorm(int i, int T, const int* pos_dev, int p0, const RowBufs& B, cudaStream_t s);
    bool finalize_sumnorm_layer(int i);
    bool finalize_mixer_state(LayerSpec& S, LayerWeights& M, int layer);   // states, frequency table and cache slot of one attention / delta mixer
    size_t sumnorm_scratch_width() const;     // floats per row of RowBufs::wide
    struct MixerBufs;
    void mixer_attention_rows(int layer, const LayerSpec& S, const LayerWeights& L, const MixerBufs& b, float* y, int T, const int* pos_dev, int p0, cudaStream_t s);
    void mixer_delta_rows(const LayerSpec& S, const LayerWeights& L, const MixerBufs& b, float* y, int T, const int* pos_dev, int p0, cudaStream_t s);
    const LayerSpec& slot_spec(int slot) const { return *slot_spec_[(size_t)slot]; }
    std::vector<const LayerSpec*> slot_spec_;   // the mixer behind every entry of kcs_ / vcs_: the layers first, then the branches that keep rows
    void layer_postnorm(int i, int T, const int* tok_dev, const int* pos_dev, int p0, const RowBufs& B, cudaStream_t s);
    void rows_matmul(float* C, const float* A, const Weight& w, int T, cudaStream_t s, bool* split_done = nullptr);      // C = A . W^T: GEMV for one row, else spec_gemm
    void pad_for_tensor_cores(Weight& w);     // gives a short BF16 matrix its zero-padded copy (Weight::tc_ptr)
    size_t row_scratch_width() const;         // widest intermediate row of any POST_NORM layer
    void cache_row_widths(int i, size_t& k, size_t& v) const;   // elements per position in layer i's two caches
    int n_streams() const { return cfg_.streams > 0 ? cfg_.streams : 1; }
    bool finalize_spec();
    void step_body_spec(cudaStream_t s);
    void step_head_spec(cudaStream_t s);
    void prefill_spec(const int* tokens, int seq_len, int start_pos);
    void ensure_prefill_buffers_spec(int tokens);
    bool spec_tc_ok(const Weight& w) const;
    void spec_gemm(float* C, const float* A, const void* A_split, const Weight& w, int T, DenseEpilogue ep, const float* row_scale, float alpha, cudaStream_t s);
    void emit_wanted(const float* x_rows, int c0, int T, cudaStream_t s);   // logits of the wanted places inside tokens [c0, c0 + T)
    const ModelFamily* family_ = nullptr;
    bool exact32_ = false;
    DType cache_dt_ = DType::F16;
    std::vector<void*> kcs_, vcs_;        // per-layer caches [max_seq, kv_heads * maps * dim] / [max_seq, kv_heads * vdim] of cache_dt_
    std::vector<char> cache_owned_;       // 0: the layer reads another layer's cache rows (LayerSpec::kv_from)
    float* streams_ = nullptr;            // decode: the residual streams [S, width]
    float* sub_y_ = nullptr;              // decode: a sublayer's output before it enters the streams [width]
    float* maps_out_ = nullptr;           // decode: the attention maps' outputs [heads * maps * vdim]
    int* moe_sel_ = nullptr;              // decode: chosen experts [top], weights [top], shared gate [1], activations [top * ff + shared_ff]
    float *moe_wt_ = nullptr, *moe_sgate_ = nullptr, *moe_act_ = nullptr;
    int* moe_offsets_host_ = nullptr;     // pinned: per-expert row offsets of the current prompt chunk (tensor-core expert GEMMs)
    float* ident_tab_ = nullptr;          // {1}: mixing matrix and write gain of a single residual stream
    Weight side_embd_;                    // second token embedding [vocab, layers * side_dim] (ModelConfig::side_dim)
    // Latent attention over a prompt portion: every visible position's per-head keys [P, heads, kd] and values [P, heads, vd] (16-bit,
    // widths padded to what the tiled attention kernel takes), rebuilt from the latent rows for each layer and portion; the portion's
    // rotated, padded queries and padded outputs; F32 staging of one block of rows for the two up-projections.
    struct LatentScratch {
        size_t rows = 0, tokens = 0, kw = 0, vw = 0, stage_w = 0, rank = 0;
        void *k = nullptr, *v = nullptr, *ws = nullptr;
        float *q = nullptr, *o = nullptr, *c32 = nullptr, *ku = nullptr, *vu = nullptr;
    } lat_;
    float* lat_part_ = nullptr;           // absorbed latent attention: (max, sum, vector) per (query, key slice, head), joined by a merge launch
    bool latent_expand_ok(const LayerSpec& S, int T) const;
    void ensure_latent_scratch(const LayerSpec& S, size_t rows, size_t tokens);
    void latent_attention_rows(int i, int T, int p0, const float* q, float* out, cudaStream_t s);   // out [T, heads * vdim]
    bool moe_glu_rows_tc(int i, int T, const float* x, cudaStream_t s);    // routed gated experts of a prompt portion on the tensor cores -> pf_.y_rows
    RowBufs dec_;                         // POST_NORM decode step: x is hidden_, the rest one scratch row each (stable addresses for the graph)
    std::vector<int> want_;               // places (indices into the current forward's tokens) whose logits are collected
    float* want_out_ = nullptr;           // device [want_cap_, vocab]
    size_t want_cap_ = 0;

    bool ensure_mega();
    void run_step_mega(bool with_head);
    void step_body(cudaStream_t s);      // embedding + all layers for the token/position in step_dev_
    void step_head(cudaStream_t s, bool from_chain = false);   // final norm + LM head (+ all-gather under TP); from_chain: norm + quantiser in the GEMV prologue
    bool chain_ok() const;               // every projection on the TMA/dp4a GEMV: the fused launch chain applies
    void run_step(bool with_head);
    void matvec(const Weight* const* ws, float* const* ys, int n, const float* x, const float* norm_w, GemvEpilogue ep,
                cudaStream_t s);
    void reduce_residual(float* partial, cudaStream_t s);
    // All prompt tokens at once: tcgen05 GEMMs (csrc/prefill_gemm.cu) + batched norm/rope/KV-write/causal attention,
    // instead of the reference's per-token loop (transformer.cpp:604-669 runs every layer's GEMVs once per token).
    void prefill_batched(const int* tokens, int seq_len, int start_pos);
    void ensure_prefill_buffers(int tokens);
    bool f16_direct(const Weight& w) const;   // F16 rows usable by TMA in place
    // C[T, w.rows] (+)= split(A)[T, w.cols] . W^T for a weight of any GGUF dtype (quantised: dequantise to hi/lo, two GEMMs)
    void prefill_gemm(float* C, const void* ws, const Weight& w, int T, bool add, cudaStream_t s);
    bool o_xq_fusable(const Weight& wo) const;
    void release_graphs();

    ModelConfig cfg_;
    GGUFVocab vocab_;
    int tp_rank_ = 0, tp_size_ = 1;
    int nh_l_ = 0, nkv_l_ = 0;           // local heads
    int inter_l_ = 0, vocab_l_ = 0;      // local FFN columns / vocab rows
    TPComm* comm_ = nullptr;

    Weight embd_, head_;
    const float* out_norm_ = nullptr;
    std::vector<LayerWeights> layers_;
    std::vector<void*> owned_;

    // device buffers
    cudaStream_t stream_ = nullptr;
    float *hidden_ = nullptr, *xnorm_ = nullptr, *q_ = nullptr, *k_ = nullptr, *v_ = nullptr, *attn_ = nullptr;
    float *act_ = nullptr, *up_ = nullptr, *part_ = nullptr, *logits_ = nullptr, *logits_l_ = nullptr, *attn_scratch_ = nullptr;
    void *xq_h_ = nullptr, *xq_a_ = nullptr, *xq_i_ = nullptr;
    unsigned* attn_tickets_ = nullptr;   // last-arriver tickets of the one-launch attention (zero between launches)
    int fuse_mask_ = 1;                  // bit 0: norm + quantiser in the GEMV prologues (default), bit 1: one-launch attention (opt-in: measured slower, profiles/r02_*), bit 2: RoPE + KV write inside the decode kernel, merge separate (NT_B200_FUSE)
    void *kc_ = nullptr, *vc_ = nullptr;
    int* step_dev_ = nullptr;            // [0] token, [1] position
    int* argmax_dev_ = nullptr;
    int* argmax_host_ = nullptr;
    int* recent_dev_ = nullptr;          // repeat-penalty window for the GPU sampler
    int recent_cap_ = 0;

    struct PrefillBuffers {
        int cap = 0;                     // tokens per chunk the buffers hold
        float *x = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *attn = nullptr;
        void *ws = nullptr, *ws2 = nullptr;   // F16 hi/lo split of the current GEMM input (ws2: SwiGLU output -> down projection)
        float *g = nullptr, *u = nullptr;     // gate / up activations (only when those weights are not F16: unfused SwiGLU)
        void *whi = nullptr, *wlo = nullptr;  // dequantised weight matrix as an F16 hi/lo pair (quantised models)
        int *tok = nullptr, *pos = nullptr;
        float *h = nullptr, *tmp = nullptr;   // layer-spec families: the block's normed input (read by both branches), a GEMM result before its scaled add
        void *hws = nullptr;                  // ... and its F16 hi/lo split
        float *xs = nullptr, *maps = nullptr;     // STREAMS: the residual streams [T, S, width]; attention maps' outputs [T, heads * maps * vdim]
        int *sel = nullptr, *work = nullptr;      // mixture of experts: chosen experts [T, top]; grouping tables
        float *g2 = nullptr; void *moe_ws = nullptr;   // tensor-core experts: rows gathered in expert order [T*top, width]; per-expert padded split workspace
        void *moe_ws2 = nullptr;                       // gated tensor-core experts: the split of act(gate) * up, input of the down GEMMs
        float *gate_rows = nullptr;                    // gated experts: W_gate h of the grouped rows [T*top, ff]
        float *wt = nullptr, *sgate = nullptr, *act_rows = nullptr, *y_rows = nullptr;   // weights [T, top], shared gate [T], grouped rows [T*top, ff | width]
        float *wide = nullptr;                         // SUM_NORM: the mixers' intermediates [T, sumnorm_scratch_width()]
    } pf_;
    // Prompts shorter than this replay token by token through the decode chain (exact-integer GEMVs); longer ones take the batched
    // tensor-core prefill, whose F32 accumulation inside the tensor cores truncates once per 16-deep MMA step: ~1e-5..1e-4 per GEMM,
    // ~3e-4 per layer on the random synthetic models (profiles/r02_parity_8b.txt) against ~1e-5 per layer for the GEMV path.
    int prefill_min_tokens_ = 32;

    bool use_graph_ = true;
    bool use_pdl_ = true;
    cudaGraphExec_t g_full_ = nullptr, g_body_ = nullptr;
    int n_full_ = 0, n_body_ = 0;        // kernels per graph replay
    bool finalized_ = false;
    double load_seconds_ = 0.0;

    // Tensor parallel: the o-projection / down-projection partials are summed through NVLink peer memory (engine/peer_xchg.h);
    // NT_B200_TP_NCCL=1 (or a failed peer mapping) keeps ncclAllReduce + add.
    std::unique_ptr<PeerXchg> xchg_;
    bool xchg_tried_ = false;
    void ensure_xchg();

    bool use_mega_ = false;
    bool mega_tried_ = false;
    std::unique_ptr<DecodeMega> mega_;
};

}}  // namespace nt::b200
