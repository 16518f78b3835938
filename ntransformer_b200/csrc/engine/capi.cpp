// capi.cpp — extern "C" surface of the engine: include/ntransformer.h and include/nt_b200_engine.h.
#include "../../../include/ntransformer.h"
#include "../../../include/nt_b200_engine.h"
#include "engine.h"
#include "tp_comm.h"
#include "json.h"
#include "model_registry.h"
#include "safetensors.h"
#include <cstring>
#include <algorithm>
#include <memory>
#include <string>

using namespace nt::b200;

namespace {
struct ModelHandle {
    std::unique_ptr<TPComm> comm;     // declared first => destroyed last: the model's graphs reference the communicator
    Model model;
};
ModelHandle* H(nt_model_t m) { return static_cast<ModelHandle*>(m); }
}  // namespace

extern "C" {

// ---- include/ntransformer.h ----
nt_engine_t nt_engine_create(void) { return new Engine(); }
void nt_engine_destroy(nt_engine_t e) { delete static_cast<Engine*>(e); }
int nt_engine_load(nt_engine_t e, const char* path) { return (e && path && static_cast<Engine*>(e)->load(path)) ? 0 : -1; }
char* nt_engine_generate(nt_engine_t e, const char* prompt, int max_tokens, float temperature, int top_k, float top_p) {
    if (!e || !prompt) return nullptr;
    GenerateConfig cfg;
    cfg.max_tokens = max_tokens; cfg.temperature = temperature; cfg.top_k = top_k; cfg.top_p = top_p; cfg.verbose = false;
    std::string out = static_cast<Engine*>(e)->generate(prompt, cfg);
    char* r = static_cast<char*>(malloc(out.size() + 1));
    if (r) memcpy(r, out.c_str(), out.size() + 1);
    return r;
}
void nt_free(char* p) { free(p); }
int nt_engine_vocab_size(nt_engine_t e) { return e ? static_cast<Engine*>(e)->config().vocab_size : 0; }
int nt_engine_n_layers(nt_engine_t e) { return e ? static_cast<Engine*>(e)->config().n_layers : 0; }
int nt_engine_hidden_size(nt_engine_t e) { return e ? static_cast<Engine*>(e)->config().hidden_size : 0; }

// ---- include/nt_b200_engine.h ----
nt_model_t nt_model_load_gguf(const char* path, int max_context, int tp_rank, int tp_size) {
    auto* h = new ModelHandle();
    if (!path || !h->model.load_gguf(path, max_context, tp_rank, tp_size)) { delete h; return nullptr; }
    return h;
}
nt_model_t nt_model_create(const nt_model_config* c, int tp_rank, int tp_size) {
    if (!c) return nullptr;
    ModelConfig cfg;
    cfg.vocab_size = c->vocab_size; cfg.hidden_size = c->hidden_size; cfg.intermediate_size = c->intermediate_size;
    cfg.n_layers = c->n_layers; cfg.n_heads = c->n_heads; cfg.n_kv_heads = c->n_kv_heads; cfg.head_dim = c->head_dim;
    cfg.max_seq_len = c->max_seq_len; cfg.norm_eps = c->norm_eps; cfg.rope_theta = c->rope_theta;
    cfg.bos_token_id = c->bos_token_id; cfg.eos_token_id = c->eos_token_id;
    auto* h = new ModelHandle();
    h->model.init(cfg, tp_rank, tp_size);
    return h;
}
nt_model_t nt_model_load_dir(const char* dir, int max_context, int exact_f32) {
    auto* h = new ModelHandle();
    h->model.set_exact_f32(exact_f32 != 0);
    if (!dir || !h->model.load_dir(dir, max_context)) { delete h; return nullptr; }
    return h;
}
nt_model_t nt_model_create_json(const char* config_json, int max_context, int exact_f32) {
    if (!config_json) return nullptr;
    Json root;
    std::string err;
    if (!Json::parse(std::string(config_json), root, &err) || !root.is_object()) { fprintf(stderr, "nt_model_create_json: %s\n", err.c_str()); return nullptr; }
    const ModelFamily* f = find_model_family(root.at("architecture").string_or(""));
    ModelConfig cfg;
    if (!f) { fprintf(stderr, "nt_model_create_json: unregistered architecture\n"); return nullptr; }
    cfg.architecture = f->architecture;
    if (!f->config_from_json(root, cfg, err)) { fprintf(stderr, "nt_model_create_json: %s\n", err.c_str()); return nullptr; }
    cfg.max_seq_len = std::max(1, max_context);
    auto* h = new ModelHandle();
    h->model.set_exact_f32(exact_f32 != 0);
    h->model.init(cfg, 0, 1);
    return h;
}
// Host only (no GPU touched): reads <dir>/config.json through the family registry and checks model.safetensors against the
// tensors the configuration needs.  Writes a text summary; returns 0, or -1 with the reason in out.
int nt_model_dir_describe(const char* dir, char* out, size_t cap) {
    if (!dir || !out || cap == 0) return -1;
    auto put = [&](const std::string& t, int rc) { snprintf(out, cap, "%s", t.c_str()); return rc; };
    ModelConfig cfg;
    const ModelFamily* fam = nullptr;
    if (!read_model_dir(dir, cfg, &fam)) return put("config.json rejected", -1);
    SafeTensorsFile f;
    if (!f.open(std::string(dir) + "/model.safetensors")) return put("model.safetensors rejected", -1);
    if (fam->sizes_from_tensors) {
        std::string err;
        const TensorShapeFn shape_of = [&](const std::string& name, std::vector<int64_t>& shape) {
            const SafeTensorInfo* ti = f.find(name);
            if (ti) shape = ti->shape;
            return ti != nullptr;
        };
        if (!fam->sizes_from_tensors(cfg, shape_of, err)) return put(err, -1);
    }
    std::string text = std::string("architecture=") + fam->architecture + " vocab=" + std::to_string(cfg.vocab_size) + " width=" + std::to_string(cfg.hidden_size) +
                       " layers=" + std::to_string(cfg.n_layers) + " eps=" + std::to_string(cfg.norm_eps) + " mult=" + std::to_string(cfg.residual_mult) + "\n";
    for (size_t i = 0; i < cfg.layers.size(); i++) {
        const LayerSpec& L = cfg.layers[i];
        text += "layer " + std::to_string(i) + ": heads=" + std::to_string(L.heads) + " kv=" + std::to_string(L.kv_heads) + " dim=" + std::to_string(L.dim) +
                " vdim=" + std::to_string(L.vdim) + " window=" + std::to_string(L.window) + " keep=" + std::to_string(L.keep_first) + " ff=" + std::to_string(L.ff) +
                " weights_of=" + std::to_string(L.weights_of);
        if (L.form == BlockForm::STREAMS)
            text += " chunk=" + std::to_string(L.chunk) + " maps=" + std::to_string(L.maps) + " rot=" + std::to_string(L.rot.dims) + " kv_from=" + std::to_string(L.kv_from) +
                    " experts=" + std::to_string(L.experts) + " top=" + std::to_string(L.top) + " shared_ff=" + std::to_string(L.shared_ff) +
                    " streams=" + std::to_string(cfg.streams);
        if (L.form == BlockForm::POST_NORM) {
            text += std::string(" mixer=") + (L.mixer == MixerKind::ATTN_LATENT ? "latent" : "scan");
            if (L.mixer == MixerKind::ATTN_LATENT)
                text += " q_rank=" + std::to_string(L.latent.q_rank) + " kv_rank=" + std::to_string(L.latent.kv_rank) + " rot_dim=" + std::to_string(L.latent.rot_dim) +
                        " rot=" + std::to_string(L.rot.dims) + " kv_from=" + std::to_string(L.kv_from);
            else
                text += " state=" + std::to_string(L.scan.state) + " groups=" + std::to_string(L.scan.groups) + " conv=" + std::to_string(L.scan.conv) +
                        " norm_groups=" + std::to_string(L.scan.norm_groups);
            text += std::string(" ff_kind=") + (L.ff == 0 ? "none" : L.ff_kind == FfKind::GLU ? "dense" : "moe") + " experts=" + std::to_string(L.experts) + " top=" +
                    std::to_string(L.top) + " route_groups=" + std::to_string(L.route.groups) + "/" + std::to_string(L.route.keep) + " side=" + std::to_string(cfg.side_dim);
        }
        if (L.form == BlockForm::SUM_NORM) {
            auto mixer_text = [](const LayerSpec& M) {
                if (M.mixer == MixerKind::DELTA_RULE)
                    return " delta(heads=" + std::to_string(M.heads) + " kv=" + std::to_string(M.kv_heads) + " dim=" + std::to_string(M.dim) + " vdim=" + std::to_string(M.vdim) +
                           " conv=" + std::to_string(M.conv) + " ranks=" + std::to_string(M.delta.decay_rank) + "/" + std::to_string(M.delta.gate_rank) + ")";
                return " attention(heads=" + std::to_string(M.heads) + " kv=" + std::to_string(M.kv_heads) + " dim=" + std::to_string(M.dim) + " vdim=" + std::to_string(M.vdim) +
                       " rot=" + std::to_string(M.rot.dims) + " divide=" + std::to_string(M.rot.divide) + " conv=" + std::to_string(M.conv) + " bias=" + std::to_string(M.qkv_bias) +
                       " temp=" + std::to_string(M.head_temp) + " talking=" + std::to_string(M.talking) + " sink=" + std::to_string(M.sink) + " v_first=" + std::to_string(M.v_first) + ")";
            };
            text += " skip=" + std::to_string(cfg.skip_scale) + " shift=" + std::to_string(L.token_shift);
            if (L.mixer == MixerKind::BRANCHES)
                for (size_t b = 0; b < L.branches.size(); b++) text += " " + std::to_string(L.branch_scale[b]) + " *" + mixer_text(L.branches[b]);
            else text += mixer_text(L);
        }
        text += "\n";
    }
    size_t n = 0;
    for (const TensorBinding& b : fam->tensors(cfg)) {
        const SafeTensorInfo* ti = f.find(b.name);
        if (!ti) return put("tensor not found: " + b.name, -1);
        const bool ok = (b.rows == 1 && b.cols == 1 && ti->shape.empty()) ||
                        ((b.rows == 1 && ti->shape.size() == 1) ? ti->shape[0] == b.cols : (ti->shape.size() == 2 && ti->shape[0] == b.rows && ti->shape[1] == b.cols));
        if (!ok) return put("tensor " + b.name + " does not have the shape the configuration needs", -1);
        n++;
    }
    text += "tensors=" + std::to_string(n) + "\n";
    return put(text, 0);
}
int nt_model_forward_logits(nt_model_t m, const int* tokens, int n, int start_pos, const int* want, int n_want, float* logits_host) {
    if (!m || !tokens || n < 1 || n_want < 0 || (n_want > 0 && (!want || !logits_host))) return -1;
    H(m)->model.forward_logits(tokens, n, start_pos, want, n_want, logits_host);
    return 0;
}
int nt_engine_load_path(nt_engine_t e, const char* path, int max_context, int exact_f32) {
    if (!e || !path) return -1;
    Engine* en = static_cast<Engine*>(e);
    en->model().set_exact_f32(exact_f32 != 0);
    return en->load(path, max_context) ? 0 : -1;
}
int nt_engine_generate_ids(nt_engine_t e, const int* prompt_ids, int n_prompt, int max_tokens, float temperature, int top_k, float top_p,
                           float repeat_penalty, unsigned long long seed, int* out_ids, int cap) {
    if (!e || !prompt_ids || n_prompt < 1) return -1;
    GenerateConfig cfg;
    cfg.max_tokens = max_tokens; cfg.temperature = temperature; cfg.top_k = top_k; cfg.top_p = top_p; cfg.repeat_penalty = repeat_penalty;
    cfg.seed = seed; cfg.verbose = false;
    const std::vector<int> ids = static_cast<Engine*>(e)->generate_ids(std::vector<int>(prompt_ids, prompt_ids + n_prompt), cfg);
    for (int i = 0; i < (int)ids.size() && i < cap; i++) out_ids[i] = ids[(size_t)i];
    return (int)ids.size();
}
// kernel-level entries of the layer-spec mechanisms (csrc/dense.cu, csrc/attention_window.cu) for numerics tests
void nt_b200_gemv_dense(float* y0, float* y1, float* y2, const void* W0, const void* W1, const void* W2, int out0, int out1, int out2, int n_mat, int K,
                        const float* x, int dtype, int epilogue, const float* row_scale, float alpha, void* stream) {
    GemvMat m[3];
    const void* Ws[3] = {W0, W1, W2}; float* ys[3] = {y0, y1, y2}; const int outs[3] = {out0, out1, out2};
    for (int i = 0; i < 3; i++) { m[i].W = Ws[i]; m[i].y = ys[i]; m[i].out = outs[i]; m[i].dtype = (nt::DType)dtype; }
    gemv_dense(m, n_mat, K, x, (DenseEpilogue)epilogue, row_scale, alpha, static_cast<cudaStream_t>(stream));
}
void nt_b200_gemm_dense(float* Cm, const float* A, const void* W, int dtype, int T, int N, int K, int epilogue, const float* row_scale, float alpha, void* stream) {
    gemm_dense(Cm, A, W, (nt::DType)dtype, 0, T, N, K, (DenseEpilogue)epilogue, row_scale, alpha, static_cast<cudaStream_t>(stream));
}
void nt_b200_attention_window(float* out, const float* Q, const void* kc, const void* vc, int cache_dtype, int tokens, int p0, int heads, int kv_heads,
                              int dim, int vdim, int window, int keep, float scale, float softcap, int max_seq, void* stream) {
    WindowAttn a;
    a.heads = heads; a.kv_heads = kv_heads; a.dim = dim; a.vdim = vdim; a.window = window; a.keep = keep; a.scale = scale; a.softcap = softcap;
    attention_window(out, Q, kc, vc, (nt::DType)cache_dtype, tokens, nullptr, p0, max_seq, a, static_cast<cudaStream_t>(stream));
}
void nt_b200_qk_norm_kv_write(float* Q, const float* K, const float* V, const float* q_gain, const float* k_gain, float eps, void* kc, void* vc,
                              int cache_dtype, int tokens, int p0, int qdim, int kdim, int vdim, void* stream) {
    qk_norm_kv_write(Q, K, V, q_gain, k_gain, eps, kc, vc, (nt::DType)cache_dtype, tokens, nullptr, p0, qdim, kdim, vdim, static_cast<cudaStream_t>(stream));
}
void nt_b200_attention_maps(float* out, const float* Q, const void* kc, const void* vc, int cache_dtype, int tokens, int p0, int heads, int kv_heads,
                            int dim, int vdim, int chunk, int maps, float scale, int max_seq, void* stream) {
    WindowAttn a;
    a.heads = heads; a.kv_heads = kv_heads; a.dim = dim; a.vdim = vdim; a.chunk = chunk; a.maps = maps; a.scale = scale;
    attention_window(out, Q, kc, vc, (nt::DType)cache_dtype, tokens, nullptr, p0, max_seq, a, static_cast<cudaStream_t>(stream));
}
float nt_b200_rotary_table(float* freq_host, int dims, float base, float factor, float original, float fast, float slow) {
    return rotary_table(freq_host, dims, base, factor, original, fast, slow);
}
void nt_b200_rope_partial_kv_write(float* Q, const float* K, const float* V, const float* freq, float mag, int dims, int interleaved, int dim, void* kc,
                                   void* vc, int cache_dtype, int tokens, int p0, int qdim, int kdim, int vdim, void* stream) {
    rope_partial_kv_write(Q, K, V, freq, mag, dims, interleaved != 0, dim, kc, vc, (nt::DType)cache_dtype, tokens, nullptr, p0, qdim, kdim, vdim,
                          static_cast<cudaStream_t>(stream));
}
void nt_b200_diff_combine(float* out, const float* A, const float* lq1, const float* lk1, const float* lq2, const float* lk2, int n_l, float diff, float eps,
                          int tokens, int heads, int vdim, void* stream) {
    diff_combine(out, A, lq1, lk1, lq2, lk2, n_l, diff, eps, tokens, heads, vdim, static_cast<cudaStream_t>(stream));
}
void nt_b200_streams_spread(float* X, const float* e, float scale, int tokens, int S, int width, void* stream) {
    streams_spread(X, e, scale, tokens, S, width, static_cast<cudaStream_t>(stream));
}
void nt_b200_streams_read(float* u, const float* X, const float* a, int tokens, int S, int width, void* stream) {
    streams_read(u, X, a, tokens, S, width, static_cast<cudaStream_t>(stream));
}
void nt_b200_streams_write(float* X, const float* y, const float* M, const float* b, int tokens, int S, int width, void* stream) {
    streams_write(X, y, M, b, tokens, S, width, static_cast<cudaStream_t>(stream));
}
void nt_b200_moe_route(int* sel, float* wt, float* sgate, const float* h, const float* router, const float* shared_gate, int experts, int top, int width,
                       int tokens, void* stream) {
    MoeWeights w;
    w.router = router; w.shared_gate = shared_gate; w.experts = experts; w.top = top; w.width = width;
    moe_route(sel, wt, sgate, h, w, tokens, static_cast<cudaStream_t>(stream));
}
// mode 0: the one-token kernels (tokens == 1; scratch: floats [top * ff + shared_ff]); mode 1: the grouped prompt-row kernels
// (scratch: ints moe work table, then floats [tokens * top * (ff + width)]; the shared expert's output, if any, comes in shared_y)
void nt_b200_moe_experts(float* y, const float* h, const int* sel, const float* wt, const float* sgate, const void* const* up_tab, const void* const* down_tab,
                         const void* shared_up, const void* shared_down, const float* shared_y, int dtype, int experts, int top, int ff, int width,
                         int shared_ff, int tokens, int mode, void* scratch, void* stream) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    MoeWeights w;
    w.up = up_tab; w.down = down_tab; w.dtype = (nt::DType)dtype; w.experts = experts; w.top = top; w.ff = ff; w.width = width;
    if (mode == 0) {
        w.shared_up = shared_up; w.shared_down = shared_down; w.shared_ff = shared_up ? shared_ff : 0;
        float* act = static_cast<float*>(scratch);
        moe_expert_up_token(act, h, sel, w, s);
        moe_expert_down_token(y, act, sel, wt, sgate, nullptr, w, s);
        return;
    }
    int* work = static_cast<int*>(scratch);
    const size_t wi = (moe_work_ints(tokens, experts, top) + 3) & ~(size_t)3;
    float* act_rows = reinterpret_cast<float*>(work + wi);
    float* y_rows = act_rows + (size_t)tokens * top * ff;
    moe_group(work, sel, tokens, experts, top, s);
    moe_expert_up_rows(act_rows, h, work, w, tokens, s);
    moe_expert_down_rows(y_rows, act_rows, work, w, tokens, s);
    moe_combine(y, y_rows, work, wt, sgate, shared_y, tokens, experts, top, width, s);
}
// ---- kernel entries of the mechanisms added with the Tanolorn family (numerics tests) ----
void nt_b200_latent_prep(float* cq, int q_rank, const float* q_gain, const float* dkv, int kv_rank, int rot_dim, const float* kv_gain, float eps, void* cache,
                         int cache_dtype, int rot_dims, int interleaved, float rot_base, int tokens, int p0, void* stream) {
    latent_prep(cq, q_rank, q_gain, dkv, kv_rank, rot_dim, kv_gain, eps, cache, (nt::DType)cache_dtype, rot_dims, interleaved != 0, rot_base, tokens, nullptr, p0,
                static_cast<cudaStream_t>(stream));
}
void nt_b200_latent_q_absorb(float* qa, const float* q, const void* W_uk, int dtype, int tokens, int heads, int dim, int rot_dim, int kv_rank, int rot_dims,
                             int interleaved, float rot_base, int p0, void* stream) {
    latent_q_absorb(qa, q, W_uk, (nt::DType)dtype, tokens, heads, dim, rot_dim, kv_rank, rot_dims, interleaved != 0, rot_base, nullptr, p0, static_cast<cudaStream_t>(stream));
}
void nt_b200_latent_v_up(float* out, const float* ol, const void* W_uv, int dtype, int tokens, int heads, int vdim, int kv_rank, void* stream) {
    latent_v_up(out, ol, W_uv, (nt::DType)dtype, tokens, heads, vdim, kv_rank, static_cast<cudaStream_t>(stream));
}
// The prompt-portion form of latent attention: every visible row's per-head keys and values expanded once (F32 GEMMs here, the engine
// uses its tensor-core GEMM where the matrices qualify), packed as 16-bit operands, then the tiled tensor-core attention kernel.
// cache: BF16 rows [rows, kv_rank + rot_dim] with rows >= p0 + tokens.  Scratch is allocated and freed here.  -1: head widths not covered.
int nt_b200_latent_attention_expanded(float* out, const float* q, const void* cache, const void* W_uk, const void* W_uv, int dtype, int tokens, int p0, int heads,
                                      int dim, int rot_dim, int vdim, int kv_rank, int rot_dims, int interleaved, float rot_base, float scale, void* stream) {
    int kw = 0, vw = 0;
    if (tokens < 16 || !attention_heads_mma_widths(dim + rot_dim, vdim, &kw, &vw)) return -1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t P = (size_t)p0 + tokens, H = (size_t)heads;
    float *c32 = nullptr, *ku = nullptr, *vu = nullptr, *qp = nullptr, *op = nullptr;
    void *kf = nullptr, *vf = nullptr;
    NT_CUDA_CHECK(cudaMalloc(&c32, sizeof(float) * P * kv_rank)); NT_CUDA_CHECK(cudaMalloc(&ku, sizeof(float) * P * H * dim)); NT_CUDA_CHECK(cudaMalloc(&vu, sizeof(float) * P * H * vdim));
    NT_CUDA_CHECK(cudaMalloc(&qp, sizeof(float) * tokens * H * kw)); NT_CUDA_CHECK(cudaMalloc(&op, sizeof(float) * tokens * H * vw));
    NT_CUDA_CHECK(cudaMalloc(&kf, 2 * P * H * kw)); NT_CUDA_CHECK(cudaMalloc(&vf, 2 * P * H * vw));
    latent_rows_f32(c32, cache, nt::DType::BF16, kv_rank + rot_dim, kv_rank, 0, (int)P, s);
    gemm_dense(ku, c32, W_uk, (nt::DType)dtype, 0, (int)P, heads * dim, kv_rank, DENSE_STORE, nullptr, 1.f, s);
    gemm_dense(vu, c32, W_uv, (nt::DType)dtype, 0, (int)P, heads * vdim, kv_rank, DENSE_STORE, nullptr, 1.f, s);
    latent_expand_pack(kf, vf, ku, vu, cache, nt::DType::BF16, kv_rank, 0, (int)P, heads, dim, rot_dim, vdim, kw, vw, s);
    latent_q_rot_pad(qp, q, tokens, heads, dim, rot_dim, kw, rot_dims, interleaved != 0, rot_base, p0, s);
    attention_heads_mma(op, qp, kf, vf, tokens, p0, (int)P, heads, kw, vw, scale, s);
    latent_unpad(out, op, tokens, heads, vdim, vw, s);
    NT_CUDA_CHECK(cudaStreamSynchronize(s));
    for (void* p : {(void*)c32, (void*)ku, (void*)vu, (void*)qp, (void*)op, kf, vf}) cudaFree(p);
    return 0;
}
// Full causal attention of `heads` query heads over ONE key / value head whose rows live in `cache` with `row` numbers per position:
// keys are the first `dim` numbers of a row, values its first `vdim` (the latent-attention layout: dim = row, vdim = kv_rank).
void nt_b200_attention_rows(float* out, const float* Q, const void* cache, int cache_dtype, int tokens, int p0, int heads, int dim, int vdim, int row, float scale,
                            int max_seq, void* stream) {
    WindowAttn a;
    a.heads = heads; a.kv_heads = 1; a.dim = dim; a.vdim = vdim; a.scale = scale; a.k_stride = row; a.v_stride = row;
    attention_window(out, Q, cache, cache, (nt::DType)cache_dtype, tokens, nullptr, p0, max_seq, a, static_cast<cudaStream_t>(stream));
}
// The same attention with every head served from one shared-memory copy of the rows (key slices merged by a second launch).
// -1: shape not covered.  Scratch is allocated and freed here.
int nt_b200_attention_rows_shared(float* out, const float* Q, const void* cache, int cache_dtype, int tokens, int p0, int heads, int dim, int vdim, int row, float scale,
                                  int max_seq, void* stream) {
    if (!attention_shared_rows_supported(heads, dim, vdim, row, (nt::DType)cache_dtype, cache)) return -1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float* scratch = nullptr;
    NT_CUDA_CHECK(cudaMalloc(&scratch, sizeof(float) * attention_shared_rows_scratch_floats(heads, vdim)));
    attention_shared_rows(out, Q, cache, (nt::DType)cache_dtype, tokens, nullptr, p0, max_seq, heads, dim, vdim, row, scale, scratch, s);
    NT_CUDA_CHECK(cudaStreamSynchronize(s));
    cudaFree(scratch);
    return 0;
}
void nt_b200_ssm_conv(float* out, const float* u, int ld, int col0, float* conv_state, const float* w, const float* b, int tokens, int ch, int taps, int p0, void* stream) {
    ssm_conv(out, u, ld, col0, conv_state, w, b, tokens, ch, taps, nullptr, p0, static_cast<cudaStream_t>(stream));
}
void nt_b200_ssm_scan(float* y, const float* xbc, const float* u, int ld, int dt_col0, float* state, const float* dt_bias, const float* A_log, const float* D,
                      int tokens, int heads, int vdim, int N, int groups, int p0, void* stream) {
    ssm_scan(y, xbc, u, ld, dt_col0, state, dt_bias, A_log, D, tokens, heads, vdim, N, groups, nullptr, p0, static_cast<cudaStream_t>(stream));
}
void nt_b200_ssm_gate_norm(float* out, const float* y, const float* u, int ld, int z_col0, const float* gain, float eps, int tokens, int inner, int norm_groups,
                           void* stream) {
    ssm_gate_norm(out, y, u, ld, z_col0, gain, eps, tokens, inner, norm_groups, static_cast<cudaStream_t>(stream));
}
void nt_b200_add_rmsnorm_rows(float* x, const float* y, const float* gain, const float* bias, int rows, int width, float eps, void* stream) {
    add_rmsnorm_rows(x, y, gain, bias, rows, width, eps, static_cast<cudaStream_t>(stream));
}
void nt_b200_glu_bias_mul(float* out, const float* gate, const float* up, const float* gate_bias, const float* up_bias, int rows, int cols, int gelu, void* stream) {
    glu_bias_mul(out, gate, up, gate_bias, up_bias, rows, cols, gelu != 0, static_cast<cudaStream_t>(stream));
}
// ---- kernels of the sum-norm block, the short convolutions, the gated delta rule and attention with per-head options ----
// Up to 6 segments: per segment u, out, w, in_bias (may be null), state (device pointers) and ch, taps, act (0 none, 1 SiLU); rows are packed (ld == ch).
void nt_b200_short_conv(const void* const* u, void* const* out, const void* const* w, const void* const* in_bias, void* const* state, const int* ch, const int* taps,
                        const int* act, int n_seg, int tokens, int p0, void* stream) {
    ConvSeg segs[SHORT_CONV_MAX_SEGS];
    NT_CHECK(n_seg >= 1 && n_seg <= SHORT_CONV_MAX_SEGS, "nt_b200_short_conv: 1..6 segments");
    for (int i = 0; i < n_seg; i++) {
        segs[i].u = static_cast<const float*>(u[i]); segs[i].ld = ch[i]; segs[i].out = static_cast<float*>(out[i]); segs[i].out_ld = ch[i]; segs[i].ch = ch[i];
        segs[i].taps = taps[i]; segs[i].w = static_cast<const float*>(w[i]); segs[i].in_bias = static_cast<const float*>(in_bias[i]);
        segs[i].state = static_cast<float*>(state[i]); segs[i].act = act[i];
    }
    short_conv(segs, n_seg, tokens, nullptr, p0, static_cast<cudaStream_t>(stream));
}
void nt_b200_delta_prep(float* q, float* k, float* a, float* beta, float* qk, const float* dt_bias, const float* A_log, int tokens, int heads, int kv_heads, int dim,
                        void* stream) {
    delta_prep(q, k, a, beta, qk, dt_bias, A_log, tokens, heads, kv_heads, dim, static_cast<cudaStream_t>(stream));
}
void nt_b200_delta_rule_rows(float* out, const float* q, const float* k, const float* v, const float* a, const float* beta, const float* qk, float* state, int tokens,
                             int heads, int kv_heads, int dim, int vdim, int p0, void* stream) {
    delta_rule_rows(out, q, k, v, a, beta, qk, state, tokens, heads, kv_heads, dim, vdim, nullptr, p0, static_cast<cudaStream_t>(stream));
}
void nt_b200_delta_gate_norm(float* out, const float* o, const float* gate_raw, const float* gain, float eps, int tokens, int heads, int vdim, void* stream) {
    delta_gate_norm(out, o, gate_raw, gain, eps, tokens, heads, vdim, static_cast<cudaStream_t>(stream));
}
// h_next / mu / carried may be null (no fused shift; it takes one row)
void nt_b200_sum_rmsnorm_rows(float* x, float a, const float* y1, float s1, const float* b1, const float* y2, float s2, const float* gain, int rows, int width, float eps,
                              float* h_next, const float* mu, float* carried, int p0, void* stream) {
    sum_rmsnorm_rows(x, a, y1, s1, b1, y2, s2, gain, rows, width, eps, static_cast<cudaStream_t>(stream), h_next, mu, carried, nullptr, p0);
}
void nt_b200_token_shift_rows(float* h, const float* x, const float* mu, float* carried, int rows, int width, int p0, void* stream) {
    token_shift_rows(h, x, mu, carried, rows, width, nullptr, p0, static_cast<cudaStream_t>(stream));
}
// q_gain / k_gain / freq / temp / v_lambda / v_first / v_publish may be null
void nt_b200_head_prep(float* Q, const float* K, const float* V, int heads, int kv_heads, int dim, int vdim, const float* q_gain, const float* k_gain, float eps,
                       int rot_dims, int interleaved, const float* freq, const float* temp, const float* v_lambda, const float* v_first, float* v_publish, void* kc,
                       void* vc, int cache_dtype, int tokens, int p0, void* stream) {
    HeadPrep p;
    p.heads = heads; p.kv_heads = kv_heads; p.dim = dim; p.vdim = vdim; p.q_gain = q_gain; p.k_gain = k_gain; p.eps = eps; p.rot_dims = rot_dims;
    p.interleaved = interleaved; p.freq = freq; p.temp = temp; p.v_lambda = v_lambda; p.v_first = v_first; p.v_publish = v_publish;
    head_prep(Q, K, V, p, kc, vc, (nt::DType)cache_dtype, tokens, nullptr, p0, static_cast<cudaStream_t>(stream));
}
// Full causal grouped-query attention over cache rows with an optional per-head sink (null: none).  talk (null: none): [heads, heads], the
// softmax weights are mixed across heads before head h applies them to its own value head; scratch [tokens, heads, kv_heads * vdim] is then needed.
// one_pass != 0 (or kv_heads * vdim > 512 is not the case): every value head in one pass; else one pass per value head.
void nt_b200_attention_heads(float* out, const float* Q, const void* kc, const void* vc, int cache_dtype, int tokens, int p0, int max_seq, int heads, int kv_heads,
                             int dim, int vdim, float scale, const float* sink, const float* talk, float* scratch, int one_pass, void* stream) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const nt::DType dt = (nt::DType)cache_dtype;
    WindowAttn a;
    a.heads = heads; a.kv_heads = kv_heads; a.dim = dim; a.vdim = vdim; a.scale = scale; a.sink = sink;
    if (!talk) { attention_window(out, Q, kc, vc, dt, tokens, nullptr, p0, max_seq, a, s); return; }
    a.joint_v = 1; a.v_stride = kv_heads * vdim;
    if (one_pass) {
        a.vdim = kv_heads * vdim;
        attention_window(scratch, Q, kc, vc, dt, tokens, nullptr, p0, max_seq, a, s);
        talk_mix(out, scratch, talk, tokens, heads, kv_heads, vdim, (size_t)heads * kv_heads * vdim, (size_t)kv_heads * vdim, (size_t)vdim, s);
        return;
    }
    for (int c = 0; c < kv_heads; c++)
        attention_window(scratch + (size_t)c * tokens * heads * vdim, Q, kc, static_cast<const uint8_t*>(vc) + (size_t)c * vdim * dtype_size(dt), dt, tokens, nullptr, p0,
                         max_seq, a, s);
    talk_mix(out, scratch, talk, tokens, heads, kv_heads, vdim, (size_t)heads * vdim, (size_t)vdim, (size_t)tokens * heads * vdim, s);
}
void nt_b200_side_gate_rows(float* g, const void* E, int dtype, int e_cols, int col0, const int* tokens_dev, int rows, int dim, void* stream) {
    side_gate_rows(g, E, (nt::DType)dtype, e_cols, col0, tokens_dev, rows, dim, static_cast<cudaStream_t>(stream));
}
// Router with sigmoid scores, a choice-only correction (may be null) and a limit to the best `keep` of `groups` runs of neighbours (groups 0: none)
void nt_b200_moe_route_scored(int* sel, float* wt, const float* h, const float* router, const float* correction, int experts, int top, int groups, int keep,
                              int width, int tokens, void* stream) {
    MoeWeights w;
    w.router = router; w.experts = experts; w.top = top; w.width = width; w.sigmoid = true; w.correction = correction; w.groups = groups; w.keep = keep;
    moe_route(sel, wt, nullptr, h, w, tokens, static_cast<cudaStream_t>(stream));
}
// Gated experts.  mode 0: the one-token kernels (scratch: floats [top * ff]); mode 1: the grouped prompt-row kernels (scratch: ints moe work
// table, then floats [tokens * top * (2 * ff + width)])
void nt_b200_moe_glu_experts(float* y, const float* h, const int* sel, const float* wt, const void* const* gate_tab, const void* const* up_tab,
                             const void* const* down_tab, int dtype, int experts, int top, int ff, int width, int tokens, int mode, void* scratch, void* stream) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    MoeWeights w;
    w.gate = gate_tab; w.up = up_tab; w.down = down_tab; w.dtype = (nt::DType)dtype; w.experts = experts; w.top = top; w.ff = ff; w.width = width;
    if (mode == 0) {
        float* act = static_cast<float*>(scratch);
        moe_expert_up_token(act, h, sel, w, s);
        moe_expert_down_token(y, act, sel, wt, nullptr, nullptr, w, s);
        return;
    }
    int* work = static_cast<int*>(scratch);
    const size_t wi = (moe_work_ints(tokens, experts, top) + 3) & ~(size_t)3;
    float* act_rows = reinterpret_cast<float*>(work + wi);
    float* gate_rows = act_rows + (size_t)tokens * top * ff;
    float* y_rows = gate_rows + (size_t)tokens * top * ff;
    moe_group(work, sel, tokens, experts, top, s);
    moe_expert_gate_rows(gate_rows, h, work, w, tokens, s);
    moe_expert_up_rows(act_rows, h, work, w, tokens, s);
    glu_bias_mul(act_rows, gate_rows, act_rows, nullptr, nullptr, tokens * top, ff, false, s);
    moe_expert_down_rows(y_rows, act_rows, work, w, tokens, s);
    moe_combine(y, y_rows, work, wt, nullptr, nullptr, tokens, experts, top, width, s);
}
void nt_b200_glu_mul(float* out, const float* gate, const float* up, long long n, int gelu, void* stream) {
    glu_mul(out, gate, up, (size_t)n, gelu != 0, static_cast<cudaStream_t>(stream));
}
int nt_model_set_tensor(nt_model_t m, const char* name, const void* p, int dtype, size_t pitch) {
    return (m && name && H(m)->model.set_tensor(name, p, (nt::DType)dtype, pitch)) ? 0 : -1;
}
int nt_model_finalize(nt_model_t m) { return (m && H(m)->model.finalize()) ? 0 : -1; }
void nt_model_free(nt_model_t m) { delete H(m); }
int nt_model_get_config(nt_model_t m, nt_model_config* o) {
    if (!m || !o) return -1;
    const ModelConfig& c = H(m)->model.config();
    *o = nt_model_config{c.vocab_size, c.hidden_size, c.intermediate_size, c.n_layers, c.n_heads, c.n_kv_heads, c.head_dim,
                         c.max_seq_len, c.norm_eps, c.rope_theta, c.bos_token_id, c.eos_token_id};
    return 0;
}
int nt_model_forward(nt_model_t m, const int* tokens, int n, int start_pos, float* logits_host) {
    if (!m || !tokens) return -1;
    float* dl = H(m)->model.forward(tokens, n, start_pos);
    if (logits_host)
        NT_CUDA_CHECK(cudaMemcpy(logits_host, dl, sizeof(float) * (size_t)H(m)->model.config().vocab_size, cudaMemcpyDeviceToHost));
    return 0;
}
int nt_model_forward_async(nt_model_t m, const int* tokens, int n, int start_pos) {
    if (!m || !tokens) return -1;
    H(m)->model.forward_async(tokens, n, start_pos);
    return 0;
}
int nt_model_sync(nt_model_t m) { return m ? H(m)->model.sync() : -1; }
float* nt_model_logits_device(nt_model_t m) { return m ? H(m)->model.logits_device() : nullptr; }
void* nt_model_stream(nt_model_t m) { return m ? (void*)H(m)->model.stream() : nullptr; }
int nt_model_argmax(nt_model_t m) { return m ? H(m)->model.argmax_last() : -1; }
void nt_model_clear_kv(nt_model_t m) { if (m) H(m)->model.clear_kv(); }
void nt_model_set_prefill_min_tokens(nt_model_t m, int n) { if (m) H(m)->model.set_prefill_min_tokens(n); }
void nt_model_use_graph(nt_model_t m, int on) { if (m) H(m)->model.set_use_graph(on != 0); }
unsigned long long nt_model_bytes_per_token(nt_model_t m, int ctx) { return m ? H(m)->model.bytes_per_token(ctx) : 0; }
int nt_model_sample(nt_model_t m, float temperature, int top_k, float top_p, float repeat_penalty, const int* recent_window, int n_window,
                    float r) {
    return m ? H(m)->model.sample_last(temperature, top_k, top_p, repeat_penalty, recent_window, n_window, r) : -1;
}
float nt_sampler_uniform(uint64_t seed, int n_draws_before) {
    SamplerConfig sc;
    sc.seed = seed;
    Sampler s;
    s.init(sc);
    for (int i = 0; i < n_draws_before; i++) s.draw();
    return s.draw();
}
void nt_model_use_megakernel(nt_model_t m, int on) { if (m) H(m)->model.set_use_megakernel(on != 0); }
double nt_model_load_seconds(nt_model_t m) { return m ? H(m)->model.load_seconds() : 0.0; }
int nt_model_tp_exchange(nt_model_t m) { return m ? H(m)->model.tp_exchange_kind() : 0; }
int nt_model_megakernel_active(nt_model_t m) { return (m && H(m)->model.megakernel_active()) ? 1 : 0; }
int nt_model_megakernel_plan(nt_model_t m, int* kinds, int cap) {
    if (!m) return -1;
    return H(m)->model.mega_plan_kinds(kinds, cap);
}
void nt_model_megakernel_trace(nt_model_t m, int on) { if (m) H(m)->model.mega_trace(on != 0); }
long long nt_model_megakernel_trace_read(nt_model_t m, unsigned long long* out_host, size_t cap) {
    return m ? (long long)H(m)->model.mega_trace_read(out_host, cap) : -1;
}
long long nt_model_debug_read(nt_model_t m, const char* name, float* out_host, size_t cap) {
    if (!m || !name) return -1;
    size_t n = 0;
    const float* p = H(m)->model.mega_debug_buffer(name, &n);
    if (!p) return -1;
    NT_CUDA_CHECK(cudaStreamSynchronize(H(m)->model.stream()));
    if (out_host) NT_CUDA_CHECK(cudaMemcpy(out_host, p, sizeof(float) * (n < cap ? n : cap), cudaMemcpyDeviceToHost));
    return (long long)n;
}

// Host-only: builds the persistent kernel's per-token program for a model of the given (per-rank) shape with placeholder
// addresses and replays its schedule on the CPU (decode_mega.h: mega_make_plan + mega_check_plan).  No CUDA call.
int nt_mega_plan_selftest(const nt_model_config* c, int tp_rank, int tp_size, const int* layer_dtypes, int head_dtype, int grid,
                          int split_fixed, int fuse, int* info, char* msg, size_t cap) {
    auto say = [&](const std::string& m) { if (msg && cap) { snprintf(msg, cap, "%s", m.c_str()); } };
    if (!c || !layer_dtypes || tp_size < 1 || c->n_heads % tp_size || c->n_kv_heads % tp_size || c->intermediate_size % tp_size) {
        say("bad arguments");
        return -1;
    }
    MegaModelView mv;
    mv.hidden = c->hidden_size; mv.nh = c->n_heads / tp_size; mv.nkv = c->n_kv_heads / tp_size; mv.hd = c->head_dim;
    mv.inter = c->intermediate_size / tp_size; mv.max_seq = c->max_seq_len; mv.n_layers = c->n_layers;
    mv.eps = c->norm_eps; mv.theta = c->rope_theta; mv.tp_rank = tp_rank; mv.tp_size = tp_size;
    uintptr_t next = 0x10000000;                       // placeholder device addresses, 256-byte aligned
    auto place = [&](size_t bytes) { void* p = reinterpret_cast<void*>(next); next += (bytes + 255) & ~(size_t)255; return p; };
    auto weight = [&](int dt, int rows, int cols, bool col_shard) {
        MegaWeight w;
        w.dtype = (nt::DType)dt; w.rows = rows; w.cols = cols;
        const size_t rb = nt::dtype_row_size(w.dtype, (size_t)cols);
        w.pitch = col_shard ? ((rb + 15) & ~(size_t)15) : rb;      // Model::upload pads column shards to a 16-byte pitch
        w.ptr = place(w.pitch * (size_t)std::max(rows, 1));
        return w;
    };
    const int qdim = mv.nh * mv.hd, kvdim = mv.nkv * mv.hd;
    for (int l = 0; l < mv.n_layers; l++) {
        const int* d = layer_dtypes + 7 * l;
        MegaLayerView L;
        L.attn_norm = static_cast<const float*>(place((size_t)mv.hidden * 4));
        L.ffn_norm = static_cast<const float*>(place((size_t)mv.hidden * 4));
        L.wq = weight(d[0], qdim, mv.hidden, false); L.wk = weight(d[1], kvdim, mv.hidden, false); L.wv = weight(d[2], kvdim, mv.hidden, false);
        L.wo = weight(d[3], mv.hidden, qdim, tp_size > 1);
        L.gate = weight(d[4], mv.inter, mv.hidden, false); L.up = weight(d[5], mv.inter, mv.hidden, false);
        L.down = weight(d[6], mv.hidden, mv.inter, tp_size > 1);
        L.kc = place((size_t)mv.max_seq * kvdim * 2); L.vc = place((size_t)mv.max_seq * kvdim * 2);
        mv.layers.push_back(L);
    }
    const int vl = (c->vocab_size + tp_size - 1) / tp_size;
    const int vrows = tp_size == 1 ? c->vocab_size : std::max(0, std::min(vl, c->vocab_size - tp_rank * vl));
    mv.head = weight(head_dtype, vrows, mv.hidden, false);
    mv.out_norm = static_cast<const float*>(place((size_t)mv.hidden * 4));
    mv.logits = static_cast<float*>(place((size_t)vl * 4));
    mv.step = static_cast<const int*>(place(8));
    MegaBuffers B;
    B.hid[0] = static_cast<float*>(place((size_t)mv.hidden * 4)); B.hid[1] = static_cast<float*>(place((size_t)mv.hidden * 4));
    B.q = static_cast<float*>(place((size_t)qdim * 4)); B.k = static_cast<float*>(place((size_t)kvdim * 4));
    B.v = static_cast<float*>(place((size_t)kvdim * 4)); B.act = static_cast<float*>(place((size_t)mv.inter * 4));
    B.xq_h = static_cast<int8_t*>(place(xq_bytes(mv.hidden))); B.xq_a = static_cast<int8_t*>(place(xq_bytes(qdim)));
    B.xq_i = static_cast<int8_t*>(place(xq_bytes(mv.inter)));
    B.cnt_quant = static_cast<unsigned*>(place((size_t)mv.inter / 32 * 4 + 4)); B.cnt_attn = static_cast<unsigned*>(place((size_t)mv.nh * 4 + 4));
    B.cnt_norm = static_cast<unsigned*>(place((size_t)mv.hidden / 32 * 4 + 4)); B.ssq = static_cast<float*>(place((size_t)mv.hidden / 32 * 4 + 4));
    MegaPlan pl;
    std::string why;
    if (!mega_make_plan(mv, B, grid, split_fixed, fuse, &pl, &why)) { say(why); return 1; }
    if (info) {
        int n_gemv = 0, min_warps = 99, min_stages = 99, n_exchange = 0;
        for (const MegaPhase& ph : pl.phases) {
            if (ph.kind == MPH_GEMV) { n_gemv++; min_warps = std::min(min_warps, ph.warps); min_stages = std::min(min_stages, ph.stages); }
            if (ph.barrier == MBAR_EXCHANGE) n_exchange++;
        }
        info[0] = (int)pl.phases.size(); info[1] = pl.n_body; info[2] = n_gemv; info[3] = min_warps; info[4] = min_stages;
        info[5] = n_exchange; info[6] = pl.n_splits_max; info[7] = pl.max_split;
    }
    const std::string bad = mega_check_plan(pl, grid, tp_size);
    if (!bad.empty()) { say(bad); return 2; }
    say("ok");
    return 0;
}

int nt_gguf_describe(const char* path, char* out, size_t cap) {
    if (!path || !out || !cap) return -1;
    GGUFFile f;
    if (!f.open(path)) return -1;
    const ModelConfig& c = f.config();
    std::string j = "{";
    auto kv = [&](const char* k, long long v) { j += "\"" + std::string(k) + "\": " + std::to_string(v) + ", "; };
    kv("vocab_size", c.vocab_size); kv("hidden_size", c.hidden_size); kv("intermediate_size", c.intermediate_size);
    kv("n_layers", c.n_layers); kv("n_heads", c.n_heads); kv("n_kv_heads", c.n_kv_heads); kv("head_dim", c.head_dim);
    kv("max_seq_len", c.max_seq_len); kv("bos_token_id", c.bos_token_id); kv("eos_token_id", c.eos_token_id);
    kv("n_vocab_tokens", (long long)f.vocab().tokens.size()); kv("data_offset", (long long)f.data_offset());
    char fl[96];
    snprintf(fl, sizeof(fl), "\"norm_eps\": %.9g, \"rope_theta\": %.9g, ", c.norm_eps, c.rope_theta);
    j += fl;
    j += "\"architecture\": \"" + c.architecture + "\", \"tensors\": [";
    bool first = true;
    for (const auto& t : f.tensors()) {
        if (!first) j += ", ";
        first = false;
        j += "{\"name\": \"" + t.name + "\", \"dtype\": " + std::to_string((int)t.dtype) + ", \"offset\": " + std::to_string(t.offset) +
             ", \"nbytes\": " + std::to_string(t.nbytes) + ", \"shape\": [";
        for (size_t d = 0; d < t.shape.size(); d++) j += (d ? ", " : "") + std::to_string(t.shape[d]);
        j += "]}";
    }
    j += "]}";
    if (j.size() + 1 > cap) return -1;
    memcpy(out, j.c_str(), j.size() + 1);
    return (int)j.size();
}
int nt_tokenize(const char* gguf_path, const char* text, int add_bos, int* ids, int cap) {
    if (!gguf_path || !text) return -1;
    GGUFFile f;
    if (!f.open(gguf_path)) return -1;
    Tokenizer t;
    t.init(f.vocab(), f.config().bos_token_id, f.config().eos_token_id);
    std::vector<int> v = t.encode(text, add_bos != 0);
    for (int i = 0; i < (int)v.size() && i < cap; i++) ids[i] = v[(size_t)i];
    return (int)v.size();
}
int nt_detokenize(const char* gguf_path, const int* ids, int n, char* out, size_t cap) {
    if (!gguf_path || !out || !cap) return -1;
    GGUFFile f;
    if (!f.open(gguf_path)) return -1;
    Tokenizer t;
    t.init(f.vocab(), f.config().bos_token_id, f.config().eos_token_id);
    std::string s = t.decode(std::vector<int>(ids, ids + n));
    if (s.size() + 1 > cap) return -1;
    memcpy(out, s.data(), s.size());
    out[s.size()] = 0;
    return (int)s.size();
}
int nt_sample_token(const float* logits, int n, float temperature, int top_k, float top_p, float repeat_penalty,
                    int repeat_window, const int* recent, int n_recent, uint64_t seed) {
    if (!logits || n <= 0) return -1;
    SamplerConfig sc;
    sc.temperature = temperature; sc.top_k = top_k; sc.top_p = top_p; sc.repeat_penalty = repeat_penalty;
    sc.repeat_window = repeat_window; sc.seed = seed;
    Sampler s;
    s.init(sc);
    std::vector<float> l(logits, logits + n);
    s.apply_repeat_penalty(l.data(), n, std::vector<int>(recent, recent + (recent ? n_recent : 0)));
    return s.sample(l.data(), n);
}

int nt_tp_unique_id(void* out128) { return TPComm::unique_id(out128) ? 0 : -1; }
int nt_tp_init(nt_model_t m, const void* id128, int rank, int size) {
    if (!m) return -1;
    auto c = std::make_unique<TPComm>();
    if (!c->init(id128, rank, size)) return -2;
    {   // NCCL builds its channels lazily on the first collective (allocations, IPC handles): do that here, eagerly,
        // so that nothing of the sort happens inside the decode step's CUDA-graph capture.
        cudaStream_t st = H(m)->model.stream();
        float* tmp = nullptr;
        NT_CUDA_CHECK(cudaMalloc(&tmp, sizeof(float) * 1024 * (size_t)(size + 1)));
        NT_CUDA_CHECK(cudaMemsetAsync(tmp, 0, sizeof(float) * 1024 * (size_t)(size + 1), st));
        c->all_reduce_sum(tmp, 1024, st);
        c->all_gather(tmp, tmp + 1024, 1024, st);
        NT_CUDA_CHECK(cudaStreamSynchronize(st));
        NT_CUDA_CHECK(cudaFree(tmp));
    }
    H(m)->model.set_comm(c.get());
    H(m)->comm = std::move(c);
    return 0;
}
}  // extern "C"
