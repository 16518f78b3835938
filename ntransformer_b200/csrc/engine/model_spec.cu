// model_spec.cu — the resident model for families described layer by layer (engine/layer_spec.h, engine/model_registry.h):
// loading a model folder, the per-token decode step and the batched prompt pass, written against LayerSpec so that the
// mechanisms (windowed / soft-capped attention, whole-projection q/k norm, parallel block with layer scale, GELU-gated unit,
// layers sharing tensors) combine freely.  Same buffers, stream, CUDA-graph replay, logits and sampler as the GGUF families
// (engine/model.cu); the KV cache is per layer because layers may differ in width.  Layers of BlockForm::SUM_NORM live in
// engine/model_sumnorm.cu.
//
// Arithmetic: the residual stream, norms, softmax and every accumulation are F32.  Weights stay in their stored dtype (BF16)
// and are widened in registers, or — exact 32-bit mode — are widened once at load.  The cache stores BF16 (F32 in exact mode).
//
// Launches per layer and decoded token (6):  [RMS norm + q/k/v GEMV, one launch]  [q/k norm + cache write]  [window attention]
//   [RMS norm + gate/up GEMV + GELU gate]  [o GEMV: x += m * ls1 * .]  [down GEMV: x += m * ls2 * .]   — the block norm lives in
//   the GEMV prologues, every residual update, gain and activation in a GEMV epilogue.
#include "model.h"
#include "safetensors.h"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <sys/stat.h>

namespace nt { namespace b200 {

namespace {
template <typename T> T* dmalloc(size_t n) {
    T* p = nullptr;
    NT_CUDA_CHECK(cudaMalloc(&p, std::max<size_t>(n, 1) * sizeof(T)));
    return p;
}
__global__ void iota_spec_kernel(int* out, int first, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = first + i;
}
constexpr int SPEC_PREFILL_CHUNK = 2048;
GemvMat mat_of(const Weight& w, float* y) { GemvMat m; m.W = w.ptr; m.y = y; m.out = w.rows; m.dtype = w.dtype; m.row_pitch = w.pitch; return m; }
}  // namespace

bool Model::load(const std::string& path, int max_context) {
    struct stat st;
    if (stat(path.c_str(), &st) == 0 && S_ISDIR(st.st_mode)) return load_dir(path, max_context);
    return load_gguf(path, max_context);
}

bool Model::bind_slot(TensorSlot slot, int layer, const void* ptr, DType dt, int rows, int cols, size_t pitch, int index, int branch) {
    auto W = [&](Weight& w) {
        if (!dense_dtype(dt)) return false;
        w.ptr = ptr; w.dtype = dt; w.rows = rows; w.cols = cols; w.pitch = pitch ? pitch : dtype_row_size(dt, (size_t)cols); w.owned = false;
        return true;
    };
    auto V = [&](const float*& v) { if (dt != DType::F32) return false; v = static_cast<const float*>(ptr); return true; };
    if (slot == TensorSlot::EMBED) return W(embd_);
    if (slot == TensorSlot::HEAD) return W(head_);
    if (slot == TensorSlot::OUT_NORM) return V(out_norm_);
    if (slot == TensorSlot::SIDE_EMBED) return W(side_embd_);
    if (layer < 0 || layer >= cfg_.n_layers) return false;
    LayerWeights* Lp = &layers_[(size_t)layer];
    if (branch >= 0) {                      // a tensor of one of the mixers that sit side by side
        const size_t nb = cfg_.layers[(size_t)layer].branches.size();
        if ((size_t)branch >= nb) return false;
        if (Lp->branch.size() != nb) Lp->branch.assign(nb, LayerWeights{});
        Lp = &Lp->branch[(size_t)branch];
    }
    LayerWeights& L = *Lp;
    switch (slot) {
        case TensorSlot::SHIFT_MU: return V(L.shift_mu);
        case TensorSlot::Q_BIAS: return V(L.q_bias);
        case TensorSlot::K_BIAS: return V(L.k_bias);
        case TensorSlot::V_BIAS: return V(L.v_bias);
        case TensorSlot::O_BIAS: return V(L.o_bias);
        case TensorSlot::Q_CONV: return V(L.q_conv);
        case TensorSlot::K_CONV: return V(L.k_conv);
        case TensorSlot::V_CONV: return V(L.v_conv);
        case TensorSlot::HEAD_TEMP: return V(L.head_temp);
        case TensorSlot::TALK: return V(L.talk);
        case TensorSlot::SINK: return V(L.sink);
        case TensorSlot::V_MIX: return V(L.v_mix);
        case TensorSlot::DELTA_BETA: return W(L.d_beta);
        case TensorSlot::DELTA_A1: return W(L.d_a1);
        case TensorSlot::DELTA_A2: return W(L.d_a2);
        case TensorSlot::DELTA_G1: return W(L.d_g1);
        case TensorSlot::DELTA_G2: return W(L.d_g2);
        case TensorSlot::DELTA_DT_BIAS: return V(L.d_dt_bias);
        case TensorSlot::DELTA_A_LOG: return V(L.d_a_log);
        case TensorSlot::DELTA_NORM: return V(L.d_norm);
        case TensorSlot::NORM1: return V(L.attn_norm);
        case TensorSlot::NORM2: return V(L.ffn_norm);
        case TensorSlot::Q_NORM: return V(L.q_norm);
        case TensorSlot::K_NORM: return V(L.k_norm);
        case TensorSlot::LS1: return V(L.ls1);
        case TensorSlot::LS2: return V(L.ls2);
        case TensorSlot::WQ: return W(L.wq);
        case TensorSlot::WK: return W(L.wk);
        case TensorSlot::WV: return W(L.wv);
        case TensorSlot::WO: return W(L.wo);
        case TensorSlot::GATE: return W(L.gate);
        case TensorSlot::UP: return W(L.up);
        case TensorSlot::DOWN: return W(L.down);
        case TensorSlot::LQ1: return V(L.lq1);
        case TensorSlot::LK1: return V(L.lk1);
        case TensorSlot::LQ2: return V(L.lq2);
        case TensorSlot::LK2: return V(L.lk2);
        case TensorSlot::HC1_IN: return V(L.hc_in[0]);
        case TensorSlot::HC1_OUT: return V(L.hc_out[0]);
        case TensorSlot::HC1_MIX: return V(L.hc_mix[0]);
        case TensorSlot::HC2_IN: return V(L.hc_in[1]);
        case TensorSlot::HC2_OUT: return V(L.hc_out[1]);
        case TensorSlot::HC2_MIX: return V(L.hc_mix[1]);
        case TensorSlot::ROUTER: return V(L.router);
        case TensorSlot::SHARED_GATE: return V(L.shared_gate);
        case TensorSlot::SHARED_UP: return W(L.sh_up);
        case TensorSlot::SHARED_DOWN: return W(L.sh_down);
        case TensorSlot::W_DQ: return W(L.w_dq);
        case TensorSlot::W_UQ: return W(L.w_uq);
        case TensorSlot::W_DKV: return W(L.w_dkv);
        case TensorSlot::W_UK: return W(L.w_uk);
        case TensorSlot::W_UV: return W(L.w_uv);
        case TensorSlot::DQ_NORM: return V(L.dq_norm);
        case TensorSlot::DKV_NORM: return V(L.dkv_norm);
        case TensorSlot::SSM_IN: return W(L.ssm_in);
        case TensorSlot::SSM_CONV: return V(L.ssm_conv);
        case TensorSlot::SSM_CONV_B: return V(L.ssm_conv_b);
        case TensorSlot::SSM_DT_BIAS: return V(L.ssm_dt_bias);
        case TensorSlot::SSM_A_LOG: return V(L.ssm_a_log);
        case TensorSlot::SSM_D: return V(L.ssm_d);
        case TensorSlot::SSM_NORM: return V(L.ssm_norm);
        case TensorSlot::GATE_B: return V(L.gate_b);
        case TensorSlot::UP_B: return V(L.up_b);
        case TensorSlot::DOWN_B: return V(L.down_b);
        case TensorSlot::ROUTE_CORRECTION: return V(L.route_corr);
        case TensorSlot::SIDE_GATE: return W(L.side_gate);
        case TensorSlot::SIDE_PROJ: return W(L.side_proj);
        case TensorSlot::SIDE_NORM: return V(L.side_norm);
        case TensorSlot::EXPERT_UP: case TensorSlot::EXPERT_DOWN: case TensorSlot::EXPERT_GATE: {
            const int E = cfg_.layers[(size_t)layer].experts;
            if (index < 0 || index >= E) return false;
            std::vector<Weight>& v = slot == TensorSlot::EXPERT_UP ? L.e_up : (slot == TensorSlot::EXPERT_GATE ? L.e_gate : L.e_down);
            if ((int)v.size() != E) v.assign((size_t)E, Weight{});
            return W(v[(size_t)index]);
        }
        default: return false;
    }
}

// config.json -> family -> LayerSpecs; model.safetensors -> one device arena.  Matrices keep their stored dtype (widened to F32
// in exact mode), gain vectors always become F32.  Shapes are checked against the configuration before anything is uploaded.
bool Model::load_dir(const std::string& dir, int max_context) {
    const auto t_start = std::chrono::steady_clock::now();
    fprintf(stderr, "Loading model folder: %s\n", dir.c_str());
    ModelConfig cfg;
    const ModelFamily* fam = nullptr;
    if (!read_model_dir(dir, cfg, &fam)) return false;
    cfg.max_seq_len = std::max(1, max_context);
    cfg.print();
    SafeTensorsFile f;
    if (!f.open(dir + "/model.safetensors")) return false;
    if (fam->sizes_from_tensors) {          // sizes only a tensor's shape gives
        std::string err;
        const TensorShapeFn shape_of = [&](const std::string& name, std::vector<int64_t>& shape) {
            const SafeTensorInfo* ti = f.find(name);
            if (ti) shape = ti->shape;
            return ti != nullptr;
        };
        if (!fam->sizes_from_tensors(cfg, shape_of, err)) { fprintf(stderr, "model: %s\n", err.c_str()); return false; }
    }
    init(cfg, 0, 1);
    const std::vector<TensorBinding> plan = fam->tensors(cfg_);
    struct Job { const SafeTensorInfo* ti; const TensorBinding* b; size_t off; DType dst; };
    std::vector<Job> jobs;
    size_t arena = 0, stage_max = 0;
    for (const TensorBinding& b : plan) {
        const SafeTensorInfo* ti = f.find(b.name);
        if (!ti) { fprintf(stderr, "model: tensor not found: %s\n", b.name.c_str()); return false; }
        const bool vec = b.rows == 1 && ti->shape.size() == 1, scalar = b.rows == 1 && b.cols == 1 && ti->shape.empty();
        if (!dense_dtype(ti->dtype) || !(scalar || (vec ? ti->shape[0] == b.cols : (ti->shape.size() == 2 && ti->shape[0] == b.rows && ti->shape[1] == b.cols)))) {
            fprintf(stderr, "model: tensor %s does not have the shape the configuration needs [%d x %d]\n", b.name.c_str(), b.rows, b.cols);
            return false;
        }
        const bool is_vec = slot_is_f32_table(b.slot);
        const DType dst = (is_vec || exact32_) ? DType::F32 : ti->dtype;
        jobs.push_back({ti, &b, arena, dst});
        arena += ((size_t)b.rows * b.cols * dtype_size(dst) + 255) & ~(size_t)255;
        stage_max = std::max(stage_max, (size_t)(ti->end - ti->begin));
    }
    uint8_t* base = nullptr;
    if (cudaMalloc(&base, std::max<size_t>(arena, 256)) != cudaSuccess) {
        cudaGetLastError();
        fprintf(stderr, "model: cannot allocate %.2f GB of device memory for the weights\n", arena / 1e9);
        return false;
    }
    owned_.push_back(base);
    cudaStream_t st = nullptr;
    NT_CUDA_CHECK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    uint8_t* host = nullptr;
    NT_CUDA_CHECK(cudaHostAlloc((void**)&host, std::max<size_t>(stage_max, 16), cudaHostAllocDefault));
    uint8_t* dev_stage = dmalloc<uint8_t>(stage_max);
    bool ok = true;
    for (const Job& j : jobs) {
        const size_t bytes = (size_t)(j.ti->end - j.ti->begin), n = (size_t)j.b->rows * j.b->cols;
        if (!f.read(*j.ti, host)) { fprintf(stderr, "model: short read of %s\n", j.b->name.c_str()); ok = false; break; }
        if (j.dst == j.ti->dtype) NT_CUDA_CHECK(cudaMemcpyAsync(base + j.off, host, bytes, cudaMemcpyHostToDevice, st));
        else {
            NT_CUDA_CHECK(cudaMemcpyAsync(dev_stage, host, bytes, cudaMemcpyHostToDevice, st));
            dense_to_f32(reinterpret_cast<float*>(base + j.off), dev_stage, j.ti->dtype, n, st);
        }
        NT_CUDA_CHECK(cudaStreamSynchronize(st));          // the staging buffers are reused by the next tensor
        if (!bind_slot(j.b->slot, j.b->layer, base + j.off, j.dst, j.b->rows, j.b->cols, 0, j.b->index, j.b->branch)) { fprintf(stderr, "model: cannot bind %s\n", j.b->name.c_str()); ok = false; break; }
    }
    cudaFreeHost(host);
    cudaFree(dev_stage);
    cudaStreamDestroy(st);
    if (!ok || !finalize()) return false;
    load_seconds_ = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_start).count();
    fprintf(stderr, "  Loaded %d layers (%s weights, %s cache): %.3f GB resident, %.2f s\nModel loaded successfully!\n", cfg_.n_layers,
            exact32_ ? "F32" : "stored-dtype", dtype_name(cache_dt_), arena / 1e9, load_seconds_);
    return true;
}

bool Model::finalize_spec() {
    const int hidden = cfg_.hidden_size, max_seq = cfg_.max_seq_len;
    if (!embd_.ptr || !out_norm_ || !head_.ptr) { fprintf(stderr, "model: embedding / final norm / head missing\n"); return false; }
    int qmax = 1, kmax = 1, vmax = 1, omax = 1, ffmax = 1, mapmax = 1, moe_act = 1, topmax = 1;
    for (int i = 0; i < cfg_.n_layers; i++) {
        const LayerSpec& S = cfg_.layers[(size_t)i];
        const LayerWeights& L = layer_weights(i);
        if (S.form == BlockForm::SUM_NORM) {
            if (!finalize_sumnorm_layer(i)) return false;
            ffmax = std::max(ffmax, S.ff);
            continue;
        }
        if (S.form == BlockForm::POST_NORM) {
            LayerWeights& M = layers_[(size_t)i];
            bool ok = L.attn_norm && L.wo.ptr;
            if (S.mixer == MixerKind::ATTN_LATENT)
                ok = ok && L.w_dq.ptr && L.dq_norm && L.w_uq.ptr && L.w_uk.ptr && L.w_uv.ptr && (S.kv_from >= 0 || (L.w_dkv.ptr && L.dkv_norm));
            else if (S.mixer == MixerKind::SSM_SCAN)
                ok = ok && L.ssm_in.ptr && L.ssm_conv && L.ssm_conv_b && L.ssm_dt_bias && L.ssm_a_log && L.ssm_d && L.ssm_norm;
            else { fprintf(stderr, "model: layer %d: this mixer has no post-norm kernels\n", i); return false; }
            if (S.ff > 0 && S.ff_kind == FfKind::GLU) ok = ok && L.ffn_norm && L.gate.ptr && L.up.ptr && L.down.ptr && (!S.ff_bias || (L.gate_b && L.up_b && L.down_b));
            if (S.ff > 0 && S.ff_kind == FfKind::MOE_GLU) {
                ok = ok && L.ffn_norm && L.router && (!S.route.correction || L.route_corr) && (int)L.e_up.size() == S.experts && (int)L.e_down.size() == S.experts &&
                     (int)L.e_gate.size() == S.experts;
                const DType edt = ok ? L.e_up[0].dtype : DType::F32;
                for (int e = 0; ok && e < S.experts; e++)
                    ok = L.e_up[(size_t)e].ptr && L.e_down[(size_t)e].ptr && L.e_gate[(size_t)e].ptr && L.e_up[(size_t)e].dtype == edt && L.e_down[(size_t)e].dtype == edt &&
                         L.e_gate[(size_t)e].dtype == edt;
            }
            if (S.ff > 0 && S.ff_kind == FfKind::MOE_RELU2) { fprintf(stderr, "model: layer %d: this feed-forward has no post-norm kernels\n", i); return false; }
            if (cfg_.side_dim > 0) ok = ok && side_embd_.ptr && L.side_gate.ptr && L.side_proj.ptr && L.side_norm;
            if (!ok) { fprintf(stderr, "model: layer %d is missing tensors\n", i); return false; }
            if (S.mixer == MixerKind::ATTN_LATENT && S.latent.kv_rank > 512) { fprintf(stderr, "model: layer %d: latents wider than 512 are not covered\n", i); return false; }
            if (S.mixer == MixerKind::SSM_SCAN) {
                if (S.scan.state > 256) { fprintf(stderr, "model: layer %d: scan states larger than 256 are not covered\n", i); return false; }
                const size_t ch = (size_t)S.heads * S.vdim + 2 * (size_t)S.scan.groups * S.scan.state;
                M.conv_state = dmalloc<float>((size_t)std::max(1, S.scan.conv - 1) * ch);
                M.ssm_state = dmalloc<float>((size_t)S.heads * S.vdim * S.scan.state);
                NT_CUDA_CHECK(cudaMemset(M.conv_state, 0, sizeof(float) * (size_t)std::max(1, S.scan.conv - 1) * ch));
                NT_CUDA_CHECK(cudaMemset(M.ssm_state, 0, sizeof(float) * (size_t)S.heads * S.vdim * S.scan.state));
            }
            if (S.ff > 0 && S.ff_kind == FfKind::MOE_GLU) {
                std::vector<const void*> up((size_t)S.experts), down((size_t)S.experts), gate((size_t)S.experts);
                for (int e = 0; e < S.experts; e++) { up[(size_t)e] = L.e_up[(size_t)e].ptr; down[(size_t)e] = L.e_down[(size_t)e].ptr; gate[(size_t)e] = L.e_gate[(size_t)e].ptr; }
                M.e_up_tab = dmalloc<const void*>((size_t)S.experts);
                M.e_down_tab = dmalloc<const void*>((size_t)S.experts);
                M.e_gate_tab = dmalloc<const void*>((size_t)S.experts);
                NT_CUDA_CHECK(cudaMemcpy(M.e_up_tab, up.data(), sizeof(void*) * up.size(), cudaMemcpyHostToDevice));
                NT_CUDA_CHECK(cudaMemcpy(M.e_down_tab, down.data(), sizeof(void*) * down.size(), cudaMemcpyHostToDevice));
                NT_CUDA_CHECK(cudaMemcpy(M.e_gate_tab, gate.data(), sizeof(void*) * gate.size(), cudaMemcpyHostToDevice));
                moe_act = std::max(moe_act, S.top * S.ff);
                topmax = std::max(topmax, S.top);
            }
            continue;
        }
        if (S.form == BlockForm::STREAMS) {
            LayerWeights& M = layers_[(size_t)i];
            const bool kv_ok = S.kv_from >= 0 || (L.wk.ptr && L.wv.ptr);
            bool ok = L.attn_norm && L.wq.ptr && kv_ok && L.wo.ptr && (S.maps == 1 || (L.lq1 && L.lk1 && L.lq2 && L.lk2));
            if (cfg_.streams > 0) ok = ok && L.hc_in[0] && L.hc_out[0] && L.hc_mix[0] && (S.ff == 0 || (L.hc_in[1] && L.hc_out[1] && L.hc_mix[1]));
            if (S.ff > 0) {
                ok = ok && S.ff_kind == FfKind::MOE_RELU2 && L.ffn_norm && L.router && (int)L.e_up.size() == S.experts && (int)L.e_down.size() == S.experts;
                const DType edt = ok ? L.e_up[0].dtype : DType::F32;
                for (int e = 0; ok && e < S.experts; e++) ok = L.e_up[(size_t)e].ptr && L.e_down[(size_t)e].ptr && L.e_up[(size_t)e].dtype == edt && L.e_down[(size_t)e].dtype == edt;
                if (S.shared_ff > 0) ok = ok && L.sh_up.ptr && L.sh_down.ptr && L.shared_gate && L.sh_up.dtype == edt && L.sh_down.dtype == edt;
            }
            if (!ok) { fprintf(stderr, "model: layer %d is missing tensors\n", i); return false; }
            if (S.mixer != MixerKind::ATTN_WINDOW || S.maps < 1 || S.maps > 2) { fprintf(stderr, "model: layer %d: this mixer has no layer-spec kernels yet\n", i); return false; }
            if (S.vdim > 256) { fprintf(stderr, "model: layer %d: value heads wider than 256 are not covered\n", i); return false; }
            if (S.ff > 0) {                                   // device tables of the experts' matrices
                std::vector<const void*> up((size_t)S.experts), down((size_t)S.experts);
                for (int e = 0; e < S.experts; e++) { up[(size_t)e] = L.e_up[(size_t)e].ptr; down[(size_t)e] = L.e_down[(size_t)e].ptr; }
                M.e_up_tab = dmalloc<const void*>((size_t)S.experts);
                M.e_down_tab = dmalloc<const void*>((size_t)S.experts);
                NT_CUDA_CHECK(cudaMemcpy(M.e_up_tab, up.data(), sizeof(void*) * up.size(), cudaMemcpyHostToDevice));
                NT_CUDA_CHECK(cudaMemcpy(M.e_down_tab, down.data(), sizeof(void*) * down.size(), cudaMemcpyHostToDevice));
                moe_act = std::max(moe_act, S.top * S.ff + S.shared_ff);
                topmax = std::max(topmax, S.top);
            }
            if (S.rot.dims > 0) {
                const RotarySpec& R = S.rot;
                std::vector<float> f((size_t)std::max(1, R.dims / 2));
                M.rot_mag = rotary_table(f.data(), R.dims, R.base, R.factor, R.original, R.fast, R.slow);
                M.rot_freq = dmalloc<float>(f.size());
                NT_CUDA_CHECK(cudaMemcpy(M.rot_freq, f.data(), sizeof(float) * f.size(), cudaMemcpyHostToDevice));
            }
            qmax = std::max(qmax, S.heads * S.maps * S.dim); kmax = std::max(kmax, S.kv_heads * S.maps * S.dim); vmax = std::max(vmax, S.kv_heads * S.vdim);
            omax = std::max(omax, S.heads * S.vdim); mapmax = std::max(mapmax, S.heads * S.maps * S.vdim);
            continue;
        }
        const bool mlp_ok = S.ff == 0 || (L.gate.ptr && L.up.ptr && L.down.ptr && (!S.layer_scale || L.ls2));
        if (!L.attn_norm || !L.wq.ptr || !L.wk.ptr || !L.wv.ptr || !L.wo.ptr || !mlp_ok || (S.layer_scale && !L.ls1) ||
            (S.qk_norm == QKNorm::WHOLE && (!L.q_norm || !L.k_norm))) {
            fprintf(stderr, "model: layer %d is missing tensors\n", i);
            return false;
        }
        if (S.mixer != MixerKind::ATTN_WINDOW || S.form != BlockForm::PARALLEL) { fprintf(stderr, "model: layer %d: this mixer / block form has no layer-spec kernels yet\n", i); return false; }
        if (S.vdim > 256) { fprintf(stderr, "model: layer %d: value heads wider than 256 are not covered\n", i); return false; }
        qmax = std::max(qmax, S.heads * S.dim); kmax = std::max(kmax, S.kv_heads * S.dim); vmax = std::max(vmax, S.kv_heads * S.vdim);
        omax = std::max(omax, S.heads * S.vdim); ffmax = std::max(ffmax, S.ff);
    }
    cache_dt_ = exact32_ ? DType::F32 : DType::BF16;
    NT_CUDA_CHECK(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
    if (cfg_.norm_gain_offset != 0.f) {
        // gains stored around zero: the offset is added once, into F32 copies the kernels read as plain gains
        auto fold = [&](const float*& g) {
            if (!g) return;
            std::vector<float> h((size_t)hidden);
            NT_CUDA_CHECK(cudaMemcpy(h.data(), g, sizeof(float) * h.size(), cudaMemcpyDeviceToHost));
            for (float& v : h) v += cfg_.norm_gain_offset;
            float* d = dmalloc<float>(h.size());
            NT_CUDA_CHECK(cudaMemcpy(d, h.data(), sizeof(float) * h.size(), cudaMemcpyHostToDevice));
            owned_.push_back(d);
            g = d;
        };
        fold(out_norm_);
        for (LayerWeights& L : layers_) { fold(L.attn_norm); fold(L.ffn_norm); }
    }
    if (cfg_.layers[0].form == BlockForm::SUM_NORM) {
        const size_t m1 = row_scratch_width();
        dec_.y = dmalloc<float>(m1);
        for (float*& t : dec_.t) t = dmalloc<float>(m1);
        dec_.wide = dmalloc<float>(sumnorm_scratch_width());
    }
    if (cfg_.layers[0].form == BlockForm::POST_NORM) {
        const size_t m1 = row_scratch_width();
        dec_.y = dmalloc<float>(m1);
        for (float*& t : dec_.t) t = dmalloc<float>(m1);
        moe_sel_ = dmalloc<int>(topmax); moe_wt_ = dmalloc<float>(topmax); moe_act_ = dmalloc<float>(moe_act);
        size_t parts = 0;                          // per-slice partial results of the attention that serves all heads from one copy of the rows
        for (const LayerSpec& S : cfg_.layers)
            if (S.mixer == MixerKind::ATTN_LATENT) parts = std::max(parts, attention_shared_rows_scratch_floats(S.heads, S.latent.kv_rank));
        if (parts) { lat_part_ = dmalloc<float>(parts); owned_.push_back(lat_part_); }
    }
    hidden_ = dmalloc<float>(hidden);
    xnorm_ = dmalloc<float>(hidden);
    q_ = dmalloc<float>(qmax); k_ = dmalloc<float>(kmax); v_ = dmalloc<float>(vmax); attn_ = dmalloc<float>(omax);
    act_ = dmalloc<float>(ffmax);
    if (cfg_.layers[0].form == BlockForm::STREAMS) {
        const int S = n_streams();
        streams_ = dmalloc<float>((size_t)S * hidden);
        sub_y_ = dmalloc<float>(hidden);
        part_ = dmalloc<float>(hidden);
        maps_out_ = dmalloc<float>(mapmax);
        moe_sel_ = dmalloc<int>(topmax); moe_wt_ = dmalloc<float>(topmax); moe_sgate_ = dmalloc<float>(1); moe_act_ = dmalloc<float>(moe_act);
        ident_tab_ = dmalloc<float>(1);
        const float one = 1.f;
        NT_CUDA_CHECK(cudaMemcpy(ident_tab_, &one, sizeof(float), cudaMemcpyHostToDevice));
    }
    logits_ = dmalloc<float>(cfg_.vocab_size);
    NT_CUDA_CHECK(cudaMemset(logits_, 0, sizeof(float) * (size_t)cfg_.vocab_size));
    // the cache table: one entry per layer, then one per mixer that sits beside another inside a layer and keeps rows of its own
    slot_spec_.clear();
    for (LayerSpec& S : cfg_.layers) { S.cache_slot = (int)slot_spec_.size(); slot_spec_.push_back(&S); }
    for (LayerSpec& S : cfg_.layers)
        for (LayerSpec& b : S.branches)
            if (b.mixer != MixerKind::DELTA_RULE && b.mixer != MixerKind::SSM_SCAN) { b.cache_slot = (int)slot_spec_.size(); slot_spec_.push_back(&b); }
    const int n_slots = (int)slot_spec_.size();
    kcs_.assign((size_t)n_slots, nullptr);
    vcs_.assign((size_t)n_slots, nullptr);
    cache_owned_.assign((size_t)n_slots, 1);
    const size_t es = dtype_size(cache_dt_);
    for (int i = 0; i < n_slots; i++) {          // every layer RUN owns a cache, also one that borrows its tensors; not one that reads another's rows
        const LayerSpec& S = slot_spec(i);
        if (S.kv_from >= 0) { kcs_[(size_t)i] = kcs_[(size_t)S.kv_from]; vcs_[(size_t)i] = vcs_[(size_t)S.kv_from]; cache_owned_[(size_t)i] = 0; continue; }
        size_t kw = 0, vw = 0;
        cache_row_widths(i, kw, vw);
        if (kw + vw == 0) continue;                        // a mixer without cache rows (state-space scan)
        const size_t kb = es * max_seq * kw, vb = es * max_seq * vw;
        if (cudaMalloc(&kcs_[(size_t)i], std::max<size_t>(kb, 16)) != cudaSuccess || cudaMalloc(&vcs_[(size_t)i], std::max<size_t>(vb, 16)) != cudaSuccess) {
            cudaGetLastError();
            fprintf(stderr, "model: cannot allocate the KV cache for %d tokens\n", max_seq);
            return false;
        }
        NT_CUDA_CHECK(cudaMemset(kcs_[(size_t)i], 0, std::max<size_t>(kb, 16)));
        NT_CUDA_CHECK(cudaMemset(vcs_[(size_t)i], 0, std::max<size_t>(vb, 16)));
    }
    step_dev_ = dmalloc<int>(2);
    argmax_dev_ = dmalloc<int>(1);
    NT_CUDA_CHECK(cudaMallocHost(&argmax_host_, sizeof(int)));
    prefill_min_tokens_ = 16;
    finalized_ = true;
    return true;
}

static WindowAttn attn_of(const LayerSpec& S) {
    WindowAttn a;
    a.heads = S.heads; a.kv_heads = S.kv_heads; a.dim = S.dim; a.vdim = S.vdim; a.window = S.window; a.keep = S.keep_first; a.scale = S.scale; a.softcap = S.softcap;
    a.chunk = S.chunk; a.maps = S.maps;
    return a;
}

void Model::step_body_spec(cudaStream_t s) {
    const int hidden = cfg_.hidden_size;
    const int* pos_dev = step_dev_ + 1;
    const float m = cfg_.residual_mult;
    embed_rows(hidden_, embd_.ptr, embd_.dtype, step_dev_, 1, hidden, s);
    if (cfg_.layers[0].form == BlockForm::POST_NORM) {
        RowBufs B = dec_;
        B.x = hidden_;
        for (int i = 0; i < cfg_.n_layers; i++) layer_postnorm(i, 1, step_dev_, pos_dev, 0, B, s);
        return;
    }
    if (cfg_.layers[0].form == BlockForm::SUM_NORM) {
        RowBufs B = dec_;
        B.x = hidden_;
        for (int i = 0; i < cfg_.n_layers; i++) layer_sumnorm(i, 1, pos_dev, 0, B, s);
        return;
    }
    if (cfg_.layers[0].form == BlockForm::STREAMS) {
        // the residual lives in streams_ [S, width]; hidden_ holds the embedding row and, at the end, the sum of the streams for the head
        streams_spread(streams_, hidden_, cfg_.embed_scale, 1, n_streams(), hidden, s);
        for (int i = 0; i < cfg_.n_layers; i++) layer_streams_token(i, s);
        streams_read(hidden_, streams_, nullptr, 1, n_streams(), hidden, s);
        return;
    }
    for (int i = 0; i < cfg_.n_layers; i++) {
        const LayerSpec& S = cfg_.layers[(size_t)i];
        const LayerWeights& L = layer_weights(i);
        // Both branches read norm(x) of the x the layer started from.  The q/k/v and the gate/up launches each normalise hidden_ in
        // their prologue (bit-identical results), and both run before the first epilogue that updates hidden_.
        GemvMat qkv[3] = {mat_of(L.wq, q_), mat_of(L.wk, k_), mat_of(L.wv, v_)};
        gemv_dense(qkv, 3, hidden, hidden_, DENSE_STORE, nullptr, 1.f, s, L.attn_norm, cfg_.norm_eps);
        qk_norm_kv_write(q_, k_, v_, L.q_norm, L.k_norm, cfg_.norm_eps, kcs_[(size_t)i], vcs_[(size_t)i], cache_dt_, 1, pos_dev, 0, S.heads * S.dim,
                         S.kv_heads * S.dim, S.kv_heads * S.vdim, s);
        attention_window(attn_, q_, kcs_[(size_t)i], vcs_[(size_t)i], cache_dt_, 1, pos_dev, 0, cfg_.max_seq_len, attn_of(S), s);
        if (S.ff > 0) {
            GemvMat gu[2] = {mat_of(L.gate, act_), mat_of(L.up, nullptr)};
            gemv_dense(gu, 2, hidden, hidden_, S.act == GluAct::GELU_TANH ? DENSE_GEGLU : DENSE_SWIGLU, nullptr, 1.f, s, L.attn_norm, cfg_.norm_eps);
        }
        GemvMat o = mat_of(L.wo, hidden_);
        gemv_dense(&o, 1, S.heads * S.vdim, attn_, DENSE_SCALED_ADD, L.ls1, m, s);
        if (S.ff > 0) {
            GemvMat d = mat_of(L.down, hidden_);
            gemv_dense(&d, 1, S.ff, act_, DENSE_SCALED_ADD, L.ls2, m, s);
        }
    }
}

void Model::step_head_spec(cudaStream_t s) {
    GemvMat h = mat_of(head_, logits_);
    gemv_dense(&h, 1, cfg_.hidden_size, hidden_, DENSE_STORE, nullptr, 1.f, s, out_norm_, cfg_.norm_eps);       // final norm in the prologue
}

void Model::ensure_prefill_buffers_spec(int tokens) {
    if (tokens <= pf_.cap) return;
    NT_CUDA_CHECK(cudaStreamSynchronize(stream_));
    for (void* p : {(void*)pf_.x, (void*)pf_.q, (void*)pf_.k, (void*)pf_.v, (void*)pf_.attn, (void*)pf_.g, (void*)pf_.u, (void*)pf_.h, (void*)pf_.tmp,
                    pf_.ws, pf_.ws2, pf_.hws, (void*)pf_.tok, (void*)pf_.xs, (void*)pf_.maps, (void*)pf_.sel, (void*)pf_.work, (void*)pf_.wt, (void*)pf_.sgate,
                    (void*)pf_.act_rows, (void*)pf_.y_rows, (void*)pf_.g2, pf_.moe_ws, pf_.moe_ws2, (void*)pf_.gate_rows, (void*)pf_.wide})
        if (p) cudaFree(p);
    pf_.moe_ws2 = nullptr; pf_.wide = nullptr;
    pf_.xs = pf_.maps = pf_.wt = pf_.sgate = pf_.act_rows = pf_.y_rows = pf_.g2 = pf_.gate_rows = nullptr; pf_.sel = pf_.work = nullptr; pf_.moe_ws = nullptr;
    const size_t T = (size_t)((tokens + 127) / 128 * 128), hidden = (size_t)cfg_.hidden_size;
    size_t qmax = 1, kmax = 1, vmax = 1, omax = 1, ffmax = 1, mapmax = 1, topmax = 0, emax = 1, effmax = 1;
    const bool sum_form = cfg_.layers[0].form == BlockForm::SUM_NORM;
    const bool post_form = cfg_.layers[0].form == BlockForm::POST_NORM || sum_form;       // both keep five scratch rows of the widest intermediate
    if (sum_form) pf_.wide = dmalloc<float>(T * sumnorm_scratch_width());
    for (const LayerSpec& S : cfg_.layers) {
        if (post_form) {                  // five scratch rows of the widest intermediate; routed experts as below
            qmax = kmax = vmax = omax = ffmax = row_scratch_width();
            if (S.ff_kind == FfKind::MOE_GLU && S.ff > 0) { topmax = std::max(topmax, (size_t)S.top); emax = std::max(emax, (size_t)S.experts); effmax = std::max(effmax, (size_t)S.ff); }
            continue;
        }
        qmax = std::max(qmax, (size_t)S.heads * S.maps * S.dim); kmax = std::max(kmax, (size_t)S.kv_heads * S.maps * S.dim); vmax = std::max(vmax, (size_t)S.kv_heads * S.vdim);
        omax = std::max(omax, (size_t)S.heads * S.vdim); mapmax = std::max(mapmax, (size_t)S.heads * S.maps * S.vdim);
        if (S.ff_kind == FfKind::MOE_RELU2 && S.ff > 0) {
            topmax = std::max(topmax, (size_t)S.top); emax = std::max(emax, (size_t)S.experts); effmax = std::max(effmax, (size_t)S.ff);
            ffmax = std::max(ffmax, std::max((size_t)S.shared_ff, hidden));       // shared expert: activations [T, shared_ff], then its output [T, width]
        } else ffmax = std::max(ffmax, (size_t)S.ff);
    }
    if (cfg_.layers[0].form == BlockForm::STREAMS || post_form) {
        if (!post_form) { pf_.xs = dmalloc<float>(T * n_streams() * hidden); pf_.maps = dmalloc<float>(T * mapmax); }
        if (topmax > 0) {
            pf_.sel = dmalloc<int>(T * topmax); pf_.wt = dmalloc<float>(T * topmax); pf_.sgate = dmalloc<float>(T);
            pf_.work = dmalloc<int>(moe_work_ints((int)T, (int)emax, (int)topmax));
            pf_.act_rows = dmalloc<float>(T * topmax * effmax); pf_.y_rows = dmalloc<float>(T * topmax * hidden);
            if (!exact32_) {       // the tensor-core path of the routed experts: gathered rows, and a split workspace with every expert's rows padded to a tile
                pf_.g2 = dmalloc<float>(T * topmax * hidden);
                pf_.moe_ws = dmalloc<uint8_t>(gemm_f16_tc_workspace_bytes((int)(T * topmax + emax * 128), (int)std::max(hidden, effmax)));
                if (!moe_offsets_host_) NT_CUDA_CHECK(cudaMallocHost(&moe_offsets_host_, sizeof(int) * 257));
            }
        }
    }
    pf_.x = dmalloc<float>(T * hidden); pf_.h = dmalloc<float>(T * hidden); pf_.tmp = dmalloc<float>(T * hidden);
    pf_.q = dmalloc<float>(T * qmax); pf_.k = dmalloc<float>(T * kmax); pf_.v = dmalloc<float>(T * vmax); pf_.attn = dmalloc<float>(T * omax);
    pf_.g = dmalloc<float>(T * ffmax); pf_.u = dmalloc<float>(T * ffmax);
    pf_.tok = dmalloc<int>(T);
    pf_.ws = pf_.ws2 = pf_.hws = nullptr;
    if (post_form && topmax > 0) pf_.gate_rows = dmalloc<float>(T * topmax * effmax);      // the gate half of the gated experts' rows
    if (post_form && topmax > 0 && !exact32_) pf_.moe_ws2 = dmalloc<uint8_t>(gemm_f16_tc_workspace_bytes((int)(T * topmax + emax * 128), (int)effmax));
    bool any_tc = false;
    for (int i = 0; i < cfg_.n_layers; i++) {
        const LayerWeights& L = layer_weights(i);
        for (const Weight* w : {&L.wq, &L.wk, &L.wv, &L.wo, &L.gate, &L.up, &L.down, &L.sh_up, &L.sh_down, &L.w_dq, &L.w_uq, &L.w_dkv, &L.ssm_in, &L.side_gate, &L.side_proj})
            any_tc = any_tc || (w->ptr && spec_tc_ok(*w));
        for (const LayerWeights& b : L.branch)
            for (const Weight* w : {&b.wq, &b.wk, &b.wv, &b.wo, &b.d_beta, &b.d_a1, &b.d_a2, &b.d_g1, &b.d_g2}) {
                any_tc = any_tc || (w->ptr && spec_tc_ok(*w));
                ffmax = std::max(ffmax, (size_t)w->cols);          // the split workspace holds the widest GEMM input
            }
        ffmax = std::max(ffmax, (size_t)L.wo.cols);
    }
    if (sum_form && any_tc) {             // the gated feed-forward's fused gate / up GEMM writes the down GEMM's split input here
        size_t ffw = 1;
        for (const LayerSpec& S : cfg_.layers) ffw = std::max(ffw, (size_t)S.ff);
        pf_.ws2 = dmalloc<uint8_t>(gemm_f16_tc_workspace_bytes((int)T, (int)ffw));
    }
    if (post_form && any_tc) {            // one split workspace: rows_matmul splits its input right before the GEMM
        pf_.ws = dmalloc<uint8_t>(gemm_f16_tc_workspace_bytes((int)T, (int)std::max(hidden, ffmax)));
        any_tc = false;
    }
    if (any_tc) {                         // BF16 hi/lo splits of the three GEMM inputs (normed block input, attention output, gated activation)
        pf_.hws = dmalloc<uint8_t>(gemm_f16_tc_workspace_bytes((int)T, (int)hidden));
        pf_.ws = dmalloc<uint8_t>(gemm_f16_tc_workspace_bytes((int)T, (int)omax));
        pf_.ws2 = dmalloc<uint8_t>(gemm_f16_tc_workspace_bytes((int)T, (int)ffmax));
    }
    pf_.cap = (int)T;
}

// BF16 rows that the tcgen05 GEMM can read in place through TMA (rows >= 128 and % 4, cols % 64, 16-byte aligned); never in exact mode.
bool Model::spec_tc_ok(const Weight& w) const {
    static const bool off = getenv("NT_B200_NO_TC_PREFILL") != nullptr;
    return !exact32_ && !off && w.dtype == DType::BF16 && gemm_f16_tc_ragged_supported(w.ptr, w.rows, w.cols, w.pitch);
}

// C (ep)= A . W^T for T prompt rows: on the tensor cores from the BF16 hi/lo split of A when the matrix qualifies, else in FP32
// on CUDA cores from A itself.  Either input may be null when the caller knows which path the matrix takes.
void Model::spec_gemm(float* C, const float* A, const void* A_split, const Weight& w, int T, DenseEpilogue ep, const float* row_scale, float alpha, cudaStream_t s) {
    if (A_split && spec_tc_ok(w)) {
        TcOpts o;
        o.bf16 = true;
        if (ep == DENSE_SCALED_ADD) { o.col_scale = row_scale; o.alpha = alpha; }
        NT_CHECK(gemm_f16_tc_ws(C, A_split, w.ptr, T, w.rows, w.cols, ep != DENSE_STORE, s, o), "prefill GEMM rejected");
        return;
    }
    NT_CHECK(A != nullptr, "spec_gemm: the FP32 input of a CUDA-core GEMM is missing");
    gemm_dense(C, A, w.ptr, w.dtype, w.pitch, T, w.rows, w.cols, ep, row_scale, alpha, s);
}

// A prompt (or a portion of one: start_pos > 0) in chunks of up to SPEC_PREFILL_CHUNK tokens.  The chunk's key / value rows go to
// the cache first, then the attention kernel reads cache rows only — earlier portions, the kept first tokens and the chunk itself
// alike — so where a prompt is cut cannot change what a query sees.
void Model::prefill_spec(const int* tokens, int seq_len, int start_pos) {
    cudaStream_t s = stream_;
    const int hidden = cfg_.hidden_size;
    const float m = cfg_.residual_mult;
    ensure_prefill_buffers_spec(std::min(seq_len, SPEC_PREFILL_CHUNK));
    int last_rows = 0;
    for (int c0 = 0; c0 < seq_len; c0 += SPEC_PREFILL_CHUNK) {
        const int T = std::min(SPEC_PREFILL_CHUNK, seq_len - c0), p0 = start_pos + c0;
        last_rows = T;
        NT_CUDA_CHECK(cudaMemcpyAsync(pf_.tok, tokens + c0, sizeof(int) * (size_t)T, cudaMemcpyHostToDevice, s));
        embed_rows(pf_.x, embd_.ptr, embd_.dtype, pf_.tok, T, hidden, s);
        const bool streams_form = cfg_.layers[0].form == BlockForm::STREAMS, post_form = cfg_.layers[0].form == BlockForm::POST_NORM;
        const bool sum_form = cfg_.layers[0].form == BlockForm::SUM_NORM;
        if (streams_form) streams_spread(pf_.xs, pf_.x, cfg_.embed_scale, T, n_streams(), hidden, s);
        RowBufs rb;
        rb.x = pf_.x; rb.y = pf_.tmp; rb.t[0] = pf_.q; rb.t[1] = pf_.k; rb.t[2] = pf_.v; rb.t[3] = pf_.attn; rb.t[4] = pf_.g; rb.wide = pf_.wide;
        for (int i = 0; i < cfg_.n_layers; i++) {
            if (streams_form) { layer_streams_rows(i, T, p0, s); continue; }
            if (sum_form) { layer_sumnorm(i, T, nullptr, p0, rb, s); continue; }
            if (post_form) { layer_postnorm(i, T, pf_.tok, nullptr, p0, rb, s); continue; }
            const LayerSpec& S = cfg_.layers[(size_t)i];
            const LayerWeights& L = layer_weights(i);
            // the block's normed input feeds q, k, v, gate and up: as FP32 rows, as a BF16 split, or both, by what those matrices take
            bool h_f32 = false, h_split = false;
            auto reads_h = [&](const Weight& w) { if (spec_tc_ok(w)) h_split = true; else h_f32 = true; };
            reads_h(L.wq); reads_h(L.wk); reads_h(L.wv);
            if (S.ff > 0) { reads_h(L.gate); reads_h(L.up); }
            if (h_f32) rmsnorm(pf_.h, pf_.x, L.attn_norm, T, hidden, cfg_.norm_eps, s);
            if (h_split) rmsnorm_split(pf_.hws, pf_.x, L.attn_norm, T, hidden, cfg_.norm_eps, s, true);
            const float* hf = h_f32 ? pf_.h : nullptr;
            const void* hs = h_split ? pf_.hws : nullptr;
            spec_gemm(pf_.q, hf, hs, L.wq, T, DENSE_STORE, nullptr, 1.f, s);
            spec_gemm(pf_.k, hf, hs, L.wk, T, DENSE_STORE, nullptr, 1.f, s);
            spec_gemm(pf_.v, hf, hs, L.wv, T, DENSE_STORE, nullptr, 1.f, s);
            qk_norm_kv_write(pf_.q, pf_.k, pf_.v, L.q_norm, L.k_norm, cfg_.norm_eps, kcs_[(size_t)i], vcs_[(size_t)i], cache_dt_, T, nullptr, p0,
                             S.heads * S.dim, S.kv_heads * S.dim, S.kv_heads * S.vdim, s);
            attention_window(pf_.attn, pf_.q, kcs_[(size_t)i], vcs_[(size_t)i], cache_dt_, T, nullptr, p0, cfg_.max_seq_len, attn_of(S), s);
            const bool o_tc = spec_tc_ok(L.wo);
            if (o_tc) split_activations(pf_.ws, pf_.attn, T, S.heads * S.vdim, s, true);
            spec_gemm(pf_.x, pf_.attn, o_tc ? pf_.ws : nullptr, L.wo, T, DENSE_SCALED_ADD, L.ls1, m, s);
            if (S.ff > 0) {
                const bool gelu = S.act == GluAct::GELU_TANH, down_tc = spec_tc_ok(L.down);
                if (spec_tc_ok(L.gate) && spec_tc_ok(L.up) && down_tc && S.ff % 128 == 0) {
                    // gate / up GEMMs with the gated activation and the split for the down projection in the epilogue: the
                    // [T, ff] activations never reach HBM in FP32
                    TcOpts o; o.bf16 = true; o.gelu = gelu;
                    NT_CHECK(gemm_f16_tc_swiglu_ws(pf_.ws2, pf_.hws, L.gate.ptr, L.up.ptr, T, S.ff, hidden, s, o), "prefill GEMM (gate/up) rejected");
                } else {
                    spec_gemm(pf_.g, hf, hs, L.gate, T, DENSE_STORE, nullptr, 1.f, s);
                    spec_gemm(pf_.u, hf, hs, L.up, T, DENSE_STORE, nullptr, 1.f, s);
                    glu_mul(pf_.g, pf_.g, pf_.u, (size_t)T * S.ff, gelu, s);
                    if (down_tc) split_activations(pf_.ws2, pf_.g, T, S.ff, s, true);
                }
                spec_gemm(pf_.x, pf_.g, down_tc ? pf_.ws2 : nullptr, L.down, T, DENSE_SCALED_ADD, L.ls2, m, s);
            }
        }
        if (streams_form) streams_read(pf_.x, pf_.xs, nullptr, T, n_streams(), hidden, s);      // the sum of the streams feeds the head
        if (!want_.empty()) emit_wanted(pf_.x, c0, T, s);
    }
    copy(hidden_, pf_.x + (size_t)(last_rows - 1) * hidden, hidden, s);
    step_head(s);
}

// ---- BlockForm::STREAMS layers (differential attention, rotary positions, block-local mask, shared caches, mixture of experts) ----

MoeWeights Model::moe_of(int i, bool with_shared) const {
    const LayerSpec& S = cfg_.layers[(size_t)i];
    const LayerWeights& L = layer_weights(i);
    MoeWeights w;
    w.router = L.router; w.shared_gate = S.shared_ff > 0 ? L.shared_gate : nullptr;
    w.up = L.e_up_tab; w.down = L.e_down_tab; w.dtype = L.e_up[0].dtype;
    w.experts = S.experts; w.top = S.top; w.ff = S.ff; w.width = cfg_.hidden_size;
    if (with_shared && S.shared_ff > 0) { w.shared_up = L.sh_up.ptr; w.shared_down = L.sh_down.ptr; w.shared_ff = S.shared_ff; }
    return w;
}

// One decoded token, 8 launches: [stream blend + norm + q/k/v GEMV] [rotary + cache write] [attention, both maps] [differential combine]
// [o GEMV -> streams]   [stream blend + norm + router] [experts up + relu^2] [experts down, weighted, + shared -> streams]
// The stream read lives in the prologue of the kernel that consumes it, the stream write in the epilogue of the one that produces y.
void Model::layer_streams_token(int i, cudaStream_t s) {
    const LayerSpec& S = cfg_.layers[(size_t)i];
    const LayerWeights& L = layer_weights(i);
    const int hidden = cfg_.hidden_size, NS = n_streams();
    const int* pos_dev = step_dev_ + 1;
    const bool one = cfg_.streams == 0;            // a single residual: identity tables
    const int qd = S.heads * S.maps * S.dim, kd = S.kv_heads * S.maps * S.dim, vd = S.kv_heads * S.vdim;
    StreamsIO rd; rd.X_in = streams_; rd.a = one ? nullptr : L.hc_in[0]; rd.S = NS;
    if (S.kv_from < 0) {
        GemvMat qkv[3] = {mat_of(L.wq, q_), mat_of(L.wk, k_), mat_of(L.wv, v_)};
        gemv_dense(qkv, 3, hidden, nullptr, DENSE_STORE, nullptr, 1.f, s, L.attn_norm, cfg_.norm_eps, &rd);
    } else {
        GemvMat q1 = mat_of(L.wq, q_);
        gemv_dense(&q1, 1, hidden, nullptr, DENSE_STORE, nullptr, 1.f, s, L.attn_norm, cfg_.norm_eps, &rd);
    }
    rope_partial_kv_write(q_, S.kv_from < 0 ? k_ : nullptr, v_, L.rot_freq, L.rot_mag, S.rot.dims, S.rot.interleaved, S.dim, kcs_[(size_t)i], vcs_[(size_t)i],
                          cache_dt_, 1, pos_dev, 0, qd, kd, vd, s);
    attention_window(S.maps > 1 ? maps_out_ : attn_, q_, kcs_[(size_t)i], vcs_[(size_t)i], cache_dt_, 1, pos_dev, 0, cfg_.max_seq_len, attn_of(S), s);
    if (S.maps > 1) diff_combine(attn_, maps_out_, L.lq1, L.lk1, L.lq2, L.lk2, S.dim, S.diff, cfg_.norm_eps, 1, S.heads, S.vdim, s);
    StreamsIO wr; wr.X_out = streams_; wr.M = one ? ident_tab_ : L.hc_mix[0]; wr.b = one ? ident_tab_ : L.hc_out[0]; wr.S = NS;
    GemvMat o = mat_of(L.wo, nullptr);
    gemv_dense(&o, 1, S.heads * S.vdim, attn_, DENSE_STREAMS, nullptr, 1.f, s, nullptr, 0.f, &wr);
    if (S.ff <= 0) return;
    rd.a = one ? nullptr : L.hc_in[1];
    wr.M = one ? ident_tab_ : L.hc_mix[1]; wr.b = one ? ident_tab_ : L.hc_out[1];
    const MoeWeights w = moe_of(i, true);
    moe_route(moe_sel_, moe_wt_, moe_sgate_, nullptr, w, 1, s, &rd, L.ffn_norm, cfg_.norm_eps, part_);
    moe_expert_up_token(moe_act_, part_, moe_sel_, w, s);
    moe_expert_down_token(nullptr, moe_act_, moe_sel_, moe_wt_, moe_sgate_, nullptr, w, s, &wr);
}

// T prompt rows at positions p0..: the same steps over rows; projections and the shared expert through spec_gemm (tensor cores
// when the matrix qualifies), routed experts as gathered GEMMs over each expert's own rows.
void Model::layer_streams_rows(int i, int T, int p0, cudaStream_t s) {
    const LayerSpec& S = cfg_.layers[(size_t)i];
    const LayerWeights& L = layer_weights(i);
    const int hidden = cfg_.hidden_size, NS = n_streams();
    const bool one = cfg_.streams == 0;
    const int qd = S.heads * S.maps * S.dim, kd = S.kv_heads * S.maps * S.dim, vd = S.kv_heads * S.vdim;
    streams_read(pf_.tmp, pf_.xs, one ? nullptr : L.hc_in[0], T, NS, hidden, s);
    bool h_f32 = false, h_split = false;
    auto reads_h = [&](const Weight& w) { if (spec_tc_ok(w)) h_split = true; else h_f32 = true; };
    reads_h(L.wq);
    if (S.kv_from < 0) { reads_h(L.wk); reads_h(L.wv); }
    if (h_f32) rmsnorm(pf_.h, pf_.tmp, L.attn_norm, T, hidden, cfg_.norm_eps, s);
    if (h_split) rmsnorm_split(pf_.hws, pf_.tmp, L.attn_norm, T, hidden, cfg_.norm_eps, s, true);
    const float* hf = h_f32 ? pf_.h : nullptr;
    const void* hs = h_split ? pf_.hws : nullptr;
    spec_gemm(pf_.q, hf, hs, L.wq, T, DENSE_STORE, nullptr, 1.f, s);
    if (S.kv_from < 0) {
        spec_gemm(pf_.k, hf, hs, L.wk, T, DENSE_STORE, nullptr, 1.f, s);
        spec_gemm(pf_.v, hf, hs, L.wv, T, DENSE_STORE, nullptr, 1.f, s);
    }
    rope_partial_kv_write(pf_.q, S.kv_from < 0 ? pf_.k : nullptr, pf_.v, L.rot_freq, L.rot_mag, S.rot.dims, S.rot.interleaved, S.dim, kcs_[(size_t)i],
                          vcs_[(size_t)i], cache_dt_, T, nullptr, p0, qd, kd, vd, s);
    attention_window(S.maps > 1 ? pf_.maps : pf_.attn, pf_.q, kcs_[(size_t)i], vcs_[(size_t)i], cache_dt_, T, nullptr, p0, cfg_.max_seq_len, attn_of(S), s);
    if (S.maps > 1) diff_combine(pf_.attn, pf_.maps, L.lq1, L.lk1, L.lq2, L.lk2, S.dim, S.diff, cfg_.norm_eps, T, S.heads, S.vdim, s);
    const bool o_tc = spec_tc_ok(L.wo);
    if (o_tc) split_activations(pf_.ws, pf_.attn, T, S.heads * S.vdim, s, true);
    spec_gemm(pf_.tmp, pf_.attn, o_tc ? pf_.ws : nullptr, L.wo, T, DENSE_STORE, nullptr, 1.f, s);
    streams_write(pf_.xs, pf_.tmp, one ? ident_tab_ : L.hc_mix[0], one ? ident_tab_ : L.hc_out[0], T, NS, hidden, s);
    if (S.ff <= 0) return;
    streams_read(pf_.tmp, pf_.xs, one ? nullptr : L.hc_in[1], T, NS, hidden, s);
    rmsnorm(pf_.h, pf_.tmp, L.ffn_norm, T, hidden, cfg_.norm_eps, s);          // the router and the gathered expert GEMMs read F32 rows
    const MoeWeights w = moe_of(i, false);
    moe_route(pf_.sel, pf_.wt, pf_.sgate, pf_.h, w, T, s);
    moe_group(pf_.work, pf_.sel, T, S.experts, S.top, s);
    bool experts_tc = pf_.moe_ws != nullptr;
    for (int e = 0; experts_tc && e < S.experts; e++) experts_tc = spec_tc_ok(L.e_up[(size_t)e]) && spec_tc_ok(L.e_down[(size_t)e]);
    if (experts_tc) {
        // Tensor cores: the per-expert row counts come to the host (one small copy and a wait per layer), then every expert with rows
        // runs the tcgen05 GEMM over exactly its rows: gather the rows in expert order, split per expert into its own padded
        // region of the workspace, up GEMM, relu^2 over all rows at once, split again, down GEMM.
        NT_CUDA_CHECK(cudaMemcpyAsync(moe_offsets_host_, pf_.work, sizeof(int) * (size_t)(S.experts + 1), cudaMemcpyDeviceToHost, s));
        NT_CUDA_CHECK(cudaStreamSynchronize(s));
        moe_gather_rows(pf_.g2, pf_.h, pf_.work, T, S.experts, S.top, hidden, s);
        auto region = [&](size_t rows_before, int K) { return static_cast<uint8_t*>(pf_.moe_ws) + gemm_f16_tc_workspace_bytes((int)rows_before, K); };
        TcOpts o; o.bf16 = true;
        size_t padded = 0;
        for (int e = 0; e < S.experts; e++) {
            const int r0 = moe_offsets_host_[e], cnt = moe_offsets_host_[e + 1] - r0;
            if (cnt <= 0) continue;
            void* ws = region(padded, hidden);
            split_activations(ws, pf_.g2 + (size_t)r0 * hidden, cnt, hidden, s, true);
            NT_CHECK(gemm_f16_tc_ws(pf_.act_rows + (size_t)r0 * S.ff, ws, L.e_up[(size_t)e].ptr, cnt, S.ff, hidden, false, s, o), "expert GEMM (up) rejected");
            padded += ((size_t)cnt + 127) / 128 * 128;
        }
        relu2(pf_.act_rows, (size_t)T * S.top * S.ff, s);
        padded = 0;
        for (int e = 0; e < S.experts; e++) {
            const int r0 = moe_offsets_host_[e], cnt = moe_offsets_host_[e + 1] - r0;
            if (cnt <= 0) continue;
            void* ws = region(padded, S.ff);
            split_activations(ws, pf_.act_rows + (size_t)r0 * S.ff, cnt, S.ff, s, true);
            NT_CHECK(gemm_f16_tc_ws(pf_.y_rows + (size_t)r0 * hidden, ws, L.e_down[(size_t)e].ptr, cnt, hidden, S.ff, false, s, o), "expert GEMM (down) rejected");
            padded += ((size_t)cnt + 127) / 128 * 128;
        }
    } else {
        moe_expert_up_rows(pf_.act_rows, pf_.h, pf_.work, w, T, s);
        moe_expert_down_rows(pf_.y_rows, pf_.act_rows, pf_.work, w, T, s);
    }
    const float* shared_y = nullptr;
    if (S.shared_ff > 0) {
        const bool up_tc = spec_tc_ok(L.sh_up), down_tc = spec_tc_ok(L.sh_down);
        if (up_tc) rmsnorm_split(pf_.hws, pf_.tmp, L.ffn_norm, T, hidden, cfg_.norm_eps, s, true);
        spec_gemm(pf_.g, pf_.h, up_tc ? pf_.hws : nullptr, L.sh_up, T, DENSE_STORE, nullptr, 1.f, s);
        relu2(pf_.g, (size_t)T * S.shared_ff, s);
        if (down_tc) split_activations(pf_.ws2, pf_.g, T, S.shared_ff, s, true);
        spec_gemm(pf_.u, pf_.g, down_tc ? pf_.ws2 : nullptr, L.sh_down, T, DENSE_STORE, nullptr, 1.f, s);
        shared_y = pf_.u;
    }
    moe_combine(pf_.tmp, pf_.y_rows, pf_.work, pf_.wt, pf_.sgate, shared_y, T, S.experts, S.top, hidden, s);
    streams_write(pf_.xs, pf_.tmp, one ? ident_tab_ : L.hc_mix[1], one ? ident_tab_ : L.hc_out[1], T, NS, hidden, s);
}

// ---- BlockForm::POST_NORM layers (latent attention, state-space scan, biased / routed gated feed-forward, per-layer token input) ----

void Model::cache_row_widths(int i, size_t& k, size_t& v) const {
    const LayerSpec& S = slot_spec(i);
    if (S.mixer == MixerKind::SSM_SCAN || S.mixer == MixerKind::DELTA_RULE || S.mixer == MixerKind::BRANCHES) { k = v = 0; return; }      // a state, no rows (branches own theirs)
    if (S.mixer == MixerKind::ATTN_LATENT) { k = (size_t)S.latent.kv_rank + S.latent.rot_dim; v = 0; return; }   // [latent | rotated key part]
    k = (size_t)S.kv_heads * S.maps * S.dim;
    v = (size_t)S.kv_heads * S.vdim;
}

size_t Model::row_scratch_width() const {
    size_t m = (size_t)cfg_.hidden_size;
    for (const LayerSpec& S : cfg_.layers) {
        if (S.form == BlockForm::SUM_NORM) { m = std::max(m, (size_t)S.ff); continue; }      // the mixers' intermediates live in RowBufs::wide
        if (S.mixer == MixerKind::ATTN_LATENT) {
            const LatentSpec& A = S.latent;
            m = std::max({m, (size_t)A.q_rank, (size_t)A.kv_rank + A.rot_dim, (size_t)S.heads * (S.dim + A.rot_dim), (size_t)S.heads * (A.kv_rank + A.rot_dim),
                          (size_t)S.heads * S.vdim});
        } else if (S.mixer == MixerKind::SSM_SCAN) {
            const size_t inner = (size_t)S.heads * S.vdim, ch = inner + 2 * (size_t)S.scan.groups * S.scan.state;
            m = std::max(m, inner + ch + S.heads);
        }
        if (S.ff_kind == FfKind::GLU) m = std::max(m, (size_t)S.ff);
        m = std::max(m, (size_t)cfg_.side_dim);
    }
    return m;
}

// Short BF16 matrices (rows below a tensor-core tile, cols a multiple of 64) get a copy with zero rows up to 128: the CUDA-core GEMM has
// one CTA per 64 x 64 outputs and leaves most SMs idle on them.  The copy must not alias the prompt pass's result row buffer: the padded
// product lands in pf_.tmp, which no caller of rows_matmul passes as A together with such a matrix.
void Model::pad_for_tensor_cores(Weight& w) {
    static const bool off = getenv("NT_B200_NO_TC_PREFILL") != nullptr;
    constexpr int kRows = 128;
    if (off || exact32_ || !w.ptr || w.dtype != DType::BF16 || w.rows >= kRows || w.cols % 64 != 0 || cfg_.hidden_size < kRows) return;
    uint8_t* p = dmalloc<uint8_t>((size_t)kRows * w.cols * 2);
    NT_CUDA_CHECK(cudaMemset(p, 0, (size_t)kRows * w.cols * 2));
    NT_CUDA_CHECK(cudaMemcpy2D(p, (size_t)w.cols * 2, w.ptr, w.pitch, (size_t)w.cols * 2, (size_t)w.rows, cudaMemcpyDeviceToDevice));
    if (!gemm_f16_tc_ragged_supported(p, kRows, w.cols, (size_t)w.cols * 2)) { cudaFree(p); return; }
    owned_.push_back(p);
    w.tc_ptr = p; w.tc_rows = kRows;
}

// C [T, w.rows] = A [T, w.cols] . W^T.  One row: the GEMV.  More: the tensor-core GEMM from a BF16 split of A made here when the matrix
// qualifies (never in exact mode), else the FP32 GEMM on CUDA cores.
void Model::rows_matmul(float* C, const float* A, const Weight& w, int T, cudaStream_t s, bool* split_done) {
    if (T == 1) {
        GemvMat m = mat_of(w, C);
        gemv_dense(&m, 1, w.cols, A, DENSE_STORE, nullptr, 1.f, s);
        return;
    }
    // split_done: several matrices read the same A one after the other; the first tensor-core one splits it, the others find it done
    auto split_once = [&]() {
        if (split_done && *split_done) return;
        split_activations(pf_.ws, A, T, w.cols, s, true);
        if (split_done) *split_done = true;
    };
    if (w.tc_ptr && pf_.ws && !exact32_) {            // a short matrix: the padded copy on the tensor cores, then the live columns
        split_once();
        TcOpts o; o.bf16 = true;
        NT_CHECK(gemm_f16_tc_ws(pf_.tmp, pf_.ws, w.tc_ptr, T, w.tc_rows, w.cols, false, s, o), "prefill GEMM (padded) rejected");
        copy_cols(C, pf_.tmp, T, w.rows, w.tc_rows, s);
        return;
    }
    const bool tc = pf_.ws && spec_tc_ok(w);
    if (tc) split_once();
    spec_gemm(C, A, tc ? pf_.ws : nullptr, w, T, DENSE_STORE, nullptr, 1.f, s);
}

// ---- latent attention over a prompt portion: expanded per-head keys / values and the tiled tensor-core attention kernel ----

constexpr int LATENT_ROW_BLOCK = 2048;      // cache rows expanded per pair of up-projection GEMMs

// 16 queries or more, BF16 cache rows, head widths the tiled kernel takes; never in exact mode (the absorbed form is all F32 there).
bool Model::latent_expand_ok(const LayerSpec& S, int T) const {
    static const bool off = getenv("NT_B200_NO_LATENT_EXPAND") != nullptr;
    int kw = 0, vw = 0;
    return !off && !exact32_ && cache_dt_ == DType::BF16 && T >= 16 && attention_heads_mma_widths(S.dim + S.latent.rot_dim, S.vdim, &kw, &vw);
}

void Model::ensure_latent_scratch(const LayerSpec& S, size_t rows, size_t tokens) {
    int kw = 0, vw = 0;
    NT_CHECK(attention_heads_mma_widths(S.dim + S.latent.rot_dim, S.vdim, &kw, &vw), "latent attention: head widths outside the tiled kernel's");
    const size_t H = (size_t)S.heads, need_k = H * kw, need_v = H * vw, need_stage = H * (size_t)std::max(S.dim, S.vdim), need_rank = (size_t)S.latent.kv_rank;
    if (rows <= lat_.rows && tokens <= lat_.tokens && need_k <= lat_.kw && need_v <= lat_.vw && need_stage <= lat_.stage_w && need_rank <= lat_.rank) return;
    NT_CUDA_CHECK(cudaStreamSynchronize(stream_));
    for (void* p : {lat_.k, lat_.v, lat_.ws, (void*)lat_.q, (void*)lat_.o, (void*)lat_.c32, (void*)lat_.ku, (void*)lat_.vu}) if (p) cudaFree(p);
    if (rows > lat_.rows) lat_.rows = std::min((size_t)cfg_.max_seq_len, std::max(2 * lat_.rows, (rows + 1023) / 1024 * 1024));     // grows geometrically up to the cache's length
    lat_.rows = std::max(lat_.rows, rows);
    lat_.tokens = std::max(lat_.tokens, (tokens + 127) / 128 * 128);
    lat_.kw = std::max(lat_.kw, need_k); lat_.vw = std::max(lat_.vw, need_v); lat_.stage_w = std::max(lat_.stage_w, need_stage); lat_.rank = std::max(lat_.rank, need_rank);
    lat_.k = dmalloc<uint16_t>(lat_.rows * lat_.kw); lat_.v = dmalloc<uint16_t>(lat_.rows * lat_.vw);
    lat_.q = dmalloc<float>(lat_.tokens * lat_.kw); lat_.o = dmalloc<float>(lat_.tokens * lat_.vw);
    lat_.c32 = dmalloc<float>((size_t)LATENT_ROW_BLOCK * lat_.rank);
    lat_.ws = dmalloc<uint8_t>(gemm_f16_tc_workspace_bytes(LATENT_ROW_BLOCK, (int)lat_.rank));
    lat_.ku = dmalloc<float>((size_t)LATENT_ROW_BLOCK * lat_.stage_w); lat_.vu = dmalloc<float>((size_t)LATENT_ROW_BLOCK * lat_.stage_w);
}

// q [T, heads, dim + rot_dim] (unrotated) at positions p0..; the layer's cache rows 0 .. p0 + T - 1 are written.  out [T, heads * vdim].
void Model::latent_attention_rows(int i, int T, int p0, const float* q, float* out, cudaStream_t s) {
    const LayerSpec& S = cfg_.layers[(size_t)i];
    const LayerWeights& L = layer_weights(i);
    const LatentSpec& A = S.latent;
    int kw = 0, vw = 0;
    attention_heads_mma_widths(S.dim + A.rot_dim, S.vdim, &kw, &vw);
    const int P = p0 + T, row = A.kv_rank + A.rot_dim;
    ensure_latent_scratch(S, (size_t)P, (size_t)T);
    const bool tk = spec_tc_ok(L.w_uk), tv = spec_tc_ok(L.w_uv);
    for (int r0 = 0; r0 < P; r0 += LATENT_ROW_BLOCK) {
        const int n = std::min(LATENT_ROW_BLOCK, P - r0);
        latent_rows_f32(lat_.c32, kcs_[(size_t)i], cache_dt_, row, A.kv_rank, r0, n, s);
        if (tk || tv) split_activations(lat_.ws, lat_.c32, n, A.kv_rank, s, true);
        spec_gemm(lat_.ku, lat_.c32, tk ? lat_.ws : nullptr, L.w_uk, n, DENSE_STORE, nullptr, 1.f, s);
        spec_gemm(lat_.vu, lat_.c32, tv ? lat_.ws : nullptr, L.w_uv, n, DENSE_STORE, nullptr, 1.f, s);
        latent_expand_pack(lat_.k, lat_.v, lat_.ku, lat_.vu, kcs_[(size_t)i], cache_dt_, A.kv_rank, r0, n, S.heads, S.dim, A.rot_dim, S.vdim, kw, vw, s);
    }
    latent_q_rot_pad(lat_.q, q, T, S.heads, S.dim, A.rot_dim, kw, S.rot.dims, S.rot.interleaved, S.rot.base, p0, s);
    float* o = vw == S.vdim ? out : lat_.o;
    attention_heads_mma(o, lat_.q, lat_.k, lat_.v, T, p0, P, S.heads, kw, vw, S.scale, s);
    if (o != out) latent_unpad(out, lat_.o, T, S.heads, S.vdim, vw, s);
}

// The routed gated experts of T prompt rows on the tensor cores: the per-expert row counts come to the host (one small copy and a wait),
// then every expert with rows runs, over exactly its rows, the gate / up GEMM pair whose epilogue applies silu(gate) * up and writes the
// down GEMM's split input, and the down GEMM.  pf_.y_rows [T * top, width] in the grouped order.  false: some matrix does not qualify.
bool Model::moe_glu_rows_tc(int i, int T, const float* x, cudaStream_t s) {
    const LayerSpec& S = cfg_.layers[(size_t)i];
    const LayerWeights& L = layer_weights(i);
    const int hidden = cfg_.hidden_size;
    if (!pf_.moe_ws || !pf_.moe_ws2 || !pf_.g2 || !moe_offsets_host_ || S.ff % 128 != 0 || S.experts > 256) return false;
    for (int e = 0; e < S.experts; e++)
        if (!spec_tc_ok(L.e_gate[(size_t)e]) || !spec_tc_ok(L.e_up[(size_t)e]) || !spec_tc_ok(L.e_down[(size_t)e])) return false;
    NT_CUDA_CHECK(cudaMemcpyAsync(moe_offsets_host_, pf_.work, sizeof(int) * (size_t)(S.experts + 1), cudaMemcpyDeviceToHost, s));
    NT_CUDA_CHECK(cudaStreamSynchronize(s));
    moe_gather_rows(pf_.g2, x, pf_.work, T, S.experts, S.top, hidden, s);
    TcOpts o; o.bf16 = true;
    size_t padded = 0;
    for (int e = 0; e < S.experts; e++) {
        const int r0 = moe_offsets_host_[e], cnt = moe_offsets_host_[e + 1] - r0;
        if (cnt <= 0) continue;
        void* wi = static_cast<uint8_t*>(pf_.moe_ws) + gemm_f16_tc_workspace_bytes((int)padded, hidden);
        void* wo = static_cast<uint8_t*>(pf_.moe_ws2) + gemm_f16_tc_workspace_bytes((int)padded, S.ff);
        split_activations(wi, pf_.g2 + (size_t)r0 * hidden, cnt, hidden, s, true);
        NT_CHECK(gemm_f16_tc_swiglu_ws(wo, wi, L.e_gate[(size_t)e].ptr, L.e_up[(size_t)e].ptr, cnt, S.ff, hidden, s, o), "expert GEMM (gate / up) rejected");
        NT_CHECK(gemm_f16_tc_ws(pf_.y_rows + (size_t)r0 * hidden, wo, L.e_down[(size_t)e].ptr, cnt, hidden, S.ff, false, s, o), "expert GEMM (down) rejected");
        padded += ((size_t)cnt + 127) / 128 * 128;
    }
    return true;
}

// One layer over T rows: x += norm1(mixer(x)); x += norm2(ff(x)); x += side(x, token).  The sublayers read x itself.
void Model::layer_postnorm(int i, int T, const int* tok_dev, const int* pos_dev, int p0, const RowBufs& B, cudaStream_t s) {
    const LayerSpec& S = cfg_.layers[(size_t)i];
    const LayerWeights& L = layer_weights(i);
    LayerWeights& M = layers_[(size_t)i];
    const int hidden = cfg_.hidden_size;
    const float eps = cfg_.norm_eps;
    if (S.mixer == MixerKind::ATTN_LATENT) {
        const LatentSpec& A = S.latent;
        const int row = A.kv_rank + A.rot_dim;
        float *cq = B.t[0], *dkv = B.t[1], *q = B.t[2], *qa = B.t[3], *ol = B.t[4], *o = B.t[2];
        if (T == 1 && S.kv_from < 0) {                  // one decoded token: both down-projections read x, one launch
            GemvMat two[2] = {mat_of(L.w_dq, cq), mat_of(L.w_dkv, dkv)};
            gemv_dense(two, 2, hidden, B.x, DENSE_STORE, nullptr, 1.f, s);
        } else {
            rows_matmul(cq, B.x, L.w_dq, T, s);
            if (S.kv_from < 0) rows_matmul(dkv, B.x, L.w_dkv, T, s);
        }
        latent_prep(cq, A.q_rank, L.dq_norm, S.kv_from < 0 ? dkv : nullptr, A.kv_rank, A.rot_dim, L.dkv_norm, eps, kcs_[(size_t)i], cache_dt_, S.rot.dims,
                    S.rot.interleaved, S.rot.base, T, pos_dev, p0, s);
        rows_matmul(q, cq, L.w_uq, T, s);
        if (!pos_dev && latent_expand_ok(S, T)) {
            latent_attention_rows(i, T, p0, q, o, s);
            rows_matmul(B.y, o, L.wo, T, s);
        } else {
        latent_q_absorb(qa, q, L.w_uk.ptr, L.w_uk.dtype, T, S.heads, S.dim, A.rot_dim, A.kv_rank, S.rot.dims, S.rot.interleaved, S.rot.base, pos_dev, p0, s);
        WindowAttn a;                       // one key / value head: keys are the whole cache rows, values their first kv_rank numbers
        a.heads = S.heads; a.kv_heads = 1; a.dim = row; a.vdim = A.kv_rank; a.scale = S.scale; a.k_stride = row; a.v_stride = row;
        if (lat_part_ && attention_shared_rows_supported(S.heads, row, A.kv_rank, row, cache_dt_, kcs_[(size_t)i]))
            attention_shared_rows(ol, qa, kcs_[(size_t)i], cache_dt_, T, pos_dev, p0, cfg_.max_seq_len, S.heads, row, A.kv_rank, row, S.scale, lat_part_, s);
        else
            attention_window(ol, qa, kcs_[(size_t)i], kcs_[(size_t)i], cache_dt_, T, pos_dev, p0, cfg_.max_seq_len, a, s);
        latent_v_up(o, ol, L.w_uv.ptr, L.w_uv.dtype, T, S.heads, S.vdim, A.kv_rank, s);
        rows_matmul(B.y, o, L.wo, T, s);
        }
    } else {
        const ScanSpec& C = S.scan;
        const int inner = S.heads * S.vdim, ch = inner + 2 * C.groups * C.state, ld = inner + ch + S.heads;
        float *u = B.t[0], *xbc = B.t[1], *ys = B.t[2], *yg = B.t[3];
        rows_matmul(u, B.x, L.ssm_in, T, s);                       // [z | x B C | dt]
        ssm_conv(xbc, u, ld, inner, M.conv_state, L.ssm_conv, L.ssm_conv_b, T, ch, C.conv, pos_dev, p0, s);
        ssm_scan(ys, xbc, u, ld, inner + ch, M.ssm_state, L.ssm_dt_bias, L.ssm_a_log, L.ssm_d, T, S.heads, S.vdim, C.state, C.groups, pos_dev, p0, s);
        ssm_gate_norm(yg, ys, u, ld, 0, L.ssm_norm, eps, T, inner, C.norm_groups, s);
        rows_matmul(B.y, yg, L.wo, T, s);
    }
    add_rmsnorm_rows(B.x, B.y, L.attn_norm, nullptr, T, hidden, eps, s);
    if (S.ff > 0 && S.ff_kind == FfKind::GLU) {
        float *g = B.t[0], *up = B.t[1];
        if (T == 1) {
            GemvMat two[2] = {mat_of(L.gate, g), mat_of(L.up, up)};
            gemv_dense(two, 2, hidden, B.x, DENSE_STORE, nullptr, 1.f, s);
        } else {
            rows_matmul(g, B.x, L.gate, T, s);
            rows_matmul(up, B.x, L.up, T, s);
        }
        glu_bias_mul(g, g, up, L.gate_b, L.up_b, T, S.ff, S.act == GluAct::GELU_TANH, s);
        rows_matmul(B.y, g, L.down, T, s);
        add_rmsnorm_rows(B.x, B.y, L.ffn_norm, L.down_b, T, hidden, eps, s);
    } else if (S.ff > 0) {
        MoeWeights w;
        w.router = L.router; w.up = L.e_up_tab; w.down = L.e_down_tab; w.gate = L.e_gate_tab; w.dtype = L.e_up[0].dtype;
        w.experts = S.experts; w.top = S.top; w.ff = S.ff; w.width = hidden;
        w.sigmoid = S.route.sigmoid; w.correction = S.route.correction ? L.route_corr : nullptr; w.groups = S.route.groups; w.keep = S.route.keep;
        if (T == 1) {
            moe_route(moe_sel_, moe_wt_, nullptr, B.x, w, 1, s);
            moe_expert_up_token(moe_act_, B.x, moe_sel_, w, s);
            moe_expert_down_token(B.y, moe_act_, moe_sel_, moe_wt_, nullptr, nullptr, w, s);
        } else {
            moe_route(pf_.sel, pf_.wt, nullptr, B.x, w, T, s);
            moe_group(pf_.work, pf_.sel, T, S.experts, S.top, s);
            if (S.act != GluAct::SILU || !moe_glu_rows_tc(i, T, B.x, s)) {
                moe_expert_gate_rows(pf_.gate_rows, B.x, pf_.work, w, T, s);
                moe_expert_up_rows(pf_.act_rows, B.x, pf_.work, w, T, s);
                glu_bias_mul(pf_.act_rows, pf_.gate_rows, pf_.act_rows, nullptr, nullptr, T * S.top, S.ff, false, s);
                moe_expert_down_rows(pf_.y_rows, pf_.act_rows, pf_.work, w, T, s);
            }
            moe_combine(B.y, pf_.y_rows, pf_.work, pf_.wt, nullptr, nullptr, T, S.experts, S.top, hidden, s);
        }
        add_rmsnorm_rows(B.x, B.y, L.ffn_norm, nullptr, T, hidden, eps, s);
    }
    if (cfg_.side_dim > 0) {
        float* g = B.t[0];
        rows_matmul(g, B.x, L.side_gate, T, s);
        side_gate_rows(g, side_embd_.ptr, side_embd_.dtype, cfg_.n_layers * cfg_.side_dim, i * cfg_.side_dim, tok_dev, T, cfg_.side_dim, s);
        rows_matmul(B.y, g, L.side_proj, T, s);
        add_rmsnorm_rows(B.x, B.y, L.side_norm, nullptr, T, hidden, eps, s);
    }
}

}}  // namespace nt::b200
