// savidra.cpp — the Savidra family: a decoder whose block norms the residual sum itself (BlockForm::SUM_NORM:
// x <- n(a x + mixer(shift(x)), g1), x <- n(a x + ff(x), g2), gains stored around zero, a = "postln_alpha") and whose mixer reads a
// per-channel blend of the token's and the previous token's input (LayerSpec::token_shift).  A layer's mixer, in whatever order the
// configuration lists them, is either
//   "attention": grouped-query attention with per-head RMS norm of q and k (QKNorm::PER_HEAD), rotate-half rotary positions on the
//                first rot.dims channels, a learned sink in the softmax denominator (LayerSpec::sink) and, where "v_mix" is set, values
//                blended with the values the first such layer computed for the same token (LayerSpec::v_first); or
//   "parallel":  two mixers side by side (MixerKind::BRANCHES) summed with the fixed weights "left_scale" / "right_scale":
//                left  — attention with biased projections, a short causal convolution on q, k and v (LayerSpec::conv), per-head q / k
//                        norm, rotary positions with linearly scaled frequencies (RotarySpec::divide), a per-head score multiplier
//                        (head_temp) and softmax weights mixed across heads (talking);
//                right — the gated delta rule (MixerKind::DELTA_RULE, DeltaSpec).
// The feed-forward is a ReLU-gated unit without biases, or absent ("mlp": null).  Every size and constant that varies between models
// of the family is read from config.json; the ranks of the delta rule's two low-rank projections are the row counts of their first
// matrices (or "decay_rank" / "gate_rank" when the configuration states them).
#include "model_registry.h"
#include <algorithm>

namespace nt { namespace b200 {

namespace {

bool need_int(const Json& o, const char* key, int& out, std::string& err, const std::string& where) {
    const Json& v = o.at(key);
    if (!v.is_number()) { err = where + ": \"" + key + "\" is missing or not a number"; return false; }
    out = (int)v.int_or(0);
    return true;
}
bool need_float(const Json& o, const char* key, float& out, std::string& err, const std::string& where) {
    const Json& v = o.at(key);
    if (!v.is_number()) { err = where + ": \"" + key + "\" is missing or not a number"; return false; }
    out = (float)v.number_or(0.0);
    return true;
}

bool rot_from_json(const Json& m, LayerSpec& L, std::string& err, const std::string& where) {
    L.rot.interleaved = false;                 // channel i pairs with channel i + dims / 2
    if (!m.has("rot") || !m.at("rot").is_object()) return true;
    const Json& r = m.at("rot");
    if (!need_int(r, "dims", L.rot.dims, err, where + ".rot") || !need_float(r, "base", L.rot.base, err, where + ".rot")) return false;
    if (L.rot.dims < 0 || L.rot.dims > L.dim || (L.rot.dims & 1) || L.rot.base <= 0.f) { err = where + ": rot.dims must be even and at most dim"; return false; }
    if (r.has("scaling") && r.at("scaling").is_object()) {
        if (!need_float(r.at("scaling"), "factor", L.rot.divide, err, where + ".rot.scaling")) return false;
        if (!(L.rot.divide > 0.f)) { err = where + ": rot.scaling.factor must be positive"; return false; }
    }
    return true;
}

bool attention_sizes(const Json& m, LayerSpec& L, std::string& err, const std::string& where) {
    L.mixer = MixerKind::ATTN_WINDOW;          // window 0: every earlier position is visible
    L.qk_norm = QKNorm::PER_HEAD;
    if (!need_int(m, "heads", L.heads, err, where) || !need_int(m, "kv_heads", L.kv_heads, err, where) || !need_int(m, "dim", L.dim, err, where) ||
        !need_int(m, "vdim", L.vdim, err, where) || !need_float(m, "scale", L.scale, err, where)) return false;
    if (L.heads <= 0 || L.kv_heads <= 0 || L.heads % L.kv_heads || L.dim <= 0 || L.vdim <= 0) { err = where + ": invalid head sizes (heads % kv_heads == 0)"; return false; }
    return rot_from_json(m, L, err, where);
}

bool conv_from_json(const Json& m, LayerSpec& L, std::string& err, const std::string& where) {
    if (!m.has("conv")) return true;
    if (!need_int(m, "conv", L.conv, err, where)) return false;
    if (L.conv < 1 || L.conv > 16) { err = where + ": 1 <= conv <= 16"; return false; }
    return true;
}

bool delta_from_json(const Json& m, LayerSpec& L, std::string& err, const std::string& where) {
    L.mixer = MixerKind::DELTA_RULE;
    if (!need_int(m, "heads", L.heads, err, where) || !need_int(m, "kv_heads", L.kv_heads, err, where) || !need_int(m, "dim", L.dim, err, where) ||
        !need_int(m, "vdim", L.vdim, err, where)) return false;
    if (L.heads <= 0 || L.kv_heads <= 0 || L.heads % L.kv_heads || L.dim <= 0 || L.vdim <= 0) { err = where + ": invalid head sizes (heads % kv_heads == 0)"; return false; }
    if (m.has("decay_rank") && !need_int(m, "decay_rank", L.delta.decay_rank, err, where)) return false;
    if (m.has("gate_rank") && !need_int(m, "gate_rank", L.delta.gate_rank, err, where)) return false;
    if (L.delta.decay_rank < 0 || L.delta.gate_rank < 0) { err = where + ": invalid ranks"; return false; }
    return conv_from_json(m, L, err, where);
}

bool config_from_json(const Json& root, ModelConfig& cfg, std::string& err) {
    if (!need_int(root, "vocab", cfg.vocab_size, err, "config") || !need_int(root, "width", cfg.hidden_size, err, "config")) return false;
    if (!need_float(root.at("norm"), "eps", cfg.norm_eps, err, "config.norm")) return false;
    if (!need_float(root, "postln_alpha", cfg.skip_scale, err, "config")) return false;
    if (cfg.vocab_size <= 0 || cfg.hidden_size <= 0) { err = "config: invalid vocab / width"; return false; }
    cfg.norm_gain_offset = 1.0f;
    const Json& layers = root.at("layers");
    if (!layers.is_array() || layers.arr.empty()) { err = "config: \"layers\" must be a non-empty list"; return false; }
    cfg.n_layers = (int)layers.arr.size();
    cfg.model_name = "savidra";
    cfg.bos_token_id = -1; cfg.eos_token_id = -1;
    int v_first = -1;
    for (size_t i = 0; i < layers.arr.size(); i++) {
        const Json& e = layers.arr[i];
        const std::string where = "config.layers[" + std::to_string(i) + "]";
        LayerSpec L;
        L.form = BlockForm::SUM_NORM;
        L.token_shift = true;
        const std::string type = e.at("type").string_or("");
        const Json& m = e.at("mixer");
        if (!m.is_object()) { err = where + ": \"mixer\" is missing"; return false; }
        if (type == "attention") {
            if (!attention_sizes(m, L, err, where)) return false;
            L.sink = true;
            if (m.at("v_mix").kind == Json::Bool && m.at("v_mix").b) {
                if (v_first < 0) v_first = (int)i;
                else {
                    const LayerSpec& F = cfg.layers[(size_t)v_first];
                    if (F.kv_heads * F.vdim != L.kv_heads * L.vdim) { err = where + ": \"v_mix\" layers must have values of one width"; return false; }
                }
                L.v_first = v_first;
            }
        } else if (type == "parallel") {
            L.mixer = MixerKind::BRANCHES;
            LayerSpec A, B;
            if (!m.at("left").is_object() || !m.at("right").is_object()) { err = where + ": \"left\" / \"right\" are missing"; return false; }
            if (!attention_sizes(m.at("left"), A, err, where + ".left") || !conv_from_json(m.at("left"), A, err, where + ".left")) return false;
            A.qkv_bias = true; A.head_temp = true; A.talking = true;
            if (!delta_from_json(m.at("right"), B, err, where + ".right")) return false;
            float ls = 1.f, rs = 1.f;
            if (!need_float(m, "left_scale", ls, err, where) || !need_float(m, "right_scale", rs, err, where)) return false;
            L.branches = {A, B};
            L.branch_scale = {ls, rs};
        } else { err = where + ": mixer type \"" + type + "\" is not part of this family"; return false; }
        const Json& mlp = e.at("mlp");
        if (mlp.is_null()) L.ff = 0;
        else {
            const std::string kind = mlp.at("kind").string_or("");
            if (kind != "dense") { err = where + ": feed-forward kind \"" + kind + "\" is not part of this family"; return false; }
            L.ff_kind = FfKind::GLU; L.act = GluAct::RELU;
            if (!need_int(mlp, "ff", L.ff, err, where + ".mlp") || L.ff <= 0) { if (err.empty()) err = where + ": invalid ff"; return false; }
        }
        cfg.layers.push_back(L);
    }
    cfg.n_heads = cfg.n_kv_heads = cfg.head_dim = cfg.intermediate_size = 0;
    auto widen = [&](const LayerSpec& L) {
        cfg.n_heads = std::max(cfg.n_heads, L.heads); cfg.n_kv_heads = std::max(cfg.n_kv_heads, L.kv_heads);
        cfg.head_dim = std::max(cfg.head_dim, L.dim);
    };
    for (const LayerSpec& L : cfg.layers) {
        widen(L);
        for (const LayerSpec& b : L.branches) widen(b);
        cfg.intermediate_size = std::max(cfg.intermediate_size, L.ff);
    }
    cfg.max_seq_len = 4096;
    return true;
}

std::string mixer_prefix(int layer, const LayerSpec& L, int branch) {
    std::string p = "l" + std::to_string(layer) + ".mix.";
    if (L.mixer == MixerKind::BRANCHES) p += branch == 0 ? "left." : "right.";
    return p;
}

// The ranks of the delta rule's low-rank projections: rows of '<mixer>.a1' and '<mixer>.g1'.
bool sizes_from_tensors(ModelConfig& cfg, const TensorShapeFn& shape_of, std::string& err) {
    for (int i = 0; i < cfg.n_layers; i++) {
        LayerSpec& L = cfg.layers[(size_t)i];
        for (size_t b = 0; b < L.branches.size(); b++) {
            LayerSpec& S = L.branches[b];
            if (S.mixer != MixerKind::DELTA_RULE) continue;
            const std::string p = mixer_prefix(i, L, (int)b);
            std::vector<int64_t> sh;
            if (S.delta.decay_rank <= 0) {
                if (!shape_of(p + "a1", sh) || sh.size() != 2 || sh[0] <= 0) { err = "tensor " + p + "a1 is missing or not a matrix"; return false; }
                S.delta.decay_rank = (int)sh[0];
            }
            if (S.delta.gate_rank <= 0) {
                if (!shape_of(p + "g1", sh) || sh.size() != 2 || sh[0] <= 0) { err = "tensor " + p + "g1 is missing or not a matrix"; return false; }
                S.delta.gate_rank = (int)sh[0];
            }
        }
    }
    return true;
}

void attention_tensors(std::vector<TensorBinding>& t, const std::string& p, const LayerSpec& S, int W, int layer, int branch) {
    auto add = [&](const std::string& name, TensorSlot slot, int rows, int cols) {
        TensorBinding b{p + name, slot, layer, rows, cols};
        b.branch = branch;
        t.push_back(b);
    };
    const int q = S.heads * S.dim, k = S.kv_heads * S.dim, v = S.kv_heads * S.vdim;
    add("q", TensorSlot::WQ, q, W); add("k", TensorSlot::WK, k, W); add("v", TensorSlot::WV, v, W);
    add("o", TensorSlot::WO, W, S.heads * S.vdim);
    add("q.norm", TensorSlot::Q_NORM, 1, S.dim); add("k.norm", TensorSlot::K_NORM, 1, S.dim);
    if (S.qkv_bias) { add("q.b", TensorSlot::Q_BIAS, 1, q); add("k.b", TensorSlot::K_BIAS, 1, k); add("v.b", TensorSlot::V_BIAS, 1, v); add("o.b", TensorSlot::O_BIAS, 1, W); }
    if (S.conv > 0) { add("q.conv", TensorSlot::Q_CONV, q, S.conv); add("k.conv", TensorSlot::K_CONV, k, S.conv); add("v.conv", TensorSlot::V_CONV, v, S.conv); }
    if (S.talking) add("talk", TensorSlot::TALK, S.heads, S.heads);
    if (S.head_temp) add("temp", TensorSlot::HEAD_TEMP, 1, S.heads);
    if (S.sink) add("sink", TensorSlot::SINK, 1, S.heads);
    if (S.v_first >= 0) add("vmix", TensorSlot::V_MIX, 1, 1);
}

void delta_tensors(std::vector<TensorBinding>& t, const std::string& p, const LayerSpec& S, int W, int layer, int branch) {
    auto add = [&](const std::string& name, TensorSlot slot, int rows, int cols) {
        TensorBinding b{p + name, slot, layer, rows, cols};
        b.branch = branch;
        t.push_back(b);
    };
    const int qk = S.kv_heads * S.dim, v = S.heads * S.vdim, hd = S.heads * S.dim;
    add("q", TensorSlot::WQ, qk, W); add("k", TensorSlot::WK, qk, W); add("v", TensorSlot::WV, v, W);
    if (S.conv > 0) { add("q.conv", TensorSlot::Q_CONV, qk, S.conv); add("k.conv", TensorSlot::K_CONV, qk, S.conv); add("v.conv", TensorSlot::V_CONV, v, S.conv); }
    add("b", TensorSlot::DELTA_BETA, S.heads, W);
    add("A_log", TensorSlot::DELTA_A_LOG, 1, S.heads);
    add("norm", TensorSlot::DELTA_NORM, 1, S.vdim);
    add("a1", TensorSlot::DELTA_A1, S.delta.decay_rank, W); add("a2", TensorSlot::DELTA_A2, hd, S.delta.decay_rank);
    add("dt_bias", TensorSlot::DELTA_DT_BIAS, 1, hd);
    add("g1", TensorSlot::DELTA_G1, S.delta.gate_rank, W); add("g2", TensorSlot::DELTA_G2, v, S.delta.gate_rank);
    add("o", TensorSlot::WO, W, v);
}

std::vector<TensorBinding> tensors(const ModelConfig& cfg) {
    std::vector<TensorBinding> t;
    const int W = cfg.hidden_size;
    t.push_back({"embed", TensorSlot::EMBED, -1, cfg.vocab_size, W});
    t.push_back({"final.norm", TensorSlot::OUT_NORM, -1, 1, W});
    t.push_back({"head", TensorSlot::HEAD, -1, cfg.vocab_size, W});
    for (int i = 0; i < cfg.n_layers; i++) {
        const LayerSpec& L = cfg.layers[(size_t)i];
        const std::string p = "l" + std::to_string(i) + ".";
        t.push_back({p + "norm1", TensorSlot::NORM1, i, 1, W});
        if (L.token_shift) t.push_back({p + "shift", TensorSlot::SHIFT_MU, i, 1, W});
        if (L.mixer == MixerKind::BRANCHES) {
            for (size_t b = 0; b < L.branches.size(); b++) {
                const LayerSpec& S = L.branches[b];
                if (S.mixer == MixerKind::DELTA_RULE) delta_tensors(t, mixer_prefix(i, L, (int)b), S, W, i, (int)b);
                else attention_tensors(t, mixer_prefix(i, L, (int)b), S, W, i, (int)b);
            }
        } else attention_tensors(t, mixer_prefix(i, L, -1), L, W, i, -1);
        if (L.ff > 0) {
            t.push_back({p + "norm2", TensorSlot::NORM2, i, 1, W});
            t.push_back({p + "mlp.gate", TensorSlot::GATE, i, L.ff, W});
            t.push_back({p + "mlp.up", TensorSlot::UP, i, L.ff, W});
            t.push_back({p + "mlp.down", TensorSlot::DOWN, i, W, L.ff});
        }
    }
    return t;
}

const ModelFamily kFamily = {"Savidra", config_from_json, tensors, sizes_from_tensors};

}  // namespace

const ModelFamily* savidra_family() { return &kFamily; }

}}  // namespace nt::b200
