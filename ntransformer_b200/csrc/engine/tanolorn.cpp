// tanolorn.cpp — the Tanolorn family: a decoder whose layers, in any order the configuration lists, mix tokens either by low-rank
// ("latent") attention (MixerKind::ATTN_LATENT: the cache row of a position is one normed latent plus one rotated key part shared
// by all heads; rotate-half rotary positions on that part and on the matching part of every query head; full causal softmax; a
// layer may read an earlier layer's cache rows, LayerSpec::kv_from) or by a selective state-space scan (MixerKind::SSM_SCAN: short
// causal convolution, per-head scalar decay, gated and group-normed output; a fixed-size state instead of cache rows).  The block
// is post-norm (BlockForm::POST_NORM: x += norm(sublayer(x)), gains stored around zero).  The feed-forward is a SiLU-gated unit with
// biases or a mixture of SiLU-gated experts chosen by sigmoid scores with a choice-only correction and a limit to the best groups
// of neighbouring experts (FfKind::MOE_GLU, RouteSpec).  After every layer a per-layer slice of a second token embedding, gated by
// the residual, is projected back and added (ModelConfig::side_dim).
// Everything that varies between models of the family is read from config.json; "mlp": null, an absent "token_side", "rot",
// "router.groups" and "kv_from" switch their mechanism off.
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

bool latent_from_json(const Json& m, LayerSpec& L, const ModelConfig& cfg, size_t i, std::string& err, const std::string& where) {
    L.mixer = MixerKind::ATTN_LATENT;
    L.kv_heads = 1;
    if (!need_int(m, "heads", L.heads, err, where) || !need_int(m, "dim", L.dim, err, where) || !need_int(m, "vdim", L.vdim, err, where) ||
        !need_int(m, "rot_dim", L.latent.rot_dim, err, where) || !need_int(m, "q_rank", L.latent.q_rank, err, where) ||
        !need_int(m, "kv_rank", L.latent.kv_rank, err, where) || !need_float(m, "scale", L.scale, err, where)) return false;
    if (L.heads <= 0 || L.dim < 0 || L.vdim <= 0 || L.latent.rot_dim < 0 || L.dim + L.latent.rot_dim <= 0 || L.latent.q_rank <= 0 || L.latent.kv_rank <= 0) {
        err = where + ": invalid mixer sizes"; return false;
    }
    L.rot.interleaved = false;                 // channel i pairs with channel i + dims / 2
    if (m.has("rot") && m.at("rot").is_object()) {
        const Json& r = m.at("rot");
        if (!need_int(r, "dims", L.rot.dims, err, where + ".rot") || !need_float(r, "base", L.rot.base, err, where + ".rot")) return false;
        if (L.rot.dims < 0 || L.rot.dims > L.latent.rot_dim || (L.rot.dims & 1) || L.rot.base <= 0.f) { err = where + ": rot.dims must be even and at most rot_dim"; return false; }
    }
    if (m.has("kv_from")) {
        L.kv_from = (int)m.at("kv_from").int_or(-1);
        if (L.kv_from < 0 || L.kv_from >= (int)i) { err = where + ": \"kv_from\" must name an earlier layer"; return false; }
        const LayerSpec& J = cfg.layers[(size_t)L.kv_from];
        if (J.mixer != MixerKind::ATTN_LATENT || J.kv_from >= 0) { err = where + ": \"kv_from\" must name a latent-attention layer that has its own key / value latent"; return false; }
        if (J.latent.kv_rank != L.latent.kv_rank || J.latent.rot_dim != L.latent.rot_dim || J.rot.dims != L.rot.dims || J.rot.base != L.rot.base) {
            err = where + ": \"kv_from\" layer has another latent size or rotation"; return false;
        }
    }
    return true;
}

bool scan_from_json(const Json& m, LayerSpec& L, std::string& err, const std::string& where) {
    L.mixer = MixerKind::SSM_SCAN;
    if (!need_int(m, "heads", L.heads, err, where) || !need_int(m, "vdim", L.vdim, err, where) || !need_int(m, "state", L.scan.state, err, where) ||
        !need_int(m, "groups", L.scan.groups, err, where) || !need_int(m, "conv", L.scan.conv, err, where) ||
        !need_int(m, "norm_groups", L.scan.norm_groups, err, where)) return false;
    if (L.heads <= 0 || L.vdim <= 0 || L.scan.state <= 0 || L.scan.groups <= 0 || L.heads % L.scan.groups || L.scan.conv <= 0 || L.scan.conv > 16 ||
        L.scan.norm_groups <= 0 || (L.heads * L.vdim) % L.scan.norm_groups) {
        err = where + ": invalid scan sizes (heads % groups == 0, 1 <= conv <= 16, heads * vdim % norm_groups == 0)"; return false;
    }
    return true;
}

bool config_from_json(const Json& root, ModelConfig& cfg, std::string& err) {
    if (!need_int(root, "vocab", cfg.vocab_size, err, "config") || !need_int(root, "width", cfg.hidden_size, err, "config")) return false;
    if (!need_float(root.at("norm"), "eps", cfg.norm_eps, err, "config.norm")) return false;
    cfg.norm_gain_offset = 1.0f;
    cfg.side_dim = 0;
    if (root.has("token_side") && root.at("token_side").is_object()) {
        if (!need_int(root.at("token_side"), "dim", cfg.side_dim, err, "config.token_side") || cfg.side_dim <= 0) { if (err.empty()) err = "config.token_side: invalid dim"; return false; }
    }
    const Json& layers = root.at("layers");
    if (!layers.is_array() || layers.arr.empty()) { err = "config: \"layers\" must be a non-empty list"; return false; }
    cfg.n_layers = (int)layers.arr.size();
    cfg.model_name = "tanolorn";
    cfg.bos_token_id = -1; cfg.eos_token_id = -1;
    for (size_t i = 0; i < layers.arr.size(); i++) {
        const Json& e = layers.arr[i];
        const std::string where = "config.layers[" + std::to_string(i) + "]";
        LayerSpec L;
        L.form = BlockForm::POST_NORM;
        const std::string type = e.at("type").string_or("");
        const Json& m = e.at("mixer");
        if (!m.is_object()) { err = where + ": \"mixer\" is missing"; return false; }
        if (type == "latent_attention") { if (!latent_from_json(m, L, cfg, i, err, where)) return false; }
        else if (type == "mamba2") { if (!scan_from_json(m, L, err, where)) return false; }
        else { err = where + ": mixer type \"" + type + "\" is not part of this family"; return false; }
        const Json& mlp = e.at("mlp");
        if (mlp.is_null()) L.ff = 0;
        else {
            const std::string kind = mlp.at("kind").string_or("");
            L.act = GluAct::SILU;
            if (kind == "dense") {
                L.ff_kind = FfKind::GLU; L.ff_bias = true;
                if (!need_int(mlp, "ff", L.ff, err, where + ".mlp") || L.ff <= 0) { if (err.empty()) err = where + ": invalid ff"; return false; }
            } else if (kind == "moe") {
                L.ff_kind = FfKind::MOE_GLU;
                L.route.sigmoid = true; L.route.correction = true;
                const Json& r = mlp.at("router");
                if (!need_int(mlp.at("expert"), "ff", L.ff, err, where + ".mlp.expert") || !need_int(r, "experts", L.experts, err, where + ".mlp.router") ||
                    !need_int(r, "top", L.top, err, where + ".mlp.router")) return false;
                if (L.ff <= 0 || L.experts <= 0 || L.top <= 0 || L.top > L.experts || L.experts > 256) { err = where + ": invalid expert sizes (1 <= top <= experts <= 256)"; return false; }
                if (r.has("groups") && r.at("groups").is_object()) {
                    if (!need_int(r.at("groups"), "count", L.route.groups, err, where + ".mlp.router.groups") ||
                        !need_int(r.at("groups"), "keep", L.route.keep, err, where + ".mlp.router.groups")) return false;
                    if (L.route.groups <= 0 || L.experts % L.route.groups || L.route.keep <= 0 || L.route.keep > L.route.groups ||
                        L.route.keep * (L.experts / L.route.groups) < L.top) {
                        err = where + ": invalid expert groups (experts % count == 0, 1 <= keep <= count, the kept groups must hold at least top experts)"; return false;
                    }
                }
            } else { err = where + ": feed-forward kind \"" + kind + "\" is not part of this family"; return false; }
        }
        cfg.layers.push_back(L);
    }
    cfg.n_heads = cfg.n_kv_heads = cfg.head_dim = cfg.intermediate_size = 0;
    for (const LayerSpec& L : cfg.layers) {
        cfg.n_heads = std::max(cfg.n_heads, L.heads); cfg.n_kv_heads = std::max(cfg.n_kv_heads, L.kv_heads);
        cfg.head_dim = std::max(cfg.head_dim, L.dim); cfg.intermediate_size = std::max(cfg.intermediate_size, L.ff);
    }
    cfg.max_seq_len = 4096;
    return true;
}

std::vector<TensorBinding> tensors(const ModelConfig& cfg) {
    std::vector<TensorBinding> t;
    const int W = cfg.hidden_size;
    t.push_back({"embed", TensorSlot::EMBED, -1, cfg.vocab_size, W});
    if (cfg.side_dim > 0) t.push_back({"side.embed", TensorSlot::SIDE_EMBED, -1, cfg.vocab_size, cfg.n_layers * cfg.side_dim});
    t.push_back({"final.norm", TensorSlot::OUT_NORM, -1, 1, W});
    t.push_back({"head", TensorSlot::HEAD, -1, cfg.vocab_size, W});
    for (int i = 0; i < cfg.n_layers; i++) {
        const LayerSpec& L = cfg.layers[(size_t)i];
        const std::string p = "l" + std::to_string(i) + ".";
        t.push_back({p + "norm1", TensorSlot::NORM1, i, 1, W});
        if (L.mixer == MixerKind::ATTN_LATENT) {
            const LatentSpec& A = L.latent;
            t.push_back({p + "mix.dq", TensorSlot::W_DQ, i, A.q_rank, W});
            t.push_back({p + "mix.dq.norm", TensorSlot::DQ_NORM, i, 1, A.q_rank});
            t.push_back({p + "mix.uq", TensorSlot::W_UQ, i, L.heads * (L.dim + A.rot_dim), A.q_rank});
            if (L.kv_from < 0) {
                t.push_back({p + "mix.dkv", TensorSlot::W_DKV, i, A.kv_rank + A.rot_dim, W});
                t.push_back({p + "mix.dkv.norm", TensorSlot::DKV_NORM, i, 1, A.kv_rank});
            }
            if (L.dim > 0) t.push_back({p + "mix.uk", TensorSlot::W_UK, i, L.heads * L.dim, A.kv_rank});
            t.push_back({p + "mix.uv", TensorSlot::W_UV, i, L.heads * L.vdim, A.kv_rank});
            t.push_back({p + "mix.o", TensorSlot::WO, i, W, L.heads * L.vdim});
        } else {
            const int inner = L.heads * L.vdim, ch = inner + 2 * L.scan.groups * L.scan.state;
            t.push_back({p + "mix.in", TensorSlot::SSM_IN, i, inner + ch + L.heads, W});
            t.push_back({p + "mix.conv", TensorSlot::SSM_CONV, i, ch, L.scan.conv});
            t.push_back({p + "mix.conv.b", TensorSlot::SSM_CONV_B, i, 1, ch});
            t.push_back({p + "mix.dt_bias", TensorSlot::SSM_DT_BIAS, i, 1, L.heads});
            t.push_back({p + "mix.A_log", TensorSlot::SSM_A_LOG, i, 1, L.heads});
            t.push_back({p + "mix.D", TensorSlot::SSM_D, i, 1, L.heads});
            t.push_back({p + "mix.norm", TensorSlot::SSM_NORM, i, 1, inner});
            t.push_back({p + "mix.o", TensorSlot::WO, i, W, inner});
        }
        if (L.ff > 0) {
            t.push_back({p + "norm2", TensorSlot::NORM2, i, 1, W});
            if (L.ff_kind == FfKind::GLU) {
                t.push_back({p + "mlp.gate", TensorSlot::GATE, i, L.ff, W});
                t.push_back({p + "mlp.up", TensorSlot::UP, i, L.ff, W});
                t.push_back({p + "mlp.down", TensorSlot::DOWN, i, W, L.ff});
                if (L.ff_bias) {
                    t.push_back({p + "mlp.gate.b", TensorSlot::GATE_B, i, 1, L.ff});
                    t.push_back({p + "mlp.up.b", TensorSlot::UP_B, i, 1, L.ff});
                    t.push_back({p + "mlp.down.b", TensorSlot::DOWN_B, i, 1, W});
                }
            } else {
                t.push_back({p + "mlp.router", TensorSlot::ROUTER, i, L.experts, W});
                if (L.route.correction) t.push_back({p + "mlp.correction", TensorSlot::ROUTE_CORRECTION, i, 1, L.experts});
                for (int e = 0; e < L.experts; e++) {
                    const std::string q = p + "mlp.e" + std::to_string(e) + ".";
                    t.push_back({q + "gate", TensorSlot::EXPERT_GATE, i, L.ff, W, e});
                    t.push_back({q + "up", TensorSlot::EXPERT_UP, i, L.ff, W, e});
                    t.push_back({q + "down", TensorSlot::EXPERT_DOWN, i, W, L.ff, e});
                }
            }
        }
        if (cfg.side_dim > 0) {
            t.push_back({p + "side.gate", TensorSlot::SIDE_GATE, i, cfg.side_dim, W});
            t.push_back({p + "side.proj", TensorSlot::SIDE_PROJ, i, W, cfg.side_dim});
            t.push_back({p + "side.norm", TensorSlot::SIDE_NORM, i, 1, W});
        }
    }
    return t;
}

const ModelFamily kFamily = {"Tanolorn", config_from_json, tensors};

}  // namespace

const ModelFamily* tanolorn_family() { return &kFamily; }

}}  // namespace nt::b200
