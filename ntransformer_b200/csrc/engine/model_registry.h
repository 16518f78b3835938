// model_registry.h — model families that load from a folder (config.json + model.safetensors).  A family is chosen by the
// config's "architecture" string; it turns the JSON into a ModelConfig with one LayerSpec per layer and lists the tensors the
// model needs, each bound to a slot of the resident model (engine/model.h).  The GGUF Llama family keeps its own loader
// (Model::load_gguf); Model::load picks by what the path is.
#pragma once
#include <functional>
#include <string>
#include <vector>
#include "gguf.h"
#include "json.h"

namespace nt { namespace b200 {

enum class TensorSlot { EMBED, HEAD, OUT_NORM, NORM1, NORM2, WQ, WK, WV, WO, Q_NORM, K_NORM, GATE, UP, DOWN, LS1, LS2,
                        LQ1, LK1, LQ2, LK2,                         // differential attention: the four vectors of lambda
                        HC1_IN, HC1_OUT, HC1_MIX, HC2_IN, HC2_OUT, HC2_MIX,   // residual streams: read blend, write gains, stream mixing [from, to]
                        ROUTER, EXPERT_UP, EXPERT_DOWN, SHARED_UP, SHARED_DOWN, SHARED_GATE,
                        EXPERT_GATE, ROUTE_CORRECTION, GATE_B, UP_B, DOWN_B,              // gated experts, choice correction, feed-forward biases
                        W_DQ, DQ_NORM, W_UQ, W_DKV, DKV_NORM, W_UK, W_UV,                 // low-rank attention (WO is shared with the other mixers)
                        SSM_IN, SSM_CONV, SSM_CONV_B, SSM_DT_BIAS, SSM_A_LOG, SSM_D, SSM_NORM,   // state-space scan
                        SIDE_EMBED, SIDE_GATE, SIDE_PROJ, SIDE_NORM,                      // per-layer token input
                        SHIFT_MU,                                                         // token shift: per-channel blend with the previous token's input
                        Q_BIAS, K_BIAS, V_BIAS, O_BIAS, Q_CONV, K_CONV, V_CONV,           // biased projections; short convolutions [channels, taps] on q, k, v
                        HEAD_TEMP, TALK, SINK, V_MIX,                                     // per-head score multiplier, head-mixing matrix [heads, heads], sink, lambda
                        DELTA_BETA, DELTA_A1, DELTA_A2, DELTA_DT_BIAS, DELTA_A_LOG, DELTA_NORM, DELTA_G1, DELTA_G2 };   // gated delta rule

struct TensorBinding {
    std::string name;      // in the checkpoint
    TensorSlot slot;
    int layer;             // -1 for model-level tensors
    int rows, cols;        // expected shape (vectors: rows == 1)
    int index = 0;         // which expert (EXPERT_UP / EXPERT_DOWN)
    int branch = -1;       // >= 0: the tensor belongs to that branch of a BRANCHES mixer
};
// Slots kept as F32 vectors / small F32 tables whatever the checkpoint stores (gains, lambda vectors, stream tables, router rows).
bool slot_is_f32_table(TensorSlot s);

// Looks a checkpoint tensor's shape up by name; false when the checkpoint has no such tensor.
using TensorShapeFn = std::function<bool(const std::string& name, std::vector<int64_t>& shape)>;

struct ModelFamily {
    const char* architecture;
    bool (*config_from_json)(const Json& root, ModelConfig& cfg, std::string& err);
    std::vector<TensorBinding> (*tensors)(const ModelConfig& cfg);
    // Optional: sizes that config.json does not state and only a tensor's shape gives (ranks of low-rank projections).  Called by the
    // folder loader between config_from_json and tensors; sizes the configuration already states are left alone.
    bool (*sizes_from_tensors)(ModelConfig& cfg, const TensorShapeFn& shape_of, std::string& err) = nullptr;
};

const ModelFamily* find_model_family(const std::string& architecture);
const std::vector<const ModelFamily*>& model_families();
// Reads <dir>/config.json; false (+ message) when it is missing, malformed or names no registered family.
bool read_model_dir(const std::string& dir, ModelConfig& cfg, const ModelFamily** family);

const ModelFamily* zelunex_family();      // engine/zelunex.cpp
const ModelFamily* vebotar_family();      // engine/vebotar.cpp
const ModelFamily* tanolorn_family();     // engine/tanolorn.cpp
const ModelFamily* savidra_family();      // engine/savidra.cpp

}}  // namespace nt::b200
