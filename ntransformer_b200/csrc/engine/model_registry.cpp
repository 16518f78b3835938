// model_registry.cpp — see model_registry.h.
#include "model_registry.h"
#include <cstdio>
#include <fstream>
#include <sstream>

namespace nt { namespace b200 {

const std::vector<const ModelFamily*>& model_families() {
    static const std::vector<const ModelFamily*> all = {zelunex_family(), vebotar_family(), tanolorn_family(), savidra_family()};
    return all;
}

bool slot_is_f32_table(TensorSlot s) {
    switch (s) {
        case TensorSlot::EMBED: case TensorSlot::HEAD: case TensorSlot::WQ: case TensorSlot::WK: case TensorSlot::WV: case TensorSlot::WO:
        case TensorSlot::GATE: case TensorSlot::UP: case TensorSlot::DOWN: case TensorSlot::EXPERT_UP: case TensorSlot::EXPERT_DOWN:
        case TensorSlot::SHARED_UP: case TensorSlot::SHARED_DOWN: case TensorSlot::EXPERT_GATE:
        case TensorSlot::W_DQ: case TensorSlot::W_UQ: case TensorSlot::W_DKV: case TensorSlot::W_UK: case TensorSlot::W_UV:
        case TensorSlot::SSM_IN: case TensorSlot::SIDE_EMBED: case TensorSlot::SIDE_GATE: case TensorSlot::SIDE_PROJ:
        case TensorSlot::DELTA_BETA: case TensorSlot::DELTA_A1: case TensorSlot::DELTA_A2: case TensorSlot::DELTA_G1: case TensorSlot::DELTA_G2: return false;
        default: return true;
    }
}

const ModelFamily* find_model_family(const std::string& architecture) {
    for (const ModelFamily* f : model_families())
        if (architecture == f->architecture) return f;
    return nullptr;
}

bool read_model_dir(const std::string& dir, ModelConfig& cfg, const ModelFamily** family) {
    const std::string path = dir + "/config.json";
    std::ifstream in(path, std::ios::binary);
    if (!in) { fprintf(stderr, "model: cannot open %s\n", path.c_str()); return false; }
    std::stringstream ss;
    ss << in.rdbuf();
    Json root;
    std::string err;
    if (!Json::parse(ss.str(), root, &err) || !root.is_object()) { fprintf(stderr, "model: %s: %s\n", path.c_str(), err.c_str()); return false; }
    const std::string arch = root.at("architecture").string_or("");
    const ModelFamily* f = find_model_family(arch);
    if (!f) {
        fprintf(stderr, "model: %s: architecture \"%s\" is not registered (known:", path.c_str(), arch.c_str());
        for (const ModelFamily* k : model_families()) fprintf(stderr, " %s", k->architecture);
        fprintf(stderr, ")\n");
        return false;
    }
    cfg = ModelConfig();
    cfg.architecture = arch;
    if (!f->config_from_json(root, cfg, err)) { fprintf(stderr, "model: %s: %s\n", path.c_str(), err.c_str()); return false; }
    if (family) *family = f;
    return true;
}

}}  // namespace nt::b200
