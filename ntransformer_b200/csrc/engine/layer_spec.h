// layer_spec.h — what one decoder layer is made of, for model families described layer by layer (a folder with config.json +
// model.safetensors) instead of by the fixed Llama block of the GGUF families.  Every mechanism is a parameter here so that
// another family can combine them differently; a Llama block would read {ROPE_CAUSAL mixer, sequential block, SiLU GLU}.
#pragma once
#include <string>
#include <vector>

namespace nt { namespace b200 {

enum class MixerKind { ATTN_ROPE_CAUSAL = 0,     // rotary positions, full causal mask (the GGUF Llama block)
                       ATTN_WINDOW = 1,          // no positions in the scores; sliding window + kept first tokens; soft-capped scores
                       ATTN_LATENT = 2,          // queries and keys / values through low-rank latents; the cache holds the normed key / value latent
                                                 // and one rotated key part shared by all heads; scored in the latent space (LatentSpec)
                       SSM_SCAN = 3,             // selective state-space recurrence with a short causal convolution in front (ScanSpec); no cache rows,
                                                 // a fixed-size state per sequence instead
                       DELTA_RULE = 4,           // gated delta-rule recurrence (DeltaSpec): a matrix state per head that is decayed per key channel,
                                                 // corrected towards the new value along the new key and read with the query; no cache rows
                       BRANCHES = 5 };           // several mixers side by side reading the same input; their outputs are summed with fixed weights
                                                 // (LayerSpec::branches / branch_scale); each branch keeps its own cache rows or state
enum class QKNorm { NONE = 0, WHOLE = 1,         // WHOLE: one RMS norm across ALL heads of the projection (gain vector of that length)
                    PER_HEAD = 2 };              // every head is RMS-normed on its own with one gain vector of the head's width shared by all heads
enum class GluAct { SILU = 0, GELU_TANH = 1, RELU = 2 };
enum class BlockForm { SEQUENTIAL = 0,           // x += mixer(norm1 x) ; x += ff(norm2 x)
                       PARALLEL = 1,             // h = norm1 x ; x += m * (ls1 * mixer(h) + ls2 * ff(h))
                       STREAMS = 2,              // SEQUENTIAL over several residual streams: a sublayer reads a learned blend of the streams and
                                                 // its output enters every stream through a learned stream-mixing matrix (ModelConfig::streams)
                       POST_NORM = 3,            // x += norm1(mixer(x)) ; x += norm2(ff(x)): the sublayers read x itself, the norm sits on their output
                       SUM_NORM = 4 };           // x <- norm1(a x + mixer(x)) ; x <- norm2(a x + ff(x)): the norm sits on the residual sum itself, the
                                                 // skip path is multiplied by a = ModelConfig::skip_scale
enum class FfKind { GLU = 0,                     // W_down (act(W_gate h) * W_up h)
                    MOE_RELU2 = 1,               // routed experts W_down relu(W_up h)^2, top-k softmax over the chosen logits, optional gated shared expert
                    MOE_GLU = 2 };               // routed gated experts W_down (act(W_gate h) * W_up h); how they are chosen and weighted: RouteSpec


// Rotary positions of one attention layer.  dims == 0: none.  The first `dims` channels of a head rotate, the rest pass.
// factor > 0 selects the long-context blend: channel pairs whose wavelength is long against `original` positions are slowed by
// `factor`, short ones are left, with a linear ramp between the pair indices that turn `fast` and `slow` times over `original`;
// cos and sin are then multiplied by 0.1 * ln(factor) + 1.
struct RotarySpec {
    int dims = 0;
    float base = 10000.f;
    bool interleaved = true;     // pairs (2i, 2i+1); false: (i, i + dims/2)
    float factor = 0.f, original = 0.f, fast = 0.f, slow = 0.f;
    float divide = 1.f;          // linear position scaling: every angular frequency is divided by this
};

// Low-rank attention.  q = W_uq rms(W_dq h): per head [dim unrotated | rot_dim rotated].  W_dkv h = [kv_rank | rot_dim]: the first part,
// RMS-normed, is the latent c; the second, rotated, is a key part common to all heads.  Head h's keys are [W_uk,h c | that part],
// its values W_uv,h c.  The cache row of a position is [c | rotated part]: kv_rank + rot_dim numbers whatever the head count.
struct LatentSpec {
    int q_rank = 0, kv_rank = 0, rot_dim = 0;
};
// State-space scan.  W_in h = [z: inner | x: inner | B: groups*state | C: groups*state | dt: heads], inner = heads * vdim.  x, B, C pass a
// causal per-channel convolution of `conv` taps and SiLU.  Per head: S <- exp(-exp(A_log) dt) S + dt B x^T (state x vdim), y = S^T C + D x,
// dt = softplus(dt + dt_bias).  y * silu(z) is RMS-normed in `norm_groups` equal parts.  The state of a sequence is S plus the last
// conv - 1 convolution inputs.
struct ScanSpec {
    int state = 0, groups = 1, conv = 0, norm_groups = 1;
};
// How a mixture of experts chooses and weights.  sigmoid: scores are sigmoid(logit) (else softmax over the chosen logits);
// correction: a per-expert vector added to the scores for the CHOICE only; groups > 0: experts form `groups` equal runs of
// neighbours, a run scores the sum of its two largest choice scores and only the best `keep` runs can be chosen from.
struct RouteSpec {
    bool sigmoid = false, correction = false;
    int groups = 0, keep = 0;
};

// Gated delta rule.  q, k [kv_heads, dim] and v [heads, vdim] come from projections followed by a short causal convolution
// (LayerSpec::conv taps) and SiLU; q and k are scaled to unit length per head (q also by dim^-1/2).  Per value head h (reading q / k head
// h / (heads / kv_heads)) with state S [dim, vdim] in F32:  S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q, where
// beta = sigmoid(W_b x) per head and g = exp(-exp(A_log_h) softplus(W_a2 W_a1 x + dt_bias)) per head and key channel (decay_rank = rows of
// W_a1).  o is RMS-normed per head (gain shared by the heads) and multiplied by sigmoid(W_g2 W_g1 x) (gate_rank = rows of W_g1).
// The sequence's state is S plus the last taps - 1 inputs of the three convolutions.
struct DeltaSpec {
    int decay_rank = 0, gate_rank = 0;
};

struct LayerSpec {
    MixerKind mixer = MixerKind::ATTN_ROPE_CAUSAL;
    BlockForm form = BlockForm::SEQUENTIAL;
    int heads = 0, kv_heads = 0;
    int dim = 0;                 // per-head query/key width
    int vdim = 0;                // per-head value width
    float scale = 0.f;           // score multiplier
    float softcap = 0.f;         // score <- softcap * tanh(score / softcap); 0 = none
    int window = 0;              // key j visible from i iff j <= i and (i - j < window or j < keep_first); 0 = full causal
    int keep_first = 0;
    QKNorm qk_norm = QKNorm::NONE;
    int ff = 0;                  // feed-forward width; 0 = the layer has no feed-forward
    GluAct act = GluAct::SILU;
    bool layer_scale = false;    // per-channel gains on each branch before the residual sum
    int weights_of = -1;         // >= 0: this layer reads that layer's tensors (own KV cache)
    // ---- mechanisms added with the Vebotar family; every one is off at its default ----
    RotarySpec rot;              // rotary positions on q and k before the cache write
    int chunk = 0;               // > 0: key j visible from i iff j <= i and j / chunk == i / chunk (blocks counted from position 0)
    int maps = 1;                // 2: differential attention — two score maps per head ([map 1 | map 2] inside each q / k head) over one
                                 // set of values, out = A1 v - lambda * A2 v, then a weightless RMS norm per head times (1 - diff)
    float diff = 0.f;            // lambda = exp(<lq1, lk1>) - exp(<lq2, lk2>) + diff
    int kv_from = -1;            // >= 0: no key / value projections; reads that layer's cache rows (rotated keys, values)
    FfKind ff_kind = FfKind::GLU;
    int experts = 0, top = 0;    // MOE_RELU2: routed experts of width ff, experts used per token
    int shared_ff = 0;           // MOE_RELU2: width of the shared expert (0 = none); its output is scaled by sigmoid(<w_sg, h>)
    // ---- mechanisms added with the Tanolorn family ----
    LatentSpec latent;           // ATTN_LATENT (heads, dim, vdim, scale, rot and kv_from above apply too)
    ScanSpec scan;               // SSM_SCAN (heads and vdim above apply too)
    RouteSpec route;             // MOE_GLU
    bool ff_bias = false;        // GLU: every projection has a bias vector
    // ---- mechanisms added with the Savidra family; every one is off at its default ----
    bool token_shift = false;    // the mixer reads h_t = x_t + (x_{t-1} - x_t) * mu (per channel, x_{-1} = 0) instead of x_t; x_{t-1} is sequence state
    int conv = 0;                // > 0: q, k and v pass a causal per-channel convolution of this many taps right after their projection
                                 // (attention: no activation; DELTA_RULE: SiLU); the last conv - 1 projected rows are sequence state
    bool qkv_bias = false;       // attention: q, k, v and the output projection have bias vectors
    bool head_temp = false;      // attention: the scores of head h are multiplied by a learned number per head
    bool talking = false;        // attention: after the softmax the heads' weights are mixed, w_h <- sum_g M[h, g] w_g, before head h applies
                                 // them to the values of its own key / value head
    bool sink = false;           // attention: the softmax denominator also holds exp(sink_h), a learned number per head without key or value
    int v_first = -1;            // attention: >= 0 and != this layer: v <- (1 - lambda) v + lambda v', v' the values layer v_first computed for the
                                 // same token (lambda a learned number); == this layer: the layer only publishes its values
    DeltaSpec delta;             // DELTA_RULE (heads, kv_heads, dim, vdim and conv above apply too)
    std::vector<LayerSpec> branches;     // BRANCHES: the mixers (their form, ff and token_shift are unused)
    std::vector<float> branch_scale;     // BRANCHES: the weight of each branch's output in the sum
    int cache_slot = -1;         // set when the model is finalized: which entry of the model's per-mixer cache table holds this mixer's rows
};

}}  // namespace nt::b200
