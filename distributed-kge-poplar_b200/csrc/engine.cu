// Host engine implementation.  See engine.hpp.
#include "engine.hpp"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>

namespace kge {

// ---------------------------------------------------------------------------
// Settings (src/poplar_kge.cpp:39-67 for the error texts, :198-246 for the keys)

namespace {

const char* type_name(int type) {
    switch (type) {
        case KGE_SET_STRING: return "string";
        case KGE_SET_BOOL: return "bool";
        case KGE_SET_FLOAT: return "float";
        case KGE_SET_UNSIGNED: return "unsigned";
    }
    return "?";
}

const SettingValue& lookup(const SettingMap& s, const std::string& key, int type) {
    auto it = s.find(key);
    if (it == s.end()) fail(KGE_INVALID_ARGUMENT, msg() << "Key not found '" << key << "'");
    if (it->second.type != type) {
        fail(KGE_INVALID_ARGUMENT, msg() << "Key '" << key
                                         << "' holds value of unexpected type. Expected: '"
                                         << type_name(type) << "', actual: '"
                                         << type_name(it->second.type) << "'.");
    }
    return it->second;
}
std::string get_string(const SettingMap& s, const std::string& k) { return lookup(s, k, KGE_SET_STRING).s; }
unsigned get_unsigned(const SettingMap& s, const std::string& k) {
    return (unsigned)lookup(s, k, KGE_SET_UNSIGNED).u;
}
float get_float(const SettingMap& s, const std::string& k) { return (float)lookup(s, k, KGE_SET_FLOAT).f; }
bool get_bool(const SettingMap& s, const std::string& k) { return lookup(s, k, KGE_SET_BOOL).u != 0; }

template <class T, class Getter>
T get_or(const SettingMap& s, const std::string& k, Getter getter, T fallback) {
    return s.count(k) ? getter(s, k) : fallback;
}

int parse_storage(const std::string& key, const std::string& value) {
    if (value == "float32") return ST_F32;
    if (value == "float16") return ST_F16;
    fail(KGE_INVALID_ARGUMENT, msg() << "'" << key << "' must either be 'float16' or 'float32', not '"
                                     << value << "'");
}

// src/poplar_kge.cpp:144-152.  A power below 1 is no norm, and pow of a negative base needs an integer power.
void read_regulariser(const SettingMap& s, const std::string& prefix, float& power, float& weight) {
    power = get_float(s, prefix + ".power");
    weight = get_float(s, prefix + ".weight");
    if (weight < 0.f) fail(KGE_INVALID_ARGUMENT, msg() << "'" << prefix << ".weight' must not be negative");
    if (weight > 0.f && !(power >= 1.f))
        fail(KGE_INVALID_ARGUMENT, msg() << "'" << prefix << ".power' must be at least 1, actual: " << power);
}

}  // namespace

Config parse_config(const SettingMap& s) {
    Config c{};
    c.n_shard = get_unsigned(s, "model.n_shard");
    const std::string device = get_string(s, "execution.device");
    if (device != "cpu" && device != "ipu" && device != "ipu_model" && device != "cuda") {
        fail(KGE_INVALID_ARGUMENT, msg() << "Unexpected setting \"device\": '" << device
                                         << "', expected \"cuda\" (or the reference's \"cpu\" / \"ipu\")");
    }
    c.seed = get_unsigned(s, "model.seed");
    const std::string score_fn = get_string(s, "model.score_fn");
    const std::string distance_fn = get_string(s, "model.distance_fn");
    c.n_entity = get_unsigned(s, "model.n_entity");
    c.n_relation_type = get_unsigned(s, "model.n_relation_type");
    c.d = get_unsigned(s, "model.embedding_size");
    c.f = get_unsigned(s, "model.entity_feature_size");
    const unsigned mlp = get_unsigned(s, "model.feature_mlp_size");
    const float dropout = get_float(s, "model.feature_dropout");
    c.share_networks = get_bool(s, "model.share_feature_networks");
    c.gamma = get_float(s, "model.gamma");
    c.init_scale = get_float(s, "model.init_scale");
    c.beta_m = get_float(s, "training.adam_beta_m");
    c.beta_v = get_float(s, "training.adam_beta_v");
    c.epsilon = get_float(s, "training.adam_epsilon");
    c.weight_decay = get_float(s, "training.weight_decay");
    const std::string mod_prefix = "training.learning_rate_modifiers.";
    for (auto& kv : s) {
        if (kv.first.compare(0, mod_prefix.size(), mod_prefix) == 0) {
            c.lr_modifiers[kv.first.substr(mod_prefix.size())] = get_float(s, kv.first);
        }
    }
    c.batch_size = get_unsigned(s, "data.batch_size");
    c.a2a_size = get_unsigned(s, "data.a2a_size");
    c.adversarial_scale = get_float(s, "model.negative_adversarial_scale");
    const std::string loss = get_string(s, "training.loss.type");
    read_regulariser(s, "training.embedding_regularisation", c.reg_power[0], c.reg_weight[0]);
    read_regulariser(s, "training.feature_regularisation", c.reg_power[1], c.reg_weight[1]);
    read_regulariser(s, "training.hidden_regularisation", c.reg_power[2], c.reg_weight[2]);
    c.correction_weight = loss == "softmax" ? get_float(s, "training.loss.correction_weight") : 0.f;
    c.loss_scale = get_float(s, "training.loss_scale");
    c.n_step = get_unsigned(s, "execution.train_steps_per_program_run");
    c.rw_batch = get_unsigned(s, "execution.rw_batch_size");
    c.predict_hr = get_unsigned(s, "execution.predict_hr_batch_size");
    c.predict_tail_batch = get_unsigned(s, "execution.predict_tail_batch_size");
    c.predict_n_best = get_unsigned(s, "execution.predict_n_best");
    c.state_type = parse_storage("execution.dtype", get_string(s, "execution.dtype"));
    c.feature_type = s.count("execution.feature_dtype")
                         ? parse_storage("execution.feature_dtype", get_string(s, "execution.feature_dtype"))
                         : c.state_type;
    c.value_bf16 = false;
    if (s.count("execution.value_dtype")) {
        const std::string v = get_string(s, "execution.value_dtype");
        if (v == "bfloat16") c.value_bf16 = true;
        else if (v != "float32" && v != "float16")
            fail(KGE_INVALID_ARGUMENT, msg() << "'execution.value_dtype' must be 'bfloat16' or the row type, not '" << v << "'");
        if (c.value_bf16 && c.state_type != ST_F32)
            fail(KGE_INVALID_ARGUMENT, "'execution.value_dtype' 'bfloat16' needs 'execution.dtype' 'float32' (the optimiser state stays float32)");
    }
    c.device_ordinal = get_or<unsigned>(s, "execution.device_ordinal", get_unsigned, 0u);
    c.rank = get_or<unsigned>(s, "execution.rank", get_unsigned, 0u);
    c.world = get_or<unsigned>(s, "execution.world_size", get_unsigned, 1u);
    c.cuda_graph = get_or<bool>(s, "execution.cuda_graph", get_bool, true);
    c.tensor_cores = get_or<bool>(s, "execution.tensor_cores", get_bool, true);
    c.l2_contraction = get_or<bool>(s, "execution.l2_contraction", get_bool, false);

    if (score_fn == "TransE") c.score_fn = SCORE_TRANSE;
    else if (score_fn == "DistMult") c.score_fn = SCORE_DISTMULT;
    else if (score_fn == "ComplEx") c.score_fn = SCORE_COMPLEX;
    else if (score_fn == "RotatE") c.score_fn = SCORE_ROTATE;
    else if (score_fn == "TransH") c.score_fn = SCORE_TRANSH;
    else
        fail(KGE_INVALID_ARGUMENT, msg() << "'model.score_fn' must be one of 'TransE', 'ComplEx', 'RotatE', "
                                            "'TransH', or 'DistMult', not '" << score_fn << "'");
    if (distance_fn == "L1" || distance_fn == "L1_old") c.dist_fn = DIST_L1;
    else if (distance_fn == "L2" || distance_fn == "L2_old") c.dist_fn = DIST_L2;
    else if (distance_fn == "MatMul") c.dist_fn = DIST_DOT;
    else
        fail(KGE_INVALID_ARGUMENT, msg() << "'model.distance_fn' must be one of 'L1', 'L1_old', 'L2', 'L2_old' "
                                            "or 'MatMul', not '" << distance_fn << "'");
    // TransH's score is the L1 form whatever the setting says (src/poplar_kge.cpp:552-565)
    if (c.score_fn == SCORE_TRANSH) c.dist_fn = DIST_L1;
    if (loss == "logsigmoid") c.loss_fn = LOSS_LOGSIGMOID;
    else if (loss == "softmax") c.loss_fn = LOSS_SOFTMAX;
    else
        fail(KGE_INVALID_ARGUMENT, msg() << "'training.loss.type' must be one of 'logsigmoid' or 'softmax', not '"
                                         << loss << "'");
    c.mlp = mlp;
    if (!(dropout >= 0.f && dropout < 1.f)) fail(KGE_INVALID_ARGUMENT, msg() << "'model.feature_dropout' must be in [0, 1), actual: " << dropout);
    c.dropout = dropout;
    if (c.state_type == ST_F16 && c.feature_type != ST_F16)
        fail(KGE_INVALID_ARGUMENT, "'execution.feature_dtype' must be 'float16' when 'execution.dtype' is 'float16'");

    // Parameters are sliced by rows over the shards (src/poplar_kge.cpp:294-300).
    auto divisible = [&](const char* name, unsigned rows, unsigned cols) {
        if (rows % c.n_shard)
            fail(KGE_INVALID_ARGUMENT, msg() << "Parameter '" << name << "' shape[0] (" << rows
                                             << ") is not divisible by n_shard (" << c.n_shard
                                             << "). Note shape: (" << rows << ", " << cols << ")");
    };
    if (c.n_shard == 0 || c.world == 0 || c.n_shard % c.world || c.rank >= c.world)
        fail(KGE_INVALID_ARGUMENT, msg() << "n_shard (" << c.n_shard << ") must be a positive multiple of "
                                            "execution.world_size (" << c.world << ") and rank < world_size");
    divisible("relation_embedding", c.n_relation_type, c.d);
    if (c.f) divisible(c.share_networks ? "feature_projection" : "head_feature_projection", c.f, c.d);
    if (c.f && c.mlp) {  // src/poplar_kge.cpp:260-265
        divisible(c.share_networks ? "mlp_up_projection" : "head_mlp_up_projection", 2 * c.d, c.mlp);
        divisible(c.share_networks ? "mlp_down_projection" : "head_mlp_down_projection", c.mlp, c.d);
    }
    for (auto& kv : c.lr_modifiers) {
        const bool known = kv.first == "entity_embedding" || kv.first == "relation_embedding" ||
                           (c.score_fn == SCORE_TRANSH && kv.first == "relation_normal") ||
                           (c.mlp && c.f && c.share_networks && (kv.first == "mlp_up_projection" || kv.first == "mlp_down_projection")) ||
                           (c.mlp && c.f && !c.share_networks &&
                            (kv.first == "head_mlp_up_projection" || kv.first == "head_mlp_down_projection" ||
                             kv.first == "tail_mlp_up_projection" || kv.first == "tail_mlp_down_projection")) ||
                           (c.share_networks ? kv.first == "feature_projection"
                                             : (kv.first == "head_feature_projection" ||
                                                kv.first == "tail_feature_projection"));
        if (!known)
            fail(KGE_INVALID_ARGUMENT, msg() << "Bad training.learning_rate_modifier: unknown parameter '"
                                             << kv.first << "'");
    }
    if (c.d == 0 || c.batch_size == 0 || c.a2a_size == 0 || c.n_step == 0 || c.n_entity == 0)
        fail(KGE_INVALID_ARGUMENT, "embedding_size, batch_size, a2a_size, n_entity and "
                                   "train_steps_per_program_run must be positive");
    if ((c.score_fn == SCORE_COMPLEX || c.score_fn == SCORE_ROTATE) && (c.d & 1))
        fail(KGE_INVALID_ARGUMENT, "ComplEx and RotatE need an even 'model.embedding_size'");
    if (c.score_fn == SCORE_ROTATE && c.dist_fn == DIST_DOT)
        fail(KGE_INVALID_ARGUMENT, "RotatE scores by a distance: 'model.distance_fn' must be 'L1' or 'L2'");
    if (c.n_tail() < 2) fail(KGE_INVALID_ARGUMENT, "n_shard * a2a_size must be at least 2");
    if ((size_t)c.batch_size + c.n_tail() > (size_t)kMaxSortItems)
        fail(KGE_INVALID_ARGUMENT, msg() << "batch_size + n_shard * a2a_size (" << c.n_remote()
                                         << ") exceeds this engine's limit of " << kMaxSortItems);
    return c;
}

// ---------------------------------------------------------------------------
// Dispatch over the row storage types.

#define KGE_DISPATCH_ROW(cfg, ...)                                          \
    do {                                                                     \
        if ((cfg).state_type == ST_F32 && (cfg).feature_type == ST_F32) {    \
            using ST = float; using FT = float; __VA_ARGS__;                 \
        } else if ((cfg).state_type == ST_F32) {                             \
            using ST = float; using FT = __half; __VA_ARGS__;                \
        } else {                                                             \
            using ST = __half; using FT = __half; __VA_ARGS__;               \
        }                                                                    \
    } while (0)

namespace {
size_t type_bytes(int storage) { return storage == ST_F32 ? 4 : 2; }
unsigned ceil_div(unsigned a, unsigned b) { return (a + b - 1) / b; }
}  // namespace

// ---------------------------------------------------------------------------
// Construction

void* Engine::device_alloc(size_t bytes) {
    void* p = nullptr;
    KGE_CUDA(cudaMalloc(&p, std::max<size_t>(bytes, 16)));
    allocations_.push_back(p);
    return p;
}

size_t Engine::arena_offset_dense(int which) const {
    const size_t flags = round_up(sizeof(unsigned) * kFlagWords, 256);
    return flags + (size_t)which * round_up(n_dense_ * sizeof(float), 256);
}
size_t Engine::arena_offset_shard(unsigned local, int which) const {
    // per local shard: tails | grad_recv | lower plane of tails
    const size_t row_block = round_up((size_t)cfg_.n_tail() * cfg_.d * sizeof(float), 256);
    const size_t per_shard = 3 * row_block;
    const size_t base = arena_offset_dense(4) + (size_t)local * per_shard;
    return base + (size_t)which * row_block;
}
// Receive buffer of the partial dense gradients: one slot of `dense_chunk_` floats per shard of the job.
size_t Engine::arena_offset_dense_recv() const { return arena_offset_predict(3); }
size_t Engine::arena_offset_predict(int which) const {
    // gathered queries [n_shard, hr, D] | result scores | result rows, each [n_local, n_shard, hr, n_best]
    // (TransH: the predicted tails, then the unit normals, src/poplar_kge.cpp:823-828)
    const size_t queries = round_up((size_t)(cfg_.score_fn == SCORE_TRANSH ? 2 : 1) * cfg_.n_shard * cfg_.predict_hr * cfg_.d * sizeof(float), 256);
    const size_t results = round_up((size_t)n_local_ * cfg_.n_shard * cfg_.predict_hr * cfg_.predict_n_best * 4, 256);
    const size_t base = arena_offset_shard(n_local_, 0);
    return base + (which == 0 ? 0 : which == 1 ? queries : which == 2 ? queries + results : queries + 2 * results);
}
size_t Engine::arena_size() const {
    return arena_offset_dense_recv() + round_up((size_t)cfg_.n_shard * dense_chunk_ * sizeof(float), 256);
}

Engine::Engine(const SettingMap& settings) : cfg_(parse_config(settings)) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || (int)cfg_.device_ordinal >= count) {
        cudaGetLastError();
        fail(KGE_RUNTIME_ERROR, msg() << "Could not attach to CUDA device " << cfg_.device_ordinal << " ("
                                      << count << " visible)");
    }
    KGE_CUDA(cudaSetDevice((int)cfg_.device_ordinal));
    n_local_ = cfg_.n_shard / cfg_.world;
    shard0_ = cfg_.rank * n_local_;

    const size_t sb = type_bytes(cfg_.state_type), fb = type_bytes(cfg_.feature_type);
    const uint32_t seg = (uint32_t)round_up(cfg_.d * sb, 16), value_seg = cfg_.value_bf16 ? (uint32_t)round_up(cfg_.d * 2, 16) : seg;
    layout_.off_m = value_seg;
    layout_.off_q = value_seg + seg;
    layout_.off_feat = value_seg + 2 * seg;
    layout_.row_bytes = layout_.off_feat + (uint32_t)round_up(cfg_.f * fb, 16);
    layout_.value_bf16 = cfg_.value_bf16 ? 1u : 0u;
    layout_.d = cfg_.d;
    layout_.f = cfg_.f;

    adam_.beta_m = cfg_.beta_m;
    adam_.beta_v = cfg_.beta_v;
    adam_.one_minus_beta_m = 1.0f - cfg_.beta_m;
    adam_.one_minus_beta_v = 1.0f - cfg_.beta_v;
    adam_.epsilon = cfg_.epsilon;
    adam_.weight_decay = cfg_.weight_decay;

    // dense vector: relation table | projection(s)
    proj_elems_ = (size_t)cfg_.f * cfg_.d;
    dense_bounds_[0] = 0;
    dense_bounds_[1] = (size_t)cfg_.n_relation_type * cfg_.d;
    dense_bounds_[2] = dense_bounds_[1] + (cfg_.n_net() >= 1 ? proj_elems_ : 0);
    dense_bounds_[3] = dense_bounds_[2] + (cfg_.n_net() >= 2 ? proj_elems_ : 0);
    dense_bounds_[4] = dense_bounds_[3] + (cfg_.score_fn == SCORE_TRANSH ? (size_t)cfg_.n_relation_type * cfg_.d : 0);
    for (unsigned net = 0; net < 2; ++net) {  // the feature MLP's projections: up [2D, M], down [M, D]
        const bool present = cfg_.mlp > 0 && net < cfg_.n_net();
        dense_bounds_[5 + 2 * net] = dense_bounds_[4 + 2 * net] + (present ? (size_t)2 * cfg_.d * cfg_.mlp : 0);
        dense_bounds_[6 + 2 * net] = dense_bounds_[5 + 2 * net] + (present ? (size_t)cfg_.mlp * cfg_.d : 0);
    }
    n_dense_ = dense_bounds_[kDenseParams];
    auto modifier = [&](const std::string& name) {
        auto it = cfg_.lr_modifiers.find(name);
        return it == cfg_.lr_modifiers.end() ? 1.0f : it->second;
    };
    entity_lr_mod_ = modifier("entity_embedding");
    dense_lr_mod_[0] = modifier("relation_embedding");
    std::vector<std::string> proj_names;
    if (cfg_.n_net() == 1) proj_names = {"feature_projection"};
    if (cfg_.n_net() == 2) proj_names = {"head_feature_projection", "tail_feature_projection"};
    // With no features the reference still declares an empty projection; it is listed with
    // shape [0, D] and carries no data.
    if (cfg_.n_net() == 0)
        proj_names = cfg_.share_networks
                         ? std::vector<std::string>{"feature_projection"}
                         : std::vector<std::string>{"head_feature_projection", "tail_feature_projection"};
    for (size_t i = 0; i < proj_names.size() && i < 2; ++i) dense_lr_mod_[1 + i] = modifier(proj_names[i]);

    auto add_variable = [&](const std::string& name, size_t rows, size_t cols, size_t offset, bool flat = false) {
        const char* suffix[3] = {"", "/adam_m", "/adam_v"};
        for (int k = 0; k < 3; ++k)
            variables_.push_back({name + suffix[k], KGE_F32, {rows, cols}, offset, k, flat});
    };
    // RotatE's relations are angles, one per complex pair (src/poplar_kge.cpp:248-251); the table keeps
    // rows of d floats all the same and uses their first half
    add_variable("relation_embedding", cfg_.n_relation_type, cfg_.score_fn == SCORE_ROTATE ? cfg_.d / 2 : cfg_.d, 0);
    for (size_t i = 0; i < proj_names.size(); ++i)
        add_variable(proj_names[i], cfg_.f, cfg_.d, cfg_.f ? dense_bounds_[1 + i] : n_dense_);
    if (cfg_.score_fn == SCORE_TRANSH) {  // src/poplar_kge.cpp:252-255
        add_variable("relation_normal", cfg_.n_relation_type, cfg_.d, dense_bounds_[3]);
        dense_lr_mod_[3] = modifier("relation_normal");
    }
    if (cfg_.mlp > 0 && cfg_.n_net() > 0)
        for (unsigned net = 0; net < cfg_.n_net(); ++net) {
            const std::string prefix = proj_names[net].substr(0, proj_names[net].size() - std::string("feature_projection").size());
            add_variable(prefix + "mlp_up_projection", 2 * cfg_.d, cfg_.mlp, dense_bounds_[4 + 2 * net], true);
            add_variable(prefix + "mlp_down_projection", cfg_.mlp, cfg_.d, dense_bounds_[5 + 2 * net]);
            dense_lr_mod_[4 + 2 * net] = modifier(prefix + "mlp_up_projection");
            dense_lr_mod_[5 + 2 * net] = modifier(prefix + "mlp_down_projection");
        }
    variables_.push_back({"step", KGE_U32, {cfg_.n_shard}, 0, 3, false});

    // Every process owns (reduces and updates) an equal share of the rows of the dense vector, dealt
    // out in turn: row r belongs to process r % world, as its row r / world.
    const size_t dense_rows = cfg_.n_relation_type + (size_t)cfg_.n_net() * cfg_.f + (cfg_.score_fn == SCORE_TRANSH ? cfg_.n_relation_type : 0) +
                              (cfg_.mlp > 0 ? (size_t)cfg_.n_net() * 3 * cfg_.mlp : 0);
    dense_chunk_rows_ = std::max<size_t>(1, (dense_rows + cfg_.world - 1) / cfg_.world);
    dense_chunk_ = dense_chunk_rows_ * cfg_.d;
    own_rows_ = dense_rows > cfg_.rank ? (dense_rows - cfg_.rank + cfg_.world - 1) / cfg_.world : 0;

    const unsigned tiles = ceil_div(cfg_.f, 64) * ceil_div(cfg_.d, 64) * std::max(1u, cfg_.n_net());
    proj_splits_ = (int)std::min(8u, std::max(1u, ceil_div(148, std::max(1u, tiles))));
    proj_rows_per_split_ = (int)round_up(ceil_div(cfg_.n_remote(), proj_splits_), 32);

    KGE_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
    KGE_CUDA(cudaStreamCreateWithFlags(&side_stream_, cudaStreamNonBlocking));
    if (const char* v = std::getenv("KGE_SPLIT_POPULAR_ROWS")) split_popular_rows_ = std::atoi(v) != 0;
    // Worth its launch only where other processes wait for the shard that holds the popular entity:
    // measured 85.0 against 82.9 us per step on one GPU, where nobody waits.
    heavy_route_ = cfg_.world >= 4;
    if (const char* v = std::getenv("KGE_ROUTE_POPULAR_ROWS")) heavy_route_ = std::atoi(v) != 0;
    if (const char* v = std::getenv("KGE_FUSE_DENSE_UPDATE")) fuse_dense_env_ = std::atoi(v) != 0;
    if (const char* v = std::getenv("KGE_PREDICT_FILTER_IN_SCORES")) filter_in_scores_ = std::atoi(v) != 0;
    // Which work runs beside the step's chain: bit 0 the relation gradients, bit 1 the next step's gather.
    side_streams_ = 3u;
    if (const char* v = std::getenv("KGE_SIDE_STREAMS")) side_streams_ = (unsigned)std::atoi(v) & 3u;
    KGE_CUDA(cudaEventCreateWithFlags(&ev_fork_, cudaEventDisableTiming));
    for (cudaEvent_t& e : ev_join_) KGE_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    KGE_CUDA(cudaEventCreate(&ev_begin_));
    KGE_CUDA(cudaEventCreate(&ev_end_));
    for (cudaEvent_t& e : ev_stage_) KGE_CUDA(cudaEventCreate(&e));
    // The plane-fed contraction needs 16-byte rows in every operand and the lookups of a block of
    // hidden rows to fit its staging area.
    planes_ = cfg_.tensor_cores && cfg_.d % 4 == 0 && cfg_.batch_size % 4 == 0 && cfg_.n_tail() % 4 == 0 &&
              cfg_.n_remote() <= (unsigned)tc::kRouteMaxLookups;
    if (const char* v = std::getenv("KGE_PLANE_CONTRACTIONS")) planes_ = planes_ && std::atoi(v) != 0;
    if (mlp_on()) planes_ = false;  // the MLP sits between the projection and the lookups: the step of separate kernels
    if (cfg_.score_fn == SCORE_TRANSH) {
        planes_ = false;  // its score has no contraction form: the step of separate kernels
        if (transh_score_smem() > 200 * 1024) fail(KGE_INVALID_ARGUMENT, "TransH: model.embedding_size is limited to 1600");
        KGE_CUDA(cudaFuncSetAttribute(k_transh_score, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)transh_score_smem()));
    }
    // With one shard in all a dense gradient has a single contributor: the projection gradient's contraction and the
    // relation rows' blocks of the entity update apply the Adam step themselves and k_dense_update is not launched.
    fuse_dense_ = fuse_dense_env_ && planes_ && cfg_.n_shard == 1 && cfg_.world == 1;
    // fp16 features are widened into rows of their own; the lower plane of fp32 features keeps the
    // stride of the rows whose feature part is its upper plane (one stride per operand)
    bf16_planes_ = planes_ && cfg_.value_bf16 && cfg_.dist_fn == DIST_DOT && cfg_.d % 8 == 0 && cfg_.n_tail() % 8 == 0 && cfg_.batch_size % 8 == 0 &&
                   (cfg_.a2a_size * cfg_.d) % 2 == 0;
    feat_stride_ = cfg_.feature_type == ST_F16 ? (uint32_t)round_up(cfg_.f, 4) : layout_.row_bytes / 4;
    allocate();
    peer_arena_.assign(cfg_.world, nullptr);
    peer_arena_[cfg_.rank] = arena_;
    if (cfg_.world == 1) {
        build_pointer_tables();
        connected_ = true;
    }
}

Engine::~Engine() {
    cudaSetDevice((int)cfg_.device_ordinal);
    if (stream_) cudaStreamSynchronize(stream_);
    if (graph_exec_) cudaGraphExecDestroy(graph_exec_);
    for (cudaEvent_t e : event_pool_) cudaEventDestroy(e);
    for (unsigned p = 0; p < peer_arena_.size(); ++p)
        if (p != cfg_.rank && peer_arena_[p]) cudaIpcCloseMemHandle(peer_arena_[p]);
    for (void* p : allocations_) cudaFree(p);
    if (pinned_) cudaFreeHost(pinned_);
    if (ev_begin_) cudaEventDestroy(ev_begin_);
    if (ev_end_) cudaEventDestroy(ev_end_);
    for (cudaEvent_t e : ev_stage_) if (e) cudaEventDestroy(e);
    if (ev_fork_) cudaEventDestroy(ev_fork_);
    for (cudaEvent_t e : ev_join_) if (e) cudaEventDestroy(e);
    if (side_stream_) cudaStreamDestroy(side_stream_);
    if (stream_) cudaStreamDestroy(stream_);
}

void Engine::allocate() {
    const unsigned B = cfg_.batch_size, T = cfg_.n_tail(), R = cfg_.n_remote(), D = cfg_.d;
    const bool two_nets = cfg_.n_net() == 2;
    const bool multiplicative = cfg_.score_fn != SCORE_TRANSE;

    arena_ = (uint8_t*)device_alloc(arena_size());
    KGE_CUDA(cudaMemset(arena_, 0, arena_size()));
    dense_ = (float*)(arena_ + arena_offset_dense(0));
    dense_m_ = (float*)(arena_ + arena_offset_dense(1));
    dense_v_ = (float*)(arena_ + arena_offset_dense(2));
    dense_lo_ = (float*)(arena_ + arena_offset_dense(3));

    shards_.resize(n_local_);
    const size_t table_bytes = (size_t)cfg_.n_entity * layout_.row_bytes;
    for (unsigned l = 0; l < n_local_; ++l) {
        ShardBuffers& b = shards_[l];
        b.table = (uint8_t*)device_alloc(table_bytes);
        KGE_CUDA(cudaMemset(b.table, 0, table_bytes));
        for (uint8_t*& rows : b.rows_c2) rows = (uint8_t*)device_alloc((size_t)R * layout_.row_bytes);
        b.hid_h = (float*)device_alloc((size_t)R * D * 4);
        b.hid_t = two_nets || dropout_on() ? (float*)device_alloc((size_t)R * D * 4) : b.hid_h;  // dropout: each call has its own mask
        b.pred = (float*)device_alloc((size_t)B * D * 4);
        b.raw = (float*)device_alloc((size_t)B * T * 4);
        b.coeff = (float*)device_alloc((size_t)B * T * 4);
        b.d_pred = (float*)device_alloc((size_t)B * D * 4);
        b.d_head = multiplicative ? (float*)device_alloc((size_t)B * D * 4) : b.d_pred;
        b.d_relrow = multiplicative ? (float*)device_alloc((size_t)B * D * 4) : b.d_pred;
        if (mlp_on()) {
            const size_t M = cfg_.mlp;
            for (unsigned net = 0; net < cfg_.n_net(); ++net) {
                b.mlp_cat[net] = (float*)device_alloc((size_t)R * 2 * D * 4);
                b.mlp_pre[net] = (float*)device_alloc((size_t)R * M * 4);
            }
            b.mlp_out = (float*)device_alloc((size_t)R * D * 4);
            b.mlp_d_pre = (float*)device_alloc((size_t)R * M * 4);
            b.mlp_d_cat = (float*)device_alloc((size_t)R * 2 * D * 4);
            b.d_val = (float*)device_alloc((size_t)R * D * 4);
            b.mlp_dw_up = (float*)device_alloc((size_t)2 * D * M * 4);
            b.mlp_dw_down = (float*)device_alloc((size_t)M * D * 4);
        }
        if (cfg_.score_fn == SCORE_TRANSH) {
            b.nrm = (float*)device_alloc((size_t)B * D * 4);
            b.d_nrm = (float*)device_alloc((size_t)B * D * 4);
            b.d_normrow = (float*)device_alloc((size_t)B * D * 4);
            b.pair_s = (float*)device_alloc((size_t)B * T * 4);
            b.pair_u = (float*)device_alloc((size_t)B * T * 4);
        }
        if (cfg_.regularised()) {
            b.reg_val = (float*)device_alloc((size_t)R * D * 4);
            b.reg_h = (float*)device_alloc((size_t)R * D * 4);
            b.reg_t = two_nets || dropout_on() ? (float*)device_alloc((size_t)R * D * 4) : nullptr;
            b.reg_loss_rows = (float*)device_alloc((size_t)R * 4);
        }
        b.d_hid_h = (float*)device_alloc((size_t)R * D * 4);
        b.d_hid_t = two_nets ? (float*)device_alloc((size_t)R * D * 4) : nullptr;
        b.proj_partial = (float*)device_alloc(std::max<size_t>(1, cfg_.n_net()) * proj_splits_ * proj_elems_ * 4);
        b.loss_rows = (float*)device_alloc((size_t)B * 4);
        b.tails = (float*)(arena_ + arena_offset_shard(l, 0));
        b.grad_recv = (float*)(arena_ + arena_offset_shard(l, 1));
        b.dense_partial = (float*)(arena_ + arena_offset_dense_recv()) + (size_t)(shard0_ + l) * dense_chunk_;
        b.dense_dst = (float**)device_alloc(sizeof(float*) * cfg_.world);
        b.heavy_partial = (float*)device_alloc((size_t)kHeavySlots * 2 * D * 4);
        b.heavy_counter = (unsigned*)device_alloc(kHeavySlots * sizeof(unsigned));
        KGE_CUDA(cudaMemset(b.heavy_counter, 0, kHeavySlots * sizeof(unsigned)));
        b.send_dst = (float**)device_alloc(sizeof(float*) * cfg_.n_shard);
        b.grad_dst = (float**)device_alloc(sizeof(float*) * cfg_.n_shard);
        b.send_lo_dst = (float**)device_alloc(sizeof(float*) * cfg_.n_shard);
        b.tails_lo = (float*)(arena_ + arena_offset_shard(l, 2));
        if (planes_) {
            for (int par = 0; par < 2; ++par) {
                if (cfg_.feature_type == ST_F16) b.feat_wide2[par] = (float*)device_alloc((size_t)R * feat_stride_ * 4);
                else b.feat_lo2[par] = (float*)device_alloc((size_t)R * feat_stride_ * 4);
            }
            b.pred_lo = (float*)device_alloc((size_t)B * D * 4);
            b.coeff_lo = (float*)device_alloc((size_t)B * T * 4);
            b.d_hid_h_lo = (float*)device_alloc((size_t)R * D * 4);
            b.d_hid_t_lo = two_nets ? (float*)device_alloc((size_t)R * D * 4) : nullptr;
        }
        b.predict_score_dst = (float**)device_alloc(sizeof(float*) * cfg_.n_shard);
        b.predict_index_dst = (uint32_t**)device_alloc(sizeof(uint32_t*) * cfg_.n_shard);
    }
    d_epoch_ = (unsigned*)device_alloc(sizeof(unsigned));
    d_xchg_words_ = (unsigned*)device_alloc(2 * XCHG_KINDS * sizeof(unsigned));
    KGE_CUDA(cudaMemset(d_xchg_words_, 0, 2 * XCHG_KINDS * sizeof(unsigned)));
    if (const char* on = std::getenv("KGE_EXCHANGE_TRACE"); on && on[0] && on[0] != '0') {
        const size_t bytes = (size_t)kTraceSlots * XCHG_KINDS * 3 * sizeof(unsigned long long);
        d_xchg_trace_ = (unsigned long long*)device_alloc(bytes);
        KGE_CUDA(cudaMemset(d_xchg_trace_, 0, bytes));
    }
    d_tc_status_ = (unsigned*)device_alloc(2 * sizeof(unsigned));  // read back together after every run
    d_status_ = d_tc_status_ + 1;
    KGE_CUDA(cudaMemset(d_epoch_, 0, sizeof(unsigned)));
    KGE_CUDA(cudaMemset(d_tc_status_, 0, 2 * sizeof(unsigned)));
    {
        // room for the two problems of the largest paired launch, kTcMaxSplits partial tiles each
        const size_t per_problem = std::max<size_t>({(size_t)R * D, (size_t)(std::max(B, T)) * D, (size_t)cfg_.f * D, (size_t)B * T});
        tc_ws_floats_ = per_problem * kTcMaxSplits;
        tc_ws_ = (float*)device_alloc(2 * tc_ws_floats_ * 4);
        tc_ws_rowsum_ = (float*)device_alloc(2 * (size_t)kTcMaxSplits * std::max(B, T) * 4);
    }
    d_peer_flags_ = (unsigned**)device_alloc(sizeof(unsigned*) * cfg_.world);
    d_partials_ = (const float**)device_alloc(sizeof(float*) * cfg_.n_shard);
    d_replicas_ = (float**)device_alloc(sizeof(float*) * cfg_.world);
    d_replicas_lo_ = (float**)device_alloc(sizeof(float*) * cfg_.world);

    const size_t steps = (size_t)n_local_ * cfg_.n_step;
    d_remote_ = (uint32_t*)device_alloc(steps * R * 4);
    d_a2a_ = (uint32_t*)device_alloc(steps * T * 4);
    d_head_ = (uint32_t*)device_alloc(steps * B * 4);
    d_relation_ = (uint32_t*)device_alloc(steps * B * 4);
    d_tail_ = (uint32_t*)device_alloc(steps * B * 4);
    d_ent_perm_ = (uint32_t*)device_alloc(steps * (B + T) * 4);
    d_ent_off_ = (uint32_t*)device_alloc(steps * (R + 1) * 4);
    d_rel_perm_ = (uint32_t*)device_alloc(steps * B * 4);
    d_rel_off_ = (uint32_t*)device_alloc(steps * (cfg_.n_relation_type + 1) * 4);
    d_first_slot_ = (uint32_t*)device_alloc(steps * R * 4);
    d_heavy_parts_ = (uint4*)device_alloc(steps * kHeavySlots * sizeof(uint4));
    d_row_info_ = (uint4*)device_alloc(steps * 2 * R * sizeof(uint4));
    d_heavy_count_ = (uint32_t*)device_alloc(steps * 4);
    KGE_CUDA(cudaMemset(d_heavy_count_, 0, steps * 4));
    d_step_size_ = (float*)device_alloc(cfg_.n_step * 4);
    d_step_key_ = (uint32_t*)device_alloc(cfg_.n_step * 4);
    d_loss_total_ = (float*)device_alloc(n_local_ * 4);
    d_loss_last_ = (float*)device_alloc(n_local_ * 4);
    d_loss_counter_ = (unsigned*)device_alloc(n_local_ * sizeof(unsigned));
    KGE_CUDA(cudaMemset(d_loss_counter_, 0, n_local_ * sizeof(unsigned)));
    if (cfg_.regularised()) {
        d_reg_loss_ = (float*)device_alloc(n_local_ * 2 * sizeof(float));
        KGE_CUDA(cudaMemset(d_reg_loss_, 0, n_local_ * 2 * sizeof(float)));
        d_reg_counter_ = (unsigned*)device_alloc(n_local_ * sizeof(unsigned));
        KGE_CUDA(cudaMemset(d_reg_counter_, 0, n_local_ * sizeof(unsigned)));
    }

    const size_t rw = (size_t)n_local_ * cfg_.rw_batch;
    d_rw_idx_ = (uint32_t*)device_alloc(std::max<size_t>(rw, (size_t)n_local_ * cfg_.predict_hr * 2) * 4);
    d_rw_data_ = (uint8_t*)device_alloc(rw * cfg_.row_width() * 4);

    pinned_bytes_ = steps * ((size_t)R + T + 3 * B) * 4 + 2 * cfg_.n_step * 4 + 256;  // index streams | step keys | step sizes | loss
    KGE_CUDA(cudaMallocHost((void**)&pinned_, pinned_bytes_));
    KGE_CUDA(cudaDeviceSynchronize());
}

void Engine::build_pointer_tables() {
    const size_t block = (size_t)cfg_.a2a_size * cfg_.d;  // floats per (src, dst) block
    std::vector<float*> send(cfg_.n_shard), grad(cfg_.n_shard), send_lo(cfg_.n_shard);
    std::vector<const float*> partials(cfg_.n_shard);
    for (unsigned l = 0; l < n_local_; ++l) {
        const unsigned me = shard0_ + l;
        for (unsigned d = 0; d < cfg_.n_shard; ++d) {
            const unsigned owner = d / n_local_, dl = d % n_local_;
            uint8_t* base = peer_arena_[owner];
            send[d] = (float*)(base + arena_offset_shard(dl, 0)) + (size_t)me * block;
            grad[d] = (float*)(base + arena_offset_shard(dl, 1)) + (size_t)me * block;
            // the companion plane holds rows of D bf16 values (half a float each) in the bf16 tier
            send_lo[d] = (float*)(base + arena_offset_shard(dl, 2)) + (size_t)me * block / (bf16_planes_ ? 2 : 1);
        }
        KGE_CUDA(cudaMemcpy(shards_[l].send_lo_dst, send_lo.data(), sizeof(float*) * cfg_.n_shard, cudaMemcpyHostToDevice));
        KGE_CUDA(cudaMemcpy(shards_[l].send_dst, send.data(), sizeof(float*) * cfg_.n_shard, cudaMemcpyHostToDevice));
        KGE_CUDA(cudaMemcpy(shards_[l].grad_dst, grad.data(), sizeof(float*) * cfg_.n_shard, cudaMemcpyHostToDevice));
        // predict: results of tail shard `me` for the queries of shard d land in d's [d_local][me] block
        std::vector<float*> pscore(cfg_.n_shard);
        std::vector<uint32_t*> pindex(cfg_.n_shard);
        const size_t result_block = (size_t)cfg_.predict_hr * cfg_.predict_n_best;
        for (unsigned d = 0; d < cfg_.n_shard; ++d) {
            uint8_t* base = peer_arena_[d / n_local_];
            const size_t slot = ((size_t)(d % n_local_) * cfg_.n_shard + me) * result_block;
            pscore[d] = (float*)(base + arena_offset_predict(1)) + slot;
            pindex[d] = (uint32_t*)(base + arena_offset_predict(2)) + slot;
        }
        KGE_CUDA(cudaMemcpy(shards_[l].predict_score_dst, pscore.data(), sizeof(float*) * cfg_.n_shard, cudaMemcpyHostToDevice));
        KGE_CUDA(cudaMemcpy(shards_[l].predict_index_dst, pindex.data(), sizeof(uint32_t*) * cfg_.n_shard, cudaMemcpyHostToDevice));
    }
    for (unsigned l = 0; l < n_local_; ++l) {
        // where shard shard0_ + l writes its partial dense gradient: its slot in every owner's receive buffer
        std::vector<float*> dst(cfg_.world);
        for (unsigned p = 0; p < cfg_.world; ++p)
            dst[p] = (float*)(peer_arena_[p] + arena_offset_dense_recv()) + (size_t)(shard0_ + l) * dense_chunk_;
        KGE_CUDA(cudaMemcpy(shards_[l].dense_dst, dst.data(), sizeof(float*) * cfg_.world, cudaMemcpyHostToDevice));
    }
    for (unsigned d = 0; d < cfg_.n_shard; ++d)
        partials[d] = (const float*)(arena_ + arena_offset_dense_recv()) + (size_t)d * dense_chunk_;
    KGE_CUDA(cudaMemcpy(d_partials_, partials.data(), sizeof(float*) * cfg_.n_shard, cudaMemcpyHostToDevice));
    std::vector<float*> replicas(cfg_.world), replicas_lo(cfg_.world);
    std::vector<unsigned*> flags(cfg_.world);
    for (unsigned p = 0; p < cfg_.world; ++p) {
        replicas[p] = (float*)(peer_arena_[p] + arena_offset_dense(0));
        replicas_lo[p] = (float*)(peer_arena_[p] + arena_offset_dense(3));
        flags[p] = (unsigned*)(peer_arena_[p] + arena_offset_flags());
    }
    KGE_CUDA(cudaMemcpy(d_replicas_, replicas.data(), sizeof(float*) * cfg_.world, cudaMemcpyHostToDevice));
    KGE_CUDA(cudaMemcpy(d_replicas_lo_, replicas_lo.data(), sizeof(float*) * cfg_.world, cudaMemcpyHostToDevice));
    KGE_CUDA(cudaMemcpy(d_peer_flags_, flags.data(), sizeof(unsigned*) * cfg_.world, cudaMemcpyHostToDevice));
}

// ---------------------------------------------------------------------------
// Multi-process set-up

namespace {
struct CommHandle {
    cudaIpcMemHandle_t mem;
    uint32_t rank, world;
    uint64_t arena_bytes;
};
}  // namespace

size_t Engine::comm_handle_bytes() { return sizeof(CommHandle); }

void Engine::comm_export(void* out) const {
    CommHandle h{};
    KGE_CUDA(cudaSetDevice((int)cfg_.device_ordinal));
    KGE_CUDA(cudaIpcGetMemHandle(&h.mem, arena_));
    h.rank = cfg_.rank;
    h.world = cfg_.world;
    h.arena_bytes = arena_size();
    std::memcpy(out, &h, sizeof(h));
}

void Engine::comm_connect(const void* handles, size_t world) {
    if (world != cfg_.world)
        fail(KGE_INVALID_ARGUMENT, msg() << "kge_comm_connect: got " << world << " handles, world_size is " << cfg_.world);
    if (connected_) fail(KGE_LOGIC_ERROR, "kge_comm_connect: already connected");
    KGE_CUDA(cudaSetDevice((int)cfg_.device_ordinal));
    const CommHandle* all = static_cast<const CommHandle*>(handles);
    for (unsigned p = 0; p < cfg_.world; ++p) {
        CommHandle h;
        std::memcpy(&h, all + p, sizeof(h));
        if (h.rank != p || h.world != cfg_.world || h.arena_bytes != arena_size())
            fail(KGE_INVALID_ARGUMENT, msg() << "kge_comm_connect: handle " << p << " does not match this engine's settings");
        if (p == cfg_.rank) continue;
        void* ptr = nullptr;
        cudaError_t err = cudaIpcOpenMemHandle(&ptr, h.mem, cudaIpcMemLazyEnablePeerAccess);
        if (err != cudaSuccess) {
            cudaGetLastError();
            fail(KGE_RUNTIME_ERROR, msg() << "Could not attach to the device memory of rank " << p << ": "
                                          << cudaGetErrorString(err));
        }
        peer_arena_[p] = (uint8_t*)ptr;
    }
    build_pointer_tables();
    connected_ = true;
}

// ---------------------------------------------------------------------------
// Host array checks (src/poplar_kge.cpp:69-106)

namespace {
const char* dtype_name(int dtype) {
    return dtype == KGE_F32 ? "float" : dtype == KGE_U32 ? "unsigned int" : "half";
}
std::string shape_string(const std::vector<size_t>& shape) {
    msg m;
    m << "(";
    for (size_t i = 0; i < shape.size(); ++i) m << (i ? ", " : "") << shape[i];
    m << ")";
    return m;
}
}  // namespace

HostArray& Engine::find_array(std::vector<HostArray>& arrays, const std::string& name, int dtype,
                              const std::vector<size_t>& shape) {
    for (HostArray& a : arrays) {
        if (a.name != name) continue;
        if (a.dtype != dtype)
            fail(KGE_INVALID_ARGUMENT, msg() << "'" << name << "' expected array of type " << dtype_name(dtype)
                                             << ", actual: " << dtype_name(a.dtype));
        if (a.shape != shape)
            fail(KGE_INVALID_ARGUMENT, msg() << "'" << name << "' expected array of shape " << shape_string(shape)
                                             << ", actual: " << shape_string(a.shape));
        if (!a.data && a.count()) fail(KGE_INVALID_ARGUMENT, msg() << "'" << name << "' has a null data pointer");
        return a;
    }
    fail(KGE_INVALID_ARGUMENT, msg() << "Key not found '" << name << "'");
}

// ---------------------------------------------------------------------------
// Commands

void Engine::run(const std::string& command, std::vector<HostArray>& arrays, const std::string& variable) {
    KGE_CUDA(cudaSetDevice((int)cfg_.device_ordinal));
    if (command == "train_step_loop") return cmd_train_step_loop(arrays);
    if (command == "predict") return cmd_predict(arrays);
    if (command == "read_entity") return cmd_read_entity(arrays);
    if (command == "write_entity") return cmd_write_entity(arrays, false);
    if (command == "write_entity_rows") return cmd_write_entity(arrays, true);
    if (command == "initialise_entities") return cmd_initialise_entities();
    if (command == "entity_layout") {
        // `layout` u32 [4]: bytes of a stored row, rows per shard, local shards, the first local shard
        HostArray& out = find_array(arrays, "layout", KGE_U32, {4});
        uint32_t* o = static_cast<uint32_t*>(out.data);
        o[0] = layout_.row_bytes, o[1] = (uint32_t)cfg_.n_entity, o[2] = (uint32_t)n_local_, o[3] = (uint32_t)(cfg_.rank * n_local_);
        return;
    }
    if (command == "dump_entity_rows") return cmd_copy_entity_range(arrays, true);
    if (command == "restore_entity_rows") return cmd_copy_entity_range(arrays, false);
    if (command == "load_triples") return cmd_load_triples(arrays);
    if (command == "sample_batch") return cmd_sample_batch(arrays, false);
    if (command == "train_step_loop_sampled") return cmd_sample_batch(arrays, true);
    if (command == "read" || command == "write") return cmd_read_write_variable(arrays, variable, command == "write");
    fail(KGE_INVALID_ARGUMENT, msg() << "Unknown command '" << command << "'");
}

void Engine::cmd_train_step_loop(std::vector<HostArray>& arrays) {
    HostArray& lr = find_array(arrays, "learning_rate", KGE_F32, {n_local_});
    HostArray& loss = find_array(arrays, "loss", KGE_F32, {n_local_});
    stage_batch(arrays);
    train_staged(static_cast<const float*>(lr.data)[0], static_cast<float*>(loss.data));
}

void Engine::stage_batch(std::vector<HostArray>& arrays) {
    KGE_CUDA(cudaSetDevice((int)cfg_.device_ordinal));
    const size_t n = n_local_, S = cfg_.n_step, B = cfg_.batch_size, T = cfg_.n_tail(), R = cfg_.n_remote();
    HostArray& remote = find_array(arrays, "remote", KGE_U32, {n, S, R});
    HostArray& a2a = find_array(arrays, "a2a", KGE_U32, {n, S, cfg_.n_shard, cfg_.a2a_size});
    HostArray& head = find_array(arrays, "head", KGE_U32, {n, S, B});
    HostArray& relation = find_array(arrays, "relation", KGE_U32, {n, S, B});
    HostArray& tail = find_array(arrays, "tail", KGE_U32, {n, S, B});
    // The reference would read out of bounds on a bad index; here it is refused on the host.
    auto check_below = [](const HostArray& a, uint32_t limit, const char* what) {
        const uint32_t* p = static_cast<const uint32_t*>(a.data);
        const size_t count = a.count();
        for (size_t i = 0; i < count; ++i)
            if (p[i] >= limit)
                fail(KGE_INVALID_ARGUMENT, msg() << "'" << a.name << "' holds index " << p[i] << " at position " << i
                                                 << ", which is not below " << what << " (" << limit << ")");
    };
    // One pass per stream: copy into the pinned buffer and take the maximum (a loop without an exit,
    // which the compiler vectorises); only a stream with a bad index is walked again for its position.
    // A batch that fails a check is not staged: the engine refuses to train until one passes all five.
    staged_ = false;
    KGE_CUDA(cudaStreamSynchronize(stream_));  // the pinned buffer may still be in flight
    uint8_t* stage = pinned_;
    struct Upload { const HostArray* a; uint32_t* dst; uint32_t limit; const char* what; };
    const Upload uploads[5] = {{&remote, d_remote_, cfg_.n_entity, "model.n_entity"},
                               {&a2a, d_a2a_, (uint32_t)R, "the number of gathered rows"},
                               {&head, d_head_, (uint32_t)R, "the number of gathered rows"},
                               {&relation, d_relation_, cfg_.n_relation_type, "model.n_relation_type"},
                               {&tail, d_tail_, (uint32_t)T, "n_shard * a2a_size"}};
    for (const Upload& u : uploads) {
        const uint32_t* __restrict__ src = static_cast<const uint32_t*>(u.a->data);
        uint32_t* __restrict__ out = reinterpret_cast<uint32_t*>(stage);
        const size_t count = u.a->count();
        uint32_t highest = 0;
        for (size_t i = 0; i < count; ++i) {
            const uint32_t v = src[i];
            out[i] = v;
            highest = v > highest ? v : highest;
        }
        if (highest >= u.limit) check_below(*u.a, u.limit, u.what);
        // the transfer of this stream runs while the next one is copied and checked
        KGE_CUDA(cudaMemcpyAsync(u.dst, stage, count * 4, cudaMemcpyHostToDevice, stream_));
        stage += count * 4;
    }
    prepare_staged();
}

// The sort-and-segment tables of the staged index streams (the backward of the row gather).
void Engine::prepare_staged() {
    const size_t n = n_local_, S = cfg_.n_step, B = cfg_.batch_size, T = cfg_.n_tail(), R = cfg_.n_remote();
    KGE_CUDA(cudaEventRecord(ev_stage_[0], stream_));
    k_prepare_segments<<<(unsigned)(n * S), 512, 0, stream_>>>(
        d_head_, d_a2a_, d_relation_, d_remote_, (int)B, (int)T, (int)R, (int)cfg_.n_relation_type, d_ent_perm_,
        d_ent_off_, d_rel_perm_, d_rel_off_, d_first_slot_, split_popular_rows_ ? d_heavy_parts_ : nullptr, d_heavy_count_, d_row_info_);
    KGE_CUDA(cudaGetLastError());
    KGE_CUDA(cudaEventRecord(ev_stage_[1], stream_));
    staged_ = true;
    stage_fresh_ = true;
}

// ---------------------------------------------------------------------------
// The batch sampler on the device (src/python/poplar_kge_dataset.py:199-263, 310-393)

// "load_triples": the training triples as local rows, sorted by (head shard, tail shard) bucket:
// `triples` u32 [3, n] (head row, relation, tail row), `bucket_offset` / `bucket_count` u32
// [n_shard, n_shard], `shard_to_count` u32 [n_shard] (real rows per shard).  All shards of the job,
// on every process: a shard's batch names positives that other shards' heads drew.
void Engine::cmd_load_triples(std::vector<HostArray>& arrays) {
    const size_t n = cfg_.n_shard;
    HostArray* triples = nullptr;
    for (HostArray& a : arrays)
        if (a.name == "triples") triples = &a;
    if (!triples) fail(KGE_INVALID_ARGUMENT, "Key not found 'triples'");
    if (triples->dtype != KGE_U32 || triples->shape.size() != 2 || triples->shape[0] != 3 || triples->shape[1] == 0)
        fail(KGE_INVALID_ARGUMENT, "'triples' expected an unsigned int array of shape (3, n_triples)");
    const size_t n_triples = triples->shape[1];
    HostArray& offset = find_array(arrays, "bucket_offset", KGE_U32, {n, n});
    HostArray& count = find_array(arrays, "bucket_count", KGE_U32, {n, n});
    HostArray& rows = find_array(arrays, "shard_to_count", KGE_U32, {n});
    const uint32_t *h_off = static_cast<const uint32_t*>(offset.data), *h_cnt = static_cast<const uint32_t*>(count.data);
    const uint32_t *h_rows = static_cast<const uint32_t*>(rows.data), *h_tri = static_cast<const uint32_t*>(triples->data);
    if (cfg_.batch_size % cfg_.n_shard || cfg_.a2a_size <= cfg_.batch_size / cfg_.n_shard)
        fail(KGE_INVALID_ARGUMENT, msg() << "Expected batch_size (" << cfg_.batch_size << ") to be a multiple of n_shard and a2a_size ("
                                         << cfg_.a2a_size << ") to be >= batch_size/n_shard");
    for (size_t b = 0; b < n * n; ++b) {
        if (h_cnt[b] == 0) fail(KGE_INVALID_ARGUMENT, msg() << "'bucket_count' has an empty (head shard, tail shard) bucket " << b);
        if ((size_t)h_off[b] + h_cnt[b] > n_triples) fail(KGE_INVALID_ARGUMENT, "'bucket_offset' + 'bucket_count' passes the end of 'triples'");
    }
    for (size_t s = 0; s < n; ++s)
        if (h_rows[s] == 0 || h_rows[s] >= cfg_.n_entity)
            fail(KGE_INVALID_ARGUMENT, msg() << "'shard_to_count' (" << h_rows[s] << ") must be between 1 and model.n_entity - 1");
    for (size_t i = 0; i < n_triples; ++i) {
        if (h_tri[i] >= cfg_.n_entity || h_tri[2 * n_triples + i] >= cfg_.n_entity || h_tri[i] == 0 || h_tri[2 * n_triples + i] == 0)
            fail(KGE_INVALID_ARGUMENT, msg() << "'triples' names a row outside [1, model.n_entity) at triple " << i);
        if (h_tri[n_triples + i] >= cfg_.n_relation_type)
            fail(KGE_INVALID_ARGUMENT, msg() << "'triples' names relation " << h_tri[n_triples + i] << " at triple " << i);
    }
    uint32_t* d_triples = (uint32_t*)device_alloc(3 * n_triples * 4);
    uint32_t* d_meta = (uint32_t*)device_alloc((2 * n * n + n) * 4);
    KGE_CUDA(cudaMemcpy(d_triples, h_tri, 3 * n_triples * 4, cudaMemcpyHostToDevice));
    KGE_CUDA(cudaMemcpy(d_meta, h_off, n * n * 4, cudaMemcpyHostToDevice));
    KGE_CUDA(cudaMemcpy(d_meta + n * n, h_cnt, n * n * 4, cudaMemcpyHostToDevice));
    KGE_CUDA(cudaMemcpy(d_meta + 2 * n * n, h_rows, n * 4, cudaMemcpyHostToDevice));
    sampler_ = SamplerData{d_triples, n_triples, d_meta, d_meta + n * n, d_meta + 2 * n * n};
}

void Engine::sample_and_stage(uint32_t seed) {
    if (!sampler_.triples) fail(KGE_LOGIC_ERROR, "no training triples: run \"load_triples\" first");
    k_sample_batch<<<(unsigned)(n_local_ * cfg_.n_step), 512, 0, stream_>>>(sampler_, seed, sample_run_++, (int)cfg_.n_shard, (int)shard0_,
                                                                             (int)cfg_.n_step, (int)cfg_.batch_size, (int)cfg_.a2a_size,
                                                                             d_remote_, d_a2a_, d_head_, d_relation_, d_tail_);
    KGE_CUDA(cudaGetLastError());
    prepare_staged();
}

// "sample_batch": draws one program run's index streams on the device (`sample_seed` u32 [1]) and
// stages them; any of remote / a2a / head / relation / tail given (local shapes of
// "train_step_loop") receives a copy.  "train_step_loop_sampled": the same, then the steps:
// `learning_rate`, `loss` as for "train_step_loop"; no index array crosses the host.
void Engine::cmd_sample_batch(std::vector<HostArray>& arrays, bool train) {
    const size_t n = n_local_, S = cfg_.n_step, B = cfg_.batch_size, T = cfg_.n_tail(), R = cfg_.n_remote();
    HostArray& seed = find_array(arrays, "sample_seed", KGE_U32, {1});
    HostArray *lr = nullptr, *loss = nullptr;
    if (train) {
        lr = &find_array(arrays, "learning_rate", KGE_F32, {n});
        loss = &find_array(arrays, "loss", KGE_F32, {n});
    }
    KGE_CUDA(cudaSetDevice((int)cfg_.device_ordinal));
    sample_and_stage(static_cast<const uint32_t*>(seed.data)[0]);
    struct Stream { const char* name; uint32_t* device; std::vector<size_t> shape; };
    const Stream streams[5] = {{"remote", d_remote_, {n, S, R}}, {"a2a", d_a2a_, {n, S, cfg_.n_shard, cfg_.a2a_size}},
                               {"head", d_head_, {n, S, B}}, {"relation", d_relation_, {n, S, B}}, {"tail", d_tail_, {n, S, B}}};
    for (const Stream& st : streams)
        for (HostArray& a : arrays)
            if (a.name == st.name) {
                HostArray& out = find_array(arrays, st.name, KGE_U32, st.shape);
                KGE_CUDA(cudaMemcpyAsync(out.data, st.device, out.count() * 4, cudaMemcpyDeviceToHost, stream_));
            }
    KGE_CUDA(cudaStreamSynchronize(stream_));
    if (train) train_staged(static_cast<const float*>(lr->data)[0], static_cast<float*>(loss->data));
}


void Engine::train_staged(float learning_rate, float* loss) {
    KGE_CUDA(cudaSetDevice((int)cfg_.device_ordinal));
    require_usable();
    if (!staged_) fail(KGE_LOGIC_ERROR, "kge_train_staged called before kge_stage_batch");
    if (!connected_) fail(KGE_LOGIC_ERROR, "world_size > 1 but kge_comm_connect has not been called");
    // Adam step sizes of the staged steps (src/fructose/frnn.cpp:42-59), in fp32.
    float* sizes = reinterpret_cast<float*>(pinned_ + pinned_bytes_ - 256 - (size_t)cfg_.n_step * 4);
    for (unsigned i = 0; i < cfg_.n_step; ++i) {
        const float t = (float)(step_ + 1 + i);
        sizes[i] = (std::sqrt(1.0f - std::pow(cfg_.beta_v, t)) / (1.0f - std::pow(cfg_.beta_m, t))) * learning_rate;
    }
    KGE_CUDA(cudaMemcpyAsync(d_step_size_, sizes, (size_t)cfg_.n_step * 4, cudaMemcpyHostToDevice, stream_));
    if (dropout_on()) {
        uint32_t* keys = reinterpret_cast<uint32_t*>(sizes) - cfg_.n_step;
        for (unsigned i = 0; i < cfg_.n_step; ++i) keys[i] = (uint32_t)(step_ + 1 + i);
        KGE_CUDA(cudaMemcpyAsync(d_step_key_, keys, (size_t)cfg_.n_step * 4, cudaMemcpyHostToDevice, stream_));
    }
    KGE_CUDA(cudaMemsetAsync(d_loss_total_, 0, n_local_ * 4, stream_));
    KGE_CUDA(cudaEventRecord(ev_begin_, stream_));
    if (cfg_.cuda_graph && !kernel_timing_) {
        if (!graph_exec_) {
            cudaGraph_t graph = nullptr;
            launch_counter_ = 0;
            KGE_CUDA(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal));
            try {
                launch_steps();
            } catch (...) {
                cudaStreamEndCapture(stream_, &graph);
                if (graph) cudaGraphDestroy(graph);
                throw;
            }
            KGE_CUDA(cudaStreamEndCapture(stream_, &graph));
            cudaError_t err = cudaGraphInstantiate(&graph_exec_, graph, 0);
            cudaGraphDestroy(graph);
            KGE_CUDA(err);
            last_launches_ = launch_counter_;
        }
        KGE_CUDA(cudaGraphLaunch(graph_exec_, stream_));
    } else {
        launch_counter_ = 0;
        if (kernel_timing_) {
            // hold the stream while the host queues the run, so the event pairs bracket kernels only
            k_delay<<<1, 1, 0, stream_>>>(20ll * 1000 * 1000);
            KGE_CUDA(cudaGetLastError());
        }
        launch_steps();
        last_launches_ = launch_counter_;
    }
    KGE_CUDA(cudaEventRecord(ev_end_, stream_));
    float* host_loss = reinterpret_cast<float*>(pinned_ + pinned_bytes_ - 256);
    if (loss)
        KGE_CUDA(cudaMemcpyAsync(host_loss, d_loss_total_, n_local_ * 4, cudaMemcpyDeviceToHost, stream_));
    KGE_CUDA(cudaStreamSynchronize(stream_));
    KGE_CUDA(cudaEventElapsedTime(&last_ms_, ev_begin_, ev_end_));
    if (stage_fresh_) {
        // the sort-and-segment preparation belongs to the step (it is the backward of the row
        // gather): its device time counts towards the first run of a staged batch
        float stage_ms = 0.f;
        KGE_CUDA(cudaEventElapsedTime(&stage_ms, ev_stage_[0], ev_stage_[1]));
        last_ms_ += stage_ms;
        stage_fresh_ = false;
    }
    timing_collect();
    step_ += cfg_.n_step;
    check_device_status();
    if (loss)
        for (unsigned l = 0; l < n_local_; ++l) loss[l] = host_loss[l] / (float)cfg_.n_step;
}

// Both status words come back in one copy (they are neighbours in device memory).  A wait that gave
// up leaves this engine's kernels out of step with the other processes' (their hand-over epochs
// disagree from then on), so the engine refuses further device commands: it must be rebuilt.
void Engine::check_device_status() {
    unsigned status[2] = {0, 0};  // [0] the tensor-core pipeline, [1] the hand-overs between processes
    KGE_CUDA(cudaMemcpyAsync(status, d_tc_status_, sizeof(status), cudaMemcpyDeviceToHost, stream_));
    KGE_CUDA(cudaStreamSynchronize(stream_));
    if (!status[0] && !status[1]) return;
    poisoned_ = true;
    KGE_CUDA(cudaMemset(d_tc_status_, 0, sizeof(status)));
    if (status[0]) fail(KGE_DEVICE_STATUS, msg() << "a bounded wait on the tensor-core pipeline gave up (code " << status[0] << ")");
    fail(KGE_DEVICE_STATUS, msg() << "a device-side wait for rank " << (status[1] - 1)
                                  << " gave up: that process did not reach the same step");
}

void Engine::require_usable() const {
    if (poisoned_)
        fail(KGE_LOGIC_ERROR, "a device-side wait of an earlier command gave up: this engine is out of step with the other "
                              "processes and must be rebuilt");
}

void Engine::set_kernel_timing(bool on) {
    kernel_timing_ = on;
    if (on) kernel_times_.clear();
}

size_t Engine::kernel_time_count() const { return kernel_times_.size(); }

void Engine::kernel_time(size_t index, const char** name, float* ms, unsigned long long* launches) const {
    if (index >= kernel_times_.size()) fail(KGE_INVALID_ARGUMENT, "kge_kernel_time: index past the end");
    auto it = kernel_times_.begin();
    std::advance(it, index);
    if (name) *name = it->first.c_str();
    if (ms) *ms = it->second.ms;
    if (launches) *launches = it->second.launches;
}

void Engine::last_run_stats(float* ms, unsigned long long* launches) const {
    if (ms) *ms = last_ms_;
    if (launches) *launches = last_launches_;
}

// Wraps one kernel launch: counts it and, when per-kernel timing is on, brackets it with a
// pair of events on the engine's stream.
#define KGE_LAUNCH(name, ...)            \
    do {                                 \
        timing_begin(name);              \
        __VA_ARGS__;                     \
        timing_end();                    \
        ++launch_counter_;               \
    } while (0)

bool dependent_launch_enabled() {
    static const bool enabled = [] {
        const char* off = std::getenv("KGE_NO_DEPENDENT_LAUNCH");
        return !(off && off[0] && off[0] != '0');
    }();
    return enabled;
}

void Engine::launch_steps() {
    launch_gather(0, stream_);
    for (unsigned step = 0; step < cfg_.n_step; ++step) launch_one_step(step);
    // The last kernel of a step only publishes its dense parameters.  The run ends when every
    // process's share has arrived in this process's copy (values and optimiser state), so that a
    // "read" or "predict" issued straight after the run sees the finished step without a host barrier.
    launch_exchange_wait(XCHG_DENSE_PARAMS);
}

// The step's rows, gathered into the compact copy every later kernel of the step reads (two
// copies, for even and odd steps).  The gather of step s + 1 needs only the rows step s has
// updated, so it runs beside the projection gradient and the dense update of step s.
void Engine::launch_gather(unsigned step, cudaStream_t stream) {
    const unsigned R = cfg_.n_remote();
    for (unsigned l = 0; l < n_local_; ++l) {
        ShardBuffers& b = shards_[l];
        const uint32_t* remote = d_remote_ + ((size_t)l * cfg_.n_step + step) * R;
        KGE_LAUNCH("gather", KGE_CUDA(launch_dependent(k_gather_step_rows, dim3(ceil_div(R, 8)), dim3(256), 0, stream, b.table,
                                                       layout_.row_bytes, remote, (int)R, b.rows_c2[step & 1], feature_planes(b, step & 1))));
    }
}

FeaturePlanes Engine::feature_planes(const ShardBuffers& b, unsigned parity) const {
    FeaturePlanes fp{};
    fp.wide = b.feat_wide2[parity];
    fp.lo = b.feat_lo2[parity];
    fp.stride = feat_stride_;
    fp.off_feat = layout_.off_feat;
    return fp;
}

// Fork: what is launched on the returned stream starts after everything queued on the main stream
// so far.  While per-kernel timing is on, everything stays on the main stream.
cudaStream_t Engine::side_begin() {
    if (kernel_timing_ || !side_streams_) return stream_;
    KGE_CUDA(cudaEventRecord(ev_fork_, stream_));
    KGE_CUDA(cudaStreamWaitEvent(side_stream_, ev_fork_, 0));
    return side_stream_;
}
// ... the side work is complete here ...
void Engine::side_end(int which) {
    if (kernel_timing_ || !side_streams_) return;
    KGE_CUDA(cudaEventRecord(ev_join_[which], side_stream_));
}
// ... and the main stream waits for it here.
void Engine::side_join(int which) {
    if (kernel_timing_ || !side_streams_) return;
    KGE_CUDA(cudaStreamWaitEvent(stream_, ev_join_[which], 0));
}

void Engine::launch_barrier() {
    if (cfg_.world == 1) return;
    BarrierArgs a;
    a.peer_flags = d_peer_flags_;
    a.my_epoch = d_epoch_;
    a.status = d_status_;
    a.rank = (int)cfg_.rank;
    a.world = (int)cfg_.world;
    a.max_spins = 2ull * 1000 * 1000;  // a second or two of 64 ns naps plus load latency
    KGE_LAUNCH("barrier", KGE_CUDA(launch_dependent(k_barrier, dim3(1), dim3(64), 0, stream_, a)));
    KGE_CUDA(cudaGetLastError());
}

// What the step's kernels need to publish and await the hand-overs between processes; with one
// process the kernels skip both.
ExchangeSync Engine::exchange_sync() const {
    ExchangeSync s{};
    s.peer_flags = d_peer_flags_;
    s.epochs = d_xchg_words_;
    s.counters = d_xchg_words_ + XCHG_KINDS;
    s.status = d_status_;
    s.rank = (int)cfg_.rank;
    s.world = (int)cfg_.world;
    s.max_spins = 1u << 28;
    s.timeout_ns = 2000ull * 1000ull * 1000ull;  // two seconds
    s.trace = d_xchg_trace_;
    return s;
}

void Engine::launch_exchange_wait(int kind) {
    if (cfg_.world == 1) return;
    KGE_LAUNCH("exchange_wait", KGE_CUDA(launch_dependent(k_exchange_wait, dim3(1), dim3(kMaxProcesses), 0, stream_, exchange_sync(), kind)));
}

void Engine::launch_exchange_signal(int kind) {
    if (cfg_.world == 1) return;
    KGE_LAUNCH("exchange_signal", KGE_CUDA(launch_dependent(k_exchange_signal, dim3(1), dim3(kMaxProcesses), 0, stream_, exchange_sync(), kind)));
}

void Engine::timing_begin(const char* name) {
    if (!kernel_timing_ || timed_.size() >= kMaxTimedLaunches) return;
    while (event_pool_.size() < 2 * (timed_.size() + 1)) {
        cudaEvent_t e = nullptr;
        KGE_CUDA(cudaEventCreate(&e));
        event_pool_.push_back(e);
    }
    timed_.push_back({name, event_pool_[2 * timed_.size()], event_pool_[2 * timed_.size() + 1]});
    timing_open_ = true;
    KGE_CUDA(cudaEventRecord(timed_.back().start, stream_));
}

void Engine::timing_end() {
    if (!timing_open_) return;
    timing_open_ = false;
    KGE_CUDA(cudaEventRecord(timed_.back().stop, stream_));
}

void Engine::timing_collect() {
    for (TimedLaunch& t : timed_) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, t.start, t.stop) == cudaSuccess) {
            KernelTime& k = kernel_times_[t.name];
            k.ms += ms;
            k.launches += 1;
        }
    }
    timed_.clear();
}

// How many k splits fill the GPU: about one block per SM, at least two 32-deep slices per split.
int Engine::tc_splits(unsigned tiles, unsigned k) const {
    const unsigned by_sms = std::max(1u, 148u / std::max(1u, tiles));
    const unsigned by_k = std::max(1u, k / 64u);
    int splits = (int)std::min<unsigned>({by_sms, by_k, (unsigned)kTcMaxSplits});
    // the splits of a tile run as one cluster: all tiles' clusters should be resident together
    while (splits > 1 && (unsigned)tc::max_resident_clusters(splits) < tiles) --splits;
    return splits;
}

// One launch for one or two contractions of the same kind (see tc_gemm.cuh).  With splits > 1
// the k range is divided and the partial tiles are reduced inside the kernel, in split order.
void Engine::launch_tc(const char* name, tc::GemmArgs* problems, int n_problems, int splits, bool a_exact, bool rowsum,
                       int wait_kind, int signal_kind) {
    for (int i = 0; i < n_problems; ++i) {
        tc::GemmArgs& g = problems[i];
        g.status = d_tc_status_;
        const unsigned tiles = ceil_div((unsigned)g.M, 128) * ceil_div((unsigned)g.N, 64);
        if (splits > 1 && tiles <= 4096 && (size_t)g.M * g.N * splits <= tc_ws_floats_) {
            g.k_per_split = (int)round_up(ceil_div((unsigned)g.K, (unsigned)splits), 32);
            g.ws = tc_ws_ + (size_t)i * tc_ws_floats_;
            g.ws_rowsum = tc_ws_rowsum_ + (size_t)i * kTcMaxSplits * std::max(cfg_.batch_size, cfg_.n_tail());
        } else {
            g.k_per_split = std::max(32, (int)round_up((unsigned)g.K, 32));
            g.ws = nullptr;
        }
    }
    if (!problems[0].ws || (n_problems > 1 && !problems[1].ws)) {
        splits = 1;
        for (int i = 0; i < n_problems; ++i) {
            problems[i].ws = nullptr;
            problems[i].k_per_split = std::max(32, (int)round_up((unsigned)problems[i].K, 32));
        }
    }
    cudaError_t err;
    timing_begin(name);
    int n_launches = 1;
    const ExchangeSync sync = exchange_sync();
    if (a_exact) err = rowsum ? tc::launch_pair<64, true, true>(problems, n_problems, splits, stream_, &n_launches, sync, wait_kind, signal_kind)
                              : tc::launch_pair<64, true, false>(problems, n_problems, splits, stream_, &n_launches, sync, wait_kind, signal_kind);
    else err = rowsum ? tc::launch_pair<64, false, true>(problems, n_problems, splits, stream_, &n_launches, sync, wait_kind, signal_kind)
                      : tc::launch_pair<64, false, false>(problems, n_problems, splits, stream_, &n_launches, sync, wait_kind, signal_kind);
    timing_end();
    launch_counter_ += (unsigned long long)n_launches;
    KGE_CUDA(err);
}

// One launch of the plane-fed contraction for one or two problems of the same shape class.  Tiles
// are 128 x 128 (128 x 64 for narrow outputs); the k range is split over the blocks of a cluster so
// that about one block per SM is busy and every split keeps at least two 32-deep slices.
void Engine::launch_planes(const char* name, tc::PlaneProblem* problems, int n_problems, int side, int wait_kind, int signal_kind,
                           const tc::RouteArgs* route) {
    int max_n = 0, max_k = 0;
    unsigned tiles = 0;
    for (int i = 0; i < n_problems; ++i) max_n = std::max(max_n, problems[i].g.N);
    const int tile_n = max_n > 64 ? 128 : 64;
    for (int i = 0; i < n_problems; ++i) {
        tiles += ceil_div((unsigned)problems[i].g.M, 128) * ceil_div((unsigned)max_n, (unsigned)tile_n);
        max_k = std::max(max_k, problems[i].g.K);
    }
    int splits = (int)std::min<unsigned>({std::max(1u, 148u / std::max(1u, tiles)), std::max(1u, (unsigned)max_k / 64u),
                                          (unsigned)tc::kMaxClusterSplits});
    while (splits > 1 && (unsigned)tc::max_resident_plane_clusters(splits) < tiles) --splits;
    for (int i = 0; i < n_problems; ++i) {
        tc::GemmArgs& g = problems[i].g;
        g.status = d_tc_status_;
        const unsigned slice = problems[i].A.elem_bytes == 2 ? 64u : 32u;  // bf16 slices are 64 deep
        g.k_per_split = (int)std::max<size_t>(slice, round_up(ceil_div((unsigned)g.K, (unsigned)splits), slice));
    }
    timing_begin(name);
    cudaError_t err;
    if (side == tc::SIDE_ROWSUM) err = tc::launch_planes<tc::SIDE_ROWSUM>(problems, n_problems, splits, tile_n, stream_, exchange_sync(), wait_kind, signal_kind, route);
    else if (side == tc::SIDE_NORMS) err = tc::launch_planes<tc::SIDE_NORMS>(problems, n_problems, splits, tile_n, stream_, exchange_sync(), wait_kind, signal_kind, route);
    else err = tc::launch_planes<tc::SIDE_NONE>(problems, n_problems, splits, tile_n, stream_, exchange_sync(), wait_kind, signal_kind, route);
    timing_end();
    ++launch_counter_;
    KGE_CUDA(err);
}

// The feature MLP on `n_rows` rows whose hidden buffer holds value + feature . W (src/poplar_kge.cpp:453-458):
// hid = value + relu(concat(value, hid - value) . up) . down, the values read from rows `index[i]` (or
// start + i) of `rows`.  Leaves the MLP's input in `cat` and its pre-activations in `pre` for the backward.
void Engine::launch_mlp_forward(const uint8_t* rows, const uint32_t* index, uint32_t start, unsigned n_rows, int net, float* hid,
                                float* cat, float* pre, float* out) {
    const unsigned D = cfg_.d, M = cfg_.mlp;
    const float* up = dense_ + dense_bounds_[4 + 2 * net];
    const float* down = dense_ + dense_bounds_[5 + 2 * net];
    const dim3 grid(std::min(ceil_div(n_rows * D, 256), 148u * 8));
    if (cfg_.state_type == ST_F32)
        KGE_LAUNCH("mlp", KGE_CUDA(launch_dependent(k_mlp_concat<float>, grid, dim3(256), 0, stream_, rows, layout_, index, start, (int)n_rows, (const float*)hid, cat)));
    else
        KGE_LAUNCH("mlp", KGE_CUDA(launch_dependent(k_mlp_concat<__half>, grid, dim3(256), 0, stream_, rows, layout_, index, start, (int)n_rows, (const float*)hid, cat)));
    SgemmArgs g{};
    g.A = cat; g.lda = 2 * D; g.B = up; g.ldb = M; g.C = pre; g.ldc = M; g.M = (int)n_rows; g.N = (int)M; g.K = (int)(2 * D);
    KGE_LAUNCH("mlp", KGE_CUDA(launch_sgemm(g, stream_)));
    g = SgemmArgs{};
    g.A = pre; g.lda = M; g.a_relu = 1; g.B = down; g.ldb = D; g.C = out; g.ldc = D; g.M = (int)n_rows; g.N = (int)D; g.K = (int)M;
    KGE_LAUNCH("mlp", KGE_CUDA(launch_sgemm(g, stream_)));
    if (cfg_.state_type == ST_F32)
        KGE_LAUNCH("mlp", KGE_CUDA(launch_dependent(k_mlp_finish<float>, grid, dim3(256), 0, stream_, rows, layout_, index, start, (int)n_rows, (const float*)out, hid)));
    else
        KGE_LAUNCH("mlp", KGE_CUDA(launch_dependent(k_mlp_finish<__half>, grid, dim3(256), 0, stream_, rows, layout_, index, start, (int)n_rows, (const float*)out, hid)));
}

// Backward of the MLP for local shard l, after the entity update has left the gradients of the
// MLP's outputs in d_hid_h / d_hid_t and the value's gradient so far in d_val: this shard's
// gradients of the up and down projections go to their owners, the input gradient's first half
// joins d_val, its second half replaces d_hid (the projection gradient's operand), and the rows
// get their Adam step.
void Engine::launch_mlp_backward(unsigned l, unsigned step) {
    ShardBuffers& b = shards_[l];
    const unsigned D = cfg_.d, M = cfg_.mlp, R = cfg_.n_remote();
    const size_t sidx = (size_t)l * cfg_.n_step + step;
    for (unsigned net = 0; net < cfg_.n_net(); ++net) {
        float* d_out = net ? b.d_hid_t : b.d_hid_h;
        const float* up = dense_ + dense_bounds_[4 + 2 * net];
        const float* down = dense_ + dense_bounds_[5 + 2 * net];
        SgemmArgs g{};  // d down = relu(pre)^T . d_out
        g.A = b.mlp_pre[net]; g.lda = M; g.a_trans = 1; g.a_relu = 1; g.B = d_out; g.ldb = D; g.C = b.mlp_dw_down; g.ldc = D;
        g.M = (int)M; g.N = (int)D; g.K = (int)R;
        KGE_LAUNCH("mlp_bwd", KGE_CUDA(launch_sgemm(g, stream_)));
        g = SgemmArgs{};  // d pre = (d_out . down^T) where pre >= 0
        g.A = d_out; g.lda = D; g.B = down; g.ldb = D; g.b_trans = 1; g.C = b.mlp_d_pre; g.ldc = M; g.M = (int)R; g.N = (int)M; g.K = (int)D;
        g.pass = b.mlp_pre[net]; g.ldpass = M;
        KGE_LAUNCH("mlp_bwd", KGE_CUDA(launch_sgemm(g, stream_)));
        g = SgemmArgs{};  // d up = cat^T . d pre
        g.A = b.mlp_cat[net]; g.lda = 2 * D; g.a_trans = 1; g.B = b.mlp_d_pre; g.ldb = M; g.C = b.mlp_dw_up; g.ldc = M;
        g.M = (int)(2 * D); g.N = (int)M; g.K = (int)R;
        KGE_LAUNCH("mlp_bwd", KGE_CUDA(launch_sgemm(g, stream_)));
        g = SgemmArgs{};  // d cat = d pre . up^T
        g.A = b.mlp_d_pre; g.lda = M; g.B = up; g.ldb = M; g.b_trans = 1; g.C = b.mlp_d_cat; g.ldc = 2 * D; g.M = (int)R; g.N = (int)(2 * D); g.K = (int)M;
        KGE_LAUNCH("mlp_bwd", KGE_CUDA(launch_sgemm(g, stream_)));
        const dim3 pgrid(std::min(ceil_div(2 * M * D, 256), 148u * 4));
        KGE_LAUNCH("mlp_bwd", KGE_CUDA(launch_dependent(k_push_dense_rows, pgrid, dim3(256), 0, stream_, (const float*)b.mlp_dw_up, (int)(2 * M),
                                                        (int)(dense_bounds_[4 + 2 * net] / D), (int)D, b.dense_dst, (int)cfg_.world)));
        KGE_LAUNCH("mlp_bwd", KGE_CUDA(launch_dependent(k_push_dense_rows, pgrid, dim3(256), 0, stream_, (const float*)b.mlp_dw_down, (int)M,
                                                        (int)(dense_bounds_[5 + 2 * net] / D), (int)D, b.dense_dst, (int)cfg_.world)));
        const dim3 sgrid(std::min(ceil_div(R * D, 256), 148u * 8));
        KGE_LAUNCH("mlp_bwd", KGE_CUDA(launch_dependent(k_mlp_split, sgrid, dim3(256), 0, stream_, (const float*)b.mlp_d_cat, b.d_val, d_out, (int)R, (int)D)));
    }
    const dim3 agrid(std::min(ceil_div(R * D, 256), 148u * 8));
    const uint8_t* rows_c = b.rows_c2[step & 1];
    const uint32_t* remote = d_remote_ + sidx * R;
    if (cfg_.state_type == ST_F32)
        KGE_LAUNCH("row_adam", KGE_CUDA(launch_dependent(k_row_adam<float>, agrid, dim3(256), 0, stream_, b.table, rows_c, layout_, remote, (const uint32_t*)(d_first_slot_ + sidx * R),
                                                         (const float*)b.d_val, (const float*)(d_step_size_ + step), entity_lr_mod_, adam_, (int)R)));
    else
        KGE_LAUNCH("row_adam", KGE_CUDA(launch_dependent(k_row_adam<__half>, agrid, dim3(256), 0, stream_, b.table, rows_c, layout_, remote, (const uint32_t*)(d_first_slot_ + sidx * R),
                                                         (const float*)b.d_val, (const float*)(d_step_size_ + step), entity_lr_mod_, adam_, (int)R)));
}

// The norm regularisers of local shard l's gathered rows (k_regularise): after the hidden rows,
// before the loss (which adds their loss term) and the entity update (which adds their gradients).
void Engine::launch_regularise(unsigned l, const uint8_t* rows_c) {
    ShardBuffers& b = shards_[l];
    const size_t R = cfg_.n_remote();
    RegParams rp{};
    for (int i = 0; i < 3; ++i) rp.power[i] = cfg_.reg_power[i], rp.weight[i] = cfg_.reg_weight[i];
    rp.loss_scale = cfg_.loss_scale;
    rp.shared = b.hid_t == b.hid_h ? 1 : 0;
    float* loss = d_reg_loss_ + 2 * l;
    if (cfg_.state_type == ST_F32)
        KGE_LAUNCH("regularise", KGE_CUDA(launch_dependent(k_regularise<float>, dim3((unsigned)ceil_div(R, 8)), dim3(256), 0, stream_, rows_c, layout_, b.hid_h,
                                                           b.hid_t, (int)R, rp, b.reg_val, b.reg_h, b.reg_t, b.reg_loss_rows, loss, loss + 1, d_reg_counter_ + l)));
    else
        KGE_LAUNCH("regularise", KGE_CUDA(launch_dependent(k_regularise<__half>, dim3((unsigned)ceil_div(R, 8)), dim3(256), 0, stream_, rows_c, layout_, b.hid_h,
                                                           b.hid_t, (int)R, rp, b.reg_val, b.reg_h, b.reg_t, b.reg_loss_rows, loss, loss + 1, d_reg_counter_ + l)));
}

RelationRows Engine::with_regularisers(RelationRows rr, unsigned l, unsigned step) const {
    const ShardBuffers& b = shards_[l];
    rr.reg_val = b.reg_val;
    rr.reg_h = b.reg_h;
    rr.reg_t = b.reg_t;
    rr.drop = dropout_params(l, step);
    rr.defer_grad = b.d_val;
    return rr;
}

DropoutParams Engine::dropout_params(unsigned l, unsigned step) const {
    DropoutParams dp{};
    if (!dropout_on()) return dp;
    dp.threshold = (uint32_t)std::lround((1.0 - (double)cfg_.dropout) * 16777216.0);
    dp.seed = cfg_.seed;
    dp.step_key = d_step_key_ + step;
    dp.shard = (uint32_t)(shard0_ + l);
    dp.scale = 1.0f / (1.0f - cfg_.dropout);
    return dp;
}

// hidden = value + dropout(hidden - value) for both calls of local shard l (k_dropout_hidden).
void Engine::launch_dropout(unsigned l, unsigned step, const uint8_t* rows_c) {
    ShardBuffers& b = shards_[l];
    const size_t R = cfg_.n_remote(), quads = ceil_div(cfg_.d, 4);
    const float* tail_in = cfg_.n_net() == 2 ? b.hid_t : b.hid_h;
    const dim3 grid((unsigned)ceil_div(R * quads, 256));
    if (cfg_.state_type == ST_F32)
        KGE_LAUNCH("dropout", KGE_CUDA(launch_dependent(k_dropout_hidden<float>, grid, dim3(256), 0, stream_, rows_c, layout_, b.hid_h, tail_in, b.hid_t,
                                                        (int)R, dropout_params(l, step))));
    else
        KGE_LAUNCH("dropout", KGE_CUDA(launch_dependent(k_dropout_hidden<__half>, grid, dim3(256), 0, stream_, rows_c, layout_, b.hid_h, tail_in, b.hid_t,
                                                        (int)R, dropout_params(l, step))));
}

// The training step with its contractions on the plane-fed kernel: seven launches on the step's
// chain (hidden + lookups + send, scores, loss, score gradients + return, segment sums + Adam +
// relation gradients, projection gradient, dense update) and the next step's gather beside the
// last two.  Every operand of a contraction is the fp32 array its producer wrote (the upper TF32
// plane) plus a lower plane the same producer wrote next to it.
void Engine::launch_step_planes(unsigned step, const LossParams& lp, float normaliser) {
    const unsigned B = cfg_.batch_size, T = cfg_.n_tail(), R = cfg_.n_remote(), D = cfg_.d, F = cfg_.f;
    const unsigned n_rel = cfg_.n_relation_type, parity = step & 1;
    const bool two_nets = cfg_.n_net() == 2, l2 = cfg_.dist_fn == DIST_L2, l1 = cfg_.dist_fn == DIST_L1;
    // bf16 embeddings: the dot-product scores and their gradients multiply bfloat16 copies of pred,
    // tails and the coefficients (written by their producers into the companion planes)
    const bool bf16 = bf16_planes_;
    auto plane16 = [](const float* values, long long row_elems, bool mn_major) {
        return tc::PlaneOperand{values, nullptr, row_elems * 2, mn_major ? 1 : 0, 2};
    };
    const bool half_features = cfg_.feature_type == ST_F16;
    const float* rel_table = dense_;
    const ExchangeSync sync = exchange_sync();
    auto step_ptr = [&](uint32_t* base, unsigned l, size_t per_step) { return base + ((size_t)l * cfg_.n_step + step) * per_step; };
    auto plane = [](const float* hi, const float* lo, long long stride_bytes, bool mn_major) {
        return tc::PlaneOperand{hi, lo, stride_bytes, mn_major ? 1 : 0};
    };
    auto features = [&](const ShardBuffers& b, bool mn_major) {
        if (half_features) return plane(b.feat_wide2[parity], nullptr, (long long)feat_stride_ * 4, mn_major);
        return plane(reinterpret_cast<const float*>(b.rows_c2[parity] + layout_.off_feat), b.feat_lo2[parity], (long long)layout_.row_bytes, mn_major);
    };

    for (unsigned l = 0; l < n_local_; ++l) {
        ShardBuffers& b = shards_[l];
        uint8_t* rows_c = b.rows_c2[parity];
        const size_t sidx = (size_t)l * cfg_.n_step + step;
        const uint32_t* a2a = step_ptr(d_a2a_, l, T);
        const uint32_t* head = step_ptr(d_head_, l, B);
        const uint32_t* relation = step_ptr(d_relation_, l, B);
        // 1. hidden = value + feature . W, and from its epilogue the lookups and the send half of the exchange
        const bool fused_route = F > 0 && cfg_.score_fn != SCORE_COMPLEX && cfg_.score_fn != SCORE_ROTATE && !dropout_on();
        if (F > 0) {
            tc::PlaneProblem nets[2] = {};
            const int n_nets = two_nets ? 2 : 1;
            for (int net = 0; net < n_nets; ++net) {
                tc::PlaneProblem& p = nets[net];
                const size_t w = dense_bounds_[1 + net];
                p.A = features(b, false);
                p.B = plane(dense_ + w, dense_lo_ + w, (long long)D * 4, true);
                tc::GemmArgs& g = p.g;
                g.M = (int)R; g.N = (int)D; g.K = (int)F;
                g.epilogue = tc::EPI_ADD_TABLE_VALUE;
                g.out = net ? b.hid_t : b.hid_h; g.ldc = D; g.block_rows = 1;
                g.x_base = rows_c; g.x_row_stride_bytes = layout_.row_bytes; g.x_is_half = cfg_.value_bf16 ? 2 : (cfg_.state_type == ST_F16 ? 1 : 0);
            }
            tc::RouteArgs route{};
            route.perm = d_ent_perm_ + sidx * (B + T);
            route.off = d_ent_off_ + sidx * (R + 1);
            route.relation = relation;
            route.rel_table = rel_table;
            route.send_dst = b.send_dst;
            route.send_lo_dst = b.send_lo_dst;
            route.pred = b.pred;
            route.pred_lo = b.pred_lo;
            route.B = (int)B; route.a2a = (int)cfg_.a2a_size; route.n_shard = (int)cfg_.n_shard; route.score_fn = cfg_.score_fn;
            route.mode[0] = two_nets ? 1 : 3;
            route.mode[1] = two_nets ? 2 : 0;
            route.lo_bf16 = bf16 ? 1 : 0;
            // rows with many lookups are routed in parts by a kernel of their own, which then publishes the tails
            const bool heavy_route = fused_route && split_popular_rows_ && heavy_route_;
            route.first_slot = heavy_route ? d_first_slot_ + sidx * R : nullptr;
            launch_planes("hidden", nets, n_nets, tc::SIDE_NONE, XCHG_DENSE_PARAMS, fused_route && !heavy_route ? XCHG_TAILS : -1,
                          fused_route ? &route : nullptr);
            if (heavy_route)
                KGE_LAUNCH("route_heavy", KGE_CUDA(launch_dependent(k_route_heavy, dim3(kHeavySlots), dim3(256), 0, stream_, (const float*)b.hid_h, (const float*)b.hid_t,
                                                                    (const uint4*)(d_heavy_parts_ + sidx * kHeavySlots), (const uint32_t*)(d_heavy_count_ + sidx),
                                                                    (const uint32_t*)(d_ent_perm_ + sidx * (B + T)), relation, rel_table, b.send_dst, b.send_lo_dst,
                                                                    b.pred, b.pred_lo, (int)B, (int)cfg_.a2a_size, (int)D, cfg_.score_fn, bf16 ? 1 : 0, sync)));
        } else {
            // no features: the hidden rows are the gathered values
            launch_exchange_wait(XCHG_DENSE_PARAMS);
            dim3 grid(ceil_div(R, 64), ceil_div(D, 64), 1);
            KGE_LAUNCH("hidden", KGE_DISPATCH_ROW(cfg_, KGE_CUDA(launch_dependent(k_hidden<ST, FT>, dim3(grid), dim3(256), 0, stream_, rows_c, layout_,
                                                                                  nullptr, 0u, (int)R, nullptr, nullptr, b.hid_h, b.hid_t))));
        }
        if (dropout_on()) launch_dropout(l, step, rows_c);
        if (!fused_route)
            KGE_LAUNCH("route", KGE_CUDA(launch_dependent(k_route<4>, dim3(T + B), dim3(64), 0, stream_, b.hid_h, b.hid_t, a2a, head, relation, rel_table,
                                                          b.send_dst, b.pred, (int)T, (int)cfg_.a2a_size, (int)B, (int)D, cfg_.score_fn, sync,
                                                          b.send_lo_dst, b.pred_lo, bf16 ? 1 : 0)));
        if (cfg_.regularised()) launch_regularise(l, rows_c);
    }
    KGE_CUDA(cudaGetLastError());

    for (unsigned l = 0; l < n_local_; ++l) {
        ShardBuffers& b = shards_[l];
        const uint32_t* head = step_ptr(d_head_, l, B);
        const uint32_t* relation = step_ptr(d_relation_, l, B);
        const uint32_t* tail = step_ptr(d_tail_, l, B);
        // 2. scores
        if (cfg_.dist_fn == DIST_DOT) {
            tc::PlaneProblem p{};
            p.A = bf16 ? plane16(b.pred_lo, D, false) : plane(b.pred, b.pred_lo, (long long)D * 4, false);
            p.B = bf16 ? plane16(b.tails_lo, D, false) : plane(b.tails, b.tails_lo, (long long)D * 4, false);
            p.g.M = (int)B; p.g.N = (int)T; p.g.K = (int)D;
            p.g.epilogue = tc::EPI_STORE; p.g.out = b.raw; p.g.ldc = T; p.g.block_rows = 1;
            launch_planes("score", &p, 1, tc::SIDE_NONE, XCHG_TAILS, -1);
        } else if (l2 && cfg_.l2_contraction) {
            // the L2 distance as |p|^2 + |t|^2 - 2 p.t on the tensor cores (direct form where that cancels)
            tc::PlaneProblem p{};
            p.A = plane(b.pred, b.pred_lo, (long long)D * 4, false);
            p.B = plane(b.tails, b.tails_lo, (long long)D * 4, false);
            p.g.M = (int)B; p.g.N = (int)T; p.g.K = (int)D;
            p.g.epilogue = tc::EPI_L2_DISTANCE; p.g.out = b.raw; p.g.ldc = T; p.g.block_rows = 1;
            launch_planes("score", &p, 1, tc::SIDE_NORMS, XCHG_TAILS, -1);
        } else {
            KGE_LAUNCH("score", KGE_CUDA(launch_score(cfg_.dist_fn, b.pred, b.tails, b.raw, (int)B, (int)T, (int)D, stream_, sync)));
        }
        // 3. loss and the coefficients of the score gradients
        // (the rows' loss terms are added up by a block of the entity update, off the chain)
        KGE_LAUNCH("loss", KGE_CUDA(launch_loss(b.raw, tail, b.coeff, b.loss_rows, lp, 1.0f / normaliser, nullptr, nullptr,
                                                d_loss_counter_ + l, l1 ? nullptr : b.coeff_lo, bf16 ? 1 : 0, (int)B, stream_, nullptr)));
        // 4. score gradients; the tails' rows go straight to the shards that own them
        if (l1) {
            PairBwdArgs pa{};
            pa.D = (int)D;
            pa.tiles_m0 = (int)ceil_div(B, 32);
            pa.p[0] = {b.pred, b.tails, b.coeff, (int)B, (int)T, (int)T, 1, b.d_pred, nullptr, 1};
            pa.p[1] = {b.tails, b.pred, b.coeff, (int)T, (int)B, 1, (int)T, nullptr, b.grad_dst, (int)cfg_.a2a_size};
            dim3 bgrid(ceil_div(B, 32) + ceil_div(T, 32), ceil_div(D, 64));
            KGE_LAUNCH("score_bwd", KGE_CUDA(launch_dependent(k_pair_bwd<DIST_L1>, dim3(bgrid), dim3(128), 0, stream_, pa)));
            launch_exchange_signal(XCHG_TAIL_GRADS);
        } else {
            //   dot:  d_pred = C . tails,                          d_tails = C^T . pred
            //   L2:   d_pred = rowsum(C) * pred - C . tails,       d_tails = colsum(C) * tails - C^T . pred
            tc::PlaneProblem both[2] = {};
            tc::PlaneProblem& g = both[0];
            g.A = bf16 ? plane16(b.coeff_lo, T, false) : plane(b.coeff, b.coeff_lo, (long long)T * 4, false);
            g.B = bf16 ? plane16(b.tails_lo, D, true) : plane(b.tails, b.tails_lo, (long long)D * 4, true);
            g.g.M = (int)B; g.g.N = (int)D; g.g.K = (int)T;
            g.g.epilogue = l2 ? tc::EPI_ROWSUM_X_MINUS : tc::EPI_STORE;
            g.g.out = b.d_pred; g.g.ldc = D; g.g.block_rows = 1;
            g.g.x_base = reinterpret_cast<const uint8_t*>(b.pred); g.g.x_row_stride_bytes = (long long)D * 4;
            tc::PlaneProblem& h = both[1];
            h.A = bf16 ? plane16(b.coeff_lo, T, true) : plane(b.coeff, b.coeff_lo, (long long)T * 4, true);
            h.B = bf16 ? plane16(b.pred_lo, D, true) : plane(b.pred, b.pred_lo, (long long)D * 4, true);
            h.g.M = (int)T; h.g.N = (int)D; h.g.K = (int)B;
            h.g.epilogue = g.g.epilogue;
            h.g.out = nullptr; h.g.out_blocks = b.grad_dst; h.g.block_rows = (int)cfg_.a2a_size; h.g.ldc = D;
            h.g.x_base = reinterpret_cast<const uint8_t*>(b.tails); h.g.x_row_stride_bytes = (long long)D * 4;
            launch_planes("score_bwd", both, 2, l2 ? tc::SIDE_ROWSUM : tc::SIDE_NONE, -1, XCHG_TAIL_GRADS);
        }
        if (cfg_.score_fn != SCORE_TRANSE)
            KGE_LAUNCH("pred_bwd", KGE_CUDA(launch_dependent(k_pred_bwd, dim3(B), dim3(64), 0, stream_, b.d_pred, b.hid_h, head, relation, rel_table, b.d_head,
                                                             b.d_relrow, (int)D, cfg_.score_fn)));
    }
    KGE_CUDA(cudaGetLastError());

    // 5. segment sums + row-wise Adam, and the relation rows of the partial dense gradient
    for (unsigned l = 0; l < n_local_; ++l) {
        ShardBuffers& b = shards_[l];
        const size_t sidx = (size_t)l * cfg_.n_step + step;
        const HeavyRows heavy{d_heavy_parts_ + sidx * kHeavySlots, d_heavy_count_ + sidx, b.heavy_partial, b.heavy_counter, d_row_info_ + sidx * 2 * R};
        const RelationRows rr = with_regularisers(RelationRows{b.d_relrow, d_rel_perm_ + sidx * B, d_rel_off_ + sidx * (n_rel + 1), b.dense_dst,
                                                               (int)n_rel, (int)cfg_.world, b.d_hid_h_lo, b.d_hid_t_lo, nullptr, nullptr, nullptr, DropoutParams{}, nullptr,
                                                               fuse_dense_ ? dense_ : nullptr, fuse_dense_ ? dense_m_ : nullptr, fuse_dense_ ? dense_v_ : nullptr,
                                                               dense_lr_mod_[0], b.loss_rows, (int)B, 1.0f / normaliser, d_loss_total_ + l, d_loss_last_ + l,
                                                               d_reg_loss_ ? d_reg_loss_ + 2 * l : nullptr}, l, step);
        const dim3 grid(kHeavySlots + ceil_div(R, kRowsPerBlock) + n_rel + 1), block(64 * kSegmentLanes);  // + the loss block
#define KGE_ENTITY_UPDATE(ST_, EXTRAS_)                                                                                                          \
    KGE_LAUNCH("entity_update", KGE_CUDA(launch_dependent(k_entity_update<ST_, 4, EXTRAS_>, grid, block, 0, stream_, b.table, b.rows_c2[parity], layout_, \
                                         step_ptr(d_remote_, l, R), d_ent_perm_ + sidx * (B + T), d_ent_off_ + sidx * (R + 1), d_first_slot_ + sidx * R,      \
                                         b.d_head, b.grad_recv, (int)B, b.d_hid_h, b.d_hid_t, d_step_size_ + step, entity_lr_mod_, adam_, sync, heavy,       \
                                         (int)R, rr)))
        const bool extras = cfg_.regularised() || dropout_on() || mlp_on();
        if (cfg_.state_type == ST_F32) {
            if (extras) KGE_ENTITY_UPDATE(float, true); else KGE_ENTITY_UPDATE(float, false);
        } else {
            if (extras) KGE_ENTITY_UPDATE(__half, true); else KGE_ENTITY_UPDATE(__half, false);
        }
#undef KGE_ENTITY_UPDATE
    }
    KGE_CUDA(cudaGetLastError());
    const bool gather_ahead = step + 1 < cfg_.n_step;
    const bool gather_beside = gather_ahead && (side_streams_ & 2u);
    if (gather_beside) {
        cudaStream_t side = side_begin();
        launch_gather(step + 1, side);
        side_end(1);
    }
    // 6. d W = feature^T . d_hidden, straight into the owners' slices of the partial dense gradient
    for (unsigned l = 0; l < n_local_; ++l) {
        ShardBuffers& b = shards_[l];
        tc::PlaneProblem nets[2] = {};
        for (unsigned net = 0; net < cfg_.n_net(); ++net) {
            tc::PlaneProblem& p = nets[net];
            p.A = features(b, true);
            p.B = plane(net ? b.d_hid_t : b.d_hid_h, net ? b.d_hid_t_lo : b.d_hid_h_lo, (long long)D * 4, true);
            tc::GemmArgs& g = p.g;
            g.M = (int)F; g.N = (int)D; g.K = (int)R;
            g.epilogue = tc::EPI_STORE;
            g.out = nullptr; g.out_blocks = b.dense_dst; g.block_rows = 1; g.block_cyclic = (int)cfg_.world;
            g.block_row_offset = (int)(n_rel + net * F); g.ldc = D;
            if (fuse_dense_) {
                // one shard in all: this gradient is the whole gradient, and the epilogue is the projection's Adam step
                g.epilogue = tc::EPI_DENSE_ADAM;
                g.out_blocks = nullptr;
                g.x_base = reinterpret_cast<const uint8_t*>(dense_ + dense_bounds_[1 + net]);
                g.x_row_stride_bytes = (long long)D * 4;
                g.adam = tc::DenseAdamArgs{dense_, dense_lo_, dense_m_, dense_v_, d_step_size_ + step, dense_lr_mod_[1 + net], adam_.beta_m, adam_.beta_v,
                                           adam_.one_minus_beta_m, adam_.one_minus_beta_v, adam_.epsilon, adam_.weight_decay};
            }
        }
        if (F > 0) launch_planes("projection_bwd", nets, (int)cfg_.n_net(), tc::SIDE_NONE, -1, XCHG_DENSE_PARTIALS);
        else launch_exchange_signal(XCHG_DENSE_PARTIALS);  // the relation rows of the entity update are all there is
    }
    KGE_CUDA(cudaGetLastError());
    if (gather_ahead && !gather_beside) launch_gather(step + 1, stream_);
    // 7. dense parameters: reduce over shards, Adam on the owned rows, new values and their lower planes into every replica
    if (!fuse_dense_) {
        DenseUpdateArgs da{};
        da.sync = sync;
        da.partials = d_partials_;
        da.n_partial = (int)cfg_.n_shard;
        da.replicas = d_replicas_;
        da.replicas_lo = d_replicas_lo_;
        da.n_replica = (int)cfg_.world;
        da.adam_m = dense_m_;
        da.adam_v = dense_v_;
        da.n_own = own_rows_;
        da.row_width = D;
        for (int i = 0; i <= kDenseParams; ++i) da.bounds[i] = dense_bounds_[i];
        for (int i = 0; i < kDenseParams; ++i) da.lr_modifier[i] = dense_lr_mod_[i];
        da.step_size = d_step_size_ + step;
        da.ap = adam_;
        const unsigned blocks = (unsigned)std::min<size_t>((own_rows_ * D / 4 + 255) / 256, 148 * 8);
        KGE_LAUNCH("dense_update", KGE_CUDA(launch_dependent(k_dense_update, dim3(std::max(1u, blocks)), dim3(256), 0, stream_, da, (int)cfg_.rank)));
    }
    KGE_CUDA(cudaGetLastError());
    if (gather_beside) side_join(1);
}

void Engine::launch_one_step(unsigned step) {
    const unsigned B = cfg_.batch_size, T = cfg_.n_tail(), R = cfg_.n_remote(), D = cfg_.d, F = cfg_.f;
    const unsigned n_rel = cfg_.n_relation_type;
    const bool two_nets = cfg_.n_net() == 2;
    const bool vec = (D % 4) == 0;
    const float* rel_table = dense_;
    const float* W0 = cfg_.n_net() >= 1 ? dense_ + dense_bounds_[1] : nullptr;
    const float* W1 = two_nets ? dense_ + dense_bounds_[2] : W0;
    const bool transh = cfg_.score_fn == SCORE_TRANSH;
    const float* normal_table = dense_ + dense_bounds_[3];

    LossParams lp{};
    lp.loss_fn = cfg_.loss_fn;
    lp.score_fn = cfg_.score_fn;
    lp.dist_fn = cfg_.dist_fn;
    lp.n_tail = (int)T;
    lp.gamma = cfg_.gamma;
    lp.adversarial_scale = cfg_.adversarial_scale;
    lp.w_neg = (0.5f * (float)T) / (float)(T - 1);
    lp.w_pos = 0.5f * (float)T;
    float normaliser;
    if (cfg_.loss_fn == LOSS_LOGSIGMOID) {
        normaliser = (float)(cfg_.n_shard * B * cfg_.a2a_size * cfg_.n_shard);
        lp.softmax_shift = 0.f;
    } else {
        normaliser = (float)(cfg_.n_shard * B);
        const float correction = (float)(std::log((double)(cfg_.n_entity * cfg_.n_shard - 1)) -
                                         std::log((double)(cfg_.n_shard * cfg_.a2a_size - 1)));
        lp.softmax_shift = cfg_.correction_weight != 0.f ? cfg_.correction_weight * correction : 0.f;
    }
    lp.grad_scale = cfg_.loss_scale / normaliser;

    if (planes_) return launch_step_planes(step, lp, normaliser);
    const ExchangeSync sync = exchange_sync();
    const bool proj_direct = cfg_.tensor_cores && F > 0;  // the projection gradient lands in the partial dense vector directly
    auto step_ptr = [&](uint32_t* base, unsigned l, size_t per_step) {
        return base + ((size_t)l * cfg_.n_step + step) * per_step;
    };

    // 1./2. hidden rows, lookups, send half of the exchange
    for (unsigned l = 0; l < n_local_; ++l) {
        ShardBuffers& b = shards_[l];
        uint8_t* rows_c = b.rows_c2[step & 1];
        if (cfg_.tensor_cores && F > 0) {
            // hidden = value + feature . W on the tensor cores: A = gathered feature rows, B = W stored [F, D]
            tc::GemmArgs nets[2] = {};
            const int n_nets = two_nets ? 2 : 1;
            for (int net = 0; net < n_nets; ++net) {
                tc::GemmArgs& g = nets[net];
                g.A = tc::make_operand(rows_c + layout_.off_feat, layout_.row_bytes, cfg_.feature_type == ST_F16, false);
                g.B = tc::make_operand(net ? W1 : W0, (long long)D * 4, false, true);
                g.M = (int)R; g.N = (int)D; g.K = (int)F; g.k_per_split = (int)round_up(F, 32);
                g.epilogue = tc::EPI_ADD_TABLE_VALUE;
                g.out = net ? b.hid_t : b.hid_h; g.ldc = D; g.block_rows = 1;
                g.x_base = rows_c; g.x_row_stride_bytes = layout_.row_bytes; g.x_gather = nullptr;
                g.x_is_half = cfg_.value_bf16 ? 2 : (cfg_.state_type == ST_F16 ? 1 : 0);
            }
            // the projection was updated by the processes that own its slices
            launch_tc("hidden", nets, n_nets, tc_splits(n_nets * ceil_div(R, 128) * ceil_div(D, 64), F), cfg_.feature_type == ST_F16, false,
                      XCHG_DENSE_PARAMS, -1);
        } else {
            launch_exchange_wait(XCHG_DENSE_PARAMS);
            dim3 grid(ceil_div(R, 64), ceil_div(D, 64), two_nets ? 2 : 1);
            KGE_LAUNCH("hidden", KGE_DISPATCH_ROW(cfg_, KGE_CUDA(launch_dependent(k_hidden<ST, FT>, dim3(grid), dim3(256), 0, stream_, 
                                                            rows_c, layout_, nullptr, 0u, (int)R, W0, W1, b.hid_h, b.hid_t))));
        }
        const uint32_t* a2a = step_ptr(d_a2a_, l, T);
        const uint32_t* head = step_ptr(d_head_, l, B);
        const uint32_t* relation = step_ptr(d_relation_, l, B);
        if (mlp_on())
            for (unsigned net = 0; net < cfg_.n_net(); ++net)
                launch_mlp_forward(rows_c, nullptr, 0u, R, (int)net, net ? b.hid_t : b.hid_h, b.mlp_cat[net], b.mlp_pre[net], b.mlp_out);
        if (dropout_on()) launch_dropout(l, step, rows_c);
        const int route_fn = transh ? SCORE_TRANSE : cfg_.score_fn;  // TransH: the tails are routed, the prediction follows
        if (vec)
            KGE_LAUNCH("route", KGE_CUDA(launch_dependent(k_route<4>, dim3(T + B), dim3(64), 0, stream_, b.hid_h, b.hid_t, a2a, head, relation, rel_table,
                                                                      b.send_dst, b.pred, (int)T, (int)cfg_.a2a_size,
                                                                      (int)B, (int)D, route_fn, sync, (float* const*)nullptr, (float*)nullptr, 0)));
        else
            KGE_LAUNCH("route", KGE_CUDA(launch_dependent(k_route<1>, dim3(T + B), dim3(64), 0, stream_, b.hid_h, b.hid_t, a2a, head, relation, rel_table,
                                                                      b.send_dst, b.pred, (int)T, (int)cfg_.a2a_size,
                                                                      (int)B, (int)D, route_fn, sync, (float* const*)nullptr, (float*)nullptr, 0)));
        if (transh)
            KGE_LAUNCH("transh_predict", KGE_CUDA(launch_dependent(k_transh_predict, dim3(B), dim3(64), 0, stream_, b.hid_h, head, relation, rel_table,
                                                                   normal_table, b.pred, b.nrm, (int)D)));
        if (cfg_.regularised()) launch_regularise(l, rows_c);
    }
    KGE_CUDA(cudaGetLastError());

    // 3./4./5a. scores, loss, score backward with the return half of the exchange
    for (unsigned l = 0; l < n_local_; ++l) {
        ShardBuffers& b = shards_[l];
        const uint32_t* head = step_ptr(d_head_, l, B);
        const uint32_t* relation = step_ptr(d_relation_, l, B);
        const uint32_t* tail = step_ptr(d_tail_, l, B);
        PairBwdArgs pa{};
        pa.D = (int)D;
        pa.tiles_m0 = (int)ceil_div(B, 32);
        pa.p[0] = {b.pred, b.tails, b.coeff, (int)B, (int)T, (int)T, 1, b.d_pred, nullptr, 1};
        pa.p[1] = {b.tails, b.pred, b.coeff, (int)T, (int)B, 1, (int)T, nullptr, b.grad_dst, (int)cfg_.a2a_size};
        dim3 bgrid(ceil_div(B, 32) + ceil_div(T, 32), ceil_div(D, 64));
        const bool tc_score = cfg_.tensor_cores && cfg_.dist_fn == DIST_DOT;
        const bool tc_bwd = cfg_.tensor_cores && cfg_.dist_fn != DIST_L1;
        if (transh) {
            const dim3 grid(ceil_div(B, kTranshRows), std::max(1u, std::min(ceil_div(T, 8), 2 * 148 / std::max(1u, ceil_div(B, kTranshRows)))));
            KGE_LAUNCH("score", KGE_CUDA(launch_dependent(k_transh_score, grid, dim3(256), transh_score_smem(), stream_, b.pred, b.nrm, b.tails, b.raw,
                                                          b.pair_s, b.pair_u, (int)B, (int)T, (int)D, sync)));
        } else if (tc_score) {
            tc::GemmArgs g{};
            g.A = tc::make_operand(b.pred, (long long)D * 4, false, false);
            g.B = tc::make_operand(b.tails, (long long)D * 4, false, false);
            g.M = (int)B; g.N = (int)T; g.K = (int)D; g.k_per_split = (int)round_up(D, 32);
            g.epilogue = tc::EPI_STORE; g.out = b.raw; g.ldc = T; g.block_rows = 1;
            launch_tc("score", &g, 1, tc_splits(ceil_div(B, 128) * ceil_div(T, 64), D), false, false, XCHG_TAILS, -1);
        } else {
            // the tail rows come from the other processes: the 16-byte-copy kernel waits for them itself
            const bool fused_wait = score_rows_aligned(b.pred, b.tails, (int)D);
            if (!fused_wait) launch_exchange_wait(XCHG_TAILS);
            KGE_LAUNCH("score", KGE_CUDA(launch_score(cfg_.dist_fn, b.pred, b.tails, b.raw, (int)B, (int)T, (int)D, stream_,
                                                      fused_wait ? sync : ExchangeSync{})));
        }
        KGE_LAUNCH("loss", KGE_CUDA(launch_loss(b.raw, tail, b.coeff, b.loss_rows, lp, 1.0f / normaliser, d_loss_total_ + l, d_loss_last_ + l,
                                                d_loss_counter_ + l, nullptr, 0, (int)B, stream_, d_reg_loss_ ? d_reg_loss_ + 2 * l : nullptr)));
        if (tc_bwd) {
            // Both input gradients are contractions with the coefficient matrix C [B, T]:
            //   dot:  d_pred = C . tails,                          d_tails = C^T . pred
            //   L2:   d_pred = rowsum(C) * pred - C . tails,       d_tails = colsum(C) * tails - C^T . pred
            // (sum_j C_ij (p_i - t_j) written out; C already holds gradient / distance).
            const bool l2 = cfg_.dist_fn == DIST_L2;
            tc::GemmArgs both[2] = {};
            tc::GemmArgs& g = both[0];
            g.A = tc::make_operand(b.coeff, (long long)T * 4, false, false);
            g.B = tc::make_operand(b.tails, (long long)D * 4, false, true);
            g.M = (int)B; g.N = (int)D; g.K = (int)T; g.k_per_split = (int)round_up(T, 32);
            g.epilogue = l2 ? tc::EPI_ROWSUM_X_MINUS : tc::EPI_STORE;
            g.out = b.d_pred; g.ldc = D; g.block_rows = 1;
            g.x_base = reinterpret_cast<const uint8_t*>(b.pred); g.x_row_stride_bytes = (long long)D * 4;
            tc::GemmArgs& h = both[1];
            h.A = tc::make_operand(b.coeff, (long long)T * 4, false, true);
            h.B = tc::make_operand(b.pred, (long long)D * 4, false, true);
            h.M = (int)T; h.N = (int)D; h.K = (int)B; h.k_per_split = (int)round_up(std::max(B, T), 32);
            h.epilogue = l2 ? tc::EPI_ROWSUM_X_MINUS : tc::EPI_STORE;
            h.out = nullptr; h.out_blocks = b.grad_dst; h.block_rows = (int)cfg_.a2a_size; h.ldc = D;
            h.x_base = reinterpret_cast<const uint8_t*>(b.tails); h.x_row_stride_bytes = (long long)D * 4;
            g.k_per_split = h.k_per_split;
            launch_tc("score_bwd", both, 2, tc_splits((ceil_div(B, 128) + ceil_div(T, 128)) * ceil_div(D, 64), std::min(B, T)), false, l2,
                      -1, XCHG_TAIL_GRADS);
        } else if (transh) {
            KGE_LAUNCH("score_bwd", KGE_CUDA(launch_dependent(k_transh_bwd, dim3(B + T), dim3(128), 0, stream_, b.pred, b.nrm, b.tails, b.coeff, b.pair_s,
                                                              b.pair_u, b.d_pred, b.d_nrm, b.grad_dst, (int)cfg_.a2a_size, (int)B, (int)T, (int)D)));
            launch_exchange_signal(XCHG_TAIL_GRADS);
        } else {
        switch (cfg_.dist_fn) {
            case DIST_L1: KGE_LAUNCH("score_bwd", KGE_CUDA(launch_dependent(k_pair_bwd<DIST_L1>, dim3(bgrid), dim3(128), 0, stream_, pa))); break;
            case DIST_L2: KGE_LAUNCH("score_bwd", KGE_CUDA(launch_dependent(k_pair_bwd<DIST_L2>, dim3(bgrid), dim3(128), 0, stream_, pa))); break;
            default: KGE_LAUNCH("score_bwd", KGE_CUDA(launch_dependent(k_pair_bwd<DIST_DOT>, dim3(bgrid), dim3(128), 0, stream_, pa))); break;
        }
        launch_exchange_signal(XCHG_TAIL_GRADS);
        }
        if (transh) {
            KGE_LAUNCH("pred_bwd", KGE_CUDA(launch_dependent(k_transh_pred_bwd, dim3(B), dim3(64), 0, stream_, b.d_pred, b.d_nrm, b.hid_h, head, relation,
                                                             normal_table, b.nrm, b.d_head, b.d_relrow, b.d_normrow, (int)D)));
            // the normals' rows of the partial dense gradient, behind the relation table and the projections
            const size_t sidx = (size_t)l * cfg_.n_step + step;
            const int normal_row0 = (int)(n_rel + cfg_.n_net() * F);
            if (vec)
                KGE_LAUNCH("dense_partial", KGE_CUDA(launch_dependent(k_dense_partial<4>, dim3(n_rel), dim3(64 * kRelationLanes), 0, stream_,
                                                b.d_normrow, d_rel_perm_ + sidx * B, d_rel_off_ + sidx * (n_rel + 1), (int)n_rel,
                                                (int)D, b.proj_partial, 0, 1, proj_elems_, b.dense_dst, (int)cfg_.world, sync, -1, normal_row0)));
            else
                KGE_LAUNCH("dense_partial", KGE_CUDA(launch_dependent(k_dense_partial<1>, dim3(n_rel), dim3(64 * kRelationLanes), 0, stream_,
                                                b.d_normrow, d_rel_perm_ + sidx * B, d_rel_off_ + sidx * (n_rel + 1), (int)n_rel,
                                                (int)D, b.proj_partial, 0, 1, proj_elems_, b.dense_dst, (int)cfg_.world, sync, -1, normal_row0)));
        } else if (cfg_.score_fn != SCORE_TRANSE)
            KGE_LAUNCH("pred_bwd", KGE_CUDA(launch_dependent(k_pred_bwd, dim3(B), dim3(64), 0, stream_, b.d_pred, b.hid_h, head, relation, rel_table, b.d_head,
                                                                     b.d_relrow, (int)D, cfg_.score_fn)));
    }
    KGE_CUDA(cudaGetLastError());

    if (proj_direct) {
        // The relation gradients depend on the score backward only: they are summed beside the entity update.
        const unsigned saved = side_streams_;
        side_streams_ = saved & 1u;
        cudaStream_t side = side_begin();
        for (unsigned l = 0; l < n_local_; ++l) {
            ShardBuffers& b = shards_[l];
            const size_t sidx = (size_t)l * cfg_.n_step + step;
            if (vec)
                KGE_LAUNCH("dense_partial", KGE_CUDA(launch_dependent(k_dense_partial<4>, dim3(n_rel), dim3(64 * kRelationLanes), 0, side,
                                                b.d_relrow, d_rel_perm_ + sidx * B, d_rel_off_ + sidx * (n_rel + 1), (int)n_rel,
                                                (int)D, b.proj_partial, 0, 1, proj_elems_, b.dense_dst, (int)cfg_.world, sync, -1, 0)));
            else
                KGE_LAUNCH("dense_partial", KGE_CUDA(launch_dependent(k_dense_partial<1>, dim3(n_rel), dim3(64 * kRelationLanes), 0, side,
                                                b.d_relrow, d_rel_perm_ + sidx * B, d_rel_off_ + sidx * (n_rel + 1), (int)n_rel,
                                                (int)D, b.proj_partial, 0, 1, proj_elems_, b.dense_dst, (int)cfg_.world, sync, -1, 0)));
        }
        side_end(0);
        side_streams_ = saved;
    }

    // 5b. segment sums + row-wise Adam; projection and relation gradients of this shard
    for (unsigned l = 0; l < n_local_; ++l) {
        ShardBuffers& b = shards_[l];
        uint8_t* rows_c = b.rows_c2[step & 1];
        const size_t sidx = (size_t)l * cfg_.n_step + step;
        const uint32_t* remote = step_ptr(d_remote_, l, R);
        const uint32_t* perm = d_ent_perm_ + sidx * (B + T);
        const uint32_t* off = d_ent_off_ + sidx * (R + 1);
        const uint32_t* first = d_first_slot_ + sidx * R;
        const float* alpha = d_step_size_ + step;
        const HeavyRows heavy{d_heavy_parts_ + sidx * kHeavySlots, d_heavy_count_ + sidx, b.heavy_partial, b.heavy_counter, d_row_info_ + sidx * 2 * R};
#define KGE_ENTITY_UPDATE(ST_, V_, EXTRAS_)                                                                                                              \
    KGE_LAUNCH("entity_update", KGE_CUDA(launch_dependent(k_entity_update<ST_, V_, EXTRAS_>, dim3(ceil_div(R, kRowsPerBlock) + kHeavySlots), dim3(64 * kSegmentLanes), \
                                         0, stream_, b.table, rows_c, layout_, remote, perm, off, first, b.d_head, b.grad_recv, (int)B, b.d_hid_h, b.d_hid_t, alpha,  \
                                         entity_lr_mod_, adam_, sync, heavy, (int)R, with_regularisers(RelationRows{}, l, step))))
        const bool extras = cfg_.regularised() || dropout_on() || mlp_on();
        if (cfg_.state_type == ST_F32) {
            if (vec) { if (extras) KGE_ENTITY_UPDATE(float, 4, true); else KGE_ENTITY_UPDATE(float, 4, false); }
            else { if (extras) KGE_ENTITY_UPDATE(float, 1, true); else KGE_ENTITY_UPDATE(float, 1, false); }
        } else {
            if (vec) { if (extras) KGE_ENTITY_UPDATE(__half, 4, true); else KGE_ENTITY_UPDATE(__half, 4, false); }
            else { if (extras) KGE_ENTITY_UPDATE(__half, 1, true); else KGE_ENTITY_UPDATE(__half, 1, false); }
        }
#undef KGE_ENTITY_UPDATE
    }
    KGE_CUDA(cudaGetLastError());
    if (mlp_on())
        for (unsigned l = 0; l < n_local_; ++l) launch_mlp_backward(l, step);
    if (proj_direct && (side_streams_ & 1u)) side_join(0);  // the relation rows of the partial dense gradient are in place
    const bool gather_ahead = step + 1 < cfg_.n_step;
    const bool gather_beside = gather_ahead && (side_streams_ & 2u);
    if (gather_beside) {
        // the next step's rows: needs only the rows just updated, runs beside the rest of this step
        cudaStream_t side = side_begin();
        launch_gather(step + 1, side);
        side_end(1);
    }
    for (unsigned l = 0; l < n_local_; ++l) {
        ShardBuffers& b = shards_[l];
        uint8_t* rows_c = b.rows_c2[step & 1];
        const size_t sidx = (size_t)l * cfg_.n_step + step;
        if (F > 0 && cfg_.tensor_cores) {
            // d W = feature^T . d_hidden: the gathered rows are the k index of both operands
            tc::GemmArgs nets[2] = {};
            for (unsigned net = 0; net < cfg_.n_net(); ++net) {
                tc::GemmArgs& g = nets[net];
                g.A = tc::make_operand(rows_c + layout_.off_feat, layout_.row_bytes, cfg_.feature_type == ST_F16, true);
                g.B = tc::make_operand(net ? b.d_hid_t : b.d_hid_h, (long long)D * 4, false, true);
                g.M = (int)F; g.N = (int)D; g.K = (int)R; g.k_per_split = proj_rows_per_split_;
                g.epilogue = tc::EPI_STORE;
                // straight into this shard's partial dense gradient, behind the relation rows: row m of
                // the projection is row n_rel + net * F + m of the dense vector, and goes to its owner
                g.out = nullptr; g.out_blocks = b.dense_dst; g.block_rows = 1; g.block_cyclic = (int)cfg_.world;
                g.block_row_offset = (int)(n_rel + net * F); g.ldc = D;
            }
            launch_tc("projection_bwd", nets, (int)cfg_.n_net(),
                      tc_splits(cfg_.n_net() * ceil_div(F, 128) * ceil_div(D, 64), R), cfg_.feature_type == ST_F16, false,
                      -1, XCHG_DENSE_PARTIALS);
        } else if (F > 0) {
            dim3 grid(ceil_div(F, 64), ceil_div(D, 64), cfg_.n_net() * proj_splits_);
            const float* dh1 = two_nets ? b.d_hid_t : b.d_hid_h;
            if (cfg_.feature_type == ST_F32)
                KGE_LAUNCH("projection_bwd", KGE_CUDA(launch_dependent(k_projection_bwd<float>, dim3(grid), dim3(256), 0, stream_, 
                                                 rows_c, layout_, nullptr, (int)R, b.d_hid_h, dh1, proj_splits_,
                                                 proj_rows_per_split_, b.proj_partial)));
            else
                KGE_LAUNCH("projection_bwd", KGE_CUDA(launch_dependent(k_projection_bwd<__half>, dim3(grid), dim3(256), 0, stream_, 
                                                 rows_c, layout_, nullptr, (int)R, b.d_hid_h, dh1, proj_splits_,
                                                 proj_rows_per_split_, b.proj_partial)));
        }
        if (!proj_direct) {
            // relation gradients and the sum of the projection gradient's row splits; completes the partial dense gradient
            const size_t proj_total = (size_t)cfg_.n_net() * proj_elems_;
            const unsigned proj_blocks = proj_total ? (unsigned)std::min<size_t>((proj_total + 511) / 512, 148 * 4) : 0;
            if (vec)
                KGE_LAUNCH("dense_partial", KGE_CUDA(launch_dependent(k_dense_partial<4>, dim3(n_rel + proj_blocks), dim3(64 * kRelationLanes), 0, stream_,
                                                b.d_relrow, d_rel_perm_ + sidx * B, d_rel_off_ + sidx * (n_rel + 1), (int)n_rel,
                                                (int)D, b.proj_partial, (int)cfg_.n_net(), proj_splits_,
                                                proj_elems_, b.dense_dst, (int)cfg_.world, sync, (int)XCHG_DENSE_PARTIALS, 0)));
            else
                KGE_LAUNCH("dense_partial", KGE_CUDA(launch_dependent(k_dense_partial<1>, dim3(n_rel + proj_blocks), dim3(64 * kRelationLanes), 0, stream_,
                                                b.d_relrow, d_rel_perm_ + sidx * B, d_rel_off_ + sidx * (n_rel + 1), (int)n_rel,
                                                (int)D, b.proj_partial, (int)cfg_.n_net(), proj_splits_,
                                                proj_elems_, b.dense_dst, (int)cfg_.world, sync, (int)XCHG_DENSE_PARTIALS, 0)));
        }
    }
    KGE_CUDA(cudaGetLastError());
    if (gather_ahead && !gather_beside) launch_gather(step + 1, stream_);  // runs while the partial dense gradients travel

    // 5c. dense parameters: reduce over shards, Adam on the owned slice, publish.  Every process
    // launches it, also one that owns nothing, since the kernel carries two hand-overs.
    {
        DenseUpdateArgs da{};
        da.sync = sync;
        da.partials = d_partials_;
        da.n_partial = (int)cfg_.n_shard;
        da.replicas = d_replicas_;
        da.n_replica = (int)cfg_.world;
        da.adam_m = dense_m_;
        da.adam_v = dense_v_;
        da.n_own = own_rows_;
        da.row_width = D;
        for (int i = 0; i <= kDenseParams; ++i) da.bounds[i] = dense_bounds_[i];
        for (int i = 0; i < kDenseParams; ++i) da.lr_modifier[i] = dense_lr_mod_[i];
        da.step_size = d_step_size_ + step;
        da.ap = adam_;
        // The parameter itself is read from this process's own replica (entry `rank`).
        const unsigned blocks = (unsigned)std::min<size_t>((own_rows_ * D / (vec ? 4 : 1) + 255) / 256, 148 * 8);
        KGE_LAUNCH("dense_update", KGE_CUDA(launch_dependent(k_dense_update, dim3(std::max(1u, blocks)), dim3(256), 0, stream_, da, (int)cfg_.rank)));
    }
    KGE_CUDA(cudaGetLastError());
    if (gather_beside) side_join(1);
}

// ---------------------------------------------------------------------------
// Table and variable I/O

void Engine::cmd_read_entity(std::vector<HostArray>& arrays) {
    const size_t n = n_local_, rw = cfg_.rw_batch, W = cfg_.row_width();
    HostArray& idx = find_array(arrays, "read_indices", KGE_U32, {n, rw});
    const int out_dtype = cfg_.state_type == ST_F32 ? KGE_F32 : KGE_F16;
    HostArray& out = find_array(arrays, "read_data", out_dtype, {n, rw, W});
    const uint32_t* h = static_cast<const uint32_t*>(idx.data);
    for (size_t i = 0; i < n * rw; ++i)
        if (h[i] >= cfg_.n_entity)
            fail(KGE_INVALID_ARGUMENT, msg() << "'read_indices' holds index " << h[i] << ", not below model.n_entity ("
                                             << cfg_.n_entity << ")");
    KGE_CUDA(cudaStreamSynchronize(stream_));
    KGE_CUDA(cudaMemcpyAsync(d_rw_idx_, idx.data, n * rw * 4, cudaMemcpyHostToDevice, stream_));
    const size_t elem = out_dtype == KGE_F32 ? 4 : 2;
    for (unsigned l = 0; l < n; ++l) {
        const uint32_t* di = d_rw_idx_ + l * rw;
        void* dout = d_rw_data_ + l * rw * W * elem;
        if (out_dtype == KGE_F32) {
            KGE_DISPATCH_ROW(cfg_, k_read_rows<ST, FT, float><<<(unsigned)rw, 128, 0, stream_>>>(shards_[l].table, layout_, di,
                                                                                                 (float*)dout));
        } else {
            k_read_rows<__half, __half, __half><<<(unsigned)rw, 128, 0, stream_>>>(shards_[l].table, layout_, di, (__half*)dout);
        }
    }
    KGE_CUDA(cudaGetLastError());
    KGE_CUDA(cudaMemcpyAsync(out.data, d_rw_data_, n * rw * W * elem, cudaMemcpyDeviceToHost, stream_));
    KGE_CUDA(cudaStreamSynchronize(stream_));
}

// "dump_entity_rows" / "restore_entity_rows": a contiguous range of one local shard's table as it
// is stored (no type conversion, optimiser state included), for checkpoints of tables too large
// to pass through host arrays of the state type at once.  `shard_range` u32 [3] = (local shard,
// first row, row count); `rows` u32 [row count, row bytes / 4].  The reference reads and writes
// the table only through indexed chunks of rw_batch_size rows (src/poplar_kge.cpp:857-871;
// read_entity_all, src/python/poplar_kge.py:583-598); a stored range is one plain copy.
void Engine::cmd_copy_entity_range(std::vector<HostArray>& arrays, bool to_host) {
    HostArray& range = find_array(arrays, "shard_range", KGE_U32, {3});
    const uint32_t* r = static_cast<const uint32_t*>(range.data);
    const size_t shard = r[0], first = r[1], count = r[2];
    if (shard >= n_local_) fail(KGE_INVALID_ARGUMENT, msg() << "'shard_range' names local shard " << shard << " of " << n_local_);
    if (first + count > cfg_.n_entity)
        fail(KGE_INVALID_ARGUMENT, msg() << "'shard_range' covers rows [" << first << ", " << first + count
                                         << "), not within model.n_entity (" << cfg_.n_entity << ")");
    HostArray& rows = find_array(arrays, "rows", KGE_U32, {count, (size_t)layout_.row_bytes / 4});
    if (!count) return;
    unsigned char* table = shards_[shard].table + first * (size_t)layout_.row_bytes;
    const size_t bytes = count * (size_t)layout_.row_bytes;
    if (to_host)
        KGE_CUDA(cudaMemcpyAsync(rows.data, table, bytes, cudaMemcpyDeviceToHost, stream_));
    else
        KGE_CUDA(cudaMemcpyAsync(table, rows.data, bytes, cudaMemcpyHostToDevice, stream_));
    KGE_CUDA(cudaStreamSynchronize(stream_));
}

void Engine::cmd_write_entity(std::vector<HostArray>& arrays, bool whole_rows) {
    const size_t n = n_local_, rw = cfg_.rw_batch, W = cfg_.row_width(), F = cfg_.f;
    HostArray& idx = find_array(arrays, "write_indices", KGE_U32, {n, rw});
    const char* data_name = whole_rows ? "write_data" : "write_features";
    const std::vector<size_t> shape = {n, rw, whole_rows ? W : F};
    // The host array is in the state type (the reference's single dtype); a float16 array is
    // also taken for features when they are stored as float16.
    HostArray* data = nullptr;
    for (HostArray& a : arrays)
        if (a.name == data_name) data = &a;
    if (!data) fail(KGE_INVALID_ARGUMENT, msg() << "Key not found '" << data_name << "'");
    const int state_dtype = cfg_.state_type == ST_F32 ? KGE_F32 : KGE_F16;
    const bool f16_features_ok = !whole_rows && cfg_.feature_type == ST_F16 && data->dtype == KGE_F16;
    find_array(arrays, data_name, f16_features_ok ? KGE_F16 : state_dtype, shape);
    const uint32_t* h = static_cast<const uint32_t*>(idx.data);
    for (size_t i = 0; i < n * rw; ++i)
        if (h[i] >= cfg_.n_entity)
            fail(KGE_INVALID_ARGUMENT, msg() << "'write_indices' holds index " << h[i] << ", not below model.n_entity ("
                                             << cfg_.n_entity << ")");
    const size_t elem = data->dtype == KGE_F32 ? 4 : 2, per_row = shape[2];
    KGE_CUDA(cudaStreamSynchronize(stream_));
    KGE_CUDA(cudaMemcpyAsync(d_rw_idx_, idx.data, n * rw * 4, cudaMemcpyHostToDevice, stream_));
    KGE_CUDA(cudaMemcpyAsync(d_rw_data_, data->data, n * rw * per_row * elem, cudaMemcpyHostToDevice, stream_));
    const float stddev = cfg_.init_scale / (float)cfg_.d;  // src/poplar_kge.cpp:865
    for (unsigned l = 0; l < n; ++l) {
        const uint32_t* di = d_rw_idx_ + l * rw;
        const uint8_t* din = d_rw_data_ + l * rw * per_row * elem;
        uint8_t* table = shards_[l].table;
        const unsigned g = (unsigned)rw;
        if (data->dtype == KGE_F32) {
            using IT = float;
            if (whole_rows) KGE_DISPATCH_ROW(cfg_, k_write_rows<ST, FT, IT><<<g, 128, 0, stream_>>>(table, layout_, di, (int)rw, (const IT*)din));
            else KGE_DISPATCH_ROW(cfg_, k_write_entity<ST, FT, IT><<<g, 128, 0, stream_>>>(table, layout_, di, (int)rw, (const IT*)din, cfg_.seed, shard0_ + l, stddev));
        } else {
            using IT = __half;
            if (whole_rows) KGE_DISPATCH_ROW(cfg_, k_write_rows<ST, FT, IT><<<g, 128, 0, stream_>>>(table, layout_, di, (int)rw, (const IT*)din));
            else KGE_DISPATCH_ROW(cfg_, k_write_entity<ST, FT, IT><<<g, 128, 0, stream_>>>(table, layout_, di, (int)rw, (const IT*)din, cfg_.seed, shard0_ + l, stddev));
        }
    }
    KGE_CUDA(cudaGetLastError());
    KGE_CUDA(cudaStreamSynchronize(stream_));
}

void Engine::cmd_initialise_entities() {
    const float stddev = cfg_.init_scale / (float)cfg_.d;
    for (unsigned l = 0; l < n_local_; ++l) {
        KGE_DISPATCH_ROW(cfg_, k_init_table<ST, FT><<<148 * 8, 256, 0, stream_>>>(shards_[l].table, layout_, (size_t)cfg_.n_entity,
                                                                               cfg_.seed, shard0_ + l, stddev));
    }
    KGE_CUDA(cudaGetLastError());
    KGE_CUDA(cudaStreamSynchronize(stream_));
}

void Engine::cmd_read_write_variable(std::vector<HostArray>& arrays, const std::string& name, bool write) {
    const Variable* var = nullptr;
    for (const Variable& v : variables_)
        if (v.name == name) var = &v;
    if (!var) fail(KGE_INVALID_ARGUMENT, msg() << "Key not found '" << name << "'");
    HostArray& value = find_array(arrays, "value", var->dtype, var->shape);
    KGE_CUDA(cudaStreamSynchronize(stream_));
    if (var->kind == 3) {  // step: one counter, presented per shard
        uint32_t* p = static_cast<uint32_t*>(value.data);
        if (write) {
            for (unsigned s = 1; s < cfg_.n_shard; ++s)
                if (p[s] != p[0]) fail(KGE_INVALID_ARGUMENT, "'step' must hold the same value for every shard");
            step_ = p[0];
        } else {
            for (unsigned s = 0; s < cfg_.n_shard; ++s) p[s] = (uint32_t)step_;
        }
        return;
    }
    const size_t count = value.count();
    if (count == 0) return;
    float* base = var->kind == 0 ? dense_ : var->kind == 1 ? dense_m_ : dense_v_;
    // Rows of the dense vector are d floats wide; a variable may show fewer columns of them to the
    // host (RotatE's angles are the first half of their rows).
    const size_t D = cfg_.d, row0 = var->offset / D, W = cfg_.world;
    const size_t cols = var->flat ? D : var->shape[1], n_rows = var->flat ? count / D : var->shape[0];
    float* host = static_cast<float*>(value.data);
    if (write) {
        // on the engine's stream, so that the kernel that derives the lower plane is ordered behind the copy
        KGE_CUDA(cudaMemcpy2DAsync(base + var->offset, D * 4, host, cols * 4, cols * 4, n_rows, cudaMemcpyHostToDevice, stream_));
        if (var->kind == 0) refresh_lower_plane(var->offset, n_rows * D);
        KGE_CUDA(cudaStreamSynchronize(stream_));
        return;
    }
    if (var->kind == 0 || cfg_.world == 1) {
        KGE_CUDA(cudaMemcpy2D(host, cols * 4, base + var->offset, D * 4, cols * 4, n_rows, cudaMemcpyDeviceToHost));
        return;
    }
    // Optimiser state lives with the process that owns the row (src/poplar_kge.cpp:329-339): row r of
    // the dense vector with process r % world.  Collect each owner's rows through its mapped arena.
    for (size_t p = 0; p < W; ++p) {
        const size_t first = row0 + (p + W - row0 % W) % W;
        if (first >= row0 + n_rows) continue;
        const size_t rows = (row0 + n_rows - first + W - 1) / W;
        const float* src = (const float*)(peer_arena_[p] + arena_offset_dense(var->kind)) + first * D;
        KGE_CUDA(cudaMemcpy2D(host + (first - row0) * cols, W * cols * 4, src, W * D * 4, cols * 4, rows, cudaMemcpyDeviceToHost));
    }
}

// The projections are tensor-core operands: their lower TF32 plane follows every change of the values.
void Engine::refresh_lower_plane(size_t offset, size_t count) {
    if (!planes_ || count == 0) return;
    k_lower_plane<<<(unsigned)std::min<size_t>((count + 255) / 256, 148 * 8), 256, 0, stream_>>>(dense_ + offset, count, dense_lo_ + offset);
    KGE_CUDA(cudaGetLastError());
    KGE_CUDA(cudaStreamSynchronize(stream_));
}

void Engine::ensure_predict_buffers() {
    if (p_raw_) return;
    const size_t Q = (size_t)cfg_.n_shard * cfg_.predict_hr, D = cfg_.d;
    p_head_hidden_ = (float*)device_alloc((size_t)cfg_.predict_hr * D * 4);
    // L1 has no contraction form; everything else ranks with the plane-fed tensor-core kernel
    predict_planes_ = planes_ && cfg_.dist_fn != DIST_L1;
    // Rows per pass over the table.  On the tensor cores: 148 tiles of 128 rows, so that the hidden
    // rows' contraction (2 column tiles) and the scores' (10 query tiles at 1250 queries) both fill
    // whole waves of 148 blocks.
    predict_chunk_ = predict_planes_ ? 148u * 128u : 4096u;
    if (const char* v = std::getenv("KGE_PREDICT_PASS_ROWS")) predict_chunk_ = std::max(64u, (unsigned)std::atoi(v) / 4u * 4u);
    p_chunk_hidden_ = (float*)device_alloc((size_t)predict_chunk_ * D * 4);
    p_raw_ = (float*)device_alloc(Q * predict_chunk_ * 4);
    if (predict_planes_) {
        p_chunk_lo_ = (float*)device_alloc((size_t)predict_chunk_ * D * 4);
        p_query_lo_ = (float*)device_alloc(Q * D * 4);
        if (cfg_.f) p_feat_ = (float*)device_alloc((size_t)predict_chunk_ * feat_stride_ * 4);
    }
    if (mlp_on()) {
        const size_t rows = std::max<size_t>(cfg_.predict_hr, predict_chunk_);
        p_mlp_cat_ = (float*)device_alloc(rows * 2 * D * 4);
        p_mlp_pre_ = (float*)device_alloc(rows * cfg_.mlp * 4);
        p_mlp_out_ = (float*)device_alloc(rows * D * 4);
    }
    p_cand_ = (unsigned long long*)device_alloc(Q * kTopkCandidates * sizeof(unsigned long long));
    p_cand_count_ = (int*)device_alloc(Q * sizeof(int));
    KGE_CUDA(cudaMemset(p_cand_count_, 0, Q * sizeof(int)));
    d_iota_ = (uint32_t*)device_alloc((size_t)cfg_.predict_hr * 4);
    std::vector<uint32_t> iota(cfg_.predict_hr);
    for (unsigned i = 0; i < cfg_.predict_hr; ++i) iota[i] = i;
    KGE_CUDA(cudaMemcpy(d_iota_, iota.data(), iota.size() * 4, cudaMemcpyHostToDevice));
    for (ShardBuffers& b : shards_) {
        b.topk_state = (unsigned long long*)device_alloc(Q * kTopkCapacity * sizeof(unsigned long long));
        b.topk_count = (int*)device_alloc(Q * sizeof(int));
    }
}

// Merges the scores of rows start .. start + c - 1 (in p_raw_) into every query's best list: the filter at
// full bandwidth, then one warp per query on what it left.
void Engine::launch_topk(ShardBuffers& b, unsigned c, uint32_t start, uint32_t last, const TopkParams& tp, bool filtered) {
    const unsigned Q = (unsigned)tp.n_query;
    const dim3 fgrid(std::max(1u, std::min(ceil_div(c, 4 * 256), 8u)), Q);
    if (!filtered)  // else the score kernel's epilogue has left the candidates
        KGE_LAUNCH("predict_topk", k_topk_filter<<<fgrid, 256, 0, stream_>>>(p_raw_, (int)c, start, last, b.topk_state, b.topk_count, p_cand_, p_cand_count_, tp));
    KGE_LAUNCH("predict_topk", k_topk_update<<<ceil_div(Q, 4), 128, 0, stream_>>>(p_raw_, (int)c, start, last, b.topk_state, b.topk_count, tp, p_cand_,
                                                                                 p_cand_count_));
}

// Ranks every real row of the local shards as a tail for the queries of all shards
// (src/poplar_kge.cpp:812-855): predicted tails of the local queries are written into every
// process's query buffer (the all-gather of :825-828); each local shard then streams its table in
// batches, scores them and keeps the n_best per query; the results go back to the asking shard's
// process (the two all-to-alls of :847-850).
void Engine::cmd_predict(std::vector<HostArray>& arrays) {
    const size_t n = n_local_, hr = cfg_.predict_hr, nb = cfg_.predict_n_best, D = cfg_.d;
    const size_t Q = (size_t)cfg_.n_shard * hr;
    HostArray& head = find_array(arrays, "predict_head", KGE_U32, {n, hr});
    HostArray& relation = find_array(arrays, "predict_relation", KGE_U32, {n, hr});
    HostArray& count = find_array(arrays, "predict_entity_count", KGE_U32, {n});
    HostArray& scores = find_array(arrays, "predict_scores", KGE_F32, {n, cfg_.n_shard, hr, nb});
    HostArray& indices = find_array(arrays, "predict_indices", KGE_U32, {n, cfg_.n_shard, hr, nb});
    if (nb == 0 || nb > kTopkCapacity / 2)
        fail(KGE_INVALID_ARGUMENT, msg() << "'execution.predict_n_best' must be between 1 and " << kTopkCapacity / 2);
    if (!connected_) fail(KGE_LOGIC_ERROR, "world_size > 1 but kge_comm_connect has not been called");
    require_usable();
    const uint32_t* h_head = static_cast<const uint32_t*>(head.data);
    const uint32_t* h_rel = static_cast<const uint32_t*>(relation.data);
    const uint32_t* h_count = static_cast<const uint32_t*>(count.data);
    for (size_t i = 0; i < n * hr; ++i) {
        if (h_head[i] >= cfg_.n_entity)
            fail(KGE_INVALID_ARGUMENT, msg() << "'predict_head' holds index " << h_head[i] << ", not below model.n_entity (" << cfg_.n_entity << ")");
        if (h_rel[i] >= cfg_.n_relation_type)
            fail(KGE_INVALID_ARGUMENT, msg() << "'predict_relation' holds index " << h_rel[i] << ", not below model.n_relation_type (" << cfg_.n_relation_type << ")");
    }
    for (size_t l = 0; l < n; ++l)
        if (h_count[l] >= cfg_.n_entity)
            fail(KGE_INVALID_ARGUMENT, msg() << "'predict_entity_count' (" << h_count[l] << ") must be below model.n_entity (" << cfg_.n_entity << ")");
    ensure_predict_buffers();
    KGE_CUDA(cudaStreamSynchronize(stream_));
    uint32_t* d_head = d_rw_idx_;
    uint32_t* d_rel = d_rw_idx_ + n * hr;
    KGE_CUDA(cudaMemcpyAsync(d_head, h_head, n * hr * 4, cudaMemcpyHostToDevice, stream_));
    KGE_CUDA(cudaMemcpyAsync(d_rel, h_rel, n * hr * 4, cudaMemcpyHostToDevice, stream_));

    const bool two_nets = cfg_.n_net() == 2, vec = (D % 4) == 0;
    const float* W_head = cfg_.n_net() >= 1 ? dense_ + dense_bounds_[1] : nullptr;
    const float* W_tail = two_nets ? dense_ + dense_bounds_[2] : W_head;
    const unsigned dtiles = ceil_div((unsigned)D, 64);
    launch_counter_ = 0;

    // 1. predicted tails of the local queries, written into every process's gathered query buffer
    for (unsigned l = 0; l < n; ++l) {
        dim3 grid(ceil_div((unsigned)hr, 64), dtiles, 1);
        KGE_LAUNCH("predict_hidden", KGE_DISPATCH_ROW(cfg_, k_hidden<ST, FT><<<grid, 256, 0, stream_>>>(
                                                                shards_[l].table, layout_, d_head + l * hr, 0u, (int)hr, W_head,
                                                                nullptr, p_head_hidden_, nullptr)));
        if (mlp_on()) launch_mlp_forward(shards_[l].table, d_head + l * hr, 0u, (unsigned)hr, 0, p_head_hidden_, p_mlp_cat_, p_mlp_pre_, p_mlp_out_);
        for (unsigned p = 0; p < cfg_.world; ++p) {
            float* dst = (float*)(peer_arena_[p] + arena_offset_predict(0)) + (size_t)(shard0_ + l) * hr * D;
            if (cfg_.score_fn == SCORE_TRANSH) {
                KGE_LAUNCH("predict_query", k_transh_predict<<<(unsigned)hr, 64, 0, stream_>>>(
                                                p_head_hidden_, d_iota_, d_rel + l * hr, dense_, dense_ + dense_bounds_[3], dst, dst + Q * D, (int)D));
                continue;
            }
            if (vec)
                KGE_LAUNCH("predict_query", k_route<4><<<(unsigned)hr, 64, 0, stream_>>>(
                                                p_head_hidden_, p_head_hidden_, nullptr, d_iota_, d_rel + l * hr, dense_, nullptr,
                                                dst, 0, 1, (int)hr, (int)D, cfg_.score_fn, ExchangeSync{}));
            else
                KGE_LAUNCH("predict_query", k_route<1><<<(unsigned)hr, 64, 0, stream_>>>(
                                                p_head_hidden_, p_head_hidden_, nullptr, d_iota_, d_rel + l * hr, dense_, nullptr,
                                                dst, 0, 1, (int)hr, (int)D, cfg_.score_fn, ExchangeSync{}));
        }
    }
    KGE_CUDA(cudaGetLastError());
    launch_barrier();

    // 2. stream each local shard's rows past all queries
    const float* queries = (const float*)(arena_ + arena_offset_predict(0));
    if (predict_planes_) {
        KGE_LAUNCH("predict_planes", k_lower_plane<<<(unsigned)std::min<size_t>((Q * D + 255) / 256, 148 * 8), 256, 0, stream_>>>(queries, Q * D, p_query_lo_));
    }
    TopkParams tp{(int)Q, (int)nb, score_is_gamma_minus_distance(cfg_.score_fn) ? 1 : 0, cfg_.gamma};
    for (unsigned l = 0; l < n; ++l) {
        ShardBuffers& b = shards_[l];
        KGE_CUDA(cudaMemsetAsync(b.topk_count, 0, Q * sizeof(int), stream_));
        const uint32_t last = h_count[l];
        for (uint32_t start = 1; start <= last; start += predict_chunk_) {
            const unsigned c = std::min<uint32_t>(predict_chunk_, last - start + 1);
            if (predict_planes_) {
                const bool filtered = predict_pass_planes(b, start, c, last, tp, queries, (unsigned)Q, W_tail == W_head ? 0 : 1);
                launch_topk(b, c, start, last, tp, filtered);
                continue;
            }
            dim3 hgrid(ceil_div(c, 64), dtiles, 1);
            KGE_LAUNCH("predict_hidden", KGE_DISPATCH_ROW(cfg_, k_hidden<ST, FT><<<hgrid, 256, 0, stream_>>>(
                                                                    b.table, layout_, nullptr, start, (int)c, W_tail, nullptr,
                                                                    p_chunk_hidden_, nullptr)));
            if (mlp_on()) launch_mlp_forward(b.table, nullptr, start, c, two_nets ? 1 : 0, p_chunk_hidden_, p_mlp_cat_, p_mlp_pre_, p_mlp_out_);
            if (cfg_.score_fn == SCORE_TRANSH) {
                const dim3 grid(ceil_div((unsigned)Q, kTranshRows), std::max(1u, std::min(ceil_div(c, 8u), 2 * 148 / std::max(1u, ceil_div((unsigned)Q, kTranshRows)))));
                KGE_LAUNCH("predict_score", k_transh_score<<<grid, 256, transh_score_smem(), stream_>>>(
                                                queries, queries + Q * D, p_chunk_hidden_, p_raw_, nullptr, nullptr, (int)Q, (int)c, (int)D, ExchangeSync{}));
            } else
            KGE_LAUNCH("predict_score", KGE_CUDA(launch_score(cfg_.dist_fn, queries, p_chunk_hidden_, p_raw_, (int)Q, (int)c, (int)D, stream_)));
            launch_topk(b, c, start, last, tp, false);
        }
        KGE_LAUNCH("predict_finish", k_topk_finish<<<(unsigned)Q, 128, 0, stream_>>>(
                                         b.topk_state, b.topk_count, (int)Q, (int)hr, (int)nb, b.predict_score_dst,
                                         b.predict_index_dst));
        KGE_CUDA(cudaGetLastError());
    }
    launch_barrier();
    const size_t result_bytes = n * cfg_.n_shard * hr * nb * 4;
    KGE_CUDA(cudaMemcpyAsync(scores.data, arena_ + arena_offset_predict(1), result_bytes, cudaMemcpyDeviceToHost, stream_));
    KGE_CUDA(cudaMemcpyAsync(indices.data, arena_ + arena_offset_predict(2), result_bytes, cudaMemcpyDeviceToHost, stream_));
    KGE_CUDA(cudaStreamSynchronize(stream_));
    timing_collect();
    last_launches_ = launch_counter_;
    check_device_status();
}

// One pass of predict on the tensor cores: hidden rows of the table rows [start, start + c) as the
// contraction feature . W + value, then their scores against all Q queries: the dot product, or
// the L2 distance as |q|^2 + |t|^2 - 2 q.t with the direct form where that cancels, so identical
// rows still score identically and an exact match still scores gamma
// (src/poplar_kge.cpp:812-855; src/poplar_extensions/distance.cpp:151-185).
// Returns whether the score kernel has also filtered the pass's scores against the queries' cut-offs
// (the L2 form; dot products leave that to k_topk_filter).
bool Engine::predict_pass_planes(ShardBuffers& b, uint32_t start, unsigned c, uint32_t last, const TopkParams& tp, const float* queries, unsigned Q,
                                 int net) {
    const unsigned D = cfg_.d, F = cfg_.f;
    const uint8_t* rows = b.table + (size_t)start * layout_.row_bytes;
    if (F > 0) {
        FeaturePlanes fp{};
        const bool half_features = cfg_.feature_type == ST_F16;
        (half_features ? fp.wide : fp.lo) = p_feat_;
        fp.stride = feat_stride_;
        fp.off_feat = layout_.off_feat;
        const size_t units = (size_t)c * ((layout_.row_bytes - layout_.off_feat) >> 4);
        KGE_LAUNCH("predict_planes", k_table_feature_planes<<<(unsigned)std::min<size_t>((units + 255) / 256, 148 * 16), 256, 0, stream_>>>(
                                         b.table, layout_, start, (int)c, fp));
        tc::PlaneProblem p{};
        p.A = half_features ? tc::PlaneOperand{p_feat_, nullptr, (long long)feat_stride_ * 4, 0, 0}
                            : tc::PlaneOperand{reinterpret_cast<const float*>(rows + layout_.off_feat), p_feat_, (long long)layout_.row_bytes, 0, 0};
        const size_t w = dense_bounds_[1 + net];
        p.B = tc::PlaneOperand{dense_ + w, dense_lo_ + w, (long long)D * 4, 1, 0};
        p.g.M = (int)c; p.g.N = (int)D; p.g.K = (int)F;
        p.g.epilogue = tc::EPI_ADD_TABLE_VALUE;
        p.g.out = p_chunk_hidden_; p.g.ldc = D; p.g.block_rows = 1;
        p.g.x_base = rows; p.g.x_row_stride_bytes = layout_.row_bytes;
        p.g.x_is_half = cfg_.value_bf16 ? 2 : (cfg_.state_type == ST_F16 ? 1 : 0);
        launch_planes("predict_hidden", &p, 1, tc::SIDE_NONE, -1, -1);
    } else {
        dim3 hgrid(ceil_div(c, 64), ceil_div(D, 64), 1);
        KGE_LAUNCH("predict_hidden", KGE_DISPATCH_ROW(cfg_, k_hidden<ST, FT><<<hgrid, 256, 0, stream_>>>(
                                                                b.table, layout_, nullptr, start, (int)c, nullptr, nullptr, p_chunk_hidden_, nullptr)));
    }
    KGE_LAUNCH("predict_planes", k_lower_plane<<<(unsigned)std::min<size_t>(((size_t)c * D + 255) / 256, 148 * 16), 256, 0, stream_>>>(
                                     p_chunk_hidden_, (size_t)c * D, p_chunk_lo_));
    tc::PlaneProblem s{};
    s.A = tc::PlaneOperand{queries, p_query_lo_, (long long)D * 4, 0, 0};
    s.B = tc::PlaneOperand{p_chunk_hidden_, p_chunk_lo_, (long long)D * 4, 0, 0};
    s.g.M = (int)Q; s.g.N = (int)c; s.g.K = (int)D;
    const bool l2 = cfg_.dist_fn == DIST_L2;
    s.g.epilogue = l2 ? tc::EPI_L2_DISTANCE : tc::EPI_STORE;
    s.g.out = p_raw_; s.g.ldc = c; s.g.block_rows = 1;
    const bool filtered = l2 && filter_in_scores_;
    if (filtered) s.filter = tc::TopkFilterArgs{b.topk_state, b.topk_count, p_cand_, p_cand_count_, start, last, tp.n_best, tp.score_is_gamma_minus, tp.gamma};
    launch_planes("predict_score", &s, 1, l2 ? tc::SIDE_NORMS : tc::SIDE_NONE, -1, -1);
    KGE_CUDA(cudaGetLastError());
    return filtered;
}

size_t Engine::debug_fetch(const std::string& what, size_t shard, float* out, size_t capacity) {
    KGE_CUDA(cudaSetDevice((int)cfg_.device_ordinal));
    if (shard >= n_local_) fail(KGE_INVALID_ARGUMENT, "kge_debug_fetch: shard out of range");
    const ShardBuffers& b = shards_[shard];
    const size_t B = cfg_.batch_size, T = cfg_.n_tail(), R = cfg_.n_remote(), D = cfg_.d;
    const float* src = nullptr;
    size_t count = 0;
    if (what == "hidden") { src = b.hid_h; count = R * D; }
    else if (what == "hidden_tail") { src = b.hid_t; count = R * D; }
    else if (what == "tails") { src = b.tails; count = T * D; }
    else if (what == "pred") { src = b.pred; count = B * D; }
    else if (what == "raw_score") { src = b.raw; count = B * T; }
    else if (what == "coeff") { src = b.coeff; count = B * T; }
    else if (what == "d_pred") { src = b.d_pred; count = B * D; }
    else if (what == "d_hidden") { src = b.d_hid_h; count = R * D; }
    else if (what == "grad_recv") { src = b.grad_recv; count = T * D; }
    else if (what == "dense_grad") {
        if (cfg_.world > 1) fail(KGE_INVALID_ARGUMENT, "kge_debug_fetch: 'dense_grad' is spread over the processes; fetch it with one process");
        src = b.dense_partial; count = n_dense_;
    }
    else if (what == "loss_last") { src = d_loss_last_ + shard; count = 1; }
    else if (what == "exchange_trace") {
        // microseconds since the earliest stamp, [kTraceSlots][XCHG_KINDS][published | wait began | wait ended]; 0 = no stamp
        const size_t n = (size_t)kTraceSlots * XCHG_KINDS * 3;
        if (!d_xchg_trace_) fail(KGE_INVALID_ARGUMENT, "kge_debug_fetch: exchange_trace needs KGE_EXCHANGE_TRACE=1 in the environment");
        if (n > capacity) fail(KGE_INVALID_ARGUMENT, msg() << "kge_debug_fetch: 'exchange_trace' needs room for " << n << " floats");
        KGE_CUDA(cudaStreamSynchronize(stream_));
        std::vector<unsigned long long> stamps(n);
        KGE_CUDA(cudaMemcpy(stamps.data(), d_xchg_trace_, n * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
        unsigned long long base = ~0ull;
        for (unsigned long long v : stamps) if (v && v < base) base = v;
        for (size_t i = 0; i < n; ++i) out[i] = stamps[i] ? (float)((double)(stamps[i] - base) * 1e-3) + 1e-3f : 0.f;
        return n;
    }
    else fail(KGE_INVALID_ARGUMENT, msg() << "kge_debug_fetch: unknown buffer '" << what << "'");
    if (count > capacity) fail(KGE_INVALID_ARGUMENT, msg() << "kge_debug_fetch: '" << what << "' needs room for " << count << " floats");
    KGE_CUDA(cudaStreamSynchronize(stream_));
    if (count) KGE_CUDA(cudaMemcpy(out, src, count * 4, cudaMemcpyDeviceToHost));
    return count;
}

}  // namespace kge
