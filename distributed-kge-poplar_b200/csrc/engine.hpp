// Host engine: owns the shard tables, the dense parameters and the per-step buffers of
// the shards this process holds, and launches the kernels of one training step in the
// order of the reference's Model::trainStep (src/poplar_kge.cpp:664-707).
#pragma once

#include <map>
#include <memory>
#include <string>
#include <vector>

#include "common.hpp"
#include "kernels.cuh"
#include "tc_gemm.cuh"
#include "tc_planes.cuh"
#include "transh.cuh"
#include "mlp.cuh"

namespace kge {

struct SettingValue {
    int type;
    std::string s;
    double f;
    unsigned long long u;
};
using SettingMap = std::map<std::string, SettingValue>;

enum StorageType : int { ST_F32 = 0, ST_F16 = 1 };

// The keys the reference's Model reads (src/poplar_kge.cpp:198-246) plus this engine's own.
struct Config {
    unsigned seed, n_shard, n_entity, n_relation_type, d, f;
    unsigned batch_size, a2a_size, n_step, rw_batch, predict_hr, predict_tail_batch, predict_n_best;
    int score_fn, dist_fn, loss_fn;
    bool share_networks;
    float gamma, init_scale, adversarial_scale, correction_weight, loss_scale;
    // Norm regularisers of the gathered rows' values, feature-network outputs and hidden rows
    // (training.embedding_regularisation, .feature_regularisation, .hidden_regularisation): power and weight.
    float reg_power[3], reg_weight[3];
    unsigned mlp;   // model.feature_mlp_size: width of the feature MLP's hidden layer, 0 = none
    float dropout;  // model.feature_dropout: drop probability of the feature network's output while training
    bool regularised() const { return reg_weight[0] > 0.f || reg_weight[1] > 0.f || reg_weight[2] > 0.f; }
    float beta_m, beta_v, epsilon, weight_decay;
    std::map<std::string, float> lr_modifiers;
    int state_type, feature_type;
    // "execution.value_dtype": "bfloat16" stores the embedding values in bf16 while adam_m and
    // sqrt(adam_v) stay float32, and runs the dot-product scores and their gradients on bf16
    // tensor-core products with fp32 accumulation (results agree with fp32 to about 1e-2).
    bool value_bf16;
    unsigned device_ordinal, rank, world;
    bool cuda_graph;
    bool tensor_cores;  // dense contractions on tcgen05 (3xTF32) instead of the FP32 pipe
    // The training step's L2 distance as |a|^2 + |b|^2 - 2 a.b on the tensor cores, with the direct form
    // wherever the expansion cancels.  Off by default: with skewed entity popularity a quarter of a
    // batch's (head, tail) pairs name the same popular entity, whose distance is the small relation
    // vector, so the direct form is needed for too many pairs and the FP32-pipe kernel is faster.
    bool l2_contraction;

    unsigned n_tail() const { return n_shard * a2a_size; }
    unsigned n_remote() const { return batch_size + n_tail(); }
    unsigned row_width() const { return 3 * d + f; }
    unsigned n_net() const { return f == 0 ? 0 : (share_networks ? 1 : 2); }
};

Config parse_config(const SettingMap& settings);

struct Variable {
    std::string name;
    int dtype;
    std::vector<size_t> shape;
    size_t offset;  // element offset inside the dense vector (params / adam_m / adam_v)
    int kind;       // 0 = parameter, 1 = adam_m, 2 = adam_v, 3 = step
    // true: stored contiguously, whatever its column count (a multiple of d floats in all); false:
    // one row of the variable per d-float row of the dense vector, of which it shows shape[1] columns
    bool flat = false;
};

struct HostArray {
    std::string name;
    int dtype;
    std::vector<size_t> shape;
    void* data;
    size_t count() const {
        size_t n = 1;
        for (size_t s : shape) n *= s;
        return n;
    }
};

class Engine {
   public:
    explicit Engine(const SettingMap& settings);
    ~Engine();
    Engine(const Engine&) = delete;
    Engine& operator=(const Engine&) = delete;

    void run(const std::string& command, std::vector<HostArray>& arrays, const std::string& variable);
    const std::vector<Variable>& variables() const { return variables_; }

    static size_t comm_handle_bytes();
    void comm_export(void* out) const;
    void comm_connect(const void* handles, size_t world);

    void stage_batch(std::vector<HostArray>& arrays);
    void train_staged(float learning_rate, float* loss);
    void last_run_stats(float* ms, unsigned long long* launches) const;
    void set_kernel_timing(bool on);
    size_t kernel_time_count() const;
    void kernel_time(size_t index, const char** name, float* ms, unsigned long long* launches) const;
    size_t debug_fetch(const std::string& what, size_t shard, float* out, size_t capacity);

    std::string last_error;

   private:
    struct ShardBuffers {
        uint8_t* table = nullptr;
        uint8_t* rows_c2[2] = {nullptr, nullptr};  // the gathered rows of even / odd steps, table row layout, [R]
        float *hid_h = nullptr, *hid_t = nullptr, *pred = nullptr, *raw = nullptr, *coeff = nullptr;
        float *d_pred = nullptr, *d_head = nullptr, *d_relrow = nullptr;
        float *d_hid_h = nullptr, *d_hid_t = nullptr, *proj_partial = nullptr, *loss_rows = nullptr;
        // TransH: unit normals of the batch's relations, n_i . t_j and the signs' sums along the normal
        // ([B, T]), gradients of the normals from the scores, per-triple gradients of the raw normals
        float *nrm = nullptr, *pair_s = nullptr, *pair_u = nullptr, *d_nrm = nullptr, *d_normrow = nullptr;
        // Feature MLP, per network: its input rows [R, 2D] and pre-activations [R, M]; then its output
        // [R, D], the gradients of the pre-activations and of the input, the value's deferred gradient,
        // and this shard's gradients of the two projections
        float *mlp_cat[2] = {nullptr, nullptr}, *mlp_pre[2] = {nullptr, nullptr};
        float *mlp_out = nullptr, *mlp_d_pre = nullptr, *mlp_d_cat = nullptr, *d_val = nullptr, *mlp_dw_up = nullptr, *mlp_dw_down = nullptr;
        float *reg_val = nullptr, *reg_h = nullptr, *reg_t = nullptr, *reg_loss_rows = nullptr;  // regularisers' terms, [R, D] and [R]
        float *tails = nullptr, *grad_recv = nullptr, *dense_partial = nullptr;  // inside the arena
        float** send_dst = nullptr;  // device table [n_shard]
        float** grad_dst = nullptr;  // device table [n_shard]
        // Lower TF32 planes of the tensor-core operands that this shard's kernels produce (the upper
        // plane is the fp32 array itself), and the widened features of the gathered rows.
        float* feat_wide2[2] = {nullptr, nullptr};  // fp16 features as fp32, [R, feat_stride], even / odd steps
        float* feat_lo2[2] = {nullptr, nullptr};    // lower plane of fp32 features
        float *pred_lo = nullptr, *coeff_lo = nullptr, *d_hid_h_lo = nullptr, *d_hid_t_lo = nullptr;
        float* tails_lo = nullptr;       // inside the arena, beside `tails`
        float** send_lo_dst = nullptr;   // device table [n_shard]
        float* heavy_partial = nullptr;   // [kHeavySlots][2][D] sums of the parts of popular rows
        unsigned* heavy_counter = nullptr;  // [kHeavySlots]
        float** dense_dst = nullptr;  // device table [world]: this shard's slot in each owner's receive buffer
        float** predict_score_dst = nullptr;     // device table [n_shard]: where each asking shard's results go
        uint32_t** predict_index_dst = nullptr;  // device table [n_shard]
        unsigned long long* topk_state = nullptr;
        int* topk_count = nullptr;
    };

    // set-up
    void allocate();
    void build_pointer_tables();
    size_t arena_offset_flags() const { return 0; }
    size_t arena_offset_dense(int which) const;
    size_t arena_offset_shard(unsigned local, int which) const;
    size_t arena_offset_predict(int which) const;
    size_t arena_offset_dense_recv() const;
    size_t arena_size() const;

    // commands
    void cmd_train_step_loop(std::vector<HostArray>& arrays);
    void cmd_read_entity(std::vector<HostArray>& arrays);
    void cmd_copy_entity_range(std::vector<HostArray>& arrays, bool to_host);
    void cmd_write_entity(std::vector<HostArray>& arrays, bool whole_rows);
    void cmd_read_write_variable(std::vector<HostArray>& arrays, const std::string& name, bool write);
    void cmd_predict(std::vector<HostArray>& arrays);
    void cmd_initialise_entities();
    void cmd_load_triples(std::vector<HostArray>& arrays);
    void cmd_sample_batch(std::vector<HostArray>& arrays, bool train);
    void sample_and_stage(uint32_t seed);
    void prepare_staged();

    // the step
    void launch_steps();
    void launch_one_step(unsigned step);
    void launch_barrier();
    ExchangeSync exchange_sync() const;
    void launch_exchange_wait(int kind);
    void launch_exchange_signal(int kind);
    void launch_gather(unsigned step, cudaStream_t stream);
    void launch_tc(const char* name, tc::GemmArgs* problems, int n_problems, int splits, bool a_exact, bool rowsum,
                   int wait_kind = -1, int signal_kind = -1);
    // the plane-fed contraction: tile width and k splits chosen here
    void launch_planes(const char* name, tc::PlaneProblem* problems, int n_problems, int side, int wait_kind, int signal_kind,
                       const tc::RouteArgs* route = nullptr);
    void launch_step_planes(unsigned step, const LossParams& lp, float normaliser);
    void refresh_lower_plane(size_t offset, size_t count);
    FeaturePlanes feature_planes(const ShardBuffers& b, unsigned parity) const;
    void check_device_status();
    void require_usable() const;
    void timing_begin(const char* name);
    void timing_end();
    void timing_collect();

    HostArray& find_array(std::vector<HostArray>& arrays, const std::string& name, int dtype,
                          const std::vector<size_t>& shape);
    void* device_alloc(size_t bytes);

    Config cfg_;
    RowLayout layout_{};
    AdamParams adam_{};
    unsigned n_local_ = 0, shard0_ = 0;
    cudaStream_t stream_ = nullptr;
    // Work that does not lie on the step's chain of dependent kernels runs beside it: forked from and
    // joined to the main stream with events (graph edges under capture).
    cudaStream_t side_stream_ = nullptr;
    unsigned side_streams_ = 0;
    bool split_popular_rows_ = true;  // rows with many lookups are summed in parts by several blocks
    bool planes_ = false;             // the step's contractions run on the plane-fed tensor-core kernel
    bool bf16_planes_ = false;        // scores and their gradients multiply bfloat16 copies of their operands
    uint32_t feat_stride_ = 0;        // floats per row of the widened / lower feature planes
    cudaEvent_t ev_fork_ = nullptr, ev_join_[2] = {nullptr, nullptr};
    cudaStream_t side_begin();
    void side_end(int which);
    void side_join(int which);
    cudaEvent_t ev_begin_ = nullptr, ev_end_ = nullptr;
    cudaEvent_t ev_stage_[2] = {nullptr, nullptr};  // around the segment preparation of a staged batch
    bool stage_fresh_ = false;                      // its time has not been counted towards a run yet
    bool poisoned_ = false;                         // a device-side wait gave up: the engine must be rebuilt
    std::vector<void*> allocations_;
    std::vector<ShardBuffers> shards_;

    // peer-visible arena
    uint8_t* arena_ = nullptr;
    std::vector<uint8_t*> peer_arena_;
    bool connected_ = false;
    unsigned* d_epoch_ = nullptr;
    unsigned* d_status_ = nullptr;
    unsigned long long* d_xchg_trace_ = nullptr;  // optional time stamps of the hand-overs (KGE_EXCHANGE_TRACE=1)
    unsigned* d_xchg_words_ = nullptr;  // [XCHG_KINDS] published epochs, [XCHG_KINDS] finished-block counters
    unsigned* d_tc_status_ = nullptr;
    // split-k workspace of the tensor-core contractions (shared by all of them: one stream)
    float *tc_ws_ = nullptr, *tc_ws_rowsum_ = nullptr;
    size_t tc_ws_floats_ = 0;
    static constexpr int kTcMaxSplits = 8;
    int tc_splits(unsigned tiles, unsigned k) const;
    unsigned** d_peer_flags_ = nullptr;
    const float** d_partials_ = nullptr;  // [n_shard]
    float** d_replicas_ = nullptr;        // [world]

    // dense parameters: relation table | projection(s)
    size_t n_dense_ = 0, proj_elems_ = 0, dense_bounds_[kDenseParams + 1] = {};  // relation table | projection(s) | TransH normals | MLP up, down per network
    float dense_lr_mod_[kDenseParams] = {1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f};
    float entity_lr_mod_ = 1.f;
    float *dense_ = nullptr, *dense_m_ = nullptr, *dense_v_ = nullptr;
    float* dense_lo_ = nullptr;      // lower TF32 plane of the dense vector (same layout, inside the arena)
    float** d_replicas_lo_ = nullptr;  // [world]
    size_t own_rows_ = 0, dense_chunk_ = 0, dense_chunk_rows_ = 1;
    std::vector<Variable> variables_;
    unsigned long long step_ = 0;
    int proj_splits_ = 1, proj_rows_per_split_ = 0;

    // staged batch
    uint32_t *d_remote_ = nullptr, *d_a2a_ = nullptr, *d_head_ = nullptr, *d_relation_ = nullptr,
             *d_tail_ = nullptr;
    uint32_t *d_ent_perm_ = nullptr, *d_ent_off_ = nullptr, *d_rel_perm_ = nullptr,
             *d_rel_off_ = nullptr, *d_first_slot_ = nullptr, *d_heavy_count_ = nullptr;
    uint4* d_heavy_parts_ = nullptr;
    uint4* d_row_info_ = nullptr;  // [n_local * n_step][R][2] per gathered row: offsets, flags, table row, first four lookups
    float *d_step_size_ = nullptr, *d_loss_total_ = nullptr, *d_loss_last_ = nullptr;
    unsigned* d_loss_counter_ = nullptr;
    size_t transh_score_smem() const { return (size_t)2 * kTranshRows * cfg_.d * sizeof(float); }
    bool mlp_on() const { return cfg_.mlp > 0 && cfg_.f > 0; }
    void launch_mlp_forward(const uint8_t* rows, const uint32_t* index, uint32_t start, unsigned n_rows, int net, float* hid,
                            float* cat, float* pre, float* out);
    void launch_mlp_backward(unsigned l, unsigned step);
    unsigned long long* p_cand_ = nullptr;  // [Q, kTopkCandidates] a batch's keys above each query's cut-off
    int* p_cand_count_ = nullptr;
    void launch_topk(ShardBuffers& b, unsigned c, uint32_t start, uint32_t last, const TopkParams& tp, bool filtered);
    float *p_mlp_cat_ = nullptr, *p_mlp_pre_ = nullptr, *p_mlp_out_ = nullptr;  // predict's MLP buffers
    bool filter_in_scores_ = true;  // predict's L2 score contraction also filters the scores against the queries' cut-offs (KGE_PREDICT_FILTER_IN_SCORES=0: k_topk_filter)
    bool heavy_route_ = false;  // rows with many lookups are routed in parts by k_route_heavy (KGE_ROUTE_POPULAR_ROWS=0: by the hidden kernel's epilogue)
    bool fuse_dense_ = false, fuse_dense_env_ = true;  // single shard: dense Adam steps inside the kernels that produce the gradients (KGE_FUSE_DENSE_UPDATE=0: k_dense_update)
    uint32_t* d_step_key_ = nullptr;   // [n_step] numbers of the staged training steps (keys of the dropout masks)
    bool dropout_on() const { return cfg_.dropout > 0.f && cfg_.f > 0; }
    DropoutParams dropout_params(unsigned l, unsigned step) const;
    void launch_dropout(unsigned l, unsigned step, const uint8_t* rows_c);
    float* d_reg_loss_ = nullptr;      // [n_local][2]: the step's regularisation loss, and a sink for its running sum
    unsigned* d_reg_counter_ = nullptr;
    void launch_regularise(unsigned l, const uint8_t* rows_c);
    RelationRows with_regularisers(RelationRows rr, unsigned l, unsigned step) const;
    uint8_t* pinned_ = nullptr;
    size_t pinned_bytes_ = 0;
    bool staged_ = false;
    // the training triples for the on-device sampler ("load_triples"), bucketed by (head shard, tail shard)
    SamplerData sampler_{};
    uint32_t sample_run_ = 0;  // program runs sampled so far: part of the generator's key
    // predict: buffers made on first use
    void ensure_predict_buffers();
    bool predict_pass_planes(ShardBuffers& b, uint32_t start, unsigned c, uint32_t last, const TopkParams& tp, const float* queries, unsigned Q, int net);
    float *p_head_hidden_ = nullptr, *p_chunk_hidden_ = nullptr, *p_raw_ = nullptr;
    uint32_t* d_iota_ = nullptr;
    // table rows scored per pass: 4096 on the FP32 pipe, 16384 when hidden rows and scores are tensor-core contractions
    unsigned predict_chunk_ = 4096;
    bool predict_planes_ = false;
    float *p_feat_ = nullptr, *p_chunk_lo_ = nullptr, *p_query_lo_ = nullptr;  // planes of a pass: widened / lower features, lower hidden rows, lower queries

    uint32_t* d_rw_idx_ = nullptr;
    uint8_t* d_rw_data_ = nullptr;

    struct TimedLaunch {
        const char* name;
        cudaEvent_t start, stop;
    };
    struct KernelTime {
        float ms = 0.f;
        unsigned long long launches = 0;
    };
    bool kernel_timing_ = false, timing_open_ = false;
    static constexpr size_t kMaxTimedLaunches = 400;  // what the launch queue holds while the stream is held
    std::vector<cudaEvent_t> event_pool_;
    std::vector<TimedLaunch> timed_;
    std::map<std::string, KernelTime> kernel_times_;

    cudaGraphExec_t graph_exec_ = nullptr;
    float last_ms_ = 0.f;
    unsigned long long last_launches_ = 0, launch_counter_ = 0;
};

}  // namespace kge
