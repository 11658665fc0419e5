/*
 * C ABI of the B200 BESS knowledge-graph-embedding engine.
 *
 * This is the boundary a binding for the reference's host API sits on: the
 * reference exposes one class, `Engine(settings, gp_folder).run(command, data)`
 * (src/lib.cpp:38-52, src/poplar_kge.hpp:57-75); the functions below carry the
 * same information with plain pointers and sizes.  All calls are synchronous
 * and must come from one thread at a time per engine, as in the reference.
 *
 * Every function returns a kge_status.  After a non-zero status,
 * kge_last_error() gives the message (for a failed kge_create pass NULL).
 * Status values map one to one to the exception classes the reference throws:
 * KGE_INVALID_ARGUMENT = std::invalid_argument (src/poplar_kge.cpp:39-47, 52-63,
 * 79-90, 961-963), KGE_RUNTIME_ERROR = std::runtime_error (:121-123),
 * KGE_LOGIC_ERROR = std::logic_error (:357).  KGE_DEVICE_STATUS has no
 * counterpart: a device-side bounded wait gave up, or a CUDA call failed.
 */
#ifndef KGE_B200_H
#define KGE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct kge_engine kge_engine;

enum kge_status {
    KGE_OK = 0,
    KGE_INVALID_ARGUMENT = 1,
    KGE_RUNTIME_ERROR = 2,
    KGE_DEVICE_STATUS = 3,
    KGE_LOGIC_ERROR = 4
};

/* Element types of host arrays (src/poplar_kge.hpp:38-50: float, uint32_t, float16). */
enum kge_dtype { KGE_F32 = 0, KGE_U32 = 1, KGE_F16 = 2 };

/* Variant tags of a settings value (the scalar alternatives of `Batch`, src/poplar_kge.hpp:38-50).
 * The reference's one map-valued setting, training.learning_rate_modifiers, is passed
 * flattened: one KGE_SET_FLOAT per entry under the key
 * "training.learning_rate_modifiers.<parameter name>". */
enum kge_setting_type { KGE_SET_STRING = 0, KGE_SET_BOOL = 1, KGE_SET_FLOAT = 2, KGE_SET_UNSIGNED = 3 };

typedef struct kge_setting {
    const char* key;      /* dotted key, e.g. "model.n_shard" (src/python/poplar_kge.py:265-278) */
    int type;             /* kge_setting_type */
    const char* s;        /* KGE_SET_STRING */
    double f;             /* KGE_SET_FLOAT */
    unsigned long long u; /* KGE_SET_UNSIGNED, KGE_SET_BOOL (0/1) */
} kge_setting;

/* A borrowed, C-contiguous host array: the `ArrayView<T>` of src/poplar_kge.hpp:20-31. */
typedef struct kge_array {
    const char* name; /* stream name, e.g. "remote", "loss", "value" */
    int dtype;        /* kge_dtype */
    int rank;
    const size_t* shape;
    void* data; /* host pointer; inputs are read, outputs are written in place */
} kge_array;

/*
 * Replaces `Engine::Engine(settings, gpFolder)` (src/poplar_kge.cpp:1001-1002, 919-948).
 * Reads the keys of src/poplar_kge.cpp:109-110,198-246 with the same types and the same
 * errors for a missing key or a wrong type.  Keys this engine adds (all optional):
 *   execution.device_ordinal (unsigned, CUDA device, default 0)
 *   execution.rank, execution.world_size (unsigned; one process per GPU, each process holds
 *       n_shard / world_size consecutive shards; default 0 / 1)
 *   execution.feature_dtype ("float16" | "float32"; storage type of the feature part of a
 *       row; default = execution.dtype)
 *   execution.cuda_graph (bool, default true: replay the step loop as one CUDA graph)
 * `artefact_dir` takes the place of gp_folder (the codelet folder); it is accepted and ignored.
 */
int kge_create(const kge_setting* settings, size_t n_settings, const char* artefact_dir,
               kge_engine** out);

/* Replaces `Engine::~Engine` (src/poplar_kge.cpp:1003). */
void kge_destroy(kge_engine* engine);

/* Message of the last failed call on this engine, or of the last failed kge_create (NULL). */
const char* kge_last_error(const kge_engine* engine);

/*
 * Replaces `Engine::run(command, data)` (src/poplar_kge.cpp:1004-1006, 950-998) for the
 * commands "train_step_loop", "predict", "read_entity", "write_entity", "read", "write".
 * Stream names, element types and shapes are those of src/poplar_kge.cpp:713-720,740,
 * 814-819,853-854,858-860,868-869, with the leading axis equal to the number of shards
 * this process holds (all of them when world_size is 1, as in the reference).  For
 * "read"/"write" the variable is named by `variable_name` and the array is called "value"
 * (src/poplar_kge.cpp:977-991).  Commands added to the reference's:
 *   "write_entity_rows" (write_indices u32 [n, rw], write_data [n, rw, 3D+F]) writes whole
 *     rows, embedding and optimiser state included, which the reference cannot do from the host.
 *   "initialise_entities" (no arrays) fills every row on the device: embeddings as
 *     "write_entity" draws them, features ~ N(0, 1), optimiser state zero.  It stands in for
 *     the reference's host loop that streams all features through "write_entity"
 *     (src/python/poplar_kge.py:690-705) when the data is synthetic.
 *   "entity_layout" (layout u32 [4]: bytes of a stored row, rows per shard, local shards, first
 *     local shard), "dump_entity_rows" and "restore_entity_rows" (shard_range u32 [3] = local
 *     shard, first row, row count; rows u32 [count, row bytes / 4]) copy a contiguous range of a
 *     shard's table as stored, for per-shard checkpoints; the reference reads the table only
 *     through read_entity chunks gathered into one host array (src/python/poplar_kge.py:583-598).
 *   "load_triples" (triples u32 [3, n_triples] sorted by bucket, bucket_offset and bucket_count
 *     u32 [n_shard, n_shard], shard_to_count u32 [n_shard]), "sample_batch" (sample_seed u32 [1];
 *     returns the five index streams of "train_step_loop") and "train_step_loop_sampled"
 *     (learning_rate, loss, sample_seed) are the reference's host-side batch sampler
 *     (src/python/poplar_kge_dataset.py:199-263, 310-393) on the device.
 */
int kge_run(kge_engine* engine, const char* command, const kge_array* arrays, size_t n_arrays,
            const char* variable_name);

/*
 * Replaces `run("variables", {})` (src/poplar_kge.cpp:993-998): the i-th variable's name and
 * global shape.  `shape` must have room for 4 entries.  Returns KGE_INVALID_ARGUMENT past the end.
 */
int kge_variable_count(kge_engine* engine, size_t* count);
int kge_variable_info(kge_engine* engine, size_t index, const char** name, int* dtype, int* rank,
                      size_t* shape);

/*
 * Multi-process set-up (no counterpart in the reference, which drives all replicas from one
 * process: src/fructose/fructose.cpp:108).  Each process exports an opaque handle of
 * kge_comm_handle_bytes() bytes, the host exchanges them (any transport), and every process
 * passes the concatenation, ordered by rank, to kge_comm_connect.  After that the training
 * step exchanges rows by direct stores into the peers' device memory over NVLink.
 */
size_t kge_comm_handle_bytes(void);
int kge_comm_export(kge_engine* engine, void* handle_out);
int kge_comm_connect(kge_engine* engine, const void* all_handles, size_t world_size);

/*
 * The two halves of "train_step_loop", separately, for callers that keep batches on the
 * device across calls (the reference's scripts/run_profile.py:43-51 re-runs one fixed batch).
 * kge_stage_batch validates and uploads the five index streams and prepares the per-step
 * segment tables; kge_train_staged runs the staged steps with the given learning rate and
 * writes the mean loss per local shard.  `loss` may be NULL to skip the read-back.
 */
int kge_stage_batch(kge_engine* engine, const kge_array* arrays, size_t n_arrays);
int kge_train_staged(kge_engine* engine, float learning_rate, float* loss);

/* Device time of the last kge_train_staged / "train_step_loop" run, from CUDA events on the
 * engine's stream, and the number of kernels it launched (graph nodes when replayed as a graph). */
int kge_last_run_stats(kge_engine* engine, float* device_ms, unsigned long long* kernel_launches);

/* Per-kernel device times.  While switched on, the step loop is launched kernel by kernel (not as
 * a graph) with a pair of CUDA events on the engine's stream around every launch; the totals per
 * kernel name accumulate until it is switched on again.  No counterpart in the reference, whose
 * profile comes from Poplar's own report (scripts/run_profile.py:22-30). */
int kge_set_kernel_timing(kge_engine* engine, int on);
int kge_kernel_time_count(kge_engine* engine, size_t* count);
int kge_kernel_time(kge_engine* engine, size_t index, const char** name, float* total_ms,
                    unsigned long long* launches);

/* Copies an intermediate of the last training step of local shard `shard` to the host, for
 * tests: "hidden", "tails", "pred", "raw_score", "coeff", "d_pred", "d_hidden", "dense_grad".
 * `capacity` is in floats; `*count` receives the number written. */
int kge_debug_fetch(kge_engine* engine, const char* what, size_t shard, float* out, size_t capacity,
                    size_t* count);

/*
 * Single operators with host buffers, mirroring the reference's operator tests
 * (tests/pag/testPag.cpp).  `fn`: 0 = L1 (src/poplar_extensions/distance.cpp:70-104),
 * 1 = L2 (:151-185), 2 = dot product (`matMul(a, b^T)`, src/poplar_kge.cpp:478-479).
 * a is [m, k], b is [n, k], out and grad_out are [m, n], row-major float32.
 */
int kge_op_pairwise(int fn, const float* a, const float* b, size_t m, size_t n, size_t k, float* out);
/* Input gradients (src/poplar_extensions/distance.cpp:106-149,187-229; src/pag/pag.cpp:685-701). */
int kge_op_pairwise_grad(int fn, const float* a, const float* b, const float* grad_out, size_t m,
                         size_t n, size_t k, float* grad_a, float* grad_b);
/* Row gather out[i] = table[indices[i]] and its backward, the duplicate-combining scatter-add
 * into a zeroed table (src/pag/pag.cpp:706-746), done by sort-and-segment. */
int kge_op_gather_rows(const float* table, size_t rows, size_t width, const uint32_t* indices,
                       size_t n, float* out);
int kge_op_scatter_add_rows(const float* grad_rows, const uint32_t* indices, size_t n, size_t rows,
                            size_t width, float* grad_table);
/*
 * The dense contraction of the step on the tensor cores, as an operator on host buffers: the fp32
 * `matMul` of src/pag/pag.cpp:673-704 (forward and both gradients are this one form).
 *   out[z, m, n] = epilogue( sum over k in split z of A[m, k] * B[n, k] )
 * a: stored matrix [a_rows, a_cols], fp32 or fp16 (a_half); A[m, k] = a[m, k], or a[k, m] when
 * a_transposed; a_gather (optional) picks the stored rows.  b: fp32, same conventions.
 * epilogue 0: acc; 1: acc + x[m, n]; 2: rowsum(A)[m] * x[m, n] - acc (x fp32 [m, n]).
 * tile_n: 64 or 128 output columns per thread block.  Products use the 3xTF32 split, so results
 * agree with an fp32 product to about 1e-6 of sum |a||b|.
 */
int kge_op_tc_gemm(const void* a, int a_half, int a_transposed, const uint32_t* a_gather, size_t a_rows,
                   size_t a_cols, const float* b, int b_transposed, size_t b_rows, size_t b_cols, size_t m,
                   size_t n, size_t k, int epilogue, const float* x, int splits, int tile_n, float* out);

/*
 * The same contraction in the form the training step runs: both operands are given to the kernel
 * as TF32-exact planes in device memory (made here from the host arrays; in the step the producing
 * kernels write them) and the TMA unit feeds the tensor core directly.  a: stored [a_rows, a_cols]
 * fp32, A[m, k] = a[m, k] or a[k, m] when a_mn_major; a_exact: every value is exact in TF32 (e.g. it
 * came from fp16 storage).  b likewise.  Stored rows must be multiples of 16 bytes.  epilogue 0-2 as
 * for kge_op_tc_gemm; 3: out[m, n] = the L2 distance of row m of A and row n of B in the form
 * sqrt(|a|^2 + |b|^2 - 2 a.b) (src/poplar_extensions/distance.cpp:151-185), recomputed directly
 * where the expansion cancels (both operands stored [mn][k]).  splits (1-8)
 * blocks share a tile's k range as one thread-block cluster; tile_n (64 or 128) is the tile's width;
 * out is [m, n].  The upper plane is the stored array itself, since the tensor core ignores the low
 * 13 bits of a TF32 operand; hi_is_cleared uses a copy with those bits cleared instead (same
 * result, bit for bit).  repeat > 0: *mean_us receives the mean device time of `repeat` further
 * launches (for the microbench; mean_us may be NULL).
 */
int kge_op_tc_planes(const float* a, int a_mn_major, int a_exact, size_t a_rows, size_t a_cols, const float* b,
                     int b_mn_major, size_t b_rows, size_t b_cols, size_t m, size_t n, size_t k, int epilogue,
                     const float* x, int splits, int tile_n, int hi_is_cleared, int repeat, float* mean_us,
                     float* out);

/*
 * The contraction on bfloat16 operands with fp32 accumulation (tcgen05.mma.kind::f16): the form in
 * which DistMult / ComplEx scores and their gradients run when the embeddings are stored in bf16
 * (`matMul`, src/poplar_kge.cpp:512-514, 571-573; the reference's reduced-precision tier is fp16
 * rows, src/poplar_kge.cpp:405-417).  Host arrays are fp32 and are rounded to bf16 on the device;
 * stored rows must be multiples of 8 elements.  Otherwise as kge_op_tc_planes with epilogue 0.
 */
int kge_op_tc_planes_bf16(const float* a, int a_mn_major, size_t a_rows, size_t a_cols, const float* b, int b_mn_major,
                          size_t b_rows, size_t b_cols, size_t m, size_t n, size_t k, int splits, int tile_n, int repeat,
                          float* mean_us, float* out);

/*
 * Device-timed kernels for the microbenchmark (BASELINE configuration 2; the reference's counterpart
 * is its operator benchmark tests/pag/testPag.cpp:321-332 and scripts/run_profile.py:43-51).  Inputs
 * are made on the device; *mean_us receives the mean device time of `repeat` back-to-back launches.
 * kge_microbench_rows: kind 0 = the step's gather of n whole rows [value | adam_m | sqrt(adam_v)]
 * (3 * d fp32) out of a table of table_rows rows; kind 1 = the row-wise Adam scatter on the same rows
 * (one lookup per row; indices distinct).  kge_microbench_scores: m queries against n shared tails,
 * k deep; fn 0 = L1, 1 = L2 (FP32 pipe), 2 = dot product, 3 = L2 as |a|^2 + |b|^2 - 2 a.b (tensor cores).
 */
int kge_microbench_rows(int kind, size_t table_rows, size_t d, const uint32_t* indices, size_t n, int repeat,
                        float* mean_us);
int kge_microbench_scores(int fn, size_t m, size_t n, size_t k, int repeat, float* mean_us);

/*
 * kge_op_scatter_add_rows for callers that cannot allocate device memory.  It has no counterpart
 * in the reference.  The operator's working memory (the sorted lookups and the per-row segment
 * starts) lives in a fixed array inside the library's device image instead of coming from
 * cudaMalloc, so this entry point calls no cudaMalloc, cudaFree or allocating library routine.
 * That is for hosts where an allocation is not allowed or not affordable: an operator running
 * inside a framework's caching allocator or a fixed memory reservation, or on a path that must not
 * take the device-wide synchronisation an allocation implies.
 *   - grad_rows [n, width], indices [n] and grad_table [rows, width] are DEVICE pointers owned by
 *     the caller; the work is queued on `cuda_stream` (a cudaStream_t, or NULL for the default
 *     stream) and the call returns without waiting for it.
 *   - Limits: n <= 4096 lookups, rows <= 65536; larger sizes are refused with KGE_INVALID_ARGUMENT.
 *     The array costs about 272 KB on every GPU that loads the library, until the process exits.
 *   - An index >= rows cannot be refused here (the indices are on the device): it is ignored.
 *   - The first call on a device looks up the array's address on that device (the device must be
 *     current); make that first call before starting any stream capture.
 *   - All calls on one device share the array.  Nothing in it needs clearing between calls (each
 *     call rewrites every entry it reads), but two calls whose kernels overlap on the GPU, from
 *     different streams or threads, race on it: keep them ordered.
 */
int kge_op_scatter_add_rows_noalloc(const float* grad_rows, const uint32_t* indices, size_t n, size_t rows,
                                    size_t width, float* grad_table, void* cuda_stream);
/* Row-wise losses with gradients: kind 0 = guarded log-sigmoid (src/pag/pag.cpp:888-910,
 * elementwise, grad_x = grad_out * d/dx), kind 1 = log-softmax over the last axis (:841-864). */
int kge_op_activation(int kind, const float* x, const float* grad_out, size_t rows, size_t cols,
                      float* y, float* grad_x);
/* The exchange on n emulated shards held in one buffer: out[dst][src] = in[src][dst] for
 * blocks of `block` floats (src/pag/pag.cpp:915-935). */
int kge_op_all_to_all(const float* in, size_t n_shard, size_t block, float* out);

#ifdef __cplusplus
}
#endif
#endif /* KGE_B200_H */
