// extern "C" surface of include/kge_b200.h: argument marshalling and error mapping for the
// engine, and the single-operator entry points.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "engine.hpp"
#include "tc_gemm.cuh"
#include "tc_planes.cuh"

#include <cuda_bf16.h>

using namespace kge;

struct kge_engine {
    std::unique_ptr<Engine> impl;
    std::string last_error;
};

namespace {

thread_local std::string g_error;  // last failure of kge_create or of an operator entry point

template <class Fn>
int guarded(std::string& error_slot, Fn&& fn) {
    try {
        fn();
        return KGE_OK;
    } catch (const Error& e) {
        error_slot = e.message;
        return e.code;
    } catch (const std::invalid_argument& e) {
        error_slot = e.what();
        return KGE_INVALID_ARGUMENT;
    } catch (const std::logic_error& e) {
        error_slot = e.what();
        return KGE_LOGIC_ERROR;
    } catch (const std::exception& e) {
        error_slot = e.what();
        return KGE_RUNTIME_ERROR;
    }
}

std::vector<HostArray> to_host_arrays(const kge_array* arrays, size_t n) {
    std::vector<HostArray> out;
    out.reserve(n);
    for (size_t i = 0; i < n; ++i) {
        const kge_array& a = arrays[i];
        if (!a.name) fail(KGE_INVALID_ARGUMENT, "array without a name");
        if (a.dtype != KGE_F32 && a.dtype != KGE_U32 && a.dtype != KGE_F16)
            fail(KGE_INVALID_ARGUMENT, msg() << "'" << a.name << "' has an unknown element type " << a.dtype);
        if (a.rank < 0 || a.rank > 8 || (a.rank && !a.shape))
            fail(KGE_INVALID_ARGUMENT, msg() << "'" << a.name << "' has a bad rank or no shape");
        out.push_back({a.name, a.dtype, std::vector<size_t>(a.shape, a.shape + a.rank), a.data});
    }
    return out;
}

// Temporary device buffers for the operator entry points.
struct DeviceBuffer {
    void* p = nullptr;
    explicit DeviceBuffer(size_t bytes) { KGE_CUDA(cudaMalloc(&p, bytes ? bytes : 16)); }
    ~DeviceBuffer() { cudaFree(p); }
    DeviceBuffer(const DeviceBuffer&) = delete;
    template <class T>
    T* as() { return static_cast<T*>(p); }
};
void to_device(DeviceBuffer& dst, const void* src, size_t bytes) {
    if (bytes) KGE_CUDA(cudaMemcpy(dst.p, src, bytes, cudaMemcpyHostToDevice));
}
void to_host(void* dst, DeviceBuffer& src, size_t bytes) {
    if (bytes) KGE_CUDA(cudaMemcpy(dst, src.p, bytes, cudaMemcpyDeviceToHost));
}
void finish_kernels() {
    KGE_CUDA(cudaGetLastError());
    KGE_CUDA(cudaDeviceSynchronize());
}
unsigned blocks_for(size_t n, unsigned per) { return (unsigned)((n + per - 1) / per); }
void require(bool ok, const char* what) {
    if (!ok) fail(KGE_INVALID_ARGUMENT, what);
}


}  // namespace

extern "C" {

int kge_create(const kge_setting* settings, size_t n_settings, const char*, kge_engine** out) {
    return guarded(g_error, [&] {
        if (!out) fail(KGE_INVALID_ARGUMENT, "kge_create: out is null");
        *out = nullptr;
        SettingMap map;
        for (size_t i = 0; i < n_settings; ++i) {
            const kge_setting& s = settings[i];
            if (!s.key) fail(KGE_INVALID_ARGUMENT, "setting without a key");
            if (s.type < KGE_SET_STRING || s.type > KGE_SET_UNSIGNED)
                fail(KGE_INVALID_ARGUMENT, msg() << "Key '" << s.key << "' holds value of unexpected type.");
            map[s.key] = SettingValue{s.type, s.s ? s.s : "", s.f, s.u};
        }
        auto engine = std::make_unique<kge_engine>();
        engine->impl = std::make_unique<Engine>(map);
        *out = engine.release();
    });
}

void kge_destroy(kge_engine* engine) { delete engine; }

const char* kge_last_error(const kge_engine* engine) {
    return engine ? engine->last_error.c_str() : g_error.c_str();
}

int kge_run(kge_engine* engine, const char* command, const kge_array* arrays, size_t n_arrays,
            const char* variable_name) {
    if (!engine) return KGE_INVALID_ARGUMENT;
    return guarded(engine->last_error, [&] {
        if (!command) fail(KGE_INVALID_ARGUMENT, "kge_run: command is null");
        auto host = to_host_arrays(arrays, n_arrays);
        const std::string cmd = command;
        if ((cmd == "read" || cmd == "write") && !variable_name) fail(KGE_INVALID_ARGUMENT, "Key not found 'name'");
        engine->impl->run(cmd, host, variable_name ? variable_name : "");
    });
}

int kge_variable_count(kge_engine* engine, size_t* count) {
    if (!engine || !count) return KGE_INVALID_ARGUMENT;
    *count = engine->impl->variables().size();
    return KGE_OK;
}

int kge_variable_info(kge_engine* engine, size_t index, const char** name, int* dtype, int* rank, size_t* shape) {
    if (!engine) return KGE_INVALID_ARGUMENT;
    return guarded(engine->last_error, [&] {
        const auto& vars = engine->impl->variables();
        if (index >= vars.size()) fail(KGE_INVALID_ARGUMENT, "kge_variable_info: index past the end");
        const Variable& v = vars[index];
        if (name) *name = v.name.c_str();
        if (dtype) *dtype = v.dtype;
        if (rank) *rank = (int)v.shape.size();
        if (shape)
            for (size_t i = 0; i < v.shape.size() && i < 4; ++i) shape[i] = v.shape[i];
    });
}

size_t kge_comm_handle_bytes(void) { return Engine::comm_handle_bytes(); }

int kge_comm_export(kge_engine* engine, void* handle_out) {
    if (!engine) return KGE_INVALID_ARGUMENT;
    return guarded(engine->last_error, [&] {
        if (!handle_out) fail(KGE_INVALID_ARGUMENT, "kge_comm_export: handle_out is null");
        engine->impl->comm_export(handle_out);
    });
}

int kge_comm_connect(kge_engine* engine, const void* all_handles, size_t world_size) {
    if (!engine) return KGE_INVALID_ARGUMENT;
    return guarded(engine->last_error, [&] {
        if (!all_handles) fail(KGE_INVALID_ARGUMENT, "kge_comm_connect: all_handles is null");
        engine->impl->comm_connect(all_handles, world_size);
    });
}

int kge_stage_batch(kge_engine* engine, const kge_array* arrays, size_t n_arrays) {
    if (!engine) return KGE_INVALID_ARGUMENT;
    return guarded(engine->last_error, [&] {
        auto host = to_host_arrays(arrays, n_arrays);
        engine->impl->stage_batch(host);
    });
}

int kge_train_staged(kge_engine* engine, float learning_rate, float* loss) {
    if (!engine) return KGE_INVALID_ARGUMENT;
    return guarded(engine->last_error, [&] { engine->impl->train_staged(learning_rate, loss); });
}

int kge_last_run_stats(kge_engine* engine, float* device_ms, unsigned long long* kernel_launches) {
    if (!engine) return KGE_INVALID_ARGUMENT;
    engine->impl->last_run_stats(device_ms, kernel_launches);
    return KGE_OK;
}

int kge_set_kernel_timing(kge_engine* engine, int on) {
    if (!engine) return KGE_INVALID_ARGUMENT;
    engine->impl->set_kernel_timing(on != 0);
    return KGE_OK;
}

int kge_kernel_time_count(kge_engine* engine, size_t* count) {
    if (!engine || !count) return KGE_INVALID_ARGUMENT;
    *count = engine->impl->kernel_time_count();
    return KGE_OK;
}

int kge_kernel_time(kge_engine* engine, size_t index, const char** name, float* total_ms, unsigned long long* launches) {
    if (!engine) return KGE_INVALID_ARGUMENT;
    return guarded(engine->last_error, [&] { engine->impl->kernel_time(index, name, total_ms, launches); });
}

int kge_debug_fetch(kge_engine* engine, const char* what, size_t shard, float* out, size_t capacity, size_t* count) {
    if (!engine) return KGE_INVALID_ARGUMENT;
    return guarded(engine->last_error, [&] {
        if (!what || !out) fail(KGE_INVALID_ARGUMENT, "kge_debug_fetch: null argument");
        const size_t n = engine->impl->debug_fetch(what, shard, out, capacity);
        if (count) *count = n;
    });
}

// ---------------------------------------------------------------------------
// Single operators on host buffers.

int kge_op_pairwise(int fn, const float* a, const float* b, size_t m, size_t n, size_t k, float* out) {
    return guarded(g_error, [&] {
        require(fn >= DIST_L1 && fn <= DIST_DOT, "kge_op_pairwise: fn must be 0 (L1), 1 (L2) or 2 (dot)");
        require(a && b && out, "kge_op_pairwise: null argument");
        if (m == 0 || n == 0) return;
        DeviceBuffer da(m * k * 4), db(n * k * 4), dout(m * n * 4);
        to_device(da, a, m * k * 4);
        to_device(db, b, n * k * 4);
        KGE_CUDA(launch_score(fn, da.as<float>(), db.as<float>(), dout.as<float>(), (int)m, (int)n, (int)k, nullptr));
        finish_kernels();
        to_host(out, dout, m * n * 4);
    });
}

int kge_op_pairwise_grad(int fn, const float* a, const float* b, const float* grad_out, size_t m, size_t n,
                         size_t k, float* grad_a, float* grad_b) {
    return guarded(g_error, [&] {
        require(fn >= DIST_L1 && fn <= DIST_DOT, "kge_op_pairwise_grad: fn must be 0 (L1), 1 (L2) or 2 (dot)");
        require(a && b && grad_out && grad_a && grad_b, "kge_op_pairwise_grad: null argument");
        if (m == 0 || n == 0 || k == 0) return;
        DeviceBuffer da(m * k * 4), db(n * k * 4), dg(m * n * 4), dga(m * k * 4), dgb(n * k * 4);
        to_device(da, a, m * k * 4);
        to_device(db, b, n * k * 4);
        std::vector<float> coeff(grad_out, grad_out + m * n);
        if (fn == DIST_L2) {
            // The L2 backward divides by the forward distance, and is zero where that is zero
            // (src/poplar_extensions/l2distance.codelet.cpp:149-158): take the distance from
            // the forward kernel, then fold the division into the coefficient.
            DeviceBuffer ddist(m * n * 4);
            KGE_CUDA(launch_score(DIST_L2, da.as<float>(), db.as<float>(), ddist.as<float>(), (int)m, (int)n, (int)k, nullptr));
            finish_kernels();
            std::vector<float> dist(m * n);
            to_host(dist.data(), ddist, m * n * 4);
            for (size_t i = 0; i < m * n; ++i) coeff[i] = dist[i] == 0.f ? 0.f : coeff[i] / dist[i];
        }
        to_device(dg, coeff.data(), m * n * 4);
        PairBwdArgs pa{};
        pa.D = (int)k;
        pa.tiles_m0 = (int)blocks_for(m, 32);
        pa.p[0] = {da.as<float>(), db.as<float>(), dg.as<float>(), (int)m, (int)n, (int)n, 1, dga.as<float>(), nullptr, 1};
        pa.p[1] = {db.as<float>(), da.as<float>(), dg.as<float>(), (int)n, (int)m, 1, (int)n, dgb.as<float>(), nullptr, 1};
        dim3 grid(blocks_for(m, 32) + blocks_for(n, 32), blocks_for(k, 64));
        if (fn == DIST_L1) k_pair_bwd<DIST_L1><<<grid, 128>>>(pa);
        else if (fn == DIST_L2) k_pair_bwd<DIST_L2><<<grid, 128>>>(pa);
        else k_pair_bwd<DIST_DOT><<<grid, 128>>>(pa);
        finish_kernels();
        to_host(grad_a, dga, m * k * 4);
        to_host(grad_b, dgb, n * k * 4);
    });
}

int kge_op_gather_rows(const float* table, size_t rows, size_t width, const uint32_t* indices, size_t n, float* out) {
    return guarded(g_error, [&] {
        require(table && indices && out, "kge_op_gather_rows: null argument");
        for (size_t i = 0; i < n; ++i)
            if (indices[i] >= rows) fail(KGE_INVALID_ARGUMENT, msg() << "kge_op_gather_rows: index " << indices[i] << " is not below " << rows);
        if (n == 0 || width == 0) return;
        DeviceBuffer dt(rows * width * 4), di(n * 4), dout(n * width * 4);
        to_device(dt, table, rows * width * 4);
        to_device(di, indices, n * 4);
        if (width % 4 == 0) k_gather_rows<4><<<(unsigned)n, 128>>>(dt.as<float>(), width, di.as<uint32_t>(), dout.as<float>());
        else k_gather_rows<1><<<(unsigned)n, 128>>>(dt.as<float>(), width, di.as<uint32_t>(), dout.as<float>());
        finish_kernels();
        to_host(out, dout, n * width * 4);
    });
}

int kge_op_scatter_add_rows(const float* grad_rows, const uint32_t* indices, size_t n, size_t rows, size_t width,
                            float* grad_table) {
    return guarded(g_error, [&] {
        require(grad_rows && indices && grad_table, "kge_op_scatter_add_rows: null argument");
        require(n <= (size_t)kMaxSortItems, "kge_op_scatter_add_rows: more rows than one sort block holds");
        for (size_t i = 0; i < n; ++i)
            if (indices[i] >= rows) fail(KGE_INVALID_ARGUMENT, msg() << "kge_op_scatter_add_rows: index " << indices[i] << " is not below " << rows);
        if (rows == 0 || width == 0) return;
        DeviceBuffer dg(n * width * 4), di(n * 4), dperm(n * 4), doff((rows + 1) * 4), dout(rows * width * 4);
        to_device(dg, grad_rows, n * width * 4);
        to_device(di, indices, n * 4);
        // All n lookups are passed as "head" lookups; there are no tail and no relation lookups.
        k_prepare_segments<<<1, 512>>>(di.as<uint32_t>(), di.as<uint32_t>(), nullptr, nullptr, (int)n, 0,
                                       (int)rows, 0, dperm.as<uint32_t>(), doff.as<uint32_t>(),
                                       nullptr, nullptr, nullptr, nullptr, nullptr, nullptr);
        k_segment_sum_rows<<<(unsigned)rows, 128>>>(dg.as<float>(), dperm.as<uint32_t>(), doff.as<uint32_t>(), width,
                                                    dout.as<float>());
        finish_kernels();
        to_host(grad_table, dout, rows * width * 4);
    });
}

int kge_op_activation(int kind, const float* x, const float* grad_out, size_t rows, size_t cols, float* y, float* grad_x) {
    return guarded(g_error, [&] {
        require(kind == 0 || kind == 1, "kge_op_activation: kind must be 0 (log-sigmoid) or 1 (log-softmax)");
        require(x && grad_out && y && grad_x, "kge_op_activation: null argument");
        const size_t n = rows * cols;
        if (n == 0) return;
        DeviceBuffer dx(n * 4), dg(n * 4), dy(n * 4), dgx(n * 4);
        to_device(dx, x, n * 4);
        to_device(dg, grad_out, n * 4);
        if (kind == 0)
            k_log_sigmoid<<<std::min(blocks_for(n, 256), 1184u), 256>>>(dx.as<float>(), dg.as<float>(), n, dy.as<float>(), dgx.as<float>());
        else
            k_log_softmax<<<(unsigned)rows, 256>>>(dx.as<float>(), dg.as<float>(), (int)cols, dy.as<float>(), dgx.as<float>());
        finish_kernels();
        to_host(y, dy, n * 4);
        to_host(grad_x, dgx, n * 4);
    });
}

int kge_op_all_to_all(const float* in, size_t n_shard, size_t block, float* out) {
    return guarded(g_error, [&] {
        require(in && out, "kge_op_all_to_all: null argument");
        const size_t total = n_shard * n_shard * block;
        if (total == 0) return;
        // Each emulated shard s holds `in[s]` = n_shard blocks and sends block d into slot s of
        // shard d's receive buffer, with the same routing kernel the training step uses: the
        // hidden table is in[s] viewed as rows of `block` floats, the lookup is the identity.
        DeviceBuffer din(total * 4), dout(total * 4), didx(n_shard * 4), dtable(n_shard * sizeof(float*));
        to_device(din, in, total * 4);
        std::vector<uint32_t> identity(n_shard);
        for (size_t i = 0; i < n_shard; ++i) identity[i] = (uint32_t)i;
        to_device(didx, identity.data(), n_shard * 4);
        for (size_t s = 0; s < n_shard; ++s) {
            std::vector<float*> dst(n_shard);
            for (size_t d = 0; d < n_shard; ++d) dst[d] = dout.as<float>() + (d * n_shard + s) * block;
            to_device(dtable, dst.data(), n_shard * sizeof(float*));
            const float* rows = din.as<float>() + s * n_shard * block;
            if (block % 4 == 0)
                k_route<4><<<(unsigned)n_shard, 64>>>(rows, rows, didx.as<uint32_t>(), nullptr, nullptr, nullptr,
                                                      dtable.as<float*>(), nullptr, (int)n_shard, 1, 0, (int)block, SCORE_TRANSE, ExchangeSync{});
            else
                k_route<1><<<(unsigned)n_shard, 64>>>(rows, rows, didx.as<uint32_t>(), nullptr, nullptr, nullptr,
                                                      dtable.as<float*>(), nullptr, (int)n_shard, 1, 0, (int)block, SCORE_TRANSE, ExchangeSync{});
            finish_kernels();
        }
        to_host(out, dout, total * 4);
    });
}

// Operator form of the tensor-core contraction (tc_gemm.cuh) on host buffers:
//   out[z, m, n] = epilogue( sum_{k in split z} A[m, k] * B[n, k] )
// `a` is the stored A matrix [a_rows, a_cols] (fp32 or fp16), read as A[m, k] = a[m, k], or
// a[k, m] when a_transposed; its stored rows may be picked by `a_gather`.  `b` likewise (fp32).
int kge_op_tc_gemm(const void* a, int a_half, int a_transposed, const uint32_t* a_gather, size_t a_rows, size_t a_cols,
                   const float* b, int b_transposed, size_t b_rows, size_t b_cols, size_t m, size_t n, size_t k,
                   int epilogue, const float* x, int splits, int tile_n, float* out) {
    return guarded(g_error, [&] {
        require(a && b && out, "kge_op_tc_gemm: null argument");
        require(epilogue >= 0 && epilogue <= 2 && (epilogue == 0 || x), "kge_op_tc_gemm: bad epilogue or missing x");
        require(splits >= 1 && (tile_n == 64 || tile_n == 128), "kge_op_tc_gemm: splits >= 1 and tile_n in {64, 128}");
        require(m > 0 && n > 0, "kge_op_tc_gemm: empty output");
        const size_t ea = a_half ? 2 : 4;
        const size_t gather_len = a_transposed ? k : m;
        if (a_gather)
            for (size_t i = 0; i < gather_len; ++i)
                if (a_gather[i] >= a_rows) fail(KGE_INVALID_ARGUMENT, "kge_op_tc_gemm: gather index out of range");
        require(a_gather || a_rows >= (a_transposed ? k : m), "kge_op_tc_gemm: a has too few rows");
        require(a_cols >= (a_transposed ? m : k), "kge_op_tc_gemm: a has too few columns");
        require(b_rows >= (b_transposed ? k : n) && b_cols >= (b_transposed ? n : k), "kge_op_tc_gemm: b is too small");
        DeviceBuffer da(a_rows * a_cols * ea), db(b_rows * b_cols * 4), dout((size_t)splits * m * n * 4), dx(m * n * 4);
        DeviceBuffer dg(gather_len * 4), dstatus(4);
        to_device(da, a, a_rows * a_cols * ea);
        to_device(db, b, b_rows * b_cols * 4);
        if (x) to_device(dx, x, m * n * 4);
        if (a_gather) to_device(dg, a_gather, gather_len * 4);
        KGE_CUDA(cudaMemset(dstatus.p, 0, 4));
        tc::GemmArgs g{};
        g.A = tc::make_operand(da.p, (long long)(a_cols * ea), a_half != 0, a_transposed != 0, a_gather ? dg.as<uint32_t>() : nullptr);
        g.B = tc::make_operand(db.p, (long long)(b_cols * 4), false, b_transposed != 0);
        g.M = (int)m; g.N = (int)n; g.K = (int)k;
        g.k_per_split = (int)(((k + splits - 1) / splits + 31) / 32 * 32);
        if (g.k_per_split == 0) g.k_per_split = 32;
        g.epilogue = epilogue;
        g.out = dout.as<float>(); g.out_blocks = nullptr; g.block_rows = 1;
        g.ldc = (long long)n; g.split_stride = (long long)(m * n);
        g.x_base = static_cast<const uint8_t*>(dx.p); g.x_row_stride_bytes = (long long)(n * 4);
        g.x_gather = nullptr; g.x_row_base = 0; g.x_is_half = 0;
        g.status = dstatus.as<unsigned>();
        const bool exact = a_half != 0, rowsum = epilogue == tc::EPI_ROWSUM_X_MINUS;
        cudaError_t err = cudaSuccess;
        KGE_CUDA(cudaMemset(dout.p, 0, (size_t)splits * m * n * 4));
        if (tile_n == 64) {
            if (exact) err = rowsum ? tc::launch_pair<64, true, true>(&g, 1, splits, nullptr) : tc::launch_pair<64, true, false>(&g, 1, splits, nullptr);
            else err = rowsum ? tc::launch_pair<64, false, true>(&g, 1, splits, nullptr) : tc::launch_pair<64, false, false>(&g, 1, splits, nullptr);
        } else {
            // the 128-column tile exists only in the unpipelined form
            if (exact) err = rowsum ? tc::launch<128, true, true>(g, splits, nullptr) : tc::launch<128, true, false>(g, splits, nullptr);
            else err = rowsum ? tc::launch<128, false, true>(g, splits, nullptr) : tc::launch<128, false, false>(g, splits, nullptr);
        }
        KGE_CUDA(err);
        finish_kernels();
        unsigned status = 0;
        KGE_CUDA(cudaMemcpy(&status, dstatus.p, 4, cudaMemcpyDeviceToHost));
        if (status) fail(KGE_DEVICE_STATUS, msg() << "kge_op_tc_gemm: a bounded wait on the tensor-core pipeline gave up (code " << status << ")");
        to_host(out, dout, (size_t)splits * m * n * 4);
    });
}

// Operator form of the plane-fed contraction (tc_planes.cuh) on host buffers.  The stored matrices
// are split into their TF32-exact planes on the device, as the producing kernels of the training
// step do, and the k splits (a thread-block cluster) are reduced inside the kernel.
//   out[m, n] = epilogue( sum_k A[m, k] * B[n, k] )
// a: stored [a_rows, a_cols] fp32; A[m, k] = a[m, k], or a[k, m] when a_mn_major.  a_exact: the
// values are exact in TF32 (they came from fp16), one plane.  b likewise.  The upper plane is the
// stored array itself (the tensor core ignores the low 13 bits of a TF32 operand);
// hi_is_cleared: a copy with those bits cleared is used instead, which must give the same bits.
// repeat > 0: the launch is repeated that many times between two events and *mean_us receives the
// mean device time per launch.
int kge_op_tc_planes(const float* a, int a_mn_major, int a_exact, size_t a_rows, size_t a_cols, const float* b, int b_mn_major,
                     size_t b_rows, size_t b_cols, size_t m, size_t n, size_t k, int epilogue, const float* x, int splits,
                     int tile_n, int hi_is_cleared, int repeat, float* mean_us, float* out) {
    return guarded(g_error, [&] {
        require(a && b && out, "kge_op_tc_planes: null argument");
        require(epilogue >= 0 && epilogue <= 3 && (epilogue == 0 || epilogue == 3 || x), "kge_op_tc_planes: bad epilogue or missing x");
        require(epilogue != 3 || (!a_mn_major && !b_mn_major), "kge_op_tc_planes: the distance epilogue needs both operands stored [mn][k]");
        require(splits >= 1 && splits <= tc::kMaxClusterSplits, "kge_op_tc_planes: splits must be between 1 and 8");
        require(tile_n == 64 || tile_n == 128, "kge_op_tc_planes: tile_n must be 64 or 128");
        require(m > 0 && n > 0 && k > 0, "kge_op_tc_planes: empty problem");
        require(a_rows >= (a_mn_major ? k : m) && a_cols >= (a_mn_major ? m : k), "kge_op_tc_planes: a is too small");
        require(b_rows >= (b_mn_major ? k : n) && b_cols >= (b_mn_major ? n : k), "kge_op_tc_planes: b is too small");
        require(a_cols % 4 == 0 && b_cols % 4 == 0, "kge_op_tc_planes: stored rows must be a multiple of 16 bytes");
        const size_t na = a_rows * a_cols, nb = b_rows * b_cols;
        DeviceBuffer da(na * 4), da_hi(na * 4), da_lo(na * 4), db(nb * 4), db_hi(nb * 4), db_lo(nb * 4);
        DeviceBuffer dout(m * n * 4), dx(m * n * 4), dstatus(4);
        to_device(da, a, na * 4);
        to_device(db, b, nb * 4);
        if (x) to_device(dx, x, m * n * 4);
        KGE_CUDA(cudaMemset(dstatus.p, 0, 4));
        tc::k_split_planes<<<std::min(blocks_for(na, 256), 1184u), 256>>>(da.as<float>(), na, da_hi.as<float>(), da_lo.as<float>());
        tc::k_split_planes<<<std::min(blocks_for(nb, 256), 1184u), 256>>>(db.as<float>(), nb, db_hi.as<float>(), db_lo.as<float>());
        KGE_CUDA(cudaGetLastError());
        tc::PlaneProblem p{};
        p.A = {hi_is_cleared ? da_hi.as<float>() : da.as<float>(), a_exact ? nullptr : da_lo.as<float>(), (long long)(a_cols * 4), a_mn_major ? 1 : 0};
        p.B = {hi_is_cleared ? db_hi.as<float>() : db.as<float>(), db_lo.as<float>(), (long long)(b_cols * 4), b_mn_major ? 1 : 0};
        tc::GemmArgs& g = p.g;
        g.M = (int)m; g.N = (int)n; g.K = (int)k;
        g.k_per_split = std::max(32, (int)(((k + splits - 1) / splits + 31) / 32 * 32));
        g.epilogue = epilogue;
        g.out = dout.as<float>(); g.out_blocks = nullptr; g.block_rows = 1;
        g.ldc = (long long)n; g.split_stride = 0;
        g.x_base = static_cast<const uint8_t*>(dx.p); g.x_row_stride_bytes = (long long)(n * 4);
        g.status = dstatus.as<unsigned>();
        tc::PlaneLaunch prepared;
        KGE_CUDA(tc::prepare_planes(&p, 1, splits, tile_n, &prepared));
        auto run = [&] {
            if (epilogue == tc::EPI_ROWSUM_X_MINUS) return tc::launch_prepared<tc::SIDE_ROWSUM>(prepared, nullptr);
            if (epilogue == tc::EPI_L2_DISTANCE) return tc::launch_prepared<tc::SIDE_NORMS>(prepared, nullptr);
            return tc::launch_prepared<tc::SIDE_NONE>(prepared, nullptr);
        };
        KGE_CUDA(run());
        finish_kernels();
        if (repeat > 0) {
            cudaEvent_t e0 = nullptr, e1 = nullptr;
            KGE_CUDA(cudaEventCreate(&e0));
            KGE_CUDA(cudaEventCreate(&e1));
            KGE_CUDA(cudaEventRecord(e0, nullptr));
            cudaError_t err = cudaSuccess;
            for (int it = 0; it < repeat && err == cudaSuccess; ++it) err = run();
            KGE_CUDA(cudaEventRecord(e1, nullptr));
            KGE_CUDA(cudaEventSynchronize(e1));
            float ms = 0.f;
            KGE_CUDA(cudaEventElapsedTime(&ms, e0, e1));
            cudaEventDestroy(e0);
            cudaEventDestroy(e1);
            KGE_CUDA(err);
            if (mean_us) *mean_us = 1e3f * ms / (float)repeat;
        }
        unsigned status = 0;
        KGE_CUDA(cudaMemcpy(&status, dstatus.p, 4, cudaMemcpyDeviceToHost));
        if (status) fail(KGE_DEVICE_STATUS, msg() << "kge_op_tc_planes: a bounded wait on the tensor-core pipeline gave up (code " << status << ")");
        to_host(out, dout, m * n * 4);
    });
}

// ---------------------------------------------------------------------------
// Device-timed single kernels for the microbenchmark (the reference's only kernel benchmark is
// tests/pag/testPag.cpp:321-332; its whole-program profile is scripts/run_profile.py).  Inputs are
// made on the device, the kernel under test is the one the training step launches, and the mean of
// `repeat` back-to-back launches between two CUDA events is returned.

}  // extern "C"

namespace {
static __global__ void k_fill_pattern(float* p, size_t n, uint32_t seed) {
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        uint32_t h = (uint32_t)e * 2654435761u + seed;
        h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
        p[e] = ((float)(h >> 8) * (1.0f / 16777216.0f) - 0.5f) * 0.25f;
    }
}
template <class Launch>
float timed_launches(int repeat, Launch&& launch) {
    KGE_CUDA(launch());
    finish_kernels();
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    KGE_CUDA(cudaEventCreate(&e0));
    KGE_CUDA(cudaEventCreate(&e1));
    KGE_CUDA(cudaEventRecord(e0, nullptr));
    cudaError_t err = cudaSuccess;
    for (int it = 0; it < repeat && err == cudaSuccess; ++it) err = launch();
    KGE_CUDA(cudaEventRecord(e1, nullptr));
    KGE_CUDA(cudaEventSynchronize(e1));
    float ms = 0.f;
    KGE_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    KGE_CUDA(err);
    return 1e3f * ms / (float)repeat;
}
}  // namespace

extern "C" {

// The same contraction on bfloat16 operands (tcgen05.mma.kind::f16, fp32 accumulation): the form of
// the 2e-2 tier (bf16 embeddings).  The host arrays are fp32; they are rounded to bf16 on the device.
int kge_op_tc_planes_bf16(const float* a, int a_mn_major, size_t a_rows, size_t a_cols, const float* b, int b_mn_major, size_t b_rows,
                          size_t b_cols, size_t m, size_t n, size_t k, int splits, int tile_n, int repeat, float* mean_us, float* out) {
    return guarded(g_error, [&] {
        require(a && b && out, "kge_op_tc_planes_bf16: null argument");
        require(splits >= 1 && splits <= tc::kMaxClusterSplits, "kge_op_tc_planes_bf16: splits must be between 1 and 8");
        require(tile_n == 64 || tile_n == 128, "kge_op_tc_planes_bf16: tile_n must be 64 or 128");
        require(m > 0 && n > 0 && k > 0, "kge_op_tc_planes_bf16: empty problem");
        require(a_rows >= (a_mn_major ? k : m) && a_cols >= (a_mn_major ? m : k), "kge_op_tc_planes_bf16: a is too small");
        require(b_rows >= (b_mn_major ? k : n) && b_cols >= (b_mn_major ? n : k), "kge_op_tc_planes_bf16: b is too small");
        require(a_cols % 8 == 0 && b_cols % 8 == 0, "kge_op_tc_planes_bf16: stored rows must be a multiple of 16 bytes");
        const size_t na = a_rows * a_cols, nb = b_rows * b_cols;
        DeviceBuffer da(na * 4), db(nb * 4), da16(na * 2), db16(nb * 2), dout(m * n * 4), dstatus(4);
        to_device(da, a, na * 4);
        to_device(db, b, nb * 4);
        KGE_CUDA(cudaMemset(dstatus.p, 0, 4));
        k_to_bf16<<<std::min(blocks_for(na, 256), 1184u), 256>>>(da.as<float>(), na, da16.as<__nv_bfloat16>());
        k_to_bf16<<<std::min(blocks_for(nb, 256), 1184u), 256>>>(db.as<float>(), nb, db16.as<__nv_bfloat16>());
        KGE_CUDA(cudaGetLastError());
        tc::PlaneProblem p{};
        p.A = {da16.as<float>(), nullptr, (long long)(a_cols * 2), a_mn_major ? 1 : 0, 2};
        p.B = {db16.as<float>(), nullptr, (long long)(b_cols * 2), b_mn_major ? 1 : 0, 2};
        tc::GemmArgs& g = p.g;
        g.M = (int)m; g.N = (int)n; g.K = (int)k;
        g.k_per_split = std::max(64, (int)(((k + splits - 1) / splits + 63) / 64 * 64));
        g.epilogue = tc::EPI_STORE;
        g.out = dout.as<float>(); g.block_rows = 1; g.ldc = (long long)n;
        g.status = dstatus.as<unsigned>();
        tc::PlaneLaunch prepared;
        KGE_CUDA(tc::prepare_planes(&p, 1, splits, tile_n, &prepared));
        auto run = [&] { return tc::launch_prepared<tc::SIDE_NONE>(prepared, nullptr); };
        if (repeat > 0 && mean_us) *mean_us = timed_launches(repeat, run);
        else {
            KGE_CUDA(run());
            finish_kernels();
        }
        unsigned status = 0;
        KGE_CUDA(cudaMemcpy(&status, dstatus.p, 4, cudaMemcpyDeviceToHost));
        if (status) fail(KGE_DEVICE_STATUS, msg() << "kge_op_tc_planes_bf16: a bounded wait on the tensor-core pipeline gave up (code " << status << ")");
        to_host(out, dout, m * n * 4);
    });
}

// kind 0: the step's row gather (k_gather_step_rows) of `n` rows of [value | adam_m | sqrt(adam_v)]
//         (3 * d fp32 per row) out of a table of `table_rows` rows into a compact copy;
// kind 1: the row-wise Adam scatter (k_entity_update with one lookup per row) on the same rows:
//         reads a gradient row and the gathered state, writes value / m / sqrt(v) back to the table.
// indices [n] are table rows (host array; for kind 1 they must be distinct).
int kge_microbench_rows(int kind, size_t table_rows, size_t d, const uint32_t* indices, size_t n, int repeat, float* mean_us) {
    return guarded(g_error, [&] {
        require(kind == 0 || kind == 1, "kge_microbench_rows: kind must be 0 (gather) or 1 (Adam scatter)");
        require(indices && mean_us && repeat > 0 && n > 0 && d > 0 && d % 4 == 0, "kge_microbench_rows: bad argument");
        for (size_t i = 0; i < n; ++i)
            if (indices[i] >= table_rows) fail(KGE_INVALID_ARGUMENT, "kge_microbench_rows: index out of range");
        RowLayout L{};
        L.d = (uint32_t)d; L.f = 0;
        L.off_m = (uint32_t)(d * 4); L.off_q = 2 * L.off_m; L.off_feat = 3 * L.off_m; L.row_bytes = L.off_feat;
        DeviceBuffer table(table_rows * L.row_bytes), rows_c(n * L.row_bytes), idx(n * 4);
        k_fill_pattern<<<1184, 256>>>(table.as<float>(), table_rows * 3 * d, 1u);
        KGE_CUDA(cudaGetLastError());
        to_device(idx, indices, n * 4);
        const FeaturePlanes no_planes{nullptr, nullptr, 0u, L.off_feat};
        auto gather = [&] {
            return launch_dependent(k_gather_step_rows, dim3(blocks_for(n, 8)), dim3(256), 0, nullptr, table.as<uint8_t>(), L.row_bytes,
                                    idx.as<uint32_t>(), (int)n, rows_c.as<uint8_t>(), no_planes);
        };
        if (kind == 0) {
            *mean_us = timed_launches(repeat, gather);
            return;
        }
        // one "head" lookup per gathered row: lookup i reads gradient row i and belongs to row i
        std::vector<uint32_t> iota(n + 1), ones(n, 1u);
        for (size_t i = 0; i <= n; ++i) iota[i] = (uint32_t)i;
        DeviceBuffer perm(n * 4), off((n + 1) * 4), first(n * 4), grads(n * d * 4), d_hid(n * d * 4), step_size(4), heavy_count(4);
        to_device(perm, iota.data(), n * 4);
        to_device(off, iota.data(), (n + 1) * 4);
        to_device(first, ones.data(), n * 4);
        const float alpha = 1e-3f;
        to_device(step_size, &alpha, 4);
        KGE_CUDA(cudaMemset(heavy_count.p, 0, 4));
        k_fill_pattern<<<1184, 256>>>(grads.as<float>(), n * d, 7u);
        KGE_CUDA(gather());
        finish_kernels();
        const AdamParams ap{0.9f, 0.999f, 0.1f, 0.001f, 1e-8f, 0.f};
        // the rows' descriptors, as k_prepare_segments leaves them: one lookup per row, every row writes
        std::vector<uint4> info(2 * n);
        for (size_t i = 0; i < n; ++i) {
            info[2 * i] = make_uint4((uint32_t)i, 1u, 1u, indices[i]);
            info[2 * i + 1] = make_uint4((uint32_t)i, 0xffffffffu, 0xffffffffu, 0xffffffffu);
        }
        DeviceBuffer row_info(2 * n * sizeof(uint4));
        to_device(row_info, info.data(), 2 * n * sizeof(uint4));
        const HeavyRows heavy{nullptr, heavy_count.as<uint32_t>(), nullptr, nullptr, row_info.as<uint4>()};
        *mean_us = timed_launches(repeat, [&] {
            return launch_dependent(k_entity_update<float, 4>, dim3((unsigned)(kHeavySlots + blocks_for(n, kRowsPerBlock))), dim3(64 * kSegmentLanes), 0, nullptr, table.as<uint8_t>(),
                                    rows_c.as<uint8_t>(), L, idx.as<uint32_t>(), perm.as<uint32_t>(), off.as<uint32_t>(), first.as<uint32_t>(),
                                    grads.as<float>(), grads.as<float>(), (int)n, d_hid.as<float>(), (float*)nullptr, step_size.as<float>(), 1.0f, ap,
                                    ExchangeSync{}, heavy, (int)n, RelationRows{});
        });
    });
}

// Scores of m queries against n shared tails, k deep, device-resident: fn 0 = L1 and 1 = L2 on the
// FP32 pipe (k_score_wide), 2 = dot product and 3 = L2 in the form |a|^2 + |b|^2 - 2 a.b on the tensor
// cores (k_tc_planes, 3xTF32).
int kge_microbench_scores(int fn, size_t m, size_t n, size_t k, int repeat, float* mean_us) {
    return guarded(g_error, [&] {
        require(fn >= 0 && fn <= 3 && mean_us && repeat > 0 && m > 0 && n > 0 && k > 0 && k % 4 == 0, "kge_microbench_scores: bad argument");
        DeviceBuffer a(m * k * 4), b(n * k * 4), a_lo(m * k * 4), b_lo(n * k * 4), out(m * n * 4), status(4);
        k_fill_pattern<<<1184, 256>>>(a.as<float>(), m * k, 3u);
        k_fill_pattern<<<1184, 256>>>(b.as<float>(), n * k, 5u);
        k_lower_plane<<<1184, 256>>>(a.as<float>(), m * k, a_lo.as<float>());
        k_lower_plane<<<1184, 256>>>(b.as<float>(), n * k, b_lo.as<float>());
        KGE_CUDA(cudaMemset(status.p, 0, 4));
        KGE_CUDA(cudaGetLastError());
        if (fn <= 1) {
            *mean_us = timed_launches(repeat, [&] { return launch_score(fn, a.as<float>(), b.as<float>(), out.as<float>(), (int)m, (int)n, (int)k, nullptr); });
            return;
        }
        tc::PlaneProblem p{};
        p.A = {a.as<float>(), a_lo.as<float>(), (long long)(k * 4), 0};
        p.B = {b.as<float>(), b_lo.as<float>(), (long long)(k * 4), 0};
        p.g.M = (int)m; p.g.N = (int)n; p.g.K = (int)k;
        p.g.epilogue = fn == 3 ? tc::EPI_L2_DISTANCE : tc::EPI_STORE;
        p.g.out = out.as<float>(); p.g.ldc = (long long)n; p.g.block_rows = 1;
        p.g.status = status.as<unsigned>();
        const unsigned tiles = blocks_for(m, 128) * blocks_for(n, 128);
        int splits = (int)std::min<unsigned>({std::max(1u, 148u / tiles), std::max(1u, (unsigned)k / 64u), (unsigned)tc::kMaxClusterSplits});
        while (splits > 1 && (unsigned)tc::max_resident_plane_clusters(splits) < tiles) --splits;
        p.g.k_per_split = std::max(32, (int)(((k + splits - 1) / splits + 31) / 32 * 32));
        tc::PlaneLaunch prepared;
        KGE_CUDA(tc::prepare_planes(&p, 1, splits, 128, &prepared));
        *mean_us = timed_launches(repeat, [&] {
            return fn == 3 ? tc::launch_prepared<tc::SIDE_NORMS>(prepared, nullptr) : tc::launch_prepared<tc::SIDE_NONE>(prepared, nullptr);
        });
    });
}

// ---------------------------------------------------------------------------
// Scatter-add for callers that must not allocate.
//
// The sort-and-segment scatter-add needs working memory beyond its inputs and outputs: the
// lookups ordered by row and the start of each row's segment.  kge_op_scatter_add_rows gets it
// from cudaMalloc.  Some callers cannot: a plugin running inside another framework's memory
// pool, where a raw cudaMalloc fragments or exceeds the pool's budget; a service with a fixed
// device-memory reservation; code on a latency path where the implicit device synchronisation
// of cudaMalloc / cudaFree is not acceptable.  For them the working memory is this fixed array
// in the library's own device image.  Every GPU that loads the library holds it (about 272 KB)
// until the process exits.
constexpr size_t kNoAllocMaxLookups = kMaxSortItems;  // 4096
constexpr size_t kNoAllocMaxRows = 65536;

struct NoAllocScratch {
    uint32_t perm[kNoAllocMaxLookups];      // lookups ordered by (row, position)
    uint32_t offsets[kNoAllocMaxRows + 1];  // segment start of each table row
};

static __device__ __align__(256) unsigned char g_no_alloc_scratch[sizeof(NoAllocScratch)];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_no_alloc_mutex;
NoAllocScratch* g_no_alloc_ptr[kMaxDevices] = {};

// The array's name is only a host-side handle; the kernels need its address on the current
// device, which the runtime hands out per device.
NoAllocScratch* no_alloc_scratch_for_current_device() {
    int device = -1;
    KGE_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) fail(KGE_RUNTIME_ERROR, "kge_op_scatter_add_rows_noalloc: device ordinal out of range");
    std::lock_guard<std::mutex> lock(g_no_alloc_mutex);
    if (!g_no_alloc_ptr[device]) {
        void* ptr = nullptr;
        KGE_CUDA(cudaGetSymbolAddress(&ptr, g_no_alloc_scratch));
        g_no_alloc_ptr[device] = static_cast<NoAllocScratch*>(ptr);
    }
    return g_no_alloc_ptr[device];
}
}  // namespace

int kge_op_scatter_add_rows_noalloc(const float* grad_rows, const uint32_t* indices, size_t n, size_t rows, size_t width,
                                    float* grad_table, void* cuda_stream) {
    return guarded(g_error, [&] {
        require(grad_table && (n == 0 || (grad_rows && indices)), "kge_op_scatter_add_rows_noalloc: null argument");
        if (n > kNoAllocMaxLookups)
            fail(KGE_INVALID_ARGUMENT, msg() << "kge_op_scatter_add_rows_noalloc: " << n << " lookups exceed the fixed working memory ("
                                             << kNoAllocMaxLookups << " lookups)");
        if (rows > kNoAllocMaxRows)
            fail(KGE_INVALID_ARGUMENT, msg() << "kge_op_scatter_add_rows_noalloc: " << rows << " table rows exceed the fixed working memory ("
                                             << kNoAllocMaxRows << " rows)");
        if (rows == 0 || width == 0) return;
        NoAllocScratch* scratch = no_alloc_scratch_for_current_device();
        cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
        // Every entry the second kernel reads (perm[0, n) and offsets[0, rows]) is rewritten by the
        // first, so nothing left by an earlier call is ever read and nothing needs clearing.
        k_prepare_segments<<<1, 512, 0, stream>>>(indices, indices, nullptr, nullptr, (int)n, 0, (int)rows, 0, scratch->perm,
                                                  scratch->offsets, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr);
        k_segment_sum_rows<<<(unsigned)rows, 128, 0, stream>>>(grad_rows, scratch->perm, scratch->offsets, width, grad_table);
        KGE_CUDA(cudaGetLastError());
    });
}

}  // extern "C"
