// The feature MLP of entityHidden (src/poplar_kge.cpp:453-458):
//   featureHidden = relu(concat(value, feature . W) . up) . down,   hidden = value + featureHidden,
// with up [2D, M] and down [M, D] per feature network.  The step computes `feature . W + value`
// with its usual kernel; what is here turns those rows into the MLP's output and carries the
// gradient back: a plain FP32 contraction kernel (any of A, A^T times B, B^T; relu on the A
// operand; a relu mask on the output), the concatenation, the final sum, the split of the input
// gradient into the value's share and the projection's, the deferred row-wise Adam step, and the
// hand-over of a parameter gradient to the processes that own its rows.  Not on any measured
// configuration's path: written for fixed summation order and parity, not for speed.
#pragma once

#include "kernels.cuh"

namespace kge {

struct SgemmArgs {
    const float* A; long long lda; int a_trans; int a_relu;  // A(m, k) = a_trans ? A[k * lda + m] : A[m * lda + k], max(., 0) when a_relu
    const float* B; long long ldb; int b_trans;              // B(k, n) = b_trans ? B[n * ldb + k] : B[k * ldb + n]
    float* C; long long ldc;
    int M, N, K;
    const float* pass; long long ldpass;  // optional [M, N]: C = acc where pass >= 0, else 0 (backward of max(x, 0), src/pag/pag.cpp:650-658)
};

// C = A . B, one 64 x 64 tile per block, 4 x 4 outputs per thread, k in steps of 16.
static __global__ void __launch_bounds__(256) k_sgemm(SgemmArgs g) {
    grid_dependency_sync();
    __shared__ float As[16][64 + 4], Bs[16][64 + 4];
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < g.K; k0 += 16) {
        for (int idx = threadIdx.x; idx < 16 * 64; idx += 256) {
            // the index that is contiguous in memory runs fastest across the threads
            const int kk_a = g.a_trans ? idx / 64 : idx % 16, mm = g.a_trans ? idx % 64 : idx / 16;
            const int m = m0 + mm, ka = k0 + kk_a;
            float a = 0.f;
            if (m < g.M && ka < g.K) a = g.a_trans ? g.A[(size_t)ka * g.lda + m] : g.A[(size_t)m * g.lda + ka];
            As[kk_a][mm] = g.a_relu ? fmaxf(a, 0.f) : a;
            const int kk_b = g.b_trans ? idx % 16 : idx / 64, nn = g.b_trans ? idx / 16 : idx % 64;
            const int n = n0 + nn, kb = k0 + kk_b;
            float b = 0.f;
            if (n < g.N && kb < g.K) b = g.b_trans ? g.B[(size_t)n * g.ldb + kb] : g.B[(size_t)kb * g.ldb + n];
            Bs[kk_b][nn] = b;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i], b[i] = Bs[kk][tx * 4 + i];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= g.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= g.N) continue;
            float v = acc[i][j];
            if (g.pass && !(g.pass[(size_t)m * g.ldpass + n] >= 0.f)) v = 0.f;
            g.C[(size_t)m * g.ldc + n] = v;
        }
    }
}

inline cudaError_t launch_sgemm(const SgemmArgs& g, cudaStream_t stream) {
    if (g.M <= 0 || g.N <= 0) return cudaSuccess;
    return launch_dependent(k_sgemm, dim3((unsigned)((g.N + 63) / 64), (unsigned)((g.M + 63) / 64)), dim3(256), 0, stream, g);
}

// Row i of the MLP's input: value | hidden - value, the value read from row `index[i]` (or
// start + i) of `rows` in the table's row layout; `hid` holds value + feature . W.
template <class ST>
static __global__ void __launch_bounds__(256)
k_mlp_concat(const uint8_t* __restrict__ rows, RowLayout L, const uint32_t* __restrict__ index, uint32_t start, int n,
             const float* __restrict__ hid, float* __restrict__ cat) {
    grid_dependency_sync();
    const int D = (int)L.d;
    for (size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x; idx < (size_t)n * D; idx += (size_t)gridDim.x * 256) {
        const int i = (int)(idx / D), c = (int)(idx - (size_t)i * D);
        const uint8_t* row = rows + (size_t)(index ? index[i] : start + (uint32_t)i) * L.row_bytes;
        const float v = load_value<ST>(L, row, c);
        cat[(size_t)i * 2 * D + c] = v;
        cat[(size_t)i * 2 * D + D + c] = hid[idx] - v;
    }
}

// hid = value + fh (same addressing of the value).
template <class ST>
static __global__ void __launch_bounds__(256)
k_mlp_finish(const uint8_t* __restrict__ rows, RowLayout L, const uint32_t* __restrict__ index, uint32_t start, int n,
             const float* __restrict__ fh, float* __restrict__ hid) {
    grid_dependency_sync();
    const int D = (int)L.d;
    for (size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x; idx < (size_t)n * D; idx += (size_t)gridDim.x * 256) {
        const int i = (int)(idx / D), c = (int)(idx - (size_t)i * D);
        const uint8_t* row = rows + (size_t)(index ? index[i] : start + (uint32_t)i) * L.row_bytes;
        hid[idx] = load_value<ST>(L, row, c) + fh[idx];
    }
}

// The gradient of the MLP's input [R, 2D]: its first half joins the value's gradient, its second
// half is the gradient of feature . W (it replaces the gradient of the MLP's output in d_hid).
static __global__ void __launch_bounds__(256)
k_mlp_split(const float* __restrict__ d_cat, float* __restrict__ d_val, float* __restrict__ d_hid, int R, int D) {
    grid_dependency_sync();
    for (size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x; idx < (size_t)R * D; idx += (size_t)gridDim.x * 256) {
        const size_t r = idx / D, c = idx - r * D;
        d_val[idx] += d_cat[r * 2 * D + c];
        d_hid[idx] = d_cat[r * 2 * D + D + c];
    }
}

// Row-wise Adam of the gathered rows from a complete gradient [R, D]: what k_entity_update does
// at the end of a row when nothing is deferred (src/poplar_kge.cpp:692-704; the row keeps
// sqrt(adam_v)).  The state before the update comes from the step's gathered copy; only the
// first slot of a table row writes.
template <class ST>
static __global__ void __launch_bounds__(256)
k_row_adam(uint8_t* __restrict__ table, const uint8_t* __restrict__ rows_c, RowLayout L, const uint32_t* __restrict__ remote,
           const uint32_t* __restrict__ first_slot, const float* __restrict__ grad, const float* __restrict__ step_size,
           float lr_modifier, AdamParams ap, int R) {
    grid_dependency_sync();
    const int D = (int)L.d;
    const float alpha = *step_size * lr_modifier;
    for (size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x; idx < (size_t)R * D; idx += (size_t)gridDim.x * 256) {
        const int r = (int)(idx / D), c = (int)(idx - (size_t)r * D);
        if (!(first_slot[r] & 1u)) continue;
        const uint8_t* src = rows_c + (size_t)r * L.row_bytes;
        uint8_t* dst = table + (size_t)remote[r] * L.row_bytes;
        float x = load_value<ST>(L, src, c);
        float m = load_as_float(reinterpret_cast<const ST*>(src + L.off_m) + c);
        const float q = load_as_float(reinterpret_cast<const ST*>(src + L.off_q) + c);
        const float g = grad[idx];
        float v = q * q;
        m = ap.beta_m * m + ap.one_minus_beta_m * g;
        v = ap.beta_v * v + ap.one_minus_beta_v * g * g;
        x = x - alpha * (m / (sqrtf(v) + ap.epsilon) + ap.weight_decay * x);
        store_value<ST>(L, dst, c, x);
        store_from_float(reinterpret_cast<ST*>(dst + L.off_m) + c, m);
        store_from_float(reinterpret_cast<ST*>(dst + L.off_q) + c, sqrtf(v));
    }
}

// A shard's gradient of a dense parameter, `n_rows` rows of D floats beginning at row `row0` of
// the dense vector, into the slots of the processes that own those rows (row r to process
// r % n_owner as its row r / n_owner).
static __global__ void __launch_bounds__(256)
k_push_dense_rows(const float* __restrict__ src, int n_rows, int row0, int D, float* const* __restrict__ dense_dst, int n_owner) {
    grid_dependency_sync();
    for (size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x; idx < (size_t)n_rows * D; idx += (size_t)gridDim.x * 256) {
        const size_t r = idx / D, c = idx - r * D, row = r + (size_t)row0;
        dense_dst[row % n_owner][(row / n_owner) * D + c] = src[idx];
    }
}

}  // namespace kge
