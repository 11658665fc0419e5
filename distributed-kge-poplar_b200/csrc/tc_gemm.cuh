// Dense contractions of the training step on the 5th-generation tensor cores (tcgen05, sm_100a).
//
//   acc[m, n] = sum_k A[m, k] * B[n, k]          A: M x K, B: N x K, fp32 result
//
// The reference multiplies in fp32 (src/pag/pag.cpp:681-699 on FLOAT tensors), and parity is
// judged at 1e-5, which a single TF32 product (11-bit significands) cannot give.  Each operand
// is therefore split into two TF32-exact parts, x = hi + lo with hi = x with its low 13
// significand bits cleared and lo = (x - hi) likewise cleared, and three products are
// accumulated in the fp32 TMEM accumulator: hi*hi + hi*lo + lo*hi (the dropped lo*lo term and
// the second truncation are each below 2^-21 of |x||y|).  An operand that comes from fp16
// storage is exact in TF32 and needs no lo part.
//
// One CTA owns a 128 x BN output tile.  Per 32-deep k slice all 128 threads bring the two operand
// tiles from global memory (L2-resident at the step's sizes; rows may be gathered through an
// index, may be fp16, and may be stored k-major or mn-major), split them and write them to
// shared memory in the K-major 128-byte-swizzled layout the UMMA descriptors describe; one thread
// then issues the tcgen05.mma instructions of the slice into a TMEM tile of its own and commits
// them to an mbarrier; while they run, the threads read the previous slice's tile from TMEM
// (tcgen05.ld, one lane = one output row) and add it to register accumulators, and then stage the
// next slice (two stages of shared memory and of TMEM).  The epilogue applies one of:
//   out = acc                                  (dot scores, projection gradient, dot backward)
//   out = acc + value[row]                     (hidden = value + feature . W)
//   out = rowsum(A)[m] * X[m, n] - acc         (L2 backward in contraction form, see engine.cu)
// Every wait on an mbarrier is bounded; on expiry the kernel records an error word and goes on
// to its clean-up (TMEM is always released).
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "exchange.cuh"
#include "pdl.cuh"

namespace kge {
namespace tc {

constexpr int kBM = 128;      // UMMA M
constexpr int kBK = 32;       // fp32 elements per k slice: one 128-byte swizzle row
constexpr int kStages = 2;
constexpr int kThreads = 128;

enum Epilogue : int { EPI_STORE = 0, EPI_ADD_TABLE_VALUE = 1, EPI_ROWSUM_X_MINUS = 2, EPI_DENSE_ADAM = 4 };  // (3: the L2 distance of tc_planes.cuh)

// EPI_DENSE_ADAM: the contraction is the gradient of a dense parameter that no other shard contributes
// to, and the epilogue is the parameter's Adam step (src/fructose/frnn.cpp:61-90) in place: output
// element (m, n) is element (m + block_row_offset) * ldc + n of the dense vector.  X is the parameter
// itself (x_base, fetched while the partial tiles travel).  Null w: not in use.
struct DenseAdamArgs {
    float* w;
    float* w_lo;  // lower TF32 plane of the parameter (null: none kept)
    float* m;
    float* v;
    const float* step_size;  // on the device: a replayed graph keeps its arguments
    float lr_modifier;
    float beta_m, beta_v, one_minus_beta_m, one_minus_beta_v, epsilon, weight_decay;
};

// One operand as it lies in global memory.  Element (r, c) of the stored matrix is at
//   base + (gather ? gather[r] : r) * row_stride_bytes + c * (is_half ? 2 : 4).
// transposed == 0: stored rows are the operand's m / n index, columns are k (k contiguous);
// transposed == 1: stored rows are k, columns are m / n.
struct Operand {
    const uint8_t* base;
    long long row_stride_bytes;
    const uint32_t* gather;
    int is_half;
    int transposed;
    int vec_ok;  // rows start on a 16-byte (fp32) / 8-byte (fp16) boundary: 4-element vector loads allowed
};

struct GemmArgs {
    Operand A, B;
    int M, N, K;
    int k_per_split;            // k range of blockIdx.z is [z * k_per_split, min(K, (z + 1) * k_per_split))
    int epilogue;
    // output: row m at out + m * ldc (+ blockIdx.z * split_stride), or, when out_blocks is set, at
    // out_blocks[(m + block_row_offset) / block_rows] + ((m + block_row_offset) % block_rows) * ldc (rows routed to their owners)
    float* out;
    float* const* out_blocks;
    int block_rows;
    int block_row_offset;  // with out_blocks: row m belongs to block (m + offset) / block_rows
    int block_cyclic;      // > 0: rows are dealt out in turn instead, row m + offset to block (m + offset) % block_cyclic, as its row (m + offset) / block_cyclic
    long long ldc;
    long long split_stride;
    // EPI_ADD_TABLE_VALUE: value row of output row m is x_base + (x_gather ? x_gather[m] : m) * x_row_stride_bytes
    // EPI_ROWSUM_X_MINUS:  X[m, n] fp32 at x_base + m * x_row_stride_bytes + n * 4
    const uint8_t* x_base;
    long long x_row_stride_bytes;
    const uint32_t* x_gather;
    uint32_t x_row_base;
    int x_is_half;              // EPI_ADD_TABLE_VALUE: 0 fp32 values, 1 fp16, 2 bfloat16
    DenseAdamArgs adam;         // EPI_DENSE_ADAM
    unsigned* status;           // device error word; non-zero = a bounded wait gave up
    // k split with a deterministic reduction (pipelined kernel only).  Every split writes its raw
    // partial tile to ws [splits, M, N] (and its partial row sums to ws_rowsum [splits, M]);
    // k_tc_reduce then adds the partials in split order and applies the epilogue.  Null ws: each
    // split applies the epilogue itself and writes its own output slice (out + z * split_stride).
    float* ws;
    float* ws_rowsum;
    int splits;
    // Set by launch_pair: the blocks of one output tile (one per split) form a thread-block cluster
    // and reduce their partial tiles through distributed shared memory; 0 = not a cluster launch.
    int cluster_splits;
};

// ---------------------------------------------------------------------------
// PTX wrappers

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.b32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after about a second and reports through `status`.
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, unsigned* status, unsigned code) {
    for (uint32_t spins = 0; spins < (1u << 22); ++spins)
        if (mbar_try_wait(bar, parity)) return;
    atomicExch(status, code);
}
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(columns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, TF32 inputs, fp32 accumulate, issued by one thread.
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The mbarrier gets one arrival when every MMA this thread has issued so far has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 consecutive accumulator columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte rows and the 128-byte swizzle:
// rows are 128 B apart, groups of 8 rows 1024 B apart (stride byte offset), leading byte offset
// 16 B (unused by this layout), descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor: fp32 accumulator (bits 4-5 = 1), A and B TF32 (format 2 at bits 7-9 and
// 10-12), both K-major (bits 15, 16 = 0), N / 8 at bits 17-22, M / 16 at bits 24-28.
__host__ __device__ constexpr uint32_t make_idesc_tf32(int m, int n) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---------------------------------------------------------------------------
// Operand staging

__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float(__float_as_uint(x) & 0xFFFFE000u); }

// Byte offset of element (row, k) inside a K-major tile with 128-byte rows under the 128-byte
// swizzle: the 16-byte chunk index is XOR-ed with the row index modulo 8.
__device__ __forceinline__ uint32_t sw128_offset(int row, int k) {
    return (uint32_t)row * 128u + ((((uint32_t)k >> 2) ^ ((uint32_t)row & 7u)) << 4) + (((uint32_t)k & 3u) << 2);
}

__device__ __forceinline__ const uint8_t* operand_row(const Operand& op, int r) {
    const size_t row = op.gather ? op.gather[r] : (uint32_t)r;
    return op.base + row * (size_t)op.row_stride_bytes;
}
__device__ __forceinline__ float operand_elem(const Operand& op, const uint8_t* row, int c) {
    return op.is_half ? __half2float(reinterpret_cast<const __half*>(row)[c]) : reinterpret_cast<const float*>(row)[c];
}

// Loads the [ROWS x 32] slice (mn0.., k0..) of an operand, splits it and stores hi (and lo) tiles.
// Elements outside [0, MN) x [k0, k_end) are zero.  With ROWSUM, each thread also adds the exact
// fp32 values it handles into per-row partial sums (the rows a thread handles never change).
template <int ROWS, bool WRITE_LO, bool ROWSUM>
__device__ __forceinline__ void stage_operand(const Operand& op, int mn0, int MN, int k0, int k_end, uint8_t* tile_hi,
                                              uint8_t* tile_lo, float (&rowsum)[ROWS / 16]) {
    const int tid = threadIdx.x;
    if (!op.transposed) {
        // 8 threads per row, 4 consecutive k each: coalesced 128-byte row segments
#pragma unroll
        for (int i = 0; i < ROWS / 16; ++i) {
            const int u = tid + i * kThreads, row = u >> 3, ch = u & 7;
            const int mn = mn0 + row, k = k0 + ch * 4;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (mn < MN && k < k_end) {
                const uint8_t* rp = operand_row(op, mn);
                if (op.vec_ok && k + 3 < k_end) {
                    if (op.is_half) {
                        const uint2 raw = *reinterpret_cast<const uint2*>(rp + (size_t)k * 2);
                        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
                        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
                    } else {
                        const float4 raw = *reinterpret_cast<const float4*>(rp + (size_t)k * 4);
                        v[0] = raw.x; v[1] = raw.y; v[2] = raw.z; v[3] = raw.w;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (k + j < k_end) v[j] = operand_elem(op, rp, k + j);
                }
            }
            if (ROWSUM) rowsum[i] += (v[0] + v[1]) + (v[2] + v[3]);
            float4 hi = make_float4(tf32_hi(v[0]), tf32_hi(v[1]), tf32_hi(v[2]), tf32_hi(v[3]));
            const uint32_t off = (uint32_t)row * 128u + (((uint32_t)ch ^ ((uint32_t)row & 7u)) << 4);
            *reinterpret_cast<float4*>(tile_hi + off) = hi;
            if (WRITE_LO) {
                float4 lo = make_float4(tf32_hi(v[0] - hi.x), tf32_hi(v[1] - hi.y), tf32_hi(v[2] - hi.z), tf32_hi(v[3] - hi.w));
                *reinterpret_cast<float4*>(tile_lo + off) = lo;
            }
        }
    } else {
        // stored rows are k: a warp covers patches of 8 consecutive m/n (32-byte global segments per
        // k) by 4 consecutive k; the 32 scalar stores of a patch fall into 32 different banks
        const int warp = tid >> 5, lane = tid & 31;
        const int r_in = lane & 7, k_in = lane >> 3;
#pragma unroll
        for (int i = 0; i < ROWS / 32; ++i) {
            const int row = (warp + 4 * i) * 8 + r_in, mn = mn0 + row;
            float part = 0.f;
#pragma unroll
            for (int kg = 0; kg < 8; ++kg) {
                const int kk = kg * 4 + k_in, k = k0 + kk;
                float v = 0.f;
                if (mn < MN && k < k_end) v = operand_elem(op, operand_row(op, k), mn);
                part += v;
                const float hi = tf32_hi(v);
                const uint32_t off = sw128_offset(row, kk);
                *reinterpret_cast<float*>(tile_hi + off) = hi;
                if (WRITE_LO) *reinterpret_cast<float*>(tile_lo + off) = tf32_hi(v - hi);
            }
            if (ROWSUM) rowsum[i] += part;
        }
    }
}

// ---------------------------------------------------------------------------
// The kernel.  Dynamic shared memory: kStages x (A_hi, A_lo, B_hi, B_lo) tiles, 1024-byte aligned.

template <int BN>
constexpr size_t smem_bytes() {
    return 1024 + (size_t)kStages * (2 * kBM * 128 + 2 * BN * 128);
}

template <int BN, bool A_EXACT, bool ROWSUM>
__global__ void __launch_bounds__(kThreads, 1) k_tc_gemm(GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bars[kStages];
    __shared__ uint32_t tmem_slot;
    __shared__ float s_rowsum[kBM];

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr uint32_t kATile = kBM * 128, kBTile = BN * 128, kStage = 2 * kATile + 2 * kBTile;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = blockIdx.x * kBM, n0 = blockIdx.y * BN;
    const int k_begin = blockIdx.z * g.k_per_split, k_end = min(g.K, k_begin + g.k_per_split);
    const int n_slices = max(0, (k_end - k_begin + kBK - 1) / kBK);

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&bars[s], 1);
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(&tmem_slot, kStages * BN);  // one accumulator tile per stage
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    grid_dependency_sync();
    const uint32_t tmem_base = tmem_slot;
    constexpr uint32_t idesc = make_idesc_tf32(kBM, BN);

    float rowsum[kBM / 16];
#pragma unroll
    for (int i = 0; i < kBM / 16; ++i) rowsum[i] = 0.f;
    float unused[BN / 16];
    // The tensor core truncates its fp32 accumulator once per MMA instruction, so a long k loop
    // accumulated in TMEM drifts by about (instructions / 2) ulp.  Each 32-deep slice is therefore
    // accumulated on its own in TMEM (12 instructions) and added here, in registers, with
    // round-to-nearest; slice j's MMAs run while slice j-1 is drained.
    float acc[BN];
#pragma unroll
    for (int j = 0; j < BN; ++j) acc[j] = 0.f;

    auto drain = [&](int slice) {
        const int b = slice % kStages;
        mbar_wait(&bars[b], (uint32_t)((slice / kStages) & 1), g.status, 1u);
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < BN; c0 += 32) {
            uint32_t r[32];
            tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(b * BN + c0), r);
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[c0 + j] += __uint_as_float(r[j]);
        }
        tc_fence_before();
    };

    for (int kc = 0; kc < n_slices; ++kc) {
        const int s = kc % kStages;
        // stage s (shared memory and TMEM tile) was released when slice kc - 2 was drained
        uint8_t* stage = smem + (size_t)s * kStage;
        uint8_t *a_hi = stage, *a_lo = stage + kATile, *b_hi = stage + 2 * kATile, *b_lo = b_hi + kBTile;
        const int k0 = k_begin + kc * kBK;
        stage_operand<kBM, !A_EXACT, ROWSUM>(g.A, m0, g.M, k0, k_end, a_hi, a_lo, rowsum);
        stage_operand<BN, true, false>(g.B, n0, g.N, k0, k_end, b_hi, b_lo, unused);
        fence_async_shared();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            const uint32_t tmem_acc = tmem_base + (uint32_t)(s * BN);
            const uint64_t da_hi = make_kmajor_sw128_desc(smem_u32(a_hi)), da_lo = make_kmajor_sw128_desc(smem_u32(a_lo));
            const uint64_t db_hi = make_kmajor_sw128_desc(smem_u32(b_hi)), db_lo = make_kmajor_sw128_desc(smem_u32(b_lo));
#pragma unroll
            for (int ks = 0; ks < kBK / 8; ++ks) {
                const uint64_t adv = (uint64_t)(ks * 32 >> 4);  // 8 TF32 = 32 bytes further along the swizzled row
                // small cross terms first, the large hi*hi term last
                umma_tf32(tmem_acc, da_hi + adv, db_lo + adv, idesc, ks > 0 ? 1u : 0u);
                if (!A_EXACT) umma_tf32(tmem_acc, da_lo + adv, db_hi + adv, idesc, 1u);
                umma_tf32(tmem_acc, da_hi + adv, db_hi + adv, idesc, 1u);
            }
            umma_commit(&bars[s]);
        }
        if (kc >= 1) drain(kc - 1);
    }
    if (n_slices > 0) drain(n_slices - 1);

    if (ROWSUM) {
        // combine the partial row sums of the threads that share a row; fixed order
        if (!g.A.transposed) {
#pragma unroll
            for (int i = 0; i < kBM / 16; ++i) {
                float v = rowsum[i];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                if ((tid & 7) == 0) s_rowsum[(tid >> 3) + 16 * i] = v;
            }
        } else {
#pragma unroll
            for (int i = 0; i < kBM / 32; ++i) {
                float v = rowsum[i];
                v += __shfl_xor_sync(0xffffffffu, v, 8);
                v += __shfl_xor_sync(0xffffffffu, v, 16);
                if (lane < 8) s_rowsum[(warp + 4 * i) * 8 + lane] = v;
            }
        }
    }
    __syncthreads();

    // epilogue: this thread holds output row m0 + tid, columns n0 .. n0 + BN
    const int row = warp * 32 + lane, m = m0 + row;
    if (m < g.M) {
        float* out_row;
        if (g.out_blocks) {
            const int gr = m + g.block_row_offset;
            const int blk = g.block_cyclic > 0 ? gr % g.block_cyclic : gr / g.block_rows;
            const int local = g.block_cyclic > 0 ? gr / g.block_cyclic : gr - blk * g.block_rows;
            out_row = g.out_blocks[blk] + (size_t)local * g.ldc;
        } else {
            out_row = g.out + (size_t)blockIdx.z * g.split_stride + (size_t)m * g.ldc;
        }
        const uint8_t* x_row = nullptr;
        if (g.epilogue != EPI_STORE) {
            const size_t xr = g.x_gather ? g.x_gather[m] : (size_t)g.x_row_base + (size_t)m;
            x_row = g.x_base + xr * (size_t)g.x_row_stride_bytes;
        }
        const float rs = ROWSUM ? s_rowsum[row] : 0.f;
        const bool vec_store = ((g.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(out_row) & 15) == 0);
#pragma unroll
        for (int j = 0; j < BN; ++j) {
            const int n = n0 + j;
            if (n < g.N) {
                if (g.epilogue == EPI_ADD_TABLE_VALUE) {
                    const float x = g.x_is_half ? __half2float(reinterpret_cast<const __half*>(x_row)[n])
                                                : reinterpret_cast<const float*>(x_row)[n];
                    acc[j] = x + acc[j];
                } else if (g.epilogue == EPI_ROWSUM_X_MINUS) {
                    acc[j] = rs * reinterpret_cast<const float*>(x_row)[n] - acc[j];
                }
            }
        }
        if (vec_store && n0 + BN <= g.N) {
#pragma unroll
            for (int j = 0; j < BN; j += 4)
                *reinterpret_cast<float4*>(out_row + n0 + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < BN; ++j)
                if (n0 + j < g.N) out_row[n0 + j] = acc[j];
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, kStages * BN);
}

// ---------------------------------------------------------------------------
// Pipelined form.  Same arithmetic as k_tc_gemm, but the operand slices travel from global
// memory to a ring of raw tiles in shared memory with cp.async (16 bytes per copy, zero-filled
// outside the matrix), three slices ahead of their use, so the L2 latency is hidden behind the
// work on earlier slices, and the block's warps are specialised (staging, issuing, accumulating:
// see the kernel).  The split pass reads the raw tile from shared memory and splits (and, for
// mn-major operands, transposes) it into the swizzled K-major hi / lo tiles.  Requires every
// operand row to start on a 16-byte boundary; otherwise the launcher falls back to k_tc_gemm.
// Two problems of the same kind (the two gradients of the score, the two feature networks) can
// share one launch: blockIdx.x picks the problem.  A k range divided over blockIdx.z is reduced
// either through the distributed shared memory of a thread-block cluster (up to 8 splits) or by
// k_tc_reduce over a workspace.

struct GemmPair {
    GemmArgs p[2];
    int tiles_m0;  // blocks with blockIdx.x < tiles_m0 work on p[0], the others on p[1]
    // hand-overs between processes folded into the launch (-1 = none): what the blocks wait for
    // before they read their operands, and what the last block to finish publishes
    ExchangeSync sync;
    int wait_kind, signal_kind;
};

__device__ __forceinline__ void cp_async16(uint8_t* dst_smem, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst_smem)), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ int clamp16(int bytes) { return bytes < 0 ? 0 : (bytes > 16 ? 16 : bytes); }

// 16 consecutive accumulator columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Queues the copies of the [ROWS x 32] slice (mn0.., k0..) into `raw`; NT threads share the work.
//   k-major operand:  raw[row][32 k]   (128-byte rows for fp32, 64-byte rows for fp16)
//   mn-major operand: raw[32 k][ROWS]  (rows of ROWS elements)
template <int ROWS, int NT>
__device__ __forceinline__ void issue_raw(const Operand& op, int mn0, int MN, int k0, int k_end, uint8_t* raw) {
    const int tid = threadIdx.x;
    if (!op.transposed) {
        if (!op.is_half) {
#pragma unroll
            for (int u = tid; u < ROWS * 8; u += NT) {
                const int row = u >> 3, ch = u & 7;
                const int mn = mn0 + row, k = k0 + ch * 4;
                const int bytes = mn < MN ? clamp16((k_end - k) * 4) : 0;
                const uint8_t* src = bytes ? operand_row(op, mn) + (size_t)k * 4 : op.base;
                cp_async16(raw + row * 128 + ch * 16, src, bytes);
            }
        } else {
#pragma unroll
            for (int u = tid; u < ROWS * 4; u += NT) {
                const int row = u >> 2, ch = u & 3;
                const int mn = mn0 + row, k = k0 + ch * 8;
                const int bytes = mn < MN ? clamp16((k_end - k) * 2) : 0;
                const uint8_t* src = bytes ? operand_row(op, mn) + (size_t)k * 2 : op.base;
                cp_async16(raw + row * 64 + ch * 16, src, bytes);
            }
        }
    } else {
        if (!op.is_half) {
            constexpr int kChunksPerRow = ROWS / 4;
#pragma unroll
            for (int u = tid; u < kBK * kChunksPerRow; u += NT) {
                const int kk = u / kChunksPerRow, c = u % kChunksPerRow;
                const int k = k0 + kk, mn = mn0 + c * 4;
                const int bytes = k < k_end ? clamp16((MN - mn) * 4) : 0;
                const uint8_t* src = bytes ? operand_row(op, k) + (size_t)mn * 4 : op.base;
                cp_async16(raw + kk * (ROWS * 4) + c * 16, src, bytes);
            }
        } else {
            constexpr int kChunksPerRow = ROWS / 8;
#pragma unroll
            for (int u = tid; u < kBK * kChunksPerRow; u += NT) {
                const int kk = u / kChunksPerRow, c = u % kChunksPerRow;
                const int k = k0 + kk, mn = mn0 + c * 8;
                const int bytes = k < k_end ? clamp16((MN - mn) * 2) : 0;
                const uint8_t* src = bytes ? operand_row(op, k) + (size_t)mn * 2 : op.base;
                cp_async16(raw + kk * (ROWS * 2) + c * 16, src, bytes);
            }
        }
    }
}

__device__ __forceinline__ void store_split(uint8_t* tile_hi, uint8_t* tile_lo, int row, int chunk, const float (&v)[4],
                                            bool write_lo) {
    const float4 hi = make_float4(tf32_hi(v[0]), tf32_hi(v[1]), tf32_hi(v[2]), tf32_hi(v[3]));
    const uint32_t off = (uint32_t)row * 128u + (((uint32_t)chunk ^ ((uint32_t)row & 7u)) << 4);
    *reinterpret_cast<float4*>(tile_hi + off) = hi;
    if (write_lo)
        *reinterpret_cast<float4*>(tile_lo + off) =
            make_float4(tf32_hi(v[0] - hi.x), tf32_hi(v[1] - hi.y), tf32_hi(v[2] - hi.z), tf32_hi(v[3] - hi.w));
}

// Raw tile -> swizzled K-major hi / lo tiles.  With ROWSUM (fp32 operands, ROWS = 128) the exact
// values are also summed: `rowsum[i]` collects what this thread handled of its i-th row
//   k-major:  rows (tid >> 3) + i * NT / 8, eight neighbouring threads share a row;
//   mn-major: row tid % 128 for every i, the threads tid, tid + 128, ... share a row.
template <int ROWS, int NT, bool WRITE_LO, bool ROWSUM>
__device__ __forceinline__ void split_raw(const Operand& op, const uint8_t* raw, uint8_t* tile_hi, uint8_t* tile_lo,
                                          float (&rowsum)[4]) {
    const int tid = threadIdx.x;
    if (!op.transposed) {
        if (!op.is_half) {
            int i = 0;
#pragma unroll
            for (int u = tid; u < ROWS * 8; u += NT, ++i) {
                const int row = u >> 3, ch = u & 7;
                const float4 x = *reinterpret_cast<const float4*>(raw + row * 128 + ch * 16);
                const float v[4] = {x.x, x.y, x.z, x.w};
                if (ROWSUM) rowsum[i & 3] += (v[0] + v[1]) + (v[2] + v[3]);
                store_split(tile_hi, tile_lo, row, ch, v, WRITE_LO);
            }
        } else {
#pragma unroll
            for (int u = tid; u < ROWS * 4; u += NT) {
                const int row = u >> 2, ch = u & 3;
                const uint4 x = *reinterpret_cast<const uint4*>(raw + row * 64 + ch * 16);
                const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&x.x));
                const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&x.y));
                const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&x.z));
                const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&x.w));
                const float v0[4] = {a.x, a.y, b.x, b.y}, v1[4] = {c.x, c.y, d.x, d.y};
                store_split(tile_hi, tile_lo, row, 2 * ch, v0, WRITE_LO);
                store_split(tile_hi, tile_lo, row, 2 * ch + 1, v1, WRITE_LO);
            }
        }
    } else {
        // unit = (row, 16-byte chunk of k): consecutive threads take consecutive rows, so the reads
        // walk along a raw row (conflict-free) and the swizzle spreads the 16-byte stores of eight
        // neighbouring rows over all banks
#pragma unroll
        for (int u = tid; u < ROWS * 8; u += NT) {
            const int row = u % ROWS, ch = u / ROWS;
            float v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int kk = ch * 4 + j;
                v[j] = op.is_half ? __half2float(reinterpret_cast<const __half*>(raw)[kk * ROWS + row])
                                  : reinterpret_cast<const float*>(raw)[kk * ROWS + row];
            }
            if (ROWSUM) rowsum[0] += (v[0] + v[1]) + (v[2] + v[3]);
            store_split(tile_hi, tile_lo, row, ch, v, WRITE_LO);
        }
    }
}

// The epilogue's second operand for four neighbouring output columns (m, n .. n+3): the value part
// of the table row (EPI_ADD_TABLE_VALUE) or X[m, n ..] (EPI_ROWSUM_X_MINUS); zeros for EPI_STORE.
// `fixed` >= 0: the epilogue is known where the call is compiled (the other kinds' code drops out).
__device__ __forceinline__ void load_x_four(const GemmArgs& g, int m, int n, float (&x)[4], int fixed = -1) {
    const int epilogue = fixed >= 0 ? fixed : g.epilogue;
    x[0] = x[1] = x[2] = x[3] = 0.f;
    if (epilogue == EPI_STORE) return;
    if (epilogue == EPI_DENSE_ADAM) {  // the moments are wanted right after X: ask L2 for them now
        const size_t e = (size_t)(m + g.block_row_offset) * g.ldc + n;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(g.adam.m + e));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(g.adam.v + e));
    }
    const size_t xr = g.x_gather ? g.x_gather[m] : (size_t)g.x_row_base + (size_t)m;
    const uint8_t* x_row = g.x_base + xr * (size_t)g.x_row_stride_bytes;
    const int narrow = epilogue == EPI_ADD_TABLE_VALUE ? g.x_is_half : 0;  // 1: fp16 values, 2: bf16 values
    if (!narrow && n + 3 < g.N && ((reinterpret_cast<uintptr_t>(x_row) + (size_t)n * 4) & 15) == 0) {
        const float4 v = *reinterpret_cast<const float4*>(x_row + (size_t)n * 4);
        x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
        return;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (n + j < g.N)
            x[j] = narrow == 1   ? __half2float(reinterpret_cast<const __half*>(x_row)[n + j])
                   : narrow == 2 ? __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(x_row)[n + j] << 16)
                                 : reinterpret_cast<const float*>(x_row)[n + j];
}

// Epilogue and store of four neighbouring output columns whose k range is complete.
__device__ __forceinline__ void finish_four(const GemmArgs& g, float* out_base, int m, int n, float (&acc)[4],
                                            const float (&x)[4], float rs, int fixed = -1) {
    const int epilogue = fixed >= 0 ? fixed : g.epilogue;
    if (epilogue == EPI_ADD_TABLE_VALUE) {
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[j] = x[j] + acc[j];
    } else if (epilogue == EPI_ROWSUM_X_MINUS) {
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[j] = rs * x[j] - acc[j];
    }
    if (epilogue == EPI_DENSE_ADAM) {
        const DenseAdamArgs& a = g.adam;
        const size_t e = (size_t)(m + g.block_row_offset) * g.ldc + n;
        const float alpha = *a.step_size * a.lr_modifier;
        const bool vec = n + 3 < g.N && (e & 3) == 0;
        float mo[4], ve[4], w[4], lo[4];
        if (vec) {
            const float4 m4 = *reinterpret_cast<const float4*>(a.m + e), v4 = *reinterpret_cast<const float4*>(a.v + e);
            mo[0] = m4.x; mo[1] = m4.y; mo[2] = m4.z; mo[3] = m4.w;
            ve[0] = v4.x; ve[1] = v4.y; ve[2] = v4.z; ve[3] = v4.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                mo[j] = n + j < g.N ? a.m[e + j] : 0.f;
                ve[j] = n + j < g.N ? a.v[e + j] : 0.f;
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float grad = acc[j];
            mo[j] = a.beta_m * mo[j] + a.one_minus_beta_m * grad;
            ve[j] = a.beta_v * ve[j] + a.one_minus_beta_v * grad * grad;
            w[j] = x[j] - alpha * (mo[j] / (sqrtf(ve[j]) + a.epsilon) + a.weight_decay * x[j]);
            const float hi = __uint_as_float(__float_as_uint(w[j]) & 0xffffe000u);
            lo[j] = __uint_as_float(__float_as_uint(w[j] - hi) & 0xffffe000u);
        }
        if (vec) {
            *reinterpret_cast<float4*>(a.m + e) = make_float4(mo[0], mo[1], mo[2], mo[3]);
            *reinterpret_cast<float4*>(a.v + e) = make_float4(ve[0], ve[1], ve[2], ve[3]);
            *reinterpret_cast<float4*>(a.w + e) = make_float4(w[0], w[1], w[2], w[3]);
            if (a.w_lo) *reinterpret_cast<float4*>(a.w_lo + e) = make_float4(lo[0], lo[1], lo[2], lo[3]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (n + j >= g.N) break;
                a.m[e + j] = mo[j];
                a.v[e + j] = ve[j];
                a.w[e + j] = w[j];
                if (a.w_lo) a.w_lo[e + j] = lo[j];
            }
        }
        return;
    }
    float* out_row;
    if (g.out_blocks) {
        const int gr = m + g.block_row_offset;
        const int blk = g.block_cyclic > 0 ? gr % g.block_cyclic : gr / g.block_rows;
        const int local = g.block_cyclic > 0 ? gr / g.block_cyclic : gr - blk * g.block_rows;
        out_row = g.out_blocks[blk] + (size_t)local * g.ldc;
    } else {
        out_row = out_base + (size_t)m * g.ldc;
    }
    if ((g.N & 3) == 0 && (g.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(out_row) & 15) == 0) {
        *reinterpret_cast<float4*>(out_row + n) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (n + j < g.N) out_row[n + j] = acc[j];
    }
}

// Thread-block cluster helpers: rank of this block, the cluster-wide barrier (a hardware barrier,
// not a spin on memory) and 128-bit / 32-bit reads of another block's shared memory.
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_map(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float4 cluster_load4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void cluster_store4(uint32_t addr, float a, float b, float c, float d) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void cluster_store1(uint32_t addr, float a) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(a) : "memory");
}
__device__ __forceinline__ float cluster_load1(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}

// Warp roles of the pipelined kernel: 8 staging warps, 8 accumulating warps, 1 issuing warp, 1 copying warp.
constexpr int kStageWarps = 8, kAccWarps = 8;
constexpr int kStageThreads = 32 * kStageWarps;
constexpr int kPipeThreads = 32 * (kStageWarps + kAccWarps + 2);
constexpr int kRawSlots = 3;   // raw slices in flight per block
constexpr int kTmemSlots = 4;  // accumulator tiles: slices whose products may be pending or unread

constexpr int kMaxClusterRows = 8;  // rows_each * splits exceeds 128 by less than the number of splits
// Rows received from the other splits of a cluster: [splits][rows_each][BN + 4] floats and their row sums.
template <int BN>
constexpr size_t cluster_receive_bytes() {
    return (size_t)(kBM + kMaxClusterRows) * (BN + 4 + 1) * 4;
}
template <int BN>
constexpr size_t smem_bytes_async() {
    return 1024 + (size_t)kStages * (2 * kBM * 128 + 2 * BN * 128) + (size_t)kRawSlots * (kBM * 128 + BN * 128) +
           cluster_receive_bytes<BN>();
}

// Tensor maps of the operands of the (up to) two problems of a launch: the copying warp moves a
// whole [rows x 32 k] (or [32 k x rows]) box per instruction with the TMA unit, which generates the
// addresses, fills what lies outside the matrix with zeros and reports the bytes to an mbarrier.
struct GemmMaps {
    CUtensorMap a[2], b[2];
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// One box of a 2-d tensor map into this block's shared memory; x is the coordinate along the
// contiguous dimension and x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint8_t* dst_smem, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst_smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}

// The groups of warps run their own loops over the k slices and meet only at mbarriers:
//
//   copying warp (17)     one thread waits until raw slot j % 4 has been read (`raw_empty`) and
//                         starts the two TMA copies of slice j into it; their bytes complete `raw_full`.
//   staging warps (0-7)   wait for `raw_full`, wait until the MMAs that read stage j % 2 have
//                         completed (`empty`), split / transpose slice j into that stage and
//                         arrive at `full` and `raw_empty`.
//   issuing warp (16)     waits for `full` and for the accumulator tile j % 4 to have been read
//                         (`acc_free`), issues the slice's tcgen05.mma instructions into it and
//                         commits them to `empty` (the stage may be overwritten) and `acc_ready`.
//   accumulating warps    wait for `acc_ready`, read their 32 lanes x 32 columns of the tile from
//   (8-15)                TMEM, arrive at `acc_free` and add the values to registers.
//
// So the copies, the split pass, the tensor core and the TMEM reads of neighbouring slices
// overlap, and no thread waits for a phase it has no part in.
template <int BN, bool A_EXACT, bool ROWSUM>
__global__ void __launch_bounds__(kPipeThreads, 1)
k_tc_gemm_async(const __grid_constant__ GemmPair gp, const __grid_constant__ GemmMaps maps) {
    static_assert(BN == 64, "an accumulating warp reads 32 of the tile's 64 columns");
    constexpr int CPT = 32;  // accumulator columns per accumulating thread
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_full[kStages], bar_empty[kStages], bar_acc_ready[kTmemSlots], bar_acc_free[kTmemSlots];
    __shared__ uint64_t bar_raw_full[kRawSlots], bar_raw_empty[kRawSlots];
    __shared__ uint32_t tmem_slot;
    __shared__ float s_rowsum[kBM];
    __shared__ float s_part[kStageThreads / kBM][kBM];

    const int which = (int)blockIdx.x >= gp.tiles_m0 ? 1 : 0;
    const GemmArgs& g = gp.p[which];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = ((int)blockIdx.x - (which ? gp.tiles_m0 : 0)) * kBM, n0 = blockIdx.y * BN;
    const unsigned total_blocks = gridDim.x * gridDim.y * gridDim.z;
    if (n0 >= g.N || m0 >= g.M) {  // the two problems may differ in size (a whole cluster leaves together)
        grid_dependency_sync();
        exchange_signal(gp.sync, gp.signal_kind, total_blocks);
        return;
    }

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr uint32_t kATile = kBM * 128, kBTile = BN * 128, kStage = 2 * kATile + 2 * kBTile, kRaw = kATile + kBTile;
    uint8_t* raw_ring = smem + (size_t)kStages * kStage;
    const int k_begin = blockIdx.z * g.k_per_split, k_end = min(g.K, k_begin + g.k_per_split);
    const int n_slices = max(0, (k_end - k_begin + kBK - 1) / kBK);

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&bar_full[s], kStageWarps);
            mbar_init(&bar_empty[s], 1);
        }
        for (int t = 0; t < kTmemSlots; ++t) {
            mbar_init(&bar_acc_ready[t], 1);
            mbar_init(&bar_acc_free[t], kAccWarps);
        }
        for (int r = 0; r < kRawSlots; ++r) {
            mbar_init(&bar_raw_full[r], 1);
            mbar_init(&bar_raw_empty[r], kStageWarps);
        }
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(&tmem_slot, kTmemSlots * BN);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    grid_dependency_sync();
    exchange_wait(gp.sync, gp.wait_kind);
    const uint32_t tmem_base = tmem_slot;

    float rowsum[4] = {0.f, 0.f, 0.f, 0.f};
    float acc[CPT];
#pragma unroll
    for (int j = 0; j < CPT; ++j) acc[j] = 0.f;

    if (warp < kStageWarps) {
        for (int kc = 0; kc < n_slices; ++kc) {
            const int s = kc % kStages, slot = kc % kRawSlots;
            mbar_wait(&bar_raw_full[slot], (uint32_t)((kc / kRawSlots) & 1), g.status, 5u);
            if (kc >= kStages) mbar_wait(&bar_empty[s], (uint32_t)(((kc / kStages) - 1) & 1), g.status, 2u);
            uint8_t* stage = smem + (size_t)s * kStage;
            uint8_t *a_hi = stage, *a_lo = stage + kATile, *b_hi = stage + 2 * kATile, *b_lo = b_hi + kBTile;
            const uint8_t* raw = raw_ring + (size_t)slot * kRaw;
            float unused[4];
            split_raw<kBM, kStageThreads, !A_EXACT, ROWSUM>(g.A, raw, a_hi, a_lo, rowsum);
            split_raw<BN, kStageThreads, true, false>(g.B, raw + kATile, b_hi, b_lo, unused);
            fence_async_shared();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&bar_full[s]);
                mbar_arrive(&bar_raw_empty[slot]);
            }
        }
    } else if (warp == kStageWarps + kAccWarps + 1) {
        const CUtensorMap* map_a = &maps.a[which];
        const CUtensorMap* map_b = &maps.b[which];
        const uint32_t bytes = (uint32_t)(kBM * kBK * (g.A.is_half ? 2 : 4) + BN * kBK * (g.B.is_half ? 2 : 4));
        for (int kc = 0; kc < n_slices; ++kc) {
            const int slot = kc % kRawSlots;
            if (kc >= kRawSlots) mbar_wait(&bar_raw_empty[slot], (uint32_t)(((kc / kRawSlots) - 1) & 1), g.status, 6u);
            if (lane == 0) {
                uint8_t* raw = raw_ring + (size_t)slot * kRaw;
                const int k0 = k_begin + kc * kBK;
                mbar_arrive_expect(&bar_raw_full[slot], bytes);
                if (g.A.transposed) tma_load_2d(raw, map_a, m0, k0, &bar_raw_full[slot]);
                else tma_load_2d(raw, map_a, k0, m0, &bar_raw_full[slot]);
                if (g.B.transposed) tma_load_2d(raw + kATile, map_b, n0, k0, &bar_raw_full[slot]);
                else tma_load_2d(raw + kATile, map_b, k0, n0, &bar_raw_full[slot]);
            }
            __syncwarp();
        }
    } else if (warp == kStageWarps + kAccWarps) {
        constexpr uint32_t idesc = make_idesc_tf32(kBM, BN);
        for (int kc = 0; kc < n_slices; ++kc) {
            const int s = kc % kStages, t = kc % kTmemSlots;
            mbar_wait(&bar_full[s], (uint32_t)((kc / kStages) & 1), g.status, 3u);
            if (kc >= kTmemSlots) mbar_wait(&bar_acc_free[t], (uint32_t)(((kc / kTmemSlots) - 1) & 1), g.status, 4u);
            tc_fence_after();
            if (lane == 0) {
                uint8_t* stage = smem + (size_t)s * kStage;
                uint8_t *a_hi = stage, *a_lo = stage + kATile, *b_hi = stage + 2 * kATile, *b_lo = b_hi + kBTile;
                const uint32_t tmem_acc = tmem_base + (uint32_t)(t * BN);
                const uint64_t da_hi = make_kmajor_sw128_desc(smem_u32(a_hi)), da_lo = make_kmajor_sw128_desc(smem_u32(a_lo));
                const uint64_t db_hi = make_kmajor_sw128_desc(smem_u32(b_hi)), db_lo = make_kmajor_sw128_desc(smem_u32(b_lo));
#pragma unroll
                for (int ks = 0; ks < kBK / 8; ++ks) {
                    const uint64_t adv = (uint64_t)(ks * 32 >> 4);
                    umma_tf32(tmem_acc, da_hi + adv, db_lo + adv, idesc, ks > 0 ? 1u : 0u);
                    if (!A_EXACT) umma_tf32(tmem_acc, da_lo + adv, db_hi + adv, idesc, 1u);
                    umma_tf32(tmem_acc, da_hi + adv, db_hi + adv, idesc, 1u);
                }
                umma_commit(&bar_empty[s]);
                umma_commit(&bar_acc_ready[t]);
            }
            __syncwarp();
        }
    } else {
        // The tensor core truncates its fp32 accumulator once per instruction, so every slice is
        // accumulated on its own in TMEM and the slices are added here with round-to-nearest.
        const int quarter = warp & 3, half = (warp - kStageWarps) >> 2;
        for (int kc = 0; kc < n_slices; ++kc) {
            const int t = kc % kTmemSlots;
            mbar_wait(&bar_acc_ready[t], (uint32_t)((kc / kTmemSlots) & 1), g.status, 1u);
            tc_fence_after();
            uint32_t r[32];
            tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(t * BN + half * CPT), r);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_acc_free[t]);
#pragma unroll
            for (int j = 0; j < CPT; ++j) acc[j] += __uint_as_float(r[j]);
        }
    }

    if (ROWSUM && warp < kStageWarps) {
        // fixed-order combination of the partial row sums of the staging threads
        if (!g.A.transposed) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float v = rowsum[i];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                if ((tid & 7) == 0) s_rowsum[(tid >> 3) + i * (kStageThreads / 8)] = v;
            }
        } else {
            s_part[tid / kBM][tid % kBM] = rowsum[0];
        }
    }
    __syncthreads();  // every slice has been read from TMEM: the operand stages are free
    if (ROWSUM && g.A.transposed) {
        if (tid < kBM) {
            float v = 0.f;
#pragma unroll
            for (int c = 0; c < kStageThreads / kBM; ++c) v += s_part[c][tid];
            s_rowsum[tid] = v;
        }
        __syncthreads();
    }

    const bool acc_warp = warp >= kStageWarps && warp < kStageWarps + kAccWarps;
    const int row = (warp & 3) * 32 + lane, m = m0 + row;
    const int nc0 = n0 + ((warp - kStageWarps) >> 2) * CPT;  // first output column of an accumulating thread
    if (g.cluster_splits > 1) {
        // The splits of this tile are the blocks of one cluster, and block z finishes rows
        // z * rows_each ... of the tile.  Every block sends each of its partial rows to the shared
        // memory of the row's owner (remote stores, nobody waits for them); after one cluster
        // barrier the owner adds what it received, in split order, and nobody reads remote memory
        // any more, so a block may leave as soon as it has stored its rows.
        constexpr int kRedStride = BN + 4;  // floats; keeps the 128-bit accesses free of bank conflicts
        const int n_split = g.cluster_splits, rank = (int)cluster_rank();
        const int rows_each = (kBM + n_split - 1) / n_split;
        // (a region of its own: a faster block may send while this one still reads its operand stages)
        float* red = reinterpret_cast<float*>(raw_ring + (size_t)kRawSlots * kRaw);  // [source block][row of mine][BN]
        float* red_rowsum = red + (size_t)n_split * rows_each * kRedStride;  // [source block][row of mine]
        if (acc_warp) {
            const int owner = row / rows_each, local = row - owner * rows_each;
            const uint32_t dst = cluster_map(smem_u32(red + ((size_t)rank * rows_each + local) * kRedStride + (nc0 - n0)), (uint32_t)owner);
#pragma unroll
            for (int j = 0; j < CPT; j += 4) cluster_store4(dst + (uint32_t)j * 4u, acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
            if (ROWSUM && nc0 == n0)
                cluster_store1(cluster_map(smem_u32(red_rowsum + rank * rows_each + local), (uint32_t)owner), s_rowsum[row]);
        }
        // the epilogue's second operand is fetched while the partial rows travel
        const int r_begin = rank * rows_each, r_end = min(kBM, r_begin + rows_each);
        constexpr int kQuads = BN / 4;
        const int n_units = max(0, r_end - r_begin) * kQuads;  // at most 64 rows x 16 = 2 per thread
        float xv[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int u = tid + i * kPipeThreads;
            const int mm = m0 + r_begin + u / kQuads, nn = n0 + (u % kQuads) * 4;
            xv[i][0] = xv[i][1] = xv[i][2] = xv[i][3] = 0.f;
            if (u < n_units && mm < g.M && nn < g.N) load_x_four(g, mm, nn, xv[i]);
        }
        cluster_sync();
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int u = tid + i * kPipeThreads;
            if (u >= n_units) continue;
            const int local = u / kQuads, c = (u % kQuads) * 4;
            float sum[4] = {0.f, 0.f, 0.f, 0.f};
            float row_total = 0.f;
            for (int z = 0; z < n_split; ++z) {
                const float4 v = *reinterpret_cast<const float4*>(red + ((size_t)z * rows_each + local) * kRedStride + c);
                sum[0] += v.x; sum[1] += v.y; sum[2] += v.z; sum[3] += v.w;
                if (ROWSUM) row_total += red_rowsum[z * rows_each + local];
            }
            const int mm = m0 + r_begin + local, nn = n0 + c;
            if (mm < g.M && nn < g.N) finish_four(g, g.out, mm, nn, sum, xv[i], row_total);
        }
    } else if (acc_warp && m < g.M && nc0 < g.N) {
        if (g.ws) {
            // split run without a cluster: leave the raw partial tile (and row sums) for k_tc_reduce
            float* w = g.ws + ((size_t)blockIdx.z * g.M + m) * g.N + nc0;
            if ((g.N & 3) == 0 && nc0 + CPT <= g.N) {
#pragma unroll
                for (int j = 0; j < CPT; j += 4) *reinterpret_cast<float4*>(w + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < CPT; ++j)
                    if (nc0 + j < g.N) w[j] = acc[j];
            }
            if (ROWSUM && blockIdx.y == 0 && nc0 == n0) g.ws_rowsum[(size_t)blockIdx.z * g.M + m] = s_rowsum[row];
        } else {
            // each split finishes its own output slice
            float* out_base = g.out_blocks ? nullptr : g.out + (size_t)blockIdx.z * g.split_stride;
            const float rs = ROWSUM ? s_rowsum[row] : 0.f;
#pragma unroll
            for (int j = 0; j < CPT; j += 4) {
                float four[4] = {acc[j], acc[j + 1], acc[j + 2], acc[j + 3]};
                float x[4];
                if (nc0 + j < g.N) {
                    load_x_four(g, m, nc0 + j, x);
                    finish_four(g, out_base, m, nc0 + j, four, x, rs);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, kTmemSlots * BN);
    exchange_signal(gp.sync, gp.signal_kind, total_blocks);
}

// Adds the partial tiles of a k split in split order and applies the epilogue of the contraction:
// one thread per output row and group of four columns, 128-bit accesses.  blockIdx.y picks the
// problem of a paired launch.
static __global__ void __launch_bounds__(256) k_tc_reduce(const __grid_constant__ GemmPair gp) {
    grid_dependency_sync();
    const GemmArgs& g = gp.p[blockIdx.y];
    const int n4 = (g.N + 3) >> 2;
    const long long unit = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (unit >= (long long)g.M * n4) return;
    const int m = (int)(unit / n4), n = (int)(unit - (long long)m * n4) * 4;
    const size_t plane = (size_t)g.M * g.N;
    const bool vec = (g.N & 3) == 0;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int z = 0; z < g.splits; ++z) {
        const float* w = g.ws + (size_t)z * plane + (size_t)m * g.N + n;
        if (vec) {
            const float4 v = *reinterpret_cast<const float4*>(w);
            acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (n + j < g.N) acc[j] += w[j];
        }
    }
    float rs = 0.f;
    if (g.epilogue == EPI_ROWSUM_X_MINUS)
        for (int z = 0; z < g.splits; ++z) rs += g.ws_rowsum[(size_t)z * g.M + m];
    float x[4];
    load_x_four(g, m, n, x);
    finish_four(g, g.out, m, n, acc, x, rs);
}

// Host side: grid = (ceil(M / 128), ceil(N / BN), splits).
template <int BN, bool A_EXACT, bool ROWSUM>
inline cudaError_t launch(const GemmArgs& g, int splits, cudaStream_t stream) {
    static bool configured[kMaxDeviceOrdinals] = {};  // one attribute call per instantiation and device is enough
    const int slot = current_device_slot();
    auto kernel = k_tc_gemm<BN, A_EXACT, ROWSUM>;
    if (slot < 0 || !configured[slot]) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<BN>());
        if (err != cudaSuccess) return err;
        if (slot >= 0) configured[slot] = true;
    }
    dim3 grid((g.M + kBM - 1) / kBM, (g.N + BN - 1) / BN, splits);
    return launch_dependent(kernel, grid, dim3(kThreads), smem_bytes<BN>(), stream, g);
}

inline bool rows_16_byte_aligned(const Operand& op) {
    return reinterpret_cast<uintptr_t>(op.base) % 16 == 0 && op.row_stride_bytes % 16 == 0;
}

// One or two problems in one launch, pipelined when every operand allows 16-byte copies.
constexpr int kMaxClusterSplits = 8;  // the portable cluster size

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda).
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &result) != cudaSuccess ||
            result != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// The map of one operand: `mn` rows (or columns, for an mn-major operand) by `k`, boxes of
// [rows x 32 k] (k-major) or [32 k x rows] (mn-major), dense in shared memory, zeros outside.
inline cudaError_t make_operand_map(const Operand& op, int mn, int k, int rows, CUtensorMap* map) {
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return cudaErrorNotSupported;
    const cuuint64_t dims[2] = {(cuuint64_t)(op.transposed ? mn : k), (cuuint64_t)(op.transposed ? k : mn)};
    const cuuint64_t strides[1] = {(cuuint64_t)op.row_stride_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)(op.transposed ? rows : kBK), (cuuint32_t)(op.transposed ? kBK : rows)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(map, op.is_half ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                              const_cast<uint8_t*>(op.base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// How many clusters of `splits` blocks of the pipelined kernel the device can hold at once
// (a cluster needs its blocks on SMs of one GPC, one block per SM).  0 when the query fails.
inline int max_resident_clusters(int splits) {
    static int cached[kMaxDeviceOrdinals][kMaxClusterSplits + 1] = {};
    static bool known[kMaxDeviceOrdinals][kMaxClusterSplits + 1] = {};
    if (splits < 1 || splits > kMaxClusterSplits) return 0;
    const int slot = current_device_slot();
    if (slot >= 0 && known[slot][splits]) return cached[slot][splits];
    auto kernel = k_tc_gemm_async<64, false, false>;
    int n = 0;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes_async<64>()) == cudaSuccess) {
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(1, 1, splits);
        config.blockDim = dim3(kPipeThreads);
        config.dynamicSmemBytes = smem_bytes_async<64>();
        cudaLaunchAttribute attribute[1];
        attribute[0].id = cudaLaunchAttributeClusterDimension;
        attribute[0].val.clusterDim.x = 1;
        attribute[0].val.clusterDim.y = 1;
        attribute[0].val.clusterDim.z = (unsigned)splits;
        config.attrs = attribute;
        config.numAttrs = 1;
        if (cudaOccupancyMaxActiveClusters(&n, kernel, &config) != cudaSuccess) {
            n = 0;
            (void)cudaGetLastError();
        }
    }
    if (slot >= 0) {
        known[slot][splits] = true;
        cached[slot][splits] = n;
    }
    return n;
}

template <int BN, bool A_EXACT, bool ROWSUM>
inline cudaError_t launch_pair(const GemmArgs* problems, int n_problems, int splits, cudaStream_t stream, int* n_launches = nullptr,
                               const ExchangeSync& sync = ExchangeSync{}, int wait_kind = -1, int signal_kind = -1) {
    if (n_launches) *n_launches = n_problems;
    bool fast = true;
    for (int i = 0; i < n_problems; ++i)
        fast = fast && rows_16_byte_aligned(problems[i].A) && rows_16_byte_aligned(problems[i].B) && !problems[i].A.gather && !problems[i].B.gather;
    const bool synced = sync.world > 1;
    if (!fast) {
        // the unpipelined kernel has no in-kernel split reduction: run each problem unsplit; the
        // hand-overs between processes become kernels of their own around it
        if (synced && wait_kind >= 0) {
            cudaError_t err = launch_dependent(k_exchange_wait, dim3(1), dim3(kMaxProcesses), 0, stream, sync, wait_kind);
            if (err != cudaSuccess) return err;
            if (n_launches) ++*n_launches;
        }
        for (int i = 0; i < n_problems; ++i) {
            GemmArgs g = problems[i];
            if (g.ws) {
                g.k_per_split = (g.K + 31) / 32 * 32;
                if (g.k_per_split == 0) g.k_per_split = 32;
            }
            cudaError_t err = launch<BN, A_EXACT, ROWSUM>(g, g.ws ? 1 : splits, stream);
            if (err != cudaSuccess) return err;
        }
        if (synced && signal_kind >= 0) {
            if (n_launches) ++*n_launches;
            return launch_dependent(k_exchange_signal, dim3(1), dim3(kMaxProcesses), 0, stream, sync, signal_kind);
        }
        return cudaSuccess;
    }
    static bool configured[kMaxDeviceOrdinals] = {};
    const int slot = current_device_slot();
    auto kernel = k_tc_gemm_async<BN, A_EXACT, ROWSUM>;
    if (slot < 0 || !configured[slot]) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes_async<BN>());
        if (err != cudaSuccess) return err;
        if (slot >= 0) configured[slot] = true;
    }
    GemmPair gp{};
    gp.p[0] = problems[0];
    gp.p[1] = problems[n_problems > 1 ? 1 : 0];
    gp.tiles_m0 = (problems[0].M + kBM - 1) / kBM;
    gp.sync = sync;
    gp.wait_kind = wait_kind;
    gp.signal_kind = signal_kind;
    int tiles_m = gp.tiles_m0, tiles_n = (problems[0].N + BN - 1) / BN;
    if (n_problems > 1) {
        tiles_m += (problems[1].M + kBM - 1) / kBM;
        tiles_n = tiles_n > (problems[1].N + BN - 1) / BN ? tiles_n : (problems[1].N + BN - 1) / BN;
    }
    GemmMaps maps;
    for (int i = 0; i < 2; ++i) {
        const GemmArgs& q = gp.p[i];
        cudaError_t e = make_operand_map(q.A, q.M, q.K, kBM, &maps.a[i]);
        if (e == cudaSuccess) e = make_operand_map(q.B, q.N, q.K, BN, &maps.b[i]);
        if (e != cudaSuccess) return e;
    }
    dim3 grid(tiles_m, tiles_n, splits);
    if (n_launches) *n_launches = 1;
    if (problems[0].ws && splits >= 2 && splits <= kMaxClusterSplits) {
        // the splits of a tile as one cluster: no workspace, no second kernel
        gp.p[0].ws = gp.p[1].ws = nullptr;
        gp.p[0].cluster_splits = gp.p[1].cluster_splits = splits;
        return launch_dependent_cluster(kernel, grid, dim3(kPipeThreads), smem_bytes_async<BN>(), stream, (unsigned)splits, gp, maps);
    }
    // with a workspace the reduction kernel writes the result, so the publishing moves behind it
    const bool reduce_after = problems[0].ws != nullptr;
    if (reduce_after) gp.signal_kind = -1;
    cudaError_t err = launch_dependent(kernel, grid, dim3(kPipeThreads), smem_bytes_async<BN>(), stream, gp, maps);
    if (err != cudaSuccess || !reduce_after) return err;
    if (n_launches) *n_launches = 2;
    gp.p[0].splits = gp.p[1].splits = splits;
    long long units = 0;
    for (int i = 0; i < n_problems; ++i) {
        const long long u = (long long)problems[i].M * ((problems[i].N + 3) / 4);
        units = u > units ? u : units;
    }
    dim3 rgrid((unsigned)((units + 255) / 256), n_problems);
    err = launch_dependent(k_tc_reduce, rgrid, dim3(256), 0, stream, gp);
    if (err != cudaSuccess || !synced || signal_kind < 0) return err;
    if (n_launches) *n_launches = 3;
    return launch_dependent(k_exchange_signal, dim3(1), dim3(kMaxProcesses), 0, stream, sync, signal_kind);
}

inline Operand make_operand(const void* base, long long row_stride_bytes, bool is_half, bool transposed,
                            const uint32_t* gather = nullptr) {
    Operand op;
    op.base = static_cast<const uint8_t*>(base);
    op.row_stride_bytes = row_stride_bytes;
    op.gather = gather;
    op.is_half = is_half ? 1 : 0;
    op.transposed = transposed ? 1 : 0;
    const uintptr_t align = is_half ? 8 : 16;
    op.vec_ok = (reinterpret_cast<uintptr_t>(base) % align == 0 && row_stride_bytes % (long long)align == 0) ? 1 : 0;
    return op;
}

}  // namespace tc
}  // namespace kge
