// The tensor-core contraction fed straight by the TMA unit (tcgen05, sm_100a).
//
//   acc[m, n] = sum_k A[m, k] * B[n, k]          fp32 operands as TF32-exact planes, fp32 result
//
// Same arithmetic as tc_gemm.cuh (three TF32 products of the hi / lo parts of each operand, every
// 32-deep k slice accumulated alone in TMEM and added in registers with round-to-nearest), but
// nobody in the block touches the operands: the kernels that PRODUCE an operand write its two
// TF32-exact parts to global memory once ("planes": hi = x with the low 13 significand bits
// cleared, lo = x - hi cut likewise; an operand that came from fp16 storage is one plane), and one
// thread moves [rows x 32 k] boxes of those planes into shared memory with cp.async.bulk.tensor
// under the 128-byte swizzle, which is exactly the layout the UMMA shared-memory descriptors read:
//
//   k-major operand  (stored [mn][k]):  one box of `rows` 128-byte rows, CU_TENSOR_MAP_SWIZZLE_128B;
//                                        descriptor "K-major, SWIZZLE_128B", 8-row groups 1024 B
//                                        apart, 32 B per 8-deep k step;
//   mn-major operand (stored [k][mn]):  rows / 32 boxes of 32 k-rows x 32 mn (4 KB each, 4096 B
//                                        apart), CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B: 32-bit
//                                        operands are transposed by the tensor core only from the
//                                        layout that swizzles 32-byte chunks; descriptor "MN-major,
//                                        SWIZZLE_128B_BASE32B", leading offset 4096 B between the
//                                        boxes, 512 B between groups of 4 k-rows, 1024 B per k step.
//
// The tensor core reads the upper 19 bits of a 32-bit TF32 operand and ignores the rest (checked
// bit for bit on the B200 against planes with those bits cleared), so the unmodified fp32 array
// serves as the hi plane and a producer only adds the lo plane.
//
// Warp roles (10 warps): warp 0 one thread issues the copies of slice j into ring stage j % 3 once
// the MMAs that read it have completed; warp 1 one thread issues the slice's tcgen05.mma
// instructions into TMEM tile j % 4 and commits them; warps 2-9 read the tile (32 lanes x 32
// columns each) and add it to registers.  With ROWSUM they also add up the rows of A from the
// staged tile (the L2 backward needs rowsum(A) . X).  The groups meet only at mbarriers; every wait
// is bounded.  The k range may be split over the blocks of a thread-block cluster, reduced through
// distributed shared memory in split order, as in tc_gemm.cuh.
#pragma once

#include <algorithm>

#include "kernels.cuh"
#include "tc_gemm.cuh"

namespace kge {
namespace tc {

struct PlaneOperand {
    const float* hi;             // TF32-exact upper part (or the value itself when it is exact in TF32)
    const float* lo;             // TF32-exact remainder; null = the operand has one plane
    long long row_stride_bytes;  // multiple of 16
    int mn_major;                // 0: stored [mn][k], k contiguous; 1: stored [k][mn], mn contiguous
    // 2: `hi` points at bfloat16 values, one plane, multiplied by tcgen05.mma.kind::f16 (the 2e-2 tier:
    // bf16 embeddings with fp32 accumulation); 0 or 4: fp32 values as above.  One kind per launch.
    int elem_bytes;
};

// One contraction: the planes of both operands and, in `g`, sizes, k split, epilogue and output
// (g.A and g.B are not used).
// EPI_L2_DISTANCE as predict's score pass: the distances of output row m (a query) that beat the
// query's cut-off as it stands before the pass go straight into its candidate list, which
// k_topk_filter would otherwise collect by reading the whole score matrix back.  Output column n is
// table row first_row + n.  Null `cand`: none.
struct TopkFilterArgs {
    const unsigned long long* state;  // [M, kTopkCapacity] the queries' lists so far
    const int* counts;                // [M]
    unsigned long long* cand;         // [M, kTopkCandidates]
    int* cand_count;                  // [M]
    uint32_t first_row, last_valid_row;
    int n_best, score_is_gamma_minus;
    float gamma;
};

struct PlaneProblem {
    PlaneOperand A, B;
    GemmArgs g;
    TopkFilterArgs filter;
};

// Folded into the epilogue of hidden = value + feature . W: the lookups of the step and the send
// half of the exchange (src/poplar_kge.cpp:676-684).  `perm` lists the lookups ordered by the hidden
// row they read, `off[r]` is where row r's begin (k_prepare_segments).  Lookup e < B is head lookup
// e: pred[e] = row (+|*) relation row; lookup e >= B is tail lookup e - B: the row goes to slot
// (e - B) % a2a of destination shard (e - B) / a2a, whose buffer may be a peer's memory.  Both also
// get their lo plane (the score gradients read them as tensor-core operands).  mode[p]: what
// problem p of the launch routes (bit 0 heads, bit 1 tails; separate head / tail networks are two
// problems).  Null `perm`: no routing.
struct RouteArgs {
    const uint32_t* perm;
    const uint32_t* off;
    const uint32_t* relation;
    const float* rel_table;
    float* const* send_dst;     // [n_shard] this shard's slot in every shard's tail buffer
    float* const* send_lo_dst;  // [n_shard] the same in the lo plane
    float* pred;
    float* pred_lo;
    int B, a2a, n_shard, score_fn;
    int mode[2];
    int lo_bf16;  // the companion planes hold the bfloat16 rounding of the rows instead of the lower TF32 part
    // Per gathered row, bit 1 set: the row has so many lookups that they are routed in parts by
    // k_route_heavy (a row that half of a step's lookups name would otherwise keep one block storing
    // for 10 us after all others are done).  Null: every row is routed here.
    const uint32_t* first_slot;
};
constexpr uint32_t kRouteSkip = 0xffffffffu;
constexpr int kRouteMaxLookups = 4096;  // lookups one block may have to route (batch_size + n_shard * a2a_size)

struct PlanePair {
    PlaneProblem p[2];
    int tiles_m0;  // blocks with blockIdx.x < tiles_m0 work on p[0], the others on p[1]
    ExchangeSync sync;
    int wait_kind, signal_kind;
    RouteArgs route;
    int n_stages[2];  // ring stages of each problem (2 to kPlMaxStages), as many as the shared memory holds
    int bf16;         // the operands are bfloat16 planes: 64-deep slices, kind::f16 products
};

struct PlaneMaps {
    CUtensorMap a_hi[2], a_lo[2], b_hi[2], b_lo[2];
};

constexpr int kPlMaxStages = 4;
constexpr int kPlAccWarps = 8;
constexpr int kPlThreads = 32 * (2 + kPlAccWarps);
constexpr int kPlTmemSlots = 4;

// Dynamic shared memory of a block: the operand ring (the partial rows of a cluster's k split land
// in the same memory once the ring is idle), after alignment to 1024 bytes.
constexpr size_t kPlRingBytes = 220 * 1024;
constexpr size_t plane_smem_bytes() { return 1024 + kPlRingBytes; }
static_assert(2 * ((size_t)(kBM + kMaxClusterRows) * (128 + 1) + 8 * 128) * 4 <= 150 * 1024, "the sent and the received rows of a k split");
static_assert(150 * 1024 + 64 * 128 * 4 <= 184 * 1024 && (128 * 128 + 128 + 128) * 4 <= 72 * 1024 && 72 * 1024 + 128 * 128 * 4 <= 184 * 1024 && 184 * 1024 + (2 * 4096 + kBM + 1) * 4 <= kPlRingBytes, "finished rows and staged lookups behind them");

// MN-major tile of 32-bit elements: atoms of 4 k-rows x 128 B (32 fp32 along mn) whose 32-byte
// chunks are XOR-ed with the k-row index modulo 4; the next 32 mn are 4096 B further (leading byte
// offset), the next 4 k 512 B further (stride byte offset).  Layout type 1 = SWIZZLE_128B_BASE32B.
__device__ __forceinline__ uint64_t make_mnmajor_sw128_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)(4096 >> 4) << 16;
    d |= (uint64_t)(512 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)1 << 61;
    return d;
}

// MN-major tile of 16-bit elements under the ordinary 128-byte swizzle: atoms of 8 k-rows x 128 B
// (64 elements along mn); a box holds 64 k-rows (8 KB), the next 64 mn are 8192 B further, the
// next 8 k 1024 B further.
__device__ __forceinline__ uint64_t make_mnmajor_sw128_desc16(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)(8192 >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// D[tmem] (+)= A[smem] * B[smem]^T, bf16 inputs, fp32 accumulate, K = 16 per instruction.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Instruction descriptor for bf16 inputs (format 1 at bits 7-9 and 10-12), fp32 accumulator.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// The copies of one slice of one plane: [ROWS x 32 k] fp32 or [ROWS x 64 k] bf16 (16 KB for 128 rows either way).
template <int ROWS>
__device__ __forceinline__ void tma_plane_tile(uint8_t* dst, const CUtensorMap* map, int mn_major, int bf16, int mn0, int k0, uint64_t* bar) {
    if (!mn_major) {
        tma_load_2d(dst, map, k0, mn0, bar);
    } else if (!bf16) {
#pragma unroll
        for (int j = 0; j < ROWS / 32; ++j) tma_load_2d(dst + j * 4096, map, mn0 + 32 * j, k0, bar);
    } else {
#pragma unroll
        for (int j = 0; j < ROWS / 64; ++j) tma_load_2d(dst + j * 8192, map, mn0 + 64 * j, k0, bar);
    }
}

// What the accumulating warps add up from the staged operand tiles while the slices pass:
//   SIDE_ROWSUM  the row sums of A (the L2 backward needs rowsum(A) . X);
//   SIDE_NORMS   the squared norms of the rows of A and of B (the L2 distance in contraction form).
enum Side : int { SIDE_NONE = 0, SIDE_ROWSUM = 1, SIDE_NORMS = 2 };
constexpr int EPI_L2_DISTANCE = 3;  // out = sqrt(|a|^2 + |b|^2 - 2 a.b), recomputed directly where that cancels

// The sum of 16 of the 32 k of row `row` of a staged A tile, added in k order.  The upper plane
// holds the operand's values themselves (the tensor core ignores their low bits), so it alone is read.
template <bool SQUARE = false>
__device__ __forceinline__ float staged_row_sum(const uint8_t* tile, int mn_major, int row, int half) {
    float s = 0.f;
    if (!mn_major) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint32_t off = (uint32_t)row * 128u + ((((uint32_t)(half * 4 + c)) ^ ((uint32_t)row & 7u)) << 4);
            const float4 v = *reinterpret_cast<const float4*>(tile + off);
            if (SQUARE) s += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
            else s += (v.x + v.y) + (v.z + v.w);
        }
    } else {
        const uint32_t base = (uint32_t)(row >> 5) * 4096u, r = (uint32_t)row & 31u;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t kk = (uint32_t)(half * 16 + i);
            s += *reinterpret_cast<const float*>(tile + base + kk * 128u + (((r >> 3) ^ (kk & 3u)) << 5) + ((r & 7u) << 2));
        }
    }
    return s;
}

__device__ __forceinline__ float tf32_lo(float v) { return tf32_hi(v - tf32_hi(v)); }

// The routing phase of a block that has finished the hidden rows [row0, row0 + n_rows) x [n0, n0 + BN)
// and left them in `fin` ([n_rows][BN], shared memory): every (lookup, 4 columns) pair is one unit
// of work, spread over all threads, so a row that hundreds of lookups name costs no thread more
// than any other.  s_look[i] = lookup | local row << 16 and s_rel[i] = relation of a head lookup
// were staged by route_stage.
template <int BN>
__device__ __forceinline__ void route_rows(const RouteArgs& rt, int mode, const float* fin, const uint32_t* s_look, const uint32_t* s_rel,
                                           int n_look, int n0, int D, int n_threads) {
    constexpr int kQuads = BN / 4;
    const int n_units = n_look * kQuads;
    for (int u0 = threadIdx.x; u0 < n_units; u0 += 4 * n_threads) {
        uint32_t look[4];
        float4 h[4], r[4];
        bool head[4], live[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int u = u0 + b * n_threads;
            live[b] = u < n_units;
            const int i = live[b] ? u / kQuads : 0, q = u % kQuads;
            look[b] = s_look[i];
            live[b] = live[b] && look[b] != kRouteSkip;
            if (!live[b]) look[b] = 0u;
            const uint32_t e = look[b] & 0xffffu;
            head[b] = e < (uint32_t)rt.B;
            live[b] = live[b] && n0 + q * 4 < D && ((head[b] ? mode & 1 : mode & 2) != 0);
            h[b] = *reinterpret_cast<const float4*>(fin + (size_t)(look[b] >> 16) * BN + q * 4);
            r[b] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (live[b] && head[b]) r[b] = *reinterpret_cast<const float4*>(rt.rel_table + (size_t)s_rel[i] * D + n0 + q * 4);
        }
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            if (!live[b]) continue;
            const int q = (u0 + b * n_threads) % kQuads;
            const uint32_t e = look[b] & 0xffffu;
            float4 o = h[b];
            float *dst, *dst_lo;
            if (head[b]) {
                // TransE / DistMult: elementwise with the relation row (ComplEx mixes the halves of a row: k_route)
                if (rt.score_fn == 0) o = make_float4(o.x + r[b].x, o.y + r[b].y, o.z + r[b].z, o.w + r[b].w);
                else o = make_float4(o.x * r[b].x, o.y * r[b].y, o.z * r[b].z, o.w * r[b].w);
                dst = rt.pred + (size_t)e * D;
                dst_lo = rt.lo_bf16 ? rt.pred_lo + (size_t)e * D / 2 : rt.pred_lo + (size_t)e * D;  // rows of D bf16 = D / 2 floats
            } else {
                const uint32_t j = e - (uint32_t)rt.B, shard = j / (uint32_t)rt.a2a, slot = j - shard * (uint32_t)rt.a2a;
                dst = rt.send_dst[shard] + (size_t)slot * D;
                dst_lo = rt.lo_bf16 ? rt.send_lo_dst[shard] + (size_t)slot * D / 2 : rt.send_lo_dst[shard] + (size_t)slot * D;
            }
            *reinterpret_cast<float4*>(dst + n0 + q * 4) = o;
            if (rt.lo_bf16) store4(reinterpret_cast<__nv_bfloat16*>(dst_lo) + n0 + q * 4, o);
            else *reinterpret_cast<float4*>(dst_lo + n0 + q * 4) = make_float4(tf32_lo(o.x), tf32_lo(o.y), tf32_lo(o.z), tf32_lo(o.w));
        }
    }
}

// Stages the lookups of the hidden rows [row0, row0 + n_rows) in shared memory and returns their
// number (at most kRouteMaxLookups: the launcher refuses larger batches).  Called by all threads.
__device__ __forceinline__ int route_stage(const RouteArgs& rt, int row0, int n_rows, uint32_t* s_off, uint32_t* s_look, uint32_t* s_rel,
                                           int n_threads) {
    if (n_rows <= 0) return 0;
    for (int r = threadIdx.x; r <= n_rows; r += n_threads) s_off[r] = rt.off[row0 + r];
    __syncthreads();
    const uint32_t q_lo = s_off[0];
    const int n_look = min((int)(s_off[n_rows] - q_lo), kRouteMaxLookups);
    for (int i = threadIdx.x; i < n_look; i += n_threads) {
        const uint32_t q = q_lo + (uint32_t)i, e = rt.perm[q];
        int lo = 0, hi = n_rows;  // the row r with s_off[r] <= q < s_off[r + 1]
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_off[mid] <= q) lo = mid; else hi = mid;
        }
        const bool elsewhere = rt.first_slot && (rt.first_slot[row0 + lo] & 2u);
        s_look[i] = elsewhere ? kRouteSkip : e | ((uint32_t)lo << 16);
        s_rel[i] = e < (uint32_t)rt.B && !elsewhere ? rt.relation[e] : 0u;
    }
    return n_look;
}

// The squared distance of two k-major rows in the direct form (the rare path: out of line).
static __device__ __noinline__ float l2_squared_direct(const float* __restrict__ a, const float* __restrict__ b, int K) {
    float s0 = 0.f, s1 = 0.f;
    int k = 0;
    for (; k + 7 < K; k += 8) {
        const float4 x0 = *reinterpret_cast<const float4*>(a + k), y0 = *reinterpret_cast<const float4*>(b + k);
        const float4 x1 = *reinterpret_cast<const float4*>(a + k + 4), y1 = *reinterpret_cast<const float4*>(b + k + 4);
        float d;
        d = x0.x - y0.x; s0 = fmaf(d, d, s0); d = x0.y - y0.y; s0 = fmaf(d, d, s0);
        d = x0.z - y0.z; s0 = fmaf(d, d, s0); d = x0.w - y0.w; s0 = fmaf(d, d, s0);
        d = x1.x - y1.x; s1 = fmaf(d, d, s1); d = x1.y - y1.y; s1 = fmaf(d, d, s1);
        d = x1.z - y1.z; s1 = fmaf(d, d, s1); d = x1.w - y1.w; s1 = fmaf(d, d, s1);
    }
    for (; k < K; ++k) {
        const float d = a[k] - b[k];
        s0 = fmaf(d, d, s0);
    }
    return s0 + s1;
}

// Distances of A row m to the B rows n .. n+3 from the contraction: d^2 = |a|^2 + |b|^2 - 2 a.b
// (src/poplar_extensions/distance.cpp:151-185 computes sqrt(sum (a - b)^2); the reference's own
// comment at src/poplar_kge.cpp:376-396 names this expansion).  The expansion loses the distance
// when the rows are close: where d^2 comes out below a fifth of |a|^2 + |b|^2 its relative error
// could pass 5e-6, so it is recomputed there in the direct form from the rows themselves, which
// also returns the exact zero for identical rows that the gradient rule tests for
// (l2distance.codelet.cpp:149-158).  Both operands are k-major; `acc` = a.b, an = |a|^2, bn = |b|^2.
// Here acc = a.b of output row m, columns n .. n + 3, becomes the distances: straight-line arithmetic
// except for one test per four outputs that sends near-cancelling pairs to the direct form.
__device__ __forceinline__ void l2_distance_four(const PlaneProblem& pp, int m, int n, float (&acc)[4], float an, const float (&bn)[4],
                                                 bool live = true) {
    const GemmArgs& g = pp.g;
    float d2[4];
    bool direct = false;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        d2[j] = an + bn[j] - 2.f * acc[j];
        direct |= n + j < g.N && d2[j] < 0.2f * (an + bn[j]);
    }
    if (direct && live) {  // not for units past the problem's edge: their rows do not exist
        const float* a = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(pp.A.hi) + (size_t)m * pp.A.row_stride_bytes);
#pragma unroll 1
        for (int j = 0; j < 4; ++j)
            if (n + j < g.N && d2[j] < 0.2f * (an + bn[j]))
                d2[j] = l2_squared_direct(a, reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(pp.B.hi) + (size_t)(n + j) * pp.B.row_stride_bytes), g.K);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = sqrtf(fmaxf(d2[j], 0.f));
}

__device__ __forceinline__ void store_four(const GemmArgs& g, int m, int n, const float (&acc)[4]) {
    float* out_row = g.out + (size_t)m * g.ldc;
    if ((g.N & 3) == 0 && (g.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(out_row) & 15) == 0) {
        *reinterpret_cast<float4*>(out_row + n) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (n + j < g.N) out_row[n + j] = acc[j];
    }
}

__device__ __forceinline__ void finish_l2_four(const PlaneProblem& pp, int m, int n, float (&acc)[4], float an, const float (&bn)[4]) {
    l2_distance_four(pp, m, n, acc, an, bn);
    store_four(pp.g, m, n, acc);
}

// predict's filter on four finished scores of query m (TopkFilterArgs): `cut` is the score of the
// query's cut-off key (+inf while there is none), `cutoff` the key itself.
__device__ __forceinline__ void topk_filter_four(const TopkFilterArgs& f, int N, int m, int n, const float (&dist)[4], float cut,
                                                 const unsigned long long* cutoff) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float score = f.score_is_gamma_minus ? f.gamma - dist[j] : dist[j];
        if (score >= cut) {  // rare once a cut-off exists; ties are decided by the keys
            const uint32_t table_row = f.first_row + (uint32_t)(n + j);
            if (n + j >= N || table_row > f.last_valid_row) continue;
            const unsigned long long key = topk_key(score, table_row);
            if (key > *cutoff) {
                const int slot = atomicAdd(f.cand_count + m, 1);
                if (slot < kTopkCandidates) f.cand[(size_t)m * kTopkCandidates + slot] = key;
            }
        }
    }
}

// 32 consecutive accumulator columns of this thread's TMEM lane, without waiting for them.
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
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
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// EPI >= 0: an instantiation for the training step's contractions, whose epilogue is known at
// compile time and which always run with fp32 planes and a k split over a cluster.  A block runs
// this kernel once on an SM whose instruction cache has never seen it, and most of it is
// straight-line code executed once: what the instantiation does not need is not fetched.
template <int BN, int SIDE, int EPI = -1>
__global__ void __launch_bounds__(kPlThreads, 1)
k_tc_planes(const __grid_constant__ PlanePair gp, const __grid_constant__ PlaneMaps maps) {
    constexpr bool kLean = EPI >= 0;
    static_assert(BN == 64 || BN == 128, "tile widths: 64 or 128 columns");
    constexpr int CPT = BN / 2;  // accumulator columns per accumulating thread: a warp reads one half of its 32 lanes' columns
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_full[kPlMaxStages], bar_empty[kPlMaxStages], bar_acc_ready[kPlTmemSlots], bar_acc_free[kPlTmemSlots];
    __shared__ uint64_t bar_reduce;
    __shared__ uint32_t tmem_slot;
    __shared__ __align__(16) float s_rowsum[2][kBM];
    __shared__ __align__(16) float s_colsum[2][BN];  // read in 16-byte pieces
    __shared__ unsigned long long s_cutoff[SIDE == SIDE_NORMS ? kBM : 1];  // the tile's queries' top-k cut-offs (TopkFilterArgs)
    __shared__ float s_cut_score[SIDE == SIDE_NORMS ? kBM : 1];            // their scores: a score below it cannot pass
    constexpr bool ROWSUM = SIDE != SIDE_NONE;

    const int which = (int)blockIdx.x >= gp.tiles_m0 ? 1 : 0;
    const PlaneProblem& pp = gp.p[which];
    const GemmArgs& g = pp.g;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = ((int)blockIdx.x - (which ? gp.tiles_m0 : 0)) * kBM, n0 = blockIdx.y * BN;
    const unsigned total_blocks = gridDim.x * gridDim.y * gridDim.z;
    if (n0 >= g.N || m0 >= g.M) {  // the two problems may differ in size (a whole cluster leaves together)
        grid_dependency_sync();
        exchange_signal(gp.sync, gp.signal_kind, total_blocks);
        return;
    }

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr uint32_t kATile = kBM * 128, kBTile = BN * 128;
    const int k_begin = blockIdx.z * g.k_per_split, k_end = min(g.K, k_begin + g.k_per_split);
    const int bf16 = kLean ? 0 : gp.bf16, slice_k = bf16 ? 64 : kBK;
    const int n_slices = max(0, (k_end - k_begin + slice_k - 1) / slice_k);
    const bool a_two = pp.A.lo != nullptr, b_two = pp.B.lo != nullptr;
    // a ring stage: A hi [| A lo] | B hi [| B lo]
    const uint32_t off_b = (a_two ? 2u : 1u) * kATile, stage_bytes = off_b + (b_two ? 2u : 1u) * kBTile;
    const int n_stages = gp.n_stages[which];

    if (tid == 0) {
        for (int s = 0; s < kPlMaxStages; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], ROWSUM ? 1 + kPlAccWarps : 1);
        }
        for (int t = 0; t < kPlTmemSlots; ++t) {
            mbar_init(&bar_acc_ready[t], 1);
            mbar_init(&bar_acc_free[t], kPlAccWarps);
        }
        mbar_init(&bar_reduce, 1);
        mbar_fence_init();
        // the TMA unit fetches the descriptors while the predecessor kernel still runs
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&maps.a_hi[which])) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&maps.b_hi[which])) : "memory");
        if (a_two) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&maps.a_lo[which])) : "memory");
        if (b_two) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&maps.b_lo[which])) : "memory");
    }
    constexpr int n_slots = kPlTmemSlots;
    if (warp == 0) tmem_alloc(&tmem_slot, (uint32_t)(n_slots * BN));
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    grid_dependency_sync();
    exchange_wait(gp.sync, gp.wait_kind);
    const uint32_t tmem_base = tmem_slot;
    if (!kLean && g.epilogue == EPI_ADD_TABLE_VALUE && g.cluster_splits <= 1 && tid >= 64 && tid < 64 + kBM && m0 + tid - 64 < g.M) {
        // A whole tile without a k split (predict's hidden rows): the table values that the epilogue
        // adds are asked into L2 now, a row per thread, so that the finishing loop, which fetches
        // them one unit after the other, waits for L2 and not for DRAM.
        const int m = m0 + tid - 64, elem = g.x_is_half ? 2 : 4;
        const size_t xr = g.x_gather ? g.x_gather[m] : (size_t)g.x_row_base + (size_t)m;
        const uint8_t* x = g.x_base + xr * (size_t)g.x_row_stride_bytes + (size_t)n0 * elem;
        const int bytes = min(BN, g.N - n0) * elem;
        for (int o = 0; o < bytes; o += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(x + o));
    }
    if (SIDE == SIDE_NORMS && pp.filter.cand != nullptr && tid >= 64 && tid < 64 + kBM) {
        const TopkFilterArgs& f = pp.filter;
        const int r = tid - 64, m = m0 + r;
        unsigned long long cutoff = ~0ull;  // rows past the problem: nothing passes
        if (m < g.M) {
            cutoff = f.counts[m] >= f.n_best ? f.state[(size_t)m * kTopkCapacity + f.n_best - 1] : 0ull;
            // no cut-off yet: every score is a candidate and the query scans its row of scores itself
            if (cutoff == 0ull && n0 == 0) f.cand_count[m] = kTopkCandidates + 1;
        }
        s_cutoff[r] = cutoff;  // read after the block-wide barrier that ends the k loop
        s_cut_score[r] = cutoff == 0ull || cutoff == ~0ull ? __int_as_float(0x7f800000) : topk_score(cutoff);
    }

    float acc[CPT];
#pragma unroll
    for (int j = 0; j < CPT; ++j) acc[j] = 0.f;
    float row_part = 0.f, col_part = 0.f;

    if (warp == 0) {
        for (int kc = 0; kc < n_slices; ++kc) {
            const int s = kc % n_stages, use = kc / n_stages;
            if (use >= 1) mbar_wait(&bar_empty[s], (uint32_t)((use - 1) & 1), g.status, 6u);
            if (lane == 0) {
                uint8_t* stage = smem + (size_t)s * stage_bytes;
                const int k0 = k_begin + kc * slice_k;
                mbar_arrive_expect(&bar_full[s], stage_bytes);
                tma_plane_tile<kBM>(stage, &maps.a_hi[which], pp.A.mn_major, bf16, m0, k0, &bar_full[s]);
                if (a_two) tma_plane_tile<kBM>(stage + kATile, &maps.a_lo[which], pp.A.mn_major, bf16, m0, k0, &bar_full[s]);
                tma_plane_tile<BN>(stage + off_b, &maps.b_hi[which], pp.B.mn_major, bf16, n0, k0, &bar_full[s]);
                if (b_two) tma_plane_tile<BN>(stage + off_b + kBTile, &maps.b_lo[which], pp.B.mn_major, bf16, n0, k0, &bar_full[s]);
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        const uint32_t idesc = make_idesc_tf32(kBM, BN) | (pp.A.mn_major ? (1u << 15) : 0u) | (pp.B.mn_major ? (1u << 16) : 0u);
        const uint64_t a_step = pp.A.mn_major ? (1024 >> 4) : (32 >> 4), b_step = pp.B.mn_major ? (1024 >> 4) : (32 >> 4);
        for (int kc = 0; kc < n_slices; ++kc) {
            const int s = kc % n_stages, t = kc % n_slots;
            mbar_wait(&bar_full[s], (uint32_t)((kc / n_stages) & 1), g.status, 3u);
            if (kc >= n_slots) mbar_wait(&bar_acc_free[t], (uint32_t)(((kc / n_slots) - 1) & 1), g.status, 4u);
            tc_fence_after();
            if (lane == 0) {
                const uint32_t a_hi = smem_u32(smem + (size_t)s * stage_bytes), a_lo = a_hi + kATile, b_hi = a_hi + off_b, b_lo = b_hi + kBTile;
                const uint32_t tmem_acc = tmem_base + (uint32_t)(t * BN);
                const uint64_t da_hi = pp.A.mn_major ? make_mnmajor_sw128_desc(a_hi) : make_kmajor_sw128_desc(a_hi);
                const uint64_t da_lo = pp.A.mn_major ? make_mnmajor_sw128_desc(a_lo) : make_kmajor_sw128_desc(a_lo);
                const uint64_t db_hi = pp.B.mn_major ? make_mnmajor_sw128_desc(b_hi) : make_kmajor_sw128_desc(b_hi);
                const uint64_t db_lo = pp.B.mn_major ? make_mnmajor_sw128_desc(b_lo) : make_kmajor_sw128_desc(b_lo);
                uint32_t accumulate = 0u;
                if (bf16) {
                    // one bf16 plane per operand, four 16-deep products per 64-deep slice
                    const uint32_t idesc16 = make_idesc_bf16(kBM, BN) | (pp.A.mn_major ? (1u << 15) : 0u) | (pp.B.mn_major ? (1u << 16) : 0u);
                    const uint64_t da = pp.A.mn_major ? make_mnmajor_sw128_desc16(a_hi) : make_kmajor_sw128_desc(a_hi);
                    const uint64_t db = pp.B.mn_major ? make_mnmajor_sw128_desc16(b_hi) : make_kmajor_sw128_desc(b_hi);
                    const uint64_t sa = pp.A.mn_major ? (2048 >> 4) : (32 >> 4), sb = pp.B.mn_major ? (2048 >> 4) : (32 >> 4);
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        umma_bf16(tmem_acc, da + (uint64_t)ks * sa, db + (uint64_t)ks * sb, idesc16, accumulate);
                        accumulate = 1u;
                    }
                } else {
#pragma unroll
                for (int ks = 0; ks < kBK / 8; ++ks) {
                    const uint64_t ka = (uint64_t)ks * a_step, kb = (uint64_t)ks * b_step;
                    // small cross terms first, the large hi*hi term last
                    if (b_two) { umma_tf32(tmem_acc, da_hi + ka, db_lo + kb, idesc, accumulate); accumulate = 1u; }
                    if (a_two) { umma_tf32(tmem_acc, da_lo + ka, db_hi + kb, idesc, accumulate); accumulate = 1u; }
                    umma_tf32(tmem_acc, da_hi + ka, db_hi + kb, idesc, accumulate);
                    accumulate = 1u;
                }
                }
                umma_commit(&bar_empty[s]);
                umma_commit(&bar_acc_ready[t]);
            }
            __syncwarp();
        }
    } else {
        const int quarter = warp & 3, half = (warp - 2) >> 2, row = quarter * 32 + lane;
        auto add_rows = [&](int kc) {
            const int s = kc % n_stages;
            mbar_wait(&bar_full[s], (uint32_t)((kc / n_stages) & 1), g.status, 7u);
            const uint8_t* stage = smem + (size_t)s * stage_bytes;
            if (SIDE == SIDE_NORMS) {  // both operands k-major
                row_part += staged_row_sum<true>(stage, 0, row, half);
                if (row < BN) col_part += staged_row_sum<true>(stage + off_b, 0, row, half);
            } else {
                row_part += staged_row_sum(stage, pp.A.mn_major, row, half);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_empty[s]);
        };
        if (ROWSUM && n_slices > 0) add_rows(0);
        for (int kc = 0; kc < n_slices; ++kc) {
            if (ROWSUM && kc + 1 < n_slices) add_rows(kc + 1);  // one slice ahead of the drain: the stage is not held back
            const int t = kc % n_slots;
            mbar_wait(&bar_acc_ready[t], (uint32_t)((kc / n_slots) & 1), g.status, 1u);
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(t * BN + half * CPT);
            uint32_t r[CPT / 32][32];
#pragma unroll
            for (int c = 0; c < CPT / 32; ++c) tmem_ld32_issue(taddr + (uint32_t)(c * 32), r[c]);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_acc_free[t]);
#pragma unroll
            for (int c = 0; c < CPT / 32; ++c)
#pragma unroll
                for (int j = 0; j < 32; ++j) acc[c * 32 + j] += __uint_as_float(r[c][j]);
        }
        if (ROWSUM) s_rowsum[half][row] = row_part;
        if (SIDE == SIDE_NORMS && row < BN) s_colsum[half][row] = col_part;
    }
    __syncthreads();  // every slice has been read from TMEM (so the ring is idle); the row sums are in place

    // Routing (hidden rows to their lookups): the finished rows and the staged lookups live in the
    // idle ring, behind what the k-split exchange uses.
    const bool routing = (!kLean || EPI == EPI_ADD_TABLE_VALUE) && gp.route.perm != nullptr && gp.route.mode[which] != 0;
    float* fin = reinterpret_cast<float*>(smem + 150 * 1024);                              // [<= 64 rows][BN], or [128][BN] at offset 0 without a k split
    uint32_t* s_look = reinterpret_cast<uint32_t*>(smem + 184 * 1024);                      // [kRouteMaxLookups]
    uint32_t* s_rel = s_look + kRouteMaxLookups;                                            // [kRouteMaxLookups]
    uint32_t* s_off = s_rel + kRouteMaxLookups;                                             // [kBM + 1]
    int route_n = 0;
    const bool acc_warp = warp >= 2;
    const int row = (warp & 3) * 32 + lane, m = m0 + row;
    const int nc0 = n0 + (acc_warp ? ((warp - 2) >> 2) * CPT : 0);  // first output column of an accumulating thread
    {
        // Block z of the cluster finishes rows z * rows_each ... of the tile.  Every block lays its
        // partial tile out in its own (now idle) operand ring, one slot per owner, and hands each
        // slot to the copy engine (cp.async.bulk from its shared memory into the owner's), which
        // reports the bytes to the owner's mbarrier; the owner then adds the slots in split order.
        // A block may be written to only after it has left its k loop: that is the first cluster
        // barrier (arrive here, wait before the copies are issued).  Without a k split the block is
        // the only owner: its rows take the same way through shared memory, which turns one thread's
        // row of the accumulator into whole rows stored by neighbouring threads.
        const bool clustered = kLean || g.cluster_splits > 1;
        if (clustered) cluster_arrive_relaxed();
        const int n_split = clustered ? g.cluster_splits : 1, rank = clustered ? (int)cluster_rank() : 0;
        const int rows_each = (kBM + n_split - 1) / n_split;
        const uint32_t off_rowsum = (uint32_t)rows_each * BN, off_colsum = off_rowsum + (uint32_t)((rows_each + 3) & ~3);
        const uint32_t slot_floats = off_colsum + (SIDE == SIDE_NORMS ? BN : 0);  // rows | row sums | column sums
        const uint32_t slot_bytes = slot_floats * 4u;
        float* staging = reinterpret_cast<float*>(smem);                   // [owner][rows_each][BN] + sums, what I send
        float* receive = staging + (size_t)n_split * slot_floats;         // [source][rows_each][BN] + sums, what I own
        if (!clustered) fin = reinterpret_cast<float*>(smem + 72 * 1024);  // one slot of 67 KB only: the finished rows follow it
        if (clustered && tid == 0) mbar_arrive_expect(&bar_reduce, (uint32_t)(n_split - 1) * slot_bytes);
        // A whole tile of distances (predict's score pass): the thread that holds a row of the
        // accumulator turns its dot products into distances before they are staged, as one stretch
        // of straight-line code, so that the arithmetic of all of them overlaps; what follows the
        // staging is then a plain copy.  The two rare cases leave a bit each and are dealt with after
        // the staging, in shared memory: near-cancelling pairs (recomputed in the direct form) and,
        // for predict's top-k (TopkFilterArgs), scores that reach the row's cut-off.  The square root
        // is the approximate one (relative error 2^-23, exact at zero): the form's own error is larger.
        uint32_t direct_bits[CPT / 32] = {}, pass_bits[CPT / 32] = {};
        const bool whole_tile = SIDE == SIDE_NORMS && !clustered && acc_warp;
        const bool filtering = whole_tile && pp.filter.cand != nullptr && m < g.M;
        if (whole_tile) {
            const float an = s_rowsum[0][row] + s_rowsum[1][row];
            const float cut = filtering ? s_cut_score[row] : __int_as_float(0x7f800000);
            const float sign = pp.filter.score_is_gamma_minus ? -1.f : 1.f, offset = pp.filter.score_is_gamma_minus ? pp.filter.gamma : 0.f;
#pragma unroll
            for (int j0 = 0; j0 < CPT; j0 += 4) {
                const int tc0 = (nc0 - n0) + j0;  // tile column of acc[j0]
                const float4 c0 = *reinterpret_cast<const float4*>(&s_colsum[0][tc0]), c1 = *reinterpret_cast<const float4*>(&s_colsum[1][tc0]);
                const float bn[4] = {c0.x + c1.x, c0.y + c1.y, c0.z + c1.z, c0.w + c1.w};
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const float both = an + bn[t], d2 = both - 2.f * acc[j0 + t];
                    direct_bits[(j0 + t) >> 5] |= (uint32_t)(d2 < 0.2f * both) << ((j0 + t) & 31);
                    float dist;
                    asm("sqrt.approx.f32 %0, %1;" : "=f"(dist) : "f"(fmaxf(d2, 0.f)));
                    acc[j0 + t] = dist;
                    pass_bits[(j0 + t) >> 5] |= (uint32_t)(fmaf(sign, dist, offset) >= cut) << ((j0 + t) & 31);
                }
            }
        }
        if (acc_warp) {
            // 16-byte chunk c of tile row `row` lies at chunk c ^ (row & 7): the lanes of a warp hold
            // 32 different rows, and this spreads their stores over all banks
            const int owner = row / rows_each, local = row - owner * rows_each;
            float* mine = staging + (size_t)owner * slot_floats + (size_t)local * BN;
            const int c0 = (nc0 - n0) >> 2;
#pragma unroll
            for (int j = 0; j < CPT; j += 4)
                *reinterpret_cast<float4*>(mine + (((c0 + (j >> 2)) ^ (row & 7)) << 2)) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
            if (ROWSUM && nc0 == n0) staging[(size_t)owner * slot_floats + off_rowsum + local] = s_rowsum[0][row] + s_rowsum[1][row];
            if (whole_tile && m < g.M) {
                const float* a_row = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(pp.A.hi) + (size_t)m * pp.A.row_stride_bytes);
#pragma unroll
                for (int w = 0; w < CPT / 32; ++w) {
                    uint32_t todo = direct_bits[w] | (filtering ? pass_bits[w] : 0u);
                    while (todo) {
                        const int bit = __ffs(todo) - 1, tcol = (nc0 - n0) + w * 32 + bit, col = n0 + tcol;
                        todo &= todo - 1;
                        if (col >= g.N) continue;
                        float* cell = mine + (((tcol >> 2) ^ (row & 7)) << 2) + (tcol & 3);
                        if ((direct_bits[w] >> bit) & 1u) {
                            const float d2 = l2_squared_direct(a_row, reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(pp.B.hi) + (size_t)col * pp.B.row_stride_bytes), g.K);
                            *cell = sqrtf(d2);
                        }
                        if (filtering) {
                            const TopkFilterArgs& f = pp.filter;
                            const float score = f.score_is_gamma_minus ? f.gamma - *cell : *cell;
                            const uint32_t table_row = f.first_row + (uint32_t)col;
                            if (table_row > f.last_valid_row) continue;
                            const unsigned long long key = topk_key(score, table_row);
                            if (key > s_cutoff[row]) {  // ties with the cut-off are decided by the keys
                                const int slot = atomicAdd(f.cand_count + m, 1);
                                if (slot < kTopkCandidates) f.cand[(size_t)m * kTopkCandidates + slot] = key;
                            }
                        }
                    }
                }
            }
        }
        if (SIDE == SIDE_NORMS)  // every owner gets this split's part of the column norms
            for (int u = tid; u < n_split * BN; u += kPlThreads)
                staging[(size_t)(u / BN) * slot_floats + off_colsum + (u % BN)] = s_colsum[0][u % BN] + s_colsum[1][u % BN];
        if (clustered) fence_async_shared();  // the copy engine reads what the threads have just written
        const int r_begin = rank * rows_each, r_end = min(kBM, r_begin + rows_each);
        constexpr int kQuads = BN / 4;
        // a split owns at most 64 rows x BN / 4 quads (22 rows in the training step's instantiations: six splits or more)
        constexpr int kUnits = ((kLean ? 22 : 64) * kQuads + kPlThreads - 1) / kPlThreads;
        const int n_units = max(0, r_end - r_begin) * kQuads;
        float xv[kUnits][4];
        if (clustered) {
#pragma unroll
            for (int i = 0; i < kUnits; ++i) {  // the epilogue's second operand is fetched while the rows travel
                const int u = tid + i * kPlThreads;
                const int mm = m0 + r_begin + u / kQuads, nn = n0 + (u % kQuads) * 4;
                xv[i][0] = xv[i][1] = xv[i][2] = xv[i][3] = 0.f;
                if (u < n_units && mm < g.M && nn < g.N) load_x_four(g, mm, nn, xv[i], EPI);
            }
        }
        if (routing) route_n = route_stage(gp.route, m0 + r_begin, max(0, min(r_end, g.M - m0) - r_begin), s_off, s_look, s_rel, kPlThreads);
        __syncthreads();
        if (clustered) {
            cluster_wait();
            if (warp == 0 && lane < n_split && lane != rank) {
                const uint32_t dst = cluster_map(smem_u32(receive + (size_t)rank * slot_floats), (uint32_t)lane);
                const uint32_t bar = cluster_map(smem_u32(&bar_reduce), (uint32_t)lane);
                asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(dst), "r"(smem_u32(staging + (size_t)lane * slot_floats)), "r"(slot_bytes), "r"(bar) : "memory");
            }
            mbar_wait(&bar_reduce, 0u, g.status, 8u);
            // Nobody may leave while the copy engine can still read its slots.  Every block reports here
            // that all of its bytes have arrived and checks before it exits that all blocks have.
            cluster_arrive_relaxed();
        }
        auto finish_unit = [&](int u, const float* x_ready) {
            const int local = u / kQuads, q = u % kQuads, trow = r_begin + local;
            const int chunk = (q ^ (trow & 7)) << 2;
            float sum[4] = {0.f, 0.f, 0.f, 0.f}, col_total[4] = {0.f, 0.f, 0.f, 0.f};
            float row_total = 0.f;
            for (int z = 0; z < n_split; ++z) {
                const float* slot = z == rank ? staging + (size_t)rank * slot_floats : receive + (size_t)z * slot_floats;
                const float4 v = *reinterpret_cast<const float4*>(slot + (size_t)local * BN + chunk);
                sum[0] += v.x; sum[1] += v.y; sum[2] += v.z; sum[3] += v.w;
                if (ROWSUM) row_total += slot[off_rowsum + local];
                if (SIDE == SIDE_NORMS) {
                    const float4 c = *reinterpret_cast<const float4*>(slot + off_colsum + q * 4);
                    col_total[0] += c.x; col_total[1] += c.y; col_total[2] += c.z; col_total[3] += c.w;
                }
            }
            const int mm = m0 + trow, nn = n0 + q * 4;
            if (mm >= g.M || nn >= g.N) return;
            if (SIDE == SIDE_NORMS) {
                finish_l2_four(pp, mm, nn, sum, row_total, col_total);
                if (pp.filter.cand != nullptr) topk_filter_four(pp.filter, g.N, mm, nn, sum, s_cut_score[trow], &s_cutoff[trow]);
            } else {
                float x[4];
                if (x_ready) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) x[j] = x_ready[j];
                } else {
                    load_x_four(g, mm, nn, x, EPI);
                }
                finish_four(g, g.out, mm, nn, sum, x, row_total, EPI);
            }
            if (routing) *reinterpret_cast<float4*>(fin + (size_t)local * BN + q * 4) = make_float4(sum[0], sum[1], sum[2], sum[3]);
        };
        if (clustered) {
#pragma unroll
            for (int i = 0; i < kUnits; ++i)
                if (tid + i * kPlThreads < n_units) finish_unit(tid + i * kPlThreads, xv[i]);
        } else if (SIDE == SIDE_NORMS || (g.epilogue == EPI_STORE && g.out_blocks == nullptr && !routing)) {
            // the staged rows are finished (distances, or a plain product): whole rows go out in 16-byte pieces
#pragma unroll 4
            for (int u = tid; u < n_units; u += kPlThreads) {
                const int local = u / kQuads, q = u % kQuads, mm = m0 + local, nn = n0 + q * 4;
                const float4 v = *reinterpret_cast<const float4*>(staging + (size_t)local * BN + ((q ^ (local & 7)) << 2));
                const float four[4] = {v.x, v.y, v.z, v.w};
                if (mm < g.M && nn < g.N) store_four(g, mm, nn, four);
            }
        } else {
            // one unit after the other: unrolling this loop costs more in instruction fetches (the body
            // holds every epilogue) than the overlap gains
            for (int u = tid; u < n_units; u += kPlThreads) finish_unit(u, nullptr);
        }
        if (clustered) cluster_wait();
    }
    if (routing) {
        __syncthreads();  // the finished rows are in `fin`
        route_rows<BN>(gp.route, gp.route.mode[which], fin, s_look, s_rel, route_n, n0, g.N, kPlThreads);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, (uint32_t)(n_slots * BN));
    exchange_signal(gp.sync, gp.signal_kind, total_blocks);
}

// Splits fp32 values into the two planes the contraction reads (for operands that no kernel of the
// step produces: parameters written by the host, operator inputs).
static __global__ void __launch_bounds__(256) k_split_planes(const float* __restrict__ x, size_t n, float* __restrict__ hi, float* __restrict__ lo) {
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const float v = x[e], h = tf32_hi(v);
        hi[e] = h;
        lo[e] = tf32_hi(v - h);
    }
}

// What a producing kernel stores for four neighbouring values.
__device__ __forceinline__ void store_planes4(float* hi, float* lo, size_t e, float a, float b, float c, float d) {
    const float4 h = make_float4(tf32_hi(a), tf32_hi(b), tf32_hi(c), tf32_hi(d));
    *reinterpret_cast<float4*>(hi + e) = h;
    *reinterpret_cast<float4*>(lo + e) = make_float4(tf32_hi(a - h.x), tf32_hi(b - h.y), tf32_hi(c - h.z), tf32_hi(d - h.w));
}

// ---------------------------------------------------------------------------
// Host side

// The map of one plane: boxes of [rows x 32 k] (k-major) or [32 k x 32 mn] (mn-major) under the
// 128-byte swizzle, zeros outside the matrix.
inline cudaError_t make_plane_map(const float* base, const PlaneOperand& op, int mn, int k, int rows, CUtensorMap* map) {
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return cudaErrorNotSupported;
    if (reinterpret_cast<uintptr_t>(base) % 16 || op.row_stride_bytes % 16) return cudaErrorInvalidValue;
    const bool bf16 = op.elem_bytes == 2;
    const cuuint64_t dims[2] = {(cuuint64_t)(op.mn_major ? mn : k), (cuuint64_t)(op.mn_major ? k : mn)};
    const cuuint64_t strides[1] = {(cuuint64_t)op.row_stride_bytes};
    // 128 bytes along the contiguous dimension; a slice is 32 k deep in fp32 and 64 k deep in bf16
    const cuuint32_t inner = bf16 ? 64u : 32u;
    const cuuint32_t box[2] = {inner, (cuuint32_t)(op.mn_major ? inner : rows)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims,
                              strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              op.mn_major && !bf16 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

inline bool planes_aligned(const PlaneOperand& op) {
    return reinterpret_cast<uintptr_t>(op.hi) % 16 == 0 && reinterpret_cast<uintptr_t>(op.lo) % 16 == 0 && op.row_stride_bytes % 16 == 0;
}

template <int BN, int SIDE, int EPI = -1>
inline cudaError_t configure_planes() {
    static bool configured[kMaxDeviceOrdinals] = {};
    const int slot = current_device_slot();
    if (slot >= 0 && configured[slot]) return cudaSuccess;
    cudaError_t err = cudaFuncSetAttribute(k_tc_planes<BN, SIDE, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plane_smem_bytes());
    if (err == cudaSuccess && slot >= 0) configured[slot] = true;
    return err;
}

// How many clusters of `splits` blocks of k_tc_planes the current device holds at once (one block
// per SM whatever the tile width, so one instantiation answers for all).
inline int max_resident_plane_clusters(int splits) {
    static int cached[kMaxDeviceOrdinals][kMaxClusterSplits + 1] = {};
    static bool known[kMaxDeviceOrdinals][kMaxClusterSplits + 1] = {};
    if (splits < 1 || splits > kMaxClusterSplits) return 0;
    const int slot = current_device_slot();
    if (slot >= 0 && known[slot][splits]) return cached[slot][splits];
    int n = 0;
    if (configure_planes<128, SIDE_NONE>() == cudaSuccess) {
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(1, 1, splits);
        config.blockDim = dim3(kPlThreads);
        config.dynamicSmemBytes = plane_smem_bytes();
        cudaLaunchAttribute attribute[1];
        attribute[0].id = cudaLaunchAttributeClusterDimension;
        attribute[0].val.clusterDim.x = 1;
        attribute[0].val.clusterDim.y = 1;
        attribute[0].val.clusterDim.z = (unsigned)splits;
        config.attrs = attribute;
        config.numAttrs = 1;
        if (cudaOccupancyMaxActiveClusters(&n, k_tc_planes<128, SIDE_NONE>, &config) != cudaSuccess) {
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

// A launch with its tensor maps encoded (encoding costs the host a few microseconds per map; a
// launch that is repeated, or captured into a graph, pays it once).
struct PlaneLaunch {
    PlanePair gp;
    PlaneMaps maps;
    dim3 grid;
    int splits, tile_n;
};

// One or two contractions of the same kind in one launch, tiles of 128 x tile_n (64 or 128).
// splits > 1: the blocks of a tile form a cluster (at most kMaxClusterSplits) and g.k_per_split
// must be set accordingly by the caller.
inline cudaError_t prepare_planes(const PlaneProblem* problems, int n_problems, int splits, int tile_n, PlaneLaunch* out,
                                  const ExchangeSync& sync = ExchangeSync{}, int wait_kind = -1, int signal_kind = -1,
                                  const RouteArgs* route = nullptr) {
    if (splits < 1 || splits > kMaxClusterSplits || (tile_n != 64 && tile_n != 128)) return cudaErrorInvalidValue;
    PlanePair& gp = out->gp;
    gp = PlanePair{};
    gp.p[0] = problems[0];
    gp.p[1] = problems[n_problems > 1 ? 1 : 0];
    gp.tiles_m0 = (problems[0].g.M + kBM - 1) / kBM;
    gp.sync = sync;
    gp.wait_kind = wait_kind;
    gp.signal_kind = signal_kind;
    if (route) gp.route = *route;
    int tiles_m = gp.tiles_m0, tiles_n = (problems[0].g.N + tile_n - 1) / tile_n;
    if (n_problems > 1) {
        tiles_m += (problems[1].g.M + kBM - 1) / kBM;
        tiles_n = std::max(tiles_n, (problems[1].g.N + tile_n - 1) / tile_n);
    }
    gp.bf16 = problems[0].A.elem_bytes == 2 ? 1 : 0;
    for (int i = 0; i < 2; ++i) {
        PlaneProblem& q = gp.p[i];
        if ((q.A.elem_bytes == 2) != (gp.bf16 != 0) || (q.B.elem_bytes == 2) != (gp.bf16 != 0)) return cudaErrorInvalidValue;
        if (gp.bf16 && (q.A.lo || q.B.lo || q.g.k_per_split % 64)) return cudaErrorInvalidValue;
        q.g.ws = nullptr;
        q.g.cluster_splits = splits > 1 ? splits : 0;
        if (!planes_aligned(q.A) || !planes_aligned(q.B)) return cudaErrorInvalidValue;
        cudaError_t err = make_plane_map(q.A.hi, q.A, q.g.M, q.g.K, kBM, &out->maps.a_hi[i]);
        if (err == cudaSuccess) err = make_plane_map(q.A.lo ? q.A.lo : q.A.hi, q.A, q.g.M, q.g.K, kBM, &out->maps.a_lo[i]);
        if (err == cudaSuccess) err = make_plane_map(q.B.hi, q.B, q.g.N, q.g.K, tile_n, &out->maps.b_hi[i]);
        if (err == cudaSuccess) err = make_plane_map(q.B.lo ? q.B.lo : q.B.hi, q.B, q.g.N, q.g.K, tile_n, &out->maps.b_lo[i]);
        if (err != cudaSuccess) return err;
        const size_t stage = (size_t)(q.A.lo ? 2 : 1) * kBM * 128 + (size_t)(q.B.lo ? 2 : 1) * tile_n * 128;
        gp.n_stages[i] = (int)std::min<size_t>(kPlMaxStages, kPlRingBytes / stage);
    }
    out->grid = dim3(tiles_m, tiles_n, splits);
    out->splits = splits;
    out->tile_n = tile_n;
    return cudaSuccess;
}

template <int SIDE, int EPI>
inline cudaError_t launch_lean(const PlaneLaunch& l, cudaStream_t stream) {
    cudaError_t err = configure_planes<128, SIDE, EPI>();
    if (err != cudaSuccess) return err;
    return launch_dependent_cluster(k_tc_planes<128, SIDE, EPI>, l.grid, dim3(kPlThreads), plane_smem_bytes(), stream, (unsigned)l.splits, l.gp,
                                    l.maps);
}

template <int SIDE>
inline cudaError_t launch_prepared(const PlaneLaunch& l, cudaStream_t stream) {
    if (SIDE != SIDE_NONE && l.gp.bf16) return cudaErrorInvalidValue;  // the side sums read fp32 tiles
    if (SIDE == SIDE_NORMS)
        for (int i = 0; i < 2; ++i)
            if (l.gp.p[i].A.mn_major || l.gp.p[i].B.mn_major || l.gp.p[i].g.out_blocks) return cudaErrorInvalidValue;
    if (l.tile_n == 128) {
        // the training step's contractions (fp32 planes, k split over a cluster, one epilogue for the launch)
        const int epilogue = l.gp.p[0].g.epilogue;
        const bool lean = SIDE != SIDE_NORMS && !l.gp.bf16 && l.splits >= 6 && l.gp.p[1].g.epilogue == epilogue;
        if constexpr (SIDE == SIDE_NONE) {
            if (lean && epilogue == EPI_ADD_TABLE_VALUE) return launch_lean<SIDE_NONE, EPI_ADD_TABLE_VALUE>(l, stream);
            if (lean && epilogue == EPI_DENSE_ADAM) return launch_lean<SIDE_NONE, EPI_DENSE_ADAM>(l, stream);
            if (lean && epilogue == EPI_STORE) return launch_lean<SIDE_NONE, EPI_STORE>(l, stream);
        } else if constexpr (SIDE == SIDE_ROWSUM) {
            if (lean && epilogue == EPI_ROWSUM_X_MINUS) return launch_lean<SIDE_ROWSUM, EPI_ROWSUM_X_MINUS>(l, stream);
        }
        cudaError_t err = configure_planes<128, SIDE>();
        if (err != cudaSuccess) return err;
        return launch_dependent_cluster(k_tc_planes<128, SIDE>, l.grid, dim3(kPlThreads), plane_smem_bytes(), stream,
                                        (unsigned)l.splits, l.gp, l.maps);
    }
    cudaError_t err = configure_planes<64, SIDE>();
    if (err != cudaSuccess) return err;
    return launch_dependent_cluster(k_tc_planes<64, SIDE>, l.grid, dim3(kPlThreads), plane_smem_bytes(), stream,
                                    (unsigned)l.splits, l.gp, l.maps);
}

template <int SIDE>
inline cudaError_t launch_planes(const PlaneProblem* problems, int n_problems, int splits, int tile_n, cudaStream_t stream,
                                 const ExchangeSync& sync = ExchangeSync{}, int wait_kind = -1, int signal_kind = -1,
                                 const RouteArgs* route = nullptr) {
    PlaneLaunch l;
    cudaError_t err = prepare_planes(problems, n_problems, splits, tile_n, &l, sync, wait_kind, signal_kind, route);
    if (err != cudaSuccess) return err;
    return launch_prepared<SIDE>(l, stream);
}

}  // namespace tc
}  // namespace kge
