// Device kernels of the BESS training step for sm_100a.
//
// Naming follows the reference's step (src/poplar_kge.cpp:664-707): rows of the stacked
// shard table are gathered by `remote`, turned into hidden vectors, looked up by `head`
// and `a2a`, exchanged, scored against the batch-shared tails, and the gradients flow
// back the same way into a row-wise Adam update.  All arithmetic is fp32.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "exchange.cuh"
#include "pdl.cuh"

namespace kge {

enum ScoreFn : int { SCORE_TRANSE = 0, SCORE_DISTMULT = 1, SCORE_COMPLEX = 2, SCORE_ROTATE = 3, SCORE_TRANSH = 4 };
// TransE, RotatE and TransH score by gamma - distance (src/poplar_kge.cpp:492-499, 532-537, 552-565); the others by the raw product.
__host__ __device__ inline bool score_is_gamma_minus_distance(int score_fn) { return score_fn == SCORE_TRANSE || score_fn == SCORE_ROTATE || score_fn == SCORE_TRANSH; }

// RotatE's relation row holds one angle per complex pair.  The reference casts the angles to
// float16 and takes sine and cosine in float16 (src/poplar_kge.cpp:522-525): restated as the
// correctly rounded float16 of the exact value (double-precision sin / cos of the rounded angle).
__device__ __forceinline__ void rotate_sin_cos(float angle, float& s, float& c) {
    const double theta = (double)__half2float(__float2half_rn(angle));
    s = __half2float(__double2half(sin(theta)));
    c = __half2float(__double2half(cos(theta)));
}
__device__ __forceinline__ float round_to_half(float x) { return __half2float(__float2half_rn(x)); }
enum DistFn : int { DIST_L1 = 0, DIST_L2 = 1, DIST_DOT = 2 };
enum LossFn : int { LOSS_LOGSIGMOID = 0, LOSS_SOFTMAX = 1 };

// Byte layout of one table row: value | adam_m | sqrt(adam_v) | feature
// (src/poplar_kge.cpp:405-417).  Every segment starts on a 16-byte boundary and
// row_bytes is a multiple of 16, so 128-bit accesses are always aligned.
struct RowLayout {
    uint32_t row_bytes;
    uint32_t off_m;
    uint32_t off_q;
    uint32_t off_feat;
    uint32_t d;
    uint32_t f;
    // 1: the value segment holds bfloat16 while adam_m and sqrt(adam_v) keep the state type (bf16
    // embeddings with fp32 optimiser state; the reference has one type per row, src/poplar_kge.cpp:405-417)
    uint32_t value_bf16;
};

struct AdamParams {
    float beta_m;
    float beta_v;
    float one_minus_beta_m;
    float one_minus_beta_v;
    float epsilon;
    float weight_decay;
};

__device__ __forceinline__ float load_as_float(const float* p) { return *p; }
__device__ __forceinline__ float load_as_float(const __half* p) { return __half2float(*p); }
__device__ __forceinline__ void store_from_float(float* p, float v) { *p = v; }
__device__ __forceinline__ void store_from_float(__half* p, float v) { *p = __float2half_rn(v); }

__device__ __forceinline__ float load_as_float(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void store_from_float(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&lo);
    raw.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}
// Element c of a row's value segment, whose type the layout names.
template <class ST>
__device__ __forceinline__ float load_value(const RowLayout& L, const uint8_t* row, int c) {
    return L.value_bf16 ? load_as_float(reinterpret_cast<const __nv_bfloat16*>(row) + c) : load_as_float(reinterpret_cast<const ST*>(row) + c);
}
template <class ST>
__device__ __forceinline__ void store_value(const RowLayout& L, uint8_t* row, int c, float v) {
    if (L.value_bf16) store_from_float(reinterpret_cast<__nv_bfloat16*>(row) + c, v);
    else store_from_float(reinterpret_cast<ST*>(row) + c, v);
}

// Four consecutive elements starting at an element index that is a multiple of 4.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __half* p) {
    uint2 raw = *reinterpret_cast<const uint2*>(p);
    __half2 lo = *reinterpret_cast<__half2*>(&raw.x);
    __half2 hi = *reinterpret_cast<__half2*>(&raw.y);
    float2 a = __half22float2(lo), b = __half22float2(hi);
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__half* p, float4 v) {
    __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&lo);
    raw.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

// Block-wide reductions with a fixed tree, so results do not depend on scheduling.
template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w) total += scratch[w];
    return total;
}
template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* scratch) {
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = scratch[0];
#pragma unroll
    for (int w = 1; w < THREADS / 32; ++w) total = fmaxf(total, scratch[w]);
    return total;
}

// Holds the stream for about `cycles` clock ticks (bounded by the argument), so that the host can
// queue the launches that follow before the first of them starts: per-kernel event timing then
// measures kernels, not the host's launch rate.
static __global__ void k_delay(long long cycles) {
    const long long start = clock64();
    while (clock64() - start < cycles) {
    }
}

// ---------------------------------------------------------------------------
// The step's row gather (fr::Buffer::read through getEntityData, src/fructose/fructose.cpp:790-798,
// src/poplar_kge.cpp:405-410): the R rows named by `remote` are copied whole, with 128-bit
// accesses, from the shard table (tens of gigabytes, so every row is a DRAM and TLB miss) into a
// compact buffer with the same row layout.  One warp per row with all of its loads in flight
// before the first store; everything after this kernel in the step reads the compact,
// L2-resident copy.
// What the tensor-core contractions read of a gathered row's features: fp16 features are widened
// to fp32 (exact, one TF32 plane) into feat_wide [R, feat_stride]; fp32 features are read in place
// (the compact copy is their upper plane) and only their lower plane feat_lo is written.  Both null:
// nothing extra.
struct FeaturePlanes {
    float* wide;   // fp16 features as fp32
    float* lo;     // lower TF32 plane of fp32 features
    uint32_t stride;    // floats per row of either
    uint32_t off_feat;  // byte offset of the features in a table row (multiple of 16)
};

__device__ __forceinline__ float tf32_upper(float x) { return __uint_as_float(__float_as_uint(x) & 0xFFFFE000u); }
__device__ __forceinline__ float tf32_lower(float x) { return tf32_upper(x - tf32_upper(x)); }
__device__ __forceinline__ float4 tf32_lower4(float4 v) { return make_float4(tf32_lower(v.x), tf32_lower(v.y), tf32_lower(v.z), tf32_lower(v.w)); }

static __global__ void __launch_bounds__(256)
k_gather_step_rows(const uint8_t* __restrict__ table, uint32_t row_bytes, const uint32_t* __restrict__ remote, int R,
                   uint8_t* __restrict__ rows_c, FeaturePlanes fp) {
    grid_dependency_sync();
    const int r = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= R) return;
    const uint4* __restrict__ src = reinterpret_cast<const uint4*>(table + (size_t)remote[r] * row_bytes);
    uint4* __restrict__ dst = reinterpret_cast<uint4*>(rows_c + (size_t)r * row_bytes);
    const int chunks = (int)(row_bytes >> 4), feat_chunk0 = (int)(fp.off_feat >> 4);
    for (int c0 = lane; c0 < chunks; c0 += 32 * 8) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (c0 + 32 * u < chunks) v[u] = src[c0 + 32 * u];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int c = c0 + 32 * u;
            if (c >= chunks) continue;
            dst[c] = v[u];
            if (c < feat_chunk0) continue;
            if (fp.wide) {  // 8 fp16 values
                const int f = (c - feat_chunk0) * 8;
                const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v[u].x)), b = __half22float2(*reinterpret_cast<const __half2*>(&v[u].y));
                const float2 cc = __half22float2(*reinterpret_cast<const __half2*>(&v[u].z)), d = __half22float2(*reinterpret_cast<const __half2*>(&v[u].w));
                float* o = fp.wide + (size_t)r * fp.stride + f;
                if (f < (int)fp.stride) *reinterpret_cast<float4*>(o) = make_float4(a.x, a.y, b.x, b.y);
                if (f + 4 < (int)fp.stride) *reinterpret_cast<float4*>(o + 4) = make_float4(cc.x, cc.y, d.x, d.y);
            } else if (fp.lo) {  // 4 fp32 values
                const int f = (c - feat_chunk0) * 4;
                if (f < (int)fp.stride)
                    *reinterpret_cast<float4*>(fp.lo + (size_t)r * fp.stride + f) =
                        tf32_lower4(make_float4(__uint_as_float(v[u].x), __uint_as_float(v[u].y), __uint_as_float(v[u].z), __uint_as_float(v[u].w)));
            }
        }
    }
}

// ---------------------------------------------------------------------------
// hidden = value + feature . W   (src/poplar_kge.cpp:439-467 with the gather of :405-410
// folded in).  A [R, F] is read straight from the gathered table rows; W is [F, D].
// Rows are table[remote[m]], or the consecutive rows row_base + m when `remote` is null
// (the tail batches of predict, src/poplar_kge.cpp:836-839).
// blockIdx.z picks the feature network (head / tail) when they are not shared.
// 64x64 output tile, 16-deep k slices, 256 threads with a 4x4 register tile each.
template <class ST, class FT>
__global__ void __launch_bounds__(256)
k_hidden(const uint8_t* __restrict__ table, RowLayout L, const uint32_t* __restrict__ remote,
         uint32_t row_base, int R, const float* __restrict__ W0, const float* __restrict__ W1,
         float* __restrict__ out0, float* __restrict__ out1) {
    grid_dependency_sync();
    constexpr int BM = 64, BN = 64, BK = 16;
    __shared__ __align__(16) float As[BK][BM + 4];
    __shared__ __align__(16) float Bs[BK][BN];
    const float* __restrict__ W = blockIdx.z ? W1 : W0;
    float* __restrict__ out = blockIdx.z ? out1 : out0;
    const int D = L.d, F = L.f;
    const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;

    const int a_row = t >> 2, a_k = (t & 3) * 4;
    const bool a_ok = m0 + a_row < R;
    const FT* __restrict__ a_ptr = nullptr;
    if (a_ok) {
        const size_t row = remote ? remote[m0 + a_row] : row_base + (uint32_t)(m0 + a_row);
        a_ptr = reinterpret_cast<const FT*>(table + row * L.row_bytes + L.off_feat);
    }
    const int b_k = t >> 4, b_n = (t & 15) * 4;
    const bool d_vec = (D & 3) == 0;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < F; k0 += BK) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        const int ka = k0 + a_k;
        if (a_ok) {
            if (ka + 3 < F) {
                a = load4(a_ptr + ka);
            } else {
                if (ka + 0 < F) a.x = load_as_float(a_ptr + ka + 0);
                if (ka + 1 < F) a.y = load_as_float(a_ptr + ka + 1);
                if (ka + 2 < F) a.z = load_as_float(a_ptr + ka + 2);
            }
        }
        float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
        const int kb = k0 + b_k, nb = n0 + b_n;
        if (kb < F) {
            const float* wp = W + (size_t)kb * D + nb;
            if (d_vec && nb + 3 < D) {
                b = load4(wp);
            } else {
                if (nb + 0 < D) b.x = wp[0];
                if (nb + 1 < D) b.y = wp[1];
                if (nb + 2 < D) b.z = wp[2];
                if (nb + 3 < D) b.w = wp[3];
            }
        }
        __syncthreads();
        As[a_k + 0][a_row] = a.x;
        As[a_k + 1][a_row] = a.y;
        As[a_k + 2][a_row] = a.z;
        As[a_k + 3][a_row] = a.w;
        store4(&Bs[b_k][b_n], b);
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 av = load4(&As[kk][ty * 4]);
            const float4 bv = load4(&Bs[kk][tx * 4]);
            const float ar[4] = {av.x, av.y, av.z, av.w};
            const float br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= R) continue;
        const size_t row = remote ? remote[m] : row_base + (uint32_t)m;
        const uint8_t* vp = table + row * L.row_bytes;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < D) out[(size_t)m * D + n] = load_value<ST>(L, vp, n) + acc[i][j];
        }
    }
}

// ---------------------------------------------------------------------------
// Lookups of the hidden table and the send half of the exchange
// (src/poplar_kge.cpp:676-684).  Blocks [0, T) copy hidden_t[a2a[q]] straight into the
// receive buffer of the destination shard (a peer's device memory when that shard lives
// in another process): `send_dst[d]` already points at this shard's slot of shard d's
// buffer.  Blocks [T, T+B) form the predicted tail h (+|*|complex*) r into `pred`.
template <int V>
__global__ void __launch_bounds__(64)
k_route(const float* __restrict__ hid_h, const float* __restrict__ hid_t,
        const uint32_t* __restrict__ a2a_idx, const uint32_t* __restrict__ head,
        const uint32_t* __restrict__ relation, const float* __restrict__ rel_table,
        float* const* __restrict__ send_dst, float* __restrict__ pred, int T, int a2a, int B, int D,
        int score_fn, ExchangeSync sync, float* const* __restrict__ send_lo_dst = nullptr, float* __restrict__ pred_lo = nullptr,
        int lo_bf16 = 0) {
    grid_dependency_sync();
    const int b = blockIdx.x;
    if (b < T) {
        const int dst = b / a2a, j = b - dst * a2a;
        const float* __restrict__ src = hid_t + (size_t)a2a_idx[b] * D;
        float* __restrict__ out = send_dst[dst] + (size_t)j * D;
        if (V == 4) {
            for (int c = threadIdx.x * 4; c < D; c += blockDim.x * 4) {
                const float4 v = load4(src + c);
                store4(out + c, v);
                if (send_lo_dst) {  // the companion plane of the tensor-core operands: lower TF32 part, or the bf16 rounding
                    if (lo_bf16) store4(reinterpret_cast<__nv_bfloat16*>(send_lo_dst[dst]) + (size_t)j * D + c, v);
                    else store4(send_lo_dst[dst] + (size_t)j * D + c, tf32_lower4(v));
                }
            }
        } else {
            for (int c = threadIdx.x; c < D; c += blockDim.x) out[c] = src[c];
        }
        exchange_signal(sync, XCHG_TAILS, gridDim.x);  // the tail rows are in their consumers' memory
        return;
    }
    const int i = b - T;
    if (i >= B) {
        exchange_signal(sync, XCHG_TAILS, gridDim.x);
        return;
    }
    const float* __restrict__ h = hid_h + (size_t)head[i] * D;
    const float* __restrict__ r = rel_table + (size_t)relation[i] * D;
    float* __restrict__ p = pred + (size_t)i * D;
    if (score_fn == SCORE_COMPLEX || score_fn == SCORE_ROTATE) {
        const int half = D / 2;
        for (int c = threadIdx.x; c < half; c += blockDim.x) {
            const float hr = h[c], hi = h[c + half];
            float rr, ri;  // the relation as a complex number: stored (ComplEx) or the unit rotation by the stored angle (RotatE)
            if (score_fn == SCORE_ROTATE) rotate_sin_cos(r[c], ri, rr);
            else { rr = r[c]; ri = r[c + half]; }
            p[c] = hr * rr - hi * ri;
            p[c + half] = hr * ri + hi * rr;
            if (pred_lo && lo_bf16) {
                __nv_bfloat16* p16 = reinterpret_cast<__nv_bfloat16*>(pred_lo) + (size_t)i * D;
                p16[c] = __float2bfloat16_rn(p[c]);
                p16[c + half] = __float2bfloat16_rn(p[c + half]);
            } else if (pred_lo) {
                pred_lo[(size_t)i * D + c] = tf32_lower(p[c]);
                pred_lo[(size_t)i * D + c + half] = tf32_lower(p[c + half]);
            }
        }
    } else if (V == 4) {
        for (int c = threadIdx.x * 4; c < D; c += blockDim.x * 4) {
            const float4 a = load4(h + c), q = load4(r + c);
            float4 o;
            if (score_fn == SCORE_TRANSE) {
                o = make_float4(a.x + q.x, a.y + q.y, a.z + q.z, a.w + q.w);
            } else {
                o = make_float4(a.x * q.x, a.y * q.y, a.z * q.z, a.w * q.w);
            }
            store4(p + c, o);
            if (pred_lo && lo_bf16) store4(reinterpret_cast<__nv_bfloat16*>(pred_lo) + (size_t)i * D + c, o);
            else if (pred_lo) store4(pred_lo + (size_t)i * D + c, tf32_lower4(o));
        }
    } else {
        for (int c = threadIdx.x; c < D; c += blockDim.x)
            p[c] = score_fn == SCORE_TRANSE ? h[c] + r[c] : h[c] * r[c];
    }
    exchange_signal(sync, XCHG_TAILS, gridDim.x);
}

// The lookups of the rows with many lookups (the parts k_prepare_segments cut them into for the
// entity update): block p copies hidden row parts[p].x to the lookups perm[parts[p].y .. parts[p].z),
// heads (+ or * their relation row) into `pred`, tails into the owning shards' buffers, each with
// its companion plane.  The hidden kernel's routing epilogue leaves these rows out, so that no
// single block stores hundreds of copies of one row; this kernel then publishes the tails hand-over.
// TransE and DistMult (the score functions whose routing is fused).
static __global__ void __launch_bounds__(256)
k_route_heavy(const float* __restrict__ hid_h, const float* __restrict__ hid_t, const uint4* __restrict__ parts,
              const uint32_t* __restrict__ count, const uint32_t* __restrict__ perm, const uint32_t* __restrict__ relation,
              const float* __restrict__ rel_table, float* const* __restrict__ send_dst, float* const* __restrict__ send_lo_dst,
              float* __restrict__ pred, float* __restrict__ pred_lo, int B, int a2a, int D, int score_fn, int lo_bf16, ExchangeSync sync) {
    grid_dependency_sync();
    if (blockIdx.x < *count) {
        // every (lookup, 4 columns) pair is one unit of work: all of a part's copies are in flight at once
        const uint4 part = parts[blockIdx.x];
        const int quads = D / 4, n_units = (int)(part.z - part.y) * quads;
        for (int u = threadIdx.x; u < n_units; u += blockDim.x) {
            const uint32_t q = part.y + (uint32_t)(u / quads), e = perm[q];
            const int c = (u % quads) * 4;
            const bool head = e < (uint32_t)B;
            float4 o = load4((head ? hid_h : hid_t) + (size_t)part.x * D + c);
            float *dst, *dst_lo;
            if (head) {
                const float4 r = load4(rel_table + (size_t)relation[e] * D + c);
                o = score_fn == SCORE_TRANSE ? make_float4(o.x + r.x, o.y + r.y, o.z + r.z, o.w + r.w)
                                             : make_float4(o.x * r.x, o.y * r.y, o.z * r.z, o.w * r.w);
                dst = pred + (size_t)e * D;
                dst_lo = lo_bf16 ? pred_lo + (size_t)e * D / 2 : pred_lo + (size_t)e * D;
            } else {
                const uint32_t j = e - (uint32_t)B, shard = j / (uint32_t)a2a, slot = j - shard * (uint32_t)a2a;
                dst = send_dst[shard] + (size_t)slot * D;
                dst_lo = lo_bf16 ? send_lo_dst[shard] + (size_t)slot * D / 2 : send_lo_dst[shard] + (size_t)slot * D;
            }
            store4(dst + c, o);
            if (lo_bf16) store4(reinterpret_cast<__nv_bfloat16*>(dst_lo) + c, o);
            else store4(dst_lo + c, tf32_lower4(o));
        }
    }
    exchange_signal(sync, XCHG_TAILS, gridDim.x);  // the tail rows are in their consumers' memory
}

// ---------------------------------------------------------------------------
// raw[i, j] = sum_k |p_ik - t_jk|  (L1),  sqrt(sum_k (p_ik - t_jk)^2)  (L2),  sum_k p_ik t_jk (dot)
// src/poplar_extensions/distance.cpp:70-104,151-185 and the codelets' l1dist / l2dist;
// the dot form is matMul(a, b^T) of src/poplar_kge.cpp:478-479.
// 32x64 output tile, 32-deep k slices staged in shared memory k-major, 128 threads, 4x4 each.
template <int FN>
__global__ void __launch_bounds__(128)
k_score(const float* __restrict__ P, const float* __restrict__ Tl, float* __restrict__ raw, int B,
        int T, int D) {
    grid_dependency_sync();
    constexpr int BM = 32, BN = 64, BK = 32;
    __shared__ __align__(16) float Ps[BK][BM];
    __shared__ __align__(16) float Ts[BK][BN];
    const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
    const int i0 = blockIdx.y * BM, j0 = blockIdx.x * BN;
    const bool vec = (D & 3) == 0;
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;

    for (int k0 = 0; k0 < D; k0 += BK) {
        __syncthreads();
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const int idx = t + it * 128, row = idx & 31, k4 = (idx >> 5) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            const int gi = i0 + row, gk = k0 + k4;
            if (gi < B) {
                const float* src = P + (size_t)gi * D + gk;
                if (vec && gk + 3 < D) {
                    v = load4(src);
                } else {
                    if (gk + 0 < D) v.x = src[0];
                    if (gk + 1 < D) v.y = src[1];
                    if (gk + 2 < D) v.z = src[2];
                    if (gk + 3 < D) v.w = src[3];
                }
            }
            Ps[k4 + 0][row] = v.x;
            Ps[k4 + 1][row] = v.y;
            Ps[k4 + 2][row] = v.z;
            Ps[k4 + 3][row] = v.w;
        }
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int idx = t + it * 128, row = idx & 63, k4 = (idx >> 6) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            const int gj = j0 + row, gk = k0 + k4;
            if (gj < T) {
                const float* src = Tl + (size_t)gj * D + gk;
                if (vec && gk + 3 < D) {
                    v = load4(src);
                } else {
                    if (gk + 0 < D) v.x = src[0];
                    if (gk + 1 < D) v.y = src[1];
                    if (gk + 2 < D) v.z = src[2];
                    if (gk + 3 < D) v.w = src[3];
                }
            }
            Ts[k4 + 0][row] = v.x;
            Ts[k4 + 1][row] = v.y;
            Ts[k4 + 2][row] = v.z;
            Ts[k4 + 3][row] = v.w;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < BK; ++kk) {
            const float4 pv = load4(&Ps[kk][ty * 4]);
            const float4 tv = load4(&Ts[kk][tx * 4]);
            const float pr[4] = {pv.x, pv.y, pv.z, pv.w};
            const float tr[4] = {tv.x, tv.y, tv.z, tv.w};
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    if (FN == DIST_L1) {
                        acc[a][b] += fabsf(pr[a] - tr[b]);
                    } else if (FN == DIST_L2) {
                        const float d = pr[a] - tr[b];
                        acc[a][b] = fmaf(d, d, acc[a][b]);
                    } else {
                        acc[a][b] = fmaf(pr[a], tr[b], acc[a][b]);
                    }
                }
        }
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int i = i0 + ty * 4 + a;
        if (i >= B) continue;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int j = j0 + tx * 4 + b;
            if (j < T) raw[(size_t)i * T + j] = FN == DIST_L2 ? sqrtf(acc[a][b]) : acc[a][b];
        }
    }
}

// The same scores for rows that allow 16-byte copies (D a multiple of 4, 16-byte aligned bases).
// A block owns a 32x32 tile of outputs and its 8 warps divide the k range in chunks of 32: warp w
// copies its own 32x32 chunk of both operands into its private part of shared memory (asynchronous
// 16-byte copies, row-major with a stride of 36 floats, which keeps the 128-bit reads below free of
// bank conflicts), accumulates a 4x8 register tile per lane over the chunk, and the 8 partial tiles
// are added through shared memory at the end.  Splitting k, not the tile, is what gives every SM
// several warps of independent work on a problem of only B x T = 512 x 768 outputs.
constexpr int kScoreStride = 36;
constexpr int kScoreWarps = 8;
constexpr size_t kScoreWideSmem = (size_t)kScoreWarps * 2 * 32 * kScoreStride * sizeof(float);

__device__ __forceinline__ void score_copy16(float* dst_smem, const float* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst_smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src));
}

template <int FN>
__global__ void __launch_bounds__(32 * kScoreWarps, 3)
k_score_wide(const float* __restrict__ P, const float* __restrict__ Tl, float* __restrict__ raw, int B,
             int T, int D, ExchangeSync sync) {
    grid_dependency_sync();
    exchange_wait(sync, XCHG_TAILS);  // the tail rows come from the other processes
    extern __shared__ __align__(16) float score_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int i0 = blockIdx.y * 32, j0 = blockIdx.x * 32;
    float* Ps = score_smem + (size_t)warp * 2 * 32 * kScoreStride;
    float* Ts = Ps + 32 * kScoreStride;
    const int ty = lane >> 2, tx = lane & 3;  // p rows ty + 8a, t rows tx + 4b
    const int n_chunks = (D + 31) / 32;
    float acc[4][8];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b) acc[a][b] = 0.f;

    for (int chunk = warp; chunk < n_chunks; chunk += kScoreWarps) {
        const int k0 = chunk * 32;
        __syncwarp();
#pragma unroll 2
        for (int it = 0; it < 8; ++it) {
            const int row = it * 4 + (lane >> 3), k4 = (lane & 7) * 4;
            float* pd = Ps + row * kScoreStride + k4;
            float* td = Ts + row * kScoreStride + k4;
            if (i0 + row < B && k0 + k4 < D) score_copy16(pd, P + (size_t)(i0 + row) * D + k0 + k4);
            else *reinterpret_cast<float4*>(pd) = make_float4(0.f, 0.f, 0.f, 0.f);
            if (j0 + row < T && k0 + k4 < D) score_copy16(td, Tl + (size_t)(j0 + row) * D + k0 + k4);
            else *reinterpret_cast<float4*>(td) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncwarp();
#pragma unroll 1
        for (int k4 = 0; k4 < 32; k4 += 4) {
            float4 pv[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) pv[a] = load4(Ps + (ty + 8 * a) * kScoreStride + k4);
#pragma unroll
            for (int half = 0; half < 4; ++half) {
                float4 tv[2];
#pragma unroll
                for (int b = 0; b < 2; ++b) tv[b] = load4(Ts + (tx + 4 * (half * 2 + b)) * kScoreStride + k4);
#pragma unroll
                for (int a = 0; a < 4; ++a)
#pragma unroll
                    for (int b = 0; b < 2; ++b) {
                        const float pr[4] = {pv[a].x, pv[a].y, pv[a].z, pv[a].w};
                        const float tr[4] = {tv[b].x, tv[b].y, tv[b].z, tv[b].w};
                        float& sum = acc[a][half * 2 + b];
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            if (FN == DIST_L1) {
                                sum += fabsf(pr[c] - tr[c]);
                            } else if (FN == DIST_L2) {
                                const float d = pr[c] - tr[c];
                                sum = fmaf(d, d, sum);
                            } else {
                                sum = fmaf(pr[c], tr[c], sum);
                            }
                        }
                    }
            }
        }
    }
    // add the warps' partial tiles: red[warp][p row][t row], stride 33
    __syncthreads();
    float* red = score_smem;
    const int n_active = n_chunks < kScoreWarps ? n_chunks : kScoreWarps;
    if (warp < n_active) {
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 8; ++b) red[(warp * 32 + ty + 8 * a) * 33 + tx + 4 * b] = acc[a][b];
    }
    __syncthreads();
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int o = threadIdx.x + it * 32 * kScoreWarps, prow = o >> 5, trow = o & 31;
        float sum = 0.f;
        for (int w = 0; w < n_active; ++w) sum += red[(w * 32 + prow) * 33 + trow];
        const int i = i0 + prow, j = j0 + trow;
        if (i < B && j < T) raw[(size_t)i * T + j] = FN == DIST_L2 ? sqrtf(sum) : sum;
    }
}

// Picks the kernel: the 16-byte-copy form when the rows allow it, the general form otherwise.
// `sync` with world > 1: the kernel waits for the tail rows of the other processes (only the
// 16-byte-copy form can; returns cudaErrorNotSupported otherwise so that the caller waits first).
template <int FN>
inline cudaError_t launch_score(const float* P, const float* Tl, float* raw, int B, int T, int D, cudaStream_t stream,
                                const ExchangeSync& sync = ExchangeSync{}) {
    const bool aligned = (D % 4) == 0 && reinterpret_cast<uintptr_t>(P) % 16 == 0 && reinterpret_cast<uintptr_t>(Tl) % 16 == 0;
    if (!aligned) {
        if (sync.world > 1) return cudaErrorNotSupported;
        return launch_dependent(k_score<FN>, dim3((T + 63) / 64, (B + 31) / 32), dim3(128), 0, stream, P, Tl, raw, B, T, D);
    }
    static bool configured[kMaxDeviceOrdinals] = {};  // one attribute call per instantiation and device is enough
    const int slot = current_device_slot();
    if (slot < 0 || !configured[slot]) {
        cudaError_t err = cudaFuncSetAttribute(k_score_wide<FN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kScoreWideSmem);
        if (err != cudaSuccess) return err;
        if (slot >= 0) configured[slot] = true;
    }
    return launch_dependent(k_score_wide<FN>, dim3((T + 31) / 32, (B + 31) / 32), dim3(32 * kScoreWarps), kScoreWideSmem, stream,
                            P, Tl, raw, B, T, D, sync);
}

inline bool score_rows_aligned(const float* P, const float* Tl, int D) {
    return (D % 4) == 0 && reinterpret_cast<uintptr_t>(P) % 16 == 0 && reinterpret_cast<uintptr_t>(Tl) % 16 == 0;
}

inline cudaError_t launch_score(int dist_fn, const float* P, const float* Tl, float* raw, int B, int T, int D, cudaStream_t stream,
                                const ExchangeSync& sync = ExchangeSync{}) {
    switch (dist_fn) {
        case DIST_L1: return launch_score<DIST_L1>(P, Tl, raw, B, T, D, stream, sync);
        case DIST_L2: return launch_score<DIST_L2>(P, Tl, raw, B, T, D, stream, sync);
        default: return launch_score<DIST_DOT>(P, Tl, raw, B, T, D, stream, sync);
    }
}

// ---------------------------------------------------------------------------
// Loss forward and backward for one row of scores per block
// (src/poplar_kge.cpp:615-660; guarded log-sigmoid src/pag/pag.cpp:888-910; log-softmax
// backward :851-860).  Reads raw distances / dot products, writes
//   loss_rows[i] = the row's un-normalised loss term, and
//   coeff[i, j]  = loss_scale * dloss/draw_ij, already divided by the distance for L2
//                  (0 where the distance is 0: l2distance.codelet.cpp:149-158),
// which is the only thing the score backward needs.
struct LossParams {
    int loss_fn;
    int score_fn;
    int dist_fn;
    int n_tail;
    float gamma;
    float softmax_shift;     // correction_weight * (log(n_entity*n_shard-1) - log(n_tail-1)), or 0
    float adversarial_scale; // 0 = off
    float w_pos, w_neg;      // log-sigmoid weights of the label / of the other columns
    float grad_scale;        // loss_scale / normaliser
};

// After its row, the block that finishes last adds the rows' loss terms in row order (a fixed
// tree: the result does not depend on which block that is) and adds the step's loss to the running
// total of the program run (src/poplar_kge.cpp:735-736).
// `extra` (may be null): a term of the step's loss that another kernel has already summed (the regularisers).
template <int THREADS>
__device__ __forceinline__ void finish_step_loss(const float* loss_rows, int B, float inv_normaliser, float* loss_total,
                                                 float* loss_last, unsigned* counter, float* scratch, const float* extra) {
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(counter, 1u) + 1u == gridDim.x ? 1 : 0;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    float part = 0.f;
    for (int i = threadIdx.x; i < B; i += THREADS) part += __ldcg(loss_rows + i);
    part = block_sum<THREADS>(part, scratch);
    if (threadIdx.x == 0) {
        const float step_loss = part * inv_normaliser + (extra ? *extra : 0.f);
        *loss_total += step_loss;
        *loss_last = step_loss;
        *counter = 0u;
    }
}

template <int THREADS>
__global__ void __launch_bounds__(THREADS)
k_loss(const float* __restrict__ raw, const uint32_t* __restrict__ label, float* __restrict__ coeff,
       float* __restrict__ loss_rows, LossParams lp, float inv_normaliser, float* __restrict__ loss_total,
       float* __restrict__ loss_last, unsigned* __restrict__ counter, float* __restrict__ coeff_lo, int lo_bf16,
       const float* __restrict__ extra_loss) {
    grid_dependency_sync();
    __shared__ float scratch[THREADS / 32];
    const int i = blockIdx.x, T = lp.n_tail;
    const float* __restrict__ r = raw + (size_t)i * T;
    float* __restrict__ c = coeff + (size_t)i * T;
    // the companion plane for the tensor-core gradients: lower TF32 part, or the bf16 rounding (rows of T bf16)
    float* __restrict__ c_lo = coeff_lo && !lo_bf16 ? coeff_lo + (size_t)i * T : nullptr;
    __nv_bfloat16* __restrict__ c16 = coeff_lo && lo_bf16 ? reinterpret_cast<__nv_bfloat16*>(coeff_lo) + (size_t)i * T : nullptr;
    const int lab = (int)label[i];
    const bool transe = score_is_gamma_minus_distance(lp.score_fn);
    auto score_of = [&](int j) { return transe ? lp.gamma - r[j] : r[j]; };
    auto to_coeff = [&](int j, float g_score) {
        float g = transe ? -g_score : g_score;  // d score / d raw
        if (lp.dist_fn == DIST_L2) {
            const float dist = r[j];
            g = dist == 0.f ? 0.f : g / dist;
        }
        return g;
    };
    if (lp.loss_fn == LOSS_SOFTMAX) {
        float mx = -INFINITY;
        for (int j = threadIdx.x; j < T; j += THREADS)
            mx = fmaxf(mx, score_of(j) + (j == lab ? 0.f : lp.softmax_shift));
        mx = block_max<THREADS>(mx, scratch);
        float sum = 0.f;
        for (int j = threadIdx.x; j < T; j += THREADS)
            sum += expf(score_of(j) + (j == lab ? 0.f : lp.softmax_shift) - mx);
        sum = block_sum<THREADS>(sum, scratch);
        const float log_z = logf(sum);
        for (int j = threadIdx.x; j < T; j += THREADS) {
            const float logp = score_of(j) + (j == lab ? 0.f : lp.softmax_shift) - mx - log_z;
            const float g = lp.grad_scale * (expf(logp) - (j == lab ? 1.f : 0.f));
            const float cj = to_coeff(j, g);
            c[j] = cj;
            if (c_lo) c_lo[j] = tf32_lower(cj);
            if (c16) c16[j] = __float2bfloat16_rn(cj);
            if (j == lab) loss_rows[i] = -logp;
        }
        if (loss_total) finish_step_loss<THREADS>(loss_rows, (int)gridDim.x, inv_normaliser, loss_total, loss_last, counter, scratch, extra_loss);
        return;
    }
    // log-sigmoid, optionally with self-adversarial weights from a detached softmax
    float adv_max = 0.f, adv_sum = 1.f;
    const bool adv = lp.adversarial_scale > 0.f;
    if (adv) {
        float mx = -INFINITY;
        for (int j = threadIdx.x; j < T; j += THREADS)
            mx = fmaxf(mx, lp.adversarial_scale * score_of(j) + (j == lab ? -10000.f : 0.f));
        adv_max = block_max<THREADS>(mx, scratch);
        float sum = 0.f;
        for (int j = threadIdx.x; j < T; j += THREADS)
            sum += expf(lp.adversarial_scale * score_of(j) + (j == lab ? -10000.f : 0.f) - adv_max);
        adv_sum = block_sum<THREADS>(sum, scratch);
    }
    float part = 0.f;
    for (int j = threadIdx.x; j < T; j += THREADS) {
        const float s = score_of(j);
        const bool pos = j == lab;
        float w = pos ? lp.w_pos : lp.w_neg;
        if (adv) {
            const float soft =
                expf(lp.adversarial_scale * s + (pos ? -10000.f : 0.f) - adv_max) / adv_sum;
            w *= (pos ? 1.f : 0.f) + (float)(T - 1) * soft;
        }
        const float x = pos ? s : -s;
        const float ls = x > -11.f ? -log1pf(expf(-fmaxf(x, -11.f))) : x;
        part += w * ls;
        const float dx = (-w * lp.grad_scale) / (1.f + expf(fminf(x, 11.f)));
        const float cj = to_coeff(j, pos ? dx : -dx);
        c[j] = cj;
        if (c_lo) c_lo[j] = tf32_lower(cj);
        if (c16) c16[j] = __float2bfloat16_rn(cj);
    }
    part = block_sum<THREADS>(part, scratch);
    if (threadIdx.x == 0) loss_rows[i] = -part;
    // (null loss_total: a later kernel of the step adds the rows' terms, off the step's critical chain)
    if (loss_total) finish_step_loss<THREADS>(loss_rows, (int)gridDim.x, inv_normaliser, loss_total, loss_last, counter, scratch, extra_loss);
}

inline cudaError_t launch_loss(const float* raw, const uint32_t* label, float* coeff, float* loss_rows, const LossParams& lp, float inv_normaliser,
                               float* loss_total, float* loss_last, unsigned* counter, float* coeff_lo, int lo_bf16, int B, cudaStream_t stream,
                               const float* extra_loss = nullptr) {
    // One block per row keeps about 130 thousand threads in flight for the metric's 512 x 768 scores; a warp
    // per row (a sixth as many threads, each with a serial chain of exponentials) measured 4 us slower.
    return launch_dependent(k_loss<256>, dim3((unsigned)B), dim3(256), 0, stream, raw, label, coeff, loss_rows, lp, inv_normaliser, loss_total,
                            loss_last, counter, coeff_lo, lo_bf16, extra_loss);
}

// ---------------------------------------------------------------------------
// Score backward: out[m, k] = sum_n C(m, n) * f(x[m, k], y[n, k]) with
//   f = sign(x - y)  (L1, sign(0) = 0: l1distance.codelet.cpp:76-79,138-145)
//   f = x - y        (L2; C already holds grad / dist)
//   f = y            (dot: src/pag/pag.cpp:685-701)
// Problem 0 is the gradient of the predicted tails (x = pred, y = tails, C = coeff);
// problem 1 the gradient of the tails (x = tails, y = pred, C = coeff transposed), whose
// rows go straight to the shard that owns them: the return half of the exchange
// (src/pag/pag.cpp:925-932).  32 rows x 64 columns per block, n in slices of 32.
struct PairBwdProblem {
    const float* X;
    const float* Y;
    const float* C;
    int M, N;
    int c_stride_m, c_stride_n;
    float* out;               // [M, D] when out_blocks is null
    float* const* out_blocks; // per block of `block_rows` rows, the base pointer of that block
    int block_rows;
};
struct PairBwdArgs {
    PairBwdProblem p[2];
    int D;
    int tiles_m0;
};

template <int FN>
__global__ void __launch_bounds__(128) k_pair_bwd(PairBwdArgs args) {
    grid_dependency_sync();
    constexpr int BM = 32, BD = 64, BN = 32;
    __shared__ float Cs[BM][BN + 1];
    __shared__ __align__(16) float Ys[BN][BD];
    const int which = (int)blockIdx.x >= args.tiles_m0 ? 1 : 0;
    const PairBwdProblem& pr = args.p[which];
    const int D = args.D;
    const int m0 = ((int)blockIdx.x - (which ? args.tiles_m0 : 0)) * BM, d0 = blockIdx.y * BD;
    const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
    const bool vec = (D & 3) == 0;

    float x[4][4], acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int m = m0 + ty * 4 + a;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int k = d0 + tx * 4 + b;
            x[a][b] = (m < pr.M && k < D) ? pr.X[(size_t)m * D + k] : 0.f;
            acc[a][b] = 0.f;
        }
    }
    const bool n_fast = pr.c_stride_n == 1;
    for (int n0 = 0; n0 < pr.N; n0 += BN) {
        __syncthreads();
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int idx = t + it * 128;
            const int m = n_fast ? (idx >> 5) : (idx & 31);
            const int n = n_fast ? (idx & 31) : (idx >> 5);
            const int gm = m0 + m, gn = n0 + n;
            float v = 0.f;
            if (gm < pr.M && gn < pr.N)
                v = pr.C[(size_t)gm * pr.c_stride_m + (size_t)gn * pr.c_stride_n];
            Cs[m][n] = v;
        }
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int idx = t + it * 128, k4 = (idx & 15) * 4, n = idx >> 4;
            const int gn = n0 + n, gk = d0 + k4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (gn < pr.N) {
                const float* src = pr.Y + (size_t)gn * D + gk;
                if (vec && gk + 3 < D) {
                    v = load4(src);
                } else {
                    if (gk + 0 < D) v.x = src[0];
                    if (gk + 1 < D) v.y = src[1];
                    if (gk + 2 < D) v.z = src[2];
                    if (gk + 3 < D) v.w = src[3];
                }
            }
            store4(&Ys[n][k4], v);
        }
        __syncthreads();
#pragma unroll 4
        for (int nn = 0; nn < BN; ++nn) {
            const float4 yv = load4(&Ys[nn][tx * 4]);
            const float yr[4] = {yv.x, yv.y, yv.z, yv.w};
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const float c = Cs[ty * 4 + a][nn];
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    if (FN == DIST_L1) {
                        const float d = x[a][b] - yr[b];
                        acc[a][b] += d > 0.f ? c : (d < 0.f ? -c : 0.f);
                    } else if (FN == DIST_L2) {
                        acc[a][b] = fmaf(c, x[a][b] - yr[b], acc[a][b]);
                    } else {
                        acc[a][b] = fmaf(c, yr[b], acc[a][b]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int m = m0 + ty * 4 + a;
        if (m >= pr.M) continue;
        float* dst;
        if (pr.out_blocks) {
            const int blk = m / pr.block_rows;
            dst = pr.out_blocks[blk] + (size_t)(m - blk * pr.block_rows) * D;
        } else {
            dst = pr.out + (size_t)m * D;
        }
        const int k = d0 + tx * 4;
        if (vec && k + 3 < D) {
            store4(dst + k, make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]));
        } else {
#pragma unroll
            for (int b = 0; b < 4; ++b)
                if (k + b < D) dst[k + b] = acc[a][b];
        }
    }
}

// Gradients of the head vector and of the relation row for the multiplicative score
// functions (backward of src/poplar_kge.cpp:501-510, 567-569).  TransE needs no kernel:
// both gradients equal d_pred.
static __global__ void __launch_bounds__(64)
k_pred_bwd(const float* __restrict__ d_pred, const float* __restrict__ hid_h,
           const uint32_t* __restrict__ head, const uint32_t* __restrict__ relation,
           const float* __restrict__ rel_table, float* __restrict__ d_head,
           float* __restrict__ d_relrow, int D, int score_fn) {
    grid_dependency_sync();
    const int i = blockIdx.x;
    const float* __restrict__ dp = d_pred + (size_t)i * D;
    const float* __restrict__ h = hid_h + (size_t)head[i] * D;
    const float* __restrict__ r = rel_table + (size_t)relation[i] * D;
    float* __restrict__ dh = d_head + (size_t)i * D;
    float* __restrict__ dr = d_relrow + (size_t)i * D;
    if (score_fn == SCORE_DISTMULT) {
        for (int c = threadIdx.x; c < D; c += blockDim.x) {
            dh[c] = dp[c] * r[c];
            dr[c] = dp[c] * h[c];
        }
    } else if (score_fn == SCORE_ROTATE) {
        // Backward of src/poplar_kge.cpp:516-530.  The gradients of sine and cosine pass back through
        // the float16 casts and the float16 sin / cos (src/pag/pag.cpp:552-595, 619-633): rounded to
        // float16 at each of those points, the angle's gradient is their float16 sum.
        const int half = D / 2;
        for (int c = threadIdx.x; c < half; c += blockDim.x) {
            const float hr = h[c], hi = h[c + half];
            float s, co;
            rotate_sin_cos(r[c], s, co);
            const float gr = dp[c], gi = dp[c + half];
            dh[c] = gr * co + gi * s;
            dh[c + half] = -gr * s + gi * co;
            const float d_sin = round_to_half(-gr * hi + gi * hr), d_cos = round_to_half(gr * hr + gi * hi);
            const float via_sin = round_to_half(d_sin * co), via_cos = round_to_half(-d_cos * s);
            dr[c] = round_to_half(via_sin + via_cos);
            dr[c + half] = 0.f;  // the table keeps rows of D floats; the upper half of an angle row is unused
        }
    } else {
        const int half = D / 2;
        for (int c = threadIdx.x; c < half; c += blockDim.x) {
            const float hr = h[c], hi = h[c + half], rr = r[c], ri = r[c + half];
            const float gr = dp[c], gi = dp[c + half];
            dh[c] = gr * rr + gi * ri;
            dh[c + half] = -gr * ri + gi * rr;
            dr[c] = gr * hr + gi * hi;
            dr[c + half] = -gr * hi + gi * hr;
        }
    }
}

// ---------------------------------------------------------------------------
// Sort-and-segment preparation, once per staged step and shard: orders the B head
// lookups and the T tail lookups by the hidden row they read (ties by position, so the
// order is unique) and records where each row's segment starts; the same for the B
// relation lookups.  The scatter-add of src/pag/pag.cpp:721-743 then becomes one
// sequential sum per row in a fixed order: no float atomics.
// One block per (shard-step); bitonic sort of (row << 32 | position) keys in shared memory.
constexpr int kMaxSortItems = 4096;

__device__ __forceinline__ void bitonic_sort(unsigned long long* keys, int padded) {
    for (int k = 2; k <= padded; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            __syncthreads();
            for (int i = threadIdx.x; i < padded; i += blockDim.x) {
                const int ixj = i ^ j;
                if (ixj > i) {
                    const unsigned long long a = keys[i], b = keys[ixj];
                    const bool ascending = (i & k) == 0;
                    if ((a > b) == ascending) {
                        keys[i] = b;
                        keys[ixj] = a;
                    }
                }
            }
        }
    }
    __syncthreads();
}

__device__ __forceinline__ int lower_bound_key(const unsigned long long* keys, int n,
                                                unsigned long long target) {
    int lo = 0, hi = n;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (keys[mid] < target) lo = mid + 1; else hi = mid;
    }
    return lo;
}

// Rows with more than kHeavyMin lookups are cut into parts of kHeavyPart lookups, at most kHeavySlots
// parts per shard and step (see k_entity_update).
constexpr int kHeavySlots = 112;
constexpr int kHeavyMin = 12;
constexpr int kHeavyPart = 16;

static __global__ void __launch_bounds__(512)
k_prepare_segments(const uint32_t* __restrict__ head, const uint32_t* __restrict__ a2a_idx,
                   const uint32_t* __restrict__ relation, const uint32_t* __restrict__ remote, int B,
                   int T, int R, int n_rel, uint32_t* __restrict__ ent_perm,
                   uint32_t* __restrict__ ent_off, uint32_t* __restrict__ rel_perm,
                   uint32_t* __restrict__ rel_off, uint32_t* __restrict__ first_slot,
                   uint4* __restrict__ heavy_parts, uint32_t* __restrict__ heavy_count, uint4* __restrict__ row_info) {
    __shared__ unsigned long long keys[kMaxSortItems];
    const int s = blockIdx.x;
    head += (size_t)s * B;
    relation += (size_t)s * B;
    a2a_idx += (size_t)s * T;
    ent_perm += (size_t)s * (B + T);
    ent_off += (size_t)s * (R + 1);
    rel_perm += (size_t)s * B;
    rel_off += (size_t)s * (n_rel + 1);

    int n = B + T, padded = 1;
    while (padded < n) padded <<= 1;
    for (int i = threadIdx.x; i < padded; i += blockDim.x) {
        unsigned long long key = ~0ull;
        if (i < B) key = ((unsigned long long)head[i] << 32) | (unsigned)i;
        else if (i < n) key = ((unsigned long long)a2a_idx[i - B] << 32) | (unsigned)i;
        keys[i] = key;
    }
    bitonic_sort(keys, padded);
    for (int i = threadIdx.x; i < n; i += blockDim.x) ent_perm[i] = (uint32_t)keys[i];
    for (int r = threadIdx.x; r <= R; r += blockDim.x)
        ent_off[r] = (uint32_t)lower_bound_key(keys, n, (unsigned long long)r << 32);
    __syncthreads();

    if (rel_perm) {  // null: the caller has no relation lookups (the operator form of the scatter-add)
        n = B;
        padded = 1;
        while (padded < n) padded <<= 1;
        for (int i = threadIdx.x; i < padded; i += blockDim.x)
            keys[i] = i < n ? (((unsigned long long)relation[i] << 32) | (unsigned)i) : ~0ull;
        bitonic_sort(keys, padded);
        for (int i = threadIdx.x; i < n; i += blockDim.x) rel_perm[i] = (uint32_t)keys[i];
        for (int r = threadIdx.x; r <= n_rel; r += blockDim.x)
            rel_off[r] = (uint32_t)lower_bound_key(keys, n, (unsigned long long)r << 32);
    }
    if (!remote) return;
    __syncthreads();

    // Which gathered slot is the first to name its table row: only that slot writes the row
    // back.  `remote` is unique apart from the zero padding at its end, whose slots all name
    // row 0; the reference computes every slot from the same gathered copy, so its duplicate
    // writes are identical, and one write reproduces them.
    remote += (size_t)s * R;
    first_slot += (size_t)s * R;
    n = R;
    padded = 1;
    while (padded < n) padded <<= 1;
    for (int i = threadIdx.x; i < padded; i += blockDim.x)
        keys[i] = i < n ? (((unsigned long long)remote[i] << 32) | (unsigned)i) : ~0ull;
    bitonic_sort(keys, padded);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const bool first = i == 0 || (keys[i - 1] >> 32) != (keys[i] >> 32);
        first_slot[(uint32_t)keys[i]] = first ? 1u : 0u;
    }
    if (heavy_parts) {
    // Rows with many lookups are cut into parts for k_entity_update (bit 1 of first_slot marks them).
    // All threads look for such rows (there are at most (B + T) / kHeavyMin of them); one thread
    // then orders them by row, so that the slots do not depend on the timing, and hands out the parts.
    constexpr int kMaxHeavyRows = 128;
    __shared__ int s_heavy_rows[kMaxHeavyRows];
    __shared__ int s_heavy_n;
    if (threadIdx.x == 0) s_heavy_n = 0;
    __syncthreads();
    for (int r = threadIdx.x; r < R; r += blockDim.x)
        if (ent_off[r + 1] - ent_off[r] > (uint32_t)kHeavyMin) {
            const int i = atomicAdd(&s_heavy_n, 1);
            if (i < kMaxHeavyRows) s_heavy_rows[i] = r;
        }
    __syncthreads();
    if (threadIdx.x == 0) {
        heavy_parts += (size_t)s * kHeavySlots;
        const int n_rows = min(s_heavy_n, kMaxHeavyRows);
        for (int i = 1; i < n_rows; ++i) {  // insertion sort, a handful of entries
            const int r = s_heavy_rows[i];
            int j = i - 1;
            for (; j >= 0 && s_heavy_rows[j] > r; --j) s_heavy_rows[j + 1] = s_heavy_rows[j];
            s_heavy_rows[j + 1] = r;
        }
        int used = 0;
        for (int i = 0; i < n_rows; ++i) {
            const int r = s_heavy_rows[i];
            const uint32_t q0 = ent_off[r], q1 = ent_off[r + 1];
            const int parts = (int)((q1 - q0 + kHeavyPart - 1) / kHeavyPart);
            if (used + parts > kHeavySlots || parts > 255) continue;  // stays with its own block
            for (int p = 0; p < parts; ++p)
                heavy_parts[used + p] = make_uint4((uint32_t)r, q0 + (uint32_t)(p * kHeavyPart),
                                                   min(q1, q0 + (uint32_t)((p + 1) * kHeavyPart)),
                                                   ((uint32_t)used << 16) | ((uint32_t)parts << 8) | (uint32_t)p);
            first_slot[r] |= 2u;
            used += parts;
        }
        heavy_count[s] = (uint32_t)used;
    }
    }
    if (!row_info) return;
    // A row's descriptor for k_entity_update: one sector holds what four scattered loads would fetch.
    __syncthreads();
    row_info += (size_t)s * 2 * R;
    for (int r = threadIdx.x; r < R; r += blockDim.x) {
        const uint32_t q0 = ent_off[r], count = ent_off[r + 1] - q0;
        uint32_t e[4];
        for (int u = 0; u < 4; ++u) e[u] = (uint32_t)u < count ? ent_perm[q0 + u] : 0xffffffffu;
        row_info[2 * r] = make_uint4(q0, count, first_slot[r], remote[r]);
        row_info[2 * r + 1] = make_uint4(e[0], e[1], e[2], e[3]);
    }
}

// ---------------------------------------------------------------------------
// Segment-sum of the lookup gradients into the hidden rows, fused with the row-wise Adam
// update and the write-back (src/pag/pag.cpp:721-743; src/poplar_kge.cpp:695-704;
// src/fructose/frnn.cpp:61-90).  One block per gathered row.  Every gathered row is
// updated, rows with a zero gradient and the padding row included, as in the reference.
// d_hid_h / d_hid_t keep the hidden-row gradients for the projection backward.
//
// Entity popularity is skewed: the shard that holds a step's most popular entity sees one row
// with hundreds of lookups, and a single block would add them sixteen at a time while the rest of
// the GPU idles.  k_prepare_segments therefore cuts every row with more than kHeavyMin lookups
// into parts of kHeavyPart lookups (at most kHeavySlots parts per shard and step).  The first
// kHeavySlots blocks of the grid take one part each, leave its sums in `heavy_partial`, and the
// block that arrives last at the row's counter adds the parts in part order and finishes the
// row; the row's own block skips it.  Nothing waits, and the order of the additions is fixed.
constexpr int kSegmentLanes = 4;  // threads groups that share the lookups of one part of a popular row
constexpr int kRowsPerBlock = 8;  // gathered rows per block of k_entity_update: one warp each

// Dropout of the feature network's output (src/poplar_kge.cpp:459-461; frnn::dropout,
// src/pag/pag.cpp:596-617): an element is kept with probability 1 - p and scaled by 1 / (1 - p);
// the backward passes g / (1 - p) through the kept elements.  (The reference tests output != 0
// instead of the mask; the two differ only where a kept element is exactly zero, which is a row
// without features, whose gradient reaches no parameter.)  The reference draws from the IPU's
// generator; here the mask is a pure function of (seed, training step, shard, call, row, column):
// Philox-4x32-10 keyed by (seed, step), one word per element, kept when word >> 8 is below
// `threshold` = round((1 - p) * 2^24).  Forward and backward recompute it, nothing is stored.
struct DropoutParams {
    uint32_t threshold;        // 0: no dropout
    uint32_t seed;
    const uint32_t* step_key;  // the training step's number, on the device (a graph replays with fixed arguments)
    uint32_t shard;            // global shard index
    float scale;               // 1 / (1 - p)
};

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1);

// Keep bits of columns 4 * col4 .. 4 * col4 + 3 of gathered row r in call `part` (0 head, 1 tail).
__device__ __forceinline__ uint32_t dropout_keep4(const DropoutParams& dp, uint32_t part, uint32_t r, uint32_t col4) {
    uint32_t c[4] = {r, col4, (dp.shard << 1) | part, 0x64726f70u};
    uint32_t k0 = dp.seed, k1 = *dp.step_key;
#pragma unroll
    for (int i = 0; i < 10; ++i) {
        philox_round(c, k0, k1);
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    uint32_t bits = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) bits |= ((c[i] >> 8) < dp.threshold ? 1u : 0u) << i;
    return bits;
}

// hidden = value + dropout(hidden - value), in place on the hidden rows of each call.  With one
// feature network both calls start from the same rows (hid_t_in == hid_h) and get their own masks.
template <class ST>
__global__ void __launch_bounds__(256)
k_dropout_hidden(const uint8_t* __restrict__ rows_c, RowLayout L, float* __restrict__ hid_h, const float* __restrict__ hid_t_in,
                 float* __restrict__ hid_t, int R, DropoutParams dp) {
    grid_dependency_sync();
    const int D = (int)L.d, quads = (D + 3) / 4;
    const int i = (int)(blockIdx.x * blockDim.x + threadIdx.x);
    if (i >= R * quads) return;
    const int r = i / quads, q = i - r * quads;
    const uint8_t* __restrict__ row = rows_c + (size_t)r * L.row_bytes;
    const uint32_t keep_h = dropout_keep4(dp, 0u, (uint32_t)r, (uint32_t)q), keep_t = dropout_keep4(dp, 1u, (uint32_t)r, (uint32_t)q);
    for (int u = 0; u < 4; ++u) {
        const int c = 4 * q + u;
        if (c >= D) break;
        const size_t o = (size_t)r * D + c;
        const float v = load_value<ST>(L, row, c);
        const float fh_h = hid_h[o] - v, fh_t = hid_t_in[o] - v;
        hid_h[o] = (keep_h >> u) & 1u ? v + fh_h * dp.scale : v;
        hid_t[o] = (keep_t >> u) & 1u ? v + fh_t * dp.scale : v;
    }
}

// Norm regularisers of the gathered rows (src/poplar_kge.cpp:430-437, 463-465): each of the two
// entityHidden calls of a step (head part, tail part) adds
//   w_e * sum_r N(value_r) + w_f * sum_r N(feature_hidden_r) + w_h * sum_r N(hidden_r),
// N(a) = (sum_k |a_k^p|)^(1/p) per row (lpnorm, :389-391), over all R gathered rows, to the shard's
// loss, not normalised.  The backward is the reference's tape: pow gives g * p * out / a with 0 where
// a is 0 (src/pag/pag.cpp:493-503), abs gives sign (:449-456), so
//   dN/da_k = N / s * |a_k|^p / a_k   (s = sum_k |a_k|^p; 0 where a_k or s is 0),
// times the weight and the loss scale (the root gradient, :691).  |a|^p stands for |a^p|: the same
// wherever a^p is defined.  The feature network's output is taken as hidden - value.
// One warp per row; writes the three gradient terms k_entity_update adds and the row's loss term;
// the last block adds the rows' terms in row order into *loss_out.
struct RegParams {
    float power[3], weight[3];  // embedding, feature, hidden
    float loss_scale;
    int shared;                 // one feature network: both calls see the same rows
};

__device__ __forceinline__ float abs_pow(float a, float p) {
    a = fabsf(a);
    return p == 2.f ? a * a : (p == 1.f ? a : powf(a, p));
}

__device__ __forceinline__ float warp_sum(float v) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <class ST>
__global__ void __launch_bounds__(256)
k_regularise(const uint8_t* __restrict__ rows_c, RowLayout L, const float* __restrict__ hid_h, const float* __restrict__ hid_t, int R,
             RegParams rp, float* __restrict__ reg_val, float* __restrict__ reg_h, float* __restrict__ reg_t,
             float* __restrict__ loss_rows, float* __restrict__ loss_out, float* __restrict__ loss_sink, unsigned* __restrict__ counter) {
    grid_dependency_sync();
    __shared__ float scratch[8];
    const int lane = threadIdx.x & 31, r = (int)blockIdx.x * 8 + (int)(threadIdx.x >> 5), D = (int)L.d;
    if (r < R) {
        const uint8_t* __restrict__ row = rows_c + (size_t)r * L.row_bytes;
        const float* __restrict__ hid[2] = {hid_h + (size_t)r * D, hid_t + (size_t)r * D};
        float* __restrict__ out[2] = {reg_h + (size_t)r * D, rp.shared ? nullptr : reg_t + (size_t)r * D};
        const int parts = rp.shared ? 1 : 2;
        const float calls = rp.shared ? 2.f : 1.f;  // how many of the two calls a part stands for
        float s_e = 0.f, s_f[2] = {0.f, 0.f}, s_h[2] = {0.f, 0.f};
        for (int c = lane; c < D; c += 32) {
            const float v = load_value<ST>(L, row, c);
            s_e += abs_pow(v, rp.power[0]);
            for (int q = 0; q < parts; ++q) {
                const float h = hid[q][c];
                s_f[q] += abs_pow(h - v, rp.power[1]);
                s_h[q] += abs_pow(h, rp.power[2]);
            }
        }
        // norm and the factor weight * loss_scale * N / s of a row's gradient
        auto norm = [&](float s, int which, float& fac) {
            s = warp_sum(s);
            const float n = s > 0.f ? powf(s, 1.f / rp.power[which]) : 0.f;
            fac = s > 0.f && rp.weight[which] > 0.f ? rp.weight[which] * rp.loss_scale * n / s : 0.f;
            return rp.weight[which] > 0.f ? rp.weight[which] * n : 0.f;
        };
        auto term = [&](float a, int which, float fac) { return a == 0.f || fac == 0.f ? 0.f : fac * abs_pow(a, rp.power[which]) / a; };
        float fac_e, fac_f[2] = {0.f, 0.f}, fac_h[2] = {0.f, 0.f};
        float loss = 2.f * norm(s_e, 0, fac_e);
        for (int q = 0; q < parts; ++q) loss += calls * (norm(s_f[q], 1, fac_f[q]) + norm(s_h[q], 2, fac_h[q]));
        for (int c = lane; c < D; c += 32) {
            const float v = load_value<ST>(L, row, c);
            float gv = 2.f * term(v, 0, fac_e);
            for (int q = 0; q < parts; ++q) {
                const float h = hid[q][c];
                const float g_h = calls * term(h, 2, fac_h[q]);
                gv += g_h;
                out[q][c] = g_h + calls * term(h - v, 1, fac_f[q]);
            }
            reg_val[(size_t)r * D + c] = gv;
        }
        if (lane == 0) loss_rows[r] = loss;
    }
    finish_step_loss<256>(loss_rows, R, 1.f, loss_sink, loss_out, counter, scratch, nullptr);
}

struct HeavyRows {
    const uint4* parts;      // [kHeavySlots] {gathered row, first lookup, end lookup, (first part's slot << 16) | (parts << 8) | part}
    const uint32_t* count;   // parts in use
    float* partial;          // [kHeavySlots][2][D] sums of a part: head lookups | tail lookups
    unsigned* counter;       // [kHeavySlots] parts of a row that have arrived (indexed by the row's first slot)
    // Optional, [R][2]: everything a row's warp needs before it can load gradient rows, in one 32-byte
    // sector: {first lookup's position, lookups, first_slot word, table row} and the row's first four
    // lookups (k_prepare_segments writes it); null: the warp reads off / first_slot / remote / perm.
    const uint4* row_info;
};

// The relation part of a shard's dense gradient, summed by blocks appended to the entity update's
// grid (both depend only on the score gradients): row rho = the sum of the per-triple relation
// gradients of the triples of relation rho, in position order (backward of the gather at
// src/poplar_kge.cpp:489), stored into the memory of the process that owns that row of the dense
// vector (row r to process r % n_owner as its row r / n_owner).  Null d_relrow: no such blocks.
struct RelationRows {
    const float* d_relrow;       // [B, D] per-triple gradients
    const uint32_t* perm;        // triples ordered by relation
    const uint32_t* off;         // [n_rel + 1]
    float* const* dense_dst;     // [n_owner] this shard's slot in each owner's receive buffer
    int n_rel, n_owner;
    float* d_hid_h_lo;           // lower TF32 planes of the hidden-row gradients (null: not needed)
    float* d_hid_t_lo;
    // Gradients of the norm regularisers (k_regularise), [R, D] each, null when all weights are 0:
    // reg_val joins the value's gradient, reg_h / reg_t the gradient of the feature network's output
    // (reg_t null with a shared network, whose reg_h then holds both calls' terms).
    const float* reg_val;
    const float* reg_h;
    const float* reg_t;
    DropoutParams drop;  // threshold 0: none.  Masks the gradients of the feature network's outputs.
    // Non-null: the value's gradient is left here ([R, D]) and the rows are not updated; k_row_adam
    // does that once the rest of the gradient is known (the feature MLP reads the value too).
    float* defer_grad;
    // Non-null (one shard in all: no other shard's gradient to wait for): a relation row's block applies
    // the row's Adam step itself instead of handing its sum to k_dense_update.
    float* rel_w;
    float* rel_m;
    float* rel_v;
    float rel_lr_modifier;
    // Non-null: one more block at the end of the grid adds the step's loss terms (loss_rows [loss_n], left by
    // k_loss) in row order into the run's total: beside the row updates instead of at the end of k_loss.
    const float* loss_rows;
    int loss_n;
    float inv_normaliser;
    float* loss_total;
    float* loss_last;
    const float* extra_loss;
};

template <int V, int LANES>
__device__ __forceinline__ void relation_row_sum(const RelationRows& rr, int rho, int D, float (*part)[64 * V], uint32_t* s_perm,
                                                 const float* __restrict__ step_size, const AdamParams& ap) {
    const int col = threadIdx.x & 63, lane = threadIdx.x >> 6;
    const uint32_t q0 = rr.off[rho], q1 = rr.off[rho + 1];
    // where the row's gradient goes: into its owner's receive buffer, or (one shard in all) straight into the row's Adam step
    auto deliver = [&](int c, float total) {
        if (!rr.rel_w) {
            rr.dense_dst[rho % rr.n_owner][(size_t)(rho / rr.n_owner) * D + c] = total;
            return;
        }
        const size_t e = (size_t)rho * D + c;
        const float alpha = *step_size * rr.rel_lr_modifier;
        const float mo = ap.beta_m * rr.rel_m[e] + ap.one_minus_beta_m * total;
        const float ve = ap.beta_v * rr.rel_v[e] + ap.one_minus_beta_v * total * total;
        const float x = rr.rel_w[e];
        rr.rel_w[e] = x - alpha * (mo / (sqrtf(ve) + ap.epsilon) + ap.weight_decay * x);
        rr.rel_m[e] = mo;
        rr.rel_v[e] = ve;
    };
    // four neighbouring columns at once where the rows allow 16-byte accesses
    auto deliver4 = [&](int c, const float (&total)[4]) {
        if (!rr.rel_w) {
            store4(rr.dense_dst[rho % rr.n_owner] + (size_t)(rho / rr.n_owner) * D + c, make_float4(total[0], total[1], total[2], total[3]));
            return;
        }
        const size_t e = (size_t)rho * D + c;
        const float alpha = *step_size * rr.rel_lr_modifier;
        const float4 m4 = load4(rr.rel_m + e), v4 = load4(rr.rel_v + e), x4 = load4(rr.rel_w + e);
        float mo[4] = {m4.x, m4.y, m4.z, m4.w}, ve[4] = {v4.x, v4.y, v4.z, v4.w}, x[4] = {x4.x, x4.y, x4.z, x4.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            mo[u] = ap.beta_m * mo[u] + ap.one_minus_beta_m * total[u];
            ve[u] = ap.beta_v * ve[u] + ap.one_minus_beta_v * total[u] * total[u];
            x[u] = x[u] - alpha * (mo[u] / (sqrtf(ve[u]) + ap.epsilon) + ap.weight_decay * x[u]);
        }
        store4(rr.rel_w + e, make_float4(x[0], x[1], x[2], x[3]));
        store4(rr.rel_m + e, make_float4(mo[0], mo[1], mo[2], mo[3]));
        store4(rr.rel_v + e, make_float4(ve[0], ve[1], ve[2], ve[3]));
    };
    if (q0 == q1) {
        if (V == 4) {
            const float zero[4] = {0.f, 0.f, 0.f, 0.f};
            for (int c = threadIdx.x * 4; c < D; c += blockDim.x * 4) deliver4(c, zero);
        } else {
            for (int c = threadIdx.x; c < D; c += blockDim.x) deliver(c, 0.f);
        }
        return;
    }
    for (int c0 = 0; c0 < D; c0 += 64 * V) {
        const int c = c0 + col * V;
        float g[V];
#pragma unroll
        for (int u = 0; u < V; ++u) g[u] = 0.f;
        for (uint32_t base = q0; base < q1; base += 64 * LANES) {
            const int count = (int)min((uint32_t)(64 * LANES), q1 - base);
            __syncthreads();
            if ((int)threadIdx.x < count) s_perm[threadIdx.x] = rr.perm[base + threadIdx.x];
            __syncthreads();
            if (c >= D) continue;
            for (int i = lane; i < count; i += 4 * LANES) {
                float4 v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int ii = i + u * LANES;
                    v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (ii < count) {
                        const float* src = rr.d_relrow + (size_t)s_perm[ii] * D + c;
                        if (V == 4) v[u] = load4(src); else v[u].x = src[0];
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (i + u * LANES >= count) continue;
                    g[0] += v[u].x;
                    if (V == 4) { g[1 % V] += v[u].y; g[2 % V] += v[u].z; g[3 % V] += v[u].w; }
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < V; ++u) part[lane][col * V + u] = g[u];
        __syncthreads();
        if (lane == 0 && c < D) {
#pragma unroll
            float totals[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int u = 0; u < V; ++u) {
                float total = part[0][col * V + u];
#pragma unroll
                for (int l = 1; l < LANES; ++l) total += part[l][col * V + u];
                totals[u] = total;
            }
            if (V == 4) {
                deliver4(c, totals);
            } else {
                deliver(c, totals[0]);
            }
        }
    }
}

// EXTRAS: the regularisers' terms, the dropout masks and the deferred row update are compiled in
// (they cost 20 registers, a third of the resident blocks, which the plain step does not pay).
template <class ST, int V, bool EXTRAS = false>
__global__ void __launch_bounds__(64 * kSegmentLanes, EXTRAS ? 2 : 4)
k_entity_update(uint8_t* __restrict__ table, const uint8_t* __restrict__ rows_c, RowLayout L,
                const uint32_t* __restrict__ remote, const uint32_t* __restrict__ perm,
                const uint32_t* __restrict__ off,
                const uint32_t* __restrict__ first_slot, const float* __restrict__ d_head,
                const float* __restrict__ grad_recv, int B,
                float* __restrict__ d_hid_h, float* __restrict__ d_hid_t,
                const float* __restrict__ step_size, float lr_modifier, AdamParams ap, ExchangeSync sync, HeavyRows heavy,
                int R, RelationRows rr) {
    grid_dependency_sync();
    const int row_blocks = (R + kRowsPerBlock - 1) / kRowsPerBlock;
    if ((int)blockIdx.x >= kHeavySlots + row_blocks) {  // a relation row: needs nothing from the other processes
        __shared__ float rel_part[kSegmentLanes][64 * V];
        __shared__ uint32_t rel_perm[64 * kSegmentLanes];
        const int rho = (int)blockIdx.x - kHeavySlots - row_blocks;
        if (rho >= rr.n_rel) {  // the loss block
            float part = 0.f;
            for (int i = threadIdx.x; i < rr.loss_n; i += 64 * kSegmentLanes) part += rr.loss_rows[i];
            part = block_sum<64 * kSegmentLanes>(part, &rel_part[0][0]);
            if (threadIdx.x == 0) {
                const float step_loss = part * rr.inv_normaliser + (rr.extra_loss ? *rr.extra_loss : 0.f);
                *rr.loss_total += step_loss;
                *rr.loss_last = step_loss;
            }
            return;
        }
        relation_row_sum<V, kSegmentLanes>(rr, rho, (int)L.d, rel_part, rel_perm, step_size, ap);
        return;
    }
    exchange_wait(sync, XCHG_TAIL_GRADS);  // grad_recv is written by the other processes
    // partial sums of the item lanes, [lane][head | tail][64 column threads][V]
    __shared__ float part[kSegmentLanes][2][64 * V];
    __shared__ uint32_t s_perm[64 * kSegmentLanes];
    __shared__ int s_last;
    const int D = L.d;
    const int col = threadIdx.x & 63, lane = threadIdx.x >> 6;
    const bool helper = (int)blockIdx.x < kHeavySlots;
    int r;
    uint32_t q0, q1, info = 0, slot_word;
    size_t row;
    uint4 first4 = make_uint4(0u, 0u, 0u, 0u);
    if (helper) {
        if (blockIdx.x >= *heavy.count) return;
        const uint4 h = heavy.parts[blockIdx.x];
        r = (int)h.x; q0 = h.y; q1 = h.z; info = h.w;
        slot_word = first_slot[r]; row = remote[r];
    } else {
        // one warp per gathered row: nothing in a row's update needs more than a warp, and a block of
        // eight independent warps keeps eight rows' loads in flight
        r = ((int)blockIdx.x - kHeavySlots) * kRowsPerBlock + (int)(threadIdx.x >> 5);
        if (r >= R) return;
        if (heavy.row_info) {
            const uint4 a = heavy.row_info[2 * r];
            first4 = heavy.row_info[2 * r + 1];
            q0 = a.x; q1 = a.x + a.y; slot_word = a.z; row = a.w;
        } else {
            slot_word = first_slot[r]; q0 = off[r]; q1 = off[r + 1]; row = remote[r];
        }
        if (slot_word & 2u) return;  // its lookups are summed part by part by the first blocks
    }
    ST* __restrict__ xv = reinterpret_cast<ST*>(table + row * L.row_bytes);
    ST* __restrict__ mv = reinterpret_cast<ST*>(table + row * L.row_bytes + L.off_m);
    ST* __restrict__ qv = reinterpret_cast<ST*>(table + row * L.row_bytes + L.off_q);
    // the state before the update comes from the step's gathered copy (slot r), not from the table
    const ST* __restrict__ xs = reinterpret_cast<const ST*>(rows_c + (size_t)r * L.row_bytes);
    const ST* __restrict__ ms = reinterpret_cast<const ST*>(rows_c + (size_t)r * L.row_bytes + L.off_m);
    const ST* __restrict__ qs = reinterpret_cast<const ST*>(rows_c + (size_t)r * L.row_bytes + L.off_q);
    const float alpha = *step_size * lr_modifier;
    const bool writes_row = (slot_word & 1u) != 0;

    // Sums of the lookups [q0, q1) for the columns c .. c+V-1, separately for head and tail lookups;
    // complete in the threads of lane 0.  Lane l sums the lookups q0 + l, q0 + l + lanes, ... in
    // that order, four loads in flight; the lanes' partial sums are then added in lane order: a
    // fixed tree, whatever the timing.  Called by all threads of the block.
    auto segment_sums = [&](int c, float (&gh)[V], float (&gt)[V]) {
#pragma unroll
        for (int u = 0; u < V; ++u) gh[u] = gt[u] = 0.f;
        for (uint32_t base = q0; base < q1; base += 64 * kSegmentLanes) {
            // the segment's lookups go through shared memory, so the row loads do not wait on them
            const int count = (int)min((uint32_t)(64 * kSegmentLanes), q1 - base);
            __syncthreads();
            if ((int)threadIdx.x < count) s_perm[threadIdx.x] = perm[base + threadIdx.x];
            __syncthreads();
            if (c >= D) continue;
            for (int q = lane; q < count; q += 4 * kSegmentLanes) {
                uint32_t e[4];
                float4 g[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) e[u] = q + u * kSegmentLanes < count ? s_perm[q + u * kSegmentLanes] : 0xffffffffu;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    g[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (e[u] == 0xffffffffu) continue;
                    const float* src = e[u] < (uint32_t)B ? d_head + (size_t)e[u] * D + c
                                                          : grad_recv + (size_t)(e[u] - B) * D + c;
                    if (V == 4) g[u] = load4(src); else g[u].x = src[0];
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (e[u] == 0xffffffffu) continue;
                    if (e[u] < (uint32_t)B) {
                        gh[0] += g[u].x;
                        if (V == 4) { gh[1 % V] += g[u].y; gh[2 % V] += g[u].z; gh[3 % V] += g[u].w; }
                    } else {
                        gt[0] += g[u].x;
                        if (V == 4) { gt[1 % V] += g[u].y; gt[2 % V] += g[u].z; gt[3 % V] += g[u].w; }
                    }
                }
            }
        }
        __syncthreads();  // the previous column block's partials have been consumed
#pragma unroll
        for (int u = 0; u < V; ++u) {
            part[lane][0][col * V + u] = gh[u];
            part[lane][1][col * V + u] = gt[u];
        }
        __syncthreads();
        if (lane != 0) return;
#pragma unroll
        for (int u = 0; u < V; ++u) {
            gh[u] = part[0][0][col * V + u];
            gt[u] = part[0][1][col * V + u];
#pragma unroll
            for (int l = 1; l < kSegmentLanes; ++l) {
                gh[u] += part[l][0][col * V + u];
                gt[u] += part[l][1][col * V + u];
            }
        }
    };

    // The row's hidden gradients and its Adam step for the columns c .. c+V-1 (one thread).
    auto finish = [&](int c, float (&gh)[V], float (&gt)[V]) {
        const size_t o = (size_t)r * D + c;
        float gv[V];  // the value's gradient: the lookups' sums (+ the regularisers' terms for the value)
#pragma unroll
        for (int u = 0; u < V; ++u) gv[u] = gh[u] + gt[u];
        if (EXTRAS && rr.reg_val) {
            // gh / gt become the gradients of the feature network's output
#pragma unroll
            for (int u = 0; u < V; ++u) {
                gv[u] += rr.reg_val[o + u];
                gh[u] += rr.reg_h[o + u];
                if (rr.reg_t) gt[u] += rr.reg_t[o + u];
            }
        }
        if (EXTRAS && rr.drop.threshold) {
            // through the dropout of each call: kept elements pass g / (1 - p)
            const uint32_t keep_h = dropout_keep4(rr.drop, 0u, (uint32_t)r, (uint32_t)c >> 2), keep_t = dropout_keep4(rr.drop, 1u, (uint32_t)r, (uint32_t)c >> 2);
#pragma unroll
            for (int u = 0; u < V; ++u) {
                const int bit = (c & 3) + u;
                gh[u] = (keep_h >> bit) & 1u ? gh[u] * rr.drop.scale : 0.f;
                gt[u] = (keep_t >> bit) & 1u ? gt[u] * rr.drop.scale : 0.f;
            }
        }
        if (V == 4) {
            if (d_hid_t) {
                const float4 a = make_float4(gh[0], gh[1 % V], gh[2 % V], gh[3 % V]), b = make_float4(gt[0], gt[1 % V], gt[2 % V], gt[3 % V]);
                store4(d_hid_h + o, a);
                store4(d_hid_t + o, b);
                if (rr.d_hid_h_lo) store4(rr.d_hid_h_lo + o, tf32_lower4(a));
                if (rr.d_hid_t_lo) store4(rr.d_hid_t_lo + o, tf32_lower4(b));
            } else {
                const float4 a = make_float4(gh[0] + gt[0], gh[1 % V] + gt[1 % V], gh[2 % V] + gt[2 % V], gh[3 % V] + gt[3 % V]);
                store4(d_hid_h + o, a);
                if (rr.d_hid_h_lo) store4(rr.d_hid_h_lo + o, tf32_lower4(a));  // lower plane for the projection gradient
            }
        } else {
            d_hid_h[o] = d_hid_t ? gh[0] : gh[0] + gt[0];
            if (d_hid_t) d_hid_t[o] = gt[0];
        }
        if (EXTRAS && rr.defer_grad) {
#pragma unroll
            for (int u = 0; u < V; ++u) rr.defer_grad[o + u] = gv[u];
            return;
        }
        if (!writes_row) return;
        float x[V], m[V], qq[V];
        if (V == 4) {
            const float4 a = L.value_bf16 ? load4(reinterpret_cast<const __nv_bfloat16*>(xs) + c) : load4(xs + c), b = load4(ms + c), d = load4(qs + c);
            x[0] = a.x; x[1 % V] = a.y; x[2 % V] = a.z; x[3 % V] = a.w;
            m[0] = b.x; m[1 % V] = b.y; m[2 % V] = b.z; m[3 % V] = b.w;
            qq[0] = d.x; qq[1 % V] = d.y; qq[2 % V] = d.z; qq[3 % V] = d.w;
        } else {
            x[0] = load_value<ST>(L, reinterpret_cast<const uint8_t*>(xs), c); m[0] = load_as_float(ms + c); qq[0] = load_as_float(qs + c);
        }
#pragma unroll
        for (int u = 0; u < V; ++u) {
            const float g = gv[u];
            float v = qq[u] * qq[u];
            m[u] = ap.beta_m * m[u] + ap.one_minus_beta_m * g;
            v = ap.beta_v * v + ap.one_minus_beta_v * g * g;
            x[u] = x[u] - alpha * (m[u] / (sqrtf(v) + ap.epsilon) + ap.weight_decay * x[u]);
            qq[u] = sqrtf(v);
        }
        if (V == 4) {
            if (L.value_bf16) store4(reinterpret_cast<__nv_bfloat16*>(xv) + c, make_float4(x[0], x[1 % V], x[2 % V], x[3 % V]));
            else store4(xv + c, make_float4(x[0], x[1 % V], x[2 % V], x[3 % V]));
            store4(mv + c, make_float4(m[0], m[1 % V], m[2 % V], m[3 % V]));
            store4(qv + c, make_float4(qq[0], qq[1 % V], qq[2 % V], qq[3 % V]));
        } else {
            store_value<ST>(L, reinterpret_cast<uint8_t*>(xv), c, x[0]);
            store_from_float(mv + c, m[0]);
            store_from_float(qv + c, qq[0]);
        }
    };

    float gh[V], gt[V];
    if (!helper) {
        // the row's lookups in position order, four lookups and two column chunks (eight loads) in
        // flight; head and tail lookups apart
        const int wl = threadIdx.x & 31;
        if (writes_row && (wl & 7) == 0) {
            // The row's state is needed only after its gradient rows have been summed, but its address is
            // known now: ask L2 for it (one request per 128-byte line, no registers held).
            for (int c = wl * V; c < D; c += 32 * V) {
                asm volatile("prefetch.global.L2 [%0];" ::"l"(L.value_bf16 ? reinterpret_cast<const void*>(reinterpret_cast<const __nv_bfloat16*>(xs) + c)
                                                                             : reinterpret_cast<const void*>(xs + c)));
                asm volatile("prefetch.global.L2 [%0];" ::"l"(ms + c));
                asm volatile("prefetch.global.L2 [%0];" ::"l"(qs + c));
            }
        }
        for (int c0 = 0; c0 < D; c0 += 64 * V) {
            const int ca = c0 + wl * V, cb = ca + 32 * V;
            if (ca >= D) continue;
            const bool two = cb < D;
            float hb[V], tb[V];
#pragma unroll
            for (int u = 0; u < V; ++u) gh[u] = gt[u] = hb[u] = tb[u] = 0.f;
            for (uint32_t q = q0; q < q1; q += 4) {
                uint32_t e[4];
                float4 ga[4], gb[4];
                if (heavy.row_info && q == q0) {  // the first four lookups came with the row's descriptor
                    e[0] = first4.x; e[1] = first4.y; e[2] = first4.z; e[3] = first4.w;
                } else {
#pragma unroll
                    for (int u = 0; u < 4; ++u) e[u] = q + u < q1 ? perm[q + u] : 0xffffffffu;
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    ga[u] = gb[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (e[u] == 0xffffffffu) continue;
                    const float* src = e[u] < (uint32_t)B ? d_head + (size_t)e[u] * D : grad_recv + (size_t)(e[u] - B) * D;
                    if (V == 4) {
                        ga[u] = load4(src + ca);
                        if (two) gb[u] = load4(src + cb);
                    } else {
                        ga[u].x = src[ca];
                        if (two) gb[u].x = src[cb];
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (e[u] == 0xffffffffu) continue;
                    if (e[u] < (uint32_t)B) {
                        gh[0] += ga[u].x; hb[0] += gb[u].x;
                        if (V == 4) {
                            gh[1 % V] += ga[u].y; gh[2 % V] += ga[u].z; gh[3 % V] += ga[u].w;
                            hb[1 % V] += gb[u].y; hb[2 % V] += gb[u].z; hb[3 % V] += gb[u].w;
                        }
                    } else {
                        gt[0] += ga[u].x; tb[0] += gb[u].x;
                        if (V == 4) {
                            gt[1 % V] += ga[u].y; gt[2 % V] += ga[u].z; gt[3 % V] += ga[u].w;
                            tb[1 % V] += gb[u].y; tb[2 % V] += gb[u].z; tb[3 % V] += gb[u].w;
                        }
                    }
                }
            }
            finish(ca, gh, gt);
            if (two) finish(cb, hb, tb);
        }
        return;
    }
    // one part of a popular row: leave its sums; the part that arrives last adds all of them
    const int first = (int)(info >> 16), parts = (int)((info >> 8) & 255u), me = (int)(info & 255u);
    for (int c0 = 0; c0 < D; c0 += 64 * V) {
        const int c = c0 + col * V;
        segment_sums(c, gh, gt);
        if (lane == 0 && c < D) {
            float* mine = heavy.partial + (size_t)(first + me) * 2 * D;
#pragma unroll
            for (int u = 0; u < V; ++u) {
                mine[c + u] = gh[u];
                mine[D + c + u] = gt[u];
            }
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned arrived = atomicAdd(&heavy.counter[first], 1u) + 1u;
        s_last = arrived == (unsigned)parts;
        if (s_last) heavy.counter[first] = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (lane != 0) return;
    for (int c = col * V; c < D; c += 64 * V) {
#pragma unroll
        for (int u = 0; u < V; ++u) gh[u] = gt[u] = 0.f;
        for (int p = 0; p < parts; ++p) {
            const float* theirs = heavy.partial + (size_t)(first + p) * 2 * D;
#pragma unroll
            for (int u = 0; u < V; ++u) {
                gh[u] += __ldcg(theirs + c + u);
                gt[u] += __ldcg(theirs + D + c + u);
            }
        }
        finish(c, gh, gt);
    }
}

// ---------------------------------------------------------------------------
// Projection backward: dW[f, d] (+)= sum_r feature[remote[r], f] * d_hidden[r, d]
// (src/pag/pag.cpp:695-700).  A = feature^T is read from the gathered table rows; the r
// range is split over blockIdx.z and each split writes its own partial, summed later in
// a fixed order.  Same 64x64x16 tiling as k_hidden.  gridDim.z = n_net * splits.
template <class FT>
__global__ void __launch_bounds__(256)
k_projection_bwd(const uint8_t* __restrict__ table, RowLayout L, const uint32_t* __restrict__ remote,
                 int R, const float* __restrict__ dh0, const float* __restrict__ dh1, int splits,
                 int rows_per_split, float* __restrict__ partial) {
    grid_dependency_sync();
    constexpr int BM = 64, BN = 64, BK = 16;
    __shared__ __align__(16) float As[BK][BM];
    __shared__ __align__(16) float Bs[BK][BN];
    const int D = L.d, F = L.f;
    const int net = blockIdx.z / splits, split = blockIdx.z - net * splits;
    const float* __restrict__ dh = net ? dh1 : dh0;
    float* __restrict__ out = partial + ((size_t)net * splits + split) * (size_t)F * D;
    const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    const int r_lo = split * rows_per_split, r_hi = min(R, r_lo + rows_per_split);
    const int ld_k = t >> 4, ld_c = (t & 15) * 4;
    const bool d_vec = (D & 3) == 0;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int r0 = r_lo; r0 < r_hi; r0 += BK) {
        const int r = r0 + ld_k;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
        if (r < r_hi) {
            const size_t row = remote ? remote[r] : (size_t)r;
            const FT* fp = reinterpret_cast<const FT*>(table + row * L.row_bytes + L.off_feat);
            const int f = m0 + ld_c;
            if (f + 3 < F) {
                a = load4(fp + f);
            } else {
                if (f + 0 < F) a.x = load_as_float(fp + f + 0);
                if (f + 1 < F) a.y = load_as_float(fp + f + 1);
                if (f + 2 < F) a.z = load_as_float(fp + f + 2);
            }
            const int n = n0 + ld_c;
            const float* gp = dh + (size_t)r * D + n;
            if (d_vec && n + 3 < D) {
                b = load4(gp);
            } else {
                if (n + 0 < D) b.x = gp[0];
                if (n + 1 < D) b.y = gp[1];
                if (n + 2 < D) b.z = gp[2];
                if (n + 3 < D) b.w = gp[3];
            }
        }
        __syncthreads();
        store4(&As[ld_k][ld_c], a);
        store4(&Bs[ld_k][ld_c], b);
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 av = load4(&As[kk][ty * 4]);
            const float4 bv = load4(&Bs[kk][tx * 4]);
            const float ar[4] = {av.x, av.y, av.z, av.w};
            const float br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int f = m0 + ty * 4 + i;
        if (f >= F) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < D) out[(size_t)f * D + n] = acc[i][j];
        }
    }
}

// This shard's contribution to the dense gradients, laid out like the dense parameter
// vector: relation table | projection(s), and written slice by slice into the memory of the
// process that owns (reduces and updates) each row: the rows are dealt out in turn, row r to
// process r % n_owner as its row r / n_owner, so that every process receives and updates an
// equal share of every parameter; dense_dst[owner] is this shard's slot in that process's
// receive buffer.  Relation rows are the segment sums of the
// per-triple relation gradients (backward of the gather at src/poplar_kge.cpp:489);
// projection entries sum the split partials of k_projection_bwd in split order.
constexpr int kRelationLanes = 8;

template <int V>
__global__ void __launch_bounds__(64 * kRelationLanes)
k_dense_partial(const float* __restrict__ d_relrow, const uint32_t* __restrict__ rel_perm,
                const uint32_t* __restrict__ rel_off, int n_rel, int D,
                const float* __restrict__ proj_partial, int n_net, int splits, size_t proj_elems,
                float* const* __restrict__ dense_dst, int n_owner, ExchangeSync sync, int signal_kind, int row_offset) {
    grid_dependency_sync();
    __shared__ float part[kRelationLanes][64 * V];
    __shared__ uint32_t s_perm[64 * kRelationLanes];
    if ((int)blockIdx.x < n_rel) {
        // One relation row.  Relation popularity is skewed, so a few rows own most of the batch's
        // triples: the row's lookups are staged in shared memory, lane l sums triples l, l + lanes,
        // ... (four loads in flight) and the lanes' partial sums are added in lane order.
        const int rho = blockIdx.x, col = threadIdx.x & 63, lane = threadIdx.x >> 6;
        const uint32_t q0 = rel_off[rho], q1 = rel_off[rho + 1];
        // the row goes to the process that owns this slice of the dense vector
        // (row_offset: where these rows begin in the dense vector; 0 for the relation table)
        const int owner = (rho + row_offset) % n_owner;
        float* __restrict__ dst_row = dense_dst[owner] + (size_t)((rho + row_offset) / n_owner) * D;
        if (q0 == q1) {
            for (int c = threadIdx.x; c < D; c += blockDim.x) dst_row[c] = 0.f;
            exchange_signal(sync, signal_kind, gridDim.x);
            return;
        }
        for (int c0 = 0; c0 < D; c0 += 64 * V) {
            const int c = c0 + col * V;
            float g[V];
#pragma unroll
            for (int u = 0; u < V; ++u) g[u] = 0.f;
            for (uint32_t base = q0; base < q1; base += 64 * kRelationLanes) {
                const int count = (int)min((uint32_t)(64 * kRelationLanes), q1 - base);
                __syncthreads();
                if ((int)threadIdx.x < count) s_perm[threadIdx.x] = rel_perm[base + threadIdx.x];
                __syncthreads();
                if (c >= D) continue;
                for (int i = lane; i < count; i += 4 * kRelationLanes) {
                    float4 v[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int ii = i + u * kRelationLanes;
                        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (ii < count) {
                            const float* src = d_relrow + (size_t)s_perm[ii] * D + c;
                            if (V == 4) v[u] = load4(src); else v[u].x = src[0];
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        if (i + u * kRelationLanes >= count) continue;
                        g[0] += v[u].x;
                        if (V == 4) { g[1 % V] += v[u].y; g[2 % V] += v[u].z; g[3 % V] += v[u].w; }
                    }
                }
            }
            __syncthreads();
#pragma unroll
            for (int u = 0; u < V; ++u) part[lane][col * V + u] = g[u];
            __syncthreads();
            if (lane == 0 && c < D) {
#pragma unroll
                for (int u = 0; u < V; ++u) {
                    float total = part[0][col * V + u];
#pragma unroll
                    for (int l = 1; l < kRelationLanes; ++l) total += part[l][col * V + u];
                    dst_row[c + u] = total;
                }
            }
        }
        exchange_signal(sync, signal_kind, gridDim.x);
        return;
    }
    const size_t rel_elems = (size_t)n_rel * D;
    const size_t total = (size_t)n_net * proj_elems;
    const size_t first = ((size_t)blockIdx.x - n_rel) * blockDim.x + threadIdx.x;
    const size_t stride = ((size_t)gridDim.x - n_rel) * blockDim.x;
    for (size_t pe = first; pe < total; pe += stride) {
        const size_t net = pe / proj_elems, idx = pe - net * proj_elems;
        float g = 0.f;
        for (int z = 0; z < splits; ++z) g += proj_partial[(net * splits + z) * proj_elems + idx];
        const size_t e = rel_elems + pe, row = e / D;
        dense_dst[row % n_owner][(row / n_owner) * D + (e - row * D)] = g;
    }
    exchange_signal(sync, signal_kind, gridDim.x);
}

// Sum of the shards' dense contributions in shard order (the reduce-scatter of
// src/pag/pag.cpp:980-994), Adam on the slice of the dense vector this process owns
// (src/poplar_kge.cpp:329-339) and the write of the new values into every replica
// (the all-gather on next use, :341-348).  Pointer tables live in device memory; entries
// may point into peers' memory.
constexpr int kDenseParams = 8;
struct DenseUpdateArgs {
    const float* const* partials;  // [n_partial] the shards' slots in this process's receive buffer
    int n_partial;
    float* const* replicas;  // [n_replica] dense parameter vectors
    float* const* replicas_lo;  // [n_replica] their lower TF32 planes (the projections are tensor-core operands); null: none
    int n_replica;
    float* adam_m;
    float* adam_v;
    // This process owns the rows self, self + n_replica, ... of the dense vector: n_own of them,
    // row_width elements each; its j-th row is row j of every slot.
    size_t n_own, row_width;
    // parameter p covers the elements [bounds[p], bounds[p+1]): relation table, projection(s), TransH
    // normals, the feature MLP's up / down projections per network; absent ones are empty
    size_t bounds[kDenseParams + 1];
    float lr_modifier[kDenseParams];
    const float* step_size;
    AdamParams ap;
    ExchangeSync sync;
};

__device__ __forceinline__ int dense_param_of(const DenseUpdateArgs& a, size_t e) {
    int p = 0;
    while (p + 1 < kDenseParams && e >= a.bounds[p + 1]) ++p;
    return p;
}

__device__ __forceinline__ float dense_adam(float x, float g, float& m, float& v, float alpha, const AdamParams& ap) {
    m = ap.beta_m * m + ap.one_minus_beta_m * g;
    v = ap.beta_v * v + ap.one_minus_beta_v * g * g;
    return x - alpha * (m / (sqrtf(v) + ap.epsilon) + ap.weight_decay * x);
}

// The shards' partial gradients of the owned slice have been written into this process's
// receive buffer by their producers; the new values are written to every process's copy of the
// parameters (posted stores over NVLink).  Four elements per access.
static __global__ void __launch_bounds__(256) k_dense_update(DenseUpdateArgs a, int self) {
    grid_dependency_sync();
    exchange_wait(a.sync, XCHG_DENSE_PARTIALS);  // every process's partial gradients are complete
    const float base_alpha = *a.step_size;
    const size_t W = a.row_width, total = a.n_own * W;
    size_t all_bounds = W;
    for (int p = 1; p <= kDenseParams; ++p) all_bounds |= a.bounds[p];
    const bool vec = (all_bounds & 3) == 0;
    if (vec) {
        for (size_t le = 4 * ((size_t)blockIdx.x * blockDim.x + threadIdx.x); le < total; le += 4 * (size_t)gridDim.x * blockDim.x) {
            const size_t j = le / W, e = (j * a.n_replica + self) * W + (le - j * W);  // slot index -> dense index
            float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
            for (int s = 0; s < a.n_partial; ++s) {
                const float4 t = *reinterpret_cast<const float4*>(a.partials[s] + le);
                g.x += t.x; g.y += t.y; g.z += t.z; g.w += t.w;
            }
            const int p = dense_param_of(a, e);
            const float alpha = base_alpha * a.lr_modifier[p];
            float4 x = *reinterpret_cast<const float4*>(a.replicas[self] + e);
            float4 m = *reinterpret_cast<const float4*>(a.adam_m + e), v = *reinterpret_cast<const float4*>(a.adam_v + e);
            x.x = dense_adam(x.x, g.x, m.x, v.x, alpha, a.ap);
            x.y = dense_adam(x.y, g.y, m.y, v.y, alpha, a.ap);
            x.z = dense_adam(x.z, g.z, m.z, v.z, alpha, a.ap);
            x.w = dense_adam(x.w, g.w, m.w, v.w, alpha, a.ap);
            *reinterpret_cast<float4*>(a.adam_m + e) = m;
            *reinterpret_cast<float4*>(a.adam_v + e) = v;
            for (int rep = 0; rep < a.n_replica; ++rep) *reinterpret_cast<float4*>(a.replicas[rep] + e) = x;
            if (a.replicas_lo && p > 0) {
                const float4 lo = tf32_lower4(x);
                for (int rep = 0; rep < a.n_replica; ++rep) *reinterpret_cast<float4*>(a.replicas_lo[rep] + e) = lo;
            }
        }
    } else {
        for (size_t le = (size_t)blockIdx.x * blockDim.x + threadIdx.x; le < total; le += (size_t)gridDim.x * blockDim.x) {
            const size_t j = le / W, e = (j * a.n_replica + self) * W + (le - j * W);
            float g = 0.f;
            for (int s = 0; s < a.n_partial; ++s) g += a.partials[s][le];
            const int p = dense_param_of(a, e);
            const float alpha = base_alpha * a.lr_modifier[p];
            float m = a.adam_m[e], v = a.adam_v[e];
            const float x = dense_adam(a.replicas[self][e], g, m, v, alpha, a.ap);
            a.adam_m[e] = m;
            a.adam_v[e] = v;
            for (int rep = 0; rep < a.n_replica; ++rep) a.replicas[rep][e] = x;
            if (a.replicas_lo && p > 0)
                for (int rep = 0; rep < a.n_replica; ++rep) a.replicas_lo[rep][e] = tf32_lower(x);
        }
    }
    exchange_signal(a.sync, XCHG_DENSE_PARAMS, gridDim.x);  // the new values are in every process's copy
}

// ---------------------------------------------------------------------------
// Cross-process barrier on flags in peer-visible memory.  Thread r publishes this
// process's new epoch into peer r's flag array, then waits until peer r's epoch has
// reached it.  The wait is bounded: on expiry the kernel records an error and returns.
struct BarrierArgs {
    unsigned* const* peer_flags;  // [world] base of each process's flag array
    unsigned* my_epoch;           // device counter, incremented once per barrier
    unsigned* status;             // device error word: non-zero = a wait gave up
    int rank, world;
    unsigned long long max_spins;
};

static __global__ void k_barrier(BarrierArgs a) {
    grid_dependency_sync();
    __shared__ unsigned epoch;
    if (threadIdx.x == 0) {
        epoch = *a.my_epoch + 1;
        *a.my_epoch = epoch;
        __threadfence_system();
    }
    __syncthreads();
    const int r = threadIdx.x;
    if (r >= a.world) return;
    volatile unsigned* remote_flag = a.peer_flags[r] + a.rank;
    __threadfence_system();
    *remote_flag = epoch;
    volatile unsigned* mine = a.peer_flags[a.rank] + r;
    // Once a wait has given up, the run is lost: later barriers of the same run do not wait again.
    if (*reinterpret_cast<volatile unsigned*>(a.status) != 0) return;
    unsigned long long spins = 0;
    while ((int)(*mine - epoch) < 0) {
        if (++spins > a.max_spins) {
            atomicExch(a.status, 1u + (unsigned)r);
            break;
        }
        __nanosleep(64);
    }
    __threadfence_system();
}

// ---------------------------------------------------------------------------
// Streaming top-k of predict (src/poplar_kge.cpp:743-810): every query keeps its n_best
// highest-scoring candidates so far; a batch of scores is merged by one warp per query.
// Candidates that beat the query's current cut-off are appended to a per-warp buffer in
// shared memory (warp ballot: the order is fixed) and the buffer is sorted down to n_best
// when it fills.  Order: higher score first, ties by lower row index, so the result does not
// depend on the batch size.  The reference leaves the tie order undefined.
constexpr int kTopkCapacity = 256;  // entries per query buffer; n_best <= capacity / 2

__device__ __forceinline__ unsigned long long topk_key(float score, uint32_t index) {
    uint32_t bits = __float_as_uint(score);
    bits = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);  // monotone in the float order
    return ((unsigned long long)bits << 32) | (uint32_t)(~index);
}
__device__ __forceinline__ float topk_score(unsigned long long key) {
    uint32_t bits = (uint32_t)(key >> 32);
    bits = (bits & 0x80000000u) ? (bits & 0x7fffffffu) : ~bits;
    return __uint_as_float(bits);
}
__device__ __forceinline__ uint32_t topk_index(unsigned long long key) { return ~(uint32_t)key; }

// Sorts the warp's buffer in descending key order (empty slots hold key 0, which sorts last).
__device__ __forceinline__ void warp_sort_desc(unsigned long long* buf) {
    const int lane = threadIdx.x & 31;
    for (int k = 2; k <= kTopkCapacity; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            __syncwarp();
            for (int i = lane; i < kTopkCapacity; i += 32) {
                const int ixj = i ^ j;
                if (ixj > i) {
                    const unsigned long long a = buf[i], b = buf[ixj];
                    const bool descending = (i & k) == 0;
                    if ((a < b) == descending) {
                        buf[i] = b;
                        buf[ixj] = a;
                    }
                }
            }
        }
    }
    __syncwarp();
}

struct TopkParams {
    int n_query, n_best;
    int score_is_gamma_minus;  // TransE: score = gamma - raw
    float gamma;
};

// A batch of scores is merged in two kernels.  k_topk_filter reads all of it at full bandwidth
// (four scores per thread) and leaves, per query, the keys that beat the query's cut-off as it
// stands before the batch in `cand` (at most kTopkCandidates; the count goes on past that).
// k_topk_update, one warp per query, then merges those few keys; a query whose candidates did not
// fit (the first batches, before a cut-off exists) scans its row of scores itself, as it would
// without the filter.  The candidates' order in `cand` depends on timing, the merged result does
// not: it is the n_best largest keys of the old list and the candidates, and keys are unique.
constexpr int kTopkCandidates = 1024;

static __global__ void __launch_bounds__(256)
k_topk_filter(const float* __restrict__ raw, int n_cols, uint32_t first_row, uint32_t last_valid_row,
              const unsigned long long* __restrict__ state, const int* __restrict__ counts,
              unsigned long long* __restrict__ cand, int* __restrict__ cand_count, TopkParams tp) {
    const int q = blockIdx.y, lane = threadIdx.x & 31;
    const unsigned long long cutoff = counts[q] >= tp.n_best ? state[(size_t)q * kTopkCapacity + tp.n_best - 1] : 0ull;
    if (cutoff == 0ull) {  // no cut-off yet: every score is a candidate, the query scans its row itself
        if (blockIdx.x == 0 && threadIdx.x == 0) cand_count[q] = kTopkCandidates + 1;
        return;
    }
    const float* __restrict__ row = raw + (size_t)q * n_cols;
    const bool vec = (n_cols & 3) == 0;
    // a warp walks 128 consecutive scores at a time; its lanes stay together for the ballots
    for (int w0 = 4 * (blockIdx.x * 256 + (threadIdx.x & ~31)); w0 < n_cols; w0 += 4 * 256 * gridDim.x) {
        const int j0 = w0 + 4 * lane;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (j0 < n_cols) {
            if (vec) {
                const float4 x = *reinterpret_cast<const float4*>(row + j0);
                v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
            } else {
                for (int u = 0; u < 4 && j0 + u < n_cols; ++u) v[u] = row[j0 + u];
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j = j0 + u;
            unsigned long long key = 0ull;
            if (j < n_cols && first_row + (uint32_t)j <= last_valid_row)
                key = topk_key(tp.score_is_gamma_minus ? tp.gamma - v[u] : v[u], first_row + (uint32_t)j);
            const bool pass = key > cutoff;
            const unsigned mask = __ballot_sync(0xffffffffu, pass);
            if (mask == 0) continue;
            int base = 0;
            if (lane == __ffs(mask) - 1) base = atomicAdd(cand_count + q, __popc(mask));  // one addition per warp
            base = __shfl_sync(0xffffffffu, base, __ffs(mask) - 1);
            const int slot = base + __popc(mask & ((1u << lane) - 1));
            if (pass && slot < kTopkCandidates) cand[(size_t)q * kTopkCandidates + slot] = key;
        }
    }
}

// raw [n_query, n_cols] holds distances / dot products against rows first_row .. first_row+n_cols-1;
// rows above last_valid_row are padding of the shard and are skipped (src/poplar_kge.cpp:836-842).
// state [n_query, kTopkCapacity] keys, counts [n_query].  4 warps per block, one query each.
// cand / cand_count (may be null): the filter's output for this batch; the counts are cleared for the next.
static __global__ void __launch_bounds__(128)
k_topk_update(const float* __restrict__ raw, int n_cols, uint32_t first_row, uint32_t last_valid_row,
              unsigned long long* __restrict__ state, int* __restrict__ counts, TopkParams tp,
              const unsigned long long* __restrict__ cand, int* __restrict__ cand_count) {
    __shared__ unsigned long long buffers[4][kTopkCapacity];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q = blockIdx.x * 4 + warp;
    if (q >= tp.n_query) return;
    unsigned long long* buf = buffers[warp];
    unsigned long long* mine = state + (size_t)q * kTopkCapacity;
    int count = counts[q];
    for (int i = lane; i < kTopkCapacity; i += 32) buf[i] = i < count ? mine[i] : 0ull;
    __syncwarp();
    unsigned long long cutoff = count >= tp.n_best ? buf[tp.n_best - 1] : 0ull;
    const int n_cand = cand_count ? cand_count[q] : kTopkCandidates + 1;
    __syncwarp();
    if (cand_count && lane == 0) cand_count[q] = 0;
    if (n_cand == 0) return;  // nothing in this batch beats the cut-off: the list stands
    if (n_cand <= kTopkCandidates) {
        // the filter's keys for this query: all beat the old cut-off; the cut-off rises as they are merged
        const unsigned long long* __restrict__ keys = cand + (size_t)q * kTopkCandidates;
        for (int base = 0; base < n_cand; base += 32) {
            const unsigned long long key = base + lane < n_cand ? keys[base + lane] : 0ull;
            const bool pass = key > cutoff;
            if (__ballot_sync(0xffffffffu, pass) == 0) continue;
            if (count + 32 > kTopkCapacity) {
                warp_sort_desc(buf);
                count = min(count, tp.n_best);
                for (int i = count + lane; i < kTopkCapacity; i += 32) buf[i] = 0ull;
                __syncwarp();
                cutoff = count >= tp.n_best ? buf[tp.n_best - 1] : 0ull;
            }
            const bool still = pass && key > cutoff;
            const unsigned mask2 = __ballot_sync(0xffffffffu, still);
            if (still) buf[count + __popc(mask2 & ((1u << lane) - 1))] = key;
            count += __popc(mask2);
            __syncwarp();
        }
        warp_sort_desc(buf);
        count = min(count, tp.n_best);
        for (int i = lane; i < kTopkCapacity; i += 32) mine[i] = i < count ? buf[i] : 0ull;
        if (lane == 0) counts[q] = count;
        return;
    }
    const float* __restrict__ row = raw + (size_t)q * n_cols;
    constexpr int kAhead = 8;  // scores fetched before the first of them is looked at: the loads overlap
    for (int base0 = 0; base0 < n_cols; base0 += 32 * kAhead) {
    float ahead[kAhead];
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
        const int j = base0 + 32 * u + lane;
        ahead[u] = j < n_cols ? row[j] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
        const int base = base0 + 32 * u;
        if (base >= n_cols) break;
        const int j = base + lane;
        unsigned long long key = 0ull;
        if (j < n_cols && first_row + (uint32_t)j <= last_valid_row) {
            const float v = ahead[u];
            key = topk_key(tp.score_is_gamma_minus ? tp.gamma - v : v, first_row + (uint32_t)j);
        }
        const bool pass = key > cutoff;
        const unsigned mask = __ballot_sync(0xffffffffu, pass);
        if (mask == 0) continue;
        if (count + 32 > kTopkCapacity) {  // no room for a full ballot: sort down to n_best first
            warp_sort_desc(buf);
            count = min(count, tp.n_best);
            for (int i = count + lane; i < kTopkCapacity; i += 32) buf[i] = 0ull;
            __syncwarp();
            cutoff = count >= tp.n_best ? buf[tp.n_best - 1] : 0ull;
        }
        const bool still = pass && key > cutoff;
        const unsigned mask2 = __ballot_sync(0xffffffffu, still);
        if (still) buf[count + __popc(mask2 & ((1u << lane) - 1))] = key;
        count += __popc(mask2);
        __syncwarp();
    }
    }
    warp_sort_desc(buf);
    count = min(count, tp.n_best);
    for (int i = lane; i < kTopkCapacity; i += 32) mine[i] = i < count ? buf[i] : 0ull;
    if (lane == 0) counts[q] = count;
}

// Writes each query's sorted candidates to the shard that asked: query q = (asking shard, slot)
// goes to out_blocks[asking shard] + slot * n_best (the return all-to-all of
// src/poplar_kge.cpp:847-850).  Missing candidates get the reference's BadScore and row 0.
static __global__ void __launch_bounds__(128)
k_topk_finish(const unsigned long long* __restrict__ state, const int* __restrict__ counts, int n_query,
              int queries_per_shard, int n_best, float* const* __restrict__ score_blocks,
              uint32_t* const* __restrict__ index_blocks) {
    const int q = blockIdx.x;
    if (q >= n_query) return;
    const int shard = q / queries_per_shard, slot = q - shard * queries_per_shard;
    float* __restrict__ so = score_blocks[shard] + (size_t)slot * n_best;
    uint32_t* __restrict__ io = index_blocks[shard] + (size_t)slot * n_best;
    const int count = counts[q];
    for (int i = threadIdx.x; i < n_best; i += blockDim.x) {
        const unsigned long long key = state[(size_t)q * kTopkCapacity + i];
        so[i] = i < count ? topk_score(key) : -1e6f;
        io[i] = i < count ? topk_index(key) : 0u;
    }
}

// ---------------------------------------------------------------------------
// The BESS batch sampler on the device (src/python/poplar_kge_dataset.py:310-393, `sample_batch`,
// with its uniform strategy; `unique_pad` :161-164).  The training triples lie in device memory
// sorted by (head shard, tail shard) bucket, as local rows: triples[0] head rows, [1] relations,
// [2] tail rows (:199-241).  One block draws everything shard s needs for step i:
//   positions [0, B)       its own positives, B / n per tail shard: head rows (and the relations);
//   positions [B, 2B)      the positives of every head shard whose tail lives on s: tail rows;
//   positions [2B, 2B + n * neg)  the negatives every head shard asks s for: uniform rows of s;
// then sorts them, keeps each row once (`remote`, zero-padded) and gives every position the slot
// of its row (`head`, `a2a`).  Draws are counter-based (Philox keyed by seed and run, counted by
// head shard, step, tail shard and slot), so the block of shard s and the block of the head
// shard that owns a positive compute the same triple without talking to each other, on any GPU.
struct SamplerData {
    const uint32_t* triples;        // [3][n_triples]
    size_t n_triples;
    const uint32_t* bucket_offset;  // [n_shard][n_shard]
    const uint32_t* bucket_count;   // [n_shard][n_shard], none empty
    const uint32_t* shard_count;    // [n_shard] real rows per shard (rows 1 .. count)
};

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1);

__device__ __forceinline__ unsigned long long sampler_draw(uint32_t seed, uint32_t run, uint32_t head_shard, uint32_t step,
                                                           uint32_t tail_shard, uint32_t slot) {
    uint32_t c[4] = {head_shard, step, tail_shard, slot};
    uint32_t k0 = seed, k1 = run ^ 0x243F6A88u;
#pragma unroll
    for (int i = 0; i < 10; ++i) {
        philox_round(c, k0, k1);
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return ((unsigned long long)c[0] << 32) | c[1];
}

constexpr uint32_t kNegativeSlot = 0x80000000u;  // slot numbers of negatives, apart from those of positives

static __global__ void __launch_bounds__(512)
k_sample_batch(SamplerData sd, uint32_t seed, uint32_t run, int n_shard, int shard0, int n_step, int B, int a2a,
               uint32_t* __restrict__ remote, uint32_t* __restrict__ a2a_out, uint32_t* __restrict__ head,
               uint32_t* __restrict__ relation, uint32_t* __restrict__ tail) {
    __shared__ unsigned long long keys[kMaxSortItems];
    __shared__ uint32_t s_scan[512];
    const int l = blockIdx.x / n_step, step = blockIdx.x % n_step, s = shard0 + l;
    const int pos = B / n_shard, neg = a2a - pos, T = n_shard * a2a, R = B + T;
    const size_t sidx = (size_t)l * n_step + step;
    remote += sidx * R;
    a2a_out += sidx * T;
    head += sidx * B;
    relation += sidx * B;
    tail += sidx * B;
    int padded = 1;
    while (padded < R) padded <<= 1;
    for (int p = threadIdx.x; p < padded; p += blockDim.x) {
        unsigned long long key = ~0ull;
        if (p < B) {
            const int ts = p / pos, k = p - ts * pos;
            const uint32_t bucket = (uint32_t)(s * n_shard + ts);
            const size_t idx = sd.bucket_offset[bucket] + sampler_draw(seed, run, (uint32_t)s, (uint32_t)step, (uint32_t)ts, (uint32_t)k) % sd.bucket_count[bucket];
            key = ((unsigned long long)sd.triples[idx] << 32) | (unsigned)p;
            relation[p] = sd.triples[sd.n_triples + idx];
            tail[p] = (uint32_t)(ts * a2a + k);  // where the exchange puts this positive's tail (:257-263)
        } else if (p < 2 * B) {
            const int q = p - B, hs = q / pos, k = q - hs * pos;
            const uint32_t bucket = (uint32_t)(hs * n_shard + s);
            const size_t idx = sd.bucket_offset[bucket] + sampler_draw(seed, run, (uint32_t)hs, (uint32_t)step, (uint32_t)s, (uint32_t)k) % sd.bucket_count[bucket];
            key = ((unsigned long long)sd.triples[2 * sd.n_triples + idx] << 32) | (unsigned)p;
        } else if (p < R) {
            const int q = p - 2 * B, hs = q / neg, k = q - hs * neg;
            const uint32_t row = 1u + (uint32_t)(sampler_draw(seed, run, (uint32_t)hs, (uint32_t)step, (uint32_t)s, kNegativeSlot | (uint32_t)k) % sd.shard_count[s]);
            key = ((unsigned long long)row << 32) | (unsigned)p;
        }
        keys[p] = key;
    }
    bitonic_sort(keys, padded);
    // rank of every sorted entry among the distinct rows: an exclusive scan of "starts a new row"
    const int per_thread = (padded + (int)blockDim.x - 1) / (int)blockDim.x, first = threadIdx.x * per_thread;
    uint32_t mine = 0;
    for (int i = first; i < first + per_thread && i < R; ++i) mine += (i == 0 || (keys[i] >> 32) != (keys[i - 1] >> 32)) ? 1u : 0u;
    s_scan[threadIdx.x] = mine;
    __syncthreads();
    for (int o = 1; o < (int)blockDim.x; o <<= 1) {  // Hillis-Steele inclusive scan over the threads' counts
        const uint32_t v = (int)threadIdx.x >= o ? s_scan[threadIdx.x - o] : 0u;
        __syncthreads();
        s_scan[threadIdx.x] += v;
        __syncthreads();
    }
    uint32_t rank = s_scan[threadIdx.x] - mine;  // distinct rows before this thread's first entry
    const uint32_t n_unique = s_scan[blockDim.x - 1];
    for (int i = first; i < first + per_thread && i < R; ++i) {
        const bool starts = i == 0 || (keys[i] >> 32) != (keys[i - 1] >> 32);
        if (starts) remote[rank++] = (uint32_t)(keys[i] >> 32);
        const uint32_t p = (uint32_t)keys[i], slot = rank - 1;
        if (p < (uint32_t)B) {
            head[p] = slot;
        } else if (p < (uint32_t)(2 * B)) {
            const uint32_t q = p - (uint32_t)B, hs = q / (uint32_t)pos;
            a2a_out[hs * a2a + (q - hs * pos)] = slot;
        } else {
            const uint32_t q = p - (uint32_t)(2 * B), hs = q / (uint32_t)neg;
            a2a_out[hs * a2a + pos + (q - hs * neg)] = slot;
        }
    }
    for (int i = (int)n_unique + (int)threadIdx.x; i < R; i += blockDim.x) remote[i] = 0u;  // unique_pad's zeros
}

// ---------------------------------------------------------------------------
// Table I/O (src/poplar_kge.cpp:857-871).

// Counter-based normal numbers (Philox-4x32-10 + Box-Muller), keyed by (seed, shard) and
// counted by (row, column / 4): the initial embedding of a row depends only on its
// address, not on which call wrote it.
__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
    c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
}
__device__ __forceinline__ float4 philox_normal4(uint32_t seed, uint32_t stream, uint32_t row,
                                                 uint32_t col4) {
    uint32_t c[4] = {row, col4, stream, 0x6b676562u};
    uint32_t k0 = seed, k1 = 0x9E3779B9u ^ stream;
#pragma unroll
    for (int i = 0; i < 10; ++i) {
        philox_round(c, k0, k1);
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    const float u0 = ((float)(c[0] >> 8) + 0.5f) * (1.0f / 16777216.0f);
    const float u1 = ((float)(c[1] >> 8) + 0.5f) * (1.0f / 16777216.0f);
    const float u2 = ((float)(c[2] >> 8) + 0.5f) * (1.0f / 16777216.0f);
    const float u3 = ((float)(c[3] >> 8) + 0.5f) * (1.0f / 16777216.0f);
    const float r0 = sqrtf(-2.f * logf(u0)), r1 = sqrtf(-2.f * logf(u2));
    float s0, c0, s1, c1;
    sincospif(2.f * u1, &s0, &c0);
    sincospif(2.f * u3, &s1, &c1);
    return make_float4(r0 * c0, r0 * s0, r1 * c1, r1 * s1);
}

// A slot writes only if no later slot names the same row, so duplicate indices (the
// overflow slots that the host redirects to row 0, src/python/poplar_kge.py:546-552)
// resolve to the last one in order, deterministically.
__device__ __forceinline__ bool is_last_writer(const uint32_t* idx, int n, int j) {
    const uint32_t mine = idx[j];
    for (int k = j + 1; k < n; ++k)
        if (idx[k] == mine) return false;
    return true;
}

// write_entity: fresh embedding ~ N(0, std), zero moments, features from the host array.
template <class ST, class FT, class IT>
__global__ void __launch_bounds__(128)
k_write_entity(uint8_t* __restrict__ table, RowLayout L, const uint32_t* __restrict__ idx, int n,
               const IT* __restrict__ features, uint32_t seed, uint32_t shard, float stddev) {
    const int j = blockIdx.x;
    __shared__ int go;
    if (threadIdx.x == 0) go = is_last_writer(idx, n, j) ? 1 : 0;
    __syncthreads();
    if (!go) return;
    const size_t row = idx[j];
    ST* xv = reinterpret_cast<ST*>(table + row * L.row_bytes);
    ST* mv = reinterpret_cast<ST*>(table + row * L.row_bytes + L.off_m);
    ST* qv = reinterpret_cast<ST*>(table + row * L.row_bytes + L.off_q);
    FT* fv = reinterpret_cast<FT*>(table + row * L.row_bytes + L.off_feat);
    const int D = L.d, F = L.f;
    for (int c4 = threadIdx.x; c4 * 4 < D; c4 += blockDim.x) {
        const float4 z = philox_normal4(seed, shard, (uint32_t)row, (uint32_t)c4);
        const float zz[4] = {z.x, z.y, z.z, z.w};
        for (int u = 0; u < 4 && c4 * 4 + u < D; ++u) {
            store_value<ST>(L, reinterpret_cast<uint8_t*>(xv), c4 * 4 + u, stddev * zz[u]);
            store_from_float(mv + c4 * 4 + u, 0.f);
            store_from_float(qv + c4 * 4 + u, 0.f);
        }
    }
    for (int c = threadIdx.x; c < F; c += blockDim.x)
        store_from_float(fv + c, load_as_float(features + (size_t)j * F + c));
}

// initialise_entities: every row of the shard on the device, no host data.  Embeddings as
// write_entity would draw them; features ~ N(0, 1) from a second stream (row 0, the padding
// row, keeps zero features); optimiser state zero.  Stands in for streaming a dataset's
// features through write_entity when the table is tens of gigabytes of synthetic data.
template <class ST, class FT>
__global__ void __launch_bounds__(256)
k_init_table(uint8_t* __restrict__ table, RowLayout L, size_t n_rows, uint32_t seed, uint32_t shard,
             float stddev) {
    const int D = L.d, F = L.f;
    const int d4 = (D + 3) / 4, f4 = (F + 3) / 4, per_row = d4 + f4;
    const size_t total = n_rows * (size_t)per_row;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (size_t)gridDim.x * blockDim.x) {
        const size_t row = e / per_row;
        const int q = (int)(e - row * per_row);
        uint8_t* base = table + row * L.row_bytes;
        if (q < d4) {
            const float4 z = philox_normal4(seed, shard, (uint32_t)row, (uint32_t)q);
            const float zz[4] = {z.x, z.y, z.z, z.w};
            for (int u = 0; u < 4 && q * 4 + u < D; ++u) {
                store_value<ST>(L, base, q * 4 + u, stddev * zz[u]);
                store_from_float(reinterpret_cast<ST*>(base + L.off_m) + q * 4 + u, 0.f);
                store_from_float(reinterpret_cast<ST*>(base + L.off_q) + q * 4 + u, 0.f);
            }
        } else {
            const int c4 = q - d4;
            const float4 z = philox_normal4(seed ^ 0x5bd1e995u, shard, (uint32_t)row, (uint32_t)c4);
            const float zz[4] = {z.x, z.y, z.z, z.w};
            for (int u = 0; u < 4 && c4 * 4 + u < F; ++u)
                store_from_float(reinterpret_cast<FT*>(base + L.off_feat) + c4 * 4 + u, row == 0 ? 0.f : zz[u]);
        }
    }
}

// write_entity_rows: whole rows [value | m | sqrt(v) | feature] from the host array.
template <class ST, class FT, class IT>
__global__ void __launch_bounds__(128)
k_write_rows(uint8_t* __restrict__ table, RowLayout L, const uint32_t* __restrict__ idx, int n,
             const IT* __restrict__ data) {
    const int j = blockIdx.x;
    __shared__ int go;
    if (threadIdx.x == 0) go = is_last_writer(idx, n, j) ? 1 : 0;
    __syncthreads();
    if (!go) return;
    const size_t row = idx[j];
    const int D = L.d, F = L.f, W = 3 * D + F;
    const IT* __restrict__ src = data + (size_t)j * W;
    uint8_t* base = table + row * L.row_bytes;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = load_as_float(src + c);
        if (c < D) store_value<ST>(L, base, c, v);
        else if (c < 2 * D) store_from_float(reinterpret_cast<ST*>(base + L.off_m) + (c - D), v);
        else if (c < 3 * D) store_from_float(reinterpret_cast<ST*>(base + L.off_q) + (c - 2 * D), v);
        else store_from_float(reinterpret_cast<FT*>(base + L.off_feat) + (c - 3 * D), v);
    }
}

// read_entity: whole rows out, in the host array's element type.
template <class ST, class FT, class OT>
__global__ void __launch_bounds__(128)
k_read_rows(const uint8_t* __restrict__ table, RowLayout L, const uint32_t* __restrict__ idx,
            OT* __restrict__ out) {
    const int j = blockIdx.x;
    const size_t row = idx[j];
    const int D = L.d, F = L.f, W = 3 * D + F;
    const uint8_t* base = table + row * L.row_bytes;
    OT* __restrict__ dst = out + (size_t)j * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float v;
        if (c < D) v = load_value<ST>(L, base, c);
        else if (c < 2 * D) v = load_as_float(reinterpret_cast<const ST*>(base + L.off_m) + (c - D));
        else if (c < 3 * D) v = load_as_float(reinterpret_cast<const ST*>(base + L.off_q) + (c - 2 * D));
        else v = load_as_float(reinterpret_cast<const FT*>(base + L.off_feat) + (c - 3 * D));
        store_from_float(dst + c, v);
    }
}

// Plain fp32 row gather with 128-bit accesses (the operator form of fr::Buffer::read,
// src/fructose/fructose.cpp:790-798), used by the operator entry point and the microbench.
template <int V>
__global__ void __launch_bounds__(128)
k_gather_rows(const float* __restrict__ table, size_t width, const uint32_t* __restrict__ idx,
              float* __restrict__ out) {
    const size_t j = blockIdx.x;
    const float* __restrict__ src = table + (size_t)idx[j] * width;
    float* __restrict__ dst = out + j * width;
    if (V == 4) {
        for (size_t c = threadIdx.x * 4; c < width; c += blockDim.x * 4) store4(dst + c, load4(src + c));
    } else {
        for (size_t c = threadIdx.x; c < width; c += blockDim.x) dst[c] = src[c];
    }
}

// y[e] = x[e] rounded to bfloat16 (operands of the bf16 contractions that the host provides).
static __global__ void __launch_bounds__(256) k_to_bf16(const float* __restrict__ x, size_t n, __nv_bfloat16* __restrict__ y) {
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) y[e] = __float2bfloat16_rn(x[e]);
}

// The feature planes of `count` consecutive table rows from `first_row` on (a pass of predict over
// the table), as k_gather_step_rows makes them for the gathered rows of a training step: fp16
// features widened to fp32 into planes.wide, or the lower TF32 plane of fp32 features into planes.lo.
static __global__ void __launch_bounds__(256)
k_table_feature_planes(const uint8_t* __restrict__ table, RowLayout L, uint32_t first_row, int count, FeaturePlanes planes) {
    const int per_row = (int)((L.row_bytes - L.off_feat) >> 4);  // 16-byte chunks of a row's feature segment
    for (size_t u = (size_t)blockIdx.x * blockDim.x + threadIdx.x; u < (size_t)count * per_row; u += (size_t)gridDim.x * blockDim.x) {
        const int r = (int)(u / per_row), c = (int)(u - (size_t)r * per_row);
        const uint4 v = *reinterpret_cast<const uint4*>(table + ((size_t)first_row + r) * L.row_bytes + L.off_feat + (size_t)c * 16);
        if (planes.wide) {
            const int f = c * 8;
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
            const float2 cc = __half22float2(*reinterpret_cast<const __half2*>(&v.z)), d = __half22float2(*reinterpret_cast<const __half2*>(&v.w));
            float* o = planes.wide + (size_t)r * planes.stride + f;
            if (f < (int)planes.stride) *reinterpret_cast<float4*>(o) = make_float4(a.x, a.y, b.x, b.y);
            if (f + 4 < (int)planes.stride) *reinterpret_cast<float4*>(o + 4) = make_float4(cc.x, cc.y, d.x, d.y);
        } else if (planes.lo) {
            const int f = c * 4;
            if (f < (int)planes.stride)
                *reinterpret_cast<float4*>(planes.lo + (size_t)r * planes.stride + f) =
                    tf32_lower4(make_float4(__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w)));
        }
    }
}

// lo[e] = the lower TF32 plane of x[e] (for parameters that the host writes).
static __global__ void __launch_bounds__(256) k_lower_plane(const float* __restrict__ x, size_t n, float* __restrict__ lo) {
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) lo[e] = tf32_lower(x[e]);
}

// Operator form of the duplicate-combining scatter-add: one block per table row, summing
// the rows of its segment in position order.
static __global__ void __launch_bounds__(128)
k_segment_sum_rows(const float* __restrict__ rows, const uint32_t* __restrict__ perm,
                   const uint32_t* __restrict__ off, size_t width, float* __restrict__ out) {
    const size_t r = blockIdx.x;
    for (size_t c = threadIdx.x; c < width; c += blockDim.x) {
        float g = 0.f;
        for (uint32_t q = off[r]; q < off[r + 1]; ++q) g += rows[(size_t)perm[q] * width + c];
        out[r * width + c] = g;
    }
}

// Operator forms of the two activations with their backward (src/pag/pag.cpp:841-864, 888-910).
static __global__ void __launch_bounds__(256)
k_log_sigmoid(const float* __restrict__ x, const float* __restrict__ grad_out, size_t n,
              float* __restrict__ y, float* __restrict__ grad_x) {
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n;
         e += (size_t)gridDim.x * blockDim.x) {
        const float v = x[e];
        y[e] = v > -11.f ? -log1pf(expf(-fmaxf(v, -11.f))) : v;
        grad_x[e] = grad_out[e] / (1.f + expf(fminf(v, 11.f)));
    }
}
static __global__ void __launch_bounds__(256)
k_log_softmax(const float* __restrict__ x, const float* __restrict__ grad_out, int cols,
              float* __restrict__ y, float* __restrict__ grad_x) {
    __shared__ float scratch[8];
    const size_t base = (size_t)blockIdx.x * cols;
    float mx = -INFINITY;
    for (int j = threadIdx.x; j < cols; j += 256) mx = fmaxf(mx, x[base + j]);
    mx = block_max<256>(mx, scratch);
    float sum = 0.f, gsum = 0.f;
    for (int j = threadIdx.x; j < cols; j += 256) {
        sum += expf(x[base + j] - mx);
        gsum += grad_out[base + j];
    }
    sum = block_sum<256>(sum, scratch);
    gsum = block_sum<256>(gsum, scratch);
    const float log_z = logf(sum);
    for (int j = threadIdx.x; j < cols; j += 256) {
        const float logp = x[base + j] - mx - log_z;
        y[base + j] = logp;
        grad_x[base + j] = grad_out[base + j] - gsum * expf(logp);
    }
}

}  // namespace kge
