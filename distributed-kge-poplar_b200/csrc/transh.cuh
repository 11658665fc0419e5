// TransH (src/poplar_kge.cpp:539-565): every relation has a translation row and a hyperplane
// normal; heads and tails are projected onto the hyperplane before the translation is compared,
//   n_i  = w_i / |w_i|                                  (w = relation_normal[relation_i])
//   pt_i = h_i - n_i (n_i . h_i) + r_i                  (the predicted tail)
//   e_ijk = pt_ik - (t_jk - n_ik (n_i . t_j))
//   score_ij = gamma - sum_k |e_ijk|                     (always the L1 form, whatever model.distance_fn says).
// Four kernels: the predicted tails of a batch, the pairwise distances with the two [B, T]
// matrices the backward needs (s_ij = n_i . t_j and u_ij = sum_k sign(e_ijk) n_ik), the gradients
// of the distance with respect to pt, n and the tails, and the backward of the prediction down to
// the head rows, the translation rows and the raw normals.  Plain FP32-pipe kernels: a row of the
// output per block, the other index walked in order, so every sum has a fixed order.
#pragma once

#include "kernels.cuh"

namespace kge {

// pred[i] = pt_i, nrm[i] = n_i.  One block of 64 threads per triple.
static __global__ void __launch_bounds__(64)
k_transh_predict(const float* __restrict__ hid_h, const uint32_t* __restrict__ head, const uint32_t* __restrict__ relation,
                 const float* __restrict__ rel_table, const float* __restrict__ normal_table, float* __restrict__ pred,
                 float* __restrict__ nrm, int D) {
    grid_dependency_sync();
    __shared__ float scratch[2];
    const int i = blockIdx.x;
    const float* __restrict__ h = hid_h + (size_t)head[i] * D;
    const float* __restrict__ r = rel_table + (size_t)relation[i] * D;
    const float* __restrict__ w = normal_table + (size_t)relation[i] * D;
    float ww = 0.f, wh = 0.f;
    for (int k = threadIdx.x; k < D; k += 64) {
        ww += w[k] * w[k];
        wh += w[k] * h[k];
    }
    ww = block_sum<64>(ww, scratch);
    wh = block_sum<64>(wh, scratch);
    const float inv = 1.f / sqrtf(ww);
    const float nh = wh * inv;  // n . h
    for (int k = threadIdx.x; k < D; k += 64) {
        const float n = w[k] * inv;
        nrm[(size_t)i * D + k] = n;
        pred[(size_t)i * D + k] = h[k] - n * nh + r[k];
    }
}

// raw[i, j] = sum_k |e_ijk|, and (when asked for) S[i, j] = n_i . t_j, U[i, j] = sum_k sign(e_ijk) n_ik.
// A block holds 16 query rows (pt and n) in shared memory and walks the tails; a warp per tail, the
// lanes split k.  `y_index` (optional) names the tail rows (predict scores chunks of the table's
// hidden rows in place).
constexpr int kTranshRows = 16;

static __global__ void __launch_bounds__(256)
k_transh_score(const float* __restrict__ pt, const float* __restrict__ nrm, const float* __restrict__ tails, float* __restrict__ raw,
               float* __restrict__ S, float* __restrict__ U, int B, int T, int D, ExchangeSync sync) {
    grid_dependency_sync();
    exchange_wait(sync, XCHG_TAILS);  // the tails come from the other processes
    extern __shared__ float smem[];
    float* sp = smem;                       // [kTranshRows][D]
    float* sn = smem + kTranshRows * D;     // [kTranshRows][D]
    const int i0 = blockIdx.x * kTranshRows, rows = min(kTranshRows, B - i0);
    for (int idx = threadIdx.x; idx < rows * D; idx += 256) {
        sp[idx] = pt[(size_t)i0 * D + idx];
        sn[idx] = nrm[(size_t)i0 * D + idx];
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int j = blockIdx.y * 8 + warp; j < T; j += gridDim.y * 8) {
        const float* __restrict__ t = tails + (size_t)j * D;
        for (int a = 0; a < rows; ++a) {
            float s = 0.f;
            for (int k = lane; k < D; k += 32) s += sn[a * D + k] * t[k];
            s = warp_sum(s);
            float dist = 0.f, u = 0.f;
            for (int k = lane; k < D; k += 32) {
                const float n = sn[a * D + k], e = sp[a * D + k] - t[k] + n * s;
                dist += fabsf(e);
                u += e > 0.f ? n : (e < 0.f ? -n : 0.f);
            }
            dist = warp_sum(dist);
            u = warp_sum(u);
            if (lane == 0) {
                const size_t o = (size_t)(i0 + a) * T + j;
                raw[o] = dist;
                if (S) S[o] = s;
                if (U) U[o] = u;
            }
        }
    }
}

// Gradients of the distances times C [B, T] (C = d loss / d raw):
//   rows i (blockIdx.x < B):  d_pt_ik = sum_j C_ij sg_ijk,   d_n_ik = sum_j C_ij (sg_ijk S_ij + U_ij t_jk)
//   rows j (the others):      d_t_jk  = sum_i C_ij (-sg_ijk + U_ij n_ik), stored to the shard that owns tail j
// with sg_ijk = sign(pt_ik - t_jk + n_ik S_ij) recomputed.  One block per output row, a thread per column.
static __global__ void __launch_bounds__(128)
k_transh_bwd(const float* __restrict__ pt, const float* __restrict__ nrm, const float* __restrict__ tails, const float* __restrict__ C,
             const float* __restrict__ S, const float* __restrict__ U, float* __restrict__ d_pt, float* __restrict__ d_n,
             float* const* __restrict__ d_tail_blocks, int block_rows, int B, int T, int D) {
    grid_dependency_sync();
    const int m = blockIdx.x;
    if (m < B) {
        const int i = m;
        for (int k = threadIdx.x; k < D; k += 128) {
            const float p = pt[(size_t)i * D + k], n = nrm[(size_t)i * D + k];
            float acc_p = 0.f, acc_n = 0.f;
            for (int j = 0; j < T; ++j) {
                const size_t o = (size_t)i * T + j;
                const float c = C[o], s = S[o], u = U[o], t = tails[(size_t)j * D + k];
                const float e = p - t + n * s;
                const float sg = e > 0.f ? 1.f : (e < 0.f ? -1.f : 0.f);
                acc_p += c * sg;
                acc_n += c * (sg * s + u * t);
            }
            d_pt[(size_t)i * D + k] = acc_p;
            d_n[(size_t)i * D + k] = acc_n;
        }
        return;
    }
    const int j = m - B;
    float* __restrict__ dst = d_tail_blocks[j / block_rows] + (size_t)(j % block_rows) * D;
    for (int k = threadIdx.x; k < D; k += 128) {
        const float t = tails[(size_t)j * D + k];
        float acc = 0.f;
        for (int i = 0; i < B; ++i) {
            const size_t o = (size_t)i * T + j;
            const float c = C[o], s = S[o], u = U[o], n = nrm[(size_t)i * D + k];
            const float e = pt[(size_t)i * D + k] - t + n * s;
            const float sg = e > 0.f ? 1.f : (e < 0.f ? -1.f : 0.f);
            acc += c * (u * n - sg);
        }
        dst[k] = acc;
    }
}

// Backward of k_transh_predict for triple i:
//   d_head = d_pt - n (n . d_pt),   d_relrow = d_pt,
//   d_n (total) = d_n - (n . h) d_pt - h (n . d_pt),   d_normrow = (d_n - n (n . d_n)) / |w|.
static __global__ void __launch_bounds__(64)
k_transh_pred_bwd(const float* __restrict__ d_pt, const float* __restrict__ d_n, const float* __restrict__ hid_h,
                  const uint32_t* __restrict__ head, const uint32_t* __restrict__ relation, const float* __restrict__ normal_table,
                  const float* __restrict__ nrm, float* __restrict__ d_head, float* __restrict__ d_relrow,
                  float* __restrict__ d_normrow, int D) {
    grid_dependency_sync();
    __shared__ float scratch[2];
    const int i = blockIdx.x;
    const float* __restrict__ h = hid_h + (size_t)head[i] * D;
    const float* __restrict__ w = normal_table + (size_t)relation[i] * D;
    const size_t o = (size_t)i * D;
    float ww = 0.f, nh = 0.f, ndp = 0.f;
    for (int k = threadIdx.x; k < D; k += 64) {
        ww += w[k] * w[k];
        nh += nrm[o + k] * h[k];
        ndp += nrm[o + k] * d_pt[o + k];
    }
    ww = block_sum<64>(ww, scratch);
    nh = block_sum<64>(nh, scratch);
    ndp = block_sum<64>(ndp, scratch);
    float ndn = 0.f;  // n . (total d_n)
    for (int k = threadIdx.x; k < D; k += 64) ndn += nrm[o + k] * (d_n[o + k] - nh * d_pt[o + k] - h[k] * ndp);
    ndn = block_sum<64>(ndn, scratch);
    const float inv = 1.f / sqrtf(ww);
    for (int k = threadIdx.x; k < D; k += 64) {
        const float n = nrm[o + k], dp = d_pt[o + k];
        d_head[o + k] = dp - n * ndp;
        d_relrow[o + k] = dp;
        d_normrow[o + k] = (d_n[o + k] - nh * dp - h[k] * ndp - n * ndn) * inv;
    }
}

}  // namespace kge
