// CPU restatement of the reference's sharded training step in C++ / OpenMP, float32.
//
// TEST INFRASTRUCTURE ONLY: the timed CPU baseline of bench.py and a second checker beside
// oracle/step_oracle.py, which pins it: tests/test_oracle_cpu.py compares the two on every
// score / loss variant (test_compiled_restatement_agrees_with_the_pinned_oracle).  It follows the reference's
// Model::trainStep (src/poplar_kge.cpp:664-707): gather rows (:405-410), hidden = value +
// feature.W (:439-467), lookups and exchange (:676-681, src/pag/pag.cpp:915-935), predicted
// tail and score (:488-613; distances as in src/poplar_extensions/l{1,2}distance.codelet.cpp),
// loss (:615-660; guarded log-sigmoid src/pag/pag.cpp:888-910), the backward of each of those
// (src/pag/pag.cpp:685-701, 721-743, 851-860), and Adam in the reference's form
// (src/fructose/frnn.cpp:42-90) on the dense parameters and on the gathered rows (:695-704).
// All shards run in this one process, as in the reference; OpenMP spreads rows over threads.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <utility>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

struct bess_config {
    int n_shard, n_entity, n_relation_type, d, f, batch, a2a;
    int score_fn;  // 0 TransE, 1 DistMult, 2 ComplEx
    int dist_fn;   // 0 L1, 1 L2, 2 dot
    int loss_fn;   // 0 logsigmoid, 1 softmax
    int share_networks;
    float gamma, correction_weight, loss_scale, beta_m, beta_v, epsilon, weight_decay;
};

int bess_oracle_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// The number of OpenMP threads of later steps (a launcher may have set OMP_NUM_THREADS=1 for its
// worker processes; the timed CPU baseline uses all host cores whatever the environment says).
void bess_oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

}  // extern "C"

namespace {

inline float sign_of(float x) { return (float)((0.f < x) - (x < 0.f)); }

void adam(float* x, float* m, float* v, const float* g, size_t n, float alpha, const bess_config& c) {
#pragma omp parallel for schedule(static)
    for (size_t e = 0; e < n; ++e) {
        m[e] = c.beta_m * m[e] + (1.0f - c.beta_m) * g[e];
        v[e] = c.beta_v * v[e] + (1.0f - c.beta_v) * g[e] * g[e];
        x[e] = x[e] - alpha * (m[e] / (std::sqrt(v[e]) + c.epsilon) + c.weight_decay * x[e]);
    }
}

}  // namespace

extern "C" int bess_oracle_step(const bess_config* cfg, float* entity_data, float* relation, float* relation_m,
                                float* relation_v, float* proj, float* proj_m, float* proj_v, unsigned* step,
                                float learning_rate, const uint32_t* remote, const uint32_t* a2a_idx,
                                const uint32_t* head, const uint32_t* rel_idx, const uint32_t* tail, float* loss_out) {
    const bess_config& c = *cfg;
    const int n = c.n_shard, D = c.d, F = c.f, B = c.batch, A = c.a2a, T = n * A, R = B + T;
    const int W = 3 * D + F, n_net = F == 0 ? 0 : (c.share_networks ? 1 : 2);
    const size_t shard_rows = (size_t)c.n_entity * W;
    std::vector<float> hid_h((size_t)n * R * D), hid_t_store(n_net == 2 ? (size_t)n * R * D : 0);
    float* hid_t = n_net == 2 ? hid_t_store.data() : hid_h.data();
    std::vector<float> tails((size_t)n * T * D), d_tails((size_t)n * T * D);
    std::vector<float> d_hid_h((size_t)n * R * D, 0.f), d_hid_t_store(n_net == 2 ? (size_t)n * R * D : 0, 0.f);
    float* d_hid_t = n_net == 2 ? d_hid_t_store.data() : d_hid_h.data();
    std::vector<float> d_rel((size_t)c.n_relation_type * D, 0.f), d_proj((size_t)n_net * F * D, 0.f);

    // 1./2. hidden rows of every shard
    for (int s = 0; s < n; ++s) {
#pragma omp parallel for schedule(static)
        for (int r = 0; r < R; ++r) {
            const float* row = entity_data + s * shard_rows + (size_t)remote[(size_t)s * R + r] * W;
            for (int net = 0; net < std::max(1, n_net); ++net) {
                float* out = (net ? hid_t : hid_h.data()) + ((size_t)s * R + r) * D;
                for (int k = 0; k < D; ++k) out[k] = row[k];
                const float* w = proj + (size_t)net * F * D;
                for (int j = 0; j < F; ++j) {
                    const float x = row[3 * D + j];
                    const float* wj = w + (size_t)j * D;
                    for (int k = 0; k < D; ++k) out[k] += x * wj[k];
                }
            }
        }
    }
    // exchange: tails[dst][src*A + j] = hid_t[src][a2a[src][dst][j]]
    for (int src = 0; src < n; ++src)
        for (int dst = 0; dst < n; ++dst)
            for (int j = 0; j < A; ++j) {
                const uint32_t r = a2a_idx[((size_t)src * n + dst) * A + j];
                std::memcpy(&tails[((size_t)dst * T + (size_t)src * A + j) * D], hid_t + ((size_t)src * R + r) * D,
                            sizeof(float) * D);
            }

    const float w_neg = (0.5f * T) / (T - 1), w_pos = 0.5f * T;
    const float normaliser = c.loss_fn == 0 ? (float)(n * B * A * n) : (float)(n * B);
    float shift = 0.f;
    if (c.loss_fn == 1 && c.correction_weight != 0.f) {
        const float correction =
            (float)(std::log((double)((unsigned)c.n_entity * (unsigned)n - 1)) - std::log((double)(T - 1)));
        shift = c.correction_weight * correction;
    }
    const float grad_scale = c.loss_scale / normaliser;
    const int half = D / 2;

    for (int s = 0; s < n; ++s) {
        std::vector<float> pred((size_t)B * D), raw((size_t)B * T), coeff((size_t)B * T), d_pred((size_t)B * D);
        std::vector<float> row_loss(B);
        const float* tl = &tails[(size_t)s * T * D];
        // 3. predicted tails and scores, 4. loss with its gradient
#pragma omp parallel for schedule(static)
        for (int i = 0; i < B; ++i) {
            const float* h = hid_h.data() + ((size_t)s * R + head[(size_t)s * B + i]) * D;
            const float* r = relation + (size_t)rel_idx[(size_t)s * B + i] * D;
            float* p = &pred[(size_t)i * D];
            if (c.score_fn == 0) for (int k = 0; k < D; ++k) p[k] = h[k] + r[k];
            else if (c.score_fn == 1) for (int k = 0; k < D; ++k) p[k] = h[k] * r[k];
            else for (int k = 0; k < half; ++k) {
                p[k] = h[k] * r[k] - h[k + half] * r[k + half];
                p[k + half] = h[k] * r[k + half] + h[k + half] * r[k];
            }
            float* rw = &raw[(size_t)i * T];
            for (int j = 0; j < T; ++j) {
                const float* t = tl + (size_t)j * D;
                float acc = 0.f;
                if (c.dist_fn == 0) for (int k = 0; k < D; ++k) acc += std::fabs(p[k] - t[k]);
                else if (c.dist_fn == 1) { for (int k = 0; k < D; ++k) { const float df = p[k] - t[k]; acc += df * df; } acc = std::sqrt(acc); }
                else for (int k = 0; k < D; ++k) acc += p[k] * t[k];
                rw[j] = acc;
            }
            const int lab = (int)tail[(size_t)s * B + i];
            float* cf = &coeff[(size_t)i * T];
            auto score_of = [&](int j) { return c.score_fn == 0 ? c.gamma - rw[j] : rw[j]; };
            if (c.loss_fn == 1) {
                float mx = -INFINITY;
                for (int j = 0; j < T; ++j) mx = std::max(mx, score_of(j) + (j == lab ? 0.f : shift));
                float sum = 0.f;
                for (int j = 0; j < T; ++j) sum += std::exp(score_of(j) + (j == lab ? 0.f : shift) - mx);
                const float log_z = std::log(sum);
                for (int j = 0; j < T; ++j) {
                    const float logp = score_of(j) + (j == lab ? 0.f : shift) - mx - log_z;
                    cf[j] = grad_scale * (std::exp(logp) - (j == lab ? 1.f : 0.f));
                    if (j == lab) row_loss[i] = -logp;
                }
            } else {
                float part = 0.f;
                for (int j = 0; j < T; ++j) {
                    const bool pos = j == lab;
                    const float w = pos ? w_pos : w_neg, x = pos ? score_of(j) : -score_of(j);
                    part += w * (x > -11.f ? -std::log1p(std::exp(-std::max(x, -11.f))) : x);
                    const float dx = (-w * grad_scale) / (1.f + std::exp(std::min(x, 11.f)));
                    cf[j] = pos ? dx : -dx;
                }
                row_loss[i] = -part;
            }
            for (int j = 0; j < T; ++j) {  // d loss / d raw, with the L2 division folded in
                float g = c.score_fn == 0 ? -cf[j] : cf[j];
                if (c.dist_fn == 1) g = rw[j] == 0.f ? 0.f : g / rw[j];
                cf[j] = g;
            }
        }
        float total = 0.f;
        for (int i = 0; i < B; ++i) total += row_loss[i];
        loss_out[s] = total / normaliser;
        // 5. score backward
#pragma omp parallel for schedule(static)
        for (int i = 0; i < B; ++i) {
            const float* p = &pred[(size_t)i * D];
            float* dp = &d_pred[(size_t)i * D];
            for (int k = 0; k < D; ++k) dp[k] = 0.f;
            for (int j = 0; j < T; ++j) {
                const float g = coeff[(size_t)i * T + j];
                const float* t = tl + (size_t)j * D;
                if (c.dist_fn == 0) for (int k = 0; k < D; ++k) dp[k] += g * sign_of(p[k] - t[k]);
                else if (c.dist_fn == 1) for (int k = 0; k < D; ++k) dp[k] += g * (p[k] - t[k]);
                else for (int k = 0; k < D; ++k) dp[k] += g * t[k];
            }
        }
#pragma omp parallel for schedule(static)
        for (int j = 0; j < T; ++j) {
            const float* t = tl + (size_t)j * D;
            float* dt = &d_tails[((size_t)s * T + j) * D];
            for (int k = 0; k < D; ++k) dt[k] = 0.f;
            for (int i = 0; i < B; ++i) {
                const float g = coeff[(size_t)i * T + j];
                const float* p = &pred[(size_t)i * D];
                if (c.dist_fn == 0) for (int k = 0; k < D; ++k) dt[k] += g * sign_of(t[k] - p[k]);
                else if (c.dist_fn == 1) for (int k = 0; k < D; ++k) dt[k] += g * (t[k] - p[k]);
                else for (int k = 0; k < D; ++k) dt[k] += g * p[k];
            }
        }
        // head / relation gradients, scattered in position order (duplicates accumulate)
        for (int i = 0; i < B; ++i) {
            const uint32_t hrow = head[(size_t)s * B + i], rrow = rel_idx[(size_t)s * B + i];
            const float* h = hid_h.data() + ((size_t)s * R + hrow) * D;
            const float* r = relation + (size_t)rrow * D;
            const float* dp = &d_pred[(size_t)i * D];
            float* dh = &d_hid_h[((size_t)s * R + hrow) * D];
            float* dr = &d_rel[(size_t)rrow * D];
            if (c.score_fn == 0) for (int k = 0; k < D; ++k) { dh[k] += dp[k]; dr[k] += dp[k]; }
            else if (c.score_fn == 1) for (int k = 0; k < D; ++k) { dh[k] += dp[k] * r[k]; dr[k] += dp[k] * h[k]; }
            else for (int k = 0; k < half; ++k) {
                const float gr = dp[k], gi = dp[k + half];
                dh[k] += gr * r[k] + gi * r[k + half];
                dh[k + half] += -gr * r[k + half] + gi * r[k];
                dr[k] += gr * h[k] + gi * h[k + half];
                dr[k + half] += -gr * h[k + half] + gi * h[k];
            }
        }
    }
    // exchange backward + tail lookups backward
    for (int src = 0; src < n; ++src)
        for (int dst = 0; dst < n; ++dst)
            for (int j = 0; j < A; ++j) {
                const uint32_t r = a2a_idx[((size_t)src * n + dst) * A + j];
                const float* g = &d_tails[((size_t)dst * T + (size_t)src * A + j) * D];
                float* out = d_hid_t + ((size_t)src * R + r) * D;
                for (int k = 0; k < D; ++k) out[k] += g[k];
            }
    // projection backward, summed over shards
    for (int net = 0; net < n_net; ++net) {
        const float* dh = net ? d_hid_t : d_hid_h.data();
        float* dw = &d_proj[(size_t)net * F * D];
#pragma omp parallel for schedule(static)
        for (int j = 0; j < F; ++j)
            for (int s = 0; s < n; ++s)
                for (int r = 0; r < R; ++r) {
                    const float x = entity_data[s * shard_rows + (size_t)remote[(size_t)s * R + r] * W + 3 * D + j];
                    const float* g = dh + ((size_t)s * R + r) * D;
                    for (int k = 0; k < D; ++k) dw[(size_t)j * D + k] += x * g[k];
                }
    }
    // update
    *step += 1;
    const float t = (float)*step;
    const float alpha = (std::sqrt(1.0f - std::pow(c.beta_v, t)) / (1.0f - std::pow(c.beta_m, t))) * learning_rate;
    adam(relation, relation_m, relation_v, d_rel.data(), d_rel.size(), alpha, c);
    if (n_net) adam(proj, proj_m, proj_v, d_proj.data(), d_proj.size(), alpha, c);
    for (int s = 0; s < n; ++s) {
        // Slots that repeat a row (the zero padding at the end of `remote`) were all gathered
        // from the same copy, so their write-backs are identical: the first slot does it.
        std::vector<std::pair<uint32_t, int>> order(R);
        for (int r = 0; r < R; ++r) order[r] = {remote[(size_t)s * R + r], r};
        std::sort(order.begin(), order.end());
        std::vector<char> first(R, 0);
        for (int q = 0; q < R; ++q) first[order[q].second] = q == 0 || order[q - 1].first != order[q].first;
#pragma omp parallel for schedule(static)
        for (int r = 0; r < R; ++r) {
            if (!first[r]) continue;
            float* row = entity_data + s * shard_rows + (size_t)remote[(size_t)s * R + r] * W;
            const float* gh = &d_hid_h[((size_t)s * R + r) * D];
            const float* gt = n_net == 2 ? d_hid_t + ((size_t)s * R + r) * D : nullptr;
            for (int k = 0; k < D; ++k) {
                const float g = gh[k] + (gt ? gt[k] : 0.f);
                float v = row[2 * D + k] * row[2 * D + k];
                const float m = c.beta_m * row[D + k] + (1.0f - c.beta_m) * g;
                v = c.beta_v * v + (1.0f - c.beta_v) * g * g;
                row[k] = row[k] - alpha * (m / (std::sqrt(v) + c.epsilon) + c.weight_decay * row[k]);
                row[D + k] = m;
                row[2 * D + k] = std::sqrt(v);
            }
        }
    }
    return 0;
}
