// CPU harness for the data-parallel step protocol (callaghandev/ml_b200/csrc/dp_protocol.h): the product's own
// dp_train_step runs here over host threads, with a toy engine (a gradient vector filled from rank-dependent values,
// the scale / norm / clip / update rules of the fused step) and an in-memory transport in which ranks can be made to
// fail.  Built by tests/test_dp_protocol.py with g++; nothing here touches a GPU.
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

#include "../callaghandev/ml_b200/csrc/dp_protocol.h"

using namespace b200dp;

namespace {

struct Shared {
    int world;
    std::mutex mu;
    std::condition_variable cv;
    std::vector<std::vector<double>> range_sum;  // per range
    std::vector<int> range_arrived;
    double scal[3] = {0, 0, 0};
    int scal_arrived = 0;
    bool aborted = false;
};

enum Scenario { HEALTHY = 0, ENGINE_ERROR = 1, RANK_ABSENT = 2, NONFINITE_SHARD = 3, EMPTY_SHARD = 4, OUT_OF_ORDER = 5 };

struct ToyEngine {
    int rank, scenario, bad_rank;
    const std::vector<Range>& ranges;
    std::vector<float>&w, &g;
    float lr, thr;
    int skipped = 0;

    int zero_grads() { std::fill(g.begin(), g.end(), 0.f); return DP_OK; }
    template <class F>
    int accumulate(F&& on_ready, double* loss_sum, int* valid) {
        const bool bad = rank == bad_rank;
        if (scenario == EMPTY_SHARD && bad) { *loss_sum = 0; *valid = 0; return DP_OK; }  // nothing to train, nothing announced
        for (size_t i = 0; i < g.size(); i++) g[i] = 0.001f * (float)((i * 7 + (size_t)rank * 13) % 29) - 0.01f;  // "unscaled gradient sum of the shard"
        if (scenario == NONFINITE_SHARD && bad) g[ranges[1].off + 3] = INFINITY;
        size_t n = ranges.size();
        for (size_t r = 0; r < n; r++) {
            if (scenario == ENGINE_ERROR && bad && r == 1) return 77;  // fails after announcing one range
            size_t idx = (scenario == OUT_OF_ORDER && bad && r == 0) ? 1 : r;
            int rc = on_ready(ranges[idx].off, ranges[idx].count);
            if (rc != DP_OK) return rc;
        }
        *loss_sum = 1.5 * (rank + 1);
        *valid = rank + 1;
        return DP_OK;
    }
    int apply_step(int global_valid, float* grad_norm) {
        if (global_valid <= 0) { *grad_norm = 0.f; return DP_OK; }
        double ss = 0;
        for (float& x : g) { x *= 1.0f / (float)global_valid; ss += (double)x * x; }
        const float norm = (float)std::sqrt(ss);
        *grad_norm = norm;
        if (!std::isfinite(norm)) { std::fill(g.begin(), g.end(), 0.f); skipped = 1; return DP_OK; }  // TransformerTrainer.cs:316-320
        const float c = norm > thr ? thr / norm : 1.f;
        for (size_t i = 0; i < g.size(); i++) { g[i] *= c; w[i] -= lr * g[i]; }
        return DP_OK;
    }
    int discard() { std::fill(g.begin(), g.end(), 0.f); return DP_OK; }
};

struct ThreadTransport {
    Shared& sh;
    std::vector<float>& g;
    const std::vector<Range>& ranges;
    std::vector<size_t> mine;  // ranges this rank has contributed to

    int allreduce_range(size_t idx, Range r) {
        std::lock_guard<std::mutex> lock(sh.mu);
        if (sh.aborted) return DP_ERR_COMM;
        auto& s = sh.range_sum[idx];
        for (int64_t i = 0; i < r.count; i++) s[(size_t)i] += g[(size_t)(r.off + i)];
        sh.range_arrived[idx]++;
        mine.push_back(idx);
        return DP_OK;
    }
    int allreduce_scalars(double* v, int n, int deadline_ms) {
        std::unique_lock<std::mutex> lock(sh.mu);
        for (int i = 0; i < n; i++) sh.scal[i] += v[i];
        sh.scal_arrived++;
        sh.cv.notify_all();
        const auto until = std::chrono::steady_clock::now() + std::chrono::milliseconds(deadline_ms);
        if (!sh.cv.wait_until(lock, until, [&] { return sh.scal_arrived == sh.world || sh.aborted; })) return DP_ERR_TIMEOUT;
        if (sh.aborted) return DP_ERR_COMM;
        for (int i = 0; i < n; i++) v[i] = sh.scal[i];
        for (size_t idx : mine)
            for (int64_t i = 0; i < ranges[idx].count; i++) g[(size_t)(ranges[idx].off + i)] = (float)sh.range_sum[idx][(size_t)i];
        return DP_OK;
    }
    void abort() {
        std::lock_guard<std::mutex> lock(sh.mu);
        sh.aborted = true;
        sh.cv.notify_all();
    }
};

}  // namespace

// Runs one step on `world` ranks.  Per rank r: rc[r], valid[r], loss[r], norm[r], elapsed_ms[r]; w_out / g_out are
// [world][total].  The gradient arena has n_ranges equal ranges announced last to first (like the trainer's).
extern "C" __attribute__((visibility("default"))) int dp_sim_run(int world, int total, int n_ranges, int scenario, int bad_rank, int deadline_ms,
                                                                  int* rc, int* valid, float* loss, float* norm, float* elapsed_ms, float* w_out,
                                                                  float* g_out, int* skipped) {
    std::vector<Range> ranges;
    const int per = total / n_ranges;
    for (int r = n_ranges - 1; r >= 0; r--) ranges.push_back(Range{(int64_t)r * per, r == n_ranges - 1 ? (int64_t)total - (int64_t)r * per : (int64_t)per});
    Shared sh;
    sh.world = world;
    sh.range_sum.resize(ranges.size());
    for (size_t i = 0; i < ranges.size(); i++) sh.range_sum[i].assign((size_t)ranges[i].count, 0.0);
    sh.range_arrived.assign(ranges.size(), 0);
    std::vector<std::vector<float>> W((size_t)world, std::vector<float>((size_t)total)), G((size_t)world, std::vector<float>((size_t)total, 0.f));
    for (int r = 0; r < world; r++)
        for (int i = 0; i < total; i++) W[(size_t)r][(size_t)i] = 0.01f * (float)(i % 17);
    std::vector<std::thread> th;
    for (int r = 0; r < world; r++) {
        rc[r] = -1; valid[r] = 0; loss[r] = 0; norm[r] = 0; elapsed_ms[r] = 0; skipped[r] = 0;
        if (scenario == RANK_ABSENT && r == bad_rank) continue;  // this rank never joins the step (it died before its first collective)
        th.emplace_back([&, r] {
            ToyEngine eng{r, scenario, bad_rank, ranges, W[(size_t)r], G[(size_t)r], 0.1f, 0.05f};
            ThreadTransport tr{sh, G[(size_t)r], ranges, {}};
            StepResult res;
            const auto t0 = std::chrono::steady_clock::now();
            rc[r] = dp_train_step(eng, tr, ranges, deadline_ms, &res);
            elapsed_ms[r] = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
            valid[r] = res.valid; loss[r] = res.loss; norm[r] = res.grad_norm; skipped[r] = eng.skipped;
        });
    }
    for (auto& t : th) t.join();
    for (int r = 0; r < world; r++) {
        memcpy(w_out + (size_t)r * total, W[(size_t)r].data(), sizeof(float) * (size_t)total);
        memcpy(g_out + (size_t)r * total, G[(size_t)r].data(), sizeof(float) * (size_t)total);
    }
    return 0;
}
