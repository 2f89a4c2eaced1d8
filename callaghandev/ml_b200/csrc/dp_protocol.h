// The data-parallel train step as a host protocol, free of CUDA and NCCL so that the very same code runs over GPUs
// (engine = the resident trainer, transport = NCCL on a communication stream) and, in the CPU tests, over host
// threads with an in-memory transport where ranks can be made to fail.
//
// The reference trains on one device (TransformerTrainer.cs:217-327); what must survive the split over ranks are its
// rules: gradients and the valid-sequence count are summed over the whole batch before scaling (:313), a failure while
// a batch is processed drops the batch and zeroes every gradient (:298-307), and a non-finite gradient norm zeroes the
// gradients and skips the update (:316-320).
//
// Rules of the protocol:
//   1. Every rank issues the same collectives in the same order, whatever happened locally: one sum per range of the
//      gradient arena, in the order of `ranges`, then one sum of three scalars {loss sum, valid count, failed ranks}.
//      A rank whose local pass failed or had nothing to train still issues every range (over whatever its arena holds)
//      and reports the failure in the third scalar.
//   2. The scalar reduction is the only blocking point and it has a deadline.  A peer that never arrives (it died, or
//      left the protocol) makes it return DP_ERR_TIMEOUT; the transport is then aborted and unusable.
//   3. If any rank reported a failure, every rank discards the step (gradients zeroed, weights untouched) and returns an
//      error: its own on the failing rank, DP_ERR_PEER elsewhere.
//   4. Otherwise every rank runs the identical step on identical reduced gradients, so the non-finite-norm rule
//      (skip and zero) is decided identically everywhere without another exchange.
#pragma once
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <vector>

namespace b200dp {

struct Range {
    int64_t off, count;
};

enum : int {
    DP_OK = 0,
    DP_ERR_PEER = 101,      // another rank failed in this step; the step was discarded everywhere
    DP_ERR_TIMEOUT = 102,   // a peer did not arrive within the deadline; the transport has been aborted
    DP_ERR_COMM = 103,      // the transport reported an error; it has been aborted
    DP_ERR_PROTOCOL = 104,  // the engine announced a range out of order
};

struct StepResult {
    float loss = 0.f, grad_norm = 0.f;
    int valid = 0;
    int local_rc = 0;  // the engine's own status on this rank (0 when the failure was a peer's)
};

// Engine:    int zero_grads();
//            template <class F> int accumulate(F&& on_ready, double* loss_sum, int* valid);
//                   on_ready(off, count) announces that [off, off+count) of the gradient arena is final; returns 0 or an error
//                   the engine should stop on.
//            int apply_step(int global_valid, float* grad_norm);
//            int discard();                                  gradients zeroed after a dropped step
// Transport: int allreduce_range(size_t index, Range r);    asynchronous sum over ranks, ordered after on_ready's point
//            int allreduce_scalars(double* v, int n, int deadline_ms);   blocking; also waits for every range issued before
//            void abort();
template <class Engine, class Transport>
int dp_train_step(Engine& eng, Transport& tr, const std::vector<Range>& ranges, int deadline_ms, StepResult* out) {
    *out = StepResult();
    size_t issued = 0;
    int comm_rc = DP_OK;
    auto on_ready = [&](int64_t off, int64_t count) -> int {
        if (comm_rc != DP_OK) return comm_rc;
        if (issued >= ranges.size() || ranges[issued].off != off || ranges[issued].count != count) return comm_rc = DP_ERR_PROTOCOL;
        comm_rc = tr.allreduce_range(issued, ranges[issued]);
        issued++;
        return comm_rc;
    };
    double loss_sum = 0.0;
    int valid = 0;
    int rc = eng.zero_grads();
    if (rc == DP_OK) rc = eng.accumulate(on_ready, &loss_sum, &valid);
    out->local_rc = rc;
    // rule 1: complete the sequence whatever happened locally
    while (comm_rc == DP_OK && issued < ranges.size()) {
        comm_rc = tr.allreduce_range(issued, ranges[issued]);
        issued++;
    }
    double s[3] = {rc == DP_OK ? loss_sum : 0.0, rc == DP_OK ? (double)valid : 0.0, rc == DP_OK ? 0.0 : 1.0};
    if (comm_rc == DP_OK) comm_rc = tr.allreduce_scalars(s, 3, deadline_ms);
    if (comm_rc != DP_OK) {  // rule 2
        tr.abort();
        eng.discard();
        return comm_rc;
    }
    if (s[2] > 0.5) {  // rule 3
        eng.discard();
        return rc != DP_OK ? rc : DP_ERR_PEER;
    }
    out->valid = (int)std::llround(s[1]);
    out->loss = out->valid > 0 ? (float)(s[0] / s[1]) : 0.f;
    return eng.apply_step(out->valid, &out->grad_norm);  // rule 4
}

// Contiguous shard of sequence indices for one rank (the batch is split by sequence; the first n % world ranks take
// one more).
inline void shard_bounds(int n_seq, int rank, int world, int* lo, int* hi) {
    const int base = n_seq / world, rem = n_seq % world;
    *lo = rank * base + (rank < rem ? rank : rem);
    *hi = *lo + base + (rank < rem ? 1 : 0);
}

}  // namespace b200dp
