// C ABI, part D: data-parallel training behind the library boundary.  The host protocol lives in dp_protocol.h (free of
// CUDA so that the CPU tests run the same code over host threads); this file supplies its two halves for real GPUs:
// the engine (the resident trainer of lm.cu, reached through its public entry points) and the transport (NCCL on a
// communication stream, loaded at run time so that the host needs no NCCL binding and the library no link-time
// dependency).  No TMA multicast, no peer-memory loads: the only cross-GPU traffic is NCCL's.
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstring>
#include <functional>
#include <thread>

#include "common.h"
#include "dp_protocol.h"

using namespace b200;

namespace {

// ---------------------------------------------------------------------------------------------------- NCCL at run time
struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommInitAll)(ncclComm_t*, int, const int*) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;  // optional (NCCL >= 2.14)
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    std::string error;
};

std::mutex g_nccl_mu;
std::string g_nccl_path;
// CTAs the communicators may use.  The all-reduce of a step moves 4 bytes per parameter in the shadow of a backward pass
// that lasts tens of milliseconds, so it needs a small fraction of NVLink's bandwidth; what it costs is the SMs its
// kernels occupy beside the GEMMs while they wait for peers, against the length of the tail that no backward hides.
// Eight GPUs, c5, ms per step: NCCL's own choice 96.2; 4 CTAs 97.7 (the tail grows to 4 ms); 8 CTAs 93.9-94.2;
// 16 CTAs 92.9 (same GEMM rate as with 8, 1.1 ms of tail).
int g_nccl_max_ctas = 16;

// ncclCommInitRank, with the CTA limit where the library supports per-communicator configuration
ncclResult_t comm_init_rank(NcclApi* api, ncclComm_t* comm, int world, ncclUniqueId id, int rank) {
    if (api->CommInitRankConfig && g_nccl_max_ctas > 0) {
        ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
        cfg.maxCTAs = g_nccl_max_ctas;
        return api->CommInitRankConfig(comm, world, id, rank, &cfg);
    }
    return api->CommInitRank(comm, world, id, rank);
}
NcclApi* g_nccl = nullptr;

NcclApi* nccl_api(std::string* why) {
    std::lock_guard<std::mutex> lock(g_nccl_mu);
    if (g_nccl) return g_nccl;
    void* h = nullptr;
    if (!g_nccl_path.empty()) h = dlopen(g_nccl_path.c_str(), RTLD_NOW | RTLD_GLOBAL);
    // a copy that the process has already loaded (for instance the one a host framework ships) comes first: two
    // different NCCL builds in one process would each bring their own proxy threads and tuning
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) {
        if (why) *why = std::string("libnccl.so.2 could not be loaded: ") + (dlerror() ? dlerror() : "unknown error");
        return nullptr;
    }
    NcclApi* a = new NcclApi();
    a->handle = h;
    bool ok = true;
    auto sym = [&](const char* name) { void* p = dlsym(h, name); if (!p) { ok = false; if (why) *why = std::string("missing NCCL symbol ") + name; } return p; };
    a->GetUniqueId = (decltype(a->GetUniqueId))sym("ncclGetUniqueId");
    a->CommInitRank = (decltype(a->CommInitRank))sym("ncclCommInitRank");
    a->CommInitAll = (decltype(a->CommInitAll))sym("ncclCommInitAll");
    a->CommInitRankConfig = (decltype(a->CommInitRankConfig))dlsym(h, "ncclCommInitRankConfig");
    a->GroupStart = (decltype(a->GroupStart))dlsym(h, "ncclGroupStart");
    a->GroupEnd = (decltype(a->GroupEnd))dlsym(h, "ncclGroupEnd");
    a->CommDestroy = (decltype(a->CommDestroy))sym("ncclCommDestroy");
    a->CommAbort = (decltype(a->CommAbort))sym("ncclCommAbort");
    a->CommGetAsyncError = (decltype(a->CommGetAsyncError))sym("ncclCommGetAsyncError");
    a->AllReduce = (decltype(a->AllReduce))sym("ncclAllReduce");
    a->Broadcast = (decltype(a->Broadcast))sym("ncclBroadcast");
    a->GetErrorString = (decltype(a->GetErrorString))sym("ncclGetErrorString");
    if (!ok) { delete a; return nullptr; }
    g_nccl = a;
    return a;
}

}  // namespace

struct b200_dp {
    b200_lm* lm = nullptr;
    b200_ctx* ctx = nullptr;
    NcclApi* api = nullptr;
    int rank = 0, world = 1;
    ncclComm_t comm = nullptr;
    bool dead = false;  // the communicator was aborted: only b200_dp_destroy is allowed
    cudaStream_t comm_stream = nullptr;
    std::vector<b200dp::Range> ranges;
    double* scal_dev = nullptr;
    double* scal_host = nullptr;  // pinned
    cudaEvent_t ev_done = nullptr, ev_bwd_end = nullptr, ev_resume = nullptr, ev_comm_first = nullptr, ev_comm_last = nullptr, ev_local = nullptr;
    int deadline_ms = 30000;
    float timings[2] = {0.f, 0.f};
    // state of the step in flight
    void* cur_event = nullptr;  // the event the trainer recorded for the range it is announcing (NULL: none, record one)
    std::function<int(int64_t, int64_t)> on_ready;
    bool first_range = true;
};

namespace {

int dp_fail(b200_dp* dp, int code, const char* what, ncclResult_t r) {
    return fail(dp->ctx, code, "%s: %s", what, dp->api && dp->api->GetErrorString ? dp->api->GetErrorString(r) : "NCCL error");
}

int map_status(int rc) {
    switch (rc) {
        case b200dp::DP_ERR_PEER: return B200_ERR_PEER;
        case b200dp::DP_ERR_TIMEOUT: return B200_ERR_TIMEOUT;
        case b200dp::DP_ERR_COMM: return B200_ERR_NCCL;
        case b200dp::DP_ERR_PROTOCOL: return B200_ERR_NCCL;
        default: return rc;
    }
}

void ready_trampoline(void* user, int64_t off, int64_t count, void* event) {
    b200_dp* dp = (b200_dp*)user;
    dp->cur_event = event;
    if (dp->on_ready) dp->on_ready(off, count);
    dp->cur_event = nullptr;
}

// The two halves the protocol is instantiated with.
struct LmEngine {
    b200_dp* dp;
    std::function<int(float*, int32_t*)> local;  // this rank's accumulate call
    float lr; int use_clip; float thr; int do_step;

    int zero_grads() { return b200_lm_zero_grads(dp->lm); }
    template <class F>
    int accumulate(F&& on_ready, double* loss_sum, int* valid) {
        dp->on_ready = on_ready;
        float ls = 0.f;
        int32_t vc = 0;
        int rc = local(&ls, &vc);
        dp->on_ready = nullptr;
        cudaEventRecord(dp->ev_bwd_end, dp->ctx->stream);  // the compute stream's own work of this step ends here
        *loss_sum = ls;
        *valid = vc;
        return rc;
    }
    int apply_step(int global_valid, float* grad_norm) { return b200_lm_apply_step(dp->lm, global_valid, lr, use_clip, thr, do_step, grad_norm); }
    int discard() { return b200_lm_zero_grads(dp->lm); }
};

struct NcclTransport {
    b200_dp* dp;

    int allreduce_range(size_t index, b200dp::Range r) {
        cudaEvent_t ev = (cudaEvent_t)dp->cur_event;
        if (!ev) {  // announced by the protocol itself (nothing local, or the local pass stopped early): order after what is enqueued now
            ev = dp->ev_local;
            if (cudaEventRecord(ev, dp->ctx->stream) != cudaSuccess) return b200dp::DP_ERR_COMM;
        }
        if (cudaStreamWaitEvent(dp->comm_stream, ev, 0) != cudaSuccess) return b200dp::DP_ERR_COMM;
        if (dp->first_range) { cudaEventRecord(dp->ev_comm_first, dp->comm_stream); dp->first_range = false; }
        float* g = b200_lm_grads_device(dp->lm) + r.off;
        ncclResult_t res = dp->api->AllReduce(g, g, (size_t)r.count, ncclFloat, ncclSum, dp->comm, dp->comm_stream);
        if (res != ncclSuccess) { dp_fail(dp, B200_ERR_NCCL, "ncclAllReduce of a gradient range failed", res); return b200dp::DP_ERR_COMM; }
        // the reduced range is final: its sum of squares (for the one-pass step) follows on the same stream
        if (lm_sumsq_range(dp->lm, (int)index, dp->comm_stream) != B200_OK) return b200dp::DP_ERR_COMM;
        return b200dp::DP_OK;
    }

    int allreduce_scalars(double* v, int n, int deadline_ms) {
        for (int i = 0; i < n; i++) dp->scal_host[i] = v[i];
        cudaEventRecord(dp->ev_comm_last, dp->comm_stream);  // end of the gradient reductions
        if (cudaMemcpyAsync(dp->scal_dev, dp->scal_host, sizeof(double) * n, cudaMemcpyHostToDevice, dp->comm_stream) != cudaSuccess) return b200dp::DP_ERR_COMM;
        ncclResult_t res = dp->api->AllReduce(dp->scal_dev, dp->scal_dev, (size_t)n, ncclDouble, ncclSum, dp->comm, dp->comm_stream);
        if (res != ncclSuccess) { dp_fail(dp, B200_ERR_NCCL, "ncclAllReduce of the step scalars failed", res); return b200dp::DP_ERR_COMM; }
        if (cudaMemcpyAsync(dp->scal_host, dp->scal_dev, sizeof(double) * n, cudaMemcpyDeviceToHost, dp->comm_stream) != cudaSuccess) return b200dp::DP_ERR_COMM;
        if (cudaEventRecord(dp->ev_done, dp->comm_stream) != cudaSuccess) return b200dp::DP_ERR_COMM;
        // the one blocking point: poll with a deadline instead of synchronising, and watch the communicator's health
        const auto t0 = std::chrono::steady_clock::now();
        for (;;) {
            cudaError_t q = cudaEventQuery(dp->ev_done);
            if (q == cudaSuccess) break;
            if (q != cudaErrorNotReady) { fail(dp->ctx, B200_ERR_CUDA, "communication stream failed: %s", cudaGetErrorString(q)); return b200dp::DP_ERR_COMM; }
            ncclResult_t async = ncclSuccess;
            if (dp->api->CommGetAsyncError(dp->comm, &async) != ncclSuccess || (async != ncclSuccess && async != ncclInProgress)) {
                dp_fail(dp, B200_ERR_NCCL, "the communicator reported an asynchronous error", async);
                return b200dp::DP_ERR_COMM;
            }
            const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
            if (ms > deadline_ms) {
                fail(dp->ctx, B200_ERR_TIMEOUT, "a data-parallel peer did not arrive within %d ms (rank %d of %d); the communicator has been aborted", deadline_ms,
                     dp->rank, dp->world);
                return b200dp::DP_ERR_TIMEOUT;
            }
            std::this_thread::sleep_for(std::chrono::microseconds(20));
        }
        for (int i = 0; i < n; i++) v[i] = dp->scal_host[i];
        // the reduced gradients are final: the step on the compute stream may follow
        if (cudaStreamWaitEvent(dp->ctx->stream, dp->ev_done, 0) != cudaSuccess) return b200dp::DP_ERR_COMM;
        cudaEventRecord(dp->ev_resume, dp->ctx->stream);
        return b200dp::DP_OK;
    }

    void abort() {
        if (dp->comm && !dp->dead) dp->api->CommAbort(dp->comm);
        dp->comm = nullptr;
        dp->dead = true;
    }
};

int dp_step(b200_dp* dp, std::function<int(float*, int32_t*)> local, float lr, int use_clip, float thr, int do_step, float* loss, float* grad_norm,
            int32_t* valid_count) {
    if (dp->dead) return fail(dp->ctx, B200_ERR_NCCL, "the communicator of this rank was aborted after an earlier failure; destroy and recreate it");
    if (cudaSetDevice(dp->ctx->device) != cudaSuccess) return fail(dp->ctx, B200_ERR_CUDA, "cudaSetDevice failed");
    dp->first_range = true;
    dp->cur_event = nullptr;
    LmEngine eng{dp, std::move(local), lr, use_clip, thr, do_step};
    NcclTransport tr{dp};
    b200dp::StepResult r;
    const int rc = b200dp::dp_train_step(eng, tr, dp->ranges, dp->deadline_ms, &r);
    if (loss) *loss = r.loss;
    if (grad_norm) *grad_norm = r.grad_norm;
    if (valid_count) *valid_count = r.valid;
    if (rc == b200dp::DP_OK) {
        float ms = 0.f;
        cudaStreamSynchronize(dp->ctx->stream);  // apply_step has synchronised already; this only makes the events below readable
        dp->timings[0] = cudaEventElapsedTime(&ms, dp->ev_bwd_end, dp->ev_resume) == cudaSuccess ? ms : 0.f;
        dp->timings[1] = cudaEventElapsedTime(&ms, dp->ev_comm_first, dp->ev_comm_last) == cudaSuccess ? ms : 0.f;
        return B200_OK;
    }
    if (rc == b200dp::DP_ERR_PEER) return fail(dp->ctx, B200_ERR_PEER, "another rank failed in this step; the step was discarded on every rank (rank %d of %d)", dp->rank, dp->world);
    if (rc == b200dp::DP_ERR_PROTOCOL) return fail(dp->ctx, B200_ERR_NCCL, "the trainer announced a gradient range out of order");
    return map_status(rc);  // the message was set where the failure was seen
}

int dp_init_common(b200_dp* dp) {
    b200_ctx* ctx = dp->ctx;
    for (const auto& r : lm_grad_ranges(dp->lm)) dp->ranges.push_back(b200dp::Range{r.first, r.second});
    int lo = 0, hi = 0;
    B200_CUDA(ctx, cudaDeviceGetStreamPriorityRange(&lo, &hi));
    B200_CUDA(ctx, cudaStreamCreateWithPriority(&dp->comm_stream, cudaStreamNonBlocking, hi));  // the reductions should not queue behind compute kernels
    B200_CUDA(ctx, cudaMalloc((void**)&dp->scal_dev, sizeof(double) * 8));
    B200_CUDA(ctx, cudaMallocHost((void**)&dp->scal_host, sizeof(double) * 8));
    cudaEvent_t* evs[] = {&dp->ev_bwd_end, &dp->ev_resume, &dp->ev_comm_first, &dp->ev_comm_last};
    for (cudaEvent_t* e : evs) B200_CUDA(ctx, cudaEventCreate(e));
    B200_CUDA(ctx, cudaEventCreateWithFlags(&dp->ev_done, cudaEventDisableTiming));
    B200_CUDA(ctx, cudaEventCreateWithFlags(&dp->ev_local, cudaEventDisableTiming));
    lm_set_external_norm(dp->lm, true);
    return b200_lm_set_grad_ready_callback(dp->lm, ready_trampoline, dp);
}

b200_dp* dp_new(b200_lm* lm, NcclApi* api, int rank, int world) {
    b200_dp* dp = new b200_dp();
    dp->lm = lm;
    dp->ctx = lm_context(lm);
    dp->api = api;
    dp->rank = rank;
    dp->world = world;
    lm_retain(lm);
    ctx_retain(dp->ctx);
    return dp;
}

}  // namespace

extern "C" {

int32_t b200_dp_set_nccl_library(const char* path) {
    std::lock_guard<std::mutex> lock(g_nccl_mu);
    if (g_nccl) return B200_ERR_INVALID_ARG;  // already loaded
    g_nccl_path = path ? path : "";
    return B200_OK;
}

int32_t b200_dp_set_nccl_max_ctas(int32_t n) {
    if (n < 0) return B200_ERR_INVALID_ARG;
    std::lock_guard<std::mutex> lock(g_nccl_mu);
    g_nccl_max_ctas = n;
    return B200_OK;
}

int32_t b200_dp_shard(int32_t n_seq, int32_t rank, int32_t world, int32_t* lo, int32_t* hi) {
    if (!lo || !hi || n_seq < 0 || world <= 0 || rank < 0 || rank >= world) return B200_ERR_INVALID_ARG;
    int l, h;
    b200dp::shard_bounds(n_seq, rank, world, &l, &h);
    *lo = l;
    *hi = h;
    return B200_OK;
}

int32_t b200_dp_unique_id(uint8_t* id128) {
    if (!id128) return B200_ERR_INVALID_ARG;
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes in every NCCL 2.x release");
    NcclApi* api = nccl_api(nullptr);
    if (!api) return B200_ERR_NCCL;
    ncclUniqueId id;
    if (api->GetUniqueId(&id) != ncclSuccess) return B200_ERR_NCCL;
    memcpy(id128, &id, 128);
    return B200_OK;
}

int32_t b200_dp_create_rank(b200_lm* lm, const uint8_t* id128, int32_t rank, int32_t world, b200_dp** out) {
    if (!lm || !id128 || !out) return B200_ERR_INVALID_ARG;
    *out = nullptr;
    b200_ctx* ctx = lm_context(lm);
    if (world <= 0 || rank < 0 || rank >= world) return fail(ctx, B200_ERR_INVALID_ARG, "rank %d outside a world of %d", rank, world);
    std::string why;
    NcclApi* api = nccl_api(&why);
    if (!api) return fail(ctx, B200_ERR_NCCL, "%s", why.c_str());
    B200_CUDA(ctx, cudaSetDevice(ctx->device));
    b200_dp* dp = dp_new(lm, api, rank, world);
    ncclUniqueId id;
    memcpy(&id, id128, 128);
    ncclResult_t r = comm_init_rank(api, &dp->comm, world, id, rank);
    if (r != ncclSuccess) {
        int rc = dp_fail(dp, B200_ERR_NCCL, "ncclCommInitRank failed", r);
        dp->comm = nullptr;
        b200_dp_destroy(dp);
        return rc;
    }
    int rc = dp_init_common(dp);
    if (rc != B200_OK) { b200_dp_destroy(dp); return rc; }
    *out = dp;
    return B200_OK;
}

int32_t b200_dp_destroy(b200_dp* dp) {
    if (!dp) return B200_OK;
    cudaSetDevice(dp->ctx->device);
    cudaStreamSynchronize(dp->ctx->stream);
    b200_lm_set_grad_ready_callback(dp->lm, nullptr, nullptr);
    lm_set_external_norm(dp->lm, false);
    if (dp->comm) {
        if (dp->comm_stream) cudaStreamSynchronize(dp->comm_stream);
        dp->api->CommDestroy(dp->comm);
    }
    if (dp->comm_stream) cudaStreamDestroy(dp->comm_stream);
    if (dp->scal_dev) cudaFree(dp->scal_dev);
    if (dp->scal_host) cudaFreeHost(dp->scal_host);
    cudaEvent_t evs[] = {dp->ev_done, dp->ev_bwd_end, dp->ev_resume, dp->ev_comm_first, dp->ev_comm_last, dp->ev_local};
    for (cudaEvent_t e : evs)
        if (e) cudaEventDestroy(e);
    b200_lm* lm = dp->lm;
    b200_ctx* ctx = dp->ctx;
    delete dp;
    b200_lm_destroy(lm);  // drops this object's reference
    ctx_release(ctx);
    return B200_OK;
}

int32_t b200_dp_set_deadline_ms(b200_dp* dp, int32_t ms) {
    if (!dp || ms <= 0) return B200_ERR_INVALID_ARG;
    dp->deadline_ms = ms;
    return B200_OK;
}

int32_t b200_dp_broadcast_params(b200_dp* dp, int32_t root) {
    if (!dp) return B200_ERR_INVALID_ARG;
    b200_ctx* ctx = dp->ctx;
    if (dp->dead) return fail(ctx, B200_ERR_NCCL, "the communicator of this rank was aborted");
    if (root < 0 || root >= dp->world) return fail(ctx, B200_ERR_INVALID_ARG, "root %d outside a world of %d", root, dp->world);
    B200_CUDA(ctx, cudaSetDevice(ctx->device));
    B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    float* p = b200_lm_params_device(dp->lm);
    ncclResult_t r = dp->api->Broadcast(p, p, (size_t)lm_param_total(dp->lm), ncclFloat, root, dp->comm, dp->comm_stream);
    if (r != ncclSuccess) return dp_fail(dp, B200_ERR_NCCL, "ncclBroadcast of the parameters failed", r);
    B200_CUDA(ctx, cudaStreamSynchronize(dp->comm_stream));
    return B200_OK;
}

int32_t b200_dp_train_step_discrete(b200_dp* dp, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq, float lr, int32_t use_clip,
                                    float clip_threshold, int32_t do_step, float* loss, float* grad_norm, int32_t* valid_count) {
    if (!dp) return B200_ERR_INVALID_ARG;
    if (!tokens || !seq_offsets || n_seq < 0) return fail(dp->ctx, B200_ERR_INVALID_ARG, "null batch argument");
    int lo, hi;
    b200dp::shard_bounds(n_seq, dp->rank, dp->world, &lo, &hi);
    // offsets are absolute positions in `tokens`, so a shard is just a window of the offset array
    auto local = [=](float* ls, int32_t* vc) { return b200_lm_accumulate_discrete(dp->lm, tokens, seq_offsets + lo, hi - lo, ls, vc); };
    return dp_step(dp, local, lr, use_clip, clip_threshold, do_step, loss, grad_norm, valid_count);
}

int32_t b200_dp_train_step_continuous(b200_dp* dp, const float* features, const float* reg_targets, const int32_t* class_targets,
                                      const int32_t* seq_offsets, int32_t n_seq, float lr, int32_t use_clip, float clip_threshold, int32_t do_step,
                                      float* loss, float* grad_norm, int32_t* valid_count) {
    if (!dp) return B200_ERR_INVALID_ARG;
    if (!features || !seq_offsets || n_seq < 0) return fail(dp->ctx, B200_ERR_INVALID_ARG, "null batch argument");
    int lo, hi;
    b200dp::shard_bounds(n_seq, dp->rank, dp->world, &lo, &hi);
    auto local = [=](float* ls, int32_t* vc) {
        return b200_lm_accumulate_continuous(dp->lm, features, reg_targets, class_targets, seq_offsets + lo, hi - lo, ls, vc);
    };
    return dp_step(dp, local, lr, use_clip, clip_threshold, do_step, loss, grad_norm, valid_count);
}

int32_t b200_dp_batch_create_discrete(b200_dp* dp, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq, b200_lm_batch** out) {
    if (!dp || !out) return B200_ERR_INVALID_ARG;
    if (!tokens || !seq_offsets || n_seq < 0) return fail(dp->ctx, B200_ERR_INVALID_ARG, "null batch argument");
    int lo, hi;
    b200dp::shard_bounds(n_seq, dp->rank, dp->world, &lo, &hi);
    // re-base the shard so that the prepared batch holds only its own tokens
    std::vector<int32_t> off((size_t)(hi - lo) + 1);
    for (int i = lo; i <= hi; i++) off[(size_t)(i - lo)] = seq_offsets[i] - seq_offsets[lo];
    return b200_lm_batch_create_discrete(dp->lm, tokens + seq_offsets[lo], off.data(), hi - lo, out);
}

int32_t b200_dp_batch_create_continuous(b200_dp* dp, const float* features, const float* reg_targets, const int32_t* class_targets,
                                        const int32_t* seq_offsets, int32_t n_seq, b200_lm_batch** out) {
    if (!dp || !out) return B200_ERR_INVALID_ARG;
    if (!features || !seq_offsets || n_seq < 0) return fail(dp->ctx, B200_ERR_INVALID_ARG, "null batch argument");
    int lo, hi;
    b200dp::shard_bounds(n_seq, dp->rank, dp->world, &lo, &hi);
    const b200_lm_config& c = lm_config_of(dp->lm);
    std::vector<int32_t> off((size_t)(hi - lo) + 1);
    for (int i = lo; i <= hi; i++) off[(size_t)(i - lo)] = seq_offsets[i] - seq_offsets[lo];
    const size_t row0 = (size_t)seq_offsets[lo];
    return b200_lm_batch_create_continuous(dp->lm, features + row0 * (size_t)c.input_feature_dim, reg_targets ? reg_targets + row0 * (size_t)c.output_dim : nullptr,
                                           class_targets ? class_targets + row0 : nullptr, off.data(), hi - lo, out);
}

int32_t b200_dp_train_step_batch(b200_dp* dp, b200_lm_batch* shard, float lr, int32_t use_clip, float clip_threshold, int32_t do_step, float* loss,
                                 float* grad_norm, int32_t* valid_count) {
    if (!dp || !shard) return B200_ERR_INVALID_ARG;
    auto local = [=](float* ls, int32_t* vc) { return b200_lm_accumulate_batch(dp->lm, shard, ls, vc); };
    return dp_step(dp, local, lr, use_clip, clip_threshold, do_step, loss, grad_norm, valid_count);
}

int32_t b200_dp_get_timings(b200_dp* dp, float* ms2) {
    if (!dp || !ms2) return B200_ERR_INVALID_ARG;
    ms2[0] = dp->timings[0];
    ms2[1] = dp->timings[1];
    return B200_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------- one process, all GPUs
struct b200_dp_group {
    std::vector<b200_ctx*> ctx;
    std::vector<b200_lm*> lm;
    std::vector<b200_dp*> dp;
    std::string err;
};

namespace {

// Runs fn(rank) on one host thread per rank and returns the first failure (the ranks' own contexts keep their messages).
int for_each_rank(b200_dp_group* g, const std::function<int(int)>& fn) {
    const int n = (int)g->dp.size();
    std::vector<int> rc((size_t)n, B200_OK);
    std::vector<std::thread> th;
    for (int r = 1; r < n; r++) th.emplace_back([&, r] { rc[(size_t)r] = fn(r); });
    rc[0] = fn(0);
    for (auto& t : th) t.join();
    // a rank's own failure says more than its peers' "another rank failed"
    int first = B200_OK, who = -1;
    for (int r = 0; r < n; r++)
        if (rc[(size_t)r] != B200_OK && (first == B200_OK || first == B200_ERR_PEER)) { first = rc[(size_t)r]; who = r; }
    if (who >= 0) g->err = "rank " + std::to_string(who) + ": " + b200_last_error(g->ctx[(size_t)who]);
    return first;
}

}  // namespace

extern "C" {

int32_t b200_dp_group_create(const int32_t* devices, int32_t n, const b200_lm_config* cfg, int32_t max_rows, int32_t gemm_mode, b200_dp_group** out) {
    if (!devices || !cfg || !out || n <= 0) return B200_ERR_INVALID_ARG;
    *out = nullptr;
    std::string why;
    NcclApi* api = nccl_api(&why);
    if (!api) return B200_ERR_NCCL;
    b200_dp_group* g = new b200_dp_group();
    int rc = B200_OK;
    for (int i = 0; i < n && rc == B200_OK; i++) {
        b200_ctx* c = nullptr;
        rc = b200_create(devices[i], &c);
        if (rc != B200_OK) break;
        g->ctx.push_back(c);
        rc = b200_set_gemm_mode(c, gemm_mode);
        if (rc != B200_OK) break;
        b200_lm* lm = nullptr;
        rc = b200_lm_create(c, cfg, nullptr, nullptr, max_rows, &lm);
        if (rc != B200_OK) break;
        g->lm.push_back(lm);
    }
    if (rc == B200_OK) {
        std::vector<ncclComm_t> comms((size_t)n);
        std::vector<int> devs(devices, devices + n);
        ncclResult_t r;
        if (api->CommInitRankConfig && api->GroupStart && api->GroupEnd && g_nccl_max_ctas > 0) {
            // ncclCommInitAll takes no configuration: the same thing by hand (one id, every rank inside one group call)
            ncclUniqueId id;
            r = api->GetUniqueId(&id);
            if (r == ncclSuccess) r = api->GroupStart();
            for (int i = 0; i < n && r == ncclSuccess; i++) {
                cudaSetDevice(devs[(size_t)i]);
                r = comm_init_rank(api, &comms[(size_t)i], n, id, i);
            }
            if (r == ncclSuccess) r = api->GroupEnd();
            else api->GroupEnd();
        } else {
            r = api->CommInitAll(comms.data(), n, devs.data());
        }
        if (r != ncclSuccess) rc = B200_ERR_NCCL;
        for (int i = 0; i < n && rc == B200_OK; i++) {
            cudaSetDevice(devices[i]);
            b200_dp* dp = dp_new(g->lm[(size_t)i], api, i, n);
            dp->comm = comms[(size_t)i];
            g->dp.push_back(dp);
            rc = dp_init_common(dp);
        }
    }
    if (rc != B200_OK) { b200_dp_group_destroy(g); return rc; }
    *out = g;
    return B200_OK;
}

int32_t b200_dp_group_destroy(b200_dp_group* g) {
    if (!g) return B200_OK;
    for (b200_dp* d : g->dp) b200_dp_destroy(d);
    for (b200_lm* l : g->lm) b200_lm_destroy(l);
    for (b200_ctx* c : g->ctx) b200_destroy(c);
    delete g;
    return B200_OK;
}

const char* b200_dp_group_last_error(b200_dp_group* g) { return g ? g->err.c_str() : "null group"; }
int32_t b200_dp_group_size(b200_dp_group* g) { return g ? (int32_t)g->dp.size() : 0; }
b200_lm* b200_dp_group_trainer(b200_dp_group* g, int32_t rank) { return (g && rank >= 0 && rank < (int)g->lm.size()) ? g->lm[(size_t)rank] : nullptr; }

int32_t b200_dp_group_set_optimizer(b200_dp_group* g, int32_t kind, float beta1, float beta2, float eps) {
    if (!g) return B200_ERR_INVALID_ARG;
    for (b200_lm* l : g->lm) B200_TRY(b200_lm_set_optimizer(l, kind, beta1, beta2, eps));
    return B200_OK;
}

int32_t b200_dp_group_upload_params(b200_dp_group* g, const float* host, int64_t offset, int64_t count) {
    if (!g) return B200_ERR_INVALID_ARG;
    return for_each_rank(g, [&](int r) { return b200_lm_upload_params(g->lm[(size_t)r], host, offset, count); });
}

int32_t b200_dp_group_train_step_discrete(b200_dp_group* g, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq, float lr, int32_t use_clip,
                                          float clip_threshold, int32_t do_step, float* loss, float* grad_norm, int32_t* valid_count) {
    if (!g) return B200_ERR_INVALID_ARG;
    return for_each_rank(g, [&](int r) {
        return b200_dp_train_step_discrete(g->dp[(size_t)r], tokens, seq_offsets, n_seq, lr, use_clip, clip_threshold, do_step, r == 0 ? loss : nullptr,
                                           r == 0 ? grad_norm : nullptr, r == 0 ? valid_count : nullptr);
    });
}

int32_t b200_dp_group_train_step_continuous(b200_dp_group* g, const float* features, const float* reg_targets, const int32_t* class_targets,
                                            const int32_t* seq_offsets, int32_t n_seq, float lr, int32_t use_clip, float clip_threshold, int32_t do_step,
                                            float* loss, float* grad_norm, int32_t* valid_count) {
    if (!g) return B200_ERR_INVALID_ARG;
    return for_each_rank(g, [&](int r) {
        return b200_dp_train_step_continuous(g->dp[(size_t)r], features, reg_targets, class_targets, seq_offsets, n_seq, lr, use_clip, clip_threshold, do_step,
                                             r == 0 ? loss : nullptr, r == 0 ? grad_norm : nullptr, r == 0 ? valid_count : nullptr);
    });
}

}  // extern "C"
