// Host-side helpers shared by the per-op entry points: a bump allocator over the context's device pool that also holds
// the context lock for the duration of one call, and the argument-check macros that map the reference's exceptions to
// status codes.
#pragma once
#include <algorithm>
#include <vector>

#include "common.h"

using namespace b200;

namespace {

// Bump allocator over the context's device pool; everything is released when the Scope dies.
struct Scope {
    b200_ctx* ctx;
    std::lock_guard<std::mutex> lock;
    std::vector<void*> overflow;
    int rc = B200_OK;
    explicit Scope(b200_ctx* c) : ctx(c), lock(c->mu) {
        ctx->pool_used = 0;
        cudaSetDevice(ctx->device);
    }
    ~Scope() {
        if (!overflow.empty()) {
            cudaStreamSynchronize(ctx->stream);
            size_t total = ctx->pool_bytes;
            for (void* p : overflow) cudaFree(p);
            // Grow the pool so the next call of this size fits without overflow blocks.
            total = std::max(total * 2, grow_to);
            if (ctx->pool) cudaFree(ctx->pool);
            ctx->pool = nullptr;
            ctx->pool_bytes = 0;
            if (cudaMalloc((void**)&ctx->pool, total) == cudaSuccess) ctx->pool_bytes = total;
            else cudaGetLastError();
        }
    }
    size_t grow_to = 0;
    void* alloc(size_t bytes) {
        bytes = (bytes + 255) & ~(size_t)255;
        if (bytes == 0) bytes = 256;
        grow_to += bytes;
        if (ctx->pool_used + bytes <= ctx->pool_bytes) {
            void* p = ctx->pool + ctx->pool_used;
            ctx->pool_used += bytes;
            return p;
        }
        void* p = nullptr;
        if (cudaMalloc(&p, bytes) != cudaSuccess) {
            rc = fail(ctx, B200_ERR_CUDA, "device allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(cudaGetLastError()));
            return nullptr;
        }
        overflow.push_back(p);
        return p;
    }
    float* floats(int64_t n) { return (float*)alloc(sizeof(float) * (size_t)std::max<int64_t>(n, 1)); }
    float* up(const float* host, int64_t n) {
        float* d = floats(n);
        if (d && n > 0 && cudaMemcpyAsync(d, host, sizeof(float) * (size_t)n, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess)
            rc = fail(ctx, B200_ERR_CUDA, "host-to-device copy failed: %s", cudaGetErrorString(cudaGetLastError()));
        return d;
    }
    int32_t* upi(const int32_t* host, int64_t n) { return (int32_t*)up((const float*)host, n); }
    uint8_t* upb(const uint8_t* host, int64_t n) {
        uint8_t* d = (uint8_t*)alloc((size_t)std::max<int64_t>(n, 1));
        if (d && n > 0 && cudaMemcpyAsync(d, host, (size_t)n, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess)
            rc = fail(ctx, B200_ERR_CUDA, "host-to-device copy failed: %s", cudaGetErrorString(cudaGetLastError()));
        return d;
    }
    int down(float* host, const float* dev, int64_t n) {
        if (n > 0) B200_CUDA(ctx, cudaMemcpyAsync(host, dev, sizeof(float) * (size_t)n, cudaMemcpyDeviceToHost, ctx->stream));
        return B200_OK;
    }
    int sync() {
        B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        return check_device_status(ctx);
    }
};

#define NEED(ctx, cond, code, ...) \
    do {                           \
        if (!(cond)) return fail(ctx, code, __VA_ARGS__); \
    } while (0)
#define NOTNULL(ctx, p) NEED(ctx, (p) != nullptr, B200_ERR_INVALID_ARG, "%s: argument '%s' is null", __func__, #p)
#define CHECK_SCOPE(s) \
    do {               \
        if ((s).rc != B200_OK) return (s).rc; \
    } while (0)

}  // namespace
