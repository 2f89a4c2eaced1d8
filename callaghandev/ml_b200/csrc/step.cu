// The parameter step as ONE cooperative kernel over the flat parameter / gradient arenas:
//   phase 1: every block sums (g * gscale)^2 over its slice (128-bit loads) and publishes one partial;
//   grid barrier;
//   phase 2: every block adds the partials in index order (so all blocks derive the bit-identical norm), forms the
//            clip factor min(1, thr/norm), and applies SGD (w -= lr*g, the reference's only optimiser) or Adam to its
//            slice, leaving the scaled-and-clipped gradient in g as the reference does.
// A non-finite norm zeroes the gradients and leaves the weights untouched (TransformerTrainer.cs:316-320).
//
// One pass over HBM: when the trainer has already summed the squares of every range of the gradient arena -- it does so
// on a side stream as each range receives its final contribution during the last pass's backward (after the range's
// all-reduce in a data-parallel job), where the sum hides under the remaining backward -- the step is
// fused_step_presummed_kernel: no norm phase, no grid barrier, the gradient is read once.  The trainer also launches
// it with write_g = 0: the scaled-and-clipped gradient is not written back (it remembers the factor and applies it
// only if somebody looks at the gradient arena before the next step zeroes it).  Bytes per parameter then: SGD read g,
// read w, write w = 12; Adam read g, w, m, v, write w, m, v = 28.
// Replaces ScaleGradients + ComputeGradientNorm + ClipGradients + UpdateParameters (TransformerTrainer.cs:1269-1383),
// which are four passes with one manager call per tensor.
#include <cooperative_groups.h>

#include "common.h"
#include "device_math.cuh"

namespace cg = cooperative_groups;

namespace b200 {

struct StepArgs {
    float *w, *g, *m, *v;
    int64_t n;
    float gscale, lr, clip_thr;
    int use_clip, do_step, optimizer;
    int write_g;  // 1: leave the scaled-and-clipped gradient in g (the reference's observable state); 0: the caller applies the factor later, on demand
    float beta1, beta2, eps;
    float alpha, rsbc2;  // Adam with the bias corrections folded in: w -= alpha * m / (sqrt(v) * rsbc2 + eps), alpha = lr / (1 - beta1^t), rsbc2 = 1 / sqrt(1 - beta2^t)
    float* partials;
    float* out;
};

__device__ __forceinline__ void step_one(const StepArgs& a, int64_t i, float factor) {
    float g = a.g[i] * factor;
    if (a.write_g) a.g[i] = g;
    if (!a.do_step) return;
    if (a.optimizer == B200_OPT_ADAM) {
        float m = a.beta1 * a.m[i] + (1.0f - a.beta1) * g;
        float v = a.beta2 * a.v[i] + (1.0f - a.beta2) * g * g;
        a.m[i] = m;
        a.v[i] = v;
        a.w[i] -= a.alpha * m / (sqrtf(v) * a.rsbc2 + a.eps);
    } else {
        a.w[i] -= a.lr * g;
    }
}

// Phase 2 of the step, shared by both kernels: t = sum of squares of the scaled gradient.
__device__ __forceinline__ void step_update(const StepArgs& a, float t, int64_t tid, int64_t stride) {
    const int64_t n4 = a.n >> 2;
    const float norm = sqrtf(t);
    const bool finite = isfinite(norm);
    const float clip = (a.use_clip && finite && norm > a.clip_thr) ? a.clip_thr / norm : 1.0f;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        a.out[0] = norm;
        a.out[1] = clip;
    }
    if (!finite) {
        float4* z4 = reinterpret_cast<float4*>(a.g);
        for (int64_t k = tid; k < n4; k += stride) z4[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int64_t k = (n4 << 2) + tid; k < a.n; k += stride) a.g[k] = 0.f;
        return;
    }
    const float factor = a.gscale * clip;
    if (!a.do_step && !a.write_g) return;  // norm only
    if (a.optimizer == B200_OPT_SGD) {
        float4* gw = reinterpret_cast<float4*>(a.g);
        float4* w4 = reinterpret_cast<float4*>(a.w);
        for (int64_t k = tid; k < n4; k += stride) {
            float4 g = gw[k];
            g.x *= factor; g.y *= factor; g.z *= factor; g.w *= factor;
            if (a.write_g) gw[k] = g;
            if (a.do_step) {
                float4 w = w4[k];
                w.x -= a.lr * g.x; w.y -= a.lr * g.y; w.z -= a.lr * g.z; w.w -= a.lr * g.w;
                w4[k] = w;
            }
        }
        for (int64_t k = (n4 << 2) + tid; k < a.n; k += stride) step_one(a, k, factor);
    } else {
        float4* gw = reinterpret_cast<float4*>(a.g);
        float4* w4 = reinterpret_cast<float4*>(a.w);
        float4* m4 = reinterpret_cast<float4*>(a.m);
        float4* v4 = reinterpret_cast<float4*>(a.v);
        const float ob1 = 1.0f - a.beta1, ob2 = 1.0f - a.beta2;
        for (int64_t k = tid; k < n4; k += stride) {
            float4 g = gw[k];
            g.x *= factor; g.y *= factor; g.z *= factor; g.w *= factor;
            if (a.write_g) gw[k] = g;
            if (a.do_step) {
                float4 m = m4[k], v = v4[k], w = w4[k];
                m.x = a.beta1 * m.x + ob1 * g.x; m.y = a.beta1 * m.y + ob1 * g.y; m.z = a.beta1 * m.z + ob1 * g.z; m.w = a.beta1 * m.w + ob1 * g.w;
                v.x = a.beta2 * v.x + ob2 * g.x * g.x; v.y = a.beta2 * v.y + ob2 * g.y * g.y;
                v.z = a.beta2 * v.z + ob2 * g.z * g.z; v.w = a.beta2 * v.w + ob2 * g.w * g.w;
                w.x -= a.alpha * m.x / (sqrtf(v.x) * a.rsbc2 + a.eps);
                w.y -= a.alpha * m.y / (sqrtf(v.y) * a.rsbc2 + a.eps);
                w.z -= a.alpha * m.z / (sqrtf(v.z) * a.rsbc2 + a.eps);
                w.w -= a.alpha * m.w / (sqrtf(v.w) * a.rsbc2 + a.eps);
                m4[k] = m; v4[k] = v; w4[k] = w;
            }
        }
        for (int64_t k = (n4 << 2) + tid; k < a.n; k += stride) step_one(a, k, factor);
    }
}

__global__ void __launch_bounds__(256) fused_step_kernel(StepArgs a) {
    __shared__ float red[32];
    cg::grid_group grid = cg::this_grid();
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t n4 = a.n >> 2;
    const float4* g4 = reinterpret_cast<const float4*>(a.g);
    float s = 0.f;
    for (int64_t k = tid; k < n4; k += stride) {
        float4 x = g4[k];
        x.x *= a.gscale; x.y *= a.gscale; x.z *= a.gscale; x.w *= a.gscale;
        s += (x.x * x.x + x.y * x.y) + (x.z * x.z + x.w * x.w);
    }
    for (int64_t k = (n4 << 2) + tid; k < a.n; k += stride) {
        float x = a.g[k] * a.gscale;
        s += x * x;
    }
    s = block_sum(s, red);
    if (threadIdx.x == 0) a.partials[blockIdx.x] = s;
    grid.sync();
    float t = 0.f;
    for (int k = threadIdx.x; k < (int)gridDim.x; k += blockDim.x) t += a.partials[k];
    t = block_sum(t, red);
    step_update(a, t, tid, stride);
}

// The same step when the sum of squares has been taken range by range beforehand: `partials` holds n_partials sums of
// UNSCALED squares in a fixed order; every block adds them in that order (bit-identical norm in all blocks).
__global__ void __launch_bounds__(256) fused_step_presummed_kernel(StepArgs a, const float* __restrict__ partials, int n_partials) {
    __shared__ float red[32];
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
    float t = 0.f;
    for (int k = threadIdx.x; k < n_partials; k += blockDim.x) t += partials[k];
    t = block_sum(t, red) * (a.gscale * a.gscale);
    step_update(a, t, tid, stride);
}

// Sum of squares of one range of the gradient arena: block b adds its fixed slice in a fixed order and writes partials[b].
__global__ void __launch_bounds__(256) sumsq_partials_kernel(const float* __restrict__ g, int64_t n, float* __restrict__ partials) {
    __shared__ float red[32];
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t head = (4 - (((uintptr_t)g >> 2) & 3)) & 3;  // elements before the first 16-byte boundary
    const int64_t h = head < n ? head : n;
    const float4* g4 = reinterpret_cast<const float4*>(g + h);
    const int64_t n4 = (n - h) >> 2;
    float s = 0.f;
    for (int64_t k = tid; k < n4; k += stride) {
        const float4 x = g4[k];
        s += (x.x * x.x + x.y * x.y) + (x.z * x.z + x.w * x.w);
    }
    if (blockIdx.x == 0) {
        for (int64_t k = threadIdx.x; k < h; k += blockDim.x) s += g[k] * g[k];
        for (int64_t k = h + (n4 << 2) + threadIdx.x; k < n; k += blockDim.x) s += g[k] * g[k];
    }
    s = block_sum(s, red);
    if (threadIdx.x == 0) partials[blockIdx.x] = s;
}

int k_fused_step(b200_ctx* ctx, float* w, float* g, float* m, float* v, int64_t n, float gscale, float lr, int use_clip, float clip_thr,
                 int do_step, int optimizer, float beta1, float beta2, float eps, int step_index, float* out_dev, int write_g) {
    if (n <= 0) return B200_OK;
    if (((uintptr_t)w | (uintptr_t)g | (uintptr_t)m | (uintptr_t)v) & 15)
        return fail(ctx, B200_ERR_INVALID_ARG, "parameter arenas must be 16-byte aligned");
    static int blocksPerSm = 0;
    if (!blocksPerSm) {
        B200_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocksPerSm, fused_step_kernel, 256, 0));
        if (blocksPerSm < 1) return fail(ctx, B200_ERR_CUDA, "fused step kernel cannot be made resident");
        if (blocksPerSm > 4) blocksPerSm = 4;
    }
    int grid = ctx->sm_count * blocksPerSm;
    int64_t need = (n / 4 + 255) / 256;
    if (need < 1) need = 1;
    if (grid > need) grid = (int)need;
    B200_TRY(ensure_ws(ctx, (size_t)grid));
    StepArgs a;
    a.w = w; a.g = g; a.m = m; a.v = v; a.n = n; a.gscale = gscale; a.lr = lr; a.clip_thr = clip_thr; a.use_clip = use_clip;
    a.do_step = do_step; a.optimizer = optimizer; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.write_g = write_g;
    a.alpha = (float)((double)lr / (1.0 - pow((double)beta1, (double)step_index)));
    a.rsbc2 = (float)(1.0 / sqrt(1.0 - pow((double)beta2, (double)step_index)));
    a.partials = ctx->ws;
    a.out = out_dev;
    void* args[] = {&a};
    B200_CUDA(ctx, cudaLaunchCooperativeKernel((void*)fused_step_kernel, dim3(grid), dim3(256), args, 0, ctx->stream));
    ctx->launches++;
    return B200_OK;
}

// Sums of squares of g[0, n) into partials[0, blocks): returns the number of partials written through *blocks.
int k_sumsq_partials(b200_ctx* ctx, const float* g, int64_t n, float* partials, int max_blocks, cudaStream_t stream, int* blocks) {
    *blocks = 0;
    if (n <= 0 || max_blocks <= 0) return B200_OK;
    int64_t want = (n / 4 + 256 * 8 - 1) / (256 * 8);  // at least eight 128-bit loads per thread
    if (want < 1) want = 1;
    if (want > max_blocks) want = max_blocks;
    sumsq_partials_kernel<<<(int)want, 256, 0, stream>>>(g, n, partials);
    B200_LAUNCH_CHECK(ctx);
    *blocks = (int)want;
    return B200_OK;
}

int k_fused_step_presummed(b200_ctx* ctx, float* w, float* g, float* m, float* v, int64_t n, const float* partials, int n_partials, float gscale,
                           float lr, int use_clip, float clip_thr, int do_step, int optimizer, float beta1, float beta2, float eps, int step_index,
                           float* out_dev, int write_g) {
    if (n <= 0) return B200_OK;
    if (((uintptr_t)w | (uintptr_t)g | (uintptr_t)m | (uintptr_t)v) & 15)
        return fail(ctx, B200_ERR_INVALID_ARG, "parameter arenas must be 16-byte aligned");
    int grid = ctx->sm_count * 5;  // 48 registers x 256 threads: five blocks per SM are resident
    int64_t need = (n / 4 + 255) / 256;
    if (need < 1) need = 1;
    if (grid > need) grid = (int)need;
    StepArgs a;
    a.w = w; a.g = g; a.m = m; a.v = v; a.n = n; a.gscale = gscale; a.lr = lr; a.clip_thr = clip_thr; a.use_clip = use_clip;
    a.do_step = do_step; a.optimizer = optimizer; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.write_g = write_g;
    a.alpha = (float)((double)lr / (1.0 - pow((double)beta1, (double)step_index)));
    a.rsbc2 = (float)(1.0 / sqrt(1.0 - pow((double)beta2, (double)step_index)));
    a.partials = nullptr;
    a.out = out_dev;
    fused_step_presummed_kernel<<<grid, 256, 0, ctx->stream>>>(a, partials, n_partials);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

// g *= factor over the whole arena: what the step leaves undone when it does not write the gradient back.
__global__ void __launch_bounds__(256) scale_arena_kernel(float* __restrict__ g, int64_t n, float factor) {
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
    float4* g4 = reinterpret_cast<float4*>(g);
    const int64_t n4 = n >> 2;
    for (int64_t k = tid; k < n4; k += stride) {
        float4 x = g4[k];
        x.x *= factor; x.y *= factor; x.z *= factor; x.w *= factor;
        g4[k] = x;
    }
    for (int64_t k = (n4 << 2) + tid; k < n; k += stride) g[k] *= factor;
}

int k_scale_arena(b200_ctx* ctx, float* g, int64_t n, float factor) {
    if (n <= 0) return B200_OK;
    int64_t need = (n / 4 + 255) / 256;
    int grid = ctx->sm_count * 8;
    if (need < 1) need = 1;
    if (grid > need) grid = (int)need;
    scale_arena_kernel<<<grid, 256, 0, ctx->stream>>>(g, n, factor);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

}  // namespace b200
