// Bandwidth-bound kernels of the training hot path: residual/LayerNorm forward and backward (warp-shuffle row
// reductions), fused softmax-cross-entropy gradient, MSE gradient, rotary embedding, embedding gather and
// deterministic scatter-add, column sums, and the small vector primitives.  All loads are 128-bit where the shape
// allows; reductions are two-stage and order-deterministic (no floating-point atomics anywhere).
#include <cmath>
#include <cstdarg>

#include "common.h"
#include "device_math.cuh"

namespace b200 {

int fail(b200_ctx* ctx, int code, const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    if (ctx) ctx->err = buf;
    return code;
}

int check_device_status(b200_ctx* ctx) {
    if (ctx->status_host && *ctx->status_host != 0) {
        int code = *ctx->status_host;
        *ctx->status_host = 0;  // reported once: the kernels that saw it have returned, the context stays usable
        return fail(ctx, B200_ERR_TIMEOUT, "a bounded device-side wait expired in a tcgen05 kernel (wait site %d: 1-3 GEMM producer / MMA issuer / epilogue, "
                    "9 the wait probe, 10 and above attention)", code);
    }
    return B200_OK;
}

int ensure_ws(b200_ctx* ctx, size_t n) {
    if (ctx->ws_floats >= n) return B200_OK;
    // The old block may still be in use by enqueued kernels: drain the stream before replacing it.
    B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->ws) cudaFree(ctx->ws);
    ctx->ws = nullptr;
    ctx->ws_floats = 0;
    size_t want = n < (1u << 20) ? (1u << 20) : n;
    B200_CUDA(ctx, cudaMalloc(&ctx->ws, want * sizeof(float)));
    ctx->ws_floats = want;
    return B200_OK;
}

int rope_table(b200_ctx* ctx, int headDim, float baseTheta, int rows, const float** out) {
    uint32_t bits;
    memcpy(&bits, &baseTheta, 4);
    RopeTable& t = ctx->rope[{headDim, bits}];
    if (t.rows < rows) {
        int want = rows < 1024 ? 1024 : rows;
        int pairs = headDim / 2;
        std::vector<float> h((size_t)want * pairs * 2);
        // Same expression order as the reference: theta = pos / pow(base, 2*pair/headDim); cos, sin of theta.
        for (int p = 0; p < pairs; p++) {
            float denom = powf(baseTheta, (2.0f * p) / headDim);
            for (int r = 0; r < want; r++) {
                float theta = r / denom;
                h[((size_t)r * pairs + p) * 2] = cosf(theta);
                h[((size_t)r * pairs + p) * 2 + 1] = sinf(theta);
            }
        }
        B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (t.dev) ctx->rope_retired.push_back(t.dev);  // a trainer or a decoding session may still hold this pointer
        t.dev = nullptr;
        t.rows = 0;
        B200_CUDA(ctx, cudaMalloc(&t.dev, h.size() * sizeof(float)));
        B200_CUDA(ctx, cudaMemcpy(t.dev, h.data(), h.size() * sizeof(float), cudaMemcpyHostToDevice));
        t.rows = want;
    }
    *out = t.dev;
    return B200_OK;
}

// ------------------------------------------------------------------------------------------------ vector primitives
static inline int grid_for(int64_t n, int per_block, int cap) {
    int64_t g = (n + per_block - 1) / per_block;
    if (g < 1) g = 1;
    if (g > cap) g = cap;
    return (int)g;
}
static inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

template <int OP>  // 0: t += a ; 1: t *= s ; 2: t -= s*a
__global__ void vec_kernel(float* __restrict__ t, const float* __restrict__ a, int64_t n, float s, int vec) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
    if (vec) {
        int64_t n4 = n >> 2;
        float4* t4 = reinterpret_cast<float4*>(t);
        const float4* a4 = reinterpret_cast<const float4*>(a);
        for (int64_t k = i; k < n4; k += stride) {
            float4 x = t4[k];
            if (OP == 1) { x.x *= s; x.y *= s; x.z *= s; x.w *= s; }
            else {
                float4 y = a4[k];
                if (OP == 0) { x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w; }
                else { x.x -= s * y.x; x.y -= s * y.y; x.z -= s * y.z; x.w -= s * y.w; }
            }
            t4[k] = x;
        }
        for (int64_t k = (n4 << 2) + i; k < n; k += stride) {
            if (OP == 0) t[k] += a[k]; else if (OP == 1) t[k] *= s; else t[k] -= s * a[k];
        }
    } else {
        for (int64_t k = i; k < n; k += stride) {
            if (OP == 0) t[k] += a[k]; else if (OP == 1) t[k] *= s; else t[k] -= s * a[k];
        }
    }
}

template <int OP>
static int vec_launch(b200_ctx* ctx, float* t, const float* a, int64_t n, float s) {
    if (n <= 0) return B200_OK;
    int vec = aligned16(t) && (a == nullptr || aligned16(a));
    vec_kernel<OP><<<grid_for(n, 256 * 8, 148 * 16), 256, 0, ctx->stream>>>(t, a, n, s, vec);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}
int k_add_inplace(b200_ctx* ctx, float* t, const float* a, int64_t n) { return vec_launch<0>(ctx, t, a, n, 0.f); }
int k_scale_inplace(b200_ctx* ctx, float* x, int64_t n, float s) { return vec_launch<1>(ctx, x, nullptr, n, s); }
int k_sgd_update(b200_ctx* ctx, float* w, const float* g, int64_t n, float lr) { return vec_launch<2>(ctx, w, g, n, lr); }

__global__ void mul_act_deriv_kernel(float* __restrict__ x, const float* __restrict__ z, int act, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        float a, d;
        ffn_act_der(z[i], act, a, d);
        x[i] *= d;
    }
}
int k_mul_act_deriv(b200_ctx* ctx, float* x, const float* z, int act, int64_t n) {
    if (n <= 0 || act == B200_ACT_NONE) return B200_OK;
    mul_act_deriv_kernel<<<grid_for(n, 256, 148 * 8), 256, 0, ctx->stream>>>(x, z, act, n);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

__global__ void sqnorm_partial_kernel(const float* __restrict__ x, int64_t n, float* __restrict__ partial, int vec) {
    __shared__ float red[32];
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
    float s = 0.f;
    if (vec) {
        int64_t n4 = n >> 2;
        const float4* x4 = reinterpret_cast<const float4*>(x);
        for (int64_t k = i; k < n4; k += stride) {
            float4 v = x4[k];
            s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        for (int64_t k = (n4 << 2) + i; k < n; k += stride) s += x[k] * x[k];
    } else {
        for (int64_t k = i; k < n; k += stride) s += x[k] * x[k];
    }
    s = block_sum(s, red);
    if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
__global__ void sum_partials_kernel(const float* __restrict__ partial, int n, float* __restrict__ out) {
    __shared__ float red[32];
    float s = 0.f;
    for (int k = threadIdx.x; k < n; k += blockDim.x) s += partial[k];
    s = block_sum(s, red);
    if (threadIdx.x == 0) out[0] = s;
}
int k_sqnorm(b200_ctx* ctx, const float* x, int64_t n, float* out_dev) {
    int g = grid_for(n, 256 * 16, 1024);
    B200_TRY(ensure_ws(ctx, 1024));
    sqnorm_partial_kernel<<<g, 256, 0, ctx->stream>>>(x, n, ctx->ws, aligned16(x));
    B200_LAUNCH_CHECK(ctx);
    sum_partials_kernel<<<1, 256, 0, ctx->stream>>>(ctx->ws, g, out_dev);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

// ------------------------------------------------------------------------------------------------ column sums
// grid (colTiles, chunks), block (32, 8): thread (x,y) sums rows y, y+8, ... of its chunk for column tile*32+x.
__global__ void colsum_partial_kernel(const float* __restrict__ x, int rows, int cols, int ld, int rowsPerChunk,
                                      float* __restrict__ partial) {
    __shared__ float sm[8][33];
    int c = blockIdx.x * 32 + threadIdx.x;
    int r0 = blockIdx.y * rowsPerChunk, r1 = min(rows, r0 + rowsPerChunk);
    float s = 0.f;
    if (c < cols)
        for (int r = r0 + threadIdx.y; r < r1; r += 8) s += x[(size_t)r * ld + c];
    sm[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && c < cols) {
        float t = 0.f;
#pragma unroll
        for (int y = 0; y < 8; y++) t += sm[y][threadIdx.x];
        partial[(size_t)blockIdx.y * cols + c] = t;
    }
}
__global__ void colsum_final_kernel(const float* __restrict__ partial, int chunks, int cols, float* __restrict__ out, int accumulate) {
    int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    float s = 0.f;
    for (int k = 0; k < chunks; k++) s += partial[(size_t)k * cols + c];
    out[c] = accumulate ? out[c] + s : s;
}
// 128-bit variant: grid (colTiles of 128 columns, chunks), block (32, 8): thread (x,y) sums rows y, y+8, ... of its chunk
// for columns tile*128 + 4x .. +3, four rows in flight per thread.
__global__ void __launch_bounds__(256) colsum_partial_vec_kernel(const float* __restrict__ x, int rows, int cols, int ld, int rowsPerChunk,
                                                                 float* __restrict__ partial) {
    __shared__ float4 sm[8][33];
    const int c = blockIdx.x * 128 + threadIdx.x * 4;
    const int r0 = blockIdx.y * rowsPerChunk, r1 = min(rows, r0 + rowsPerChunk);
    float4 s0 = make_float4(0.f, 0.f, 0.f, 0.f), s1 = s0, s2 = s0, s3 = s0;
    if (c < cols) {
        const float* base = x + c;
        int r = r0 + threadIdx.y;
        for (; r + 24 < r1; r += 32) {
            const float4 a = *reinterpret_cast<const float4*>(base + (size_t)r * ld), b = *reinterpret_cast<const float4*>(base + (size_t)(r + 8) * ld),
                         cc = *reinterpret_cast<const float4*>(base + (size_t)(r + 16) * ld), d = *reinterpret_cast<const float4*>(base + (size_t)(r + 24) * ld);
            s0.x += a.x; s0.y += a.y; s0.z += a.z; s0.w += a.w;
            s1.x += b.x; s1.y += b.y; s1.z += b.z; s1.w += b.w;
            s2.x += cc.x; s2.y += cc.y; s2.z += cc.z; s2.w += cc.w;
            s3.x += d.x; s3.y += d.y; s3.z += d.z; s3.w += d.w;
        }
        for (; r < r1; r += 8) {
            const float4 a = *reinterpret_cast<const float4*>(base + (size_t)r * ld);
            s0.x += a.x; s0.y += a.y; s0.z += a.z; s0.w += a.w;
        }
    }
    sm[threadIdx.y][threadIdx.x] = make_float4((s0.x + s1.x) + (s2.x + s3.x), (s0.y + s1.y) + (s2.y + s3.y), (s0.z + s1.z) + (s2.z + s3.z),
                                               (s0.w + s1.w) + (s2.w + s3.w));
    __syncthreads();
    if (threadIdx.y == 0 && c < cols) {
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int y = 0; y < 8; y++) {
            const float4 v = sm[y][threadIdx.x];
            t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
        }
        *reinterpret_cast<float4*>(partial + (size_t)blockIdx.y * cols + c) = t;
    }
}
int k_colsum(b200_ctx* ctx, const float* x, int rows, int cols, int ld, float* out, int accumulate) {
    if (cols <= 0) return B200_OK;
    const bool vec = (cols % 4 == 0) && (ld % 4 == 0) && aligned16(x);
    int colTiles = vec ? (cols + 127) / 128 : (cols + 31) / 32;
    int chunks = (148 * 8 + colTiles - 1) / colTiles;
    if (chunks > (vec ? 256 : 64)) chunks = vec ? 256 : 64;
    int maxChunks = (rows + 63) / 64;
    if (maxChunks < 1) maxChunks = 1;
    if (chunks > maxChunks) chunks = maxChunks;
    int rowsPerChunk = (rows + chunks - 1) / chunks;
    if (rowsPerChunk < 1) rowsPerChunk = 1;
    B200_TRY(ensure_ws(ctx, (size_t)chunks * cols));
    if (vec) colsum_partial_vec_kernel<<<dim3(colTiles, chunks), dim3(32, 8), 0, ctx->stream>>>(x, rows, cols, ld, rowsPerChunk, ctx->ws);
    else colsum_partial_kernel<<<dim3(colTiles, chunks), dim3(32, 8), 0, ctx->stream>>>(x, rows, cols, ld, rowsPerChunk, ctx->ws);
    B200_LAUNCH_CHECK(ctx);
    colsum_final_kernel<<<(cols + 255) / 256, 256, 0, ctx->stream>>>(ctx->ws, chunks, cols, out, accumulate);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

// ------------------------------------------------------------------------------------------------ argmax (greedy decoding)
// out[0] = index of the largest of x[0..n) (the lowest index among equals); one block.
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ x, int n, int32_t* __restrict__ out) {
    __shared__ float sv[32];
    __shared__ int si[32];
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = x[i];
        if (v > bv || (v == bv && i < bi) || bi == 0x7fffffff) { if (v > bv || bi == 0x7fffffff || (v == bv && i < bi)) { bv = v; bi = i; } }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int warps = (blockDim.x + 31) >> 5;
        bv = threadIdx.x < warps ? sv[threadIdx.x] : -INFINITY;
        bi = threadIdx.x < warps ? si[threadIdx.x] : 0x7fffffff;
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (threadIdx.x == 0) out[0] = bi == 0x7fffffff ? 0 : bi;
    }
}
int k_argmax(b200_ctx* ctx, const float* x, int n, int32_t* out) {
    if (n <= 0) return B200_OK;
    argmax_kernel<<<1, 1024, 0, ctx->stream>>>(x, n, out);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

// ------------------------------------------------------------------------------------------------ embedding
__global__ void embed_kernel(const int32_t* __restrict__ ids, int count, const float* __restrict__ emb, int d, float* __restrict__ out, int vec) {
    int row = blockIdx.x;
    if (row >= count) return;
    const float* src = emb + (size_t)ids[row] * d;
    float* dst = out + (size_t)row * d;
    if (vec) {
        const float4* s4 = reinterpret_cast<const float4*>(src);
        float4* d4 = reinterpret_cast<float4*>(dst);
        for (int k = threadIdx.x; k < (d >> 2); k += blockDim.x) d4[k] = s4[k];
    } else {
        for (int k = threadIdx.x; k < d; k += blockDim.x) dst[k] = src[k];
    }
}
int k_embed(b200_ctx* ctx, const int32_t* ids, int count, const float* emb, int d, float* out) {
    if (count <= 0) return B200_OK;
    int vec = (d % 4 == 0) && aligned16(emb) && aligned16(out);
    embed_kernel<<<count, d >= 512 ? 128 : 64, 0, ctx->stream>>>(ids, count, emb, d, out, vec);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

// One block column-slice per vocabulary row that occurs in the batch; rows are added in ascending original order,
// exactly the order of the reference's serial scatter, so the result does not depend on scheduling.
__global__ void embed_scatter_kernel(float* __restrict__ eg, const float* __restrict__ a, const float* __restrict__ b,
                                     const int32_t* __restrict__ seg_id, const int32_t* __restrict__ seg_off,
                                     const int32_t* __restrict__ perm, int d) {
    int s = blockIdx.x;
    int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= d) return;
    int lo = seg_off[s], hi = seg_off[s + 1];
    float* dst = eg + (size_t)seg_id[s] * d + c;
    float acc = *dst;
    for (int k = lo; k < hi; k++) {
        size_t r = (size_t)perm[k] * d + c;
        float v = a[r];
        if (b) v += b[r];
        acc += v;
    }
    *dst = acc;
}

// The same for row widths that are multiples of 4 (16-byte aligned arenas): four columns per thread, and the rows of a
// segment are fetched U at a time before they are added -- in the same ascending order, so the sums are bit for bit those
// of the serial loop.  A token that fills a tenth of the batch (Zipf ids) is a chain of thousands of dependent
// additions for one block; issuing its loads one by one made that chain, not the memory system, set the kernel's time.
template <int U>
__global__ void __launch_bounds__(128) embed_scatter_vec_kernel(float* __restrict__ eg, const float* __restrict__ a,
                                                                const int32_t* __restrict__ seg_id, const int32_t* __restrict__ seg_off,
                                                                const int32_t* __restrict__ perm, int d) {
    const int s = blockIdx.x;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (c >= d) return;
    const int lo = seg_off[s], hi = seg_off[s + 1];
    float4* dst = reinterpret_cast<float4*>(eg + (size_t)seg_id[s] * d + c);
    float4 acc = *dst;
    int k = lo;
    // Index -> row is a chain of two loads, and one group's rows in flight do not fill the memory pipeline of a block that
    // owns a long segment: the indices run two groups ahead of the additions, and the rows of the NEXT group are asked
    // of L2 (prefetch, no registers) while this group's rows travel.
    int cur[U], nx[U];
    if (k + U <= hi) {
#pragma unroll
        for (int u = 0; u < U; u++) cur[u] = perm[k + u];
    }
    if (k + 2 * U <= hi) {
#pragma unroll
        for (int u = 0; u < U; u++) nx[u] = perm[k + U + u];
    }
    for (; k + U <= hi; k += U) {
        float4 v[U];
#pragma unroll
        for (int u = 0; u < U; u++) v[u] = *reinterpret_cast<const float4*>(a + (size_t)cur[u] * d + c);
        int nn[U];
        if (k + 2 * U <= hi) {
#pragma unroll
            for (int u = 0; u < U; u++) asm volatile("prefetch.global.L2 [%0];" ::"l"(a + (size_t)nx[u] * d + c));
        }
        if (k + 3 * U <= hi) {
#pragma unroll
            for (int u = 0; u < U; u++) nn[u] = perm[k + 2 * U + u];
        }
#pragma unroll
        for (int u = 0; u < U; u++) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
#pragma unroll
        for (int u = 0; u < U; u++) { cur[u] = nx[u]; nx[u] = nn[u]; }
    }
    for (; k < hi; k++) {
        const float4 x = *reinterpret_cast<const float4*>(a + (size_t)perm[k] * d + c);
        acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
    }
    *dst = acc;
}

int k_embed_scatter(b200_ctx* ctx, float* eg, const float* a, const float* b, const int32_t* seg_id, const int32_t* seg_off,
                    const int32_t* perm, int nSeg, int d) {
    if (nSeg <= 0) return B200_OK;
    if (!b && d % 4 == 0 && aligned16(eg) && aligned16(a)) {
        const int threads = d >= 512 ? 128 : ((d / 4 + 31) / 32) * 32;
        embed_scatter_vec_kernel<16><<<dim3(nSeg, (d / 4 + threads - 1) / threads), threads, 0, ctx->stream>>>(eg, a, seg_id, seg_off, perm, d);
        B200_LAUNCH_CHECK(ctx);
        return B200_OK;
    }
    int threads = d >= 128 ? 128 : ((d + 31) / 32) * 32;
    embed_scatter_kernel<<<dim3(nSeg, (d + threads - 1) / threads), threads, 0, ctx->stream>>>(eg, a, b, seg_id, seg_off, perm, d);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

// ------------------------------------------------------------------------------------------------ rotary embedding
__global__ void rope_kernel(float* __restrict__ base, int64_t matStride, int count, int rows, int ld, int startCol, int numHeads,
                            int headDim, const float2* __restrict__ table, const int32_t* __restrict__ pos, int inverse, int round_tf32) {
    int pairs = headDim >> 1;
    int64_t perMat = (int64_t)rows * numHeads * pairs;
    int64_t total = perMat * count;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int m = (int)(i / perMat);
        int64_t r = i - (int64_t)m * perMat;
        int row = (int)(r / (numHeads * pairs));
        int hp = (int)(r - (int64_t)row * numHeads * pairs);
        int h = hp / pairs, p = hp - h * pairs;
        int ps = pos ? pos[row] : row;
        float2 cs = table[(size_t)ps * pairs + p];
        float sn = inverse ? -cs.y : cs.y;
        float2* ptr = reinterpret_cast<float2*>(base + m * matStride + (size_t)row * ld + startCol + h * headDim + 2 * p);
        float2 x = *ptr;
        float2 y;
        y.x = x.x * cs.x - x.y * sn;
        y.y = x.x * sn + x.y * cs.x;
        if (round_tf32) {
            uint32_t u0, u1;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u0) : "f"(y.x));
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u1) : "f"(y.y));
            y.x = __uint_as_float(u0); y.y = __uint_as_float(u1);
        }
        *ptr = y;
    }
}
__global__ void rope_kernel_scalar(float* __restrict__ base, int64_t matStride, int count, int rows, int ld, int startCol, int numHeads,
                                   int headDim, const float* __restrict__ table, const int32_t* __restrict__ pos, int inverse, int round_tf32) {
    int pairs = headDim >> 1;
    int64_t perMat = (int64_t)rows * numHeads * pairs;
    int64_t total = perMat * count;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int m = (int)(i / perMat);
        int64_t r = i - (int64_t)m * perMat;
        int row = (int)(r / (numHeads * pairs));
        int hp = (int)(r - (int64_t)row * numHeads * pairs);
        int h = hp / pairs, p = hp - h * pairs;
        int ps = pos ? pos[row] : row;
        float c = table[((size_t)ps * pairs + p) * 2], sn = table[((size_t)ps * pairs + p) * 2 + 1];
        if (inverse) sn = -sn;
        float* ptr = base + m * matStride + (size_t)row * ld + startCol + h * headDim + 2 * p;
        float x0 = ptr[0], x1 = ptr[1];
        float y0 = x0 * c - x1 * sn, y1 = x0 * sn + x1 * c;
        if (round_tf32) {
            uint32_t u0, u1;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u0) : "f"(y0));
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u1) : "f"(y1));
            y0 = __uint_as_float(u0); y1 = __uint_as_float(u1);
        }
        ptr[0] = y0;
        ptr[1] = y1;
    }
}
int k_rope(b200_ctx* ctx, float* base, int64_t matStride, int count, int rows, int ld, int startCol, int numHeads, int headDim,
           const float* table, const int32_t* pos, int inverse, int round_tf32) {
    int64_t total = (int64_t)count * rows * numHeads * (headDim / 2);
    if (total <= 0) return B200_OK;
    int g = grid_for(total, 256, 148 * 16);
    bool vec = ((uintptr_t)base % 8 == 0) && (matStride % 2 == 0) && (ld % 2 == 0) && (startCol % 2 == 0) && (headDim % 2 == 0);
    if (vec)
        rope_kernel<<<g, 256, 0, ctx->stream>>>(base, matStride, count, rows, ld, startCol, numHeads, headDim,
                                                reinterpret_cast<const float2*>(table), pos, inverse, round_tf32);
    else
        rope_kernel_scalar<<<g, 256, 0, ctx->stream>>>(base, matStride, count, rows, ld, startCol, numHeads, headDim, table, pos, inverse, round_tf32);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

// ------------------------------------------------------------------------------------------------ LayerNorm
// One warp per row.  When the row fits (d % 4 == 0, d <= 1024) it is held in registers as up to 8 float4 per lane, so
// every input is read from memory exactly once; other widths take the looping fallback.
constexpr int LN_MAXV = 8;

template <bool HAS_SUB>
__global__ void __launch_bounds__(128) ln_fwd_vec_kernel(const float* __restrict__ x, const float* __restrict__ sub,
                                                         const float* __restrict__ gamma, const float* __restrict__ beta, int rows,
                                                         int d, float eps, float* __restrict__ out, float* __restrict__ mean,
                                                         float* __restrict__ var, float* __restrict__ normalized,
                                                         float* __restrict__ residual) {
    int lane = threadIdx.x & 31;
    int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    int d4 = d >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x + (size_t)row * d);
    const float4* s4 = HAS_SUB ? reinterpret_cast<const float4*>(sub + (size_t)row * d) : nullptr;
    float4 v[LN_MAXV];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < LN_MAXV; i++) {
        int c = lane + 32 * i;
        if (c < d4) {
            float4 a = x4[c];
            if (HAS_SUB) { float4 b = s4[c]; a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }
            v[i] = a;
            sum += (a.x + a.y) + (a.z + a.w);
        }
    }
    float mu = warp_sum(sum) / d;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < LN_MAXV; i++) {
        int c = lane + 32 * i;
        if (c < d4) {
            float a = v[i].x - mu, b = v[i].y - mu, e = v[i].z - mu, f = v[i].w - mu;
            sq += (a * a + b * b) + (e * e + f * f);
        }
    }
    float vr = warp_sum(sq) / d;
    float inv = 1.0f / sqrtf(vr + eps);
    if (lane == 0) {
        if (mean) mean[row] = mu;
        if (var) var[row] = vr;
    }
    const float4* g4 = reinterpret_cast<const float4*>(gamma);
    const float4* b4 = reinterpret_cast<const float4*>(beta);
#pragma unroll
    for (int i = 0; i < LN_MAXV; i++) {
        int c = lane + 32 * i;
        if (c < d4) {
            float4 a = v[i], g = g4[c], b = b4[c], n, o;
            n.x = (a.x - mu) * inv; n.y = (a.y - mu) * inv; n.z = (a.z - mu) * inv; n.w = (a.w - mu) * inv;
            o.x = g.x * n.x + b.x; o.y = g.y * n.y + b.y; o.z = g.z * n.z + b.z; o.w = g.w * n.w + b.w;
            reinterpret_cast<float4*>(out + (size_t)row * d)[c] = o;
            if (normalized) reinterpret_cast<float4*>(normalized + (size_t)row * d)[c] = n;
            if (residual) reinterpret_cast<float4*>(residual + (size_t)row * d)[c] = a;
        }
    }
}

__global__ void ln_fwd_generic_kernel(const float* __restrict__ x, const float* __restrict__ sub, const float* __restrict__ gamma,
                                      const float* __restrict__ beta, int rows, int d, float eps, float* __restrict__ out,
                                      float* __restrict__ mean, float* __restrict__ var, float* __restrict__ normalized,
                                      float* __restrict__ residual) {
    int lane = threadIdx.x & 31;
    int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float* xr = x + (size_t)row * d;
    const float* sr = sub ? sub + (size_t)row * d : nullptr;
    float sum = 0.f;
    for (int c = lane; c < d; c += 32) sum += xr[c] + (sr ? sr[c] : 0.f);
    float mu = warp_sum(sum) / d;
    float sq = 0.f;
    for (int c = lane; c < d; c += 32) {
        float a = xr[c] + (sr ? sr[c] : 0.f) - mu;
        sq += a * a;
    }
    float vr = warp_sum(sq) / d;
    float inv = 1.0f / sqrtf(vr + eps);
    if (lane == 0) {
        if (mean) mean[row] = mu;
        if (var) var[row] = vr;
    }
    for (int c = lane; c < d; c += 32) {
        float a = xr[c] + (sr ? sr[c] : 0.f);
        float n = (a - mu) * inv;
        out[(size_t)row * d + c] = gamma[c] * n + beta[c];
        if (normalized) normalized[(size_t)row * d + c] = n;
        if (residual) residual[(size_t)row * d + c] = a;
    }
}

int k_ln_forward(b200_ctx* ctx, const float* x, const float* sub, const float* gamma, const float* beta, int rows, int d, float eps,
                 float* out, float* mean, float* var, float* normalized, float* residual) {
    if (rows <= 0 || d <= 0) return B200_OK;
    bool vec = (d % 4 == 0) && d <= 128 * LN_MAXV && aligned16(x) && (!sub || aligned16(sub)) && aligned16(gamma) && aligned16(beta) &&
               aligned16(out) && (!normalized || aligned16(normalized)) && (!residual || aligned16(residual));
    int grid = (rows + 3) / 4;
    if (vec) {
        if (sub) ln_fwd_vec_kernel<true><<<grid, 128, 0, ctx->stream>>>(x, sub, gamma, beta, rows, d, eps, out, mean, var, normalized, residual);
        else ln_fwd_vec_kernel<false><<<grid, 128, 0, ctx->stream>>>(x, sub, gamma, beta, rows, d, eps, out, mean, var, normalized, residual);
    } else {
        ln_fwd_generic_kernel<<<grid, 128, 0, ctx->stream>>>(x, sub, gamma, beta, rows, d, eps, out, mean, var, normalized, residual);
    }
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

// Backward: each warp walks rows row0, row0+W, ... (W = warps in the grid), keeps its columns' dGamma/dBeta partial
// sums in registers, and the block writes one partial row per block; a second kernel adds the partial rows in block
// order (deterministic).  dx = dNorm*invStd + (2/n)*dVar*(x-mean) + dMean/n with
// dVar = -0.5*invStd^3*sum(dNorm*(x-mean)), dMean = -invStd*sum(dNorm)  (the reference's formulation).
template <bool HAS_B, bool DXSUM = false>
__global__ void __launch_bounds__(128, 4) ln_bwd_vec_kernel(const float* __restrict__ dOutA, const float* __restrict__ dOutB,
                                                            const float* __restrict__ x, const float* __restrict__ gamma,
                                                            const float* __restrict__ mean, const float* __restrict__ var, int rows,
                                                            int d, float eps, float* __restrict__ dx, float* __restrict__ partial) {
    // The dGamma/dBeta partial sums of a warp live in its own shared-memory slice (every lane owns its columns, so
    // there is nothing to synchronise) instead of 64 registers per thread: the kernel is bound by how many rows are in
    // flight per SM, and the registers it does not hold become resident warps.
    // With DXSUM a third slice accumulates the column sums of dx: the bias gradient of the linear layer that feeds
    // this LayerNorm, which would otherwise cost another pass over dx.
    constexpr int NACC = DXSUM ? 3 : 2;
    extern __shared__ float sm[];  // [warps][NACC*d]
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    int d4 = d >> 2;
    const float4* g4 = reinterpret_cast<const float4*>(gamma);
    float4* smg = reinterpret_cast<float4*>(sm + (size_t)warp * NACC * d);
    float4* smb = reinterpret_cast<float4*>(sm + (size_t)warp * NACC * d + d);
    float4* smx = reinterpret_cast<float4*>(sm + (size_t)warp * NACC * d + 2 * d);  // only touched with DXSUM
#pragma unroll
    for (int i = 0; i < LN_MAXV; i++) {
        int c = lane + 32 * i;
        if (c < d4) {
            smg[c] = make_float4(0, 0, 0, 0); smb[c] = make_float4(0, 0, 0, 0);
            if (DXSUM) smx[c] = make_float4(0, 0, 0, 0);
        }
    }
    float invN = 1.0f / d;
    for (int row = blockIdx.x * warps + warp; row < rows; row += gridDim.x * warps) {
        const float4* a4 = reinterpret_cast<const float4*>(dOutA + (size_t)row * d);
        const float4* b4 = HAS_B ? reinterpret_cast<const float4*>(dOutB + (size_t)row * d) : nullptr;
        const float4* x4 = reinterpret_cast<const float4*>(x + (size_t)row * d);
        float mu = mean[row];
        float inv = 1.0f / sqrtf(var[row] + eps);
        {   // ask L2 for this warp's next row while this one is worked on (one lane per 128-byte line)
            const int nrow = row + gridDim.x * warps;
            if (nrow < rows && (lane & 7) == 0) {
#pragma unroll
                for (int i = 0; i < LN_MAXV; i++) {
                    const int c = lane + 32 * i;
                    if (c < d4) {
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(dOutA + (size_t)nrow * d + 4 * c));
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(x + (size_t)nrow * d + 4 * c));
                        if (HAS_B) asm volatile("prefetch.global.L2 [%0];" ::"l"(dOutB + (size_t)nrow * d + 4 * c));
                    }
                }
            }
        }
        float4 dn[LN_MAXV], xm[LN_MAXV];
#pragma unroll
        for (int i = 0; i < LN_MAXV; i++) {  // all loads of the row first
            int c = lane + 32 * i;
            if (c < d4) {
                float4 o = a4[c];
                if (HAS_B) { float4 p = b4[c]; o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w; }
                dn[i] = o;
                xm[i] = x4[c];
            }
        }
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int i = 0; i < LN_MAXV; i++) {
            int c = lane + 32 * i;
            if (c < d4) {
                const float4 o = dn[i];
                float4 xv = xm[i];
                xv.x -= mu; xv.y -= mu; xv.z -= mu; xv.w -= mu;
                xm[i] = xv;
                float4 g = smg[c], bb = smb[c];
                g.x += o.x * (xv.x * inv); g.y += o.y * (xv.y * inv); g.z += o.z * (xv.z * inv); g.w += o.w * (xv.w * inv);
                bb.x += o.x; bb.y += o.y; bb.z += o.z; bb.w += o.w;
                smg[c] = g; smb[c] = bb;
                const float4 gm = __ldg(g4 + c);
                float4 n;
                n.x = o.x * gm.x; n.y = o.y * gm.y; n.z = o.z * gm.z; n.w = o.w * gm.w;
                dn[i] = n;
                s1 += (n.x * xv.x + n.y * xv.y) + (n.z * xv.z + n.w * xv.w);
                s2 += (n.x + n.y) + (n.z + n.w);
            }
        }
        s1 = warp_sum(s1);
        s2 = warp_sum(s2);
        float dVarScale = s1 * (-0.5f) * inv * inv * inv * 2.0f * invN;
        float dMeanScale = s2 * (-inv) * invN;
#pragma unroll
        for (int i = 0; i < LN_MAXV; i++) {
            int c = lane + 32 * i;
            if (c < d4) {
                float4 r;
                r.x = dn[i].x * inv + dVarScale * xm[i].x + dMeanScale;
                r.y = dn[i].y * inv + dVarScale * xm[i].y + dMeanScale;
                r.z = dn[i].z * inv + dVarScale * xm[i].z + dMeanScale;
                r.w = dn[i].w * inv + dVarScale * xm[i].w + dMeanScale;
                reinterpret_cast<float4*>(dx + (size_t)row * d)[c] = r;
                if (DXSUM) {
                    float4 sx = smx[c];
                    sx.x += r.x; sx.y += r.y; sx.z += r.z; sx.w += r.w;
                    smx[c] = sx;
                }
            }
        }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < NACC * d; c += blockDim.x) {
        float s = 0.f;
        for (int w = 0; w < warps; w++) s += sm[(size_t)w * NACC * d + c];
        partial[(size_t)blockIdx.x * NACC * d + c] = s;
    }
}

__global__ void ln_bwd_generic_kernel(const float* __restrict__ dOutA, const float* __restrict__ dOutB, const float* __restrict__ x,
                                      const float* __restrict__ gamma, const float* __restrict__ mean, const float* __restrict__ var,
                                      int rows, int d, float eps, float* __restrict__ dx) {
    int lane = threadIdx.x & 31;
    int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    float mu = mean[row], inv = 1.0f / sqrtf(var[row] + eps);
    float s1 = 0.f, s2 = 0.f;
    for (int c = lane; c < d; c += 32) {
        float o = dOutA[(size_t)row * d + c] + (dOutB ? dOutB[(size_t)row * d + c] : 0.f);
        float n = o * gamma[c], xm = x[(size_t)row * d + c] - mu;
        s1 += n * xm;
        s2 += n;
    }
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    float invN = 1.0f / d;
    float dVarScale = s1 * (-0.5f) * inv * inv * inv * 2.0f * invN;
    float dMeanScale = s2 * (-inv) * invN;
    for (int c = lane; c < d; c += 32) {
        float o = dOutA[(size_t)row * d + c] + (dOutB ? dOutB[(size_t)row * d + c] : 0.f);
        float n = o * gamma[c], xm = x[(size_t)row * d + c] - mu;
        dx[(size_t)row * d + c] = n * inv + dVarScale * xm + dMeanScale;
    }
}
// grid (colTiles, chunks) like colsum: partial[chunk][0..d) = dGamma, [d..2d) = dBeta.
__global__ void ln_bwd_generic_cols_kernel(const float* __restrict__ dOutA, const float* __restrict__ dOutB, const float* __restrict__ x,
                                           const float* __restrict__ mean, const float* __restrict__ var, int rows, int d, float eps,
                                           int rowsPerChunk, float* __restrict__ partial) {
    __shared__ float sg[8][33], sb[8][33];
    int c = blockIdx.x * 32 + threadIdx.x;
    int r0 = blockIdx.y * rowsPerChunk, r1 = min(rows, r0 + rowsPerChunk);
    float g = 0.f, b = 0.f;
    if (c < d)
        for (int r = r0 + threadIdx.y; r < r1; r += 8) {
            float o = dOutA[(size_t)r * d + c] + (dOutB ? dOutB[(size_t)r * d + c] : 0.f);
            float inv = 1.0f / sqrtf(var[r] + eps);
            g += o * ((x[(size_t)r * d + c] - mean[r]) * inv);
            b += o;
        }
    sg[threadIdx.y][threadIdx.x] = g;
    sb[threadIdx.y][threadIdx.x] = b;
    __syncthreads();
    if (threadIdx.y == 0 && c < d) {
        float tg = 0.f, tb = 0.f;
#pragma unroll
        for (int y = 0; y < 8; y++) { tg += sg[y][threadIdx.x]; tb += sb[y][threadIdx.x]; }
        partial[(size_t)blockIdx.y * 2 * d + c] = tg;
        partial[(size_t)blockIdx.y * 2 * d + d + c] = tb;
    }
}
__global__ void ln_bwd_final_kernel(const float* __restrict__ partial, int parts, int d, float* __restrict__ dGamma,
                                    float* __restrict__ dBeta, int accumulate) {
    int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= 2 * d) return;
    float s = 0.f;
    for (int k = 0; k < parts; k++) s += partial[(size_t)k * 2 * d + c];
    float* dst = c < d ? dGamma + c : dBeta + (c - d);
    *dst = accumulate ? *dst + s : s;
}

// The same final reduction for the training path, where it runs twice per block and pass: 32 columns x 8 slices of
// the partial rows per CTA (a thread of the kernels above walks every partial row of its column, one dependent load
// after the other, which costs ~28 us for 592 rows).  The order of the adds is fixed, so results repeat bit for bit.
// Column index c runs over [dGamma | dBeta | dxColSum] (the third only when dxColSum is given, always accumulated).
__global__ void __launch_bounds__(256) ln_bwd_final_sliced_kernel(const float* __restrict__ partial, int parts, int d, int nacc, float* __restrict__ dGamma,
                                                                  float* __restrict__ dBeta, float* __restrict__ dxColSum, int accumulate) {
    __shared__ float sm[8][33];
    const int c = blockIdx.x * 32 + threadIdx.x, width = nacc * d;
    float s0 = 0.f, s1 = 0.f;
    if (c < width) {
        int k = threadIdx.y;
        for (; k + 8 < parts; k += 16) { s0 += partial[(size_t)k * width + c]; s1 += partial[(size_t)(k + 8) * width + c]; }
        if (k < parts) s0 += partial[(size_t)k * width + c];
    }
    sm[threadIdx.y][threadIdx.x] = s0 + s1;
    __syncthreads();
    if (threadIdx.y != 0 || c >= width) return;
    float s = 0.f;
#pragma unroll
    for (int y = 0; y < 8; y++) s += sm[y][threadIdx.x];
    if (c >= 2 * d) { dxColSum[c - 2 * d] += s; return; }
    float* dst = c < d ? dGamma + c : dBeta + (c - d);
    *dst = accumulate ? *dst + s : s;
}

int k_ln_backward(b200_ctx* ctx, const float* dOutA, const float* dOutB, const float* x, const float* gamma, const float* mean,
                  const float* var, int rows, int d, float eps, float* dx, float* dGamma, float* dBeta, int accumulate, float* dxColSum) {
    if (d <= 0) return B200_OK;
    if (rows <= 0) {
        if (!accumulate) {
            B200_CUDA(ctx, cudaMemsetAsync(dGamma, 0, sizeof(float) * d, ctx->stream));
            B200_CUDA(ctx, cudaMemsetAsync(dBeta, 0, sizeof(float) * d, ctx->stream));
        }
        return B200_OK;
    }
    bool vec = (d % 4 == 0) && d <= 128 * LN_MAXV && aligned16(dOutA) && (!dOutB || aligned16(dOutB)) && aligned16(x) &&
               aligned16(gamma) && aligned16(dx);
    int parts;
    if (vec) {
        int warps = 4;
        int grid = (rows + warps - 1) / warps;
        int cap = ctx->sm_count > 0 ? ctx->sm_count * 4 : 592;
        if (grid > cap) grid = cap;
        parts = grid;
        const int nacc = dxColSum ? 3 : 2;
        B200_TRY(ensure_ws(ctx, (size_t)parts * nacc * d));
        size_t smem = (size_t)warps * nacc * d * sizeof(float);
        if (dxColSum) {
            if (dOutB) ln_bwd_vec_kernel<true, true><<<grid, warps * 32, smem, ctx->stream>>>(dOutA, dOutB, x, gamma, mean, var, rows, d, eps, dx, ctx->ws);
            else ln_bwd_vec_kernel<false, true><<<grid, warps * 32, smem, ctx->stream>>>(dOutA, dOutB, x, gamma, mean, var, rows, d, eps, dx, ctx->ws);
            B200_LAUNCH_CHECK(ctx);
            ln_bwd_final_sliced_kernel<<<(3 * d + 31) / 32, dim3(32, 8), 0, ctx->stream>>>(ctx->ws, parts, d, 3, dGamma, dBeta, dxColSum, accumulate);
            B200_LAUNCH_CHECK(ctx);
            return B200_OK;
        }
        if (dOutB) ln_bwd_vec_kernel<true><<<grid, warps * 32, smem, ctx->stream>>>(dOutA, dOutB, x, gamma, mean, var, rows, d, eps, dx, ctx->ws);
        else ln_bwd_vec_kernel<false><<<grid, warps * 32, smem, ctx->stream>>>(dOutA, dOutB, x, gamma, mean, var, rows, d, eps, dx, ctx->ws);
        B200_LAUNCH_CHECK(ctx);
    } else {
        ln_bwd_generic_kernel<<<(rows + 3) / 4, 128, 0, ctx->stream>>>(dOutA, dOutB, x, gamma, mean, var, rows, d, eps, dx);
        B200_LAUNCH_CHECK(ctx);
        int colTiles = (d + 31) / 32;
        int chunks = (rows + 63) / 64;
        if (chunks > 64) chunks = 64;
        int rowsPerChunk = (rows + chunks - 1) / chunks;
        parts = chunks;
        B200_TRY(ensure_ws(ctx, (size_t)parts * 2 * d));
        ln_bwd_generic_cols_kernel<<<dim3(colTiles, chunks), dim3(32, 8), 0, ctx->stream>>>(dOutA, dOutB, x, mean, var, rows, d, eps,
                                                                                         rowsPerChunk, ctx->ws);
        B200_LAUNCH_CHECK(ctx);
    }
    ln_bwd_final_sliced_kernel<<<(2 * d + 31) / 32, dim3(32, 8), 0, ctx->stream>>>(ctx->ws, parts, d, 2, dGamma, dBeta, nullptr, accumulate);
    B200_LAUNCH_CHECK(ctx);
    if (dxColSum) return k_colsum(ctx, dx, rows, d, d, dxColSum, 1);  // paths without the fused column sum
    return B200_OK;
}

// ------------------------------------------------------------------------------------------------ LayerNorm backward without any allocation
// Scratch for b200_LayerNormBackward_noalloc: the per-block dGamma/dBeta partial rows of the two-stage column
// reduction.  It is part of the library image, so every GPU that loads the library holds these 2.3 MiB until the
// process exits; in exchange the entry point below never asks the driver (or any allocator) for memory.
constexpr int NOALLOC_LN_MAX_FEATURES = 1024;  // widest row the entry point accepts
constexpr int NOALLOC_LN_MAX_PARTS = 296;      // partial rows (blocks) the scratch has room for
static __device__ __align__(256) float g_noalloc_ln_scratch[NOALLOC_LN_MAX_PARTS * 2 * NOALLOC_LN_MAX_FEATURES];

constexpr int NOALLOC_MAX_DEVICES = 64;
static float* g_noalloc_ln_ptr[NOALLOC_MAX_DEVICES];  // device address of the scratch, per device ordinal (0 = not set up yet)
static std::mutex g_noalloc_mu;

}  // namespace b200

extern "C" int32_t b200_LayerNormBackward_noalloc(void* cuda_stream, const float* dOut, const float* input, const float* gamma, const float* mean,
                                                  const float* variance, int32_t rows, int32_t features, float eps, float* dInput, float* dGamma,
                                                  float* dBeta) {
    using namespace b200;
    auto reject = [](int code, const char* why) {
        fprintf(stderr, "b200_LayerNormBackward_noalloc: %s\n", why);
        return code;
    };
    if (!dOut || !input || !gamma || !mean || !variance || !dInput || !dGamma || !dBeta) return reject(B200_ERR_INVALID_ARG, "null device pointer");
    if (rows <= 0 || features <= 0) return reject(B200_ERR_INVALID_ARG, "rows and features must be positive");
    if (features > NOALLOC_LN_MAX_FEATURES)
        return reject(B200_ERR_OUT_OF_RANGE, "features exceeds the built-in scratch (maximum 1024 columns); use b200_LayerNormBackward");
    if (features % 4 != 0) return reject(B200_ERR_UNSUPPORTED, "features must be a multiple of 4");
    if (!aligned16(dOut) || !aligned16(input) || !aligned16(gamma) || !aligned16(dInput))
        return reject(B200_ERR_UNSUPPORTED, "dOut, input, gamma and dInput must be 16-byte aligned");
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) return reject(B200_ERR_CUDA, "no current CUDA device");
    float* scratch = nullptr;
    {
        // Set-up, once per device, with that device current: in host code the array's name is only a stand-in for
        // the device object, so its device address has to be asked for before a kernel can be given it.
        std::lock_guard<std::mutex> lock(g_noalloc_mu);
        if (!g_noalloc_ln_ptr[dev]) {
            float* p = nullptr;
            cudaError_t e = cudaGetSymbolAddress((void**)&p, g_noalloc_ln_scratch);
            if (e != cudaSuccess || !p) {
                fprintf(stderr, "b200_LayerNormBackward_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
                return B200_ERR_CUDA;
            }
            g_noalloc_ln_ptr[dev] = p;
        }
        scratch = g_noalloc_ln_ptr[dev];
    }
    cudaStream_t st = (cudaStream_t)cuda_stream;
    (void)cudaGetLastError();  // a stale error of an earlier, unrelated call must not be reported as this call's launch failure
    const int warps = 4;
    int grid = (rows + warps - 1) / warps;
    if (grid > NOALLOC_LN_MAX_PARTS) grid = NOALLOC_LN_MAX_PARTS;
    const size_t smem = (size_t)warps * 2 * features * sizeof(float);
    // Every partial row the second kernel reads (grid of them) is written in full by the first one, so nothing in the
    // scratch has to start at zero and nothing left by an earlier call can leak into this one.
    ln_bwd_vec_kernel<false><<<grid, warps * 32, smem, st>>>(dOut, nullptr, input, gamma, mean, variance, rows, features, eps, dInput, scratch);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) {
        ln_bwd_final_kernel<<<(2 * features + 255) / 256, 256, 0, st>>>(scratch, grid, features, dGamma, dBeta, 0);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) {
        fprintf(stderr, "b200_LayerNormBackward_noalloc: kernel launch failed: %s\n", cudaGetErrorString(e));
        return B200_ERR_CUDA;
    }
    return B200_OK;
}

namespace b200 {

// ------------------------------------------------------------------------------------------------ losses
// One block per row; the row lives in registers (up to 32 values per thread), so logits are read once and the
// gradient written once even when it overwrites the logits.
constexpr int CE_ITEMS = 32;

template <int THREADS>
__global__ void __launch_bounds__(THREADS) ce_kernel(const float* __restrict__ logits, int V, const int32_t* __restrict__ targets,
                                                     int effRows, const float* __restrict__ row_scale_dev, float row_scale,
                                                     float* __restrict__ dLogits, float* __restrict__ row_loss,
                                                     int32_t* __restrict__ row_ok) {
    __shared__ float red[32];
    __shared__ float s_pt;
    int row = blockIdx.x;
    float* dl = dLogits + (size_t)row * V;
    if (row >= effRows) {
        for (int j = threadIdx.x; j < V; j += THREADS) dl[j] = 0.f;
        return;
    }
    const float* l = logits + (size_t)row * V;
    if (threadIdx.x == 0) s_pt = 0.f;  // ordered before its use by the barriers inside the reductions
    float v[CE_ITEMS];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < CE_ITEMS; i++) {
        int j = threadIdx.x + i * THREADS;
        v[i] = j < V ? l[j] : -INFINITY;
        mx = fmaxf(mx, v[i]);
    }
    mx = block_max(mx, red);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < CE_ITEMS; i++) {
        int j = threadIdx.x + i * THREADS;
        if (j < V) { v[i] = expf(v[i] - mx); sum += v[i]; }
    }
    sum = block_sum(sum, red);
    float inv = 1.0f / sum;
    int t = targets[row];
    float sc = row_scale_dev ? row_scale_dev[row] : row_scale;
    int ok = (unsigned)t < (unsigned)V ? 1 : 0;  // a target outside the row marks the row invalid instead of reading out of range
#pragma unroll
    for (int i = 0; i < CE_ITEMS; i++) {
        int j = threadIdx.x + i * THREADS;
        if (j < V) {
            if (j == t) s_pt = v[i];
            float g = (v[i] * inv) * sc;
            if (j == t) g -= sc;
            ok &= isfinite(g) ? 1 : 0;
            dl[j] = g;
        }
    }
    ok = __syncthreads_and(ok);
    if (threadIdx.x == 0) {
        row_loss[row] = -logf(s_pt * inv + 1e-10f);
        row_ok[row] = ok;
    }
}

// Larger vocabularies, or V not a multiple of 16 (V a multiple of 4, 16-byte aligned rows): one block of 256 threads per row, several blocks per SM.
// Pass 1 streams the row once with 128-bit loads and keeps a running (max, sum of exp) pair per thread; pass 2 reads the
// row again (about a third of those reads still hit L2 with eight blocks per SM in flight; capping the blocks per SM to
// raise the hit rate cost more in latency hiding than it saved in traffic) and writes the gradient.  The loads of one
// block overlap the reductions and stores of the others, which the one-block-per-SM register-resident kernel cannot do.
// (Up to 32768 classes ce_cluster_kernel reads the row once.  A persistent block per SM that stages the row through shared
// memory and prefetches the next one was built too: 10 % faster than this kernel alone under the profiler, 5-9 % slower
// inside the power-capped step, where a single block per SM cannot hide latency at the lower clock: not kept.)
__global__ void __launch_bounds__(256) ce_twopass_kernel(const float* __restrict__ logits, int V, const int32_t* __restrict__ targets,
                                                         int effRows, const float* __restrict__ row_scale_dev, float row_scale,
                                                         float* __restrict__ dLogits, float* __restrict__ row_loss,
                                                         int32_t* __restrict__ row_ok) {
    __shared__ float red_m[8], red_s[8];
    __shared__ float s_pt;
    const int row = blockIdx.x, V4 = V >> 2, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float4* dl4 = reinterpret_cast<float4*>(dLogits + (size_t)row * V);
    if (row >= effRows) {
        for (int j = threadIdx.x; j < V4; j += 256) dl4[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        return;
    }
    const float4* l4 = reinterpret_cast<const float4*>(logits + (size_t)row * V);
    if (threadIdx.x == 0) s_pt = 0.f;
    float m = -INFINITY, sum = 0.f;
    for (int j = threadIdx.x; j < V4; j += 256) {
        const float4 x = l4[j];
        const float m4 = fmaxf(fmaxf(x.x, x.y), fmaxf(x.z, x.w));
        if (m4 > m) {  // -inf rows stay at (m = -inf, sum = 0) until a finite value arrives
            sum *= __expf(m - m4);
            m = m4;
        }
        if (m != -INFINITY) sum += (__expf(x.x - m) + __expf(x.y - m)) + (__expf(x.z - m) + __expf(x.w - m));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float mo = __shfl_xor_sync(0xffffffffu, m, o), so = __shfl_xor_sync(0xffffffffu, sum, o);
        const float mn = fmaxf(m, mo);
        sum = (mn == -INFINITY) ? 0.f : sum * __expf(m - mn) + so * __expf(mo - mn);
        m = mn;
    }
    if (lane == 0) { red_m[warp] = m; red_s[warp] = sum; }
    __syncthreads();
    float M = red_m[0];
#pragma unroll
    for (int w = 1; w < 8; w++) M = fmaxf(M, red_m[w]);
    float S = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) S += (red_m[w] == -INFINITY) ? 0.f : red_s[w] * __expf(red_m[w] - M);
    const float inv = 1.0f / S;
    const int t = targets[row];
    const float sc = row_scale_dev ? row_scale_dev[row] : row_scale;
    int ok = (unsigned)t < (unsigned)V ? 1 : 0;  // a target outside the row marks the row invalid instead of reading out of range
    for (int j = threadIdx.x; j < V4; j += 256) {
        const float4 x = l4[j];
        float e[4] = {expf(x.x - M), expf(x.y - M), expf(x.z - M), expf(x.w - M)};
        float g[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            g[k] = (e[k] * inv) * sc;
            if (4 * j + k == t) { s_pt = e[k]; g[k] -= sc; }
            ok &= isfinite(g[k]) ? 1 : 0;
        }
        dl4[j] = make_float4(g[0], g[1], g[2], g[3]);
    }
    ok = __syncthreads_and(ok);
    if (threadIdx.x == 0) {
        row_loss[row] = -logf(s_pt * inv + 1e-10f);
        row_ok[row] = ok;
    }
}

// Vocabularies of 8192..32768 classes (V a multiple of 16, 16-byte aligned rows) on devices with thread-block clusters:
// a cluster of four blocks of 256 threads per row, each block holding its quarter of the row in registers (8 x float4
// per thread).  The quarter maxima and the quarter sums of exp are exchanged through distributed shared memory (two
// cluster barriers per row); logits are read once and the gradient is written once from registers -- 8 B per element,
// against the 12 B of the two-pass kernel below, whose second read misses L2 two times out of three -- and with five
// blocks resident per SM the loads of one row overlap the reductions and stores of the others.  Same arithmetic as
// ce_kernel: maximum, exp(x - max), sum, p / sum.  A row is non-finite exactly when its sum of exp (or its scale) is:
// every exp lies in [0, sum], and a NaN or +inf logit makes the sum NaN.
constexpr int CE_CL = 4, CE_CL_THREADS = 256, CE_CL_ITEMS = 8;
__global__ void __launch_bounds__(CE_CL_THREADS, 5) ce_cluster_kernel(const float* __restrict__ logits, int V, const int32_t* __restrict__ targets,
                                                                      int effRows, const float* __restrict__ row_scale_dev, float row_scale,
                                                                      float* __restrict__ dLogits, float* __restrict__ row_loss,
                                                                      int32_t* __restrict__ row_ok) {
    __shared__ float red[8];
    __shared__ float xmax[CE_CL], xsum[CE_CL];  // written by the four blocks of the cluster, one slot each
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int row = blockIdx.x / CE_CL, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int Q4 = V >> 4;                 // float4 per quarter row
    const int base4 = (int)rank * Q4;      // this block's first float4 of the row
    float4* dl4 = reinterpret_cast<float4*>(dLogits + (size_t)row * V) + base4;
    if (row >= effRows) {  // all four blocks of a cluster take this branch together: no barrier is skipped by a part of it
        for (int j = tid; j < Q4; j += CE_CL_THREADS) dl4[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        return;
    }
    const float4* l4 = reinterpret_cast<const float4*>(logits + (size_t)row * V) + base4;
    float4 v[CE_CL_ITEMS];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < CE_CL_ITEMS; i++) {
        const int j = tid + i * CE_CL_THREADS;
        v[i] = j < Q4 ? l4[j] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        mx = fmaxf(mx, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
    }
    auto publish = [&](float* slot_array, float value) {  // value of this block into slot [rank] of every block of the cluster
        const uint32_t local = (uint32_t)__cvta_generic_to_shared(slot_array + rank);
#pragma unroll
        for (uint32_t r = 0; r < CE_CL; r++) {
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(r));
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(value) : "memory");
        }
    };
    auto cluster_barrier = [] {
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    };
    mx = warp_max(mx);
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    if (tid == 0) {
        float m = red[0];
#pragma unroll
        for (int w = 1; w < 8; w++) m = fmaxf(m, red[w]);
        publish(xmax, m);
    }
    cluster_barrier();
    const float M = fmaxf(fmaxf(xmax[0], xmax[1]), fmaxf(xmax[2], xmax[3]));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < CE_CL_ITEMS; i++) {  // padding lanes hold -inf: exp gives 0
        v[i].x = expf(v[i].x - M); v[i].y = expf(v[i].y - M); v[i].z = expf(v[i].z - M); v[i].w = expf(v[i].w - M);
        sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
    sum = warp_sum(sum);
    if (lane == 0) red[warp] = sum;  // the maxima in red were consumed before the cluster barrier
    __syncthreads();
    if (tid == 0) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 8; w++) t += red[w];
        publish(xsum, t);
    }
    cluster_barrier();
    const float S = (xsum[0] + xsum[1]) + (xsum[2] + xsum[3]);
    const float inv = 1.0f / S;
    const int t = targets[row];
    const float sc = row_scale_dev ? row_scale_dev[row] : row_scale;
    const int tq = t - 4 * base4;  // the target's column within this quarter (outside [0, 4*Q4): another block's, or invalid)
#pragma unroll
    for (int i = 0; i < CE_CL_ITEMS; i++) {
        const int j = tid + i * CE_CL_THREADS;
        if (j < Q4) {
            float e[4] = {v[i].x, v[i].y, v[i].z, v[i].w}, g[4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                g[k] = (e[k] * inv) * sc;
                if (4 * j + k == tq) {  // exactly one thread of the cluster owns the target column: it reports the row
                    g[k] -= sc;
                    row_loss[row] = -logf(e[k] * inv + 1e-10f);
                }
            }
            dl4[j] = make_float4(g[0], g[1], g[2], g[3]);
        }
    }
    if (rank == 0 && tid == 0) {
        const bool in_range = (unsigned)t < (unsigned)V;  // a target outside the row marks the row invalid instead of reading out of range
        if (!in_range) row_loss[row] = -logf(1e-10f);     // what the other kernels report when no column matches (s_pt = 0)
        row_ok[row] = (in_range && isfinite(S) && isfinite(sc)) ? 1 : 0;
    }
}

// Any vocabulary size: three passes over the row in global memory (not in-place safe w.r.t. partial overwrite, so the
// gradient is written only in the last pass, after every read of the same element by the same thread).
__global__ void ce_generic_kernel(const float* __restrict__ logits, int V, const int32_t* __restrict__ targets, int effRows,
                                  const float* __restrict__ row_scale_dev, float row_scale, float* __restrict__ dLogits,
                                  float* __restrict__ row_loss, int32_t* __restrict__ row_ok) {
    __shared__ float red[32];
    int row = blockIdx.x;
    float* dl = dLogits + (size_t)row * V;
    if (row >= effRows) {
        for (int j = threadIdx.x; j < V; j += blockDim.x) dl[j] = 0.f;
        return;
    }
    const float* l = logits + (size_t)row * V;
    float mx = -INFINITY;
    for (int j = threadIdx.x; j < V; j += blockDim.x) mx = fmaxf(mx, l[j]);
    mx = block_max(mx, red);
    float sum = 0.f;
    for (int j = threadIdx.x; j < V; j += blockDim.x) sum += expf(l[j] - mx);
    sum = block_sum(sum, red);
    float inv = 1.0f / sum;
    int t = targets[row];
    float sc = row_scale_dev ? row_scale_dev[row] : row_scale;
    int ok = (unsigned)t < (unsigned)V ? 1 : 0;
    float pt = ok ? expf(l[t] - mx) : 0.f;
    __syncthreads();  // every thread has read l[t] before any thread overwrites it
    for (int j = threadIdx.x; j < V; j += blockDim.x) {
        float g = (expf(l[j] - mx) * inv) * sc;
        if (j == t) g -= sc;
        ok &= isfinite(g) ? 1 : 0;
        dl[j] = g;
    }
    ok = __syncthreads_and(ok);
    if (threadIdx.x == 0) {
        row_loss[row] = -logf(pt * inv + 1e-10f);
        row_ok[row] = ok;
    }
}

int k_cross_entropy(b200_ctx* ctx, const float* logits, int rows, int V, const int32_t* targets, int effRows, const float* row_scale_dev,
                    float row_scale, float* dLogits, float* row_loss, int32_t* row_ok) {
    if (rows <= 0 || V <= 0) return B200_OK;
    const bool big = V >= 8192 && (V % 4 == 0) && aligned16(logits) && aligned16(dLogits);
    if (big && V % 16 == 0 && V <= CE_CL * CE_CL_THREADS * CE_CL_ITEMS * 4 && ctx->cc_major >= 9) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)rows * CE_CL);
        cfg.blockDim = dim3(CE_CL_THREADS);
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = CE_CL; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        B200_CUDA(ctx, cudaLaunchKernelEx(&cfg, ce_cluster_kernel, logits, V, targets, effRows, row_scale_dev, row_scale, dLogits, row_loss, row_ok));
    } else if (big) ce_twopass_kernel<<<rows, 256, 0, ctx->stream>>>(logits, V, targets, effRows, row_scale_dev, row_scale, dLogits, row_loss, row_ok);
    else if (V <= 128 * CE_ITEMS) ce_kernel<128><<<rows, 128, 0, ctx->stream>>>(logits, V, targets, effRows, row_scale_dev, row_scale, dLogits, row_loss, row_ok);
    else if (V <= 256 * CE_ITEMS) ce_kernel<256><<<rows, 256, 0, ctx->stream>>>(logits, V, targets, effRows, row_scale_dev, row_scale, dLogits, row_loss, row_ok);
    else if (V <= 1024 * CE_ITEMS) ce_kernel<1024><<<rows, 1024, 0, ctx->stream>>>(logits, V, targets, effRows, row_scale_dev, row_scale, dLogits, row_loss, row_ok);
    else ce_generic_kernel<<<rows, 1024, 0, ctx->stream>>>(logits, V, targets, effRows, row_scale_dev, row_scale, dLogits, row_loss, row_ok);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

__global__ void mse_kernel(const float* __restrict__ pred, int rows, int O, const float* __restrict__ targets, int effRows,
                           const float* __restrict__ row_scale_dev, float row_scale, float* __restrict__ dOut,
                           float* __restrict__ row_loss, int32_t* __restrict__ row_ok) {
    int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) return;
    if (row >= effRows) {
        for (int j = 0; j < O; j++) dOut[(size_t)row * O + j] = 0.f;
        return;
    }
    float sc = row_scale_dev ? row_scale_dev[row] : row_scale;
    float loss = 0.f;
    int ok = 1;
    for (int j = 0; j < O; j++) {
        float diff = pred[(size_t)row * O + j] - targets[(size_t)row * O + j];
        loss += diff * diff;
        float g = 2.0f * diff * sc;
        ok &= isfinite(g) ? 1 : 0;
        dOut[(size_t)row * O + j] = g;
    }
    row_loss[row] = loss;
    row_ok[row] = ok;
}
int k_mse(b200_ctx* ctx, const float* pred, int rows, int O, const float* targets, int effRows, const float* row_scale_dev, float row_scale,
          float* dOut, float* row_loss, int32_t* row_ok) {
    if (rows <= 0 || O <= 0) return B200_OK;
    mse_kernel<<<(rows + 127) / 128, 128, 0, ctx->stream>>>(pred, rows, O, targets, effRows, row_scale_dev, row_scale, dOut, row_loss, row_ok);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

// ------------------------------------------------------------------------------------------------ batch-MLP helpers
__global__ void mlp_output_delta_kernel(const float* __restrict__ A, const float* __restrict__ D, const float* __restrict__ Y, int64_t n,
                                        int cost, float huberDelta, float* __restrict__ delta) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        delta[i] = -mlp_cost_deriv(cost, A[i], Y[i], huberDelta) * D[i];
}
int k_mlp_output_delta(b200_ctx* ctx, const float* A, const float* D, const float* Y, int64_t n, int cost, float huberDelta, float* delta) {
    if (n <= 0) return B200_OK;
    mlp_output_delta_kernel<<<grid_for(n, 256, 148 * 8), 256, 0, ctx->stream>>>(A, D, Y, n, cost, huberDelta, delta);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}
__global__ void mlp_scale_inputs_kernel(const float* __restrict__ X, int B, int F, const float* __restrict__ mn, const float* __restrict__ mx,
                                        float* __restrict__ out) {
    int64_t n = (int64_t)B * F;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int j = (int)(i % F);
        float range = mx[j] - mn[j];
        out[i] = range <= 0.f ? 0.f : (X[i] - mn[j]) / range;
    }
}
int k_mlp_scale_inputs(b200_ctx* ctx, const float* X, int B, int F, const float* mn, const float* mx, float* out) {
    int64_t n = (int64_t)B * F;
    if (n <= 0) return B200_OK;
    mlp_scale_inputs_kernel<<<grid_for(n, 256, 148 * 8), 256, 0, ctx->stream>>>(X, B, F, mn, mx, out);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}
__global__ void mlp_clip_scale_kernel(const float* __restrict__ sumsq, int nParts, float thr, float* __restrict__ out) {
    float s = 0.f;
    for (int i = 0; i < nParts; i++) s += sumsq[i];
    float norm = sqrtf(s);
    out[0] = norm > thr ? thr / norm : 1.0f;
    out[1] = norm;
}
int k_mlp_clip_scale(b200_ctx* ctx, const float* sumsq_dev, int nParts, float thr, float* scale_norm_dev) {
    mlp_clip_scale_kernel<<<1, 1, 0, ctx->stream>>>(sumsq_dev, nParts, thr, scale_norm_dev);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}
// b[j] -= slr * scale * sum_i delta[i,j]   (GPUB:302-313 BiasSumKernel + GPUB:350-358 BiasUpdateKernel)
__global__ void bias_update_kernel(float* __restrict__ b, const float* __restrict__ delta, int rows, int cols, float slr,
                                   const float* __restrict__ scale_dev) {
    int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= cols) return;
    float s = 0.f;
    for (int i = 0; i < rows; i++) s += delta[(size_t)i * cols + j];
    b[j] = b[j] - slr * (s * scale_dev[0]);
}
int k_bias_update(b200_ctx* ctx, float* b, const float* delta, int rows, int cols, float slr, const float* scale_dev) {
    if (cols <= 0) return B200_OK;
    bias_update_kernel<<<(cols + 127) / 128, 128, 0, ctx->stream>>>(b, delta, rows, cols, slr, scale_dev);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

}  // namespace b200
