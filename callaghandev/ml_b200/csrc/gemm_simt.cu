// FP32 SIMT GEMM: shared-memory staged, register tiled, any shape and any of the four operand layouts, with the fused
// epilogue.  This is the engine below the tensor-core threshold (a dimension under 128) and the 1e-5 parity path:
// every output element accumulates its K products in ascending k order in FP32 (fused multiply-add), with no split-K
// and no re-association across threads.
#include "common.h"
#include "gemm_epilogue.cuh"

namespace b200 {

template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_simt_kernel(int M, int N, int K, const float* __restrict__ A, int lda, int transA, const float* __restrict__ B, int ldb,
                 int transB, Epilogue ep) {
    constexpr int THREADS = (BM / TM) * (BN / TN);
    constexpr int RB = TM / 4, CB = TN / 4;          // 4-wide sub-blocks per thread in each direction
    constexpr int RSTRIDE = BM / RB, CSTRIDE = BN / CB;
    __shared__ __align__(16) float As[BK][BM + 4];
    __shared__ __align__(16) float Bs[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // ---- stage A tile (BM x BK) as As[k][m]
#pragma unroll
        for (int it = 0; it < (BM * BK) / THREADS; it++) {
            int idx = tid + it * THREADS;
            int m, k;
            if (transA) { k = idx / BM; m = idx % BM; } else { m = idx / BK; k = idx % BK; }
            int gm = m0 + m, gk = k0 + k;
            float v = 0.f;
            if (gm < M && gk < K) v = transA ? A[(size_t)gk * lda + gm] : A[(size_t)gm * lda + gk];
            As[k][m] = v;
        }
        // ---- stage B tile (BK x BN) as Bs[k][n]
#pragma unroll
        for (int it = 0; it < (BN * BK) / THREADS; it++) {
            int idx = tid + it * THREADS;
            int n, k;
            if (transB) { n = idx / BK; k = idx % BK; } else { k = idx / BN; n = idx % BN; }
            int gn = n0 + n, gk = k0 + k;
            float v = 0.f;
            if (gn < N && gk < K) v = transB ? B[(size_t)gn * ldb + gk] : B[(size_t)gk * ldb + gn];
            Bs[k][n] = v;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; k++) {
            float a[TM], b[TN];
#pragma unroll
            for (int rb = 0; rb < RB; rb++) {
                float4 t = *reinterpret_cast<const float4*>(&As[k][rb * RSTRIDE + ty * 4]);
                a[rb * 4 + 0] = t.x; a[rb * 4 + 1] = t.y; a[rb * 4 + 2] = t.z; a[rb * 4 + 3] = t.w;
            }
#pragma unroll
            for (int cb = 0; cb < CB; cb++) {
                float4 t = *reinterpret_cast<const float4*>(&Bs[k][cb * CSTRIDE + tx * 4]);
                b[cb * 4 + 0] = t.x; b[cb * 4 + 1] = t.y; b[cb * 4 + 2] = t.z; b[cb * 4 + 3] = t.w;
            }
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < TN; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }

    float alpha = ep.alpha;
    if (ep.alpha_dev) alpha *= ep.alpha_dev[0];
#pragma unroll
    for (int i = 0; i < TM; i++) {
        int m = m0 + (i / 4) * RSTRIDE + ty * 4 + (i % 4);
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; j++) {
            int n = n0 + (j / 4) * CSTRIDE + tx * 4 + (j % 4);
            if (n < N) epilogue_store(ep, m, n, acc[i][j], alpha);
        }
    }
}

static Epilogue make_epilogue(const Gemm& g) {
    Epilogue e;
    e.C = g.C; e.ldc = g.ldc; e.alpha = g.alpha; e.alpha_dev = g.alpha_dev; e.accumulate = g.accumulate; e.bias = g.bias;
    e.zout = g.zout; e.ldz = g.ldz; e.act = g.act; e.act_conv = g.act_conv; e.dout = g.dout; e.lddo = g.lddo;
    e.mulz = g.mulz; e.ldmulz = g.ldmulz; e.mulz_act = g.mulz_act; e.mulmat = g.mulmat; e.ldmul = g.ldmul;
    e.act_sign_zero = g.act_sign_zero; e.mulz_is_act = g.mulz_is_act;
    e.addmat = g.addmat; e.ldadd = g.ldadd; e.sgd_lr = g.sgd_lr; e.sgd_lambda = g.sgd_lambda; e.round_tf32 = g.round_tf32;
    e.rope_table = nullptr; e.rope_pos = nullptr; e.rope_cols = 0; e.rope_hd = 0;  // the rotation is a separate kernel behind this engine
    return e;
}

int gemm_simt(b200_ctx* ctx, const Gemm& g) {
    if (g.M <= 0 || g.N <= 0) return B200_OK;
    ctx->engine_launches[B200_ENGINE_GEMM_SIMT]++;
    Epilogue e = make_epilogue(g);
    // K == 0 still runs: the accumulator is zero and the epilogue (bias, assign) must happen.
    if (g.M >= 256 && g.N >= 128) {
        dim3 grid((g.N + 127) / 128, (g.M + 127) / 128);
        gemm_simt_kernel<128, 128, 16, 8, 8><<<grid, 256, 0, ctx->stream>>>(g.M, g.N, g.K, g.A, g.lda, g.transA, g.B, g.ldb, g.transB, e);
    } else {
        dim3 grid((g.N + 63) / 64, (g.M + 63) / 64);
        gemm_simt_kernel<64, 64, 16, 4, 4><<<grid, 256, 0, ctx->stream>>>(g.M, g.N, g.K, g.A, g.lda, g.transA, g.B, g.ldb, g.transB, e);
    }
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

// ------------------------------------------------------------------------------------------------ few-row products
// C[m,n] = A[m,:] . B[n,:] for M <= 4 rows (incremental decoding: one token at a time).  The product is bound by
// reading B once, which the tiled kernels above would do at 1/64 efficiency for a single row; what bounds a single
// launch, though, is latency: a weight row is a chain of dependent loop iterations for its warp, and a layer has only
// 1024..4096 rows.  So `wpc` warps share one output column (each a contiguous slice of K, summed in slice order through
// shared memory: deterministic), every lane keeps four independent 128-bit loads in flight, and the grid is sized so
// that a few thousand warps are resident whatever N is.  Same fused epilogue.
template <int MR>
__global__ void __launch_bounds__(256) gemv_rows_kernel(int M, int N, int K, const float* __restrict__ A, int lda, const float* __restrict__ B,
                                                        int ldb, int vec, int wpc, Epilogue ep) {
    __shared__ float part[8][MR];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * (8 / wpc) + warp / wpc, seg = warp % wpc;
    float acc[MR];
#pragma unroll
    for (int m = 0; m < MR; m++) acc[m] = 0.f;
    if (n < N) {
        const float* w = B + (size_t)n * ldb;
        int chunk = (K + wpc - 1) / wpc;
        chunk = (chunk + 127) & ~127;  // whole 128-element strides per warp slice
        const int k0 = seg * chunk, k1 = min(K, k0 + chunk);
        if (vec) {
            int k = k0 + lane * 4;
            for (; k + 384 < k1; k += 512) {
                float4 wv[4];
#pragma unroll
                for (int u = 0; u < 4; u++) wv[u] = *reinterpret_cast<const float4*>(w + k + 128 * u);
#pragma unroll
                for (int u = 0; u < 4; u++)
#pragma unroll
                    for (int m = 0; m < MR; m++)
                        if (m < M) {
                            const float4 xv = *reinterpret_cast<const float4*>(A + (size_t)m * lda + k + 128 * u);
                            acc[m] += (wv[u].x * xv.x + wv[u].y * xv.y) + (wv[u].z * xv.z + wv[u].w * xv.w);
                        }
            }
            for (; k < k1; k += 128) {
                const float4 wv = *reinterpret_cast<const float4*>(w + k);
#pragma unroll
                for (int m = 0; m < MR; m++)
                    if (m < M) {
                        const float4 xv = *reinterpret_cast<const float4*>(A + (size_t)m * lda + k);
                        acc[m] += (wv.x * xv.x + wv.y * xv.y) + (wv.z * xv.z + wv.w * xv.w);
                    }
            }
        } else {
            for (int k = k0 + lane; k < k1; k += 32) {
                const float wv = w[k];
#pragma unroll
                for (int m = 0; m < MR; m++)
                    if (m < M) acc[m] += wv * A[(size_t)m * lda + k];
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MR; m++) {
        const float v = warp_sum(acc[m]);
        if (lane == 0) part[warp][m] = v;
    }
    __syncthreads();
    if (n < N && seg == 0 && lane == 0) {
        float alpha = ep.alpha;
        if (ep.alpha_dev) alpha *= ep.alpha_dev[0];
        for (int m = 0; m < MR && m < M; m++) {
            float v = part[warp][m];
            for (int s2 = 1; s2 < wpc; s2++) v += part[warp + s2][m];
            epilogue_store(ep, m, n, v, alpha);
        }
    }
}

static bool gemv_eligible(const Gemm& g) { return g.M >= 1 && g.M <= 4 && !g.transA && g.transB && g.N >= 1 && g.K >= 1; }

static int gemv_rows(b200_ctx* ctx, const Gemm& g) {
    ctx->engine_launches[B200_ENGINE_GEMM_SIMT]++;
    Epilogue e = make_epilogue(g);
    const int vec = (g.K % 4 == 0) && (g.lda % 4 == 0) && (g.ldb % 4 == 0) && (((uintptr_t)g.A | (uintptr_t)g.B) & 15) == 0;
    int wpc = 1;  // warps per output column: aim at ~8192 warps in the grid, never less than 256 elements of K per warp
    while (wpc < 8 && (int64_t)g.N * wpc < 8192 && g.K / (2 * wpc) >= 256) wpc *= 2;
    const int cols_per_block = 8 / wpc;
    const int blocks = (g.N + cols_per_block - 1) / cols_per_block;
    gemv_rows_kernel<4><<<blocks, 256, 0, ctx->stream>>>(g.M, g.N, g.K, g.A, g.lda, g.B, g.ldb, vec, wpc, e);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

static int gemm_dispatch(b200_ctx* ctx, const Gemm& g0, int* engine) {
    Gemm g = g0;
    const bool rope_after = g.rope_table && !(ctx->gemm_mode != B200_GEMM_FP32_SIMT && gemm_tcgen05_fuses_rope(ctx, g));
    if (rope_after) {  // not fusable here: plain GEMM, then the rotation as its own kernel (TF32 rounding moves there too)
        g.rope_table = nullptr;
        g.round_tf32 = 0;
        B200_TRY(gemm_dispatch(ctx, g, engine));
        const int heads = g0.rope_cols / g0.rope_head_dim;
        return k_rope(ctx, g0.C, 0, 1, g0.M, g0.ldc, 0, heads, g0.rope_head_dim, g0.rope_table, g0.rope_pos, 0, g0.round_tf32);
    }
    if (ctx->gemm_mode != B200_GEMM_FP32_SIMT && gemm_tcgen05_eligible(ctx, g)) {
        *engine = 1;
        return gemm_tcgen05(ctx, g);
    }
    if (gemv_eligible(g)) {
        *engine = 0;
        return gemv_rows(ctx, g);
    }
    if (ctx->gemm_mode == B200_GEMM_TF32_TCGEN05 && g.M >= 128 && g.N >= 128 && g.K >= 128)
        return fail(ctx, B200_ERR_UNSUPPORTED, "TF32 tcgen05 GEMM requested but shape/alignment/device does not qualify (M=%d N=%d K=%d)", g.M, g.N, g.K);
    *engine = 0;
    return gemm_simt(ctx, g);
}

int gemm(b200_ctx* ctx, const Gemm& g) {
    int engine = 0;
    if (!ctx->profile) return gemm_dispatch(ctx, g, &engine);
    while (ctx->prof_events.size() < ctx->prof_used + 2) {
        cudaEvent_t e;
        B200_CUDA(ctx, cudaEventCreate(&e));
        ctx->prof_events.push_back(e);
    }
    cudaEvent_t e0 = ctx->prof_events[ctx->prof_used], e1 = ctx->prof_events[ctx->prof_used + 1];
    B200_CUDA(ctx, cudaEventRecord(e0, ctx->stream));
    B200_TRY(gemm_dispatch(ctx, g, &engine));
    B200_CUDA(ctx, cudaEventRecord(e1, ctx->stream));
    ctx->prof_used += 2;
    ctx->prof_flops.push_back(2.0 * g.M * g.N * g.K);
    ctx->prof_engine.push_back(engine);
    ctx->prof_shape.push_back(b200_ctx::ProfShape{g.M, g.N, g.K, g.transA, g.transB});
    return B200_OK;
}

int linear_fwd(b200_ctx* ctx, const float* X, int rows, int inDim, const float* W, const float* bias, int outDim, float* Y, int ldy) {
    Gemm g;
    g.M = rows; g.N = outDim; g.K = inDim;
    g.A = X; g.lda = inDim; g.transA = 0;
    g.B = W; g.ldb = inDim; g.transB = 1;
    g.C = Y; g.ldc = ldy; g.bias = bias;
    return gemm(ctx, g);
}
int wgrad(b200_ctx* ctx, const float* dY, int lddy, const float* X, int ldx, int rows, int outDim, int inDim, float* Wg, float* bg) {
    Gemm g;
    g.M = outDim; g.N = inDim; g.K = rows;
    g.A = dY; g.lda = lddy; g.transA = 1;
    g.B = X; g.ldb = ldx; g.transB = 0;
    g.C = Wg; g.ldc = inDim; g.accumulate = 1;
    B200_TRY(gemm(ctx, g));
    return bg ? k_colsum(ctx, dY, rows, outDim, lddy, bg, 1) : B200_OK;
}
int dgrad(b200_ctx* ctx, const float* dY, int lddy, const float* W, int rows, int outDim, int inDim, float* dX, int accumulate) {
    Gemm g;
    g.M = rows; g.N = inDim; g.K = outDim;
    g.A = dY; g.lda = lddy; g.transA = 0;
    g.B = W; g.ldb = inDim; g.transB = 0;
    g.C = dX; g.ldc = inDim; g.accumulate = accumulate;
    return gemm(ctx, g);
}

}  // namespace b200
