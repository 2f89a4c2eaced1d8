/*
 * oracle.c -- CPU restatement of the CallaghanDev.ML training hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA library is
 * compared against; nothing in the shipped package calls it.  It restates, in
 * plain C, the arithmetic of the reference's single-thread CPU manager
 * (CallaghanDev.ML/AccelerationManagers/AccelerationCPU.cs, "CPU" below), the
 * trainer orchestration (CallaghanDev.ML/Transformers/MultiTypeTransformer/
 * TransformerTrainer.cs, "TT"), the feed-forward network batch paths
 * (CallaghanDev.ML/Neural Network/NeuralNetwork.cs, "NN") and the batched MLP
 * kernels (CallaghanDev.ML/AccelerationManagers/BatchedAccelerationGPU.cs,
 * "GPUB").  Each function cites the lines it follows.
 *
 * Parity status: the reference is C#/.NET and cannot be built where this was
 * written, so no output of the reference itself is available.  The op-level
 * functions are pinned by the known-answer tests the reference's own test
 * suite carries (matmul-transpose values, RoPE known rotations, LayerNorm
 * statistics, masked-row zeros, causal-flag == causal-mask, the independent
 * BackpropQKV restatement).  The trainer-level step (lm_*) and the MLP batch
 * step (mlp_*) have no stored results in the reference's active tests:
 * PARITY UNPINNED there; they are validated op by op and by double-precision
 * finite differences (build with -DORACLE_F64).
 *
 * Third-party arithmetic not present in the reference tree: .NET MathF
 * (Exp/Log/Sqrt/Pow/Cos/Sin/Tanh) is restated with C libm; System.Numerics
 * Vector<float> is restated as 8 independent lanes (AVX2 width).
 *
 * real = float (default) or double (-DORACLE_F64, finite-difference checks).
 * Threading: ref_set_threads(n>1) enables OpenMP loops over the axes the
 * reference's multi-thread manager uses (rows for dX, outputs for dW,
 * segment x head for attention); per-element summation order is unchanged, so
 * results are bit-identical to the single-thread order.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#ifdef ORACLE_F64
typedef double real;
#define R_EXP exp
#define R_LOG log
#define R_SQRT sqrt
#define R_POW pow
#define R_COS cos
#define R_SIN sin
#define R_TANH tanh
#define R_FABS fabs
#else
typedef float real;
#define R_EXP expf
#define R_LOG logf
#define R_SQRT sqrtf
#define R_POW powf
#define R_COS cosf
#define R_SIN sinf
#define R_TANH tanhf
#define R_FABS fabsf
#endif

#define API __attribute__((visibility("default")))

static int g_threads = 1;
API void ref_set_threads(int n) { g_threads = n < 1 ? 1 : n; }
API int ref_get_threads(void) { return g_threads; }
API int ref_real_size(void) { return (int)sizeof(real); }
API int ref_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
#define PAR _Pragma("omp parallel for schedule(static) if(g_threads > 1) num_threads(g_threads)")
#define PAR_DYN _Pragma("omp parallel for schedule(dynamic,1) if(g_threads > 1) num_threads(g_threads)")

/* CPU:65-104 Dot: 8 vector lanes when length >= 16, then 4-unrolled, then tail. */
static real dot(const real* a, const real* b, int n) {
    real sum = 0;
    int i = 0;
    if (n >= 16) {
        int vend = n - (n % 8);
        real acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (; i < vend; i += 8)
            for (int l = 0; l < 8; l++) acc[l] += a[i + l] * b[i + l];
        for (int l = 0; l < 8; l++) sum += acc[l];
    }
    int end4 = i + ((n - i) & ~3);
    for (; i < end4; i += 4) {
        sum += a[i] * b[i];
        sum += a[i + 1] * b[i + 1];
        sum += a[i + 2] * b[i + 2];
        sum += a[i + 3] * b[i + 3];
    }
    for (; i < n; i++) sum += a[i] * b[i];
    return sum;
}

/* ---------------------------------------------------------------- tensor primitives */

/* CPU:159-210 MatrixMultiply: C[i,j] = Dot(A row i, B column j). */
API void ref_MatrixMultiply(const real* A, int rowsA, int colsA, const real* B, int colsB, real* C) {
    if (rowsA == 0 || colsB == 0) return;
    if (colsA == 0) { memset(C, 0, sizeof(real) * (size_t)rowsA * colsB); return; }
    real* bT = (real*)malloc(sizeof(real) * (size_t)colsA * colsB);
    for (int k = 0; k < colsA; k++)
        for (int j = 0; j < colsB; j++) bT[(size_t)j * colsA + k] = B[(size_t)k * colsB + j];
    PAR
    for (int i = 0; i < rowsA; i++)
        for (int j = 0; j < colsB; j++)
            C[(size_t)i * colsB + j] = dot(A + (size_t)i * colsA, bT + (size_t)j * colsA, colsA);
    free(bT);
}

/* MatrixMultiplyTranspose: C = A * B^T (known-answer test TTT:664-674). */
API void ref_MatrixMultiplyTranspose(const real* A, int rowsA, int colsA, const real* B, int rowsB, real* C) {
    PAR
    for (int i = 0; i < rowsA; i++)
        for (int j = 0; j < rowsB; j++)
            C[(size_t)i * rowsB + j] = dot(A + (size_t)i * colsA, B + (size_t)j * colsA, colsA);
}

/* CPU:352-404 BatchDotProductAddBias (offset-aware): y[i,j] = Dot(W row j, x row rowStart+i) + bias[j]. */
API void ref_BatchDotProductAddBias(const real* W, int outDim, int inDim, const real* X, int rowStart, int rowCount,
                                    const real* bias, real* Y) {
    PAR
    for (int i = 0; i < rowCount; i++)
        for (int j = 0; j < outDim; j++)
            Y[(size_t)i * outDim + j] = dot(W + (size_t)j * inDim, X + (size_t)(rowStart + i) * inDim, inDim) + bias[j];
}

/* CPU:2694-2715 ProjectOutputBatch: p[i,j] = bias[j] + Dot(proj row j, hidden row i). */
API void ref_ProjectOutputBatch(const real* hidden, int embDim, const real* proj, const real* bias, int seqLen,
                                int outputDim, real* pred) {
    PAR
    for (int i = 0; i < seqLen; i++)
        for (int j = 0; j < outputDim; j++)
            pred[(size_t)i * outputDim + j] = bias[j] + dot(proj + (size_t)j * embDim, hidden + (size_t)i * embDim, embDim);
}

/* CPU:522-546 MatrixAddInPlace / CPU:548-566 VectorAccumulate. */
API void ref_AddInPlace(real* target, const real* addend, int64_t n) {
    for (int64_t i = 0; i < n; i++) target[i] += addend[i];
}

/* ---------------------------------------------------------------- layer norm */

/* CPU:1440-1514 ResidualLayerNormForward. */
API void ref_ResidualLayerNormForward(const real* input, const real* subLayer, const real* gamma, const real* beta,
                                      int rows, int features, real eps, real* output, real* means, real* variances,
                                      real* normalized, real* residual) {
    PAR
    for (int i = 0; i < rows; i++) {
        size_t row = (size_t)i * features;
        real mean = 0;
        for (int j = 0; j < features; j++) {
            real v = input[row + j] + (subLayer ? subLayer[row + j] : 0);
            residual[row + j] = v;
            mean += v;
        }
        mean /= features;
        means[i] = mean;
        real var = 0;
        for (int j = 0; j < features; j++) {
            real d = residual[row + j] - mean;
            var += d * d;
        }
        var /= features;
        variances[i] = var;
        real invStd = (real)1 / R_SQRT(var + eps);
        for (int j = 0; j < features; j++) {
            real n = (residual[row + j] - mean) * invStd;
            normalized[row + j] = n;
            output[row + j] = gamma[j] * n + beta[j];
        }
    }
}

/* CPU:1516-1564 LayerNormBackward.  dGamma/dBeta are fresh (zeroed here). */
API void ref_LayerNormBackward(const real* dOut, const real* normalized, const real* gamma, const real* input,
                               const real* mean, const real* variance, int rows, int features, real eps,
                               real* dInput, real* dGamma, real* dBeta) {
    for (int j = 0; j < features; j++) { dGamma[j] = 0; dBeta[j] = 0; }
    for (int i = 0; i < rows; i++) {
        size_t row = (size_t)i * features;
        for (int j = 0; j < features; j++) {
            dGamma[j] += dOut[row + j] * normalized[row + j];
            dBeta[j] += dOut[row + j];
        }
    }
    PAR
    for (int i = 0; i < rows; i++) {
        size_t row = (size_t)i * features;
        real invStd = (real)1 / R_SQRT(variance[i] + eps);
        real invStd3 = invStd * invStd * invStd;
        real dVar = 0, dMean = 0, m = mean[i];
        for (int j = 0; j < features; j++) {
            real dNorm = dOut[row + j] * gamma[j];
            real xm = input[row + j] - m;
            dVar += dNorm * xm * (real)(-0.5) * invStd3;
            dMean += dNorm * (-invStd);
        }
        real invN = (real)1 / features;
        real dVarScale = dVar * (real)2 * invN;
        real dMeanScale = dMean * invN;
        for (int j = 0; j < features; j++) {
            real dNorm = dOut[row + j] * gamma[j];
            real xm = input[row + j] - m;
            dInput[row + j] = dNorm * invStd + dVarScale * xm + dMeanScale;
        }
    }
}

/* ---------------------------------------------------------------- attention */

/* CPU:1797-1956 ScaledDotProductAttention.  mask: NULL or [queryLen,keyLen] bytes (non-zero = visible). */
API void ref_ScaledDotProductAttention(const real* q, const real* k, const real* v, int queryLen, int keyLen,
                                       int embDim, int numHeads, const uint8_t* mask, int causal, real* out) {
    int headDim = embDim / numHeads;
    real scale = (real)1 / R_SQRT((real)headDim);
    memset(out, 0, sizeof(real) * (size_t)queryLen * embDim);
    PAR
    for (int head = 0; head < numHeads; head++) {
        real* scores = (real*)malloc(sizeof(real) * (size_t)keyLen);
        int off = head * headDim;
        for (int qi = 0; qi < queryLen; qi++) {
            int usable = causal ? (qi + 1 < keyLen ? qi + 1 : keyLen) : keyLen;
            const real* qr = q + (size_t)qi * embDim + off;
            real* orow = out + (size_t)qi * embDim + off;
            real maxS = -INFINITY;
            for (int kj = 0; kj < usable; kj++) {
                if (mask && !mask[(size_t)qi * keyLen + kj]) { scores[kj] = -INFINITY; continue; }
                real s = dot(qr, k + (size_t)kj * embDim + off, headDim) * scale;
                scores[kj] = s;
                if (s > maxS) maxS = s;
            }
            if (isinf(maxS) && maxS < 0) continue;
            real sumExp = 0;
            for (int kj = 0; kj < usable; kj++) {
                if (isinf(scores[kj]) && scores[kj] < 0) { scores[kj] = 0; continue; }
                real e = R_EXP(scores[kj] - maxS);
                scores[kj] = e;
                sumExp += e;
            }
            if (sumExp <= 0 || isnan(sumExp) || isinf(sumExp)) continue;
            real inv = (real)1 / sumExp;
            for (int kj = 0; kj < usable; kj++) {
                real w = scores[kj] * inv;
                if (w == 0) continue;
                const real* vr = v + (size_t)kj * embDim + off;
                for (int d = 0; d < headDim; d++) orow[d] += w * vr[d];
            }
        }
        free(scores);
    }
}

/* One (head, query-row) step shared by CPU:1037-1284 MultiHeadAttentionBackwardCore and
 * TT:989-1121 SegmentedMultiHeadAttentionBackward.  Rows are addressed relative to the
 * given base pointers, heads are column slices. */
static void mha_bwd_row(const real* Q, const real* K, const real* V, const real* dO, int embDim, int off, int headDim,
                        int qi, int seqLenK, const uint8_t* maskRow, int visible, real scale, real* dQ, real* dK,
                        real* dV, real* weights, real* dAttn) {
    const real* qr = Q + (size_t)qi * embDim + off;
    const real* dor = dO + (size_t)qi * embDim + off;
    real maxS = -INFINITY;
    int active = 0;
    for (int j = 0; j < visible; j++) {
        if (maskRow && !maskRow[j]) { weights[j] = -INFINITY; continue; }
        real s = dot(qr, K + (size_t)j * embDim + off, headDim) * scale;
        weights[j] = s;
        active++;
        if (s > maxS) maxS = s;
    }
    (void)seqLenK;
    if (active == 0 || (isinf(maxS) && maxS < 0)) return;
    real sumExp = 0;
    for (int j = 0; j < visible; j++) {
        if (maskRow && !maskRow[j]) { weights[j] = 0; continue; }
        real w = R_EXP(weights[j] - maxS);
        weights[j] = w;
        sumExp += w;
    }
    if (sumExp <= 0) return;
    real inv = (real)1 / sumExp;
    real rowDot = 0;
    for (int j = 0; j < visible; j++) {
        if (maskRow && !maskRow[j]) continue;
        weights[j] *= inv;
        real w = weights[j];
        real dA = 0;
        const real* vr = V + (size_t)j * embDim + off;
        real* dvr = dV + (size_t)j * embDim + off;
        for (int d = 0; d < headDim; d++) {
            dvr[d] += w * dor[d];
            dA += dor[d] * vr[d];
        }
        dAttn[j] = dA;
        rowDot += w * dA;
    }
    real* dqr = dQ + (size_t)qi * embDim + off;
    for (int j = 0; j < visible; j++) {
        if (maskRow && !maskRow[j]) continue;
        real dDot = weights[j] * (dAttn[j] - rowDot) * scale;
        if (dDot == 0) continue;
        const real* kr = K + (size_t)j * embDim + off;
        real* dkr = dK + (size_t)j * embDim + off;
        for (int d = 0; d < headDim; d++) {
            dqr[d] += dDot * kr[d];
            dkr[d] += dDot * qr[d];
        }
    }
}

/* CPU:1037-1284 MultiHeadAttentionBackward (both overloads): mask NULL + useDecoderMask, or explicit mask. */
API void ref_MultiHeadAttentionBackward(const real* Q, const real* K, const real* V, const real* dConcat, int seqLenQ,
                                        int seqLenK, int embDim, int numHeads, real scale, const uint8_t* mask,
                                        int useDecoderMask, real* dQ, real* dK, real* dV) {
    int headDim = embDim / numHeads;
    memset(dQ, 0, sizeof(real) * (size_t)seqLenQ * embDim);
    memset(dK, 0, sizeof(real) * (size_t)seqLenK * embDim);
    memset(dV, 0, sizeof(real) * (size_t)seqLenK * embDim);
    PAR
    for (int head = 0; head < numHeads; head++) {
        real* weights = (real*)malloc(sizeof(real) * (size_t)(seqLenK + 1));
        real* dAttn = (real*)malloc(sizeof(real) * (size_t)(seqLenK + 1));
        for (int i = 0; i < seqLenQ; i++) {
            int visible = mask ? seqLenK : (useDecoderMask ? (i + 1 < seqLenK ? i + 1 : seqLenK) : seqLenK);
            mha_bwd_row(Q, K, V, dConcat, embDim, head * headDim, headDim, i, seqLenK,
                        mask ? mask + (size_t)i * seqLenK : NULL, visible, scale, dQ, dK, dV, weights, dAttn);
        }
        free(weights);
        free(dAttn);
    }
}

/* TT:723-809 segmented attention forward (Q,K already rotated): segment s owns rows [s*L, (s+1)*L). */
API void ref_SegmentedAttentionForward(const real* Q, const real* K, const real* V, int segLen, int segCount,
                                       int embDim, int numHeads, int causal, real* out) {
    int headDim = embDim / numHeads;
    real scale = (real)1 / R_SQRT((real)headDim);
    memset(out, 0, sizeof(real) * (size_t)segLen * segCount * embDim);
    PAR_DYN
    for (int work = 0; work < segCount * numHeads; work++) {
        int seg = work / numHeads, head = work - seg * numHeads;
        size_t rowBase = (size_t)seg * segLen;
        int off = head * headDim;
        real* scores = (real*)malloc(sizeof(real) * (size_t)segLen);
        for (int qi = 0; qi < segLen; qi++) {
            const real* qr = Q + (rowBase + qi) * embDim + off;
            int visible = causal ? qi + 1 : segLen;
            real maxS = -INFINITY;
            for (int kj = 0; kj < visible; kj++) {
                const real* kr = K + (rowBase + kj) * embDim + off;
                real d = 0;
                for (int c = 0; c < headDim; c++) d += qr[c] * kr[c];
                real s = d * scale;
                scores[kj] = s;
                if (s > maxS) maxS = s;
            }
            real sumExp = 0;
            for (int kj = 0; kj < visible; kj++) {
                real e = R_EXP(scores[kj] - maxS);
                scores[kj] = e;
                sumExp += e;
            }
            real inv = sumExp > 0 ? (real)1 / sumExp : 0;
            real* orow = out + (rowBase + qi) * embDim + off;
            for (int kj = 0; kj < visible; kj++) {
                real w = scores[kj] * inv;
                if (w == 0) continue;
                const real* vr = V + (rowBase + kj) * embDim + off;
                for (int c = 0; c < headDim; c++) orow[c] += w * vr[c];
            }
        }
        free(scores);
    }
}

/* TT:989-1121 SegmentedMultiHeadAttentionBackward. */
API void ref_SegmentedAttentionBackward(const real* Q, const real* K, const real* V, const real* dConcat, int segLen,
                                        int segCount, int embDim, int numHeads, real scale, int causal, real* dQ,
                                        real* dK, real* dV) {
    int headDim = embDim / numHeads;
    size_t total = (size_t)segLen * segCount * embDim;
    memset(dQ, 0, sizeof(real) * total);
    memset(dK, 0, sizeof(real) * total);
    memset(dV, 0, sizeof(real) * total);
    PAR_DYN
    for (int work = 0; work < segCount * numHeads; work++) {
        int seg = work / numHeads, head = work - seg * numHeads;
        size_t base = (size_t)seg * segLen * embDim;
        real* weights = (real*)malloc(sizeof(real) * (size_t)(segLen + 1));
        real* dAttn = (real*)malloc(sizeof(real) * (size_t)(segLen + 1));
        for (int qi = 0; qi < segLen; qi++) {
            int visible = causal ? qi + 1 : segLen;
            mha_bwd_row(Q + base, K + base, V + base, dConcat + base, embDim, head * headDim, headDim, qi, segLen, NULL,
                        visible, scale, dQ + base, dK + base, dV + base, weights, dAttn);
        }
        free(weights);
        free(dAttn);
    }
}

/* CPU:4929-4982 rotary core for one head; position = row index (or row % segLen, TT:811-848, when segLen > 0). */
static void rope_head(real* m, int rows, int embDim, int startCol, int headDim, real baseTheta, int inverse, int segLen) {
    int pairs = headDim / 2;
    if (rows == 0 || pairs == 0) return;
    real* denom = (real*)malloc(sizeof(real) * (size_t)pairs);
    for (int p = 0; p < pairs; p++) denom[p] = R_POW(baseTheta, ((real)2 * p) / headDim);
    for (int r = 0; r < rows; r++) {
        int pos = segLen > 0 ? r % segLen : r;
        real* row = m + (size_t)r * embDim + startCol;
        for (int p = 0; p < pairs; p++) {
            real theta = pos / denom[p];
            real c = R_COS(theta), s = R_SIN(theta);
            if (inverse) s = -s;
            real x0 = row[2 * p], x1 = row[2 * p + 1];
            row[2 * p] = x0 * c - x1 * s;
            row[2 * p + 1] = x0 * s + x1 * c;
        }
    }
    free(denom);
}

/* CPU:4855-4893 ApplyRotaryPositionEmbeddingInPlace; segLen > 0 gives TT:811-848 ApplySegmentedRotaryInPlace. */
API void ref_ApplyRotaryPositionEmbeddingInPlace(real* m, int rows, int embDim, int numHeads, real baseTheta,
                                                 int inverse, int segLen) {
    int headDim = embDim / numHeads;
    for (int h = 0; h < numHeads; h++) rope_head(m, rows, embDim, h * headDim, headDim, baseTheta, inverse, segLen);
}

/* CPU:4894-4928 ApplyRotaryPositionEmbeddingHeadInPlace. */
API void ref_ApplyRotaryPositionEmbeddingHeadInPlace(real* m, int rows, int embDim, int startCol, int headDim,
                                                     real baseTheta, int inverse) {
    rope_head(m, rows, embDim, startCol, headDim, baseTheta, inverse, 0);
}

/* ---------------------------------------------------------------- projections */

/* CPU:2005-2069 ProjectQKV. */
API void ref_ProjectQKV(const real* x, int rows, int inDim, const real* WQ, const real* bQ, const real* WK,
                        const real* bK, const real* WV, const real* bV, int outDim, real* Q, real* K, real* V) {
    PAR
    for (int i = 0; i < rows; i++)
        for (int o = 0; o < outDim; o++) {
            const real* xr = x + (size_t)i * inDim;
            Q[(size_t)i * outDim + o] = bQ[o] + dot(WQ + (size_t)o * inDim, xr, inDim);
            K[(size_t)i * outDim + o] = bK[o] + dot(WK + (size_t)o * inDim, xr, inDim);
            V[(size_t)i * outDim + o] = bV[o] + dot(WV + (size_t)o * inDim, xr, inDim);
        }
}

/* Generic "W grads += dY^T x, bias grads += colsum(dY)" with the reference's per-element order
 * (row index ascending), threaded over outputs as MT:921-953 does. */
static void accum_wgrad(const real* dY, int ldDy, const real* x, int ldX, int rows, int outDim, int inDim, real* Wg,
                        real* bg) {
    PAR
    for (int j = 0; j < outDim; j++) {
        real b = bg[j];
        for (int i = 0; i < rows; i++) b += dY[(size_t)i * ldDy + j];
        bg[j] = b;
        real* wr = Wg + (size_t)j * inDim;
        for (int i = 0; i < rows; i++) {
            real d = dY[(size_t)i * ldDy + j];
            const real* xr = x + (size_t)i * ldX;
            for (int k = 0; k < inDim; k++) wr[k] += d * xr[k];
        }
    }
}

/* CPU:2071-2182 BackpropQKV: grads +=, dInput fresh.  dx accumulates per (o,d) the sum dq*wq+dk*wk+dv*wv. */
API void ref_BackpropQKV(const real* x, int rows, int inDim, const real* dQ, const real* dK, const real* dV,
                         int outDim, const real* WQ, const real* WK, const real* WV, real* WQg, real* bQg, real* WKg,
                         real* bKg, real* WVg, real* bVg, real* dInput) {
    accum_wgrad(dQ, outDim, x, inDim, rows, outDim, inDim, WQg, bQg);
    accum_wgrad(dK, outDim, x, inDim, rows, outDim, inDim, WKg, bKg);
    accum_wgrad(dV, outDim, x, inDim, rows, outDim, inDim, WVg, bVg);
    PAR
    for (int i = 0; i < rows; i++) {
        real* dx = dInput + (size_t)i * inDim;
        for (int d = 0; d < inDim; d++) dx[d] = 0;
        for (int o = 0; o < outDim; o++) {
            real dq = dQ[(size_t)i * outDim + o], dk = dK[(size_t)i * outDim + o], dv = dV[(size_t)i * outDim + o];
            const real *wq = WQ + (size_t)o * inDim, *wk = WK + (size_t)o * inDim, *wv = WV + (size_t)o * inDim;
            for (int d = 0; d < inDim; d++) dx[d] += dq * wq[d] + dk * wk[d] + dv * wv[d];
        }
    }
}

/* CPU:4361-4417 ProjectKV: K = x WK^T + bK, V = x WV^T + bV (the bias starts each sum). */
API void ref_ProjectKV(const real* x, int rows, int inDim, const real* WK, const real* bK, const real* WV, const real* bV, int outDim,
                       real* K, real* V) {
    PAR
    for (int i = 0; i < rows; i++)
        for (int o = 0; o < outDim; o++) {
            const real* xr = x + (size_t)i * inDim;
            real sk = 0, sv = 0;
            for (int d = 0; d < inDim; d++) { sk += WK[(size_t)o * inDim + d] * xr[d]; sv += WV[(size_t)o * inDim + d] * xr[d]; }
            K[(size_t)i * outDim + o] = bK[o] + sk;
            V[(size_t)i * outDim + o] = bV[o] + sv;
        }
}

/* CPU:4419-4532 BackpropKV: weight and bias gradients accumulate, dInput is a fresh array. */
API void ref_BackpropKV(const real* x, int rows, int inDim, const real* dK, const real* dV, int outDim, const real* WK, const real* WV,
                        real* WKg, real* bKg, real* WVg, real* bVg, real* dInput) {
    accum_wgrad(dK, outDim, x, inDim, rows, outDim, inDim, WKg, bKg);
    accum_wgrad(dV, outDim, x, inDim, rows, outDim, inDim, WVg, bVg);
    PAR
    for (int i = 0; i < rows; i++) {
        real* dx = dInput + (size_t)i * inDim;
        for (int d = 0; d < inDim; d++) dx[d] = 0;
        for (int o = 0; o < outDim; o++) {
            real dk = dK[(size_t)i * outDim + o], dv = dV[(size_t)i * outDim + o];
            const real *wk = WK + (size_t)o * inDim, *wv = WV + (size_t)o * inDim;
            for (int d = 0; d < inDim; d++) dx[d] += dk * wk[d] + dv * wv[d];
        }
    }
}

/* CPU:2188-2229 BackpropLinearProjection: weightGrad, biasGrad and dInput all accumulate. */
API void ref_BackpropLinearProjection(const real* x, const real* dY, const real* W, int seqLen, int inDim, int outDim,
                                      real* Wg, real* bg, real* dInput) {
    accum_wgrad(dY, outDim, x, inDim, seqLen, outDim, inDim, Wg, bg);
    PAR
    for (int i = 0; i < seqLen; i++)
        for (int k = 0; k < inDim; k++) {
            real s = 0;
            for (int j = 0; j < outDim; j++) s += dY[(size_t)i * outDim + j] * W[(size_t)j * inDim + k];
            dInput[(size_t)i * inDim + k] += s;
        }
}

/* CPU:2231-2273 BackpropOutputProjection: grads +=, dX assigned. */
API void ref_BackpropOutputProjection(const real* dLogits, const real* x, const real* W, real* Wg, real* bg,
                                      int seqLen, int outputDim, int embDim, real* dX) {
    accum_wgrad(dLogits, outputDim, x, embDim, seqLen, outputDim, embDim, Wg, bg);
    PAR
    for (int i = 0; i < seqLen; i++)
        for (int e = 0; e < embDim; e++) {
            real s = 0;
            for (int v = 0; v < outputDim; v++) s += dLogits[(size_t)i * outputDim + v] * W[(size_t)v * embDim + e];
            dX[(size_t)i * embDim + e] = s;
        }
}

/* CPU:2280-2332 BackpropInputProjection (offset-aware). */
API void ref_BackpropInputProjection(const real* dX, const real* cont, int contCols, int inputRowStart, real* Wg,
                                     real* bg, int seqLen, int embDim, int inputFeatureDim) {
    accum_wgrad(dX, embDim, cont + (size_t)inputRowStart * contCols, contCols, seqLen, embDim, inputFeatureDim, Wg, bg);
}

/* CPU:3473-3515 EmbedTokenIds: returns -1 if an id is outside [0, vocab). */
API int ref_EmbedTokenIds(const int32_t* ids, int tokenStart, int tokenCount, const real* emb, int vocab, int embDim,
                          real* out) {
    for (int i = 0; i < tokenCount; i++) {
        int id = ids[tokenStart + i];
        if ((uint32_t)id >= (uint32_t)vocab) return -1;
        memcpy(out + (size_t)i * embDim, emb + (size_t)id * embDim, sizeof(real) * (size_t)embDim);
    }
    return 0;
}

/* CPU:2339-2370 AccumulateTokenEmbeddingGrad: serial scatter in row order. */
API void ref_AccumulateTokenEmbeddingGrad(real* eg, const real* dX, const int32_t* ids, int tokenStart, int seqLen,
                                          int embDim) {
    for (int i = 0; i < seqLen; i++) {
        real* g = eg + (size_t)ids[tokenStart + i] * embDim;
        const real* d = dX + (size_t)i * embDim;
        for (int j = 0; j < embDim; j++) g[j] += d[j];
    }
}

/* ---------------------------------------------------------------- losses */

/* CPU:2377-2440 CrossEntropyLossAndGradient.  dLogits is [rows,outputDim]; rows >= effectiveLen stay zero. */
API real ref_CrossEntropyLossAndGradient(const real* logits, int rows, int outputDim, const int32_t* targets,
                                         int targetStart, int effectiveLen, real* dLogits) {
    memset(dLogits, 0, sizeof(real) * (size_t)rows * outputDim);
    if (effectiveLen == 0) return 0;
    real loss = 0;
    real invLen = (real)1 / effectiveLen;
    for (int i = 0; i < effectiveLen; i++) {
        const real* l = logits + (size_t)i * outputDim;
        real* dl = dLogits + (size_t)i * outputDim;
        real mx = -INFINITY;
        for (int j = 0; j < outputDim; j++) mx = l[j] > mx ? l[j] : (mx == mx && l[j] == l[j] ? mx : NAN);
        real sum = 0;
        for (int j = 0; j < outputDim; j++) {
            real p = R_EXP(l[j] - mx);
            dl[j] = p;
            sum += p;
        }
        real inv = (real)1 / sum;
        int t = targets[targetStart + i];
        loss -= R_LOG(dl[t] * inv + (real)1e-10);
        for (int j = 0; j < outputDim; j++) {
            real g = (dl[j] * inv) * invLen;
            if (j == t) g -= invLen;
            dl[j] = g;
        }
    }
    return loss / effectiveLen;
}

/* CPU:2447-2491 MSELossAndGradient. */
API real ref_MSELossAndGradient(const real* pred, int rows, int outputDim, const real* targets, int targetStart,
                                int effectiveLen, real* dOut) {
    memset(dOut, 0, sizeof(real) * (size_t)rows * outputDim);
    if (effectiveLen == 0 || outputDim == 0) return 0;
    real loss = 0;
    real invLen = (real)1 / ((real)effectiveLen * outputDim);
    for (int i = 0; i < effectiveLen; i++)
        for (int j = 0; j < outputDim; j++) {
            real diff = pred[(size_t)i * outputDim + j] - targets[(size_t)(targetStart + i) * outputDim + j];
            loss += diff * diff;
            dOut[(size_t)i * outputDim + j] = (real)2 * diff * invLen;
        }
    return loss / ((real)effectiveLen * outputDim);
}

/* ---------------------------------------------------------------- step primitives */

/* CPU:2493-2513 MatrixSquaredNorm / VectorSquaredNorm. */
API real ref_SquaredNorm(const real* m, int64_t n) {
    real s = 0;
    for (int64_t i = 0; i < n; i++) s += m[i] * m[i];
    return s;
}
/* CPU:2515-2546 MatrixScaleInPlace / VectorScaleInPlace. */
API void ref_ScaleInPlace(real* m, int64_t n, real scale) {
    for (int64_t i = 0; i < n; i++) m[i] *= scale;
}
/* CPU:2548-2590 MatrixUpdate / VectorUpdate: w -= lr * g. */
API void ref_Update(real* w, const real* g, int64_t n, real lr) {
    for (int64_t i = 0; i < n; i++) w[i] -= lr * g[i];
}

/* ---------------------------------------------------------------- feed-forward network (transformer FFN path) */

enum { ACT_NONE = 0, ACT_SIGMOID = 1, ACT_TANH = 2, ACT_RELU = 3, ACT_LEAKYRELU = 4, ACT_SWISH = 5 };

/* NN:704-716 StableSigmoidLocal. */
static real stable_sigmoid(real x) {
    if (x >= 0) { real z = R_EXP(-x); return (real)1 / ((real)1 + z); }
    real z = R_EXP(x);
    return z / ((real)1 + z);
}
/* NN:670-702 ApplyActivationInPlace (forward-only path). */
static real ffn_act(real x, int t) {
    switch (t) {
        case ACT_SIGMOID: return stable_sigmoid(x);
        case ACT_TANH: return R_TANH(x);
        case ACT_RELU: return x > 0 ? x : 0;
        case ACT_LEAKYRELU: return x > 0 ? x : (real)0.01 * x;
        case ACT_SWISH: return x * stable_sigmoid(x);
        default: return x;
    }
}
/* NN:886-946 FillActivationAndDerivative (backward path; note ReLU'(0)=1 and LeakyReLU' = 0.1 for z<=0). */
static void ffn_act_der(real z, int t, real* a, real* d) {
    switch (t) {
        case ACT_SIGMOID: { real s = stable_sigmoid(z); *a = s; *d = s * ((real)1 - s); break; }
        case ACT_TANH: { real th = R_TANH(z); *a = th; *d = (real)1 - th * th; break; }
        case ACT_RELU: *a = z > 0 ? z : 0; *d = z >= 0 ? 1 : 0; break;
        case ACT_LEAKYRELU: *a = z > 0 ? z : (real)0.01 * z; *d = z <= 0 ? (real)0.1 : 1; break;
        case ACT_SWISH: { real s = stable_sigmoid(z); *a = z * s; *d = s + z * s * ((real)1 - s); break; }
        default: *a = z; *d = 1; break;
    }
}

/* NN:629-668 ForwardPassOnlyBatch for a network given as layer widths [nLayers], activations [nLayers]
 * (entry 0 unused) and per-layer weights[l] ([width l, width l-1]) / biases[l], l = 1..nLayers-1. */
API void ref_FFNForwardBatch(const real* input, int rows, int nLayers, const int32_t* widths, const int32_t* acts,
                             const real* const* weights, const real* const* biases, real* out) {
    const real* cur = input;
    real* buf = NULL;
    for (int l = 1; l < nLayers; l++) {
        real* next = (l == nLayers - 1) ? out : (real*)malloc(sizeof(real) * (size_t)rows * widths[l]);
        ref_BatchDotProductAddBias(weights[l], widths[l], widths[l - 1], cur, 0, rows, biases[l], next);
        size_t n = (size_t)rows * widths[l];
        for (size_t i = 0; i < n; i++) next[i] = ffn_act(next[i], acts[l]);
        if (buf) free(buf);
        buf = (l == nLayers - 1) ? NULL : next;
        cur = next;
    }
}

/* NN:773-884 ComputeInputGradientBatch (+ NN:948-987 AccumulateGradientsBatch): recompute forward, deltas,
 * accumulate weightGrads[l]/biasGrads[l] (l = 1..nLayers-1; may be NULL arrays), return dInput [rows, widths[0]]. */
API void ref_FFNInputGradientBatch(const real* input, const real* dOutput, int rows, int nLayers, const int32_t* widths,
                                   const int32_t* acts, const real* const* weights, const real* const* biases,
                                   real* const* weightGrads, real* const* biasGrads, real* dInput) {
    int L = nLayers - 1;
    real** act = (real**)calloc((size_t)nLayers, sizeof(real*));
    real** der = (real**)calloc((size_t)nLayers, sizeof(real*));
    act[0] = (real*)input;
    for (int l = 1; l <= L; l++) {
        size_t n = (size_t)rows * widths[l];
        real* z = (real*)malloc(sizeof(real) * n);
        ref_BatchDotProductAddBias(weights[l], widths[l], widths[l - 1], act[l - 1], 0, rows, biases[l], z);
        act[l] = (real*)malloc(sizeof(real) * n);
        der[l] = (real*)malloc(sizeof(real) * n);
        for (size_t i = 0; i < n; i++) ffn_act_der(z[i], acts[l], &act[l][i], &der[l][i]);
        free(z);
    }
    size_t nOut = (size_t)rows * widths[L];
    real* cur = (real*)malloc(sizeof(real) * nOut);
    for (size_t i = 0; i < nOut; i++) cur[i] = dOutput[i] * der[L][i];
    for (int l = L; l >= 1; l--) {
        if (weightGrads && biasGrads) {
            /* deltaT x prevActivations via MatrixMultiply (Dot order over rows), then wGrad += ; bias sums rows. */
            int ls = widths[l], ps = widths[l - 1];
            real* dT = (real*)malloc(sizeof(real) * (size_t)ls * rows);
            for (int r = 0; r < rows; r++)
                for (int c = 0; c < ls; c++) dT[(size_t)c * rows + r] = cur[(size_t)r * ls + c];
            real* wd = (real*)malloc(sizeof(real) * (size_t)ls * ps);
            ref_MatrixMultiply(dT, ls, rows, act[l - 1], ps, wd);
            for (int i = 0; i < ls; i++) {
                real b = biasGrads[l][i];
                for (int r = 0; r < rows; r++) b += cur[(size_t)r * ls + i];
                biasGrads[l][i] = b;
                for (int j = 0; j < ps; j++) weightGrads[l][(size_t)i * ps + j] += wd[(size_t)i * ps + j];
            }
            free(dT);
            free(wd);
        }
        int below = widths[l - 1];
        real* nxt = (l == 1) ? dInput : (real*)malloc(sizeof(real) * (size_t)rows * below);
        ref_MatrixMultiply(cur, rows, widths[l], weights[l], below, nxt);
        if (l > 1) {
            size_t n = (size_t)rows * below;
            for (size_t i = 0; i < n; i++) nxt[i] *= der[l - 1][i];
        }
        free(cur);
        cur = (l == 1) ? NULL : nxt;
    }
    for (int l = 1; l <= L; l++) { free(act[l]); free(der[l]); }
    free(act);
    free(der);
}

/* ---------------------------------------------------------------- language-model train step (TT) */

/* Flat parameter layout shared with the CUDA library: see lm_layout() below.  Tensor order follows the
 * reference's weights.bin (LM:737-765) with each block's FFN tensors appended to the block. */
typedef struct {
    int32_t vocab_size;        /* discrete models */
    int32_t input_feature_dim; /* continuous models */
    int32_t output_dim;        /* EffectiveOutputDim: vocab for text, OutputDim otherwise */
    int32_t embedding_dim, num_heads, num_layers, ffn_dim;
    int32_t ffn_activation;    /* ACT_* */
    int32_t discrete;          /* 1: token ids in, cross-entropy; 0: continuous features in */
    int32_t loss_kind;         /* 0 cross-entropy, 1 MSE (time-series regression) */
    int32_t causal;            /* UseDecoderOnly */
    int32_t align_floats;      /* every tensor offset is rounded up to this many elements (>=1) */
} ref_lm_config;

typedef struct {
    int64_t emb, inW, inB;
    int64_t total;
} lm_head_off;

static int64_t al(int64_t x, int a) { return a <= 1 ? x : (x + a - 1) / a * a; }

/* Per-layer tensor offsets relative to the start of the arena. */
typedef struct {
    int64_t WQ, WK, WV, WO, bQ, bK, bV, bO, g1, b1n, g2, b2n, W1, fb1, W2, fb2;
} lm_layer_off;

typedef struct {
    int64_t in0, in1; /* embedding (discrete) or input projection W and bias (continuous; in1 = bias) */
    lm_layer_off* layer;
    int64_t Wout, bout, total;
} lm_off;

static void lm_layout(const ref_lm_config* c, lm_off* o) {
    int a = c->align_floats, d = c->embedding_dim, f = c->ffn_dim;
    int64_t p = 0;
    if (c->discrete) { o->in0 = p; p = al(p + (int64_t)c->vocab_size * d, a); o->in1 = -1; }
    else { o->in0 = p; p = al(p + (int64_t)d * c->input_feature_dim, a); o->in1 = p; p = al(p + d, a); }
    o->layer = (lm_layer_off*)calloc((size_t)c->num_layers, sizeof(lm_layer_off));
    for (int l = 0; l < c->num_layers; l++) {
        lm_layer_off* L = &o->layer[l];
        L->WQ = p; p = al(p + (int64_t)d * d, a);
        L->WK = p; p = al(p + (int64_t)d * d, a);
        L->WV = p; p = al(p + (int64_t)d * d, a);
        L->WO = p; p = al(p + (int64_t)d * d, a);
        L->bQ = p; p = al(p + d, a);
        L->bK = p; p = al(p + d, a);
        L->bV = p; p = al(p + d, a);
        L->bO = p; p = al(p + d, a);
        L->g1 = p; p = al(p + d, a);
        L->b1n = p; p = al(p + d, a);
        L->g2 = p; p = al(p + d, a);
        L->b2n = p; p = al(p + d, a);
        L->W1 = p; p = al(p + (int64_t)f * d, a);
        L->fb1 = p; p = al(p + f, a);
        L->W2 = p; p = al(p + (int64_t)d * f, a);
        L->fb2 = p; p = al(p + d, a);
    }
    o->Wout = p; p = al(p + (int64_t)c->output_dim * d, a);
    o->bout = p; p = al(p + c->output_dim, a);
    o->total = p;
}

API int64_t ref_lm_param_count(const ref_lm_config* c) {
    lm_off o;
    lm_layout(c, &o);
    free(o.layer);
    return o.total;
}

/* Number of tensors and (offset, rows, cols) of tensor `idx` in arena order. */
API int ref_lm_tensor_count(const ref_lm_config* c) { return (c->discrete ? 1 : 2) + 16 * c->num_layers + 2; }
API int ref_lm_tensor_info(const ref_lm_config* c, int idx, int64_t* off, int32_t* rows, int32_t* cols) {
    lm_off o;
    lm_layout(c, &o);
    int d = c->embedding_dim, f = c->ffn_dim, n0 = c->discrete ? 1 : 2, rc = 0;
    if (idx < n0) {
        if (c->discrete) { *off = o.in0; *rows = c->vocab_size; *cols = d; }
        else if (idx == 0) { *off = o.in0; *rows = d; *cols = c->input_feature_dim; }
        else { *off = o.in1; *rows = 1; *cols = d; }
    } else if (idx < n0 + 16 * c->num_layers) {
        int l = (idx - n0) / 16, t = (idx - n0) % 16;
        lm_layer_off* L = &o.layer[l];
        int64_t offs[16] = {L->WQ, L->WK, L->WV, L->WO, L->bQ, L->bK, L->bV, L->bO,
                            L->g1, L->b1n, L->g2, L->b2n, L->W1, L->fb1, L->W2, L->fb2};
        int rws[16] = {d, d, d, d, 1, 1, 1, 1, 1, 1, 1, 1, f, 1, d, 1};
        int cls[16] = {d, d, d, d, d, d, d, d, d, d, d, d, d, f, f, d};
        *off = offs[t]; *rows = rws[t]; *cols = cls[t];
    } else if (idx == n0 + 16 * c->num_layers) { *off = o.Wout; *rows = c->output_dim; *cols = d; }
    else if (idx == n0 + 16 * c->num_layers + 1) { *off = o.bout; *rows = 1; *cols = c->output_dim; }
    else rc = -1;
    free(o.layer);
    return rc;
}

typedef struct {
    real *x, *Q, *K, *V, *attnOut, *ln1In, *ln1Mean, *ln1Var, *ln1Norm, *normed1, *ln2In, *ln2Mean, *ln2Var, *ln2Norm;
} layer_cache;

static real* ralloc(size_t n) { return (real*)calloc(n ? n : 1, sizeof(real)); }

/* One bucket (TT:247-296): `count` sequences of equal input length `len`, rows = count*len.
 * Forward with cache (TT:540-590), loss, dOut *= count (TT:292), BackpropFromOutput (TT:874-987).
 * Returns the bucket loss (already the mean over rows) through *lossOut and 1 if finite, else 0 (skipped). */
static int lm_bucket(const ref_lm_config* c, const lm_off* o, const real* P, real* G, const int32_t* ids,
                     const real* cont, const int32_t* tgtIds, const real* tgtReg, int len, int count, real* lossOut) {
    int d = c->embedding_dim, H = c->num_heads, f = c->ffn_dim, Lc = c->num_layers, O = c->output_dim;
    int N = len * count;
    size_t Nd = (size_t)N * d;
    real eps = (real)1e-5;
    layer_cache* cache = (layer_cache*)calloc((size_t)Lc, sizeof(layer_cache));
    real* x = ralloc(Nd);
    if (c->discrete) {
        if (ref_EmbedTokenIds(ids, 0, N, P + o->in0, c->vocab_size, d, x) != 0) { free(x); free(cache); return 0; }
    } else {
        ref_BatchDotProductAddBias(P + o->in0, d, c->input_feature_dim, cont, 0, N, P + o->in1, x);
    }
    int32_t widths[3] = {d, f, d};
    int32_t acts[3] = {ACT_NONE, c->ffn_activation, ACT_NONE};
    for (int l = 0; l < Lc; l++) {
        const lm_layer_off* L = &o->layer[l];
        layer_cache* k = &cache[l];
        k->x = x;
        k->Q = ralloc(Nd); k->K = ralloc(Nd); k->V = ralloc(Nd); k->attnOut = ralloc(Nd);
        ref_ProjectQKV(x, N, d, P + L->WQ, P + L->bQ, P + L->WK, P + L->bK, P + L->WV, P + L->bV, d, k->Q, k->K, k->V);
        /* TT:735 / TT:1130: rotary on Q and K, position = row % segment length. */
        ref_ApplyRotaryPositionEmbeddingInPlace(k->Q, N, d, H, (real)10000, 0, len);
        ref_ApplyRotaryPositionEmbeddingInPlace(k->K, N, d, H, (real)10000, 0, len);
        /* TT:560-562: a bucket of one sequence takes the manager's attention, larger buckets the trainer's own. */
        if (count == 1) ref_ScaledDotProductAttention(k->Q, k->K, k->V, N, N, d, H, NULL, c->causal, k->attnOut);
        else ref_SegmentedAttentionForward(k->Q, k->K, k->V, len, count, d, H, c->causal, k->attnOut);
        real* proj = ralloc(Nd);
        ref_ProjectOutputBatch(k->attnOut, d, P + L->WO, P + L->bO, N, d, proj);
        k->ln1In = ralloc(Nd); k->ln1Norm = ralloc(Nd); k->normed1 = ralloc(Nd);
        k->ln1Mean = ralloc((size_t)N); k->ln1Var = ralloc((size_t)N);
        ref_ResidualLayerNormForward(x, proj, P + L->g1, P + L->b1n, N, d, eps, k->normed1, k->ln1Mean, k->ln1Var,
                                     k->ln1Norm, k->ln1In);
        free(proj);
        real* ff = ralloc(Nd);
        const real* W[3] = {NULL, P + L->W1, P + L->W2};
        const real* B[3] = {NULL, P + L->fb1, P + L->fb2};
        ref_FFNForwardBatch(k->normed1, N, 3, widths, acts, W, B, ff);
        k->ln2In = ralloc(Nd); k->ln2Norm = ralloc(Nd);
        k->ln2Mean = ralloc((size_t)N); k->ln2Var = ralloc((size_t)N);
        real* nx = ralloc(Nd);
        ref_ResidualLayerNormForward(k->normed1, ff, P + L->g2, P + L->b2n, N, d, eps, nx, k->ln2Mean, k->ln2Var,
                                     k->ln2Norm, k->ln2In);
        free(ff);
        x = nx;
    }
    real* finalHidden = x;
    real* out = ralloc((size_t)N * O);
    ref_ProjectOutputBatch(finalHidden, d, P + o->Wout, P + o->bout, N, O, out);
    real* dOut = ralloc((size_t)N * O);
    real loss;
    if (c->loss_kind == 0) loss = ref_CrossEntropyLossAndGradient(out, N, O, tgtIds, 0, N, dOut);
    else loss = ref_MSELossAndGradient(out, N, O, tgtReg, 0, N, dOut);
    int ok = isfinite(loss);
    for (size_t i = 0; ok && i < (size_t)N * O; i++) if (!isfinite(dOut[i])) ok = 0;
    if (ok) {
        if (count > 1) for (size_t i = 0; i < (size_t)N * O; i++) dOut[i] *= (real)count;
        real* dX = ralloc(Nd);
        ref_BackpropOutputProjection(dOut, finalHidden, P + o->Wout, G + o->Wout, G + o->bout, N, O, d, dX);
        real* dg = ralloc((size_t)d);
        real* db = ralloc((size_t)d);
        for (int l = Lc - 1; l >= 0; l--) {
            const lm_layer_off* L = &o->layer[l];
            layer_cache* k = &cache[l];
            /* TT:898-921 BackpropBlock */
            real* dFF = ralloc(Nd);
            ref_LayerNormBackward(dX, k->ln2Norm, P + L->g2, k->ln2In, k->ln2Mean, k->ln2Var, N, d, eps, dFF, dg, db);
            ref_AddInPlace(G + L->g2, dg, d);
            ref_AddInPlace(G + L->b2n, db, d);
            real* dN1 = ralloc(Nd);
            const real* W[3] = {NULL, P + L->W1, P + L->W2};
            const real* B[3] = {NULL, P + L->fb1, P + L->fb2};
            real* WG[3] = {NULL, G + L->W1, G + L->W2};
            real* BG[3] = {NULL, G + L->fb1, G + L->fb2};
            ref_FFNInputGradientBatch(k->normed1, dFF, N, 3, widths, acts, W, B, WG, BG, dN1);
            ref_AddInPlace(dN1, dFF, (int64_t)Nd);
            real* dAR = ralloc(Nd);
            ref_LayerNormBackward(dN1, k->ln1Norm, P + L->g1, k->ln1In, k->ln1Mean, k->ln1Var, N, d, eps, dAR, dg, db);
            ref_AddInPlace(G + L->g1, dg, d);
            ref_AddInPlace(G + L->b1n, db, d);
            /* TT:933-987 BackpropAttention */
            real* dCat = ralloc(Nd);
            ref_BackpropLinearProjection(k->attnOut, dAR, P + L->WO, N, d, d, G + L->WO, G + L->bO, dCat);
            real *dQ = ralloc(Nd), *dK = ralloc(Nd), *dV = ralloc(Nd);
            real scale = (real)1 / R_SQRT((real)(d / H));
            if (count == 1) ref_MultiHeadAttentionBackward(k->Q, k->K, k->V, dCat, N, N, d, H, scale, NULL, c->causal, dQ, dK, dV);
            else ref_SegmentedAttentionBackward(k->Q, k->K, k->V, dCat, len, count, d, H, scale, c->causal, dQ, dK, dV);
            ref_ApplyRotaryPositionEmbeddingInPlace(dQ, N, d, H, (real)10000, 1, len);
            ref_ApplyRotaryPositionEmbeddingInPlace(dK, N, d, H, (real)10000, 1, len);
            real* dXa = ralloc(Nd);
            ref_BackpropQKV(k->x, N, d, dQ, dK, dV, d, P + L->WQ, P + L->WK, P + L->WV, G + L->WQ, G + L->bQ,
                            G + L->WK, G + L->bK, G + L->WV, G + L->bV, dXa);
            ref_AddInPlace(dXa, dAR, (int64_t)Nd);
            free(dFF); free(dN1); free(dAR); free(dCat); free(dQ); free(dK); free(dV); free(dX);
            dX = dXa;
        }
        /* TT:887-896 BackpropInput */
        if (c->discrete) ref_AccumulateTokenEmbeddingGrad(G + o->in0, dX, ids, 0, N, d);
        else ref_BackpropInputProjection(dX, cont, c->input_feature_dim, 0, G + o->in0, G + o->in1, N, d,
                                         c->input_feature_dim);
        free(dX); free(dg); free(db);
    }
    *lossOut = loss;
    for (int l = 0; l < Lc; l++) {
        layer_cache* k = &cache[l];
        free(k->x); free(k->Q); free(k->K); free(k->V); free(k->attnOut); free(k->ln1In); free(k->ln1Mean);
        free(k->ln1Var); free(k->ln1Norm); free(k->normed1); free(k->ln2In); free(k->ln2Mean); free(k->ln2Var);
        free(k->ln2Norm);
    }
    free(finalHidden); free(out); free(dOut); free(cache);
    return ok;
}

/* TT:217-327 TrainBatchDiscrete / TT:337-486 TrainBatchContinuous on a flat arena.
 *   tokens/seqOff : discrete sequences, sequence s = tokens[seqOff[s] .. seqOff[s+1]) (inputs are all but the
 *                   last id, targets all but the first);
 *   contIn/regTgt/clsTgt : continuous sequences with seqOff counting rows; features [rows,F], regression targets
 *                   [rows,O] or class targets [rows]; row t is trained against target row t+1 (TT:703).
 * Gradients are zeroed, accumulated bucket by bucket in order of first appearance of each length
 * (Dictionary insertion order), scaled by 1/validCount, clipped by global norm, and applied with SGD when
 * doStep != 0.  Returns totalLoss/validCount (0 if nothing valid). */
API real ref_lm_train_step(const ref_lm_config* c, real* P, real* G, const int32_t* tokens, const real* contIn,
                           const real* regTgt, const int32_t* clsTgt, const int32_t* seqOff, int nSeq, real lr,
                           int useClip, real clipThr, int doStep, real* gradNormOut, int32_t* validOut) {
    lm_off o;
    lm_layout(c, &o);
    memset(G, 0, sizeof(real) * (size_t)o.total);
    int* lens = (int*)malloc(sizeof(int) * (size_t)(nSeq + 1));
    char* used = (char*)calloc((size_t)nSeq + 1, 1);
    int F = c->input_feature_dim, O = c->output_dim;
    for (int s = 0; s < nSeq; s++) {
        int n = seqOff[s + 1] - seqOff[s];
        int valid = n >= 2;
        if (valid && c->discrete) /* TT:1467-1478 TokensAreValid */
            for (int t = 0; t < n; t++) {
                int id = tokens[seqOff[s] + t];
                if (id < 0 || id >= c->vocab_size) { valid = 0; break; }
            }
        lens[s] = valid ? n - 1 : -1;
    }
    real totalLoss = 0;
    int validCount = 0;
    for (int s0 = 0; s0 < nSeq; s0++) {
        if (used[s0] || lens[s0] < 0) continue;
        int len = lens[s0], count = 0;
        for (int s = s0; s < nSeq; s++) if (!used[s] && lens[s] == len) count++;
        int N = len * count;
        int32_t* ids = (int32_t*)calloc((size_t)N + 1, sizeof(int32_t));
        int32_t* tgt = (int32_t*)calloc((size_t)N + 1, sizeof(int32_t));
        real* cont = c->discrete ? NULL : ralloc((size_t)N * F);
        real* rt = (c->loss_kind == 1) ? ralloc((size_t)N * O) : NULL;
        int b = 0;
        for (int s = s0; s < nSeq; s++) {
            if (used[s] || lens[s] != len) continue;
            used[s] = 1;
            int base = seqOff[s];
            for (int t = 0; t < len; t++) {
                if (c->discrete) { ids[b * len + t] = tokens[base + t]; tgt[b * len + t] = tokens[base + t + 1]; }
                else {
                    memcpy(cont + ((size_t)b * len + t) * F, contIn + (size_t)(base + t) * F, sizeof(real) * (size_t)F);
                    if (c->loss_kind == 1)
                        memcpy(rt + ((size_t)b * len + t) * O, regTgt + (size_t)(base + t + 1) * O, sizeof(real) * (size_t)O);
                    else tgt[b * len + t] = clsTgt[base + t + 1];
                }
            }
            b++;
        }
        real loss = 0;
        if (lm_bucket(c, &o, P, G, ids, cont, tgt, rt, len, count, &loss)) {
            totalLoss += loss * (real)count;
            validCount += count;
        }
        free(ids); free(tgt); free(cont); free(rt);
    }
    free(lens); free(used);
    if (validOut) *validOut = validCount;
    if (gradNormOut) *gradNormOut = 0;
    if (validCount == 0) { free(o.layer); return 0; }
    ref_ScaleInPlace(G, o.total, (real)1 / validCount); /* TT:313 */
    real norm = R_SQRT(ref_SquaredNorm(G, o.total));    /* TT:1319-1352 */
    if (gradNormOut) *gradNormOut = norm;
    if (!isfinite(norm)) { memset(G, 0, sizeof(real) * (size_t)o.total); free(o.layer); return totalLoss / validCount; }
    if (useClip && norm > clipThr) ref_ScaleInPlace(G, o.total, clipThr / norm); /* TT:1311-1318 */
    if (doStep) ref_Update(P, G, o.total, lr);                                   /* TT:1269-1305 */
    free(o.layer);
    return totalLoss / validCount;
}

/* TT:1142-1184 Validate / TT:1185-1268 ValidateContinuous: every valid sequence on its own, forward and loss only
 * (the forward of a single sequence is the count == 1 path of lm_bucket; its gradients go to a scratch arena and are
 * dropped).  totalLoss += loss * effectiveLen, totalItems += effectiveLen; sequences with a non-finite loss are skipped.
 * Returns totalLoss / totalItems (0 when nothing contributed). */
API real ref_lm_validate(const ref_lm_config* c, const real* P, const int32_t* tokens, const real* contIn, const real* regTgt,
                         const int32_t* clsTgt, const int32_t* seqOff, int nSeq, int32_t* itemsOut) {
    lm_off o;
    lm_layout(c, &o);
    real* G = ralloc((size_t)o.total);
    int F = c->input_feature_dim, O = c->output_dim;
    real totalLoss = 0;
    int totalItems = 0;
    for (int s = 0; s < nSeq; s++) {
        int n = seqOff[s + 1] - seqOff[s];
        if (n < 2) continue;
        int base = seqOff[s], len = n - 1, valid = 1;
        if (c->discrete) /* TT:1467-1478 TokensAreValid */
            for (int t = 0; t < n; t++) {
                int id = tokens[base + t];
                if (id < 0 || id >= c->vocab_size) { valid = 0; break; }
            }
        if (!valid) continue;
        int32_t* ids = (int32_t*)calloc((size_t)len + 1, sizeof(int32_t));
        int32_t* tgt = (int32_t*)calloc((size_t)len + 1, sizeof(int32_t));
        real* cont = c->discrete ? NULL : ralloc((size_t)len * F);
        real* rt = (c->loss_kind == 1) ? ralloc((size_t)len * O) : NULL;
        for (int t = 0; t < len; t++) {
            if (c->discrete) { ids[t] = tokens[base + t]; tgt[t] = tokens[base + t + 1]; }
            else {
                memcpy(cont + (size_t)t * F, contIn + (size_t)(base + t) * F, sizeof(real) * (size_t)F);
                if (c->loss_kind == 1) memcpy(rt + (size_t)t * O, regTgt + (size_t)(base + t + 1) * O, sizeof(real) * (size_t)O);
                else tgt[t] = clsTgt[base + t + 1];
            }
        }
        real loss = 0;
        lm_bucket(c, &o, P, G, ids, cont, tgt, rt, len, 1, &loss);
        if (isfinite(loss)) {
            totalLoss += loss * (real)len;
            totalItems += len;
        }
        free(ids); free(tgt); free(cont); free(rt);
    }
    free(G); free(o.layer);
    if (itemsOut) *itemsOut = totalItems;
    return totalItems > 0 ? totalLoss / (real)totalItems : 0;
}

/* LM:293-537 incremental decoding with a per-layer key/value cache: every token (prompt tokens included, LM:517-520) is
 * pushed through ForwardDecoderTokenFromId at its absolute position; after each one ProjectLastTokenOnly (LM:235-268)
 * gives the next-token logits.  logitsOut[t*O .. ) = logits after token t.  The rotary angle uses the absolute position
 * (LM:450-476); attention is the three-pass loop of LM:378-428 over the cached keys, no mask (all keys are in the past).
 * Returns 0, or -1 for an invalid token id / too many tokens. */
API int ref_lm_decode_logits(const ref_lm_config* c, const real* P, const int32_t* tokens, int n, int maxLen, real* logitsOut) {
    if (n > maxLen) return -1;
    lm_off o;
    lm_layout(c, &o);
    int d = c->embedding_dim, H = c->num_heads, hd = d / H, f = c->ffn_dim, Lc = c->num_layers, O = c->output_dim;
    real eps = (real)1e-5;
    real** Kc = (real**)calloc((size_t)Lc, sizeof(real*));
    real** Vc = (real**)calloc((size_t)Lc, sizeof(real*));
    for (int l = 0; l < Lc; l++) { Kc[l] = ralloc((size_t)maxLen * d); Vc[l] = ralloc((size_t)maxLen * d); }
    int32_t widths[3] = {d, f, d};
    int32_t acts[3] = {ACT_NONE, c->ffn_activation, ACT_NONE};
    real *x = ralloc((size_t)d), *q = ralloc((size_t)d), *k = ralloc((size_t)d), *v = ralloc((size_t)d), *cat = ralloc((size_t)d),
         *proj = ralloc((size_t)d), *n1 = ralloc((size_t)d), *ff = ralloc((size_t)d), *nx = ralloc((size_t)d), *tmpN = ralloc((size_t)d),
         *tmpR = ralloc((size_t)d);
    real mean, var;
    int rc = 0;
    for (int pos = 0; pos < n && rc == 0; pos++) {
        int id = tokens[pos];
        if (id < 0 || id >= c->vocab_size) { rc = -1; break; }
        memcpy(x, P + o.in0 + (size_t)id * d, sizeof(real) * (size_t)d);
        for (int l = 0; l < Lc; l++) {
            const lm_layer_off* L = &o.layer[l];
            ref_ProjectQKV(x, 1, d, P + L->WQ, P + L->bQ, P + L->WK, P + L->bK, P + L->WV, P + L->bV, d, q, k, v);
            for (int h = 0; h < H; h++) /* LM:450-476 ApplyRotaryPositionSingleRow */
                for (int pr = 0; pr < hd / 2; pr++) {
                    real theta = (real)pos / R_POW((real)10000, ((real)2 * pr) / hd);
                    real cs = R_COS(theta), sn = R_SIN(theta);
                    int e = h * hd + 2 * pr;
                    real q0 = q[e], q1 = q[e + 1], k0 = k[e], k1 = k[e + 1];
                    q[e] = q0 * cs - q1 * sn; q[e + 1] = q0 * sn + q1 * cs;
                    k[e] = k0 * cs - k1 * sn; k[e + 1] = k0 * sn + k1 * cs;
                }
            memcpy(Kc[l] + (size_t)pos * d, k, sizeof(real) * (size_t)d);
            memcpy(Vc[l] + (size_t)pos * d, v, sizeof(real) * (size_t)d);
            int keyLen = pos + 1;
            real scale = (real)1 / R_SQRT((real)hd);
            for (int e = 0; e < d; e++) cat[e] = 0;
            for (int h = 0; h < H; h++) { /* LM:378-428 */
                int off = h * hd;
                real maxS = -INFINITY;
                for (int kj = 0; kj < keyLen; kj++) {
                    real dot = 0;
                    for (int e = 0; e < hd; e++) dot += q[off + e] * Kc[l][(size_t)kj * d + off + e];
                    real sc = dot * scale;
                    if (sc > maxS) maxS = sc;
                }
                real sumExp = 0;
                for (int kj = 0; kj < keyLen; kj++) {
                    real dot = 0;
                    for (int e = 0; e < hd; e++) dot += q[off + e] * Kc[l][(size_t)kj * d + off + e];
                    sumExp += R_EXP(dot * scale - maxS);
                }
                real inv = sumExp > 0 ? (real)1 / sumExp : 0;
                for (int kj = 0; kj < keyLen; kj++) {
                    real dot = 0;
                    for (int e = 0; e < hd; e++) dot += q[off + e] * Kc[l][(size_t)kj * d + off + e];
                    real w = R_EXP(dot * scale - maxS) * inv;
                    if (w == 0) continue;
                    for (int e = 0; e < hd; e++) cat[off + e] += w * Vc[l][(size_t)kj * d + off + e];
                }
            }
            ref_ProjectOutputBatch(cat, d, P + L->WO, P + L->bO, 1, d, proj);
            ref_ResidualLayerNormForward(x, proj, P + L->g1, P + L->b1n, 1, d, eps, n1, &mean, &var, tmpN, tmpR);
            const real* W[3] = {NULL, P + L->W1, P + L->W2};
            const real* B[3] = {NULL, P + L->fb1, P + L->fb2};
            ref_FFNForwardBatch(n1, 1, 3, widths, acts, W, B, ff);
            ref_ResidualLayerNormForward(n1, ff, P + L->g2, P + L->b2n, 1, d, eps, nx, &mean, &var, tmpN, tmpR);
            memcpy(x, nx, sizeof(real) * (size_t)d);
        }
        for (int oi = 0; oi < O; oi++) { /* LM:235-268 ProjectLastTokenOnly: the bias starts the sum */
            real sum = P[o.bout + oi];
            for (int e = 0; e < d; e++) sum += P[o.Wout + (size_t)oi * d + e] * x[e];
            logitsOut[(size_t)pos * O + oi] = sum;
        }
    }
    for (int l = 0; l < Lc; l++) { free(Kc[l]); free(Vc[l]); }
    free(Kc); free(Vc); free(x); free(q); free(k); free(v); free(cat); free(proj); free(n1); free(ff); free(nx); free(tmpN); free(tmpR);
    free(o.layer);
    return rc;
}

/* ---------------------------------------------------------------- MLP mini-batch step (NN:499-610, GPUB:251-358) */

enum { COST_MSE = 0, COST_ZERO_WEIGHTED_MSE = 1, COST_BCE = 2, COST_MAE = 3, COST_CCE = 4, COST_HUBER = 5 };

/* GPUB:251-290 BatchKernel activation and derivative conventions (ReLU'(0)=0, LeakyReLU' = 0.01, Swish -> 0). */
static void mlp_act_der(real z, int t, real* a, real* d) {
    switch (t) {
        case ACT_NONE: *a = z; *d = 1; break;
        case ACT_SIGMOID: { real e = R_EXP(z); *a = e / ((real)1 + e); *d = *a * ((real)1 - *a); break; }
        case ACT_TANH: *a = R_TANH(z); *d = (real)1 - *a * *a; break;
        case ACT_RELU: *a = z > 0 ? z : 0; *d = z > 0 ? 1 : 0; break;
        case ACT_LEAKYRELU: *a = z > 0 ? z : (real)0.01 * z; *d = z > 0 ? 1 : (real)0.01; break;
        default: *a = 0; *d = 0; break;
    }
}

/* NN:314-390 CostFunctionDeriv(ActualValue := activation a, predicted := target y) as called at NN:514. */
static real cost_deriv(int kind, real a, real y, real huberDelta) {
    switch (kind) {
        case COST_MSE: return (real)2 * (y - a);
        case COST_ZERO_WEIGHTED_MSE: return (real)2 * (a == 0 ? (real)0.25 : (real)1) * (y - a);
        case COST_BCE: return (y - a) / (y * ((real)1 - y));
        case COST_MAE: return a > y ? (real)-1 : (real)1;
        case COST_CCE: return y - a;
        default: {
            real diff = a - y;
            if (R_FABS(diff) <= huberDelta) return diff;
            return huberDelta * (real)((diff > 0) - (diff < 0));
        }
    }
}

/* NN:499-520 LearnBatch + NN:542-553 BackPropagateBatch on one mini-batch X [B, widths[0]] (already input-scaled),
 * Y [B, widths[L]].  weights[l]/biases[l] (l = 1..nLayers-1) are updated in place.  Returns the delta norm. */
API real ref_mlp_learn_batch(int nLayers, const int32_t* widths, const int32_t* acts, real* const* weights,
                             real* const* biases, const real* X, const real* Y, int B, int costKind, real huberDelta,
                             real lr, real lambda, real clipThr) {
    int L = nLayers - 1;
    real** A = (real**)calloc((size_t)nLayers, sizeof(real*));
    real** D = (real**)calloc((size_t)nLayers, sizeof(real*));
    real** dl = (real**)calloc((size_t)nLayers, sizeof(real*));
    A[0] = (real*)X;
    for (int l = 1; l <= L; l++) { /* NN:522-541 ForwardPropagateBatch -> GPUB:251-290 */
        int n = widths[l], kdim = widths[l - 1];
        A[l] = ralloc((size_t)B * n);
        D[l] = ralloc((size_t)B * n);
        PAR
        for (int i = 0; i < B; i++)
            for (int j = 0; j < n; j++) {
                real sum = 0;
                for (int k = 0; k < kdim; k++) sum += A[l - 1][(size_t)i * kdim + k] * weights[l][(size_t)j * kdim + k];
                mlp_act_der(sum + biases[l][j], acts[l], &A[l][(size_t)i * n + j], &D[l][(size_t)i * n + j]);
            }
    }
    int nOut = widths[L];
    dl[L] = ralloc((size_t)B * nOut); /* GPUB:315-322: delta = -cost * deriv */
    for (size_t i = 0; i < (size_t)B * nOut; i++) dl[L][i] = -cost_deriv(costKind, A[L][i], Y[i], huberDelta) * D[L][i];
    for (int l = L - 1; l >= 1; l--) { /* GPUB:324-335 */
        int n = widths[l], nn = widths[l + 1];
        dl[l] = ralloc((size_t)B * n);
        PAR
        for (int i = 0; i < B; i++)
            for (int j = 0; j < n; j++) {
                real sum = 0;
                for (int k = 0; k < nn; k++) sum += dl[l + 1][(size_t)i * nn + k] * weights[l + 1][(size_t)k * n + j];
                dl[l][(size_t)i * n + j] = sum * D[l][(size_t)i * n + j];
            }
    }
    real sumSq = 0; /* NN:571-580 */
    for (int l = L; l >= 1; l--)
        for (size_t i = 0; i < (size_t)B * widths[l]; i++) sumSq += dl[l][i] * dl[l][i];
    real norm = R_SQRT(sumSq);
    real scale = norm > clipThr ? clipThr / norm : (real)1; /* NN:242-245 */
    if (scale != (real)1)
        for (int l = L; l >= 1; l--)
            for (size_t i = 0; i < (size_t)B * widths[l]; i++) dl[l][i] *= scale;
    real slr = lr / B;
    for (int l = L; l >= 1; l--) { /* GPUB:209-234, 292-358 */
        int n = widths[l], kdim = widths[l - 1];
        PAR
        for (int r = 0; r < n; r++) {
            for (int cc = 0; cc < kdim; cc++) {
                real sum = 0;
                for (int i = 0; i < B; i++) sum += dl[l][(size_t)i * n + r] * A[l - 1][(size_t)i * kdim + cc];
                real w = weights[l][(size_t)r * kdim + cc];
                weights[l][(size_t)r * kdim + cc] = w - slr * (sum + lambda * w);
            }
            real bs = 0;
            for (int i = 0; i < B; i++) bs += dl[l][(size_t)i * n + r];
            biases[l][r] = biases[l][r] - slr * bs;
        }
    }
    for (int l = 1; l <= L; l++) { free(A[l]); free(D[l]); free(dl[l]); }
    free(A); free(D); free(dl);
    return norm;
}

/* NN:121-134 ScaleInput with NN:135-157 CalibrateInputs ranges: x' = (x-min)/(max-min), 0 when the range is <= 0. */
API void ref_mlp_scale_inputs(const real* X, int B, int F, const real* mn, const real* mx, real* out) {
    for (int i = 0; i < B; i++)
        for (int j = 0; j < F; j++) {
            real range = mx[j] - mn[j];
            out[(size_t)i * F + j] = range <= 0 ? 0 : (X[(size_t)i * F + j] - mn[j]) / range;
        }
}

/* ===================================================================================================================
 * Operators of the sibling trainers (TACAMT / MMTAC / PriceTAC) on the same interface, restated in the reference's
 * loop order.  Rank-3 arrays are flat in the reference's element order.  PARITY UNPINNED: the reference's tests for
 * these operators compare its back ends with each other and hold no known-answer values; the restatement is checked
 * against an independent float64 statement of the same mathematics instead. */

/* CPU:3076-3270 ContentAwareCrossAttentionForward.  bias [q,k,H] or NULL; W and S are [H,q,k] (always written here;
 * the wrapper drops them for needBackwardCache = false, the output is the same on both branches). */
API void ref_ContentAwareCrossAttentionForward(const real* Q, int qLen, const real* K, const real* V, int kLen, int E, int H, real scale,
                                               const real* bias, real* out, real* W, real* S) {
    const int hd = E / H;
    for (size_t i = 0; i < (size_t)qLen * E; i++) out[i] = 0;
    for (size_t i = 0; i < (size_t)H * qLen * kLen; i++) { W[i] = 0; S[i] = 0; }
    for (int h = 0; h < H; h++) {
        const int off = h * hd;
        for (int q = 0; q < qLen; q++) {
            real* s = S + ((size_t)h * qLen + q) * kLen;
            real* w = W + ((size_t)h * qLen + q) * kLen;
            real mx = -INFINITY;
            for (int k = 0; k < kLen; k++) {
                real dot = 0;
                for (int d = 0; d < hd; d++) dot += Q[(size_t)q * E + off + d] * K[(size_t)k * E + off + d];
                real sc = dot * scale;
                if (bias) sc += bias[((size_t)q * kLen + k) * H + h];
                s[k] = sc;
                if (!(isinf(sc) && sc < 0) && sc > mx) mx = sc;
            }
            if (isinf(mx) && mx < 0) continue;
            real sum = 0;
            for (int k = 0; k < kLen; k++) {
                if (isinf(s[k]) && s[k] < 0) { w[k] = 0; continue; }
                w[k] = R_EXP(s[k] - mx);
                sum += w[k];
            }
            if (sum > 0) {
                const real inv = (real)1 / sum;
                for (int k = 0; k < kLen; k++) w[k] *= inv;
            }
            for (int k = 0; k < kLen; k++)
                if (w[k] != 0)
                    for (int d = 0; d < hd; d++) out[(size_t)q * E + off + d] += w[k] * V[(size_t)k * E + off + d];
        }
    }
}

/* CPU:3748-3857 BackpropTimeDecayedAttention.  W is [H,q,k]; dBias [q,k,H] or NULL; dQ, dK, dV start at zero. */
API void ref_BackpropTimeDecayedAttention(const real* q, int qLen, const real* k, const real* v, int kLen, const real* dO, const real* W, int E,
                                          int H, real* dQ, real* dK, real* dV, real* dBias) {
    const int hd = E / H;
    const real scale = (real)1 / R_SQRT((real)hd);
    for (size_t i = 0; i < (size_t)qLen * E; i++) dQ[i] = 0;
    for (size_t i = 0; i < (size_t)kLen * E; i++) { dK[i] = 0; dV[i] = 0; }
    if (dBias) for (size_t i = 0; i < (size_t)qLen * kLen * H; i++) dBias[i] = 0;
    real* dW = (real*)malloc(sizeof(real) * (size_t)(kLen > 0 ? kLen : 1));
    for (int h = 0; h < H; h++) {
        const int off = h * hd;
        for (int p = 0; p < qLen; p++) {
            const real* w = W + ((size_t)h * qLen + p) * kLen;
            for (int s = 0; s < kLen; s++) {
                real dot = 0;
                for (int d = 0; d < hd; d++) {
                    const real g = dO[(size_t)p * E + off + d];
                    dV[(size_t)s * E + off + d] += w[s] * g;
                    dot += g * v[(size_t)s * E + off + d];
                }
                dW[s] = dot;
            }
            real dotwg = 0;
            for (int s = 0; s < kLen; s++) dotwg += w[s] * dW[s];
            for (int s = 0; s < kLen; s++) {
                const real ds = w[s] * (dW[s] - dotwg), dsc = ds * scale;
                for (int d = 0; d < hd; d++) {
                    dQ[(size_t)p * E + off + d] += dsc * k[(size_t)s * E + off + d];
                    dK[(size_t)s * E + off + d] += dsc * q[(size_t)p * E + off + d];
                }
                if (dBias) dBias[((size_t)p * kLen + s) * H + h] += ds;
            }
        }
    }
    free(dW);
}

/* CPU:2596-2644 */
API void ref_ApplyContextTypeEmbedding(real* hidden, int rows, int E, const real* typeEmb, const int* idx) {
    for (int i = 0; i < rows; i++)
        for (int d = 0; d < E; d++) hidden[(size_t)i * E + d] += typeEmb[(size_t)idx[i] * E + d];
}
/* CPU:2646-2674 */
API void ref_ComputeTimeDiffMatrix(int rows, const real* keyTimes, int keys, real* out) {
    for (int p = 0; p < rows; p++)
        for (int s = 0; s < keys; s++) out[(size_t)p * keys + s] = (real)p - keyTimes[s];
}
/* CPU:2676-2692 */
API void ref_ComputeMemoryAttentionScores(const real* price, int E, int lastPos, const real* ctx, int totalCtx, real scale, real* scores) {
    for (int s = 0; s < totalCtx; s++) {
        real dot = 0;
        for (int d = 0; d < E; d++) dot += price[(size_t)lastPos * E + d] * ctx[(size_t)s * E + d];
        scores[s] = dot * scale;
    }
}
/* CPU:3424-3461 */
API void ref_ProjectGlobalFeatures(const real* g, int gd, const real* proj, const real* bias, int ed, real* out) {
    for (int d = 0; d < ed; d++) {
        real dot = 0;
        for (int j = 0; j < gd; j++) dot += proj[(size_t)d * gd + j] * g[j];
        out[d] = bias[d] + dot;
    }
}
/* CPU:3517-3552 */
API void ref_MeanPoolRows(const real* m, int rows, int cols, real* out) {
    for (int d = 0; d < cols; d++) out[d] = 0;
    if (rows == 0) return;
    for (int r = 0; r < rows; r++)
        for (int d = 0; d < cols; d++) out[d] += m[(size_t)r * cols + d];
    const real inv = (real)1 / (real)rows;
    for (int d = 0; d < cols; d++) out[d] *= inv;
}
/* CPU:4321-4359 */
API void ref_ExpandMeanPoolGradient(const real* pooled, int pooledCols, int rowIndex, int rowCount, int E, real* out) {
    const real inv = (real)1 / (real)rowCount;
    for (int t = 0; t < rowCount; t++)
        for (int d = 0; d < E; d++) out[(size_t)t * E + d] = pooled[(size_t)rowIndex * pooledCols + d] * inv;
}
/* CPU:3700-3746 */
API void ref_SoftmaxVector(const real* x, int n, real* out) {
    if (n == 0) return;
    real mx = -INFINITY, sum = 0;
    for (int i = 0; i < n; i++) if (x[i] > mx) mx = x[i];
    for (int i = 0; i < n; i++) { out[i] = R_EXP(x[i] - mx); sum += out[i]; }
    if (sum <= 0) return;
    const real inv = (real)1 / sum;
    for (int i = 0; i < n; i++) out[i] *= inv;
}
/* CPU:4985-4992 (StableSigmoidCore, CPU:143-153) */
API void ref_SigmoidInPlace(real* m, long long n) { for (long long i = 0; i < n; i++) m[i] = stable_sigmoid(m[i]); }
/* CPU:5016-5035 */
API void ref_ZeroMatrixColumns(real* m, int rows, int cols, int count) {
    if (count <= 0) return;
    if (count > cols) count = cols;
    for (int i = 0; i < rows; i++)
        for (int c = 0; c < count; c++) m[(size_t)i * cols + c] = 0;
}
/* CPU:5037-5056 */
API void ref_VectorUpdateClamped(real* w, const real* g, long long n, real lr, real lo, real hi) {
    for (long long i = 0; i < n; i++) {
        const real v = w[i] - lr * g[i];
        w[i] = v < lo ? lo : (v > hi ? hi : v);
    }
}
/* CPU:4296-4319 */
API void ref_AccumulateGlobalProjectionGradients(const real* dGlobal, int ed, const real* feat, int gd, real* projGrad, real* biasGrad) {
    for (int d = 0; d < ed; d++) {
        biasGrad[d] += dGlobal[d];
        for (int g = 0; g < gd; g++) projGrad[(size_t)d * gd + g] += dGlobal[d] * feat[g];
    }
}
