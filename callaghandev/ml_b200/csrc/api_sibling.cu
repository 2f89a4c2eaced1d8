// C ABI, part C: the operators the reference's sibling trainers (TACAMT / MMTAC / PriceTAC) share with the
// language-model path: cross-attention with an additive per-head decay bias and its backward pass over materialised
// attention weights, and the small context / pooling / update helpers around them
// (IAccelerationManager.cs:251-361).  Same contract as the other per-op entry points: host arrays in, host arrays out,
// arguments checked on the host, one synchronisation before returning.
#include <cmath>

#include "api_scope.cuh"
#include "device_math.cuh"

namespace {

constexpr int ATT_THREADS = 128;

// ---------------------------------------------------------------------------------------------------------------
// Forward (AccelerationCPU.cs:3076-3270).  One block per (query row, head): scores over all keys, a soft-max that
// skips -inf scores (a row whose scores are all -inf keeps zero weights and a zero output), then the weighted sum of
// the value rows.  Scores and weights are materialised in [head][query][key] order because the backward pass and
// the callers' caches consume them in that form.
__global__ void __launch_bounds__(ATT_THREADS) decay_attn_fwd_kernel(const float* __restrict__ Q, const float* __restrict__ K,
                                                                      const float* __restrict__ V, const float* __restrict__ bias,
                                                                      int qLen, int kLen, int E, int H, float scale,
                                                                      float* __restrict__ out, float* __restrict__ weights,
                                                                      float* __restrict__ scores) {
    __shared__ float red[32];
    extern __shared__ float qrow[];  // headDim floats
    const int q = blockIdx.x, h = blockIdx.y, hd = E / H, off = h * hd;
    const int tid = threadIdx.x;
    for (int d = tid; d < hd; d += ATT_THREADS) qrow[d] = Q[(size_t)q * E + off + d];
    __syncthreads();
    float* srow = scores + ((size_t)h * qLen + q) * kLen;
    float* wrow = weights + ((size_t)h * qLen + q) * kLen;
    float mx = -INFINITY;
    for (int s = tid; s < kLen; s += ATT_THREADS) {
        const float* kr = K + (size_t)s * E + off;
        float acc = 0.f;
        for (int d = 0; d < hd; d++) acc = fmaf(qrow[d], kr[d], acc);
        float sc = acc * scale;
        if (bias) sc += bias[((size_t)q * kLen + s) * H + h];
        srow[s] = sc;
        if (sc != -INFINITY && sc > mx) mx = sc;
    }
    mx = block_max(mx, red);
    if (mx == -INFINITY) {  // nothing to attend to: weights and output stay zero
        for (int s = tid; s < kLen; s += ATT_THREADS) wrow[s] = 0.f;
        for (int d = tid; d < hd; d += ATT_THREADS) out[(size_t)q * E + off + d] = 0.f;
        return;
    }
    float sum = 0.f;
    for (int s = tid; s < kLen; s += ATT_THREADS) {
        const float sc = srow[s];
        const float w = sc == -INFINITY ? 0.f : expf(sc - mx);
        wrow[s] = w;
        sum += w;
    }
    sum = block_sum(sum, red);
    const float inv = sum > 0.f ? 1.f / sum : 1.f;
    for (int s = tid; s < kLen; s += ATT_THREADS) wrow[s] *= inv;
    __syncthreads();
    for (int d = tid; d < hd; d += ATT_THREADS) {
        float acc = 0.f;
        for (int s = 0; s < kLen; s++) acc = fmaf(wrow[s], V[(size_t)s * E + off + d], acc);
        out[(size_t)q * E + off + d] = acc;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Backward over given weights (AccelerationCPU.cs:3748-3857), in two deterministic passes without atomics.
// Pass 1, one block per (query row, head): dWeights, the soft-max Jacobian, dScore (also the decay-bias gradient)
// and this row's dQ.
__global__ void __launch_bounds__(ATT_THREADS) decay_attn_bwd_rows_kernel(const float* __restrict__ K, const float* __restrict__ V,
                                                                           const float* __restrict__ dO, const float* __restrict__ W,
                                                                           int qLen, int kLen, int E, int H, float scale,
                                                                           float* __restrict__ dS, float* __restrict__ dQ,
                                                                           float* __restrict__ dBias) {
    __shared__ float red[32];
    extern __shared__ float dorow[];  // headDim floats
    const int p = blockIdx.x, h = blockIdx.y, hd = E / H, off = h * hd, tid = threadIdx.x;
    for (int d = tid; d < hd; d += ATT_THREADS) dorow[d] = dO[(size_t)p * E + off + d];
    __syncthreads();
    const float* wrow = W + ((size_t)h * qLen + p) * kLen;
    float* dsrow = dS + ((size_t)h * qLen + p) * kLen;
    float dotwg = 0.f;
    for (int s = tid; s < kLen; s += ATT_THREADS) {
        const float* vr = V + (size_t)s * E + off;
        float acc = 0.f;
        for (int d = 0; d < hd; d++) acc = fmaf(dorow[d], vr[d], acc);
        dsrow[s] = acc;  // dWeights for now
        dotwg = fmaf(wrow[s], acc, dotwg);
    }
    dotwg = block_sum(dotwg, red);
    for (int s = tid; s < kLen; s += ATT_THREADS) {
        const float ds = wrow[s] * (dsrow[s] - dotwg);
        dsrow[s] = ds;
        if (dBias) dBias[((size_t)p * kLen + s) * H + h] = ds;
    }
    __syncthreads();
    for (int d = tid; d < hd; d += ATT_THREADS) {
        float acc = 0.f;
        for (int s = 0; s < kLen; s++) acc = fmaf(dsrow[s] * scale, K[(size_t)s * E + off + d], acc);
        dQ[(size_t)p * E + off + d] = acc;
    }
}
// Pass 2, one block per (key row, head): dK and dV gather over the query rows.
__global__ void __launch_bounds__(ATT_THREADS) decay_attn_bwd_keys_kernel(const float* __restrict__ Q, const float* __restrict__ dO,
                                                                           const float* __restrict__ W, const float* __restrict__ dS,
                                                                           int qLen, int kLen, int E, int H, float scale,
                                                                           float* __restrict__ dK, float* __restrict__ dV) {
    const int s = blockIdx.x, h = blockIdx.y, hd = E / H, off = h * hd, tid = threadIdx.x;
    for (int d = tid; d < hd; d += ATT_THREADS) {
        float ak = 0.f, av = 0.f;
        for (int p = 0; p < qLen; p++) {
            const size_t i = ((size_t)h * qLen + p) * kLen + s;
            ak = fmaf(dS[i] * scale, Q[(size_t)p * E + off + d], ak);
            av = fmaf(W[i], dO[(size_t)p * E + off + d], av);
        }
        dK[(size_t)s * E + off + d] = ak;
        dV[(size_t)s * E + off + d] = av;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Small helpers.
__global__ void time_diff_kernel(const float* __restrict__ keyTimes, int rows, int keys, float* __restrict__ out) {
    const int64_t n = (int64_t)rows * keys;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = (float)(i / keys) - keyTimes[i % keys];
}
__global__ void add_type_embedding_kernel(float* __restrict__ hidden, const float* __restrict__ typeEmb, const int32_t* __restrict__ idx,
                                          int rows, int E) {
    const int64_t n = (int64_t)rows * E;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        hidden[i] += typeEmb[(size_t)idx[i / E] * E + i % E];
}
// One warp per output row: out[r] = scale * <M[r,:], x> (+ bias[r]).
__global__ void rows_dot_kernel(const float* __restrict__ M, int rows, int cols, const float* __restrict__ x, const float* __restrict__ bias,
                                float scale, float* __restrict__ out) {
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= rows) return;
    float acc = 0.f;
    for (int c = lane; c < cols; c += 32) acc = fmaf(M[(size_t)r * cols + c], x[c], acc);
    acc = warp_sum(acc);
    if (lane == 0) out[r] = acc * scale + (bias ? bias[r] : 0.f);
}
__global__ void sigmoid_kernel(float* __restrict__ x, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) x[i] = stable_sigmoid(x[i]);
}
__global__ void zero_columns_kernel(float* __restrict__ x, int rows, int cols, int count) {
    const int64_t n = (int64_t)rows * count;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        x[(i / count) * cols + i % count] = 0.f;
}
__global__ void update_clamped_kernel(float* __restrict__ w, const float* __restrict__ g, int64_t n, float lr, float lo, float hi) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    {
        const float v = w[i] - lr * g[i];
        w[i] = v < lo ? lo : (v > hi ? hi : v);  // a NaN stays a NaN, as with Math.Clamp
    }
}
// Soft-max of one vector, one block (AccelerationCPU.cs:3700-3746): a non-positive sum leaves the exponentials as they are.
__global__ void __launch_bounds__(256) softmax_vector_kernel(const float* __restrict__ x, int n, float* __restrict__ out) {
    __shared__ float red[32];
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < n; i += 256) mx = fmaxf(mx, x[i]);
    mx = block_max(mx, red);
    float sum = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) {
        const float e = expf(x[i] - mx);
        out[i] = e;
        sum += e;
    }
    sum = block_sum(sum, red);
    if (!(sum > 0.f)) return;
    const float inv = 1.f / sum;
    for (int i = threadIdx.x; i < n; i += 256) out[i] *= inv;
}
// Rank-one accumulation G[d, g] += a[d] * b[g], biasGrad[d] += a[d] (AccelerationCPU.cs:4296-4319).
__global__ void outer_accumulate_kernel(const float* __restrict__ a, const float* __restrict__ b, int rows, int cols, float* __restrict__ G,
                                        float* __restrict__ biasGrad) {
    const int64_t n = (int64_t)rows * cols;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int d = (int)(i / cols), g = (int)(i % cols);
        G[i] = fmaf(a[d], b[g], G[i]);
        if (g == 0) biasGrad[d] += a[d];
    }
}
__global__ void broadcast_row_kernel(const float* __restrict__ row, int rows, int cols, float scale, float* __restrict__ out) {
    const int64_t n = (int64_t)rows * cols;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) out[i] = row[i % cols] * scale;
}

inline int blocks_for(int64_t n) { return (int)std::min<int64_t>((n + 255) / 256, 148 * 16); }

}  // namespace

extern "C" {

// IAccelerationManager.cs:263 / AccelerationCPU.cs:3076-3270.  decayBias is [queryLen, keyLen, numHeads] or null;
// attentionWeights / scoresPreSoftmax are [numHeads, queryLen, keyLen] or null (needBackwardCache = false).
int32_t b200_ContentAwareCrossAttentionForward(b200_ctx* ctx, const float* Q, int32_t queryLen, const float* K, const float* V, int32_t keyLen,
                                               int32_t embDim, int32_t numHeads, float scale, const float* decayBias, float* output,
                                               float* attentionWeights, float* scoresPreSoftmax) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, Q); NOTNULL(ctx, K); NOTNULL(ctx, V); NOTNULL(ctx, output);
    NEED(ctx, queryLen >= 0 && keyLen >= 0 && embDim > 0, B200_ERR_INVALID_ARG, "negative length");
    NEED(ctx, numHeads > 0 && numHeads <= 65535 && embDim % numHeads == 0, B200_ERR_INVALID_ARG, "embedding dimension %d is not divisible by %d heads", embDim, numHeads);
    if (queryLen == 0) return B200_OK;
    const int64_t nq = (int64_t)queryLen * embDim, nk = (int64_t)keyLen * embDim, nw = (int64_t)numHeads * queryLen * keyLen;
    if (keyLen == 0) {  // no keys: every row is an empty soft-max
        std::fill(output, output + nq, 0.f);
        return B200_OK;
    }
    Scope s(ctx);
    float *dQ = s.up(Q, nq), *dK = s.up(K, nk), *dV = s.up(V, nk), *dB = decayBias ? s.up(decayBias, nw) : nullptr;
    float *dO = s.floats(nq), *dW = s.floats(nw), *dS = s.floats(nw);
    CHECK_SCOPE(s);
    decay_attn_fwd_kernel<<<dim3(queryLen, numHeads), ATT_THREADS, sizeof(float) * (embDim / numHeads), ctx->stream>>>(
        dQ, dK, dV, dB, queryLen, keyLen, embDim, numHeads, scale, dO, dW, dS);
    B200_LAUNCH_CHECK(ctx);
    B200_TRY(s.down(output, dO, nq));
    if (attentionWeights) B200_TRY(s.down(attentionWeights, dW, nw));
    if (scoresPreSoftmax) B200_TRY(s.down(scoresPreSoftmax, dS, nw));
    return s.sync();
}

// IAccelerationManager.cs:287 / AccelerationCPU.cs:3748-3857.  attentionWeights is [numHeads, queryLen, keyLen];
// dDecayBias is [queryLen, keyLen, numHeads] or null (the reference returns null when it is given no time differences).
// scale is 1/sqrt(headDim), as in the reference.
int32_t b200_BackpropTimeDecayedAttention(b200_ctx* ctx, const float* q, int32_t queryLen, const float* k, const float* v, int32_t keyLen,
                                          const float* dOutput, const float* attentionWeights, int32_t embeddingDim, int32_t numHeads,
                                          float* dQ, float* dK, float* dV, float* dDecayBias) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, q); NOTNULL(ctx, k); NOTNULL(ctx, v); NOTNULL(ctx, dOutput); NOTNULL(ctx, attentionWeights);
    NOTNULL(ctx, dQ); NOTNULL(ctx, dK); NOTNULL(ctx, dV);
    NEED(ctx, queryLen >= 0 && keyLen >= 0 && embeddingDim > 0, B200_ERR_INVALID_ARG, "negative length");
    NEED(ctx, numHeads > 0 && numHeads <= 65535 && embeddingDim % numHeads == 0, B200_ERR_INVALID_ARG, "embedding dimension %d is not divisible by %d heads", embeddingDim, numHeads);
    const int64_t nq = (int64_t)queryLen * embeddingDim, nk = (int64_t)keyLen * embeddingDim, nw = (int64_t)numHeads * queryLen * keyLen;
    std::fill(dQ, dQ + nq, 0.f); std::fill(dK, dK + nk, 0.f); std::fill(dV, dV + nk, 0.f);
    if (queryLen == 0 || keyLen == 0) return B200_OK;
    const int hd = embeddingDim / numHeads;
    const float scale = 1.0f / sqrtf((float)hd);
    Scope s(ctx);
    float *gQ = s.up(q, nq), *gK = s.up(k, nk), *gV = s.up(v, nk), *gdO = s.up(dOutput, nq), *gW = s.up(attentionWeights, nw);
    float *gdS = s.floats(nw), *gdQ = s.floats(nq), *gdK = s.floats(nk), *gdV = s.floats(nk), *gdB = dDecayBias ? s.floats(nw) : nullptr;
    CHECK_SCOPE(s);
    decay_attn_bwd_rows_kernel<<<dim3(queryLen, numHeads), ATT_THREADS, sizeof(float) * hd, ctx->stream>>>(
        gK, gV, gdO, gW, queryLen, keyLen, embeddingDim, numHeads, scale, gdS, gdQ, gdB);
    B200_LAUNCH_CHECK(ctx);
    decay_attn_bwd_keys_kernel<<<dim3(keyLen, numHeads), ATT_THREADS, 0, ctx->stream>>>(gQ, gdO, gW, gdS, queryLen, keyLen, embeddingDim, numHeads,
                                                                                      scale, gdK, gdV);
    B200_LAUNCH_CHECK(ctx);
    B200_TRY(s.down(dQ, gdQ, nq));
    B200_TRY(s.down(dK, gdK, nk));
    B200_TRY(s.down(dV, gdV, nk));
    if (dDecayBias) B200_TRY(s.down(dDecayBias, gdB, nw));
    return s.sync();
}

// IAccelerationManager.cs:253 / AccelerationCPU.cs:2596-2644.
int32_t b200_ApplyContextTypeEmbedding(b200_ctx* ctx, float* contextHidden, int32_t rows, int32_t embDim, const float* typeEmbedding,
                                       int32_t typeCount, const int32_t* typeIndices) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, contextHidden); NOTNULL(ctx, typeEmbedding); NOTNULL(ctx, typeIndices);
    NEED(ctx, rows >= 0 && embDim >= 0 && typeCount >= 0, B200_ERR_INVALID_ARG, "negative dimension");
    for (int i = 0; i < rows; i++)
        NEED(ctx, (uint32_t)typeIndices[i] < (uint32_t)typeCount, B200_ERR_OUT_OF_RANGE, "Invalid context type index %d at row %d.", typeIndices[i], i);
    const int64_t n = (int64_t)rows * embDim;
    if (n == 0) return B200_OK;
    Scope s(ctx);
    float *dH = s.up(contextHidden, n), *dT = s.up(typeEmbedding, (int64_t)typeCount * embDim);
    int32_t* dI = s.upi(typeIndices, rows);
    CHECK_SCOPE(s);
    add_type_embedding_kernel<<<blocks_for(n), 256, 0, ctx->stream>>>(dH, dT, dI, rows, embDim);
    B200_LAUNCH_CHECK(ctx);
    B200_TRY(s.down(contextHidden, dH, n));
    return s.sync();
}

// IAccelerationManager.cs:255 / AccelerationCPU.cs:2646-2674: out[p, s] = p - keyArrivalTimes[s].
int32_t b200_ComputeTimeDiffMatrix(b200_ctx* ctx, int32_t priceSeqLen, const float* keyArrivalTimes, int32_t numKeys, float* out) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NEED(ctx, priceSeqLen > 0, B200_ERR_OUT_OF_RANGE, "priceSeqLen must be positive.");
    NOTNULL(ctx, keyArrivalTimes);
    NEED(ctx, numKeys >= 0, B200_ERR_INVALID_ARG, "negative key count");
    if (numKeys == 0) return B200_OK;
    NOTNULL(ctx, out);
    const int64_t n = (int64_t)priceSeqLen * numKeys;
    Scope s(ctx);
    float *dT = s.up(keyArrivalTimes, numKeys), *dO = s.floats(n);
    CHECK_SCOPE(s);
    time_diff_kernel<<<blocks_for(n), 256, 0, ctx->stream>>>(dT, priceSeqLen, numKeys, dO);
    B200_LAUNCH_CHECK(ctx);
    B200_TRY(s.down(out, dO, n));
    return s.sync();
}

// IAccelerationManager.cs:257 / AccelerationCPU.cs:2676-2692: scores[s] = <priceHidden[lastPos], contextHidden[s]> * scale.
int32_t b200_ComputeMemoryAttentionScores(b200_ctx* ctx, const float* priceHidden, int32_t priceRows, int32_t embDim, int32_t lastPos,
                                          const float* contextHidden, int32_t totalCtx, float scale, float* scores) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, priceHidden); NOTNULL(ctx, contextHidden);
    NEED(ctx, embDim >= 0 && totalCtx >= 0, B200_ERR_INVALID_ARG, "negative dimension");
    NEED(ctx, lastPos >= 0 && lastPos < priceRows, B200_ERR_OUT_OF_RANGE, "lastPos %d outside the %d price rows", lastPos, priceRows);
    if (totalCtx == 0) return B200_OK;
    NOTNULL(ctx, scores);
    Scope s(ctx);
    float *dP = s.up(priceHidden + (size_t)lastPos * embDim, embDim), *dC = s.up(contextHidden, (int64_t)totalCtx * embDim), *dO = s.floats(totalCtx);
    CHECK_SCOPE(s);
    rows_dot_kernel<<<(totalCtx + 7) / 8, 256, 0, ctx->stream>>>(dC, totalCtx, embDim, dP, nullptr, scale, dO);
    B200_LAUNCH_CHECK(ctx);
    B200_TRY(s.down(scores, dO, totalCtx));
    return s.sync();
}

// IAccelerationManager.cs:273 / AccelerationCPU.cs:3424-3461: out[d] = bias[d] + <projection[d,:], globalFeatures>.
int32_t b200_ProjectGlobalFeatures(b200_ctx* ctx, const float* globalFeatures, int32_t featureDim, const float* projection, const float* bias,
                                   int32_t embDim, float* out) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, globalFeatures); NOTNULL(ctx, projection); NOTNULL(ctx, bias);
    NEED(ctx, featureDim >= 0 && embDim >= 0, B200_ERR_INVALID_ARG, "negative dimension");
    if (embDim == 0) return B200_OK;
    NOTNULL(ctx, out);
    Scope s(ctx);
    float *dG = s.up(globalFeatures, featureDim), *dP = s.up(projection, (int64_t)embDim * featureDim), *dB = s.up(bias, embDim), *dO = s.floats(embDim);
    CHECK_SCOPE(s);
    rows_dot_kernel<<<(embDim + 7) / 8, 256, 0, ctx->stream>>>(dP, embDim, featureDim, dG, dB, 1.0f, dO);
    B200_LAUNCH_CHECK(ctx);
    B200_TRY(s.down(out, dO, embDim));
    return s.sync();
}

// IAccelerationManager.cs:279 / AccelerationCPU.cs:3517-3552: column means (zeros for an empty matrix).
int32_t b200_MeanPoolRows(b200_ctx* ctx, const float* matrix, int32_t rows, int32_t cols, float* out) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, matrix);
    NEED(ctx, rows >= 0 && cols >= 0, B200_ERR_INVALID_ARG, "negative dimension");
    if (cols == 0) return B200_OK;
    NOTNULL(ctx, out);
    std::fill(out, out + cols, 0.f);
    if (rows == 0) return B200_OK;
    Scope s(ctx);
    float *dM = s.up(matrix, (int64_t)rows * cols), *dO = s.floats(cols);
    CHECK_SCOPE(s);
    B200_TRY(k_colsum(ctx, dM, rows, cols, cols, dO, 0));
    B200_TRY(k_scale_inplace(ctx, dO, cols, 1.0f / (float)rows));
    B200_TRY(s.down(out, dO, cols));
    return s.sync();
}

// IAccelerationManager.cs:285 / AccelerationCPU.cs:3700-3746.
int32_t b200_SoftmaxVector(b200_ctx* ctx, const float* scores, int32_t n, float* out) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, scores);
    NEED(ctx, n >= 0, B200_ERR_INVALID_ARG, "negative length");
    if (n == 0) return B200_OK;
    NOTNULL(ctx, out);
    Scope s(ctx);
    float *dX = s.up(scores, n), *dO = s.floats(n);
    CHECK_SCOPE(s);
    softmax_vector_kernel<<<1, 256, 0, ctx->stream>>>(dX, n, dO);
    B200_LAUNCH_CHECK(ctx);
    B200_TRY(s.down(out, dO, n));
    return s.sync();
}

// IAccelerationManager.cs:324 / AccelerationCPU.cs:4985-4992.
int32_t b200_SigmoidInPlace(b200_ctx* ctx, float* matrix, int64_t count) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, matrix);
    NEED(ctx, count >= 0, B200_ERR_INVALID_ARG, "negative count");
    if (count == 0) return B200_OK;
    Scope s(ctx);
    float* dM = s.up(matrix, count);
    CHECK_SCOPE(s);
    sigmoid_kernel<<<blocks_for(count), 256, 0, ctx->stream>>>(dM, count);
    B200_LAUNCH_CHECK(ctx);
    B200_TRY(s.down(matrix, dM, count));
    return s.sync();
}

// IAccelerationManager.cs:327 / AccelerationCPU.cs:5016-5035: clears the first min(columnCount, cols) columns of every row.
int32_t b200_ZeroMatrixColumns(b200_ctx* ctx, float* matrix, int32_t rows, int32_t cols, int32_t columnCount) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, matrix);
    NEED(ctx, rows >= 0 && cols >= 0, B200_ERR_INVALID_ARG, "negative dimension");
    const int count = std::min(columnCount, cols);
    if (count <= 0 || rows == 0) return B200_OK;
    const int64_t n = (int64_t)rows * cols;
    Scope s(ctx);
    float* dM = s.up(matrix, n);
    CHECK_SCOPE(s);
    zero_columns_kernel<<<blocks_for((int64_t)rows * count), 256, 0, ctx->stream>>>(dM, rows, cols, count);
    B200_LAUNCH_CHECK(ctx);
    B200_TRY(s.down(matrix, dM, n));
    return s.sync();
}

// IAccelerationManager.cs:337 / AccelerationCPU.cs:5037-5056: w = clamp(w - lr * g, minValue, maxValue).
int32_t b200_VectorUpdateClamped(b200_ctx* ctx, float* weights, const float* gradients, int64_t count, float learningRate, float minValue,
                                 float maxValue) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, weights); NOTNULL(ctx, gradients);
    NEED(ctx, count >= 0, B200_ERR_INVALID_ARG, "negative count");
    NEED(ctx, !(minValue > maxValue), B200_ERR_INVALID_ARG, "'%g' cannot be greater than %g.", minValue, maxValue);
    if (count == 0) return B200_OK;
    Scope s(ctx);
    float *dW = s.up(weights, count), *dG = s.up(gradients, count);
    CHECK_SCOPE(s);
    update_clamped_kernel<<<blocks_for(count), 256, 0, ctx->stream>>>(dW, dG, count, learningRate, minValue, maxValue);
    B200_LAUNCH_CHECK(ctx);
    B200_TRY(s.down(weights, dW, count));
    return s.sync();
}

// IAccelerationManager.cs:358 / AccelerationCPU.cs:4296-4319: biasGrad += dGlobalHidden, projectionGrad += dGlobalHidden (x) globalFeatures.
int32_t b200_AccumulateGlobalProjectionGradients(b200_ctx* ctx, const float* dGlobalHidden, int32_t embDim, const float* globalFeatures,
                                                 int32_t featureDim, float* projectionGrad, float* biasGrad) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    if (!dGlobalHidden || !globalFeatures || !projectionGrad || !biasGrad) return B200_OK;  // the reference returns silently
    NEED(ctx, embDim >= 0 && featureDim >= 0, B200_ERR_INVALID_ARG, "negative dimension");
    if (embDim == 0) return B200_OK;
    if (featureDim == 0) {
        for (int d = 0; d < embDim; d++) biasGrad[d] += dGlobalHidden[d];
        return B200_OK;
    }
    const int64_t n = (int64_t)embDim * featureDim;
    Scope s(ctx);
    float *dA = s.up(dGlobalHidden, embDim), *dB = s.up(globalFeatures, featureDim), *dG = s.up(projectionGrad, n), *dBg = s.up(biasGrad, embDim);
    CHECK_SCOPE(s);
    outer_accumulate_kernel<<<blocks_for(n), 256, 0, ctx->stream>>>(dA, dB, embDim, featureDim, dG, dBg);
    B200_LAUNCH_CHECK(ctx);
    B200_TRY(s.down(projectionGrad, dG, n));
    B200_TRY(s.down(biasGrad, dBg, embDim));
    return s.sync();
}

// IAccelerationManager.cs:360 / AccelerationCPU.cs:4321-4359: rowCount copies of pooledGradient[rowIndex, 0:embeddingDim] / rowCount.
int32_t b200_ExpandMeanPoolGradient(b200_ctx* ctx, const float* pooledGradient, int32_t pooledRows, int32_t pooledCols, int32_t rowIndex,
                                    int32_t rowCount, int32_t embeddingDim, float* out) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, pooledGradient);
    if (rowCount <= 0) return B200_OK;
    NEED(ctx, rowIndex >= 0 && rowIndex < pooledRows, B200_ERR_OUT_OF_RANGE, "rowIndex %d outside the %d pooled rows", rowIndex, pooledRows);
    NEED(ctx, embeddingDim >= 0 && embeddingDim <= pooledCols, B200_ERR_OUT_OF_RANGE, "embeddingDim %d exceeds the %d pooled columns", embeddingDim, pooledCols);
    if (embeddingDim == 0) return B200_OK;
    NOTNULL(ctx, out);
    const int64_t n = (int64_t)rowCount * embeddingDim;
    Scope s(ctx);
    float *dR = s.up(pooledGradient + (size_t)rowIndex * pooledCols, embeddingDim), *dO = s.floats(n);
    CHECK_SCOPE(s);
    broadcast_row_kernel<<<blocks_for(n), 256, 0, ctx->stream>>>(dR, rowCount, embeddingDim, 1.0f / (float)rowCount, dO);
    B200_LAUNCH_CHECK(ctx);
    B200_TRY(s.down(out, dO, n));
    return s.sync();
}

// IAccelerationManager.cs:267-269, 333-335: the rank-3 forms are the flat element-wise operations on d0*d1*d2 values.
int32_t b200_Matrix3DScaleInPlace(b200_ctx* ctx, float* matrix, int64_t count, float scale) { return b200_MatrixScaleInPlace(ctx, matrix, count, scale); }
int32_t b200_MatrixSquaredNorm3D(b200_ctx* ctx, const float* matrix, int64_t count, float* out) { return b200_MatrixSquaredNorm(ctx, matrix, count, out); }
int32_t b200_Matrix3DAddInPlace(b200_ctx* ctx, float* target, const float* addend, int64_t count) { return b200_MatrixAddInPlace(ctx, target, addend, count); }
int32_t b200_Matrix3DUpdate(b200_ctx* ctx, float* weights, const float* gradients, int64_t count, float learningRate) {
    return b200_MatrixUpdate(ctx, weights, gradients, count, learningRate);
}

}  // extern "C"
