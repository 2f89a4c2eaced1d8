// C ABI, part A: context management and the per-op entry points that mirror IAccelerationManager one to one.
// Every function validates its arguments on the host (the reference's null / shape / range checks, mapped to status
// codes), stages host arrays into a grow-only device pool, runs the same kernels the resident trainer uses, copies
// the results back and synchronises before returning.
#include <algorithm>
#include <cstring>

#include "api_scope.cuh"


extern "C" {

int32_t b200_create(int32_t device, b200_ctx** out) {
    if (!out) return B200_ERR_INVALID_ARG;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) return B200_ERR_CUDA;  // no CPU fallback exists
    if (device < 0 || device >= count) return B200_ERR_OUT_OF_RANGE;
    if (cudaSetDevice(device) != cudaSuccess) return B200_ERR_CUDA;
    b200_ctx* c = new b200_ctx();
    c->device = device;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { delete c; return B200_ERR_CUDA; }
    c->cc_major = prop.major;
    c->sm_count = prop.multiProcessorCount;
    c->clock_khz = prop.clockRate;
    if (cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking) != cudaSuccess) { delete c; return B200_ERR_CUDA; }
    c->stream = c->own_stream;
    if (cudaMallocHost((void**)&c->pinned, 4096) != cudaSuccess) { cudaStreamDestroy(c->own_stream); delete c; return B200_ERR_CUDA; }
    *out = c;
    return B200_OK;
}

int32_t b200_destroy(b200_ctx* ctx) {
    if (ctx) ctx_release(ctx);
    return B200_OK;
}

}  // extern "C"

void b200::ctx_release(b200_ctx* ctx) {
    if (ctx->refs.fetch_sub(1) != 1) return;  // a trainer or session still uses it: the last of them frees it
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->pool) cudaFree(ctx->pool);
    if (ctx->ws) cudaFree(ctx->ws);
    if (ctx->pinned) cudaFreeHost(ctx->pinned);
    if (ctx->status_host) cudaFreeHost(ctx->status_host);
    for (auto& kv : ctx->rope)
        if (kv.second.dev) cudaFree(kv.second.dev);
    for (float* old : ctx->rope_retired) cudaFree(old);
    for (cudaEvent_t e : ctx->prof_events) cudaEventDestroy(e);
    if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
    delete ctx;
}

extern "C" {

const char* b200_last_error(b200_ctx* ctx) { return ctx ? ctx->err.c_str() : "null context"; }

int32_t b200_set_stream(b200_ctx* ctx, void* s) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    cudaStreamSynchronize(ctx->stream);
    ctx->stream = s ? (cudaStream_t)s : ctx->own_stream;
    return B200_OK;
}
int32_t b200_set_gemm_mode(b200_ctx* ctx, int32_t mode) {
    if (!ctx || mode < 0 || mode > 2) return B200_ERR_INVALID_ARG;
    ctx->gemm_mode = mode;
    return B200_OK;
}
int32_t b200_synchronize(b200_ctx* ctx) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return check_device_status(ctx);
}
int64_t b200_kernel_launches(b200_ctx* ctx) { return ctx ? ctx->launches : 0; }
int32_t b200_engine_launches(b200_ctx* ctx, int64_t* out) {
    if (!ctx || !out) return B200_ERR_INVALID_ARG;
    for (int i = 0; i < B200_ENGINE_COUNT; i++) out[i] = ctx->engine_launches[i];
    return B200_OK;
}
int32_t b200_set_gemm_kernel(b200_ctx* ctx, int32_t kernel) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    if (kernel != 0 && kernel != 1 && kernel != 128 && kernel != 256 && kernel != 512) return fail(ctx, B200_ERR_INVALID_ARG, "gemm kernel must be 0, 1, 128, 256 or 512");
    ctx->gemm_tile_n = kernel;
    return B200_OK;
}
int32_t b200_set_wait_budget_us(b200_ctx* ctx, int64_t microseconds) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    if (microseconds <= 0 || microseconds > 60ll * 1000 * 1000) return fail(ctx, B200_ERR_OUT_OF_RANGE, "wait budget must be within (0, 60 s]");
    std::lock_guard<std::mutex> lock(ctx->mu);
    B200_CUDA(ctx, cudaSetDevice(ctx->device));
    B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    const long long clocks = (long long)((double)microseconds * (double)(ctx->clock_khz > 0 ? ctx->clock_khz : 2000000) / 1000.0);
    B200_TRY(gemm_tcgen05_set_wait_budget(ctx, clocks));
    return attn_umma_set_wait_budget(ctx, clocks);
}
int32_t b200_probe_wait_timeout(b200_ctx* ctx) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    std::lock_guard<std::mutex> lock(ctx->mu);
    B200_CUDA(ctx, cudaSetDevice(ctx->device));
    return gemm_tcgen05_probe_wait(ctx);
}
int32_t b200_has_tcgen05(b200_ctx* ctx) { return ctx && ctx->cc_major == 10 ? 1 : 0; }

int32_t b200_profile_gemm(b200_ctx* ctx, int32_t enable) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->profile = enable ? 1 : 0;
    ctx->prof_used = 0;
    ctx->prof_flops.clear();
    ctx->prof_engine.clear();
    ctx->prof_shape.clear();
    return B200_OK;
}

int64_t b200_gemm_profile_csv(b200_ctx* ctx, char* buf, int64_t cap) {
    if (!ctx || !buf || cap <= 0) return -1;
    std::lock_guard<std::mutex> lock(ctx->mu);
    cudaSetDevice(ctx->device);
    if (cudaStreamSynchronize(ctx->stream) != cudaSuccess) return -1;
    struct Agg { int64_t n = 0; double ms = 0, flops = 0; };
    std::map<std::vector<int>, Agg> agg;
    for (size_t i = 0; i < ctx->prof_flops.size(); i++) {
        float t = 0.f;
        if (cudaEventElapsedTime(&t, ctx->prof_events[2 * i], ctx->prof_events[2 * i + 1]) != cudaSuccess) continue;
        const auto& sh = ctx->prof_shape[i];
        Agg& a = agg[{ctx->prof_engine[i], sh.M, sh.N, sh.K, sh.tA, sh.tB}];
        a.n++; a.ms += t; a.flops += ctx->prof_flops[i];
    }
    std::string out = "engine,M,N,K,transA,transB,launches,total_ms,tflops\n";
    char line[256];
    for (auto& kv : agg) {
        snprintf(line, sizeof(line), "%d,%d,%d,%d,%d,%d,%lld,%.4f,%.2f\n", kv.first[0], kv.first[1], kv.first[2], kv.first[3], kv.first[4], kv.first[5],
                 (long long)kv.second.n, kv.second.ms, kv.second.ms > 0 ? kv.second.flops / (kv.second.ms * 1e-3) / 1e12 : 0.0);
        out += line;
    }
    int64_t n = (int64_t)out.size() < cap - 1 ? (int64_t)out.size() : cap - 1;
    memcpy(buf, out.data(), (size_t)n);
    buf[n] = 0;
    return n;
}

int32_t b200_gemm_profile(b200_ctx* ctx, int32_t engine, int64_t* launches, double* flops, double* ms) {
    if (!ctx || !launches || !flops || !ms) return B200_ERR_INVALID_ARG;
    std::lock_guard<std::mutex> lock(ctx->mu);
    B200_CUDA(ctx, cudaSetDevice(ctx->device));
    B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    *launches = 0; *flops = 0; *ms = 0;
    for (size_t i = 0; i < ctx->prof_flops.size(); i++) {
        if (ctx->prof_engine[i] != engine) continue;
        float t = 0.f;
        B200_CUDA(ctx, cudaEventElapsedTime(&t, ctx->prof_events[2 * i], ctx->prof_events[2 * i + 1]));
        *launches += 1; *flops += ctx->prof_flops[i]; *ms += t;
    }
    return B200_OK;
}

// ------------------------------------------------------------------------------------------------ tensor primitives
int32_t b200_MatrixMultiply(b200_ctx* ctx, const float* A, int32_t rowsA, int32_t colsA, const float* B, int32_t rowsB, int32_t colsB, float* C) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, A); NOTNULL(ctx, B); NOTNULL(ctx, C);
    NEED(ctx, rowsA >= 0 && colsA >= 0 && rowsB >= 0 && colsB >= 0, B200_ERR_INVALID_ARG, "MatrixMultiply: negative dimension");
    NEED(ctx, colsA == rowsB, B200_ERR_SHAPE, "MatrixMultiply: A columns (%d) must equal B rows (%d)", colsA, rowsB);
    if (rowsA == 0 || colsB == 0) return B200_OK;
    Scope s(ctx);
    float *dA = s.up(A, (int64_t)rowsA * colsA), *dB = s.up(B, (int64_t)rowsB * colsB), *dC = s.floats((int64_t)rowsA * colsB);
    CHECK_SCOPE(s);
    Gemm g;
    g.M = rowsA; g.N = colsB; g.K = colsA; g.A = dA; g.lda = colsA; g.B = dB; g.ldb = colsB; g.C = dC; g.ldc = colsB;
    B200_TRY(gemm(ctx, g));
    B200_TRY(s.down(C, dC, (int64_t)rowsA * colsB));
    return s.sync();
}

int32_t b200_MatrixMultiplyTranspose(b200_ctx* ctx, const float* A, int32_t rowsA, int32_t colsA, const float* B, int32_t rowsB, int32_t colsB, float* C) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, A); NOTNULL(ctx, B); NOTNULL(ctx, C);
    NEED(ctx, rowsA >= 0 && colsA >= 0 && rowsB >= 0 && colsB >= 0, B200_ERR_INVALID_ARG, "MatrixMultiplyTranspose: negative dimension");
    NEED(ctx, colsA == colsB, B200_ERR_SHAPE, "MatrixMultiplyTranspose: A columns (%d) must equal B columns (%d)", colsA, colsB);
    if (rowsA == 0 || rowsB == 0) return B200_OK;
    Scope s(ctx);
    float *dA = s.up(A, (int64_t)rowsA * colsA), *dB = s.up(B, (int64_t)rowsB * colsB), *dC = s.floats((int64_t)rowsA * rowsB);
    CHECK_SCOPE(s);
    Gemm g;
    g.M = rowsA; g.N = rowsB; g.K = colsA; g.A = dA; g.lda = colsA; g.B = dB; g.ldb = colsB; g.transB = 1; g.C = dC; g.ldc = rowsB;
    B200_TRY(gemm(ctx, g));
    B200_TRY(s.down(C, dC, (int64_t)rowsA * rowsB));
    return s.sync();
}

int32_t b200_BatchDotProductAddBias(b200_ctx* ctx, const float* W, int32_t outDim, int32_t inDim, const float* X, int32_t xRows, int32_t xCols,
                                    int32_t rowStart, int32_t rowCount, const float* bias, int32_t biasLen, float* Y) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, W); NOTNULL(ctx, X); NOTNULL(ctx, bias); NOTNULL(ctx, Y);
    NEED(ctx, rowStart >= 0 && rowCount >= 0 && (int64_t)rowStart + rowCount <= xRows, B200_ERR_OUT_OF_RANGE,
         "BatchDotProductAddBias: rows [%d,%d) outside the %d input rows", rowStart, rowStart + rowCount, xRows);
    NEED(ctx, xCols == inDim, B200_ERR_SHAPE, "Expected input columns %d, got %d", inDim, xCols);
    NEED(ctx, biasLen == outDim, B200_ERR_SHAPE, "Bias length must match output dimension.");
    if (rowCount == 0 || outDim == 0) return B200_OK;
    Scope s(ctx);
    float* dW = s.up(W, (int64_t)outDim * inDim);
    float* dX = s.up(X + (size_t)rowStart * inDim, (int64_t)rowCount * inDim);
    float* dB = s.up(bias, outDim);
    float* dY = s.floats((int64_t)rowCount * outDim);
    CHECK_SCOPE(s);
    B200_TRY(linear_fwd(ctx, dX, rowCount, inDim, dW, dB, outDim, dY, outDim));
    B200_TRY(s.down(Y, dY, (int64_t)rowCount * outDim));
    return s.sync();
}

int32_t b200_ProjectOutputBatch(b200_ctx* ctx, const float* hidden, int32_t hiddenRows, int32_t embDim, const float* proj, const float* bias,
                                int32_t seqLen, int32_t outputDim, float* pred) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, hidden); NOTNULL(ctx, proj); NOTNULL(ctx, bias); NOTNULL(ctx, pred);
    NEED(ctx, seqLen >= 0 && seqLen <= hiddenRows, B200_ERR_OUT_OF_RANGE, "ProjectOutputBatch: seqLen %d outside the %d hidden rows", seqLen, hiddenRows);
    if (seqLen == 0 || outputDim <= 0) return B200_OK;
    Scope s(ctx);
    float *dH = s.up(hidden, (int64_t)seqLen * embDim), *dW = s.up(proj, (int64_t)outputDim * embDim), *dB = s.up(bias, outputDim);
    float* dY = s.floats((int64_t)seqLen * outputDim);
    CHECK_SCOPE(s);
    B200_TRY(linear_fwd(ctx, dH, seqLen, embDim, dW, dB, outputDim, dY, outputDim));
    B200_TRY(s.down(pred, dY, (int64_t)seqLen * outputDim));
    return s.sync();
}

int32_t b200_MatrixAddInPlace(b200_ctx* ctx, float* target, const float* addend, int64_t count) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, target); NOTNULL(ctx, addend);
    NEED(ctx, count >= 0, B200_ERR_INVALID_ARG, "negative count");
    if (count == 0) return B200_OK;
    Scope s(ctx);
    float *dT = s.up(target, count), *dA = s.up(addend, count);
    CHECK_SCOPE(s);
    B200_TRY(k_add_inplace(ctx, dT, dA, count));
    B200_TRY(s.down(target, dT, count));
    return s.sync();
}
int32_t b200_VectorAccumulate(b200_ctx* ctx, float* target, const float* source, int64_t count) { return b200_MatrixAddInPlace(ctx, target, source, count); }

int32_t b200_ZeroMatrix(b200_ctx* ctx, float* matrix, int64_t count) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, matrix);
    NEED(ctx, count >= 0, B200_ERR_INVALID_ARG, "negative count");
    // The array lives in host memory and the call is defined as "all elements become +0": a device round trip
    // would only copy zeros back, so it is cleared in place.
    memset(matrix, 0, sizeof(float) * (size_t)count);
    return B200_OK;
}
int32_t b200_ZeroVector(b200_ctx* ctx, float* vector, int64_t count) { return b200_ZeroMatrix(ctx, vector, count); }

// ------------------------------------------------------------------------------------------------ layer norm
int32_t b200_ResidualLayerNormForward(b200_ctx* ctx, const float* input, const float* subLayer, const float* gamma, const float* beta, int32_t rows,
                                      int32_t features, float eps, float* output, float* means, float* variances, float* normalized,
                                      float* residual) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, input); NOTNULL(ctx, gamma); NOTNULL(ctx, beta); NOTNULL(ctx, output);
    NEED(ctx, rows >= 0 && features >= 0, B200_ERR_INVALID_ARG, "negative dimension");
    if (rows == 0 || features == 0) return B200_OK;
    int64_t n = (int64_t)rows * features;
    Scope s(ctx);
    float* dX = s.up(input, n);
    float* dS = subLayer ? s.up(subLayer, n) : nullptr;
    float *dG = s.up(gamma, features), *dB = s.up(beta, features);
    float* dO = s.floats(n);
    float *dM = s.floats(rows), *dV = s.floats(rows);
    float* dN = normalized ? s.floats(n) : nullptr;
    float* dR = residual ? s.floats(n) : nullptr;
    CHECK_SCOPE(s);
    B200_TRY(k_ln_forward(ctx, dX, dS, dG, dB, rows, features, eps, dO, dM, dV, dN, dR));
    B200_TRY(s.down(output, dO, n));
    if (means) B200_TRY(s.down(means, dM, rows));
    if (variances) B200_TRY(s.down(variances, dV, rows));
    if (normalized) B200_TRY(s.down(normalized, dN, n));
    if (residual) B200_TRY(s.down(residual, dR, n));
    return s.sync();
}

int32_t b200_LayerNormBackward(b200_ctx* ctx, const float* dOut, const float* normalized, const float* gamma, const float* input, const float* mean,
                               const float* variance, int32_t rows, int32_t features, float eps, float* dInput, float* dGamma, float* dBeta) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, dOut); NOTNULL(ctx, gamma); NOTNULL(ctx, input); NOTNULL(ctx, mean); NOTNULL(ctx, variance);
    NOTNULL(ctx, dInput); NOTNULL(ctx, dGamma); NOTNULL(ctx, dBeta);
    (void)normalized;  // recomputed from input, mean and variance: (x - mean) / sqrt(var + eps), the forward's own expression
    NEED(ctx, rows >= 0 && features >= 0, B200_ERR_INVALID_ARG, "negative dimension");
    if (features == 0) return B200_OK;
    int64_t n = (int64_t)rows * features;
    Scope s(ctx);
    float *dD = s.up(dOut, n), *dX = s.up(input, n), *dG = s.up(gamma, features), *dM = s.up(mean, rows), *dV = s.up(variance, rows);
    float *dI = s.floats(n), *dGg = s.floats(features), *dBg = s.floats(features);
    CHECK_SCOPE(s);
    B200_TRY(k_ln_backward(ctx, dD, nullptr, dX, dG, dM, dV, rows, features, eps, dI, dGg, dBg, 0));
    B200_TRY(s.down(dInput, dI, n));
    B200_TRY(s.down(dGamma, dGg, features));
    B200_TRY(s.down(dBeta, dBg, features));
    return s.sync();
}

// ------------------------------------------------------------------------------------------------ attention
static int attn_common_checks(b200_ctx* ctx, const char* fn, int qLen, int kLen, int embDim, int numHeads) {
    NEED(ctx, numHeads > 0, B200_ERR_OUT_OF_RANGE, "%s: numHeads must be positive", fn);
    NEED(ctx, qLen >= 0 && kLen >= 0 && embDim > 0, B200_ERR_INVALID_ARG, "%s: bad dimensions", fn);
    NEED(ctx, embDim % numHeads == 0, B200_ERR_SHAPE, "%s: embedding dimension must be divisible by numHeads", fn);
    NEED(ctx, embDim / numHeads <= 128, B200_ERR_UNSUPPORTED, "%s: head dimension above 128", fn);
    return B200_OK;
}

static int sdpa_impl(b200_ctx* ctx, const float* q, const float* k, const float* v, int qLen, int kLen, int embDim, int numHeads, float scale,
                     const uint8_t* mask, int causal, float* out) {
    int64_t nq = (int64_t)qLen * embDim, nk = (int64_t)kLen * embDim;
    Scope s(ctx);
    float *dQ = s.up(q, nq), *dK = s.up(k, nk), *dV = s.up(v, nk), *dO = s.floats(nq);
    uint8_t* dM = mask ? s.upb(mask, (int64_t)qLen * kLen) : nullptr;
    AttnSeg seg{0, qLen, 0, kLen};
    AttnSeg* dSeg = (AttnSeg*)s.alloc(sizeof(AttnSeg));
    CHECK_SCOPE(s);
    B200_CUDA(ctx, cudaMemcpyAsync(dSeg, &seg, sizeof(seg), cudaMemcpyHostToDevice, ctx->stream));
    Attn a;
    a.Q = dQ; a.K = dK; a.V = dV; a.ldq = a.ldk = a.ldv = embDim; a.numHeads = numHeads; a.headDim = embDim / numHeads; a.scale = scale;
    a.causal = causal; a.mask = dM; a.segs_dev = dSeg; a.nSeg = 1; a.maxQLen = qLen; a.maxKLen = kLen; a.totalQ = qLen; a.totalK = kLen;
    a.O = dO; a.ldo = embDim;
    B200_TRY(attn_forward(ctx, a));
    B200_TRY(s.down(out, dO, nq));
    B200_TRY(s.sync());  // seg is read by the async copy until here
    return B200_OK;
}

int32_t b200_ScaledDotProductAttention(b200_ctx* ctx, const float* q, const float* k, const float* v, int32_t queryLen, int32_t keyLen, int32_t embDim,
                                       int32_t numHeads, const uint8_t* mask, int32_t causal, float* out) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, q); NOTNULL(ctx, k); NOTNULL(ctx, v); NOTNULL(ctx, out);
    B200_TRY(attn_common_checks(ctx, "ScaledDotProductAttention", queryLen, keyLen, embDim, numHeads));
    NEED(ctx, queryLen > 0, B200_ERR_INVALID_ARG, "Q must contain at least one row.");
    NEED(ctx, keyLen > 0, B200_ERR_INVALID_ARG, "K must contain at least one row.");
    NEED(ctx, !(causal && queryLen != keyLen), B200_ERR_INVALID_ARG,
         "The simple causal path assumes queryLen == keyLen. Use an explicit mask for cross-attention or cached decoding.");
    float scale = 1.0f / sqrtf((float)(embDim / numHeads));
    return sdpa_impl(ctx, q, k, v, queryLen, keyLen, embDim, numHeads, scale, mask, causal ? 1 : 0, out);
}

int32_t b200_MultiHeadAttentionForward(b200_ctx* ctx, const float* q, const float* k, const float* v, int32_t queryLen, int32_t keyLen, int32_t embDim,
                                       int32_t numHeads, float scale, const uint8_t* mask, float* out) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, q); NOTNULL(ctx, k); NOTNULL(ctx, v); NOTNULL(ctx, out);
    B200_TRY(attn_common_checks(ctx, "MultiHeadAttentionForward", queryLen, keyLen, embDim, numHeads));
    if (queryLen == 0) return B200_OK;
    return sdpa_impl(ctx, q, k, v, queryLen, keyLen, embDim, numHeads, scale, mask, 0, out);
}

static int mha_bwd_impl(b200_ctx* ctx, const float* Q, const float* K, const float* V, const float* dO, const std::vector<AttnSeg>& segs,
                        int totalQ, int totalK, int maxQ, int maxK, int embDim, int numHeads, float scale, const uint8_t* mask, int causal,
                        float* dQ, float* dK, float* dV, float* fwdOut) {
    int64_t nq = (int64_t)totalQ * embDim, nk = (int64_t)totalK * embDim;
    Scope s(ctx);
    float *dq = s.up(Q, nq), *dk = s.up(K, nk), *dv = s.up(V, nk);
    float* ddo = dO ? s.up(dO, nq) : nullptr;
    float* dOo = s.floats(nq);
    float *rm = s.floats((int64_t)totalQ * numHeads), *rs = s.floats((int64_t)totalQ * numHeads), *rd = s.floats((int64_t)totalQ * numHeads);
    float *gq = s.floats(nq), *gk = s.floats(nk), *gv = s.floats(nk);
    uint8_t* dM = mask ? s.upb(mask, (int64_t)totalQ * totalK) : nullptr;
    AttnSeg* dSeg = (AttnSeg*)s.alloc(sizeof(AttnSeg) * segs.size());
    CHECK_SCOPE(s);
    B200_CUDA(ctx, cudaMemcpyAsync(dSeg, segs.data(), sizeof(AttnSeg) * segs.size(), cudaMemcpyHostToDevice, ctx->stream));
    Attn a;
    a.Q = dq; a.K = dk; a.V = dv; a.ldq = a.ldk = a.ldv = embDim; a.numHeads = numHeads; a.headDim = embDim / numHeads; a.scale = scale;
    a.causal = causal; a.mask = dM; a.segs_dev = dSeg; a.nSeg = (int)segs.size(); a.maxQLen = maxQ; a.maxKLen = maxK; a.totalQ = totalQ;
    a.totalK = totalK; a.O = dOo; a.ldo = embDim; a.rowMax = rm; a.rowSum = rs; a.rowDot = rd;
    B200_TRY(attn_forward(ctx, a));
    if (fwdOut) B200_TRY(s.down(fwdOut, dOo, nq));
    if (ddo) {
        a.dO = ddo; a.lddo = embDim; a.dQ = gq; a.dK = gk; a.dV = gv; a.lddq = a.lddk = a.lddv = embDim;
        B200_TRY(attn_backward(ctx, a));
        B200_TRY(s.down(dQ, gq, nq));
        B200_TRY(s.down(dK, gk, nk));
        B200_TRY(s.down(dV, gv, nk));
    }
    return s.sync();
}

int32_t b200_MultiHeadAttentionBackward(b200_ctx* ctx, const float* Q, const float* K, const float* V, const float* dConcat, int32_t seqLenQ,
                                        int32_t seqLenK, int32_t embDim, int32_t numHeads, float scale, const uint8_t* mask, int32_t useDecoderMask,
                                        float* dQ, float* dK, float* dV) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, Q); NOTNULL(ctx, K); NOTNULL(ctx, V); NOTNULL(ctx, dConcat); NOTNULL(ctx, dQ); NOTNULL(ctx, dK); NOTNULL(ctx, dV);
    B200_TRY(attn_common_checks(ctx, "MultiHeadAttentionBackward", seqLenQ, seqLenK, embDim, numHeads));
    memset(dQ, 0, sizeof(float) * (size_t)seqLenQ * embDim);
    memset(dK, 0, sizeof(float) * (size_t)seqLenK * embDim);
    memset(dV, 0, sizeof(float) * (size_t)seqLenK * embDim);
    if (seqLenQ == 0 || seqLenK == 0) return B200_OK;
    std::vector<AttnSeg> segs{AttnSeg{0, seqLenQ, 0, seqLenK}};
    return mha_bwd_impl(ctx, Q, K, V, dConcat, segs, seqLenQ, seqLenK, seqLenQ, seqLenK, embDim, numHeads, scale, mask,
                        (!mask && useDecoderMask) ? 1 : 0, dQ, dK, dV, nullptr);
}

static std::vector<AttnSeg> uniform_segs(int segLen, int segCount) {
    std::vector<AttnSeg> v((size_t)segCount);
    for (int i = 0; i < segCount; i++) v[i] = AttnSeg{i * segLen, segLen, i * segLen, segLen};
    return v;
}

int32_t b200_SegmentedAttentionForward(b200_ctx* ctx, const float* Q, const float* K, const float* V, int32_t segLen, int32_t segCount, int32_t embDim,
                                       int32_t numHeads, int32_t causal, float* out) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, Q); NOTNULL(ctx, K); NOTNULL(ctx, V); NOTNULL(ctx, out);
    NEED(ctx, segLen > 0 && segCount > 0, B200_ERR_INVALID_ARG, "Invalid segmented attention shape.");
    NEED(ctx, segCount <= 65535, B200_ERR_UNSUPPORTED, "more than 65535 segments in one call");
    B200_TRY(attn_common_checks(ctx, "SegmentedAttentionForward", segLen, segLen, embDim, numHeads));
    int total = segLen * segCount;
    float scale = 1.0f / sqrtf((float)(embDim / numHeads));
    return mha_bwd_impl(ctx, Q, K, V, nullptr, uniform_segs(segLen, segCount), total, total, segLen, segLen, embDim, numHeads, scale, nullptr,
                        causal ? 1 : 0, nullptr, nullptr, nullptr, out);
}

int32_t b200_SegmentedAttentionBackward(b200_ctx* ctx, const float* Q, const float* K, const float* V, const float* dConcat, int32_t segLen,
                                        int32_t segCount, int32_t embDim, int32_t numHeads, float scale, int32_t causal, float* dQ, float* dK,
                                        float* dV) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, Q); NOTNULL(ctx, K); NOTNULL(ctx, V); NOTNULL(ctx, dConcat); NOTNULL(ctx, dQ); NOTNULL(ctx, dK); NOTNULL(ctx, dV);
    NEED(ctx, segLen > 0 && segCount > 0, B200_ERR_INVALID_ARG, "Invalid segmented attention backward shape.");
    NEED(ctx, segCount <= 65535, B200_ERR_UNSUPPORTED, "more than 65535 segments in one call");
    B200_TRY(attn_common_checks(ctx, "SegmentedAttentionBackward", segLen, segLen, embDim, numHeads));
    int total = segLen * segCount;
    return mha_bwd_impl(ctx, Q, K, V, dConcat, uniform_segs(segLen, segCount), total, total, segLen, segLen, embDim, numHeads, scale, nullptr,
                        causal ? 1 : 0, dQ, dK, dV, nullptr);
}

int32_t b200_ApplyRotaryPositionEmbeddingInPlace(b200_ctx* ctx, float* matrix, int32_t rows, int32_t embDim, int32_t numHeads, float baseTheta,
                                                 int32_t inverse, int32_t segLen) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, matrix);
    NEED(ctx, numHeads > 0, B200_ERR_OUT_OF_RANGE, "numHeads must be positive");
    NEED(ctx, baseTheta > 0.f && std::isfinite(baseTheta), B200_ERR_OUT_OF_RANGE, "baseTheta must be finite and positive");
    NEED(ctx, rows >= 0 && embDim >= 0 && segLen >= 0, B200_ERR_INVALID_ARG, "negative dimension");
    NEED(ctx, embDim % numHeads == 0, B200_ERR_SHAPE, "embedding dimension must be divisible by numHeads");
    int hd = embDim / numHeads;
    NEED(ctx, (hd & 1) == 0, B200_ERR_SHAPE, "head dimension must be even");
    if (rows == 0 || hd == 0) return B200_OK;
    int maxPos = segLen > 0 ? std::min(segLen, rows) : rows;
    const float* table = nullptr;
    std::unique_lock<std::mutex> pre(ctx->mu);
    cudaSetDevice(ctx->device);
    B200_TRY(rope_table(ctx, hd, baseTheta, maxPos, &table));
    pre.unlock();
    Scope s(ctx);
    float* dM = s.up(matrix, (int64_t)rows * embDim);
    int32_t* dPos = nullptr;
    std::vector<int32_t> pos;
    if (segLen > 0) {
        pos.resize((size_t)rows);
        for (int r = 0; r < rows; r++) pos[r] = r % segLen;
        dPos = s.upi(pos.data(), rows);
    }
    CHECK_SCOPE(s);
    B200_TRY(k_rope(ctx, dM, 0, 1, rows, embDim, 0, numHeads, hd, table, dPos, inverse ? 1 : 0));
    B200_TRY(s.down(matrix, dM, (int64_t)rows * embDim));
    return s.sync();
}

int32_t b200_ApplyRotaryPositionEmbeddingHeadInPlace(b200_ctx* ctx, float* matrix, int32_t rows, int32_t embDim, int32_t startCol, int32_t headDim,
                                                     float baseTheta, int32_t inverse) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, matrix);
    NEED(ctx, startCol >= 0 && headDim >= 0, B200_ERR_OUT_OF_RANGE, "startCol and headDim must be non-negative");
    NEED(ctx, (headDim & 1) == 0, B200_ERR_SHAPE, "head dimension must be even");
    NEED(ctx, baseTheta > 0.f && std::isfinite(baseTheta), B200_ERR_OUT_OF_RANGE, "baseTheta must be finite and positive");
    NEED(ctx, startCol + headDim <= embDim, B200_ERR_OUT_OF_RANGE, "head slice exceeds the matrix width");
    if (rows <= 0 || headDim == 0) return B200_OK;
    const float* table = nullptr;
    std::unique_lock<std::mutex> pre(ctx->mu);
    cudaSetDevice(ctx->device);
    B200_TRY(rope_table(ctx, headDim, baseTheta, rows, &table));
    pre.unlock();
    Scope s(ctx);
    float* dM = s.up(matrix, (int64_t)rows * embDim);
    CHECK_SCOPE(s);
    B200_TRY(k_rope(ctx, dM, 0, 1, rows, embDim, startCol, 1, headDim, table, nullptr, inverse ? 1 : 0));
    B200_TRY(s.down(matrix, dM, (int64_t)rows * embDim));
    return s.sync();
}

// ------------------------------------------------------------------------------------------------ projections
// n (2 or 3) projections of the same input with separate weights: staged contiguously so that one [n*out, in] GEMM
// produces them side by side.
static int project_many(b200_ctx* ctx, const float* input, int rows, int inDim, int n, const float* const* Ws, const float* const* Bs, int outDim,
                        float* const* outs) {
    NEED(ctx, rows >= 0 && inDim >= 0 && outDim >= 0, B200_ERR_INVALID_ARG, "negative dimension");
    if (rows == 0 || outDim == 0) return B200_OK;
    int64_t nw = (int64_t)outDim * inDim, ny = (int64_t)rows * outDim;
    Scope s(ctx);
    float* dX = s.up(input, (int64_t)rows * inDim);
    float* dW = s.floats(n * nw);
    float* dB = s.floats(n * (int64_t)outDim);
    float* dY = s.floats(n * ny);
    CHECK_SCOPE(s);
    for (int i = 0; i < n; i++) {
        B200_CUDA(ctx, cudaMemcpyAsync(dW + i * nw, Ws[i], sizeof(float) * nw, cudaMemcpyHostToDevice, ctx->stream));
        B200_CUDA(ctx, cudaMemcpyAsync(dB + i * outDim, Bs[i], sizeof(float) * outDim, cudaMemcpyHostToDevice, ctx->stream));
    }
    B200_TRY(linear_fwd(ctx, dX, rows, inDim, dW, dB, n * outDim, dY, n * outDim));
    for (int i = 0; i < n; i++)
        B200_CUDA(ctx, cudaMemcpy2DAsync(outs[i], sizeof(float) * outDim, dY + i * outDim, sizeof(float) * n * outDim, sizeof(float) * outDim, rows,
                                         cudaMemcpyDeviceToHost, ctx->stream));
    return s.sync();
}

// Backward of project_many: the 2n parameter gradients accumulate, dInput is assigned.
static int backprop_many(b200_ctx* ctx, const float* input, int rows, int inDim, int n, const float* const* Ys, int outDim, const float* const* Ws,
                         float* const* Wg, float* const* Bg, float* dInput) {
    NEED(ctx, rows >= 0 && inDim >= 0 && outDim >= 0, B200_ERR_INVALID_ARG, "negative dimension");
    int64_t nw = (int64_t)outDim * inDim, ny = (int64_t)rows * outDim, nx = (int64_t)rows * inDim;
    if (nx == 0) return B200_OK;
    Scope s(ctx);
    float* dX = s.up(input, nx);
    float *dW = s.floats(n * nw), *dWg = s.floats(n * nw), *dBg = s.floats(n * (int64_t)outDim), *dY = s.floats(n * ny), *dIn = s.floats(nx);
    CHECK_SCOPE(s);
    for (int i = 0; i < n; i++) {
        B200_CUDA(ctx, cudaMemcpyAsync(dW + i * nw, Ws[i], sizeof(float) * nw, cudaMemcpyHostToDevice, ctx->stream));
        B200_CUDA(ctx, cudaMemcpyAsync(dWg + i * nw, Wg[i], sizeof(float) * nw, cudaMemcpyHostToDevice, ctx->stream));
        B200_CUDA(ctx, cudaMemcpyAsync(dBg + i * outDim, Bg[i], sizeof(float) * outDim, cudaMemcpyHostToDevice, ctx->stream));
        B200_CUDA(ctx, cudaMemcpy2DAsync(dY + i * outDim, sizeof(float) * n * outDim, Ys[i], sizeof(float) * outDim, sizeof(float) * outDim, rows,
                                         cudaMemcpyHostToDevice, ctx->stream));
    }
    B200_TRY(wgrad(ctx, dY, n * outDim, dX, inDim, rows, n * outDim, inDim, dWg, dBg));
    B200_TRY(dgrad(ctx, dY, n * outDim, dW, rows, n * outDim, inDim, dIn, 0));
    for (int i = 0; i < n; i++) {
        B200_TRY(s.down(Wg[i], dWg + i * nw, nw));
        B200_TRY(s.down(Bg[i], dBg + i * outDim, outDim));
    }
    B200_TRY(s.down(dInput, dIn, nx));
    return s.sync();
}

int32_t b200_ProjectQKV(b200_ctx* ctx, const float* input, int32_t rows, int32_t inDim, const float* WQ, const float* bQ, const float* WK, const float* bK,
                        const float* WV, const float* bV, int32_t outDim, float* Q, float* K, float* V) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, input); NOTNULL(ctx, WQ); NOTNULL(ctx, WK); NOTNULL(ctx, WV); NOTNULL(ctx, bQ); NOTNULL(ctx, bK); NOTNULL(ctx, bV);
    NOTNULL(ctx, Q); NOTNULL(ctx, K); NOTNULL(ctx, V);
    const float* Ws[3] = {WQ, WK, WV};
    const float* Bs[3] = {bQ, bK, bV};
    float* outs[3] = {Q, K, V};
    return project_many(ctx, input, rows, inDim, 3, Ws, Bs, outDim, outs);
}

int32_t b200_ProjectKV(b200_ctx* ctx, const float* input, int32_t rows, int32_t inDim, const float* WK, const float* bK, const float* WV, const float* bV,
                       int32_t outDim, float* K, float* V) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, input); NOTNULL(ctx, WK); NOTNULL(ctx, WV); NOTNULL(ctx, bK); NOTNULL(ctx, bV); NOTNULL(ctx, K); NOTNULL(ctx, V);
    const float* Ws[2] = {WK, WV};
    const float* Bs[2] = {bK, bV};
    float* outs[2] = {K, V};
    return project_many(ctx, input, rows, inDim, 2, Ws, Bs, outDim, outs);
}

int32_t b200_BackpropQKV(b200_ctx* ctx, const float* input, int32_t rows, int32_t inDim, const float* dQ, const float* dK, const float* dV, int32_t outDim,
                         const float* WQ, const float* WK, const float* WV, float* WQGrad, float* bQGrad, float* WKGrad, float* bKGrad,
                         float* WVGrad, float* bVGrad, float* dInput) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, input); NOTNULL(ctx, dQ); NOTNULL(ctx, dK); NOTNULL(ctx, dV); NOTNULL(ctx, WQ); NOTNULL(ctx, WK); NOTNULL(ctx, WV);
    NOTNULL(ctx, WQGrad); NOTNULL(ctx, bQGrad); NOTNULL(ctx, WKGrad); NOTNULL(ctx, bKGrad); NOTNULL(ctx, WVGrad); NOTNULL(ctx, bVGrad);
    NOTNULL(ctx, dInput);
    const float* Ws[3] = {WQ, WK, WV};
    const float* Ys[3] = {dQ, dK, dV};
    float* Wg[3] = {WQGrad, WKGrad, WVGrad};
    float* Bg[3] = {bQGrad, bKGrad, bVGrad};
    return backprop_many(ctx, input, rows, inDim, 3, Ys, outDim, Ws, Wg, Bg, dInput);
}

int32_t b200_BackpropKV(b200_ctx* ctx, const float* input, int32_t rows, int32_t inDim, const float* dK, const float* dV, int32_t outDim, const float* WK,
                        const float* WV, float* WKGrad, float* bKGrad, float* WVGrad, float* bVGrad, float* dInput) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, input); NOTNULL(ctx, dK); NOTNULL(ctx, dV); NOTNULL(ctx, WK); NOTNULL(ctx, WV);
    NOTNULL(ctx, WKGrad); NOTNULL(ctx, bKGrad); NOTNULL(ctx, WVGrad); NOTNULL(ctx, bVGrad); NOTNULL(ctx, dInput);
    const float* Ws[2] = {WK, WV};
    const float* Ys[2] = {dK, dV};
    float* Wg[2] = {WKGrad, WVGrad};
    float* Bg[2] = {bKGrad, bVGrad};
    return backprop_many(ctx, input, rows, inDim, 2, Ys, outDim, Ws, Wg, Bg, dInput);
}

int32_t b200_BackpropLinearProjection(b200_ctx* ctx, const float* input, const float* dOutput, const float* weights, int32_t seqLen, int32_t inDim,
                                      int32_t outDim, float* weightGrad, float* biasGrad, float* dInput) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, input); NOTNULL(ctx, dOutput); NOTNULL(ctx, weights); NOTNULL(ctx, weightGrad); NOTNULL(ctx, biasGrad); NOTNULL(ctx, dInput);
    NEED(ctx, seqLen >= 0 && inDim >= 0 && outDim >= 0, B200_ERR_INVALID_ARG, "negative dimension");
    int64_t nw = (int64_t)outDim * inDim, ny = (int64_t)seqLen * outDim, nx = (int64_t)seqLen * inDim;
    if (seqLen == 0) return B200_OK;
    Scope s(ctx);
    float *dX = s.up(input, nx), *dY = s.up(dOutput, ny), *dW = s.up(weights, nw), *dWg = s.up(weightGrad, nw), *dBg = s.up(biasGrad, outDim),
          *dIn = s.up(dInput, nx);
    CHECK_SCOPE(s);
    B200_TRY(wgrad(ctx, dY, outDim, dX, inDim, seqLen, outDim, inDim, dWg, dBg));
    B200_TRY(dgrad(ctx, dY, outDim, dW, seqLen, outDim, inDim, dIn, 1));
    B200_TRY(s.down(weightGrad, dWg, nw));
    B200_TRY(s.down(biasGrad, dBg, outDim));
    B200_TRY(s.down(dInput, dIn, nx));
    return s.sync();
}

int32_t b200_BackpropOutputProjection(b200_ctx* ctx, const float* dLogits, const float* input, const float* weights, float* weightGrad, float* biasGrad,
                                      int32_t seqLen, int32_t outputDim, int32_t embDim, float* dX) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, dLogits); NOTNULL(ctx, input); NOTNULL(ctx, weights); NOTNULL(ctx, weightGrad); NOTNULL(ctx, biasGrad); NOTNULL(ctx, dX);
    NEED(ctx, seqLen >= 0 && outputDim >= 0 && embDim >= 0, B200_ERR_INVALID_ARG, "negative dimension");
    int64_t nw = (int64_t)outputDim * embDim, ny = (int64_t)seqLen * outputDim, nx = (int64_t)seqLen * embDim;
    if (seqLen == 0) return B200_OK;
    Scope s(ctx);
    float *dXi = s.up(input, nx), *dY = s.up(dLogits, ny), *dW = s.up(weights, nw), *dWg = s.up(weightGrad, nw), *dBg = s.up(biasGrad, outputDim),
          *dOutX = s.floats(nx);
    CHECK_SCOPE(s);
    B200_TRY(wgrad(ctx, dY, outputDim, dXi, embDim, seqLen, outputDim, embDim, dWg, dBg));
    B200_TRY(dgrad(ctx, dY, outputDim, dW, seqLen, outputDim, embDim, dOutX, 0));
    B200_TRY(s.down(weightGrad, dWg, nw));
    B200_TRY(s.down(biasGrad, dBg, outputDim));
    B200_TRY(s.down(dX, dOutX, nx));
    return s.sync();
}

int32_t b200_BackpropInputProjection(b200_ctx* ctx, const float* dX, int32_t dXRows, int32_t dXCols, const float* continuousInput, int32_t contRows,
                                     int32_t contCols, int32_t inputRowStart, float* weightGrad, float* biasGrad, int32_t seqLen, int32_t embDim,
                                     int32_t inputFeatureDim) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, dX); NOTNULL(ctx, continuousInput); NOTNULL(ctx, weightGrad); NOTNULL(ctx, biasGrad);
    NEED(ctx, inputRowStart >= 0 && seqLen >= 0 && (int64_t)inputRowStart + seqLen <= contRows, B200_ERR_OUT_OF_RANGE,
         "BackpropInputProjection: rows [%d,%d) outside the %d input rows", inputRowStart, inputRowStart + seqLen, contRows);
    NEED(ctx, inputFeatureDim <= contCols && dXRows >= seqLen && dXCols >= embDim, B200_ERR_SHAPE, "BackpropInputProjection: shape mismatch");
    if (seqLen == 0 || embDim <= 0 || inputFeatureDim <= 0) return B200_OK;
    int64_t nw = (int64_t)embDim * inputFeatureDim;
    Scope s(ctx);
    float* dD = s.up(dX, (int64_t)seqLen * dXCols);
    float* dC = s.up(continuousInput + (size_t)inputRowStart * contCols, (int64_t)seqLen * contCols);
    float *dWg = s.up(weightGrad, nw), *dBg = s.up(biasGrad, embDim);
    CHECK_SCOPE(s);
    B200_TRY(wgrad(ctx, dD, dXCols, dC, contCols, seqLen, embDim, inputFeatureDim, dWg, dBg));
    B200_TRY(s.down(weightGrad, dWg, nw));
    B200_TRY(s.down(biasGrad, dBg, embDim));
    return s.sync();
}

int32_t b200_EmbedTokenIds(b200_ctx* ctx, const int32_t* tokenIds, int32_t nIds, int32_t tokenStart, int32_t tokenCount, const float* embedding,
                           int32_t vocab, int32_t embDim, float* out) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, tokenIds);
    if (nIds == 0 || tokenCount == 0) return B200_OK;
    NOTNULL(ctx, embedding); NOTNULL(ctx, out);
    NEED(ctx, tokenStart >= 0 && tokenCount >= 0 && (int64_t)tokenStart + tokenCount <= nIds, B200_ERR_OUT_OF_RANGE,
         "EmbedTokenIds: tokens [%d,%d) outside the %d ids", tokenStart, tokenStart + tokenCount, nIds);
    for (int i = 0; i < tokenCount; i++)
        NEED(ctx, (uint32_t)tokenIds[tokenStart + i] < (uint32_t)vocab, B200_ERR_OUT_OF_RANGE, "Token id %d at position %d is outside [0,%d)",
             tokenIds[tokenStart + i], tokenStart + i, vocab);
    Scope s(ctx);
    int32_t* dI = s.upi(tokenIds + tokenStart, tokenCount);
    float *dE = s.up(embedding, (int64_t)vocab * embDim), *dO = s.floats((int64_t)tokenCount * embDim);
    CHECK_SCOPE(s);
    B200_TRY(k_embed(ctx, dI, tokenCount, dE, embDim, dO));
    B200_TRY(s.down(out, dO, (int64_t)tokenCount * embDim));
    return s.sync();
}

}  // extern "C"

namespace b200 {
// Stable counting sort of rows by token id: seg_id = distinct ids ascending, rows of each id in ascending row order.
void sort_rows_by_id(const int32_t* ids, int n, int vocab, std::vector<int32_t>& seg_id, std::vector<int32_t>& seg_off, std::vector<int32_t>& perm) {
    std::vector<int32_t> count((size_t)vocab + 1, 0);
    for (int i = 0; i < n; i++) count[(size_t)ids[i] + 1]++;
    seg_id.clear();
    seg_off.clear();
    std::vector<int32_t> start((size_t)vocab, 0);
    int32_t run = 0;
    for (int v = 0; v < vocab; v++) {
        start[v] = run;
        if (count[(size_t)v + 1] > 0) {
            seg_id.push_back(v);
            seg_off.push_back(run);
        }
        run += count[(size_t)v + 1];
    }
    seg_off.push_back(run);
    perm.assign((size_t)n, 0);
    for (int i = 0; i < n; i++) perm[(size_t)start[ids[i]]++] = i;
}
}  // namespace b200

extern "C" {

int32_t b200_AccumulateTokenEmbeddingGrad(b200_ctx* ctx, float* embeddingGrad, int32_t vocab, const float* dX, const int32_t* tokenIds, int32_t nIds,
                                          int32_t tokenStart, int32_t seqLen, int32_t embDim) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, embeddingGrad); NOTNULL(ctx, dX); NOTNULL(ctx, tokenIds);
    NEED(ctx, tokenStart >= 0 && seqLen >= 0 && (int64_t)tokenStart + seqLen <= nIds, B200_ERR_OUT_OF_RANGE,
         "AccumulateTokenEmbeddingGrad: tokens [%d,%d) outside the %d ids", tokenStart, tokenStart + seqLen, nIds);
    for (int i = 0; i < seqLen; i++)
        NEED(ctx, (uint32_t)tokenIds[tokenStart + i] < (uint32_t)vocab, B200_ERR_OUT_OF_RANGE, "Token id %d is outside [0,%d)", tokenIds[tokenStart + i], vocab);
    if (seqLen == 0 || embDim <= 0) return B200_OK;
    std::vector<int32_t> seg_id, seg_off, perm;
    sort_rows_by_id(tokenIds + tokenStart, seqLen, vocab, seg_id, seg_off, perm);
    Scope s(ctx);
    float *dE = s.up(embeddingGrad, (int64_t)vocab * embDim), *dD = s.up(dX, (int64_t)seqLen * embDim);
    int32_t *dSid = s.upi(seg_id.data(), (int64_t)seg_id.size()), *dSoff = s.upi(seg_off.data(), (int64_t)seg_off.size()), *dPerm = s.upi(perm.data(), seqLen);
    CHECK_SCOPE(s);
    B200_TRY(k_embed_scatter(ctx, dE, dD, nullptr, dSid, dSoff, dPerm, (int)seg_id.size(), embDim));
    B200_TRY(s.down(embeddingGrad, dE, (int64_t)vocab * embDim));
    return s.sync();
}

// ------------------------------------------------------------------------------------------------ losses
int32_t b200_CrossEntropyLossAndGradient(b200_ctx* ctx, const float* logits, int32_t rows, int32_t outputDim, const int32_t* targets, int32_t nTargets,
                                         int32_t targetStart, int32_t effectiveLen, float* loss, float* dLogits) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, logits); NOTNULL(ctx, targets); NOTNULL(ctx, loss); NOTNULL(ctx, dLogits);
    NEED(ctx, targetStart >= 0 && effectiveLen >= 0 && (int64_t)targetStart + effectiveLen <= nTargets, B200_ERR_OUT_OF_RANGE,
         "CrossEntropyLossAndGradient: targets [%d,%d) outside the %d targets", targetStart, targetStart + effectiveLen, nTargets);
    NEED(ctx, effectiveLen <= rows, B200_ERR_OUT_OF_RANGE, "effectiveLen %d exceeds the %d logit rows", effectiveLen, rows);
    for (int i = 0; i < effectiveLen; i++)
        NEED(ctx, (uint32_t)targets[targetStart + i] < (uint32_t)outputDim, B200_ERR_OUT_OF_RANGE, "target %d outside [0,%d)", targets[targetStart + i], outputDim);
    *loss = 0.f;
    int64_t n = (int64_t)rows * outputDim;
    if (effectiveLen == 0 || n == 0) {
        memset(dLogits, 0, sizeof(float) * (size_t)n);
        return B200_OK;
    }
    Scope s(ctx);
    float* dL = s.up(logits, n);
    int32_t* dT = s.upi(targets + targetStart, effectiveLen);
    float* dRl = s.floats(rows);
    int32_t* dOk = (int32_t*)s.floats(rows);
    CHECK_SCOPE(s);
    B200_TRY(k_cross_entropy(ctx, dL, rows, outputDim, dT, effectiveLen, nullptr, 1.0f / effectiveLen, dL, dRl, dOk));
    B200_TRY(s.down(dLogits, dL, n));
    std::vector<float> rl((size_t)effectiveLen);
    B200_TRY(s.down(rl.data(), dRl, effectiveLen));
    B200_TRY(s.sync());
    float acc = 0.f;  // the reference's serial loop: loss -= log(...), then loss /= effectiveLen
    for (int i = 0; i < effectiveLen; i++) acc += rl[i];
    *loss = acc / effectiveLen;
    return B200_OK;
}

int32_t b200_MSELossAndGradient(b200_ctx* ctx, const float* predictions, int32_t rows, int32_t outputDim, const float* targets, int32_t targetRows,
                                int32_t targetStart, int32_t effectiveLen, float* loss, float* dOutput) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, predictions); NOTNULL(ctx, targets); NOTNULL(ctx, loss); NOTNULL(ctx, dOutput);
    NEED(ctx, targetStart >= 0 && effectiveLen >= 0 && (int64_t)targetStart + effectiveLen <= targetRows, B200_ERR_OUT_OF_RANGE,
         "MSELossAndGradient: targets [%d,%d) outside the %d target rows", targetStart, targetStart + effectiveLen, targetRows);
    NEED(ctx, effectiveLen <= rows, B200_ERR_OUT_OF_RANGE, "effectiveLen %d exceeds the %d prediction rows", effectiveLen, rows);
    *loss = 0.f;
    int64_t n = (int64_t)rows * outputDim;
    if (effectiveLen == 0 || outputDim == 0) {
        memset(dOutput, 0, sizeof(float) * (size_t)n);
        return B200_OK;
    }
    Scope s(ctx);
    float* dP = s.up(predictions, n);
    float* dT = s.up(targets + (size_t)targetStart * outputDim, (int64_t)effectiveLen * outputDim);
    float* dD = s.floats(n);
    float* dRl = s.floats(rows);
    int32_t* dOk = (int32_t*)s.floats(rows);
    CHECK_SCOPE(s);
    float invLen = 1.0f / ((float)effectiveLen * outputDim);
    B200_TRY(k_mse(ctx, dP, rows, outputDim, dT, effectiveLen, nullptr, invLen, dD, dRl, dOk));
    B200_TRY(s.down(dOutput, dD, n));
    std::vector<float> rl((size_t)effectiveLen);
    B200_TRY(s.down(rl.data(), dRl, effectiveLen));
    B200_TRY(s.sync());
    float acc = 0.f;
    for (int i = 0; i < effectiveLen; i++) acc += rl[i];
    *loss = acc / ((float)effectiveLen * outputDim);
    return B200_OK;
}

// ------------------------------------------------------------------------------------------------ step primitives
int32_t b200_MatrixSquaredNorm(b200_ctx* ctx, const float* matrix, int64_t count, float* out) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, matrix); NOTNULL(ctx, out);
    NEED(ctx, count >= 0, B200_ERR_INVALID_ARG, "negative count");
    *out = 0.f;
    if (count == 0) return B200_OK;
    Scope s(ctx);
    float *dM = s.up(matrix, count), *dO = s.floats(1);
    CHECK_SCOPE(s);
    B200_TRY(k_sqnorm(ctx, dM, count, dO));
    B200_TRY(s.down(out, dO, 1));
    return s.sync();
}
int32_t b200_VectorSquaredNorm(b200_ctx* ctx, const float* vector, int64_t count, float* out) { return b200_MatrixSquaredNorm(ctx, vector, count, out); }

int32_t b200_MatrixScaleInPlace(b200_ctx* ctx, float* matrix, int64_t count, float scale) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, matrix);
    NEED(ctx, count >= 0, B200_ERR_INVALID_ARG, "negative count");
    if (count == 0) return B200_OK;
    Scope s(ctx);
    float* dM = s.up(matrix, count);
    CHECK_SCOPE(s);
    B200_TRY(k_scale_inplace(ctx, dM, count, scale));
    B200_TRY(s.down(matrix, dM, count));
    return s.sync();
}
int32_t b200_VectorScaleInPlace(b200_ctx* ctx, float* vector, int64_t count, float scale) { return b200_MatrixScaleInPlace(ctx, vector, count, scale); }

int32_t b200_MatrixUpdate(b200_ctx* ctx, float* weights, const float* gradients, int64_t count, float learningRate) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, weights); NOTNULL(ctx, gradients);
    NEED(ctx, count >= 0, B200_ERR_INVALID_ARG, "negative count");
    if (count == 0) return B200_OK;
    Scope s(ctx);
    float *dW = s.up(weights, count), *dG = s.up(gradients, count);
    CHECK_SCOPE(s);
    B200_TRY(k_sgd_update(ctx, dW, dG, count, learningRate));
    B200_TRY(s.down(weights, dW, count));
    return s.sync();
}
int32_t b200_VectorUpdate(b200_ctx* ctx, float* weights, const float* gradients, int64_t count, float learningRate) {
    return b200_MatrixUpdate(ctx, weights, gradients, count, learningRate);
}

// ------------------------------------------------------------------------------------------------ feed-forward network
static int ffn_checks(b200_ctx* ctx, int nLayers, const int32_t* widths, const int32_t* acts, const float* const* weights, const float* const* biases) {
    NEED(ctx, nLayers >= 2, B200_ERR_INVALID_ARG, "Neural network must have at least input and output layers.");
    NOTNULL(ctx, widths); NOTNULL(ctx, acts); NOTNULL(ctx, weights); NOTNULL(ctx, biases);
    for (int l = 0; l < nLayers; l++) NEED(ctx, widths[l] > 0, B200_ERR_INVALID_ARG, "layer %d has non-positive width", l);
    for (int l = 1; l < nLayers; l++) {
        NEED(ctx, weights[l] && biases[l], B200_ERR_INVALID_ARG, "layer %d weights/biases are null", l);
        NEED(ctx, acts[l] >= 0 && acts[l] <= 5, B200_ERR_INVALID_ARG, "layer %d has an unknown activation", l);
    }
    return B200_OK;
}

int32_t b200_FFNForwardBatch(b200_ctx* ctx, const float* input, int32_t rows, int32_t nLayers, const int32_t* widths, const int32_t* acts,
                             const float* const* weights, const float* const* biases, float* out) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, input); NOTNULL(ctx, out);
    B200_TRY(ffn_checks(ctx, nLayers, widths, acts, weights, biases));
    if (rows <= 0) return B200_OK;
    Scope s(ctx);
    float* cur = s.up(input, (int64_t)rows * widths[0]);
    for (int l = 1; l < nLayers; l++) {
        float *dW = s.up(weights[l], (int64_t)widths[l] * widths[l - 1]), *dB = s.up(biases[l], widths[l]);
        float* nxt = s.floats((int64_t)rows * widths[l]);
        CHECK_SCOPE(s);
        Gemm g;
        g.M = rows; g.N = widths[l]; g.K = widths[l - 1]; g.A = cur; g.lda = widths[l - 1]; g.B = dW; g.ldb = widths[l - 1]; g.transB = 1;
        g.C = nxt; g.ldc = widths[l]; g.bias = dB; g.act = acts[l]; g.act_conv = 0;
        B200_TRY(gemm(ctx, g));
        cur = nxt;
    }
    B200_TRY(s.down(out, cur, (int64_t)rows * widths[nLayers - 1]));
    return s.sync();
}

int32_t b200_FFNInputGradientBatch(b200_ctx* ctx, const float* input, const float* dOutput, int32_t rows, int32_t nLayers, const int32_t* widths,
                                   const int32_t* acts, const float* const* weights, const float* const* biases, float* const* weightGrads,
                                   float* const* biasGrads, float* dInput) {
    if (!ctx) return B200_ERR_INVALID_ARG;
    NOTNULL(ctx, input); NOTNULL(ctx, dOutput); NOTNULL(ctx, dInput);
    B200_TRY(ffn_checks(ctx, nLayers, widths, acts, weights, biases));
    NEED(ctx, (weightGrads == nullptr) == (biasGrads == nullptr), B200_ERR_INVALID_ARG,
         "weightGradients and biasGradients must either both be null or both be supplied.");
    if (rows <= 0) return B200_OK;
    int L = nLayers - 1;
    Scope s(ctx);
    std::vector<float*> act((size_t)nLayers), z((size_t)nLayers), W((size_t)nLayers);
    act[0] = s.up(input, (int64_t)rows * widths[0]);
    for (int l = 1; l <= L; l++) {
        W[l] = s.up(weights[l], (int64_t)widths[l] * widths[l - 1]);
        float* dB = s.up(biases[l], widths[l]);
        z[l] = s.floats((int64_t)rows * widths[l]);
        act[l] = s.floats((int64_t)rows * widths[l]);
        CHECK_SCOPE(s);
        Gemm g;
        g.M = rows; g.N = widths[l]; g.K = widths[l - 1]; g.A = act[l - 1]; g.lda = widths[l - 1]; g.B = W[l]; g.ldb = widths[l - 1]; g.transB = 1;
        g.C = act[l]; g.ldc = widths[l]; g.bias = dB; g.zout = z[l]; g.ldz = widths[l]; g.act = acts[l];
        B200_TRY(gemm(ctx, g));
    }
    // delta_L = dOutput o act'(z_L)   (NeuralNetwork.cs:842-848)
    float* cur = s.up(dOutput, (int64_t)rows * widths[L]);
    CHECK_SCOPE(s);
    B200_TRY(k_mul_act_deriv(ctx, cur, z[L], acts[L], (int64_t)rows * widths[L]));
    for (int l = L; l >= 1; l--) {
        if (weightGrads) {
            NEED(ctx, weightGrads[l] && biasGrads[l], B200_ERR_INVALID_ARG, "Gradient storage must contain one entry per non-input layer.");
            int64_t nw = (int64_t)widths[l] * widths[l - 1];
            float *dWg = s.up(weightGrads[l], nw), *dBg = s.up(biasGrads[l], widths[l]);
            CHECK_SCOPE(s);
            B200_TRY(wgrad(ctx, cur, widths[l], act[l - 1], widths[l - 1], rows, widths[l], widths[l - 1], dWg, dBg));
            B200_TRY(s.down(weightGrads[l], dWg, nw));
            B200_TRY(s.down(biasGrads[l], dBg, widths[l]));
        }
        float* nxt = s.floats((int64_t)rows * widths[l - 1]);
        CHECK_SCOPE(s);
        Gemm g;
        g.M = rows; g.N = widths[l - 1]; g.K = widths[l]; g.A = cur; g.lda = widths[l]; g.B = W[l]; g.ldb = widths[l - 1]; g.C = nxt; g.ldc = widths[l - 1];
        if (l > 1) { g.mulz = z[l - 1]; g.ldmulz = widths[l - 1]; g.mulz_act = acts[l - 1]; }
        B200_TRY(gemm(ctx, g));
        cur = nxt;
    }
    B200_TRY(s.down(dInput, cur, (int64_t)rows * widths[0]));
    return s.sync();
}

}  // extern "C"
