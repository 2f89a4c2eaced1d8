// C ABI, part C: the resident mini-batch trainer of the feed-forward NeuralNetwork (NeuralNetwork.TrainBatch /
// LearnBatch, NeuralNetwork.cs:420-610, with the kernel math of BatchedAccelerationGPU.cs:251-358).  Weights and
// biases stay on the device across batches.  Per batch:
//   forward   A_l = act(A_{l-1} W_l^T + b_l), D_l = act'(.)              one GEMM per layer, activation fused
//   deltas    delta_L = -costDeriv(A_L, Y) o D_L ; delta_l = (delta_{l+1} W_{l+1}) o D_l   derivative fused in the GEMM
//   clip      s = min(1, thr / ||all deltas||_2)                         two-stage deterministic reduction
//   update    W_l -= (lr/B) (s delta_l^T A_{l-1} + lambda W_l)           L2 term and SGD fused in the dW GEMM epilogue
//             b_l -= (lr/B) s sum_i delta_l[i]
// All deltas are formed from the pre-update weights before any layer is updated.
#include <algorithm>

#include "common.h"

using namespace b200;

struct b200_mlp {
    b200_ctx* ctx = nullptr;
    int nLayers = 0, cost = 0, maxB = 0;
    float huber = 1.f, lambda = 0.f, clip = 1.f;
    std::vector<int> widths, acts;
    std::vector<float*> W, B, A, D, delta;
    float *Xraw = nullptr, *Y = nullptr, *mn = nullptr, *mx = nullptr, *sumsq = nullptr, *scaleNorm = nullptr;
    char* block = nullptr;
};

extern "C" {

int32_t b200_mlp_create(b200_ctx* ctx, int32_t nLayers, const int32_t* widths, const int32_t* acts, int32_t cost, float huber_delta, float l2_lambda,
                        float clip_threshold, int32_t max_batch, b200_mlp** out) {
    if (!ctx || !out) return B200_ERR_INVALID_ARG;
    *out = nullptr;
    if (nLayers < 2 || !widths || !acts || max_batch <= 0) return fail(ctx, B200_ERR_INVALID_ARG, "Neural network must have at least input and output layers.");
    if (cost < 0 || cost > 5) return fail(ctx, B200_ERR_INVALID_ARG, "Unsupported cost function type");
    for (int l = 0; l < nLayers; l++)
        if (widths[l] <= 0 || (l > 0 && (acts[l] < 0 || acts[l] > 5))) return fail(ctx, B200_ERR_INVALID_ARG, "bad layer %d", l);
    std::lock_guard<std::mutex> lock(ctx->mu);
    B200_CUDA(ctx, cudaSetDevice(ctx->device));
    b200_mlp* m = new b200_mlp();
    m->ctx = ctx; m->nLayers = nLayers; m->cost = cost; m->maxB = max_batch; m->huber = huber_delta; m->lambda = l2_lambda; m->clip = clip_threshold;
    m->widths.assign(widths, widths + nLayers);
    m->acts.assign(acts, acts + nLayers);
    auto rnd = [](size_t n) { return (n + 63) & ~(size_t)63; };
    size_t Bz = (size_t)max_batch, total = rnd(Bz * widths[0]) * 2 + rnd(Bz * widths[nLayers - 1]) + 2 * rnd((size_t)widths[0]) + 128;
    for (int l = 1; l < nLayers; l++) total += rnd((size_t)widths[l] * widths[l - 1]) + rnd((size_t)widths[l]) + 3 * rnd(Bz * widths[l]);
    cudaError_t e = cudaMalloc((void**)&m->block, total * sizeof(float));
    if (e != cudaSuccess) { delete m; return fail(ctx, B200_ERR_CUDA, "MLP allocation failed: %s", cudaGetErrorString(e)); }
    cudaMemsetAsync(m->block, 0, total * sizeof(float), ctx->stream);
    float* q = (float*)m->block;
    auto take = [&](size_t n) { float* r = q; q += rnd(n); return r; };
    m->W.assign((size_t)nLayers, nullptr); m->B = m->W; m->A = m->W; m->D = m->W; m->delta = m->W;
    m->Xraw = take(Bz * widths[0]); m->A[0] = take(Bz * widths[0]); m->Y = take(Bz * widths[nLayers - 1]);
    m->mn = take((size_t)widths[0]); m->mx = take((size_t)widths[0]); m->sumsq = take(64); m->scaleNorm = take(64);
    for (int l = 1; l < nLayers; l++) {
        m->W[l] = take((size_t)widths[l] * widths[l - 1]); m->B[l] = take((size_t)widths[l]);
        m->A[l] = take(Bz * widths[l]); m->D[l] = take(Bz * widths[l]); m->delta[l] = take(Bz * widths[l]);
    }
    ctx_retain(ctx);
    *out = m;
    return B200_OK;
}

int32_t b200_mlp_destroy(b200_mlp* m) {
    if (!m) return B200_OK;
    cudaSetDevice(m->ctx->device);
    cudaStreamSynchronize(m->ctx->stream);
    if (m->block) cudaFree(m->block);
    b200_ctx* ctx = m->ctx;
    delete m;
    ctx_release(ctx);
    return B200_OK;
}

int32_t b200_mlp_upload_layer(b200_mlp* m, int32_t layer, const float* weights, const float* biases) {
    if (!m) return B200_ERR_INVALID_ARG;
    b200_ctx* ctx = m->ctx;
    if (layer < 1 || layer >= m->nLayers || !weights || !biases) return fail(ctx, B200_ERR_INVALID_ARG, "bad layer index or null array");
    std::lock_guard<std::mutex> lock(ctx->mu);
    B200_CUDA(ctx, cudaSetDevice(ctx->device));
    B200_CUDA(ctx, cudaMemcpyAsync(m->W[layer], weights, sizeof(float) * (size_t)m->widths[layer] * m->widths[layer - 1], cudaMemcpyHostToDevice, ctx->stream));
    B200_CUDA(ctx, cudaMemcpyAsync(m->B[layer], biases, sizeof(float) * (size_t)m->widths[layer], cudaMemcpyHostToDevice, ctx->stream));
    B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return B200_OK;
}

int32_t b200_mlp_download_layer(b200_mlp* m, int32_t layer, float* weights, float* biases) {
    if (!m) return B200_ERR_INVALID_ARG;
    b200_ctx* ctx = m->ctx;
    if (layer < 1 || layer >= m->nLayers || !weights || !biases) return fail(ctx, B200_ERR_INVALID_ARG, "No GPU buffers for layer %d", layer);
    std::lock_guard<std::mutex> lock(ctx->mu);
    B200_CUDA(ctx, cudaSetDevice(ctx->device));
    B200_CUDA(ctx, cudaMemcpyAsync(weights, m->W[layer], sizeof(float) * (size_t)m->widths[layer] * m->widths[layer - 1], cudaMemcpyDeviceToHost, ctx->stream));
    B200_CUDA(ctx, cudaMemcpyAsync(biases, m->B[layer], sizeof(float) * (size_t)m->widths[layer], cudaMemcpyDeviceToHost, ctx->stream));
    B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return B200_OK;
}

int32_t b200_mlp_learn_batch(b200_mlp* m, const float* X, const float* Y, int32_t Bn, float lr, const float* in_min, const float* in_max, float* delta_norm) {
    if (!m) return B200_ERR_INVALID_ARG;
    b200_ctx* ctx = m->ctx;
    if (!X || !Y) return fail(ctx, B200_ERR_INVALID_ARG, "xBatch must be non-empty.");
    if (Bn <= 0 || Bn > m->maxB) return fail(ctx, B200_ERR_OUT_OF_RANGE, "batch size %d outside [1,%d]", Bn, m->maxB);
    if ((in_min == nullptr) != (in_max == nullptr)) return fail(ctx, B200_ERR_INVALID_ARG, "input range needs both min and max");
    std::lock_guard<std::mutex> lock(ctx->mu);
    B200_CUDA(ctx, cudaSetDevice(ctx->device));
    const int L = m->nLayers - 1;
    const std::vector<int>& w = m->widths;
    cudaStream_t st = ctx->stream;
    B200_CUDA(ctx, cudaMemcpyAsync(m->Y, Y, sizeof(float) * (size_t)Bn * w[L], cudaMemcpyHostToDevice, st));
    if (in_min) {
        B200_CUDA(ctx, cudaMemcpyAsync(m->Xraw, X, sizeof(float) * (size_t)Bn * w[0], cudaMemcpyHostToDevice, st));
        B200_CUDA(ctx, cudaMemcpyAsync(m->mn, in_min, sizeof(float) * w[0], cudaMemcpyHostToDevice, st));
        B200_CUDA(ctx, cudaMemcpyAsync(m->mx, in_max, sizeof(float) * w[0], cudaMemcpyHostToDevice, st));
        B200_TRY(k_mlp_scale_inputs(ctx, m->Xraw, Bn, w[0], m->mn, m->mx, m->A[0]));
    } else {
        B200_CUDA(ctx, cudaMemcpyAsync(m->A[0], X, sizeof(float) * (size_t)Bn * w[0], cudaMemcpyHostToDevice, st));
    }
    for (int l = 1; l <= L; l++) {  // NeuralNetwork.cs:522-541 -> BatchedAccelerationGPU.cs:251-290
        Gemm g;
        g.M = Bn; g.N = w[l]; g.K = w[l - 1]; g.A = m->A[l - 1]; g.lda = w[l - 1]; g.B = m->W[l]; g.ldb = w[l - 1]; g.transB = 1;
        g.C = m->A[l]; g.ldc = w[l]; g.bias = m->B[l]; g.act = m->acts[l]; g.act_conv = 1; g.dout = m->D[l]; g.lddo = w[l];
        B200_TRY(gemm(ctx, g));
    }
    B200_TRY(k_mlp_output_delta(ctx, m->A[L], m->D[L], m->Y, (int64_t)Bn * w[L], m->cost, m->huber, m->delta[L]));
    for (int l = L - 1; l >= 1; l--) {  // BatchedAccelerationGPU.cs:324-335
        Gemm g;
        g.M = Bn; g.N = w[l]; g.K = w[l + 1]; g.A = m->delta[l + 1]; g.lda = w[l + 1]; g.B = m->W[l + 1]; g.ldb = w[l]; g.C = m->delta[l]; g.ldc = w[l];
        g.mulmat = m->D[l]; g.ldmul = w[l];
        B200_TRY(gemm(ctx, g));
    }
    for (int l = 1; l <= L; l++) B200_TRY(k_sqnorm(ctx, m->delta[l], (int64_t)Bn * w[l], m->sumsq + (l - 1)));  // NeuralNetwork.cs:571-580
    B200_TRY(k_mlp_clip_scale(ctx, m->sumsq, L, m->clip, m->scaleNorm));
    const float slr = lr / (float)Bn;
    for (int l = L; l >= 1; l--) {  // BatchedAccelerationGPU.cs:209-234, :292-358
        Gemm g;
        g.M = w[l]; g.N = w[l - 1]; g.K = Bn; g.A = m->delta[l]; g.lda = w[l]; g.transA = 1; g.B = m->A[l - 1]; g.ldb = w[l - 1];
        g.C = m->W[l]; g.ldc = w[l - 1]; g.alpha_dev = m->scaleNorm; g.sgd_lr = slr; g.sgd_lambda = m->lambda;
        B200_TRY(gemm(ctx, g));
        B200_TRY(k_bias_update(ctx, m->B[l], m->delta[l], Bn, w[l], slr, m->scaleNorm));
    }
    B200_CUDA(ctx, cudaMemcpyAsync(ctx->pinned, m->scaleNorm, 2 * sizeof(float), cudaMemcpyDeviceToHost, st));
    B200_CUDA(ctx, cudaStreamSynchronize(st));
    B200_TRY(check_device_status(ctx));
    if (delta_norm) *delta_norm = ctx->pinned[1];
    return B200_OK;
}

}  // extern "C"
