/*
 * callaghan_b200.h -- C ABI of libcallaghan_b200.so, the sm_100a (B200) training back end that plugs in behind
 * CallaghanDev.ML's IAccelerationManager (CallaghanDev.ML/AccelerationManagers/IAccelerationManager.cs:13-361).
 *
 * Conventions
 *   - Every entry point returns an int32 status (B200_OK == 0).  b200_last_error() gives the message of the last
 *     failure on that context.  Nothing throws, nothing traps on the device.
 *   - Section A ("per-op") functions mirror one IAccelerationManager method each: all pointers are HOST pointers to
 *     row-major float32 / int32 / uint8 arrays owned by the caller, the call is blocking, and no pointer is retained.
 *     The accumulate-vs-assign behaviour of each output is the reference's (noted per function).
 *   - Section B ("resident") functions keep a model's weights, gradients and activation caches on the device and run
 *     whole train steps; they are what the trainer hooks call.
 *   - A context is thread-compatible: one call at a time per context; different contexts may be used concurrently.
 *   - The library never falls back to the CPU: a missing/unsupported device is an error.
 */
#ifndef CALLAGHAN_B200_H
#define CALLAGHAN_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define B200_API __attribute__((visibility("default")))
#else
#define B200_API
#endif

enum {
    B200_OK = 0,
    B200_ERR_INVALID_ARG = 1,  /* null pointer, non-positive count: ArgumentNullException / ArgumentException */
    B200_ERR_SHAPE = 2,        /* dimension mismatch: ArgumentException */
    B200_ERR_OUT_OF_RANGE = 3, /* row window or token id out of range: ArgumentOutOfRangeException */
    B200_ERR_CUDA = 4,         /* CUDA runtime/driver error */
    B200_ERR_NCCL = 5,         /* the collective library reported an error (or could not be loaded); the communicator is aborted */
    B200_ERR_TIMEOUT = 6,      /* a bounded wait gave up: a device-side wait of a kernel, or a data-parallel peer that did not arrive */
    B200_ERR_NONFINITE = 7,    /* reserved */
    B200_ERR_UNSUPPORTED = 8,  /* e.g. head dimension above 128 */
    B200_ERR_PEER = 9          /* another data-parallel rank failed in this step; the step was discarded on every rank */
};

/* Activation ids = CallaghanDev.ML.Enums.ActivationType; cost ids = CostFunctionType (Neural Network/Enums). */
enum { B200_ACT_NONE = 0, B200_ACT_SIGMOID = 1, B200_ACT_TANH = 2, B200_ACT_RELU = 3, B200_ACT_LEAKYRELU = 4, B200_ACT_SWISH = 5 };
enum { B200_COST_MSE = 0, B200_COST_ZERO_WEIGHTED_MSE = 1, B200_COST_BCE = 2, B200_COST_MAE = 3, B200_COST_CCE = 4, B200_COST_HUBER = 5 };
/* GEMM engine selection (b200_set_gemm_mode): AUTO = TF32 tcgen05 tiles when every dimension >= 128, FP32 SIMT below. */
enum { B200_GEMM_AUTO = 0, B200_GEMM_FP32_SIMT = 1, B200_GEMM_TF32_TCGEN05 = 2 };
enum { B200_OPT_SGD = 0, B200_OPT_ADAM = 1 };

typedef struct b200_ctx b200_ctx;
typedef struct b200_lm b200_lm;
typedef struct b200_mlp b200_mlp;
typedef struct b200_lm_batch b200_lm_batch;

/* ------------------------------------------------------------------------------------------------ context */
/* Replaces the backend construction in AccelerationFactory.Create (AccelerationManagers/AccelerationFactory.cs:31-45)
 * and NeuralNetwork.InitAcceleration (Neural Network/NeuralNetwork.cs:37-58).  device = CUDA ordinal. */
B200_API int32_t b200_create(int32_t device, b200_ctx** out);
/* IAccelerationManager.Dispose (IAccelerationManager.cs:325). */
B200_API int32_t b200_destroy(b200_ctx* ctx);
B200_API const char* b200_last_error(b200_ctx* ctx);
/* Run all work of this context on a caller-owned cudaStream_t (NULL restores the context's own stream). */
B200_API int32_t b200_set_stream(b200_ctx* ctx, void* cuda_stream);
B200_API int32_t b200_set_gemm_mode(b200_ctx* ctx, int32_t mode);
B200_API int32_t b200_synchronize(b200_ctx* ctx);
/* Number of kernels this context has launched so far (launch accounting for benchmarks). */
B200_API int64_t b200_kernel_launches(b200_ctx* ctx);
/* Per-launch GEMM timing for roofline reports: while enabled, a CUDA-event pair brackets every GEMM launch on the
 * context's stream.  b200_gemm_profile sums, for one engine (0 = FP32 SIMT, 1 = TF32 tcgen05), the launches, their
 * algorithmic FLOPs (2*M*N*K) and their device time since the last b200_profile_gemm call. */
B200_API int32_t b200_profile_gemm(b200_ctx* ctx, int32_t enable);
B200_API int32_t b200_gemm_profile(b200_ctx* ctx, int32_t engine, int64_t* launches, double* flops, double* ms);
/* The same data grouped by (engine, M, N, K, transA, transB) as CSV text; returns the number of bytes written. */
B200_API int64_t b200_gemm_profile_csv(b200_ctx* ctx, char* buf, int64_t capacity);
/* 1 if the device is compute capability 10.x (tcgen05 path usable), else 0. */
B200_API int32_t b200_has_tcgen05(b200_ctx* ctx);
/* Launch counts per engine since the context was created, out[B200_ENGINE_COUNT]: lets a caller (and the parity
 * tests) see which kernel family a call really ran on instead of trusting the dispatcher's rules. */
enum {
    B200_ENGINE_GEMM_SIMT = 0,        /* FP32 shared-memory GEMM */
    B200_ENGINE_GEMM_TILE = 1,        /* tcgen05, one 128x128 tile per CTA */
    B200_ENGINE_GEMM_PERSISTENT = 2,  /* tcgen05, one persistent CTA per SM */
    B200_ENGINE_GEMM_PAIR = 3,        /* tcgen05 cta_group::2, two SMs per 256x256 tile */
    B200_ENGINE_ATTN_FP32 = 4,        /* FP32 attention (forward or backward call) */
    B200_ENGINE_ATTN_MMA_SYNC = 5,    /* TF32 mma.sync attention */
    B200_ENGINE_ATTN_TCGEN05 = 6,     /* TF32 tcgen05 attention (head dim 64) */
    B200_ENGINE_CE_FUSED = 7,         /* soft-max cross-entropy fused with the vocabulary projection, per row chunk */
    B200_ENGINE_COUNT = 8
};
B200_API int32_t b200_engine_launches(b200_ctx* ctx, int64_t* out);
/* Forces one tcgen05 GEMM kernel for every qualifying shape of this context: 0 = choose by shape (default), 1 = one
 * tile per CTA, 128 / 256 = one-CTA persistent kernel of that tile width, 512 = two-SM kernel.  For tests and A/B
 * measurements; the reference has no counterpart. */
B200_API int32_t b200_set_gemm_kernel(b200_ctx* ctx, int32_t kernel);
/* Every device-side wait of the tcgen05 kernels (on an mbarrier that a TMA copy, an MMA commit or another warp
 * completes) is bounded: when the budget runs out the kernel raises a status word, unwinds and returns, and the next
 * synchronising call reports B200_ERR_TIMEOUT instead of the process hanging.  The budget is held per device by the
 * library (default 2 s); this call sets it for the context's device, in microseconds.
 * b200_probe_wait_timeout launches one tiny kernel (one warp, no tensor memory, no copy) that waits on a barrier
 * nobody completes, so that the expiry path and its host-side reporting can be exercised without any real failure:
 * it returns B200_ERR_TIMEOUT when the path works, and the context stays usable.  No counterpart in the reference. */
B200_API int32_t b200_set_wait_budget_us(b200_ctx* ctx, int64_t microseconds);
B200_API int32_t b200_probe_wait_timeout(b200_ctx* ctx);

/* ------------------------------------------------------------------------------------------------ A. per-op */
/* IAccelerationManager.MatrixMultiply (IAccelerationManager.cs:20; AccelerationCPU.cs:159-210): C[rowsA,colsB] = A*B. */
B200_API int32_t b200_MatrixMultiply(b200_ctx*, const float* A, int32_t rowsA, int32_t colsA, const float* B, int32_t rowsB, int32_t colsB, float* C);
/* MatrixMultiplyTranspose (IAccelerationManager.cs:26): C[rowsA,rowsB] = A*B^T. */
B200_API int32_t b200_MatrixMultiplyTranspose(b200_ctx*, const float* A, int32_t rowsA, int32_t colsA, const float* B, int32_t rowsB, int32_t colsB, float* C);
/* BatchDotProductAddBias, both overloads (IAccelerationManager.cs:45,50; AccelerationCPU.cs:342-404):
 * Y[rowCount,outDim] = X[rowStart..rowStart+rowCount) * W^T + bias. */
B200_API int32_t b200_BatchDotProductAddBias(b200_ctx*, const float* W, int32_t outDim, int32_t inDim, const float* X, int32_t xRows, int32_t xCols,
                                             int32_t rowStart, int32_t rowCount, const float* bias, int32_t biasLen, float* Y);
/* ProjectOutputBatch (IAccelerationManager.cs:259; AccelerationCPU.cs:2694-2715). */
B200_API int32_t b200_ProjectOutputBatch(b200_ctx*, const float* hidden, int32_t hiddenRows, int32_t embDim, const float* proj, const float* bias,
                                         int32_t seqLen, int32_t outputDim, float* pred);
/* MatrixAddInPlace / VectorAccumulate (IAccelerationManager.cs:91,97): target += addend. */
B200_API int32_t b200_MatrixAddInPlace(b200_ctx*, float* target, const float* addend, int64_t count);
B200_API int32_t b200_VectorAccumulate(b200_ctx*, float* target, const float* source, int64_t count);
/* ZeroMatrix / ZeroVector (IAccelerationManager.cs:80,86). */
B200_API int32_t b200_ZeroMatrix(b200_ctx*, float* matrix, int64_t count);
B200_API int32_t b200_ZeroVector(b200_ctx*, float* vector, int64_t count);

/* ResidualLayerNormForward (IAccelerationManager.cs:138; AccelerationCPU.cs:1440-1514).  subLayer may be NULL
 * (= LayerNormForward, IAccelerationManager.cs:127); normalized/residual/means/variances may be NULL when not wanted
 * (= ResidualLayerNorm / LayerNorm, IAccelerationManager.cs:122,132). */
B200_API int32_t b200_ResidualLayerNormForward(b200_ctx*, const float* input, const float* subLayer, const float* gamma, const float* beta,
                                               int32_t rows, int32_t features, float eps, float* output, float* means, float* variances,
                                               float* normalized, float* residual);
/* LayerNormBackward (IAccelerationManager.cs:143; AccelerationCPU.cs:1516-1564): all three outputs are assigned. */
B200_API int32_t b200_LayerNormBackward(b200_ctx*, const float* dOut, const float* normalized, const float* gamma, const float* input,
                                        const float* mean, const float* variance, int32_t rows, int32_t features, float eps,
                                        float* dInput, float* dGamma, float* dBeta);

/* No counterpart in the reference.  LayerNormBackward for callers that must not cause a device allocation while they
 * run: a host framework that has handed all device memory to its own pool, or a training loop that cannot afford the
 * device-wide synchronisation and possible out-of-memory failure of a driver allocation in the middle of a step.
 * Every pointer is a DEVICE pointer supplied by the caller (inputs and the three outputs, which are assigned as in
 * b200_LayerNormBackward); the call enqueues two kernels on cuda_stream (NULL = default stream) and returns without
 * synchronising.  It takes no context and calls neither cudaMalloc/cudaFree nor any allocating routine: the scratch of
 * the column reduction is a fixed array inside the library (2.3 MiB per GPU, held until the process exits).
 * Limits: features <= 1024 and a multiple of 4 (otherwise B200_ERR_OUT_OF_RANGE / B200_ERR_UNSUPPORTED with a message on
 * stderr); dOut, input, gamma, dInput 16-byte aligned.  The first call on each device looks up the scratch's device
 * address; make that first call before starting any stream capture.  All calls share the one scratch array, so two
 * calls that can overlap on the GPU (different streams without an ordering between them) race: keep calls on one
 * device ordered.  Nothing in the scratch needs clearing between calls.  The looked-up address is kept per device
 * ordinal for the life of the process: after an in-process cudaDeviceReset it is stale, so a process that resets a
 * device must not call this entry point on it again. */
B200_API int32_t b200_LayerNormBackward_noalloc(void* cuda_stream, const float* dOut, const float* input, const float* gamma, const float* mean,
                                                const float* variance, int32_t rows, int32_t features, float eps, float* dInput,
                                                float* dGamma, float* dBeta);

/* ScaledDotProductAttention (IAccelerationManager.cs:167; AccelerationCPU.cs:1797-1956).  mask: NULL or
 * [queryLen,keyLen] bytes, non-zero = visible.  causal with queryLen != keyLen is B200_ERR_INVALID_ARG. */
B200_API int32_t b200_ScaledDotProductAttention(b200_ctx*, const float* q, const float* k, const float* v, int32_t queryLen, int32_t keyLen,
                                                int32_t embDim, int32_t numHeads, const uint8_t* mask, int32_t causal, float* out);
/* MultiHeadAttentionForward (IAccelerationManager.cs:155): same kernel with an explicit scale. */
B200_API int32_t b200_MultiHeadAttentionForward(b200_ctx*, const float* q, const float* k, const float* v, int32_t queryLen, int32_t keyLen,
                                                int32_t embDim, int32_t numHeads, float scale, const uint8_t* mask, float* out);
/* MultiHeadAttentionBackward, both overloads (IAccelerationManager.cs:161,163; AccelerationCPU.cs:1037-1284). */
B200_API int32_t b200_MultiHeadAttentionBackward(b200_ctx*, const float* Q, const float* K, const float* V, const float* dConcat, int32_t seqLenQ,
                                                 int32_t seqLenK, int32_t embDim, int32_t numHeads, float scale, const uint8_t* mask,
                                                 int32_t useDecoderMask, float* dQ, float* dK, float* dV);
/* Trainer-side batched attention that today is C# inside TransformerTrainer
 * (TransformerTrainer.cs:723-809 forward, :989-1121 backward): segment s owns rows [s*segLen,(s+1)*segLen). */
B200_API int32_t b200_SegmentedAttentionForward(b200_ctx*, const float* Q, const float* K, const float* V, int32_t segLen, int32_t segCount,
                                                int32_t embDim, int32_t numHeads, int32_t causal, float* out);
B200_API int32_t b200_SegmentedAttentionBackward(b200_ctx*, const float* Q, const float* K, const float* V, const float* dConcat, int32_t segLen,
                                                 int32_t segCount, int32_t embDim, int32_t numHeads, float scale, int32_t causal,
                                                 float* dQ, float* dK, float* dV);
/* ApplyRotaryPositionEmbeddingInPlace (IAccelerationManager.cs:320; AccelerationCPU.cs:4855-4982); segLen > 0 makes the
 * position row % segLen (TransformerTrainer.cs:811-848 ApplySegmentedRotaryInPlace). */
B200_API int32_t b200_ApplyRotaryPositionEmbeddingInPlace(b200_ctx*, float* matrix, int32_t rows, int32_t embDim, int32_t numHeads,
                                                          float baseTheta, int32_t inverse, int32_t segLen);
/* ApplyRotaryPositionEmbeddingHeadInPlace (IAccelerationManager.cs:319). */
B200_API int32_t b200_ApplyRotaryPositionEmbeddingHeadInPlace(b200_ctx*, float* matrix, int32_t rows, int32_t embDim, int32_t startCol,
                                                              int32_t headDim, float baseTheta, int32_t inverse);

/* ProjectQKV (IAccelerationManager.cs:169; AccelerationCPU.cs:2005-2069). */
B200_API int32_t b200_ProjectQKV(b200_ctx*, const float* input, int32_t rows, int32_t inDim, const float* WQ, const float* bQ, const float* WK,
                                 const float* bK, const float* WV, const float* bV, int32_t outDim, float* Q, float* K, float* V);
/* BackpropQKV (IAccelerationManager.cs:171; AccelerationCPU.cs:2071-2182): the six gradients accumulate, dInput is assigned. */
B200_API int32_t b200_BackpropQKV(b200_ctx*, const float* input, int32_t rows, int32_t inDim, const float* dQ, const float* dK, const float* dV,
                                  int32_t outDim, const float* WQ, const float* WK, const float* WV, float* WQGrad, float* bQGrad,
                                  float* WKGrad, float* bKGrad, float* WVGrad, float* bVGrad, float* dInput);
/* ProjectKV (IAccelerationManager.cs:329; AccelerationCPU.cs:4361-4417) and BackpropKV (IAccelerationManager.cs:331;
 * AccelerationCPU.cs:4419-4560): the key/value halves of the two above, used by the cross-attention of the sibling trainers;
 * the four gradients accumulate, dInput is assigned. */
B200_API int32_t b200_ProjectKV(b200_ctx*, const float* input, int32_t rows, int32_t inDim, const float* WK, const float* bK, const float* WV,
                                const float* bV, int32_t outDim, float* K, float* V);
B200_API int32_t b200_BackpropKV(b200_ctx*, const float* input, int32_t rows, int32_t inDim, const float* dK, const float* dV, int32_t outDim,
                                 const float* WK, const float* WV, float* WKGrad, float* bKGrad, float* WVGrad, float* bVGrad, float* dInput);
/* BackpropLinearProjection (IAccelerationManager.cs:182; AccelerationCPU.cs:2188-2229): weightGrad, biasGrad AND dInput accumulate. */
B200_API int32_t b200_BackpropLinearProjection(b200_ctx*, const float* input, const float* dOutput, const float* weights, int32_t seqLen,
                                               int32_t inDim, int32_t outDim, float* weightGrad, float* biasGrad, float* dInput);
/* BackpropOutputProjection (IAccelerationManager.cs:184; AccelerationCPU.cs:2231-2273): grads accumulate, dX assigned. */
B200_API int32_t b200_BackpropOutputProjection(b200_ctx*, const float* dLogits, const float* input, const float* weights, float* weightGrad,
                                               float* biasGrad, int32_t seqLen, int32_t outputDim, int32_t embDim, float* dX);
/* BackpropInputProjection, both overloads (IAccelerationManager.cs:190,197; AccelerationCPU.cs:2275-2332). */
B200_API int32_t b200_BackpropInputProjection(b200_ctx*, const float* dX, int32_t dXRows, int32_t dXCols, const float* continuousInput,
                                              int32_t contRows, int32_t contCols, int32_t inputRowStart, float* weightGrad, float* biasGrad,
                                              int32_t seqLen, int32_t embDim, int32_t inputFeatureDim);
/* EmbedTokenIds, both overloads (IAccelerationManager.cs:275,277; AccelerationCPU.cs:3473-3515).  An id outside
 * [0,vocab) is B200_ERR_OUT_OF_RANGE, checked on the host before any launch. */
B200_API int32_t b200_EmbedTokenIds(b200_ctx*, const int32_t* tokenIds, int32_t nIds, int32_t tokenStart, int32_t tokenCount,
                                    const float* embedding, int32_t vocab, int32_t embDim, float* out);
/* AccumulateTokenEmbeddingGrad, both overloads (IAccelerationManager.cs:203,205; AccelerationCPU.cs:2334-2370):
 * embeddingGrad[ids[tokenStart+i],:] += dX[i,:], duplicates summed in row order (deterministic). */
B200_API int32_t b200_AccumulateTokenEmbeddingGrad(b200_ctx*, float* embeddingGrad, int32_t vocab, const float* dX, const int32_t* tokenIds,
                                                   int32_t nIds, int32_t tokenStart, int32_t seqLen, int32_t embDim);
/* CrossEntropyLossAndGradient, both overloads (IAccelerationManager.cs:207,209; AccelerationCPU.cs:2372-2440).
 * dLogits is [rows,outputDim]; rows at and beyond effectiveLen are zero. */
B200_API int32_t b200_CrossEntropyLossAndGradient(b200_ctx*, const float* logits, int32_t rows, int32_t outputDim, const int32_t* targets,
                                                  int32_t nTargets, int32_t targetStart, int32_t effectiveLen, float* loss, float* dLogits);
/* MSELossAndGradient, both overloads (IAccelerationManager.cs:212,214; AccelerationCPU.cs:2442-2491). */
B200_API int32_t b200_MSELossAndGradient(b200_ctx*, const float* predictions, int32_t rows, int32_t outputDim, const float* targets,
                                         int32_t targetRows, int32_t targetStart, int32_t effectiveLen, float* loss, float* dOutput);
/* MatrixSquaredNorm / VectorSquaredNorm (IAccelerationManager.cs:221,228). */
B200_API int32_t b200_MatrixSquaredNorm(b200_ctx*, const float* matrix, int64_t count, float* out);
B200_API int32_t b200_VectorSquaredNorm(b200_ctx*, const float* vector, int64_t count, float* out);
/* MatrixScaleInPlace / VectorScaleInPlace (IAccelerationManager.cs:235,240). */
B200_API int32_t b200_MatrixScaleInPlace(b200_ctx*, float* matrix, int64_t count, float scale);
B200_API int32_t b200_VectorScaleInPlace(b200_ctx*, float* vector, int64_t count, float scale);
/* MatrixUpdate / VectorUpdate (IAccelerationManager.cs:246,248; AccelerationCPU.cs:2548-2590): w -= lr*g. */
B200_API int32_t b200_MatrixUpdate(b200_ctx*, float* weights, const float* gradients, int64_t count, float learningRate);
B200_API int32_t b200_VectorUpdate(b200_ctx*, float* weights, const float* gradients, int64_t count, float learningRate);

/* FFNForwardBatch (IAccelerationManager.cs:165) for the case the reference itself special-cases: the delegate's target
 * is a NeuralNetwork (AccelerationCPU.cs:1975-1985 -> NeuralNetwork.ForwardPassOnlyBatch, NeuralNetwork.cs:629-668).
 * The network is passed as nLayers widths/activations (entry 0 = input layer) and, for l = 1..nLayers-1,
 * weights[l] ([widths[l], widths[l-1]]) and biases[l]; entry 0 of the pointer arrays is ignored. */
B200_API int32_t b200_FFNForwardBatch(b200_ctx*, const float* input, int32_t rows, int32_t nLayers, const int32_t* widths, const int32_t* activations,
                                      const float* const* weights, const float* const* biases, float* out);
/* NeuralNetwork.ComputeInputGradientBatch (NeuralNetwork.cs:773-987), the FFN backward the trainer calls at
 * TransformerTrainer.cs:923-931.  weightGrads/biasGrads may both be NULL; otherwise they accumulate. */
B200_API int32_t b200_FFNInputGradientBatch(b200_ctx*, const float* input, const float* dOutput, int32_t rows, int32_t nLayers, const int32_t* widths,
                                            const int32_t* activations, const float* const* weights, const float* const* biases,
                                            float* const* weightGrads, float* const* biasGrads, float* dInput);

/* ------------------------------------------------------------------------------------------------ A2. sibling trainers' ops
 * The operators the TACAMT / MMTAC / PriceTAC trainers call on the same interface (IAccelerationManager.cs:251-361).
 * Rank-3 arrays are passed flat in the reference's own element order. */
/* ContentAwareCrossAttentionForward (IAccelerationManager.cs:263; AccelerationCPU.cs:3076-3270).  decayBias is
 * [queryLen, keyLen, numHeads] or NULL; attentionWeights and scoresPreSoftmax are [numHeads, queryLen, keyLen] or NULL
 * (needBackwardCache = false).  -inf scores get weight 0; a row of only -inf scores gives zero weights and output. */
B200_API int32_t b200_ContentAwareCrossAttentionForward(b200_ctx*, const float* Q, int32_t queryLen, const float* K, const float* V,
                                                        int32_t keyLen, int32_t embDim, int32_t numHeads, float scale, const float* decayBias,
                                                        float* output, float* attentionWeights, float* scoresPreSoftmax);
/* BackpropTimeDecayedAttention (IAccelerationManager.cs:287; AccelerationCPU.cs:3748-3857).  attentionWeights is
 * [numHeads, queryLen, keyLen]; dDecayBias is [queryLen, keyLen, numHeads], or NULL where the reference is called without
 * time differences; dQ, dK, dV are assigned.  The scale is 1/sqrt(embeddingDim / numHeads). */
B200_API int32_t b200_BackpropTimeDecayedAttention(b200_ctx*, const float* q, int32_t queryLen, const float* k, const float* v, int32_t keyLen,
                                                   const float* dOutput, const float* attentionWeights, int32_t embeddingDim, int32_t numHeads,
                                                   float* dQ, float* dK, float* dV, float* dDecayBias);
/* ApplyContextTypeEmbedding (IAccelerationManager.cs:253; AccelerationCPU.cs:2596-2644): contextHidden[i,:] += typeEmbedding[typeIndices[i],:]. */
B200_API int32_t b200_ApplyContextTypeEmbedding(b200_ctx*, float* contextHidden, int32_t rows, int32_t embDim, const float* typeEmbedding,
                                                int32_t typeCount, const int32_t* typeIndices);
/* ComputeTimeDiffMatrix (IAccelerationManager.cs:255; AccelerationCPU.cs:2646-2674): out[p, s] = p - keyArrivalTimes[s]. */
B200_API int32_t b200_ComputeTimeDiffMatrix(b200_ctx*, int32_t priceSeqLen, const float* keyArrivalTimes, int32_t numKeys, float* out);
/* ComputeMemoryAttentionScores (IAccelerationManager.cs:257; AccelerationCPU.cs:2676-2692). */
B200_API int32_t b200_ComputeMemoryAttentionScores(b200_ctx*, const float* priceHidden, int32_t priceRows, int32_t embDim, int32_t lastPos,
                                                   const float* contextHidden, int32_t totalCtx, float scale, float* scores);
/* ProjectGlobalFeatures (IAccelerationManager.cs:273; AccelerationCPU.cs:3424-3461): out = bias + projection[embDim, featureDim] * globalFeatures. */
B200_API int32_t b200_ProjectGlobalFeatures(b200_ctx*, const float* globalFeatures, int32_t featureDim, const float* projection, const float* bias,
                                            int32_t embDim, float* out);
/* MeanPoolRows (IAccelerationManager.cs:279; AccelerationCPU.cs:3517-3552) and its gradient ExpandMeanPoolGradient
 * (IAccelerationManager.cs:360; AccelerationCPU.cs:4321-4359). */
B200_API int32_t b200_MeanPoolRows(b200_ctx*, const float* matrix, int32_t rows, int32_t cols, float* out);
B200_API int32_t b200_ExpandMeanPoolGradient(b200_ctx*, const float* pooledGradient, int32_t pooledRows, int32_t pooledCols, int32_t rowIndex,
                                             int32_t rowCount, int32_t embeddingDim, float* out);
/* SoftmaxVector (IAccelerationManager.cs:285; AccelerationCPU.cs:3700-3746). */
B200_API int32_t b200_SoftmaxVector(b200_ctx*, const float* scores, int32_t n, float* out);
/* SigmoidInPlace (IAccelerationManager.cs:324; AccelerationCPU.cs:143-153, 4985-4992). */
B200_API int32_t b200_SigmoidInPlace(b200_ctx*, float* matrix, int64_t count);
/* ZeroMatrixColumns (IAccelerationManager.cs:327; AccelerationCPU.cs:5016-5035): the first min(columnCount, cols) columns of every row. */
B200_API int32_t b200_ZeroMatrixColumns(b200_ctx*, float* matrix, int32_t rows, int32_t cols, int32_t columnCount);
/* VectorUpdateClamped (IAccelerationManager.cs:337; AccelerationCPU.cs:5037-5056). */
B200_API int32_t b200_VectorUpdateClamped(b200_ctx*, float* weights, const float* gradients, int64_t count, float learningRate, float minValue,
                                          float maxValue);
/* AccumulateGlobalProjectionGradients (IAccelerationManager.cs:358; AccelerationCPU.cs:4296-4319); any NULL array: no-op, as in the reference. */
B200_API int32_t b200_AccumulateGlobalProjectionGradients(b200_ctx*, const float* dGlobalHidden, int32_t embDim, const float* globalFeatures,
                                                          int32_t featureDim, float* projectionGrad, float* biasGrad);
/* Matrix3DScaleInPlace, MatrixSquaredNorm3D (IAccelerationManager.cs:267,269; AccelerationCPU.cs:3388-3422), Matrix3DAddInPlace,
 * Matrix3DUpdate (IAccelerationManager.cs:333,335; AccelerationCPU.cs:5058-5130): count = d0 * d1 * d2. */
B200_API int32_t b200_Matrix3DScaleInPlace(b200_ctx*, float* matrix, int64_t count, float scale);
B200_API int32_t b200_MatrixSquaredNorm3D(b200_ctx*, const float* matrix, int64_t count, float* out);
B200_API int32_t b200_Matrix3DAddInPlace(b200_ctx*, float* target, const float* addend, int64_t count);
B200_API int32_t b200_Matrix3DUpdate(b200_ctx*, float* weights, const float* gradients, int64_t count, float learningRate);

/* ------------------------------------------------------------------------------------------------ B. resident LM */
/* Model shape = TransformerConfig (Transformers/MultiTypeTransformer/TransformerConfig.cs:17-103). */
typedef struct {
    int32_t vocab_size;        /* VocabSize (discrete models) */
    int32_t input_feature_dim; /* InputFeatureDim (continuous models) */
    int32_t output_dim;        /* EffectiveOutputDim */
    int32_t embedding_dim, num_heads, num_layers, ffn_dim;
    int32_t ffn_activation;    /* B200_ACT_* of the FFN hidden layer */
    int32_t discrete;          /* Data.UsesDiscreteTokens */
    int32_t loss_kind;         /* 0 cross-entropy, 1 MSE (TimeSeriesRegression) */
    int32_t causal;            /* UseDecoderOnly */
    int32_t align_floats;      /* tensor offsets in the flat arena are multiples of this (>= 1; 64 recommended) */
} b200_lm_config;

/* Flat parameter arena.  Tensor order = the reference's weights.bin (LanguageModel.cs:737-765) with each block's FFN
 * appended to the block: [TokenEmbedding | InputProjection, InputProjectionBias], then per layer WQ WK WV WO bQ bK bV bO
 * LN1Gamma LN1Beta LN2Gamma LN2Beta W1 b1 W2 b2, then OutputProjection, OutputBias. */
B200_API int64_t b200_lm_param_count(const b200_lm_config* cfg);
B200_API int32_t b200_lm_tensor_count(const b200_lm_config* cfg);
B200_API int32_t b200_lm_tensor_info(const b200_lm_config* cfg, int32_t index, int64_t* offset, int32_t* rows, int32_t* cols);

/* Replaces the construction of TransformerTrainer's state (TransformerTrainer.cs:17-41: model, TransformerGradients,
 * FFN gradient storage).  params_dev / grads_dev: optional caller-owned DEVICE buffers of b200_lm_param_count floats
 * (e.g. tensors of a host framework that all-reduces the gradients); NULL lets the library allocate.
 * max_rows_per_pass bounds the rows (tokens) of one forward/backward pass; larger batches are split. */
B200_API int32_t b200_lm_create(b200_ctx*, const b200_lm_config* cfg, float* params_dev, float* grads_dev, int32_t max_rows_per_pass, b200_lm** out);
B200_API int32_t b200_lm_destroy(b200_lm*);
B200_API int32_t b200_lm_upload_params(b200_lm*, const float* host, int64_t offset, int64_t count);
B200_API int32_t b200_lm_download_params(b200_lm*, float* host, int64_t offset, int64_t count);
B200_API int32_t b200_lm_download_grads(b200_lm*, float* host, int64_t offset, int64_t count);
B200_API float* b200_lm_params_device(b200_lm*);
/* The gradient arena on the device.  A step does not write the scaled-and-clipped gradient back; the factor is applied
 * (one kernel on the context's stream) the first time the arena is looked at through this call or b200_lm_download_grads,
 * or added to by a further b200_lm_accumulate_*, so every observer sees what the reference leaves behind. */
B200_API float* b200_lm_grads_device(b200_lm*);
B200_API int32_t b200_lm_set_optimizer(b200_lm*, int32_t kind, float beta1, float beta2, float eps);

/* TransformerTrainer.TrainBatchDiscrete (TransformerTrainer.cs:217-327) on one batch: sequence s is
 * tokens[seq_offsets[s] .. seq_offsets[s+1]).  Zeroes the gradients, runs forward + loss + backward for every valid
 * sequence, scales by 1/validCount, computes the global gradient norm, clips and (do_step != 0) applies the update.
 * Outputs: *loss = totalLoss/validCount, *grad_norm (before clipping), *valid_count. */
B200_API int32_t b200_lm_train_step_discrete(b200_lm*, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq, float lr, int32_t use_clip,
                                             float clip_threshold, int32_t do_step, float* loss, float* grad_norm, int32_t* valid_count);
/* TransformerTrainer.TrainBatchContinuous (TransformerTrainer.cs:337-486): features [rows,F]; regression targets
 * [rows,O] (loss_kind 1) or class targets [rows] (loss_kind 0); seq_offsets count rows; row t trains against row t+1. */
B200_API int32_t b200_lm_train_step_continuous(b200_lm*, const float* features, const float* reg_targets, const int32_t* class_targets,
                                               const int32_t* seq_offsets, int32_t n_seq, float lr, int32_t use_clip, float clip_threshold,
                                               int32_t do_step, float* loss, float* grad_norm, int32_t* valid_count);

/* Device-resident batches (no counterpart in the reference, whose trainers re-read managed arrays every step): the
 * batch is validated, bucketed, packed into passes and copied to the device ONCE; training on it afterwards moves no
 * input bytes from the host.  Semantics of b200_lm_train_step_batch = b200_lm_train_step_discrete/continuous. */
B200_API int32_t b200_lm_batch_create_discrete(b200_lm*, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq, b200_lm_batch** out);
B200_API int32_t b200_lm_batch_create_continuous(b200_lm*, const float* features, const float* reg_targets, const int32_t* class_targets,
                                                 const int32_t* seq_offsets, int32_t n_seq, b200_lm_batch** out);
B200_API int32_t b200_lm_batch_destroy(b200_lm_batch*);
B200_API int32_t b200_lm_accumulate_batch(b200_lm*, b200_lm_batch*, float* loss_sum, int32_t* valid_count);
B200_API int32_t b200_lm_train_step_batch(b200_lm*, b200_lm_batch*, float lr, int32_t use_clip, float clip_threshold, int32_t do_step,
                                          float* loss, float* grad_norm, int32_t* valid_count);

/* Data-parallel decomposition of the same step (no counterpart in the reference, which is single-device):
 *   b200_lm_zero_grads -> b200_lm_accumulate_* (this rank's sequences; gradients summed, unscaled)
 *   -> the host all-reduces the gradient arena, loss sum and valid count -> b200_lm_apply_step on every rank.
 * The callback, when set, fires on the calling thread during the LAST pass of b200_lm_accumulate_* each time a
 * contiguous range of the gradient arena [offset, offset+count) has received its final contribution; `event` is a
 * cudaEvent_t recorded on the compute stream after that contribution (make the communication stream wait on it). */
typedef void (*b200_grad_ready_fn)(void* user, int64_t offset, int64_t count, void* event);
B200_API int32_t b200_lm_set_grad_ready_callback(b200_lm*, b200_grad_ready_fn fn, void* user);
B200_API int32_t b200_lm_zero_grads(b200_lm*);
B200_API int32_t b200_lm_accumulate_discrete(b200_lm*, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq, float* loss_sum, int32_t* valid_count);
B200_API int32_t b200_lm_accumulate_continuous(b200_lm*, const float* features, const float* reg_targets, const int32_t* class_targets,
                                               const int32_t* seq_offsets, int32_t n_seq, float* loss_sum, int32_t* valid_count);
B200_API int32_t b200_lm_apply_step(b200_lm*, int32_t global_valid_count, float lr, int32_t use_clip, float clip_threshold, int32_t do_step, float* grad_norm);
/* TransformerTrainer.Validate (TransformerTrainer.cs:1142-1184) / ValidateContinuous (:1185-1268): forward and loss
 * only, on the device.  Every valid sequence contributes its mean loss times its trained rows (len-1); sequences that are
 * too short, hold invalid ids or produce a non-finite loss are skipped; *mean_loss = sum / contributing rows (0 when
 * none), *items = contributing rows. */
B200_API int32_t b200_lm_validate_discrete(b200_lm*, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq, float* mean_loss, int32_t* items);
B200_API int32_t b200_lm_validate_continuous(b200_lm*, const float* features, const float* reg_targets, const int32_t* class_targets,
                                             const int32_t* seq_offsets, int32_t n_seq, float* mean_loss, int32_t* items);
/* Optimiser state for checkpoints that resume without leaving the resident path (LanguageModel.Save/Load,
 * LanguageModel.cs:706-839, write weights only; the Adam moments are this library's extension).  which = 0: first
 * moments, 1: second moments; same layout and offsets as the parameter arena.  The step index drives the bias
 * correction. */
B200_API int32_t b200_lm_download_optimizer_state(b200_lm*, int32_t which, float* host, int64_t offset, int64_t count);
B200_API int32_t b200_lm_upload_optimizer_state(b200_lm*, int32_t which, const float* host, int64_t offset, int64_t count);
B200_API int32_t b200_lm_get_step_index(b200_lm*, int32_t* step_index);
B200_API int32_t b200_lm_set_step_index(b200_lm*, int32_t step_index);
/* Incremental decoding with a device key/value cache (LanguageModel.Generate, decoder path, LanguageModel.cs:270-537):
 * b200_lm_gen_step pushes one token through the model at position = current length (ForwardDecoderTokenFromId) and
 * returns the next-token logits (ProjectLastTokenOnly) -- temperature and sampling stay with the caller, as the
 * reference draws from its own random generator.  b200_lm_gen_greedy runs prompt + arg-max continuation without a host
 * round trip per token.  max_len = capacity of the cache (the reference's MaxSequenceLength). */
typedef struct b200_lm_gen b200_lm_gen;
B200_API int32_t b200_lm_gen_create(b200_lm*, int32_t max_len, b200_lm_gen** out);
B200_API int32_t b200_lm_gen_destroy(b200_lm_gen*);
B200_API int32_t b200_lm_gen_reset(b200_lm_gen*);
B200_API int32_t b200_lm_gen_length(b200_lm_gen*, int32_t* length);
/* How a token is executed.  Every decoding kernel takes the token's position from device memory, so nothing in the
 * launch sequence depends on the host.  Preferred: ONE cooperative kernel per token, its phases separated by grid barriers
 * (b200_lm_gen_single_kernel returns 1).  Otherwise -- tensors of the arena not 16-byte aligned, Q/K/V weights not back to
 * back, no cooperative launch, or b200_lm_gen_set_single_kernel(g, 0) -- the phases are separate launches (six per block),
 * captured into a CUDA graph when the session processes its second token and replayed afterwards; *nodes = launches per
 * replay (0 = plain launches so far). */
B200_API int32_t b200_lm_gen_single_kernel(b200_lm_gen*);
B200_API int32_t b200_lm_gen_set_single_kernel(b200_lm_gen*, int32_t on);
B200_API int32_t b200_lm_gen_graph_nodes(b200_lm_gen*, int32_t* nodes);
B200_API int32_t b200_lm_gen_step(b200_lm_gen*, int32_t token_id, float* logits);
B200_API int32_t b200_lm_gen_greedy(b200_lm_gen*, const int32_t* prompt, int32_t n_prompt, int32_t max_new, int32_t* out_tokens, int32_t* n_out);
/* Device time of the phases of the last step in milliseconds: [0] forward, [1] loss, [2] backward, [3] step. */
B200_API int32_t b200_lm_get_timings(b200_lm*, float* ms4);

/* ------------------------------------------------------------------------------------------------ D. data parallel */
/* No counterpart in the reference, which trains on one device (AccelerationFactory.cs:31-45 builds one manager for one
 * device id).  The batch is split by sequence over the ranks, every rank holds the full model, the gradient arena is
 * summed with NCCL all-reduces issued on a communication stream as each range becomes final during the last pass's
 * backward (output projection, blocks last to first, embedding), one more all-reduce carries {loss sum, valid count,
 * failed ranks}, and every rank applies the identical fused step -- TransformerTrainer.cs:313-326 over the whole
 * batch.  The collective library is loaded at run time (libnccl.so.2 as already loaded in the process, else from the
 * loader path, else from b200_dp_set_nccl_library's path); the host needs no NCCL binding of its own.
 *
 * Failure rules (TransformerTrainer.cs:298-307, 316-320 carried over to several ranks): every rank issues the same
 * collectives in the same order whatever happened locally; a rank whose pass failed reports it in the scalar
 * all-reduce and then every rank zeroes its gradients, leaves the weights untouched and returns an error (its own on
 * the failing rank, B200_ERR_PEER elsewhere); a peer that does not arrive within the deadline (default 30 s) gives
 * B200_ERR_TIMEOUT after the communicator has been aborted (the object must then be destroyed); a non-finite gradient
 * norm skips the update and zeroes the gradients on every rank alike, because all ranks hold identical sums.
 *
 * One process per GPU: rank 0 calls b200_dp_unique_id, the host hands the 128 bytes to the other processes (any
 * channel), every process calls b200_dp_create_rank on its own trainer.  One process for all GPUs:
 * b200_dp_group_create(devices, n, ...) builds a context, a trainer and a rank per listed device and drives them with
 * one host thread each. */
typedef struct b200_dp b200_dp;
typedef struct b200_dp_group b200_dp_group;
B200_API int32_t b200_dp_set_nccl_library(const char* path);
/* CTAs a communicator created after this call may use (ncclConfig_t.maxCTAs; default 16, 0 = NCCL's own choice).  A step's
 * all-reduce needs a small fraction of NVLink's bandwidth; what it costs is the SMs its kernels hold beside the backward
 * GEMMs while they wait for peers. */
B200_API int32_t b200_dp_set_nccl_max_ctas(int32_t n);
B200_API int32_t b200_dp_unique_id(uint8_t* id128);
B200_API int32_t b200_dp_create_rank(b200_lm* lm, const uint8_t* id128, int32_t rank, int32_t world, b200_dp** out);
B200_API int32_t b200_dp_destroy(b200_dp*);
/* [lo, hi) of the sequences of a global batch that `rank` trains (contiguous; the first n_seq % world ranks take one more). */
B200_API int32_t b200_dp_shard(int32_t n_seq, int32_t rank, int32_t world, int32_t* lo, int32_t* hi);
B200_API int32_t b200_dp_set_deadline_ms(b200_dp*, int32_t milliseconds);
/* Copies rank `root`'s parameter arena to every rank (after root uploaded or loaded weights). */
B200_API int32_t b200_dp_broadcast_params(b200_dp*, int32_t root);
/* One step on a GLOBAL batch in host memory (same arrays on every rank; each trains its shard).  Outputs as
 * b200_lm_train_step_discrete, identical on every rank. */
B200_API int32_t b200_dp_train_step_discrete(b200_dp*, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq, float lr, int32_t use_clip,
                                             float clip_threshold, int32_t do_step, float* loss, float* grad_norm, int32_t* valid_count);
B200_API int32_t b200_dp_train_step_continuous(b200_dp*, const float* features, const float* reg_targets, const int32_t* class_targets,
                                               const int32_t* seq_offsets, int32_t n_seq, float lr, int32_t use_clip, float clip_threshold,
                                               int32_t do_step, float* loss, float* grad_norm, int32_t* valid_count);
/* The same on a device-resident shard: b200_dp_batch_create_discrete keeps this rank's part of the global batch on
 * the device (an empty shard is valid); release it with b200_lm_batch_destroy. */
B200_API int32_t b200_dp_batch_create_discrete(b200_dp*, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq, b200_lm_batch** out);
B200_API int32_t b200_dp_batch_create_continuous(b200_dp*, const float* features, const float* reg_targets, const int32_t* class_targets,
                                                 const int32_t* seq_offsets, int32_t n_seq, b200_lm_batch** out);
B200_API int32_t b200_dp_train_step_batch(b200_dp*, b200_lm_batch* shard, float lr, int32_t use_clip, float clip_threshold, int32_t do_step,
                                          float* loss, float* grad_norm, int32_t* valid_count);
/* Communication of the last step, milliseconds on the device: [0] exposed = how long the compute stream waited for the
 * last all-reduce after its own backward had finished; [1] span from the first all-reduce's start to the last one's end. */
B200_API int32_t b200_dp_get_timings(b200_dp*, float* ms2);

B200_API int32_t b200_dp_group_create(const int32_t* devices, int32_t n_devices, const b200_lm_config* cfg, int32_t max_rows_per_pass,
                                      int32_t gemm_mode, b200_dp_group** out);
B200_API int32_t b200_dp_group_destroy(b200_dp_group*);
B200_API const char* b200_dp_group_last_error(b200_dp_group*);
B200_API int32_t b200_dp_group_size(b200_dp_group*);
B200_API b200_lm* b200_dp_group_trainer(b200_dp_group*, int32_t rank);  /* the rank's trainer, e.g. for downloads */
B200_API int32_t b200_dp_group_set_optimizer(b200_dp_group*, int32_t kind, float beta1, float beta2, float eps);
B200_API int32_t b200_dp_group_upload_params(b200_dp_group*, const float* host, int64_t offset, int64_t count);  /* to every rank */
B200_API int32_t b200_dp_group_train_step_discrete(b200_dp_group*, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq, float lr,
                                                   int32_t use_clip, float clip_threshold, int32_t do_step, float* loss, float* grad_norm,
                                                   int32_t* valid_count);
B200_API int32_t b200_dp_group_train_step_continuous(b200_dp_group*, const float* features, const float* reg_targets, const int32_t* class_targets,
                                                     const int32_t* seq_offsets, int32_t n_seq, float lr, int32_t use_clip, float clip_threshold,
                                                     int32_t do_step, float* loss, float* grad_norm, int32_t* valid_count);

/* ------------------------------------------------------------------------------------------------ C. resident MLP */
/* NeuralNetwork.TrainBatch state (NeuralNetwork.cs:420-477 + BatchedAccelerationGPU.cs:12-149): weights stay on the
 * device across batches.  widths/activations have nLayers entries (entry 0 = input layer, its activation unused). */
B200_API int32_t b200_mlp_create(b200_ctx*, int32_t nLayers, const int32_t* widths, const int32_t* activations, int32_t cost, float huber_delta,
                                 float l2_lambda, float clip_threshold, int32_t max_batch, b200_mlp** out);
B200_API int32_t b200_mlp_destroy(b200_mlp*);
/* layer = 1..nLayers-1.  download = AccelerationGPUBatch.CopyLayerToCPU (BatchedAccelerationGPU.cs:236-247). */
B200_API int32_t b200_mlp_upload_layer(b200_mlp*, int32_t layer, const float* weights, const float* biases);
B200_API int32_t b200_mlp_download_layer(b200_mlp*, int32_t layer, float* weights, float* biases);
/* NeuralNetwork.LearnBatch (NeuralNetwork.cs:499-520, 542-610): X [B,widths[0]] already input-scaled, Y [B,widths[last]].
 * in_min/in_max non-NULL applies ScaleInput (NeuralNetwork.cs:121-134) to X on the device first. */
B200_API int32_t b200_mlp_learn_batch(b200_mlp*, const float* X, const float* Y, int32_t B, float lr, const float* in_min, const float* in_max,
                                      float* delta_norm);

#ifdef __cplusplus
}
#endif
#endif
