// CudaB200AccelerationManager.cs -- the C# side of the boundary: CallaghanDev.ML's IAccelerationManager
// (CallaghanDev.ML/AccelerationManagers/IAccelerationManager.cs:13-361) implemented over libcallaghan_b200.so, plus the two
// small interfaces the resident trainers are reached through (IB200TrainStep for TransformerTrainer, IB200MlpBatch for
// NeuralNetwork.TrainBatch).  Add this file to CallaghanDev.ML/AccelerationManagers/ together with the five host edits
// listed in INTEGRATION.md; AllowUnsafeBlocks is already on (CallaghanDev.ML/CallaghanDev.ML.csproj:8).
//
// Status of this file: written against include/callaghan_b200.h (every DllImport below was generated from that header)
// and against the interface as it stands in the reference; it has NOT been compiled -- no .NET toolchain exists where
// the library is built.  The Python class callaghandev.ml_b200.CudaB200AccelerationManager binds the same symbols with
// the same argument meaning and is what the parity tests drive.
//
// Rules every method follows (the places a binding goes wrong):
//   * null checks and the shape checks that the reference performs BEFORE touching data stay in C#, with the
//     reference's exception types (ArgumentNullException / ArgumentException / ArgumentOutOfRangeException,
//     e.g. AccelerationCPU.cs:354-380, 1859-1862, 3506-3509); everything else is validated by the library, whose
//     status codes map back to the same types in Check();
//   * float[,] is contiguous row-major: `fixed (float* p = m)` is the (pointer, rows, cols) the ABI takes;
//   * accumulate-vs-assign is the reference's: *Grad arrays, embeddingGrad and BackpropLinearProjection's dInput are
//     added to in place; returned arrays are freshly allocated here and assigned by the library;
//   * nothing is retained by the library after a per-op call returns;
//   * methods outside the training hot path (tokenizer strings, MMTAC context builders and heads, the TACAMT decay
//     network, per-sample NeuralNetwork helpers, small host-side utilities) delegate to an owned AccelerationCPU, as
//     AccelerationGPU delegates to its CPU manager (GPU/AccelerationGPU.cs:17,138).
using System;
using System.Collections.Generic;
using System.Runtime.InteropServices;
using CallaghanDev.ML.Enums;
using CallaghanDev.ML.Transformers.TACAMT;

namespace CallaghanDev.ML.AccelerationManagers
{
    /// <summary>TransformerTrainer routes TrainBatchDiscrete / TrainBatchContinuous / Validate here when its manager
    /// implements this interface (host edit 4).</summary>
    public interface IB200TrainStep
    {
        void AttachModel(B200ModelShape shape, float[] flatParameters, int maxRowsPerPass);
        (float loss, float gradNorm, int validCount) TrainBatchDiscrete(int[] tokens, int[] seqOffsets, float learningRate, bool useClip, float clipThreshold);
        (float loss, float gradNorm, int validCount) TrainBatchContinuous(float[,] features, float[,] regressionTargets, int[] classTargets, int[] seqOffsets,
                                                                           float learningRate, bool useClip, float clipThreshold);
        (float meanLoss, int items) ValidateDiscrete(int[] tokens, int[] seqOffsets);
        float[] DownloadParameters();
    }

    /// <summary>NeuralNetwork.TrainBatch uses this in place of the concrete AccelerationGPUBatch (host edit 5).</summary>
    public interface IB200MlpBatch
    {
        IntPtr CreateMlp(int[] widths, ActivationType[] activations, CostFunctionType cost, float huberDelta, float l2Lambda, float clipThreshold, int maxBatch);
        void UploadLayer(IntPtr mlp, int layer, float[,] weights, float[] biases);
        void DownloadLayer(IntPtr mlp, int layer, float[,] weights, float[] biases);
        float LearnBatch(IntPtr mlp, float[,] x, float[,] y, float learningRate, float[] inputMin, float[] inputMax);
        void DestroyMlp(IntPtr mlp);
    }

    /// <summary>b200_lm_config (include/callaghan_b200.h): the TransformerConfig fields that shape the trained tensors.</summary>
    [StructLayout(LayoutKind.Sequential)]
    public struct LmConfig
    {
        public int vocab_size, input_feature_dim, output_dim, embedding_dim, num_heads, num_layers, ffn_dim, ffn_activation, discrete, loss_kind, causal, align_floats;
    }

    public struct B200ModelShape
    {
        public int VocabSize, InputFeatureDim, OutputDim, EmbeddingDim, NumHeads, NumLayers, FeedForwardDim;
        public ActivationType FfnActivation;
        public bool Discrete, MseLoss, Causal;
    }

    [UnmanagedFunctionPointer(CallingConvention.Cdecl)]
    public delegate void GradReadyFn(IntPtr user, long offset, long count, IntPtr cudaEvent);

    internal static unsafe class Native
    {
        const string Lib = "callaghan_b200";
    [DllImport(Lib)] internal static extern int b200_create(int device, out IntPtr @out);
    [DllImport(Lib)] internal static extern int b200_destroy(IntPtr ctx);
    [DllImport(Lib)] internal static extern IntPtr b200_last_error(IntPtr ctx);
    [DllImport(Lib)] internal static extern int b200_set_stream(IntPtr ctx, IntPtr cuda_stream);
    [DllImport(Lib)] internal static extern int b200_set_gemm_mode(IntPtr ctx, int mode);
    [DllImport(Lib)] internal static extern int b200_synchronize(IntPtr ctx);
    [DllImport(Lib)] internal static extern long b200_kernel_launches(IntPtr ctx);
    [DllImport(Lib)] internal static extern int b200_profile_gemm(IntPtr ctx, int enable);
    [DllImport(Lib)] internal static extern int b200_gemm_profile(IntPtr ctx, int engine, long* launches, double* flops, double* ms);
    [DllImport(Lib)] internal static extern long b200_gemm_profile_csv(IntPtr ctx, byte* buf, long capacity);
    [DllImport(Lib)] internal static extern int b200_has_tcgen05(IntPtr ctx);
    [DllImport(Lib)] internal static extern int b200_engine_launches(IntPtr ctx, long* @out);
    [DllImport(Lib)] internal static extern int b200_set_gemm_kernel(IntPtr ctx, int kernel);
    [DllImport(Lib)] internal static extern int b200_set_wait_budget_us(IntPtr ctx, long microseconds);
    [DllImport(Lib)] internal static extern int b200_probe_wait_timeout(IntPtr ctx);
    [DllImport(Lib)] internal static extern int b200_MatrixMultiply(IntPtr h, float* A, int rowsA, int colsA, float* B, int rowsB, int colsB, float* C);
    [DllImport(Lib)] internal static extern int b200_MatrixMultiplyTranspose(IntPtr h, float* A, int rowsA, int colsA, float* B, int rowsB, int colsB, float* C);
    [DllImport(Lib)] internal static extern int b200_BatchDotProductAddBias(IntPtr h, float* W, int outDim, int inDim, float* X, int xRows, int xCols, int rowStart, int rowCount, float* bias, int biasLen, float* Y);
    [DllImport(Lib)] internal static extern int b200_ProjectOutputBatch(IntPtr h, float* hidden, int hiddenRows, int embDim, float* proj, float* bias, int seqLen, int outputDim, float* pred);
    [DllImport(Lib)] internal static extern int b200_MatrixAddInPlace(IntPtr h, float* target, float* addend, long count);
    [DllImport(Lib)] internal static extern int b200_VectorAccumulate(IntPtr h, float* target, float* source, long count);
    [DllImport(Lib)] internal static extern int b200_ZeroMatrix(IntPtr h, float* matrix, long count);
    [DllImport(Lib)] internal static extern int b200_ZeroVector(IntPtr h, float* vector, long count);
    [DllImport(Lib)] internal static extern int b200_ResidualLayerNormForward(IntPtr h, float* input, float* subLayer, float* gamma, float* beta, int rows, int features, float eps, float* output, float* means, float* variances, float* normalized, float* residual);
    [DllImport(Lib)] internal static extern int b200_LayerNormBackward(IntPtr h, float* dOut, float* normalized, float* gamma, float* input, float* mean, float* variance, int rows, int features, float eps, float* dInput, float* dGamma, float* dBeta);
    [DllImport(Lib)] internal static extern int b200_LayerNormBackward_noalloc(IntPtr cuda_stream, float* dOut, float* input, float* gamma, float* mean, float* variance, int rows, int features, float eps, float* dInput, float* dGamma, float* dBeta);
    [DllImport(Lib)] internal static extern int b200_ScaledDotProductAttention(IntPtr h, float* q, float* k, float* v, int queryLen, int keyLen, int embDim, int numHeads, byte* mask, int causal, float* @out);
    [DllImport(Lib)] internal static extern int b200_MultiHeadAttentionForward(IntPtr h, float* q, float* k, float* v, int queryLen, int keyLen, int embDim, int numHeads, float scale, byte* mask, float* @out);
    [DllImport(Lib)] internal static extern int b200_MultiHeadAttentionBackward(IntPtr h, float* Q, float* K, float* V, float* dConcat, int seqLenQ, int seqLenK, int embDim, int numHeads, float scale, byte* mask, int useDecoderMask, float* dQ, float* dK, float* dV);
    [DllImport(Lib)] internal static extern int b200_SegmentedAttentionForward(IntPtr h, float* Q, float* K, float* V, int segLen, int segCount, int embDim, int numHeads, int causal, float* @out);
    [DllImport(Lib)] internal static extern int b200_SegmentedAttentionBackward(IntPtr h, float* Q, float* K, float* V, float* dConcat, int segLen, int segCount, int embDim, int numHeads, float scale, int causal, float* dQ, float* dK, float* dV);
    [DllImport(Lib)] internal static extern int b200_ApplyRotaryPositionEmbeddingInPlace(IntPtr h, float* matrix, int rows, int embDim, int numHeads, float baseTheta, int inverse, int segLen);
    [DllImport(Lib)] internal static extern int b200_ApplyRotaryPositionEmbeddingHeadInPlace(IntPtr h, float* matrix, int rows, int embDim, int startCol, int headDim, float baseTheta, int inverse);
    [DllImport(Lib)] internal static extern int b200_ProjectQKV(IntPtr h, float* input, int rows, int inDim, float* WQ, float* bQ, float* WK, float* bK, float* WV, float* bV, int outDim, float* Q, float* K, float* V);
    [DllImport(Lib)] internal static extern int b200_BackpropQKV(IntPtr h, float* input, int rows, int inDim, float* dQ, float* dK, float* dV, int outDim, float* WQ, float* WK, float* WV, float* WQGrad, float* bQGrad, float* WKGrad, float* bKGrad, float* WVGrad, float* bVGrad, float* dInput);
    [DllImport(Lib)] internal static extern int b200_ProjectKV(IntPtr h, float* input, int rows, int inDim, float* WK, float* bK, float* WV, float* bV, int outDim, float* K, float* V);
    [DllImport(Lib)] internal static extern int b200_BackpropKV(IntPtr h, float* input, int rows, int inDim, float* dK, float* dV, int outDim, float* WK, float* WV, float* WKGrad, float* bKGrad, float* WVGrad, float* bVGrad, float* dInput);
    [DllImport(Lib)] internal static extern int b200_BackpropLinearProjection(IntPtr h, float* input, float* dOutput, float* weights, int seqLen, int inDim, int outDim, float* weightGrad, float* biasGrad, float* dInput);
    [DllImport(Lib)] internal static extern int b200_BackpropOutputProjection(IntPtr h, float* dLogits, float* input, float* weights, float* weightGrad, float* biasGrad, int seqLen, int outputDim, int embDim, float* dX);
    [DllImport(Lib)] internal static extern int b200_BackpropInputProjection(IntPtr h, float* dX, int dXRows, int dXCols, float* continuousInput, int contRows, int contCols, int inputRowStart, float* weightGrad, float* biasGrad, int seqLen, int embDim, int inputFeatureDim);
    [DllImport(Lib)] internal static extern int b200_EmbedTokenIds(IntPtr h, int* tokenIds, int nIds, int tokenStart, int tokenCount, float* embedding, int vocab, int embDim, float* @out);
    [DllImport(Lib)] internal static extern int b200_AccumulateTokenEmbeddingGrad(IntPtr h, float* embeddingGrad, int vocab, float* dX, int* tokenIds, int nIds, int tokenStart, int seqLen, int embDim);
    [DllImport(Lib)] internal static extern int b200_CrossEntropyLossAndGradient(IntPtr h, float* logits, int rows, int outputDim, int* targets, int nTargets, int targetStart, int effectiveLen, float* loss, float* dLogits);
    [DllImport(Lib)] internal static extern int b200_MSELossAndGradient(IntPtr h, float* predictions, int rows, int outputDim, float* targets, int targetRows, int targetStart, int effectiveLen, float* loss, float* dOutput);
    [DllImport(Lib)] internal static extern int b200_MatrixSquaredNorm(IntPtr h, float* matrix, long count, float* @out);
    [DllImport(Lib)] internal static extern int b200_VectorSquaredNorm(IntPtr h, float* vector, long count, float* @out);
    [DllImport(Lib)] internal static extern int b200_MatrixScaleInPlace(IntPtr h, float* matrix, long count, float scale);
    [DllImport(Lib)] internal static extern int b200_VectorScaleInPlace(IntPtr h, float* vector, long count, float scale);
    [DllImport(Lib)] internal static extern int b200_MatrixUpdate(IntPtr h, float* weights, float* gradients, long count, float learningRate);
    [DllImport(Lib)] internal static extern int b200_VectorUpdate(IntPtr h, float* weights, float* gradients, long count, float learningRate);
    [DllImport(Lib)] internal static extern int b200_FFNForwardBatch(IntPtr h, float* input, int rows, int nLayers, int* widths, int* activations, float** weights, float** biases, float* @out);
    [DllImport(Lib)] internal static extern int b200_FFNInputGradientBatch(IntPtr h, float* input, float* dOutput, int rows, int nLayers, int* widths, int* activations, float** weights, float** biases, float** weightGrads, float** biasGrads, float* dInput);
    [DllImport(Lib)] internal static extern int b200_ContentAwareCrossAttentionForward(IntPtr h, float* Q, int queryLen, float* K, float* V, int keyLen, int embDim, int numHeads, float scale, float* decayBias, float* output, float* attentionWeights, float* scoresPreSoftmax);
    [DllImport(Lib)] internal static extern int b200_BackpropTimeDecayedAttention(IntPtr h, float* q, int queryLen, float* k, float* v, int keyLen, float* dOutput, float* attentionWeights, int embeddingDim, int numHeads, float* dQ, float* dK, float* dV, float* dDecayBias);
    [DllImport(Lib)] internal static extern int b200_ApplyContextTypeEmbedding(IntPtr h, float* contextHidden, int rows, int embDim, float* typeEmbedding, int typeCount, int* typeIndices);
    [DllImport(Lib)] internal static extern int b200_ComputeTimeDiffMatrix(IntPtr h, int priceSeqLen, float* keyArrivalTimes, int numKeys, float* @out);
    [DllImport(Lib)] internal static extern int b200_ComputeMemoryAttentionScores(IntPtr h, float* priceHidden, int priceRows, int embDim, int lastPos, float* contextHidden, int totalCtx, float scale, float* scores);
    [DllImport(Lib)] internal static extern int b200_ProjectGlobalFeatures(IntPtr h, float* globalFeatures, int featureDim, float* projection, float* bias, int embDim, float* @out);
    [DllImport(Lib)] internal static extern int b200_MeanPoolRows(IntPtr h, float* matrix, int rows, int cols, float* @out);
    [DllImport(Lib)] internal static extern int b200_ExpandMeanPoolGradient(IntPtr h, float* pooledGradient, int pooledRows, int pooledCols, int rowIndex, int rowCount, int embeddingDim, float* @out);
    [DllImport(Lib)] internal static extern int b200_SoftmaxVector(IntPtr h, float* scores, int n, float* @out);
    [DllImport(Lib)] internal static extern int b200_SigmoidInPlace(IntPtr h, float* matrix, long count);
    [DllImport(Lib)] internal static extern int b200_ZeroMatrixColumns(IntPtr h, float* matrix, int rows, int cols, int columnCount);
    [DllImport(Lib)] internal static extern int b200_VectorUpdateClamped(IntPtr h, float* weights, float* gradients, long count, float learningRate, float minValue, float maxValue);
    [DllImport(Lib)] internal static extern int b200_AccumulateGlobalProjectionGradients(IntPtr h, float* dGlobalHidden, int embDim, float* globalFeatures, int featureDim, float* projectionGrad, float* biasGrad);
    [DllImport(Lib)] internal static extern int b200_Matrix3DScaleInPlace(IntPtr h, float* matrix, long count, float scale);
    [DllImport(Lib)] internal static extern int b200_MatrixSquaredNorm3D(IntPtr h, float* matrix, long count, float* @out);
    [DllImport(Lib)] internal static extern int b200_Matrix3DAddInPlace(IntPtr h, float* target, float* addend, long count);
    [DllImport(Lib)] internal static extern int b200_Matrix3DUpdate(IntPtr h, float* weights, float* gradients, long count, float learningRate);
    [DllImport(Lib)] internal static extern long b200_lm_param_count(ref LmConfig cfg);
    [DllImport(Lib)] internal static extern int b200_lm_tensor_count(ref LmConfig cfg);
    [DllImport(Lib)] internal static extern int b200_lm_tensor_info(ref LmConfig cfg, int index, long* offset, int* rows, int* cols);
    [DllImport(Lib)] internal static extern int b200_lm_create(IntPtr h, ref LmConfig cfg, float* params_dev, float* grads_dev, int max_rows_per_pass, out IntPtr @out);
    [DllImport(Lib)] internal static extern int b200_lm_destroy(IntPtr h);
    [DllImport(Lib)] internal static extern int b200_lm_upload_params(IntPtr h, float* host, long offset, long count);
    [DllImport(Lib)] internal static extern int b200_lm_download_params(IntPtr h, float* host, long offset, long count);
    [DllImport(Lib)] internal static extern int b200_lm_download_grads(IntPtr h, float* host, long offset, long count);
    [DllImport(Lib)] internal static extern float* b200_lm_params_device(IntPtr h);
    [DllImport(Lib)] internal static extern float* b200_lm_grads_device(IntPtr h);
    [DllImport(Lib)] internal static extern int b200_lm_set_optimizer(IntPtr h, int kind, float beta1, float beta2, float eps);
    [DllImport(Lib)] internal static extern int b200_lm_train_step_discrete(IntPtr h, int* tokens, int* seq_offsets, int n_seq, float lr, int use_clip, float clip_threshold, int do_step, float* loss, float* grad_norm, int* valid_count);
    [DllImport(Lib)] internal static extern int b200_lm_train_step_continuous(IntPtr h, float* features, float* reg_targets, int* class_targets, int* seq_offsets, int n_seq, float lr, int use_clip, float clip_threshold, int do_step, float* loss, float* grad_norm, int* valid_count);
    [DllImport(Lib)] internal static extern int b200_lm_batch_create_discrete(IntPtr h, int* tokens, int* seq_offsets, int n_seq, out IntPtr @out);
    [DllImport(Lib)] internal static extern int b200_lm_batch_create_continuous(IntPtr h, float* features, float* reg_targets, int* class_targets, int* seq_offsets, int n_seq, out IntPtr @out);
    [DllImport(Lib)] internal static extern int b200_lm_batch_destroy(IntPtr h);
    [DllImport(Lib)] internal static extern int b200_lm_accumulate_batch(IntPtr h, IntPtr a1, float* loss_sum, int* valid_count);
    [DllImport(Lib)] internal static extern int b200_lm_train_step_batch(IntPtr h, IntPtr a1, float lr, int use_clip, float clip_threshold, int do_step, float* loss, float* grad_norm, int* valid_count);
    [DllImport(Lib)] internal static extern int b200_lm_set_grad_ready_callback(IntPtr h, GradReadyFn @fn, IntPtr user);
    [DllImport(Lib)] internal static extern int b200_lm_zero_grads(IntPtr h);
    [DllImport(Lib)] internal static extern int b200_lm_accumulate_discrete(IntPtr h, int* tokens, int* seq_offsets, int n_seq, float* loss_sum, int* valid_count);
    [DllImport(Lib)] internal static extern int b200_lm_accumulate_continuous(IntPtr h, float* features, float* reg_targets, int* class_targets, int* seq_offsets, int n_seq, float* loss_sum, int* valid_count);
    [DllImport(Lib)] internal static extern int b200_lm_apply_step(IntPtr h, int global_valid_count, float lr, int use_clip, float clip_threshold, int do_step, float* grad_norm);
    [DllImport(Lib)] internal static extern int b200_lm_validate_discrete(IntPtr h, int* tokens, int* seq_offsets, int n_seq, float* mean_loss, int* items);
    [DllImport(Lib)] internal static extern int b200_lm_validate_continuous(IntPtr h, float* features, float* reg_targets, int* class_targets, int* seq_offsets, int n_seq, float* mean_loss, int* items);
    [DllImport(Lib)] internal static extern int b200_lm_download_optimizer_state(IntPtr h, int which, float* host, long offset, long count);
    [DllImport(Lib)] internal static extern int b200_lm_upload_optimizer_state(IntPtr h, int which, float* host, long offset, long count);
    [DllImport(Lib)] internal static extern int b200_lm_get_step_index(IntPtr h, int* step_index);
    [DllImport(Lib)] internal static extern int b200_lm_set_step_index(IntPtr h, int step_index);
    [DllImport(Lib)] internal static extern int b200_lm_gen_create(IntPtr h, int max_len, out IntPtr @out);
    [DllImport(Lib)] internal static extern int b200_lm_gen_destroy(IntPtr h);
    [DllImport(Lib)] internal static extern int b200_lm_gen_reset(IntPtr h);
    [DllImport(Lib)] internal static extern int b200_lm_gen_length(IntPtr h, int* length);
    [DllImport(Lib)] internal static extern int b200_lm_gen_step(IntPtr h, int token_id, float* logits);
    [DllImport(Lib)] internal static extern int b200_lm_gen_greedy(IntPtr h, int* prompt, int n_prompt, int max_new, int* out_tokens, int* n_out);
    [DllImport(Lib)] internal static extern int b200_lm_gen_graph_nodes(IntPtr h, int* nodes);
    [DllImport(Lib)] internal static extern int b200_lm_gen_single_kernel(IntPtr h);
    [DllImport(Lib)] internal static extern int b200_lm_gen_set_single_kernel(IntPtr h, int on);
    [DllImport(Lib)] internal static extern int b200_lm_get_timings(IntPtr h, float* ms4);
    [DllImport(Lib)] internal static extern int b200_dp_set_nccl_library(byte* path);
    [DllImport(Lib)] internal static extern int b200_dp_set_nccl_max_ctas(int n);
    [DllImport(Lib)] internal static extern int b200_dp_unique_id(byte* id128);
    [DllImport(Lib)] internal static extern int b200_dp_create_rank(IntPtr lm, byte* id128, int rank, int world, out IntPtr @out);
    [DllImport(Lib)] internal static extern int b200_dp_destroy(IntPtr h);
    [DllImport(Lib)] internal static extern int b200_dp_shard(int n_seq, int rank, int world, int* lo, int* hi);
    [DllImport(Lib)] internal static extern int b200_dp_set_deadline_ms(IntPtr h, int milliseconds);
    [DllImport(Lib)] internal static extern int b200_dp_broadcast_params(IntPtr h, int root);
    [DllImport(Lib)] internal static extern int b200_dp_train_step_discrete(IntPtr h, int* tokens, int* seq_offsets, int n_seq, float lr, int use_clip, float clip_threshold, int do_step, float* loss, float* grad_norm, int* valid_count);
    [DllImport(Lib)] internal static extern int b200_dp_train_step_continuous(IntPtr h, float* features, float* reg_targets, int* class_targets, int* seq_offsets, int n_seq, float lr, int use_clip, float clip_threshold, int do_step, float* loss, float* grad_norm, int* valid_count);
    [DllImport(Lib)] internal static extern int b200_dp_batch_create_discrete(IntPtr h, int* tokens, int* seq_offsets, int n_seq, out IntPtr @out);
    [DllImport(Lib)] internal static extern int b200_dp_batch_create_continuous(IntPtr h, float* features, float* reg_targets, int* class_targets, int* seq_offsets, int n_seq, out IntPtr @out);
    [DllImport(Lib)] internal static extern int b200_dp_train_step_batch(IntPtr h, IntPtr shard, float lr, int use_clip, float clip_threshold, int do_step, float* loss, float* grad_norm, int* valid_count);
    [DllImport(Lib)] internal static extern int b200_dp_get_timings(IntPtr h, float* ms2);
    [DllImport(Lib)] internal static extern int b200_dp_group_create(int* devices, int n_devices, ref LmConfig cfg, int max_rows_per_pass, int gemm_mode, out IntPtr @out);
    [DllImport(Lib)] internal static extern int b200_dp_group_destroy(IntPtr h);
    [DllImport(Lib)] internal static extern IntPtr b200_dp_group_last_error(IntPtr h);
    [DllImport(Lib)] internal static extern int b200_dp_group_size(IntPtr h);
    [DllImport(Lib)] internal static extern IntPtr b200_dp_group_trainer(IntPtr h, int rank);
    [DllImport(Lib)] internal static extern int b200_dp_group_set_optimizer(IntPtr h, int kind, float beta1, float beta2, float eps);
    [DllImport(Lib)] internal static extern int b200_dp_group_upload_params(IntPtr h, float* host, long offset, long count);
    [DllImport(Lib)] internal static extern int b200_dp_group_train_step_discrete(IntPtr h, int* tokens, int* seq_offsets, int n_seq, float lr, int use_clip, float clip_threshold, int do_step, float* loss, float* grad_norm, int* valid_count);
    [DllImport(Lib)] internal static extern int b200_dp_group_train_step_continuous(IntPtr h, float* features, float* reg_targets, int* class_targets, int* seq_offsets, int n_seq, float lr, int use_clip, float clip_threshold, int do_step, float* loss, float* grad_norm, int* valid_count);
    [DllImport(Lib)] internal static extern int b200_mlp_create(IntPtr h, int nLayers, int* widths, int* activations, int cost, float huber_delta, float l2_lambda, float clip_threshold, int max_batch, out IntPtr @out);
    [DllImport(Lib)] internal static extern int b200_mlp_destroy(IntPtr h);
    [DllImport(Lib)] internal static extern int b200_mlp_upload_layer(IntPtr h, int layer, float* weights, float* biases);
    [DllImport(Lib)] internal static extern int b200_mlp_download_layer(IntPtr h, int layer, float* weights, float* biases);
    [DllImport(Lib)] internal static extern int b200_mlp_learn_batch(IntPtr h, float* X, float* Y, int B, float lr, float* in_min, float* in_max, float* delta_norm);
    }

    public sealed unsafe class CudaB200AccelerationManager : IAccelerationManager, IB200TrainStep, IB200MlpBatch, IDisposable
    {
        readonly IntPtr _ctx;
        readonly AccelerationCPU _cpu = new AccelerationCPU();
        IntPtr _lm = IntPtr.Zero;
        long _paramCount;
        bool _disposed;

        public CudaB200AccelerationManager(int deviceId = 0)
        {
            int rc = Native.b200_create(deviceId, out _ctx);
            if (rc != 0) throw new InvalidOperationException($"b200_create(device {deviceId}) failed with status {rc}: a CUDA device is required, there is no CPU fallback.");
        }

        public void Dispose()
        {
            if (_disposed) return;
            _disposed = true;
            if (_lm != IntPtr.Zero) Native.b200_lm_destroy(_lm);   // handles are reference counted in the library: any order is safe
            Native.b200_destroy(_ctx);
        }

        // ---- status -> exception, with the reference's types
        void Check(int rc)
        {
            if (rc == 0) return;
            string msg = Marshal.PtrToStringUTF8(Native.b200_last_error(_ctx)) ?? "";
            switch (rc)
            {
                case 1: case 2: throw new ArgumentException(msg);                   // B200_ERR_INVALID_ARG, B200_ERR_SHAPE
                case 3: throw new ArgumentOutOfRangeException(null, msg);           // B200_ERR_OUT_OF_RANGE
                case 8: throw new NotSupportedException(msg);                       // B200_ERR_UNSUPPORTED
                case 6: throw new TimeoutException(msg);                            // B200_ERR_TIMEOUT
                default: throw new InvalidOperationException($"b200 status {rc}: {msg}");   // CUDA, NCCL, PEER
            }
        }

        static void NotNull(object o, string name) { if (o == null) throw new ArgumentNullException(name); }
        static int B(bool v) => v ? 1 : 0;

        static float[][,] Unflatten(float[] flat, int heads, int q, int k)
        {
            var r = new float[heads][,];
            for (int h = 0; h < heads; h++)
            {
                r[h] = new float[q, k];
                Buffer.BlockCopy(flat, h * q * k * sizeof(float), r[h], 0, q * k * sizeof(float));
            }
            return r;
        }

        static float[] Flatten(float[][,] a, int heads, int q, int k)
        {
            var flat = new float[(long)heads * q * k];
            for (int h = 0; h < heads; h++)
            {
                if (a[h] == null || a[h].GetLength(0) != q || a[h].GetLength(1) != k) throw new ArgumentException("attentionWeights has ragged heads");
                Buffer.BlockCopy(a[h], 0, flat, h * q * k * sizeof(float), q * k * sizeof(float));
            }
            return flat;
        }

        // =====================================================================================  shared tensor primitives
        public float[,] MatrixMultiply(float[,] A, float[,] B)
        {
            NotNull(A, nameof(A)); NotNull(B, nameof(B));
            var C = new float[A.GetLength(0), B.GetLength(1)];
            fixed (float* a = A, b = B, c = C)
                Check(Native.b200_MatrixMultiply(_ctx, a, A.GetLength(0), A.GetLength(1), b, B.GetLength(0), B.GetLength(1), c));
            return C;
        }

        public float[,] MatrixMultiplyTranspose(float[,] A, float[,] B)
        {
            NotNull(A, nameof(A)); NotNull(B, nameof(B));
            var C = new float[A.GetLength(0), B.GetLength(0)];
            fixed (float* a = A, b = B, c = C)
                Check(Native.b200_MatrixMultiplyTranspose(_ctx, a, A.GetLength(0), A.GetLength(1), b, B.GetLength(0), B.GetLength(1), c));
            return C;
        }

        public float[,] BatchDotProductAddBias(float[,] weights, float[,] inputMatrix, float[] bias)
        {
            NotNull(inputMatrix, nameof(inputMatrix));
            return BatchDotProductAddBias(weights, inputMatrix, 0, inputMatrix.GetLength(0), bias);
        }

        public float[,] BatchDotProductAddBias(float[,] weights, float[,] inputMatrix, int rowStart, int rowCount, float[] bias)
        {
            NotNull(weights, nameof(weights)); NotNull(inputMatrix, nameof(inputMatrix)); NotNull(bias, nameof(bias));
            if (rowCount < 0) throw new ArgumentOutOfRangeException(nameof(rowCount));
            var Y = new float[rowCount, weights.GetLength(0)];
            fixed (float* w = weights, x = inputMatrix, b = bias, y = Y)
                Check(Native.b200_BatchDotProductAddBias(_ctx, w, weights.GetLength(0), weights.GetLength(1), x, inputMatrix.GetLength(0), inputMatrix.GetLength(1),
                                                         rowStart, rowCount, b, bias.Length, y));
            return Y;
        }

        public void ZeroMatrix(float[,] matrix) { NotNull(matrix, nameof(matrix)); fixed (float* p = matrix) Check(Native.b200_ZeroMatrix(_ctx, p, matrix.LongLength)); }
        public void ZeroVector(float[] vector) { NotNull(vector, nameof(vector)); fixed (float* p = vector) Check(Native.b200_ZeroVector(_ctx, p, vector.LongLength)); }

        public void MatrixAddInPlace(float[,] target, float[,] addend)
        {
            NotNull(target, nameof(target)); NotNull(addend, nameof(addend));
            if (target.GetLength(0) != addend.GetLength(0) || target.GetLength(1) != addend.GetLength(1)) throw new ArgumentException("Matrix dimensions must match.");
            fixed (float* t = target, a = addend) Check(Native.b200_MatrixAddInPlace(_ctx, t, a, target.LongLength));
        }

        public void VectorAccumulate(float[] target, float[] source)
        {
            NotNull(target, nameof(target)); NotNull(source, nameof(source));
            if (target.Length != source.Length) throw new ArgumentException("Vector lengths must match.");
            fixed (float* t = target, s = source) Check(Native.b200_VectorAccumulate(_ctx, t, s, target.LongLength));
        }

        // small host-side utilities: no device work to win
        public float[,] MatrixScale(float[,] matrix, float scalar) => _cpu.MatrixScale(matrix, scalar);
        public float[,] MatrixAdd(float[,] A, float[,] B) => _cpu.MatrixAdd(A, B);
        public float[,] MatrixAddBias(float[,] matrix, float[] bias) => _cpu.MatrixAddBias(matrix, bias);
        public float[,] BatchDotProduct(float[,] weights, float[,] inputMatrix) => _cpu.BatchDotProduct(weights, inputMatrix);
        public float[,] BatchDotProduct(float[,] weights, float[,] inputMatrix, int rowStart, int rowCount) => _cpu.BatchDotProduct(weights, inputMatrix, rowStart, rowCount);
        public float[,] SliceRows(float[,] matrix, int startRow, int endRow) => _cpu.SliceRows(matrix, startRow, endRow);
        public float[] ExtractRow(float[,] matrix, int rowIndex, int cols) => _cpu.ExtractRow(matrix, rowIndex, cols);
        public void SetRow(float[,] matrix, int rowIndex, float[] values, int cols) => _cpu.SetRow(matrix, rowIndex, values, cols);

        // =====================================================================================  per-sample neural network (not on the batch path)
        public float[] CalculateDotProduct(float[,] matrix, float[] vector) => _cpu.CalculateDotProduct(matrix, vector);
        public (float[] activation, float[] derivative) ActivateLayer(float[] dot, float[] bias, ActivationType activationType) => _cpu.ActivateLayer(dot, bias, activationType);
        public float[] CalculateOutputGradients(float[] cost, float[] derivative) => _cpu.CalculateOutputGradients(cost, derivative);
        public float[] CalculateHiddenGradients(float[,] weights, float[] nextDeltas, float[] derivative) => _cpu.CalculateHiddenGradients(weights, nextDeltas, derivative);
        public float[,] UpdateWeights(float[,] weights, float[] deltas, float[] prevActivations, float learningRate, float lambda) => _cpu.UpdateWeights(weights, deltas, prevActivations, learningRate, lambda);
        public float[] UpdateBias(float[] bias, float[] deltas, float learningRate) => _cpu.UpdateBias(bias, deltas, learningRate);

        // =====================================================================================  transformer core
        public float[,] Softmax(float[,] matrix, bool[,] mask = null) => _cpu.Softmax(matrix, mask);
        public bool[,] CreateCausalMask(int seqLen) => _cpu.CreateCausalMask(seqLen);

        (float[,] output, float[] means, float[] variances, float[,] normalized, float[,] residual) LayerNormCore(
            float[,] input, float[,] subLayer, float[] gamma, float[] beta, float epsilon, bool wantStats, bool wantResidual)
        {
            NotNull(input, nameof(input)); NotNull(gamma, nameof(gamma)); NotNull(beta, nameof(beta));
            int rows = input.GetLength(0), f = input.GetLength(1);
            if (subLayer != null && (subLayer.GetLength(0) != rows || subLayer.GetLength(1) != f)) throw new ArgumentException("subLayer must have the shape of input.");
            var output = new float[rows, f];
            float[] means = wantStats ? new float[rows] : null, variances = wantStats ? new float[rows] : null;
            float[,] normalized = wantStats ? new float[rows, f] : null, residual = wantResidual ? new float[rows, f] : null;
            fixed (float* x = input, s = subLayer, g = gamma, b = beta, o = output, m = means, v = variances, n = normalized, r = residual)   // a null array pins to a null pointer
                Check(Native.b200_ResidualLayerNormForward(_ctx, x, s, g, b, rows, f, epsilon, o, m, v, n, r));
            return (output, means, variances, normalized, residual);
        }

        public float[,] LayerNorm(float[,] input, float[] gamma, float[] beta, float epsilon = 1e-5f) => LayerNormCore(input, null, gamma, beta, epsilon, false, false).output;

        public (float[,] output, float[] means, float[] variances, float[,] normalized) LayerNormForward(float[,] input, float[] gamma, float[] beta, float epsilon = 1e-5f)
        {
            var r = LayerNormCore(input, null, gamma, beta, epsilon, true, false);
            return (r.output, r.means, r.variances, r.normalized);
        }

        public float[,] ResidualLayerNorm(float[,] input, float[,] subLayer, float[] gamma, float[] beta, float epsilon = 1e-5f)
        {
            NotNull(subLayer, nameof(subLayer));
            return LayerNormCore(input, subLayer, gamma, beta, epsilon, false, false).output;
        }

        public (float[,] output, float[] means, float[] variances, float[,] normalized, float[,] residual) ResidualLayerNormForward(
            float[,] input, float[,] subLayer, float[] gamma, float[] beta, float epsilon = 1e-5f)
        {
            NotNull(subLayer, nameof(subLayer));
            return LayerNormCore(input, subLayer, gamma, beta, epsilon, true, true);
        }

        public (float[,] dInput, float[] dGamma, float[] dBeta) LayerNormBackward(float[,] dOut, float[,] normalized, float[] gamma, float[,] input, float[] mean,
                                                                                 float[] variance, float epsilon = 1e-5f)
        {
            NotNull(dOut, nameof(dOut)); NotNull(normalized, nameof(normalized)); NotNull(gamma, nameof(gamma)); NotNull(input, nameof(input));
            NotNull(mean, nameof(mean)); NotNull(variance, nameof(variance));
            int rows = dOut.GetLength(0), f = dOut.GetLength(1);
            var dIn = new float[rows, f]; var dG = new float[f]; var dB = new float[f];   // all three are assigned (AccelerationCPU.cs:1516-1564)
            fixed (float* pd = dOut, pn = normalized, pg = gamma, px = input, pm = mean, pv = variance, o1 = dIn, o2 = dG, o3 = dB)
                Check(Native.b200_LayerNormBackward(_ctx, pd, pn, pg, px, pm, pv, rows, f, epsilon, o1, o2, o3));
            return (dIn, dG, dB);
        }

        public float[,] MultiHeadAttentionForward(float[,] Q, float[,] K, float[,] V, int numHeads, float scale, bool[,] mask = null)
        {
            NotNull(Q, nameof(Q)); NotNull(K, nameof(K)); NotNull(V, nameof(V));
            int q = Q.GetLength(0), k = K.GetLength(0), e = Q.GetLength(1);
            var output = new float[q, e];
            fixed (float* pq = Q, pk = K, pv = V, po = output)
            fixed (bool* pm = mask)   // bool[,] stores one byte per element: non-zero = visible
                Check(Native.b200_MultiHeadAttentionForward(_ctx, pq, pk, pv, q, k, e, numHeads, scale, (byte*)pm, po));
            return output;
        }

        public float[,] ScaledDotProductAttention(float[,] q, float[,] k, float[,] v, int numHeads, bool[,] mask = null, bool causal = false)
        {
            NotNull(q, nameof(q)); NotNull(k, nameof(k)); NotNull(v, nameof(v));
            int ql = q.GetLength(0), kl = k.GetLength(0), e = q.GetLength(1);
            if (causal && ql != kl) throw new ArgumentException("Causal attention requires queryLen == keyLen.");   // AccelerationCPU.cs:1859-1862
            var output = new float[ql, e];
            fixed (float* pq = q, pk = k, pv = v, po = output)
            fixed (bool* pm = mask)
                Check(Native.b200_ScaledDotProductAttention(_ctx, pq, pk, pv, ql, kl, e, numHeads, (byte*)pm, B(causal), po));
            return output;
        }

        (float[,] dQ, float[,] dK, float[,] dV) AttentionBackwardCore(float[,] Q, float[,] K, float[,] V, float[,] dConcatenated, int numHeads, float scale, bool[,] mask, bool decoder)
        {
            NotNull(Q, nameof(Q)); NotNull(K, nameof(K)); NotNull(V, nameof(V)); NotNull(dConcatenated, nameof(dConcatenated));
            int ql = Q.GetLength(0), kl = K.GetLength(0), e = Q.GetLength(1);
            var dQ = new float[ql, e]; var dK = new float[kl, e]; var dV = new float[kl, e];   // fresh: assigned by the library
            fixed (float* pq = Q, pk = K, pv = V, pd = dConcatenated, oq = dQ, ok = dK, ov = dV)
            fixed (bool* pm = mask)
                Check(Native.b200_MultiHeadAttentionBackward(_ctx, pq, pk, pv, pd, ql, kl, e, numHeads, scale, (byte*)pm, B(decoder), oq, ok, ov));
            return (dQ, dK, dV);
        }

        public (float[,] dQ, float[,] dK, float[,] dV) MultiHeadAttentionBackward(float[,] Q, float[,] K, float[,] V, float[,] dConcatenated, int numHeads, float scale, bool useDecoderMask = false)
            => AttentionBackwardCore(Q, K, V, dConcatenated, numHeads, scale, null, useDecoderMask);

        public (float[,] dQ, float[,] dK, float[,] dV) MultiHeadAttentionBackward(float[,] Q, float[,] K, float[,] V, float[,] dConcatenated, int numHeads, float scale, bool[,] mask)
            => AttentionBackwardCore(Q, K, V, dConcatenated, numHeads, scale, mask, false);

        /// <summary>The reference special-cases a delegate whose target is a NeuralNetwork (AccelerationCPU.cs:1975-1985); that case
        /// runs on the device with the network's own layers, any other delegate is called row by row like the reference does.</summary>
        public float[,] FFNForwardBatch(float[,] input, int seqLen, int outputDim, Func<float[], float[]> forwardPassFn)
        {
            NotNull(input, nameof(input)); NotNull(forwardPassFn, nameof(forwardPassFn));
            if (!(forwardPassFn.Target is NeuralNetwork nn)) return _cpu.FFNForwardBatch(input, seqLen, outputDim, forwardPassFn);
            Data data = nn.GetInternalData();
            int n = data.layers.Length;
            var widths = new int[n]; var acts = new int[n];
            for (int l = 0; l < n; l++) { widths[l] = data.layers[l].Size; acts[l] = (int)data.layers[l].ActivationType; }
            var output = new float[seqLen, outputDim];
            var handles = new List<GCHandle>();
            try
            {
                float** w = stackalloc float*[n]; float** b = stackalloc float*[n];
                w[0] = null; b[0] = null;
                for (int l = 1; l < n; l++)
                {
                    var hw = GCHandle.Alloc(data.layers[l].Weights, GCHandleType.Pinned); handles.Add(hw);
                    var hb = GCHandle.Alloc(data.layers[l].Biases, GCHandleType.Pinned); handles.Add(hb);
                    w[l] = (float*)hw.AddrOfPinnedObject(); b[l] = (float*)hb.AddrOfPinnedObject();
                }
                fixed (float* x = input, o = output)
                fixed (int* pw = widths, pa = acts)
                    Check(Native.b200_FFNForwardBatch(_ctx, x, seqLen, n, pw, pa, w, b, o));
            }
            finally { foreach (var h in handles) h.Free(); }
            return output;
        }

        public (float[,] Q, float[,] K, float[,] V) ProjectQKV(float[,] input, float[,] WQ, float[] biasQ, float[,] WK, float[] biasK, float[,] WV, float[] biasV)
        {
            NotNull(input, nameof(input)); NotNull(WQ, nameof(WQ)); NotNull(WK, nameof(WK)); NotNull(WV, nameof(WV));
            NotNull(biasQ, nameof(biasQ)); NotNull(biasK, nameof(biasK)); NotNull(biasV, nameof(biasV));
            int rows = input.GetLength(0), inDim = input.GetLength(1), outDim = WQ.GetLength(0);
            var Q = new float[rows, outDim]; var K = new float[rows, outDim]; var V = new float[rows, outDim];
            fixed (float* x = input, wq = WQ, bq = biasQ, wk = WK, bk = biasK, wv = WV, bv = biasV, oq = Q, ok = K, ov = V)
                Check(Native.b200_ProjectQKV(_ctx, x, rows, inDim, wq, bq, wk, bk, wv, bv, outDim, oq, ok, ov));
            return (Q, K, V);
        }

        public float[,] BackpropQKV(float[,] input, float[,] dQ, float[,] dK, float[,] dV, float[,] WQ, float[,] WK, float[,] WV, float[,] WQGrad, float[] biasQGrad,
                                    float[,] WKGrad, float[] biasKGrad, float[,] WVGrad, float[] biasVGrad)
        {
            NotNull(input, nameof(input)); NotNull(dQ, nameof(dQ)); NotNull(dK, nameof(dK)); NotNull(dV, nameof(dV));
            int rows = input.GetLength(0), inDim = input.GetLength(1), outDim = dQ.GetLength(1);
            var dInput = new float[rows, inDim];   // assigned; the six gradients accumulate (AccelerationCPU.cs:2071-2182)
            fixed (float* x = input, q = dQ, k = dK, v = dV, wq = WQ, wk = WK, wv = WV, gq = WQGrad, bq = biasQGrad, gk = WKGrad, bk = biasKGrad, gv = WVGrad, bv = biasVGrad, o = dInput)
                Check(Native.b200_BackpropQKV(_ctx, x, rows, inDim, q, k, v, outDim, wq, wk, wv, gq, bq, gk, bk, gv, bv, o));
            return dInput;
        }

        public (float[,] K, float[,] V) ProjectKV(float[,] input, float[,] WK, float[] biasK, float[,] WV, float[] biasV)
        {
            NotNull(input, nameof(input)); NotNull(WK, nameof(WK)); NotNull(WV, nameof(WV)); NotNull(biasK, nameof(biasK)); NotNull(biasV, nameof(biasV));
            int rows = input.GetLength(0), inDim = input.GetLength(1), outDim = WK.GetLength(0);
            var K = new float[rows, outDim]; var V = new float[rows, outDim];
            fixed (float* x = input, wk = WK, bk = biasK, wv = WV, bv = biasV, ok = K, ov = V)
                Check(Native.b200_ProjectKV(_ctx, x, rows, inDim, wk, bk, wv, bv, outDim, ok, ov));
            return (K, V);
        }

        public float[,] BackpropKV(float[,] input, float[,] dK, float[,] dV, float[,] WK, float[,] WV, float[,] WKGrad, float[] biasKGrad, float[,] WVGrad, float[] biasVGrad)
        {
            NotNull(input, nameof(input)); NotNull(dK, nameof(dK)); NotNull(dV, nameof(dV));
            int rows = input.GetLength(0), inDim = input.GetLength(1), outDim = dK.GetLength(1);
            var dInput = new float[rows, inDim];
            fixed (float* x = input, k = dK, v = dV, wk = WK, wv = WV, gk = WKGrad, bk = biasKGrad, gv = WVGrad, bv = biasVGrad, o = dInput)
                Check(Native.b200_BackpropKV(_ctx, x, rows, inDim, k, v, outDim, wk, wv, gk, bk, gv, bv, o));
            return dInput;
        }

        // =====================================================================================  transformer training
        public void BackpropLinearProjection(float[,] input, float[,] dOutput, float[,] weights, float[,] weightGrad, float[] biasGrad, float[,] dInput)
        {
            NotNull(input, nameof(input)); NotNull(dOutput, nameof(dOutput)); NotNull(weights, nameof(weights));
            NotNull(weightGrad, nameof(weightGrad)); NotNull(biasGrad, nameof(biasGrad)); NotNull(dInput, nameof(dInput));
            fixed (float* x = input, dy = dOutput, w = weights, wg = weightGrad, bg = biasGrad, di = dInput)   // all three outputs accumulate (AccelerationCPU.cs:2188-2229)
                Check(Native.b200_BackpropLinearProjection(_ctx, x, dy, w, input.GetLength(0), input.GetLength(1), dOutput.GetLength(1), wg, bg, di));
        }

        public float[,] BackpropOutputProjection(float[,] dLogits, float[,] input, float[,] weights, float[,] weightGrad, float[] biasGrad, int seqLen, int outputDim, int embeddingDim)
        {
            NotNull(dLogits, nameof(dLogits)); NotNull(input, nameof(input)); NotNull(weights, nameof(weights)); NotNull(weightGrad, nameof(weightGrad)); NotNull(biasGrad, nameof(biasGrad));
            var dX = new float[seqLen, embeddingDim];   // assigned; the two gradients accumulate
            fixed (float* dl = dLogits, x = input, w = weights, wg = weightGrad, bg = biasGrad, o = dX)
                Check(Native.b200_BackpropOutputProjection(_ctx, dl, x, w, wg, bg, seqLen, outputDim, embeddingDim, o));
            return dX;
        }

        public void BackpropInputProjection(float[,] dX, float[,] continuousInput, float[,] weightGrad, float[] biasGrad, int seqLen, int embeddingDim, int inputFeatureDim)
            => BackpropInputProjection(dX, continuousInput, 0, weightGrad, biasGrad, seqLen, embeddingDim, inputFeatureDim);

        public void BackpropInputProjection(float[,] dX, float[,] continuousInput, int inputRowStart, float[,] weightGrad, float[] biasGrad, int seqLen, int embeddingDim, int inputFeatureDim)
        {
            NotNull(dX, nameof(dX)); NotNull(continuousInput, nameof(continuousInput)); NotNull(weightGrad, nameof(weightGrad)); NotNull(biasGrad, nameof(biasGrad));
            fixed (float* d = dX, c = continuousInput, wg = weightGrad, bg = biasGrad)
                Check(Native.b200_BackpropInputProjection(_ctx, d, dX.GetLength(0), dX.GetLength(1), c, continuousInput.GetLength(0), continuousInput.GetLength(1), inputRowStart,
                                                          wg, bg, seqLen, embeddingDim, inputFeatureDim));
        }

        public void AccumulateTokenEmbeddingGrad(float[,] embeddingGrad, float[,] dX, int[] tokenIds, int seqLen, int embeddingDim)
            => AccumulateTokenEmbeddingGrad(embeddingGrad, dX, tokenIds, 0, seqLen, embeddingDim);

        public void AccumulateTokenEmbeddingGrad(float[,] embeddingGrad, float[,] dX, int[] tokenIds, int tokenStart, int seqLen, int embeddingDim)
        {
            NotNull(embeddingGrad, nameof(embeddingGrad)); NotNull(dX, nameof(dX)); NotNull(tokenIds, nameof(tokenIds));
            fixed (float* eg = embeddingGrad, d = dX)
            fixed (int* ids = tokenIds)
                Check(Native.b200_AccumulateTokenEmbeddingGrad(_ctx, eg, embeddingGrad.GetLength(0), d, ids, tokenIds.Length, tokenStart, seqLen, embeddingDim));
        }

        public (float loss, float[,] dLogits) CrossEntropyLossAndGradient(float[,] logits, int[] targets, int effectiveLen) => CrossEntropyLossAndGradient(logits, targets, 0, effectiveLen);

        public (float loss, float[,] dLogits) CrossEntropyLossAndGradient(float[,] logits, int[] targets, int targetStart, int effectiveLen)
        {
            NotNull(logits, nameof(logits)); NotNull(targets, nameof(targets));
            int rows = logits.GetLength(0), outDim = logits.GetLength(1);
            var dLogits = new float[rows, outDim];
            float loss = 0f;
            fixed (float* l = logits, d = dLogits)
            fixed (int* t = targets)
                Check(Native.b200_CrossEntropyLossAndGradient(_ctx, l, rows, outDim, t, targets.Length, targetStart, effectiveLen, &loss, d));
            return (loss, dLogits);
        }

        public (float loss, float[,] dOutput) MSELossAndGradient(float[,] predictions, float[,] targets, int effectiveLen) => MSELossAndGradient(predictions, targets, 0, effectiveLen);

        public (float loss, float[,] dOutput) MSELossAndGradient(float[,] predictions, float[,] targets, int targetStart, int effectiveLen)
        {
            NotNull(predictions, nameof(predictions)); NotNull(targets, nameof(targets));
            int rows = predictions.GetLength(0), outDim = predictions.GetLength(1);
            var dOutput = new float[rows, outDim];
            float loss = 0f;
            fixed (float* p = predictions, t = targets, d = dOutput)
                Check(Native.b200_MSELossAndGradient(_ctx, p, rows, outDim, t, targets.GetLength(0), targetStart, effectiveLen, &loss, d));
            return (loss, dOutput);
        }

        public float MatrixSquaredNorm(float[,] matrix) { NotNull(matrix, nameof(matrix)); float r = 0f; fixed (float* p = matrix) Check(Native.b200_MatrixSquaredNorm(_ctx, p, matrix.LongLength, &r)); return r; }
        public float VectorSquaredNorm(float[] vector) { NotNull(vector, nameof(vector)); float r = 0f; fixed (float* p = vector) Check(Native.b200_VectorSquaredNorm(_ctx, p, vector.LongLength, &r)); return r; }
        public void MatrixScaleInPlace(float[,] matrix, float scale) { NotNull(matrix, nameof(matrix)); fixed (float* p = matrix) Check(Native.b200_MatrixScaleInPlace(_ctx, p, matrix.LongLength, scale)); }
        public void VectorScaleInPlace(float[] vector, float scale) { NotNull(vector, nameof(vector)); fixed (float* p = vector) Check(Native.b200_VectorScaleInPlace(_ctx, p, vector.LongLength, scale)); }

        public void MatrixUpdate(float[,] weights, float[,] gradients, float learningRate)
        {
            NotNull(weights, nameof(weights)); NotNull(gradients, nameof(gradients));
            if (weights.GetLength(0) != gradients.GetLength(0) || weights.GetLength(1) != gradients.GetLength(1)) throw new ArgumentException("Matrix dimensions must match.");
            fixed (float* w = weights, g = gradients) Check(Native.b200_MatrixUpdate(_ctx, w, g, weights.LongLength, learningRate));
        }

        public void VectorUpdate(float[] weights, float[] gradients, float learningRate)
        {
            NotNull(weights, nameof(weights)); NotNull(gradients, nameof(gradients));
            if (weights.Length != gradients.Length) throw new ArgumentException("Vector lengths must match.");
            fixed (float* w = weights, g = gradients) Check(Native.b200_VectorUpdate(_ctx, w, g, weights.LongLength, learningRate));
        }

        // =====================================================================================  sibling trainers' operators
        public void ApplyContextTypeEmbedding(float[,] contextHidden, float[,] typeEmbedding, int[] typeIndices)
        {
            NotNull(contextHidden, nameof(contextHidden)); NotNull(typeEmbedding, nameof(typeEmbedding)); NotNull(typeIndices, nameof(typeIndices));
            fixed (float* c = contextHidden, t = typeEmbedding)
            fixed (int* i = typeIndices)
                Check(Native.b200_ApplyContextTypeEmbedding(_ctx, c, contextHidden.GetLength(0), contextHidden.GetLength(1), t, typeEmbedding.GetLength(0), i));
        }

        public float[,] ComputeTimeDiffMatrix(int priceSeqLen, float[] keyArrivalTimes)
        {
            NotNull(keyArrivalTimes, nameof(keyArrivalTimes));
            var r = new float[priceSeqLen, keyArrivalTimes.Length];
            fixed (float* k = keyArrivalTimes, o = r) Check(Native.b200_ComputeTimeDiffMatrix(_ctx, priceSeqLen, k, keyArrivalTimes.Length, o));
            return r;
        }

        public float[] ComputeMemoryAttentionScores(float[,] priceHidden, int lastPos, float[,] contextHidden, int totalCtx, float scale)
        {
            NotNull(priceHidden, nameof(priceHidden)); NotNull(contextHidden, nameof(contextHidden));
            var scores = new float[totalCtx];
            fixed (float* p = priceHidden, c = contextHidden, s = scores)
                Check(Native.b200_ComputeMemoryAttentionScores(_ctx, p, priceHidden.GetLength(0), priceHidden.GetLength(1), lastPos, c, totalCtx, scale, s));
            return scores;
        }

        public float[,] ProjectOutputBatch(float[,] hidden, float[,] outputProjection, float[] outputBias, int seqLen, int outputDim)
        {
            NotNull(hidden, nameof(hidden)); NotNull(outputProjection, nameof(outputProjection)); NotNull(outputBias, nameof(outputBias));
            var pred = new float[seqLen, outputDim];
            fixed (float* h = hidden, w = outputProjection, b = outputBias, o = pred)
                Check(Native.b200_ProjectOutputBatch(_ctx, h, hidden.GetLength(0), hidden.GetLength(1), w, b, seqLen, outputDim, o));
            return pred;
        }

        // these two take the TACAMT model objects themselves (decay network, block caches): that model family's own code
        public (float[,,] decayBias, ContentAwareDecayCache cache) ContentAwareDecayForward(float[,] queryEmbeddings, float[,] keyEmbeddings, float[,] timeDiffs, float[] keyTimesFromRef,
            ContentAwareDecayNetwork network, bool isTraining = false, Random dropoutRng = null)
            => _cpu.ContentAwareDecayForward(queryEmbeddings, keyEmbeddings, timeDiffs, keyTimesFromRef, network, isTraining, dropoutRng);

        public float[,] ContentAwareCrossAttentionWithCache(float[,] Q, float[,] K, float[,] V, float[,] timeDiffs, float[] keyTimesFromRef, float[,] queryEmbeddings, float[,] keyEmbeddings,
            TacamtBlock block, BlockCache bc, int PriceEmbeddingDim, int PriceNumHeads, bool enableDecayBias = true, bool isTraining = false, Random dropoutRng = null)
            => _cpu.ContentAwareCrossAttentionWithCache(Q, K, V, timeDiffs, keyTimesFromRef, queryEmbeddings, keyEmbeddings, block, bc, PriceEmbeddingDim, PriceNumHeads, enableDecayBias, isTraining, dropoutRng);

        /// <summary>float[numHeads][,] caches and float[,,] tensors cross the boundary flat: the library writes [numHeads, queryLen, keyLen]
        /// and this method slices it into the jagged array the callers keep.</summary>
        public float[,] ContentAwareCrossAttentionForward(float[,] Q, float[,] K, float[,] V, int numHeads, float scale, float[,,] decayBias,
            out float[][,] attentionWeights, out float[][,] scoresPreSoftmax, bool needBackwardCache = true)
        {
            NotNull(Q, nameof(Q)); NotNull(K, nameof(K)); NotNull(V, nameof(V));
            int q = Q.GetLength(0), k = K.GetLength(0), e = Q.GetLength(1);
            var output = new float[q, e];
            float[] w = needBackwardCache ? new float[(long)numHeads * q * k] : null, s = needBackwardCache ? new float[(long)numHeads * q * k] : null;
            fixed (float* pq = Q, pk = K, pv = V, pb = decayBias, po = output, pw = w, ps = s)
                Check(Native.b200_ContentAwareCrossAttentionForward(_ctx, pq, q, pk, pv, k, e, numHeads, scale, pb, po, pw, ps));
            attentionWeights = needBackwardCache ? Unflatten(w, numHeads, q, k) : null;
            scoresPreSoftmax = needBackwardCache ? Unflatten(s, numHeads, q, k) : null;
            return output;
        }

        public (float[,] dQ, float[,] dK, float[,] dV, float[,,] dDecayBias) BackpropTimeDecayedAttention(float[,] q, float[,] k, float[,] v, float[,] dOutput, float[][,] attentionWeights,
            float[,] timeDiffs, int embeddingDim, int numHeads)
        {
            NotNull(q, nameof(q)); NotNull(k, nameof(k)); NotNull(v, nameof(v)); NotNull(dOutput, nameof(dOutput)); NotNull(attentionWeights, nameof(attentionWeights));
            int ql = q.GetLength(0), kl = k.GetLength(0);
            float[] w = Flatten(attentionWeights, numHeads, ql, kl);
            var dQ = new float[ql, embeddingDim]; var dK = new float[kl, embeddingDim]; var dV = new float[kl, embeddingDim];
            float[,,] dBias = timeDiffs != null ? new float[ql, kl, numHeads] : null;   // the reference returns null without time differences
            fixed (float* pq = q, pk = k, pv = v, pd = dOutput, pw = w, oq = dQ, ok = dK, ov = dV, ob = dBias)
                Check(Native.b200_BackpropTimeDecayedAttention(_ctx, pq, ql, pk, pv, kl, pd, pw, embeddingDim, numHeads, oq, ok, ov, ob));
            return (dQ, dK, dV, dBias);
        }

        public void Matrix3DScaleInPlace(float[,,] matrix, float scale) { NotNull(matrix, nameof(matrix)); fixed (float* p = matrix) Check(Native.b200_Matrix3DScaleInPlace(_ctx, p, matrix.LongLength, scale)); }
        public float MatrixSquaredNorm3D(float[,,] matrix) { NotNull(matrix, nameof(matrix)); float r = 0f; fixed (float* p = matrix) Check(Native.b200_MatrixSquaredNorm3D(_ctx, p, matrix.LongLength, &r)); return r; }

        public void Matrix3DAddInPlace(float[,,] target, float[,,] addend)
        {
            NotNull(target, nameof(target)); NotNull(addend, nameof(addend));
            if (target.LongLength != addend.LongLength) throw new ArgumentException("Tensor dimensions must match.");
            fixed (float* t = target, a = addend) Check(Native.b200_Matrix3DAddInPlace(_ctx, t, a, target.LongLength));
        }

        public void Matrix3DUpdate(float[,,] weights, float[,,] gradients, float learningRate)
        {
            NotNull(weights, nameof(weights)); NotNull(gradients, nameof(gradients));
            if (weights.LongLength != gradients.LongLength) throw new ArgumentException("Tensor dimensions must match.");
            fixed (float* w = weights, g = gradients) Check(Native.b200_Matrix3DUpdate(_ctx, w, g, weights.LongLength, learningRate));
        }

        public float[] ProjectGlobalFeatures(float[] globalFeatures, float[,] projection, float[] bias)
        {
            NotNull(globalFeatures, nameof(globalFeatures)); NotNull(projection, nameof(projection)); NotNull(bias, nameof(bias));
            var r = new float[projection.GetLength(0)];
            fixed (float* g = globalFeatures, p = projection, b = bias, o = r)
                Check(Native.b200_ProjectGlobalFeatures(_ctx, g, globalFeatures.Length, p, b, projection.GetLength(0), o));
            return r;
        }

        public float[,] EmbedTokenIds(int[] tokenIds, float[,] embedding, int embeddingDim)
        {
            NotNull(tokenIds, nameof(tokenIds));
            return EmbedTokenIds(tokenIds, 0, tokenIds.Length, embedding, embeddingDim);
        }

        public float[,] EmbedTokenIds(int[] tokenIds, int tokenStart, int tokenCount, float[,] embedding, int embeddingDim)
        {
            NotNull(tokenIds, nameof(tokenIds)); NotNull(embedding, nameof(embedding));
            if (tokenCount < 0) throw new ArgumentOutOfRangeException(nameof(tokenCount));
            var r = new float[tokenCount, embeddingDim];
            fixed (int* ids = tokenIds)
            fixed (float* e = embedding, o = r)   // an id outside [0, vocab) comes back as B200_ERR_OUT_OF_RANGE -> ArgumentOutOfRangeException (AccelerationCPU.cs:3506-3509)
                Check(Native.b200_EmbedTokenIds(_ctx, ids, tokenIds.Length, tokenStart, tokenCount, e, embedding.GetLength(0), embeddingDim, o));
            return r;
        }

        public float[] MeanPoolRows(float[,] matrix)
        {
            NotNull(matrix, nameof(matrix));
            var r = new float[matrix.GetLength(1)];
            fixed (float* m = matrix, o = r) Check(Native.b200_MeanPoolRows(_ctx, m, matrix.GetLength(0), matrix.GetLength(1), o));
            return r;
        }

        public float[,] ExpandMeanPoolGradient(float[,] pooledGradient, int rowIndex, int rowCount, int embeddingDim)
        {
            NotNull(pooledGradient, nameof(pooledGradient));
            var r = new float[rowCount, embeddingDim];
            fixed (float* p = pooledGradient, o = r)
                Check(Native.b200_ExpandMeanPoolGradient(_ctx, p, pooledGradient.GetLength(0), pooledGradient.GetLength(1), rowIndex, rowCount, embeddingDim, o));
            return r;
        }

        public float[] SoftmaxVector(float[] scores)
        {
            NotNull(scores, nameof(scores));
            var r = new float[scores.Length];
            fixed (float* s = scores, o = r) Check(Native.b200_SoftmaxVector(_ctx, s, scores.Length, o));
            return r;
        }

        public void SigmoidInPlace(float[,] matrix) { NotNull(matrix, nameof(matrix)); fixed (float* p = matrix) Check(Native.b200_SigmoidInPlace(_ctx, p, matrix.LongLength)); }

        public void ZeroMatrixColumns(float[,] matrix, int columnCount)
        {
            NotNull(matrix, nameof(matrix));
            fixed (float* p = matrix) Check(Native.b200_ZeroMatrixColumns(_ctx, p, matrix.GetLength(0), matrix.GetLength(1), columnCount));
        }

        public void VectorUpdateClamped(float[] weights, float[] gradients, float learningRate, float minValue, float maxValue)
        {
            NotNull(weights, nameof(weights)); NotNull(gradients, nameof(gradients));
            if (weights.Length != gradients.Length) throw new ArgumentException("Vector lengths must match.");
            fixed (float* w = weights, g = gradients) Check(Native.b200_VectorUpdateClamped(_ctx, w, g, weights.LongLength, learningRate, minValue, maxValue));
        }

        public void AccumulateGlobalProjectionGradients(float[] dGlobalHidden, float[] globalFeatures, float[,] projectionGrad, float[] biasGrad)
        {
            if (dGlobalHidden == null || globalFeatures == null || projectionGrad == null || biasGrad == null) return;   // a no-op in the reference too (AccelerationCPU.cs:4296-4300)
            fixed (float* d = dGlobalHidden, f = globalFeatures, p = projectionGrad, b = biasGrad)
                Check(Native.b200_AccumulateGlobalProjectionGradients(_ctx, d, dGlobalHidden.Length, f, globalFeatures.Length, p, b));
        }

        // MMTAC context builders and output heads: that model family's own code
        public (float[,] contextHidden, float[] contextTimes, int numGlobal, int numNews) BuildMmtacContext(float[,] newsHidden, float[] newsTimes, float[] globalToken, float[,] contextTypeEmbedding)
            => _cpu.BuildMmtacContext(newsHidden, newsTimes, globalToken, contextTypeEmbedding);

        public (float[,] contextHidden, float[] contextTimes, int numGlobal, int numNews, int numPrice) BuildMmtacContextWithPrice(float[,] newsHidden, float[] newsTimes, float[] globalToken,
            float[,] priceContextHidden, float[] priceContextTimes, float[,] contextTypeEmbedding)
            => _cpu.BuildMmtacContextWithPrice(newsHidden, newsTimes, globalToken, priceContextHidden, priceContextTimes, contextTypeEmbedding);

        public (float[,] regression, float[,] range, float[,] quality, float[,] direction, float[,] midDirection, float[,] confidence, float[,] regressionLogits, float[] rangeLogits, float[] qualityLogits)
            ProjectMmtacOutputHeads(float[,] hidden, float[,] regressionProjection, float[] regressionBias, float[,] rangeProjection, float[] rangeBias, float[,] qualityProjection, float[] qualityBias,
                                    float[,] directionProjection, float[] directionBias, float[,] midDirectionProjection, float[] midDirectionBias, float[,] confidenceProjection,
                                    float[] confidenceBias, bool useConfidenceHead)
            => _cpu.ProjectMmtacOutputHeads(hidden, regressionProjection, regressionBias, rangeProjection, rangeBias, qualityProjection, qualityBias, directionProjection, directionBias,
                                            midDirectionProjection, midDirectionBias, confidenceProjection, confidenceBias, useConfidenceHead);

        public (float loss, float[,] dHidden) BackpropMmtacOutputHeads(
            float[,] regression, float[,] range, float[,] quality, float[,] direction, float[,] midDirection, float[,] confidence,
            float[,] targetRegression, float[,] targetRange, float[,] targetQuality, float[,] targetDirection, float[,] targetMidDirection,
            float[] previousClose, float[] confidenceTargets,
            float[,] hidden, float[,] regressionLogits, float[] rangeLogits,
            float[,] regressionProjection, float[,] rangeProjection, float[,] qualityProjection, float[,] directionProjection, float[,] midDirectionProjection, float[,] confidenceProjection,
            float[,] regressionProjectionGrad, float[] regressionBiasGrad,
            float[,] rangeProjectionGrad, float[] rangeBiasGrad,
            float[,] qualityProjectionGrad, float[] qualityBiasGrad,
            float[,] directionProjectionGrad, float[] directionBiasGrad,
            float[,] midDirectionProjectionGrad, float[] midDirectionBiasGrad,
            float[,] confidenceProjectionGrad, float[] confidenceBiasGrad,
            float rangeLossWeight, float qualityLossWeight, float directionLossWeight, float midDirectionLossWeight,
            float closeDirectionConsistencyWeight, float closeDirectionConsistencyMargin, float confidenceLossWeight, bool useConfidenceHead)
            => _cpu.BackpropMmtacOutputHeads(regression, range, quality, direction, midDirection, confidence, targetRegression, targetRange, targetQuality, targetDirection, targetMidDirection,
                                             previousClose, confidenceTargets, hidden, regressionLogits, rangeLogits, regressionProjection, rangeProjection, qualityProjection, directionProjection,
                                             midDirectionProjection, confidenceProjection, regressionProjectionGrad, regressionBiasGrad, rangeProjectionGrad, rangeBiasGrad, qualityProjectionGrad,
                                             qualityBiasGrad, directionProjectionGrad, directionBiasGrad, midDirectionProjectionGrad, midDirectionBiasGrad, confidenceProjectionGrad,
                                             confidenceBiasGrad, rangeLossWeight, qualityLossWeight, directionLossWeight, midDirectionLossWeight, closeDirectionConsistencyWeight,
                                             closeDirectionConsistencyMargin, confidenceLossWeight, useConfidenceHead);

        public void AccumulateMmtacContextGradients(float[,] dContextA, float[,] dContextB, float[,] contextTypeEmbeddingGrad, float[,] dLiveNewsHidden, float[] dGlobalHidden, int numGlobal,
            int numStoredNews, int numNews, int numLiveNews, int numPriceContext, int totalContext, int priceOffset)
            => _cpu.AccumulateMmtacContextGradients(dContextA, dContextB, contextTypeEmbeddingGrad, dLiveNewsHidden, dGlobalHidden, numGlobal, numStoredNews, numNews, numLiveNews,
                                                    numPriceContext, totalContext, priceOffset);

        // =====================================================================================  tokenizer (host string work)
        public string[] PreTokenize(string text) => _cpu.PreTokenize(text);
        public Dictionary<string, int> GetWordFrequencies(string[] texts, bool lowerCase) => _cpu.GetWordFrequencies(texts, lowerCase);
        public HashSet<string> BuildCharacterVocabulary(Dictionary<string, int> wordFreqs) => _cpu.BuildCharacterVocabulary(wordFreqs);
        public List<string> ApplyMerge(List<string> word, string left, string right) => _cpu.ApplyMerge(word, left, right);
        public List<int> EncodeWord(string word, Dictionary<(string, string), int> mergePriority, Dictionary<string, int> vocabToId, int unkTokenId) => _cpu.EncodeWord(word, mergePriority, vocabToId, unkTokenId);
        public Dictionary<(string left, string right), int> CountPairFrequencies(Dictionary<List<string>, int> words) => _cpu.CountPairFrequencies(words);
        public ((string left, string right) pair, int frequency) SelectBestPair(Dictionary<(string left, string right), int> pairCounts, int minFrequency) => _cpu.SelectBestPair(pairCounts, minFrequency);
        public Dictionary<List<string>, int> ApplyMergeToVocabulary(Dictionary<List<string>, int> words, string left, string right) => _cpu.ApplyMergeToVocabulary(words, left, right);
        public string DecodeTokens(int[] tokenIds, Dictionary<int, string> idToVocab, string unkToken, bool skipSpecialTokens) => _cpu.DecodeTokens(tokenIds, idToVocab, unkToken, skipSpecialTokens);
        public int[] PadOrTruncate(int[] tokenIds, int maxLength, bool addSpecialTokens, int padTokenId, int endTokenId) => _cpu.PadOrTruncate(tokenIds, maxLength, addSpecialTokens, padTokenId, endTokenId);

        // =====================================================================================  rotary position embeddings
        public void ApplyRotaryPositionEmbeddingHeadInPlace(float[,] matrix, int startCol, int headDim, float baseTheta, bool inverse)
        {
            NotNull(matrix, nameof(matrix));
            fixed (float* p = matrix) Check(Native.b200_ApplyRotaryPositionEmbeddingHeadInPlace(_ctx, p, matrix.GetLength(0), matrix.GetLength(1), startCol, headDim, baseTheta, B(inverse)));
        }

        public void ApplyRotaryPositionEmbeddingInPlace(float[,] matrix, int numHeads, float baseTheta, bool inverse)
        {
            NotNull(matrix, nameof(matrix));
            fixed (float* p = matrix) Check(Native.b200_ApplyRotaryPositionEmbeddingInPlace(_ctx, p, matrix.GetLength(0), matrix.GetLength(1), numHeads, baseTheta, B(inverse), 0));
        }

        // =====================================================================================  IB200TrainStep: the resident trainer (host edit 4)
        public void AttachModel(B200ModelShape s, float[] flatParameters, int maxRowsPerPass)
        {
            var cfg = new LmConfig
            {
                vocab_size = s.Discrete ? s.VocabSize : 0, input_feature_dim = s.Discrete ? 0 : s.InputFeatureDim, output_dim = s.Discrete ? s.VocabSize : s.OutputDim,
                embedding_dim = s.EmbeddingDim, num_heads = s.NumHeads, num_layers = s.NumLayers, ffn_dim = s.FeedForwardDim, ffn_activation = (int)s.FfnActivation,
                discrete = B(s.Discrete), loss_kind = s.MseLoss ? 1 : 0, causal = B(s.Causal), align_floats = 64
            };
            _paramCount = Native.b200_lm_param_count(ref cfg);
            if (_paramCount < 0) throw new ArgumentException("invalid model configuration");
            if (flatParameters == null || flatParameters.LongLength != _paramCount) throw new ArgumentException($"expected {_paramCount} parameters in arena order (b200_lm_tensor_info)");
            if (_lm != IntPtr.Zero) { Native.b200_lm_destroy(_lm); _lm = IntPtr.Zero; }
            Check(Native.b200_lm_create(_ctx, ref cfg, null, null, maxRowsPerPass, out _lm));
            fixed (float* p = flatParameters) Check(Native.b200_lm_upload_params(_lm, p, 0, _paramCount));
        }

        public (float loss, float gradNorm, int validCount) TrainBatchDiscrete(int[] tokens, int[] seqOffsets, float learningRate, bool useClip, float clipThreshold)
        {
            NotNull(tokens, nameof(tokens)); NotNull(seqOffsets, nameof(seqOffsets));
            float loss = 0f, norm = 0f; int valid = 0;
            fixed (int* t = tokens, o = seqOffsets)
                Check(Native.b200_lm_train_step_discrete(_lm, t, o, seqOffsets.Length - 1, learningRate, B(useClip), clipThreshold, 1, &loss, &norm, &valid));
            return (loss, norm, valid);
        }

        public (float loss, float gradNorm, int validCount) TrainBatchContinuous(float[,] features, float[,] regressionTargets, int[] classTargets, int[] seqOffsets,
                                                                                  float learningRate, bool useClip, float clipThreshold)
        {
            NotNull(features, nameof(features)); NotNull(seqOffsets, nameof(seqOffsets));
            float loss = 0f, norm = 0f; int valid = 0;
            fixed (float* x = features, r = regressionTargets)
            fixed (int* c = classTargets, o = seqOffsets)
                Check(Native.b200_lm_train_step_continuous(_lm, x, r, c, o, seqOffsets.Length - 1, learningRate, B(useClip), clipThreshold, 1, &loss, &norm, &valid));
            return (loss, norm, valid);
        }

        public (float meanLoss, int items) ValidateDiscrete(int[] tokens, int[] seqOffsets)
        {
            NotNull(tokens, nameof(tokens)); NotNull(seqOffsets, nameof(seqOffsets));
            float loss = 0f; int items = 0;
            fixed (int* t = tokens, o = seqOffsets) Check(Native.b200_lm_validate_discrete(_lm, t, o, seqOffsets.Length - 1, &loss, &items));
            return (loss, items);
        }

        public float[] DownloadParameters()
        {
            var r = new float[_paramCount];
            fixed (float* p = r) Check(Native.b200_lm_download_params(_lm, p, 0, _paramCount));
            return r;
        }

        // =====================================================================================  IB200MlpBatch (host edit 5)
        public IntPtr CreateMlp(int[] widths, ActivationType[] activations, CostFunctionType cost, float huberDelta, float l2Lambda, float clipThreshold, int maxBatch)
        {
            NotNull(widths, nameof(widths)); NotNull(activations, nameof(activations));
            var acts = new int[activations.Length];
            for (int i = 0; i < acts.Length; i++) acts[i] = (int)activations[i];
            IntPtr h;
            fixed (int* w = widths, a = acts) Check(Native.b200_mlp_create(_ctx, widths.Length, w, a, (int)cost, huberDelta, l2Lambda, clipThreshold, maxBatch, out h));
            return h;
        }

        public void UploadLayer(IntPtr mlp, int layer, float[,] weights, float[] biases) { fixed (float* w = weights, b = biases) Check(Native.b200_mlp_upload_layer(mlp, layer, w, b)); }
        public void DownloadLayer(IntPtr mlp, int layer, float[,] weights, float[] biases) { fixed (float* w = weights, b = biases) Check(Native.b200_mlp_download_layer(mlp, layer, w, b)); }

        public float LearnBatch(IntPtr mlp, float[,] x, float[,] y, float learningRate, float[] inputMin, float[] inputMax)
        {
            NotNull(x, nameof(x)); NotNull(y, nameof(y));
            float norm = 0f;
            fixed (float* px = x, py = y, mn = inputMin, mx = inputMax) Check(Native.b200_mlp_learn_batch(mlp, px, py, x.GetLength(0), learningRate, mn, mx, &norm));
            return norm;
        }

        public void DestroyMlp(IntPtr mlp) => Native.b200_mlp_destroy(mlp);
    }
}
