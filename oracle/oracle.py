"""ctypes front end of the CPU oracle (oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke`` and by
``bench.py``'s CPU-baseline / reference arm.  The shipped package never imports it.

The method names and argument meaning mirror the reference's ``IAccelerationManager``
(CallaghanDev.ML/AccelerationManagers/IAccelerationManager.cs:13-361) so that a parity
test reads ``oracle.LayerNormBackward(...)`` against ``manager.LayerNormBackward(...)``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent

ACT = {"None": 0, "Sigmoid": 1, "Tanh": 2, "Relu": 3, "Leakyrelu": 4, "Swish": 5}
COST = {"mse": 0, "ZeroWeightedMSE": 1, "binaryCrossEntropy": 2, "mae": 3, "categoricalCrossEntropy": 4, "huberLoss": 5}


def build(force: bool = False) -> None:
    """Compile liboracle.so / liboracle_f64.so next to this file (gcc, a few seconds)."""
    targets = [_HERE / "liboracle.so", _HERE / "liboracle_f64.so"]
    src = _HERE / "oracle.c"
    if not force and all(t.exists() and t.stat().st_mtime >= src.stat().st_mtime for t in targets):
        return
    subprocess.run(["make", "-C", str(_HERE), "-s", "-B"], check=True, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)


class LMConfig(C.Structure):
    """Field-for-field image of ``ref_lm_config`` / ``b200_lm_config``."""

    _fields_ = [
        ("vocab_size", C.c_int32),
        ("input_feature_dim", C.c_int32),
        ("output_dim", C.c_int32),
        ("embedding_dim", C.c_int32),
        ("num_heads", C.c_int32),
        ("num_layers", C.c_int32),
        ("ffn_dim", C.c_int32),
        ("ffn_activation", C.c_int32),
        ("discrete", C.c_int32),
        ("loss_kind", C.c_int32),
        ("causal", C.c_int32),
        ("align_floats", C.c_int32),
    ]


def _mask(m):
    if m is None:
        return None
    return np.ascontiguousarray(np.asarray(m).astype(np.uint8))


class Oracle:
    def __init__(self, f64: bool = False, threads: int = 1):
        build()
        self.lib = C.CDLL(str(_HERE / ("liboracle_f64.so" if f64 else "liboracle.so")))
        self.dt = np.float64 if f64 else np.float32
        self.real = C.c_double if f64 else C.c_float
        lib = self.lib
        lib.ref_CrossEntropyLossAndGradient.restype = self.real
        lib.ref_MSELossAndGradient.restype = self.real
        lib.ref_SquaredNorm.restype = self.real
        lib.ref_lm_train_step.restype = self.real
        lib.ref_lm_validate.restype = self.real
        lib.ref_mlp_learn_batch.restype = self.real
        lib.ref_lm_param_count.restype = C.c_int64
        assert lib.ref_real_size() == np.dtype(self.dt).itemsize
        self.set_threads(threads)

    # ------------------------------------------------------------------ helpers
    def set_threads(self, n: int) -> None:
        self.lib.ref_set_threads(int(n))

    def max_threads(self) -> int:
        return int(self.lib.ref_max_threads())

    def a(self, x):
        return np.ascontiguousarray(np.asarray(x, dtype=self.dt))

    def p(self, x):
        return None if x is None else x.ctypes.data_as(C.c_void_p)

    def r(self, v):
        return self.real(float(v))

    # ------------------------------------------------------------------ tensor primitives
    def MatrixMultiply(self, A, B):
        A, B = self.a(A), self.a(B)
        out = np.zeros((A.shape[0], B.shape[1]), self.dt)
        self.lib.ref_MatrixMultiply(self.p(A), A.shape[0], A.shape[1], self.p(B), B.shape[1], self.p(out))
        return out

    def MatrixMultiplyTranspose(self, A, B):
        A, B = self.a(A), self.a(B)
        out = np.zeros((A.shape[0], B.shape[0]), self.dt)
        self.lib.ref_MatrixMultiplyTranspose(self.p(A), A.shape[0], A.shape[1], self.p(B), B.shape[0], self.p(out))
        return out

    def BatchDotProductAddBias(self, W, X, bias, rowStart=0, rowCount=None):
        W, X, bias = self.a(W), self.a(X), self.a(bias)
        rowCount = X.shape[0] - rowStart if rowCount is None else rowCount
        out = np.zeros((rowCount, W.shape[0]), self.dt)
        self.lib.ref_BatchDotProductAddBias(self.p(W), W.shape[0], W.shape[1], self.p(X), rowStart, rowCount, self.p(bias), self.p(out))
        return out

    def ProjectOutputBatch(self, hidden, proj, bias, seqLen, outputDim):
        hidden, proj, bias = self.a(hidden), self.a(proj), self.a(bias)
        out = np.zeros((seqLen, outputDim), self.dt)
        self.lib.ref_ProjectOutputBatch(self.p(hidden), hidden.shape[1], self.p(proj), self.p(bias), seqLen, outputDim, self.p(out))
        return out

    def MatrixAddInPlace(self, target, addend):
        addend = self.a(addend)
        self.lib.ref_AddInPlace(self.p(target), self.p(addend), C.c_int64(target.size))

    VectorAccumulate = MatrixAddInPlace

    # ------------------------------------------------------------------ layer norm
    def ResidualLayerNormForward(self, input, subLayer, gamma, beta, eps=1e-5):
        input, gamma, beta = self.a(input), self.a(gamma), self.a(beta)
        subLayer = None if subLayer is None else self.a(subLayer)
        rows, feat = input.shape
        out, norm, res = (np.zeros((rows, feat), self.dt) for _ in range(3))
        means, var = np.zeros(rows, self.dt), np.zeros(rows, self.dt)
        self.lib.ref_ResidualLayerNormForward(self.p(input), self.p(subLayer), self.p(gamma), self.p(beta), rows, feat, self.r(eps),
                                              self.p(out), self.p(means), self.p(var), self.p(norm), self.p(res))
        return out, means, var, norm, res

    def LayerNormForward(self, input, gamma, beta, eps=1e-5):
        return self.ResidualLayerNormForward(input, None, gamma, beta, eps)[:4]

    def LayerNormBackward(self, dOut, normalized, gamma, input, mean, variance, eps=1e-5):
        dOut, normalized, gamma, input, mean, variance = map(self.a, (dOut, normalized, gamma, input, mean, variance))
        rows, feat = dOut.shape
        dIn, dG, dB = np.zeros((rows, feat), self.dt), np.zeros(feat, self.dt), np.zeros(feat, self.dt)
        self.lib.ref_LayerNormBackward(self.p(dOut), self.p(normalized), self.p(gamma), self.p(input), self.p(mean), self.p(variance),
                                       rows, feat, self.r(eps), self.p(dIn), self.p(dG), self.p(dB))
        return dIn, dG, dB

    # ------------------------------------------------------------------ attention
    def ScaledDotProductAttention(self, q, k, v, numHeads, mask=None, causal=False):
        q, k, v = self.a(q), self.a(k), self.a(v)
        if causal and q.shape[0] != k.shape[0]:
            raise ValueError("The simple causal path assumes queryLen == keyLen.")
        m = _mask(mask)
        out = np.zeros_like(q)
        self.lib.ref_ScaledDotProductAttention(self.p(q), self.p(k), self.p(v), q.shape[0], k.shape[0], q.shape[1], numHeads,
                                               self.p(m), int(bool(causal)), self.p(out))
        return out

    def MultiHeadAttentionBackward(self, Q, K, V, dConcat, numHeads, scale, mask=None, useDecoderMask=False):
        Q, K, V, dConcat = map(self.a, (Q, K, V, dConcat))
        m = _mask(mask)
        dQ, dK, dV = np.zeros_like(Q), np.zeros_like(K), np.zeros_like(V)
        self.lib.ref_MultiHeadAttentionBackward(self.p(Q), self.p(K), self.p(V), self.p(dConcat), Q.shape[0], K.shape[0], Q.shape[1],
                                                numHeads, self.r(scale), self.p(m), int(bool(useDecoderMask)),
                                                self.p(dQ), self.p(dK), self.p(dV))
        return dQ, dK, dV

    def SegmentedAttentionForward(self, Q, K, V, segLen, segCount, numHeads, causal=True):
        Q, K, V = map(self.a, (Q, K, V))
        out = np.zeros_like(Q)
        self.lib.ref_SegmentedAttentionForward(self.p(Q), self.p(K), self.p(V), segLen, segCount, Q.shape[1], numHeads,
                                               int(bool(causal)), self.p(out))
        return out

    def SegmentedAttentionBackward(self, Q, K, V, dConcat, segLen, segCount, numHeads, scale, causal=True):
        Q, K, V, dConcat = map(self.a, (Q, K, V, dConcat))
        dQ, dK, dV = np.zeros_like(Q), np.zeros_like(K), np.zeros_like(V)
        self.lib.ref_SegmentedAttentionBackward(self.p(Q), self.p(K), self.p(V), self.p(dConcat), segLen, segCount, Q.shape[1], numHeads,
                                                self.r(scale), int(bool(causal)), self.p(dQ), self.p(dK), self.p(dV))
        return dQ, dK, dV

    def ApplyRotaryPositionEmbeddingInPlace(self, matrix, numHeads, baseTheta=10000.0, inverse=False, segLen=0):
        assert matrix.dtype == self.dt and matrix.flags.c_contiguous
        self.lib.ref_ApplyRotaryPositionEmbeddingInPlace(self.p(matrix), matrix.shape[0], matrix.shape[1], numHeads, self.r(baseTheta),
                                                         int(bool(inverse)), segLen)

    def ApplyRotaryPositionEmbeddingHeadInPlace(self, matrix, startCol, headDim, baseTheta=10000.0, inverse=False):
        assert matrix.dtype == self.dt and matrix.flags.c_contiguous
        self.lib.ref_ApplyRotaryPositionEmbeddingHeadInPlace(self.p(matrix), matrix.shape[0], matrix.shape[1], startCol, headDim,
                                                             self.r(baseTheta), int(bool(inverse)))

    # ------------------------------------------------------------------ projections
    def ProjectQKV(self, input, WQ, bQ, WK, bK, WV, bV):
        input, WQ, bQ, WK, bK, WV, bV = map(self.a, (input, WQ, bQ, WK, bK, WV, bV))
        rows, out = input.shape[0], WQ.shape[0]
        Q, K, V = (np.zeros((rows, out), self.dt) for _ in range(3))
        self.lib.ref_ProjectQKV(self.p(input), rows, input.shape[1], self.p(WQ), self.p(bQ), self.p(WK), self.p(bK), self.p(WV), self.p(bV),
                                out, self.p(Q), self.p(K), self.p(V))
        return Q, K, V

    def BackpropQKV(self, input, dQ, dK, dV, WQ, WK, WV, WQg, bQg, WKg, bKg, WVg, bVg):
        input, dQ, dK, dV, WQ, WK, WV = map(self.a, (input, dQ, dK, dV, WQ, WK, WV))
        dIn = np.zeros_like(input)
        self.lib.ref_BackpropQKV(self.p(input), input.shape[0], input.shape[1], self.p(dQ), self.p(dK), self.p(dV), WQ.shape[0],
                                 self.p(WQ), self.p(WK), self.p(WV), self.p(WQg), self.p(bQg), self.p(WKg), self.p(bKg),
                                 self.p(WVg), self.p(bVg), self.p(dIn))
        return dIn

    def ProjectKV(self, input, WK, bK, WV, bV):
        input, WK, bK, WV, bV = map(self.a, (input, WK, bK, WV, bV))
        rows, out = input.shape[0], WK.shape[0]
        K, V = (np.zeros((rows, out), self.dt) for _ in range(2))
        self.lib.ref_ProjectKV(self.p(input), rows, input.shape[1], self.p(WK), self.p(bK), self.p(WV), self.p(bV), out, self.p(K), self.p(V))
        return K, V

    def BackpropKV(self, input, dK, dV, WK, WV, WKg, bKg, WVg, bVg):
        input, dK, dV, WK, WV = map(self.a, (input, dK, dV, WK, WV))
        dIn = np.zeros_like(input)
        self.lib.ref_BackpropKV(self.p(input), input.shape[0], input.shape[1], self.p(dK), self.p(dV), WK.shape[0], self.p(WK), self.p(WV),
                                self.p(WKg), self.p(bKg), self.p(WVg), self.p(bVg), self.p(dIn))
        return dIn

    # ------------------------------------------------------------------ sibling trainers' operators
    def ContentAwareCrossAttentionForward(self, Q, K, V, numHeads, scale, decayBias=None, needBackwardCache=True):
        Q, K, V = self.a(Q), self.a(K), self.a(V)
        b = None if decayBias is None else self.a(decayBias)
        qn, e, kn = Q.shape[0], Q.shape[1], K.shape[0]
        out = np.zeros((qn, e), self.dt)
        W, S = np.zeros((numHeads, qn, kn), self.dt), np.zeros((numHeads, qn, kn), self.dt)
        self.lib.ref_ContentAwareCrossAttentionForward(self.p(Q), qn, self.p(K), self.p(V), kn, e, numHeads, self.r(scale), self.p(b),
                                                       self.p(out), self.p(W), self.p(S))
        return (out, W, S) if needBackwardCache else (out, None, None)

    def BackpropTimeDecayedAttention(self, q, k, v, dOutput, attentionWeights, timeDiffs, embeddingDim, numHeads):
        q, k, v, dO, W = map(self.a, (q, k, v, dOutput, attentionWeights))
        qn, kn = q.shape[0], k.shape[0]
        dQ, dK, dV = np.zeros_like(q), np.zeros_like(k), np.zeros_like(v)
        dB = np.zeros((qn, kn, numHeads), self.dt) if timeDiffs is not None else None
        self.lib.ref_BackpropTimeDecayedAttention(self.p(q), qn, self.p(k), self.p(v), kn, self.p(dO), self.p(W), embeddingDim, numHeads,
                                                  self.p(dQ), self.p(dK), self.p(dV), self.p(dB))
        return dQ, dK, dV, dB

    def ApplyContextTypeEmbedding(self, contextHidden, typeEmbedding, typeIndices):
        t, idx = self.a(typeEmbedding), np.ascontiguousarray(np.asarray(typeIndices, np.int32))
        self.lib.ref_ApplyContextTypeEmbedding(self.p(contextHidden), contextHidden.shape[0], contextHidden.shape[1], self.p(t), self.p(idx))

    def ComputeTimeDiffMatrix(self, priceSeqLen, keyArrivalTimes):
        t = self.a(keyArrivalTimes)
        out = np.zeros((priceSeqLen, len(t)), self.dt)
        self.lib.ref_ComputeTimeDiffMatrix(priceSeqLen, self.p(t), len(t), self.p(out))
        return out

    def ComputeMemoryAttentionScores(self, priceHidden, lastPos, contextHidden, totalCtx, scale):
        p_, c = self.a(priceHidden), self.a(contextHidden)
        out = np.zeros(totalCtx, self.dt)
        self.lib.ref_ComputeMemoryAttentionScores(self.p(p_), p_.shape[1], lastPos, self.p(c), totalCtx, self.r(scale), self.p(out))
        return out

    def ProjectGlobalFeatures(self, globalFeatures, projection, bias):
        g, P, b = self.a(globalFeatures), self.a(projection), self.a(bias)
        out = np.zeros(P.shape[0], self.dt)
        self.lib.ref_ProjectGlobalFeatures(self.p(g), P.shape[1], self.p(P), self.p(b), P.shape[0], self.p(out))
        return out

    def MeanPoolRows(self, matrix):
        m = self.a(matrix)
        out = np.zeros(m.shape[1], self.dt)
        self.lib.ref_MeanPoolRows(self.p(m), m.shape[0], m.shape[1], self.p(out))
        return out

    def ExpandMeanPoolGradient(self, pooledGradient, rowIndex, rowCount, embeddingDim):
        g = self.a(pooledGradient)
        out = np.zeros((max(rowCount, 0), embeddingDim), self.dt)
        if rowCount > 0:
            self.lib.ref_ExpandMeanPoolGradient(self.p(g), g.shape[1], rowIndex, rowCount, embeddingDim, self.p(out))
        return out

    def SoftmaxVector(self, scores):
        s = self.a(scores)
        out = np.zeros(len(s), self.dt)
        self.lib.ref_SoftmaxVector(self.p(s), len(s), self.p(out))
        return out

    def SigmoidInPlace(self, matrix):
        self.lib.ref_SigmoidInPlace(self.p(matrix), C.c_longlong(matrix.size))

    def ZeroMatrixColumns(self, matrix, columnCount):
        self.lib.ref_ZeroMatrixColumns(self.p(matrix), matrix.shape[0], matrix.shape[1], columnCount)

    def VectorUpdateClamped(self, weights, gradients, learningRate, minValue, maxValue):
        g = self.a(gradients)
        self.lib.ref_VectorUpdateClamped(self.p(weights), self.p(g), C.c_longlong(weights.size), self.r(learningRate), self.r(minValue),
                                         self.r(maxValue))

    def AccumulateGlobalProjectionGradients(self, dGlobalHidden, globalFeatures, projectionGrad, biasGrad):
        d, g = self.a(dGlobalHidden), self.a(globalFeatures)
        self.lib.ref_AccumulateGlobalProjectionGradients(self.p(d), len(d), self.p(g), len(g), self.p(projectionGrad), self.p(biasGrad))

    def BackpropLinearProjection(self, input, dOutput, weights, weightGrad, biasGrad, dInput):
        input, dOutput, weights = map(self.a, (input, dOutput, weights))
        self.lib.ref_BackpropLinearProjection(self.p(input), self.p(dOutput), self.p(weights), input.shape[0], input.shape[1],
                                              dOutput.shape[1], self.p(weightGrad), self.p(biasGrad), self.p(dInput))

    def BackpropOutputProjection(self, dLogits, input, weights, weightGrad, biasGrad, seqLen, outputDim, embeddingDim):
        dLogits, input, weights = map(self.a, (dLogits, input, weights))
        dX = np.zeros((seqLen, embeddingDim), self.dt)
        self.lib.ref_BackpropOutputProjection(self.p(dLogits), self.p(input), self.p(weights), self.p(weightGrad), self.p(biasGrad),
                                              seqLen, outputDim, embeddingDim, self.p(dX))
        return dX

    def BackpropInputProjection(self, dX, continuousInput, weightGrad, biasGrad, seqLen, embeddingDim, inputFeatureDim, inputRowStart=0):
        dX, continuousInput = self.a(dX), self.a(continuousInput)
        self.lib.ref_BackpropInputProjection(self.p(dX), self.p(continuousInput), continuousInput.shape[1], inputRowStart,
                                             self.p(weightGrad), self.p(biasGrad), seqLen, embeddingDim, inputFeatureDim)

    def EmbedTokenIds(self, tokenIds, embedding, embeddingDim, tokenStart=0, tokenCount=None):
        ids = np.ascontiguousarray(np.asarray(tokenIds, np.int32))
        embedding = self.a(embedding)
        tokenCount = len(ids) - tokenStart if tokenCount is None else tokenCount
        out = np.zeros((tokenCount, embeddingDim), self.dt)
        rc = self.lib.ref_EmbedTokenIds(self.p(ids), tokenStart, tokenCount, self.p(embedding), embedding.shape[0], embeddingDim, self.p(out))
        if rc != 0:
            raise IndexError("token id outside the embedding table")
        return out

    def AccumulateTokenEmbeddingGrad(self, embeddingGrad, dX, tokenIds, seqLen, embeddingDim, tokenStart=0):
        ids = np.ascontiguousarray(np.asarray(tokenIds, np.int32))
        dX = self.a(dX)
        self.lib.ref_AccumulateTokenEmbeddingGrad(self.p(embeddingGrad), self.p(dX), self.p(ids), tokenStart, seqLen, embeddingDim)

    # ------------------------------------------------------------------ losses
    def CrossEntropyLossAndGradient(self, logits, targets, effectiveLen, targetStart=0):
        logits = self.a(logits)
        t = np.ascontiguousarray(np.asarray(targets, np.int32))
        d = np.zeros_like(logits)
        loss = self.lib.ref_CrossEntropyLossAndGradient(self.p(logits), logits.shape[0], logits.shape[1], self.p(t), targetStart, effectiveLen, self.p(d))
        return self.dt(loss), d

    def MSELossAndGradient(self, predictions, targets, effectiveLen, targetStart=0):
        predictions, targets = self.a(predictions), self.a(targets)
        d = np.zeros_like(predictions)
        loss = self.lib.ref_MSELossAndGradient(self.p(predictions), predictions.shape[0], predictions.shape[1], self.p(targets), targetStart, effectiveLen, self.p(d))
        return self.dt(loss), d

    # ------------------------------------------------------------------ step primitives
    def MatrixSquaredNorm(self, m):
        m = self.a(m)
        return self.dt(self.lib.ref_SquaredNorm(self.p(m), C.c_int64(m.size)))

    VectorSquaredNorm = MatrixSquaredNorm

    def MatrixScaleInPlace(self, m, scale):
        self.lib.ref_ScaleInPlace(self.p(m), C.c_int64(m.size), self.r(scale))

    VectorScaleInPlace = MatrixScaleInPlace

    def MatrixUpdate(self, w, g, lr):
        g = self.a(g)
        self.lib.ref_Update(self.p(w), self.p(g), C.c_int64(w.size), self.r(lr))

    VectorUpdate = MatrixUpdate

    # ------------------------------------------------------------------ feed-forward network
    def _net(self, widths, acts, weights, biases, grads=False):
        n = len(widths)
        w_arr = (C.c_void_p * n)()
        b_arr = (C.c_void_p * n)()
        keep = []
        for l in range(1, n):
            w = weights[l - 1] if grads else self.a(weights[l - 1])
            b = biases[l - 1] if grads else self.a(biases[l - 1])
            keep += [w, b]
            w_arr[l] = w.ctypes.data
            b_arr[l] = b.ctypes.data
        wd = np.asarray(widths, np.int32)
        ac = np.asarray([ACT[x] if isinstance(x, str) else int(x) for x in acts], np.int32)
        return wd, ac, w_arr, b_arr, keep

    def FFNForwardBatch(self, input, widths, acts, weights, biases):
        input = self.a(input)
        wd, ac, w, b, keep = self._net(widths, acts, weights, biases)
        out = np.zeros((input.shape[0], widths[-1]), self.dt)
        self.lib.ref_FFNForwardBatch(self.p(input), input.shape[0], len(widths), self.p(wd), self.p(ac), w, b, self.p(out))
        return out

    def FFNInputGradientBatch(self, input, dOutput, widths, acts, weights, biases, weightGrads=None, biasGrads=None):
        """NeuralNetwork.ComputeInputGradientBatch; weightGrads/biasGrads are accumulated in place when given."""
        input, dOutput = self.a(input), self.a(dOutput)
        wd, ac, w, b, keep = self._net(widths, acts, weights, biases)
        gw = gb = None
        if weightGrads is not None:
            _, _, gw, gb, keep2 = self._net(widths, acts, weightGrads, biasGrads, grads=True)
        dIn = np.zeros_like(input)
        self.lib.ref_FFNInputGradientBatch(self.p(input), self.p(dOutput), input.shape[0], len(widths), self.p(wd), self.p(ac), w, b, gw, gb, self.p(dIn))
        return dIn

    # ------------------------------------------------------------------ language-model step
    def lm_param_count(self, cfg: LMConfig) -> int:
        return int(self.lib.ref_lm_param_count(C.byref(cfg)))

    def lm_tensors(self, cfg: LMConfig):
        """[(offset, rows, cols)] in arena order."""
        out = []
        for i in range(self.lib.ref_lm_tensor_count(C.byref(cfg))):
            off, r, c = C.c_int64(), C.c_int32(), C.c_int32()
            self.lib.ref_lm_tensor_info(C.byref(cfg), i, C.byref(off), C.byref(r), C.byref(c))
            out.append((off.value, r.value, c.value))
        return out

    def lm_train_step(self, cfg: LMConfig, params, grads, seq_offsets, tokens=None, cont=None, reg_targets=None, cls_targets=None,
                      lr=1e-3, use_clip=True, clip_thr=1.0, do_step=True):
        """Returns (loss, grad_norm, valid_count); params (when do_step) and grads are updated in place."""
        assert params.dtype == self.dt and grads.dtype == self.dt
        off = np.ascontiguousarray(np.asarray(seq_offsets, np.int32))
        tok = None if tokens is None else np.ascontiguousarray(np.asarray(tokens, np.int32))
        cont = None if cont is None else self.a(cont)
        reg = None if reg_targets is None else self.a(reg_targets)
        cls = None if cls_targets is None else np.ascontiguousarray(np.asarray(cls_targets, np.int32))
        norm, valid = self.real(0), C.c_int32(0)
        loss = self.lib.ref_lm_train_step(C.byref(cfg), self.p(params), self.p(grads), self.p(tok), self.p(cont), self.p(reg), self.p(cls),
                                          self.p(off), len(off) - 1, self.r(lr), int(bool(use_clip)), self.r(clip_thr), int(bool(do_step)),
                                          C.byref(norm), C.byref(valid))
        return float(loss), float(norm.value), int(valid.value)

    def lm_validate(self, cfg: LMConfig, params, seq_offsets, tokens=None, cont=None, reg_targets=None, cls_targets=None):
        """TransformerTrainer.Validate / ValidateContinuous: (mean loss over contributing rows, contributing rows)."""
        assert params.dtype == self.dt
        off = np.ascontiguousarray(np.asarray(seq_offsets, np.int32))
        tok = None if tokens is None else np.ascontiguousarray(np.asarray(tokens, np.int32))
        cont = None if cont is None else self.a(cont)
        reg = None if reg_targets is None else self.a(reg_targets)
        cls = None if cls_targets is None else np.ascontiguousarray(np.asarray(cls_targets, np.int32))
        items = C.c_int32(0)
        loss = self.lib.ref_lm_validate(C.byref(cfg), self.p(params), self.p(tok), self.p(cont), self.p(reg), self.p(cls), self.p(off), len(off) - 1,
                                        C.byref(items))
        return float(loss), int(items.value)

    def lm_decode_logits(self, cfg: LMConfig, params, tokens, max_len=None):
        """LanguageModel incremental decoding (KV cache, one token at a time): logits [len(tokens), output_dim], row t =
        next-token logits after token t."""
        assert params.dtype == self.dt
        tok = np.ascontiguousarray(np.asarray(tokens, np.int32))
        out = np.zeros((len(tok), cfg.output_dim), self.dt)
        rc = self.lib.ref_lm_decode_logits(C.byref(cfg), self.p(params), self.p(tok), len(tok), int(max_len or len(tok)), self.p(out))
        if rc != 0:
            raise ValueError("invalid token id or sequence longer than the cache")
        return out

    # ------------------------------------------------------------------ MLP batch step
    def mlp_learn_batch(self, widths, acts, weights, biases, X, Y, cost="mse", huber_delta=1.0, lr=0.01, lam=0.0, clip_thr=1.0):
        """weights/biases: lists (per non-input layer) of arrays updated in place.  Returns the delta norm."""
        X, Y = self.a(X), self.a(Y)
        wd, ac, w, b, keep = self._net(widths, acts, weights, biases, grads=True)
        ck = COST[cost] if isinstance(cost, str) else int(cost)
        return float(self.lib.ref_mlp_learn_batch(len(widths), self.p(wd), self.p(ac), w, b, self.p(X), self.p(Y), X.shape[0], ck,
                                                  self.r(huber_delta), self.r(lr), self.r(lam), self.r(clip_thr)))

    def mlp_scale_inputs(self, X, mn, mx):
        X, mn, mx = self.a(X), self.a(mn), self.a(mx)
        out = np.zeros_like(X)
        self.lib.ref_mlp_scale_inputs(self.p(X), X.shape[0], X.shape[1], self.p(mn), self.p(mx), self.p(out))
        return out


# Closed-form input generators of the reference's parity tests
# (CallaghanDev.ML.TestConsoleApp/Tests/AccelerationManagerParityTests.cs:2180-2212).
def pt_matrix(rows, cols, seed, dtype=np.float32):
    i = np.arange(1, rows + 1, dtype=np.float64)[:, None]
    j = np.arange(1, cols + 1, dtype=np.float64)[None, :]
    return (np.sin(i * 12.9898 + j * 78.233 + seed * 0.137) * 0.25).astype(np.float32).astype(dtype)


def pt_vector(n, seed, dtype=np.float32):
    i = np.arange(1, n + 1, dtype=np.float64)
    return (np.sin(i * 19.19 + seed * 0.313) * 0.25).astype(np.float32).astype(dtype)


def pt_tensor3(d0, d1, d2, seed, dtype=np.float32):
    """Tensor3 of the same test file (AccelerationManagerParityTests.cs:2239-2254)."""
    i = np.arange(1, d0 + 1, dtype=np.float64)[:, None, None]
    j = np.arange(1, d1 + 1, dtype=np.float64)[None, :, None]
    k = np.arange(1, d2 + 1, dtype=np.float64)[None, None, :]
    return (np.sin(i * 3.1 + j * 5.7 + k * 7.9 + seed * 0.101) * 0.1).astype(np.float32).astype(dtype)


def pt_positive_vector(n, seed, dtype=np.float32):
    return (np.abs(pt_vector(n, seed)) + np.float32(0.5)).astype(dtype)
