"""CudaB200AccelerationManager: the host-side mirror of the reference's IAccelerationManager for the training hot path.

Method names, argument order and meaning, accumulate-vs-assign behaviour and error behaviour follow
CallaghanDev.ML/AccelerationManagers/IAccelerationManager.cs:13-361 (numpy ``float32`` C-contiguous arrays stand in
for ``float[,]`` / ``float[]``, ``int32`` for ``int[]``, ``bool`` for ``bool[,]``).  Every call goes through the
C ABI of libcallaghan_b200.so; in-place methods mutate the caller's array exactly as the reference does.
Exceptions: ValueError <- ArgumentNullException/ArgumentException, IndexError <- ArgumentOutOfRangeException.
"""
from __future__ import annotations

import ctypes as C
import weakref

import numpy as np

from . import _lib as L


def _f(x):
    if x is None:
        raise ValueError("argument is null")
    a = np.asarray(x, dtype=np.float32)
    return a if a.flags.c_contiguous else np.ascontiguousarray(a)


def _inplace(x, name="array"):
    if x is None:
        raise ValueError(f"{name} is null")
    if not (isinstance(x, np.ndarray) and x.dtype == np.float32 and x.flags.c_contiguous and x.flags.writeable):
        raise TypeError(f"{name} is modified in place: pass a writable C-contiguous float32 numpy array")
    return x


def _i(x):
    if x is None:
        raise ValueError("argument is null")
    return np.ascontiguousarray(np.asarray(x, dtype=np.int32))


def _pf(a):
    return None if a is None else a.ctypes.data_as(C.POINTER(C.c_float))


def _pi(a):
    return a.ctypes.data_as(C.POINTER(C.c_int32))


def _mask(m):
    if m is None:
        return None, None
    a = np.ascontiguousarray(np.asarray(m).astype(np.uint8))
    return a, a.ctypes.data_as(C.POINTER(C.c_uint8))


class CudaB200AccelerationManager:
    def __init__(self, device: int = 0, gemm_mode: int = L.GEMM_AUTO):
        self.lib = L.load()
        h = C.c_void_p()
        rc = self.lib.b200_create(int(device), C.byref(h))
        if rc != L.OK:
            raise L.B200Error(f"b200_create(device={device}) failed with status {rc}: a CUDA device is required (no CPU fallback)")
        self.ctx = h
        self.device = device
        self._children = weakref.WeakSet()  # resident trainers: they must be destroyed before the context
        self.set_gemm_mode(gemm_mode)

    # ------------------------------------------------------------------ plumbing
    def _ck(self, rc):
        L.check(self.lib, self.ctx, rc)

    def set_gemm_mode(self, mode: int):
        self._ck(self.lib.b200_set_gemm_mode(self.ctx, int(mode)))

    def set_stream(self, cuda_stream_ptr):
        self._ck(self.lib.b200_set_stream(self.ctx, C.c_void_p(cuda_stream_ptr or 0)))

    def synchronize(self):
        self._ck(self.lib.b200_synchronize(self.ctx))

    def kernel_launches(self) -> int:
        return int(self.lib.b200_kernel_launches(self.ctx))

    def profile_gemm(self, enable: bool):
        self._ck(self.lib.b200_profile_gemm(self.ctx, int(bool(enable))))

    def gemm_profile(self, engine: int):
        """(launches, algorithmic FLOPs, device milliseconds) of the GEMM launches of one engine since profiling was enabled."""
        n, fl, ms = C.c_int64(0), C.c_double(0), C.c_double(0)
        self._ck(self.lib.b200_gemm_profile(self.ctx, int(engine), C.byref(n), C.byref(fl), C.byref(ms)))
        return n.value, fl.value, ms.value

    def gemm_profile_csv(self) -> str:
        buf = C.create_string_buffer(1 << 20)
        n = self.lib.b200_gemm_profile_csv(self.ctx, buf, len(buf))
        return buf.raw[:max(n, 0)].decode()

    def has_tcgen05(self) -> bool:
        return bool(self.lib.b200_has_tcgen05(self.ctx))

    def engine_launches(self) -> dict:
        """Launch counts per kernel family since the context was created (which path a call really took)."""
        out = (C.c_int64 * len(L.ENGINES))()
        self._ck(self.lib.b200_engine_launches(self.ctx, out))
        return dict(zip(L.ENGINES, (int(v) for v in out)))

    def set_gemm_kernel(self, kernel: int):
        """0 choose by shape; 1 / 128 / 256 / 512 force one tcgen05 GEMM kernel (tests, A/B measurements)."""
        self._ck(self.lib.b200_set_gemm_kernel(self.ctx, int(kernel)))

    def set_wait_budget_us(self, microseconds: int):
        self._ck(self.lib.b200_set_wait_budget_us(self.ctx, int(microseconds)))

    def probe_wait_timeout(self):
        """Runs the wait-expiry probe; raises B200Error(status 6, timeout) when the expiry path works."""
        self._ck(self.lib.b200_probe_wait_timeout(self.ctx))

    def Dispose(self):
        if getattr(self, "ctx", None):
            for child in list(self._children):
                child.close()
            self.lib.b200_destroy(self.ctx)
            self.ctx = None

    def __del__(self):
        try:
            self.Dispose()
        except Exception:
            pass

    # ------------------------------------------------------------------ shared tensor primitives
    def MatrixMultiply(self, A, B):
        A, B = _f(A), _f(B)
        out = np.zeros((A.shape[0], B.shape[1]), np.float32)
        self._ck(self.lib.b200_MatrixMultiply(self.ctx, _pf(A), A.shape[0], A.shape[1], _pf(B), B.shape[0], B.shape[1], _pf(out)))
        return out

    def MatrixMultiplyTranspose(self, A, B):
        A, B = _f(A), _f(B)
        out = np.zeros((A.shape[0], B.shape[0]), np.float32)
        self._ck(self.lib.b200_MatrixMultiplyTranspose(self.ctx, _pf(A), A.shape[0], A.shape[1], _pf(B), B.shape[0], B.shape[1], _pf(out)))
        return out

    def BatchDotProductAddBias(self, weights, inputMatrix, bias, rowStart=0, rowCount=None):
        W, X, b = _f(weights), _f(inputMatrix), _f(bias)
        rowCount = X.shape[0] - rowStart if rowCount is None else rowCount
        out = np.zeros((max(rowCount, 0), W.shape[0]), np.float32)
        self._ck(self.lib.b200_BatchDotProductAddBias(self.ctx, _pf(W), W.shape[0], W.shape[1], _pf(X), X.shape[0], X.shape[1], rowStart, rowCount,
                                                      _pf(b), b.shape[0], _pf(out)))
        return out

    def ProjectOutputBatch(self, hidden, outputProjection, outputBias, seqLen, outputDim):
        h, W, b = _f(hidden), _f(outputProjection), _f(outputBias)
        out = np.zeros((seqLen, outputDim), np.float32)
        self._ck(self.lib.b200_ProjectOutputBatch(self.ctx, _pf(h), h.shape[0], h.shape[1], _pf(W), _pf(b), seqLen, outputDim, _pf(out)))
        return out

    def MatrixAddInPlace(self, target, addend):
        t, a = _inplace(target, "target"), _f(addend)
        if a.shape != t.shape:
            raise ValueError("Matrix dimensions must match.")
        self._ck(self.lib.b200_MatrixAddInPlace(self.ctx, _pf(t), _pf(a), t.size))

    def VectorAccumulate(self, target, source):
        t, a = _inplace(target, "target"), _f(source)
        self._ck(self.lib.b200_VectorAccumulate(self.ctx, _pf(t), _pf(a), t.size))

    def ZeroMatrix(self, matrix):
        m = _inplace(matrix, "matrix")
        self._ck(self.lib.b200_ZeroMatrix(self.ctx, _pf(m), m.size))

    def ZeroVector(self, vector):
        v = _inplace(vector, "vector")
        self._ck(self.lib.b200_ZeroVector(self.ctx, _pf(v), v.size))

    # ------------------------------------------------------------------ layer norm
    def ResidualLayerNormForward(self, input, subLayer, gamma, beta, epsilon=1e-5):
        x, g, b = _f(input), _f(gamma), _f(beta)
        s = None if subLayer is None else _f(subLayer)
        if s is not None and s.shape != x.shape:
            raise ValueError("Residual input dimensions must match.")
        if g.shape[0] != x.shape[1] or b.shape[0] != x.shape[1]:
            raise ValueError("Layer norm gamma/beta must match the feature dimension.")
        rows, feat = x.shape
        out, norm, res = (np.zeros((rows, feat), np.float32) for _ in range(3))
        mean, var = np.zeros(rows, np.float32), np.zeros(rows, np.float32)
        self._ck(self.lib.b200_ResidualLayerNormForward(self.ctx, _pf(x), _pf(s), _pf(g), _pf(b), rows, feat, epsilon, _pf(out), _pf(mean), _pf(var),
                                                        _pf(norm), _pf(res)))
        return out, mean, var, norm, res

    def LayerNormForward(self, input, gamma, beta, epsilon=1e-5):
        return self.ResidualLayerNormForward(input, None, gamma, beta, epsilon)[:4]

    def LayerNorm(self, input, gamma, beta, epsilon=1e-5):
        return self.ResidualLayerNormForward(input, None, gamma, beta, epsilon)[0]

    def ResidualLayerNorm(self, input, subLayer, gamma, beta, epsilon=1e-5):
        return self.ResidualLayerNormForward(input, subLayer, gamma, beta, epsilon)[0]

    def LayerNormBackward(self, dOut, normalized, gamma, input, mean, variance, epsilon=1e-5):
        d, n, g, x, m, v = _f(dOut), _f(normalized), _f(gamma), _f(input), _f(mean), _f(variance)
        rows, feat = d.shape
        dIn, dG, dB = np.zeros((rows, feat), np.float32), np.zeros(feat, np.float32), np.zeros(feat, np.float32)
        self._ck(self.lib.b200_LayerNormBackward(self.ctx, _pf(d), _pf(n), _pf(g), _pf(x), _pf(m), _pf(v), rows, feat, epsilon, _pf(dIn), _pf(dG), _pf(dB)))
        return dIn, dG, dB

    # ------------------------------------------------------------------ attention
    def ScaledDotProductAttention(self, q, k, v, numHeads, mask=None, causal=False):
        q, k, v = _f(q), _f(k), _f(v)
        if k.shape[1] != q.shape[1] or v.shape[1] != q.shape[1]:
            raise ValueError("K/V width must match Q width.")
        if v.shape[0] != k.shape[0]:
            raise ValueError("V row count must match K row count.")
        keep, pm = _mask(mask)
        if keep is not None and keep.shape != (q.shape[0], k.shape[0]):
            raise ValueError(f"Mask shape must be [{q.shape[0]},{k.shape[0]}], got {list(keep.shape)}.")
        out = np.zeros_like(q)
        self._ck(self.lib.b200_ScaledDotProductAttention(self.ctx, _pf(q), _pf(k), _pf(v), q.shape[0], k.shape[0], q.shape[1], numHeads, pm,
                                                         int(bool(causal)), _pf(out)))
        return out

    def MultiHeadAttentionForward(self, Q, K, V, numHeads, scale, mask=None):
        q, k, v = _f(Q), _f(K), _f(V)
        keep, pm = _mask(mask)
        out = np.zeros_like(q)
        self._ck(self.lib.b200_MultiHeadAttentionForward(self.ctx, _pf(q), _pf(k), _pf(v), q.shape[0], k.shape[0], q.shape[1], numHeads, scale, pm, _pf(out)))
        return out

    def MultiHeadAttentionBackward(self, Q, K, V, dConcatenated, numHeads, scale, mask=None, useDecoderMask=False):
        """Both reference overloads: pass ``useDecoderMask=True`` or an explicit boolean ``mask``."""
        q, k, v, d = _f(Q), _f(K), _f(V), _f(dConcatenated)
        if k.shape[1] != q.shape[1] or v.shape[1] != q.shape[1]:
            raise ValueError("Q, K and V must have the same embedding dimension.")
        if v.shape[0] != k.shape[0]:
            raise ValueError("K and V must have the same sequence length.")
        if d.shape != q.shape:
            raise ValueError("dConcatenated shape must match Q shape.")
        keep, pm = _mask(mask)
        if keep is not None and keep.shape != (q.shape[0], k.shape[0]):
            raise ValueError(f"Mask shape must be [{q.shape[0]},{k.shape[0]}], got {list(keep.shape)}.")
        dQ, dK, dV = np.zeros_like(q), np.zeros_like(k), np.zeros_like(v)
        self._ck(self.lib.b200_MultiHeadAttentionBackward(self.ctx, _pf(q), _pf(k), _pf(v), _pf(d), q.shape[0], k.shape[0], q.shape[1], numHeads, scale,
                                                          pm, int(bool(useDecoderMask)), _pf(dQ), _pf(dK), _pf(dV)))
        return dQ, dK, dV

    def SegmentedAttentionForward(self, Q, K, V, segmentLength, segmentCount, numHeads, causal=True):
        q, k, v = _f(Q), _f(K), _f(V)
        if q.shape[0] != segmentLength * segmentCount:
            raise ValueError("Invalid segmented attention shape.")
        out = np.zeros_like(q)
        self._ck(self.lib.b200_SegmentedAttentionForward(self.ctx, _pf(q), _pf(k), _pf(v), segmentLength, segmentCount, q.shape[1], numHeads,
                                                         int(bool(causal)), _pf(out)))
        return out

    def SegmentedAttentionBackward(self, Q, K, V, dConcatenated, segmentLength, segmentCount, numHeads, scale, causal=True):
        q, k, v, d = _f(Q), _f(K), _f(V), _f(dConcatenated)
        if q.shape[0] != segmentLength * segmentCount:
            raise ValueError("Invalid segmented attention backward shape.")
        dQ, dK, dV = np.zeros_like(q), np.zeros_like(k), np.zeros_like(v)
        self._ck(self.lib.b200_SegmentedAttentionBackward(self.ctx, _pf(q), _pf(k), _pf(v), _pf(d), segmentLength, segmentCount, q.shape[1], numHeads,
                                                          scale, int(bool(causal)), _pf(dQ), _pf(dK), _pf(dV)))
        return dQ, dK, dV

    def ApplyRotaryPositionEmbeddingInPlace(self, matrix, numHeads, baseTheta=10000.0, inverse=False, segmentLength=0):
        m = _inplace(matrix, "matrix")
        self._ck(self.lib.b200_ApplyRotaryPositionEmbeddingInPlace(self.ctx, _pf(m), m.shape[0], m.shape[1], numHeads, baseTheta, int(bool(inverse)),
                                                                   segmentLength))

    def ApplyRotaryPositionEmbeddingHeadInPlace(self, matrix, startCol, headDim, baseTheta=10000.0, inverse=False):
        m = _inplace(matrix, "matrix")
        self._ck(self.lib.b200_ApplyRotaryPositionEmbeddingHeadInPlace(self.ctx, _pf(m), m.shape[0], m.shape[1], startCol, headDim, baseTheta,
                                                                       int(bool(inverse))))

    # ------------------------------------------------------------------ projections
    def ProjectQKV(self, input, WQ, biasQ, WK, biasK, WV, biasV):
        x, wq, bq, wk, bk, wv, bv = map(_f, (input, WQ, biasQ, WK, biasK, WV, biasV))
        for w, n in ((wq, "WQ"), (wk, "WK"), (wv, "WV")):
            if w.shape[1] != x.shape[1]:
                raise ValueError(f"{n} input dimension does not match input width.")
        if not (wq.shape[0] == wk.shape[0] == wv.shape[0]):
            raise ValueError("Q, K and V output dimensions must match.")
        for b, w, n in ((bq, wq, "biasQ"), (bk, wk, "biasK"), (bv, wv, "biasV")):
            if b.shape[0] != w.shape[0]:
                raise ValueError(f"{n} length does not match the output dimension.")
        rows, out = x.shape[0], wq.shape[0]
        Q, K, V = (np.zeros((rows, out), np.float32) for _ in range(3))
        self._ck(self.lib.b200_ProjectQKV(self.ctx, _pf(x), rows, x.shape[1], _pf(wq), _pf(bq), _pf(wk), _pf(bk), _pf(wv), _pf(bv), out, _pf(Q), _pf(K), _pf(V)))
        return Q, K, V

    def ProjectKV(self, input, WK, biasK, WV, biasV):
        x, wk, bk, wv, bv = map(_f, (input, WK, biasK, WV, biasV))
        if wk.shape[0] != wv.shape[0]:
            raise ValueError("K and V output dimensions must match.")
        for w, n in ((wk, "WK"), (wv, "WV")):
            if w.shape[1] != x.shape[1]:
                raise ValueError(f"{n} input dimension does not match input width.")
        for b, w, n in ((bk, wk, "biasK"), (bv, wv, "biasV")):
            if b.shape[0] != w.shape[0]:
                raise ValueError(f"{n} length does not match the output dimension.")
        rows, out = x.shape[0], wk.shape[0]
        K, V = (np.zeros((rows, out), np.float32) for _ in range(2))
        self._ck(self.lib.b200_ProjectKV(self.ctx, _pf(x), rows, x.shape[1], _pf(wk), _pf(bk), _pf(wv), _pf(bv), out, _pf(K), _pf(V)))
        return K, V

    def BackpropKV(self, input, dK, dV, WK, WV, WKGrad, biasKGrad, WVGrad, biasVGrad):
        x, dk, dv, wk, wv = map(_f, (input, dK, dV, WK, WV))
        grads = [_inplace(g, "gradient") for g in (WKGrad, biasKGrad, WVGrad, biasVGrad)]
        rows, inp, out = x.shape[0], x.shape[1], wk.shape[0]
        if not (wk.shape == wv.shape == (out, inp)):
            raise ValueError("K/V weight input dimensions must match input width.")
        if not (dk.shape == dv.shape == (rows, out)):
            raise ValueError("dK and dV must be [rows, outputDim].")
        for g in grads[0::2]:
            if g.shape != (out, inp):
                raise ValueError("Weight gradient shape mismatch.")
        for g in grads[1::2]:
            if g.shape != (out,):
                raise ValueError("K/V bias gradient lengths must match output dimension.")
        dIn = np.zeros_like(x)
        self._ck(self.lib.b200_BackpropKV(self.ctx, _pf(x), rows, inp, _pf(dk), _pf(dv), out, _pf(wk), _pf(wv), *[_pf(g) for g in grads], _pf(dIn)))
        return dIn

    def BackpropQKV(self, input, dQ, dK, dV, WQ, WK, WV, WQGrad, biasQGrad, WKGrad, biasKGrad, WVGrad, biasVGrad):
        x, dq, dk, dv, wq, wk, wv = map(_f, (input, dQ, dK, dV, WQ, WK, WV))
        grads = [_inplace(g, "gradient") for g in (WQGrad, biasQGrad, WKGrad, biasKGrad, WVGrad, biasVGrad)]
        rows, inp, out = x.shape[0], x.shape[1], wq.shape[0]
        if not (wq.shape == wk.shape == wv.shape == (out, inp)):
            raise ValueError("Weight shapes must match [outputDim, inputDim].")
        if not (dq.shape == dk.shape == dv.shape == (rows, out)):
            raise ValueError("dQ, dK and dV must be [rows, outputDim].")
        for g in grads[0::2]:
            if g.shape != (out, inp):
                raise ValueError("Weight gradient shape mismatch.")
        for g in grads[1::2]:
            if g.shape != (out,):
                raise ValueError("Bias gradient length mismatch.")
        dIn = np.zeros_like(x)
        self._ck(self.lib.b200_BackpropQKV(self.ctx, _pf(x), rows, inp, _pf(dq), _pf(dk), _pf(dv), out, _pf(wq), _pf(wk), _pf(wv), *[_pf(g) for g in grads],
                                           _pf(dIn)))
        return dIn

    def BackpropLinearProjection(self, input, dOutput, weights, weightGrad, biasGrad, dInput):
        x, dy, w = _f(input), _f(dOutput), _f(weights)
        wg, bg, di = _inplace(weightGrad, "weightGrad"), _inplace(biasGrad, "biasGrad"), _inplace(dInput, "dInput")
        self._ck(self.lib.b200_BackpropLinearProjection(self.ctx, _pf(x), _pf(dy), _pf(w), x.shape[0], x.shape[1], dy.shape[1], _pf(wg), _pf(bg), _pf(di)))

    def BackpropOutputProjection(self, dLogits, input, weights, weightGrad, biasGrad, seqLen, outputDim, embeddingDim):
        dl, x, w = _f(dLogits), _f(input), _f(weights)
        wg, bg = _inplace(weightGrad, "weightGrad"), _inplace(biasGrad, "biasGrad")
        dX = np.zeros((seqLen, embeddingDim), np.float32)
        self._ck(self.lib.b200_BackpropOutputProjection(self.ctx, _pf(dl), _pf(x), _pf(w), _pf(wg), _pf(bg), seqLen, outputDim, embeddingDim, _pf(dX)))
        return dX

    def BackpropInputProjection(self, dX, continuousInput, weightGrad, biasGrad, seqLen, embeddingDim, inputFeatureDim, inputRowStart=0):
        d, c = _f(dX), _f(continuousInput)
        wg, bg = _inplace(weightGrad, "weightGrad"), _inplace(biasGrad, "biasGrad")
        self._ck(self.lib.b200_BackpropInputProjection(self.ctx, _pf(d), d.shape[0], d.shape[1], _pf(c), c.shape[0], c.shape[1], inputRowStart, _pf(wg), _pf(bg),
                                                       seqLen, embeddingDim, inputFeatureDim))

    def EmbedTokenIds(self, tokenIds, embedding, embeddingDim, tokenStart=0, tokenCount=None):
        ids = _i(tokenIds)
        tokenCount = len(ids) - tokenStart if tokenCount is None else tokenCount
        if len(ids) == 0 or tokenCount == 0:
            return np.zeros((0, embeddingDim), np.float32)
        E = _f(embedding)
        if E.shape[1] != embeddingDim:
            raise ValueError("Embedding width must match embeddingDim.")
        out = np.zeros((max(tokenCount, 0), embeddingDim), np.float32)
        self._ck(self.lib.b200_EmbedTokenIds(self.ctx, _pi(ids), len(ids), tokenStart, tokenCount, _pf(E), E.shape[0], embeddingDim, _pf(out)))
        return out

    def AccumulateTokenEmbeddingGrad(self, embeddingGrad, dX, tokenIds, seqLen, embeddingDim, tokenStart=0):
        eg, d, ids = _inplace(embeddingGrad, "embeddingGrad"), _f(dX), _i(tokenIds)
        self._ck(self.lib.b200_AccumulateTokenEmbeddingGrad(self.ctx, _pf(eg), eg.shape[0], _pf(d), _pi(ids), len(ids), tokenStart, seqLen, embeddingDim))

    # ------------------------------------------------------------------ losses
    def CrossEntropyLossAndGradient(self, logits, targets, effectiveLen, targetStart=0):
        l, t = _f(logits), _i(targets)
        d = np.zeros_like(l)
        loss = C.c_float(0)
        self._ck(self.lib.b200_CrossEntropyLossAndGradient(self.ctx, _pf(l), l.shape[0], l.shape[1], _pi(t), len(t), targetStart, effectiveLen,
                                                           C.byref(loss), _pf(d)))
        return np.float32(loss.value), d

    def MSELossAndGradient(self, predictions, targets, effectiveLen, targetStart=0):
        p, t = _f(predictions), _f(targets)
        if t.ndim != 2 or t.shape[1] != p.shape[1]:
            raise IndexError("targets must be [rows, outputDim]")
        d = np.zeros_like(p)
        loss = C.c_float(0)
        self._ck(self.lib.b200_MSELossAndGradient(self.ctx, _pf(p), p.shape[0], p.shape[1], _pf(t), t.shape[0], targetStart, effectiveLen, C.byref(loss), _pf(d)))
        return np.float32(loss.value), d

    # ------------------------------------------------------------------ step primitives
    def MatrixSquaredNorm(self, matrix):
        m = _f(matrix)
        out = C.c_float(0)
        self._ck(self.lib.b200_MatrixSquaredNorm(self.ctx, _pf(m), m.size, C.byref(out)))
        return np.float32(out.value)

    VectorSquaredNorm = MatrixSquaredNorm

    def MatrixScaleInPlace(self, matrix, scale):
        m = _inplace(matrix, "matrix")
        self._ck(self.lib.b200_MatrixScaleInPlace(self.ctx, _pf(m), m.size, scale))

    VectorScaleInPlace = MatrixScaleInPlace

    def MatrixUpdate(self, weights, gradients, learningRate):
        w, g = _inplace(weights, "weights"), _f(gradients)
        if g.shape != w.shape:
            raise ValueError("Gradient shape must match weight shape.")
        self._ck(self.lib.b200_MatrixUpdate(self.ctx, _pf(w), _pf(g), w.size, learningRate))

    VectorUpdate = MatrixUpdate

    # ------------------------------------------------------------------ feed-forward network (NeuralNetwork batch paths)
    def _net(self, widths, acts, weights, biases, writable=False):
        n = len(widths)
        if len(weights) != n - 1 or len(biases) != n - 1:
            raise ValueError("one weight matrix and one bias vector per non-input layer")
        wa, ba = (C.c_void_p * n)(), (C.c_void_p * n)()
        keep = []
        for l in range(1, n):
            w = _inplace(weights[l - 1], "weight gradient") if writable else _f(weights[l - 1])
            b = _inplace(biases[l - 1], "bias gradient") if writable else _f(biases[l - 1])
            if w.shape != (widths[l], widths[l - 1]) or b.shape != (widths[l],):
                raise ValueError(f"layer {l}: expected weights {(widths[l], widths[l - 1])} and bias {(widths[l],)}")
            keep += [w, b]
            wa[l], ba[l] = w.ctypes.data, b.ctypes.data
        wd = np.asarray(widths, np.int32)
        ac = np.asarray([L.ACT[a] if isinstance(a, str) else int(a) for a in acts], np.int32)
        return wd, ac, wa, ba, keep

    def FFNForwardBatch(self, input, widths, activations, weights, biases):
        """IAccelerationManager.FFNForwardBatch for a delegate bound to a NeuralNetwork (= ForwardPassOnlyBatch)."""
        x = _f(input)
        if x.shape[1] != widths[0]:
            raise ValueError(f"Input matrix column count ({x.shape[1]}) must match network input size ({widths[0]}).")
        wd, ac, wa, ba, keep = self._net(widths, activations, weights, biases)
        out = np.zeros((x.shape[0], widths[-1]), np.float32)
        self._ck(self.lib.b200_FFNForwardBatch(self.ctx, _pf(x), x.shape[0], len(widths), _pi(wd), _pi(ac), wa, ba, _pf(out)))
        return out

    def FFNInputGradientBatch(self, input, dOutput, widths, activations, weights, biases, weightGradients=None, biasGradients=None):
        """NeuralNetwork.ComputeInputGradientBatch; gradient lists (one entry per non-input layer) accumulate in place."""
        x, d = _f(input), _f(dOutput)
        if d.shape[0] != x.shape[0]:
            raise ValueError("dOutput row count must match input row count.")
        if (weightGradients is None) != (biasGradients is None):
            raise ValueError("weightGradients and biasGradients must either both be null or both be supplied.")
        wd, ac, wa, ba, keep = self._net(widths, activations, weights, biases)
        ga = gb = None
        if weightGradients is not None:
            _, _, ga, gb, keep2 = self._net(widths, activations, weightGradients, biasGradients, writable=True)
        dIn = np.zeros_like(x)
        self._ck(self.lib.b200_FFNInputGradientBatch(self.ctx, _pf(x), _pf(d), x.shape[0], len(widths), _pi(wd), _pi(ac), wa, ba, ga, gb, _pf(dIn)))
        return dIn

    # ------------------------------------------------------------------ sibling trainers' operators (TACAMT / MMTAC / PriceTAC)
    def ContentAwareCrossAttentionForward(self, Q, K, V, numHeads, scale, decayBias=None, needBackwardCache=True):
        """Returns (output, attentionWeights, scoresPreSoftmax); the last two are [numHeads, queryLen, keyLen] arrays
        (the reference's float[numHeads][,]) or None when needBackwardCache is false."""
        q, k, v = _f(Q), _f(K), _f(V)
        qn, e, kn = q.shape[0], q.shape[1], k.shape[0]
        if k.shape != (kn, e) or v.shape != (kn, e):
            raise ValueError("K and V must be [keyLen, embDim] with Q's embedding width.")
        b = None
        if decayBias is not None:
            b = _f(decayBias)
            if b.shape != (qn, kn, numHeads):
                raise ValueError("decayBias must be [queryLen, keyLen, numHeads].")
        out = np.zeros((qn, e), np.float32)
        w = np.zeros((numHeads, qn, kn), np.float32) if needBackwardCache else None
        s = np.zeros((numHeads, qn, kn), np.float32) if needBackwardCache else None
        self._ck(self.lib.b200_ContentAwareCrossAttentionForward(self.ctx, _pf(q), qn, _pf(k), _pf(v), kn, e, int(numHeads), float(scale), _pf(b),
                                                                 _pf(out), _pf(w), _pf(s)))
        return out, w, s

    def BackpropTimeDecayedAttention(self, q, k, v, dOutput, attentionWeights, timeDiffs, embeddingDim, numHeads):
        """Returns (dQ, dK, dV, dDecayBias); dDecayBias is None when timeDiffs is None, as in the reference."""
        qq, kk, vv, do = _f(q), _f(k), _f(v), _f(dOutput)
        w = _f(attentionWeights)
        qn, kn = qq.shape[0], kk.shape[0]
        if w.shape != (numHeads, qn, kn):
            raise ValueError("attentionWeights must be [numHeads, queryLen, keyLen].")
        if qq.shape[1] != embeddingDim or kk.shape != (kn, embeddingDim) or vv.shape != (kn, embeddingDim) or do.shape != (qn, embeddingDim):
            raise ValueError("q, k, v and dOutput must have embeddingDim columns and matching row counts.")
        dQ, dK, dV = np.zeros_like(qq), np.zeros_like(kk), np.zeros_like(vv)
        dB = np.zeros((qn, kn, numHeads), np.float32) if timeDiffs is not None else None
        self._ck(self.lib.b200_BackpropTimeDecayedAttention(self.ctx, _pf(qq), qn, _pf(kk), _pf(vv), kn, _pf(do), _pf(w), int(embeddingDim),
                                                            int(numHeads), _pf(dQ), _pf(dK), _pf(dV), _pf(dB)))
        return dQ, dK, dV, dB

    def ApplyContextTypeEmbedding(self, contextHidden, typeEmbedding, typeIndices):
        h, t, idx = _inplace(contextHidden, "contextHidden"), _f(typeEmbedding), _i(typeIndices)
        if len(idx) != h.shape[0]:
            raise ValueError("typeIndices length must match contextHidden row count.")
        if t.shape[1] != h.shape[1]:
            raise ValueError("typeEmbedding dimension must match contextHidden embedding dimension.")
        self._ck(self.lib.b200_ApplyContextTypeEmbedding(self.ctx, _pf(h), h.shape[0], h.shape[1], _pf(t), t.shape[0], _pi(idx)))

    def ComputeTimeDiffMatrix(self, priceSeqLen, keyArrivalTimes):
        t = _f(keyArrivalTimes)
        out = np.zeros((max(int(priceSeqLen), 0), len(t)), np.float32)
        self._ck(self.lib.b200_ComputeTimeDiffMatrix(self.ctx, int(priceSeqLen), _pf(t), len(t), _pf(out)))
        return out

    def ComputeMemoryAttentionScores(self, priceHidden, lastPos, contextHidden, totalCtx, scale):
        p, c = _f(priceHidden), _f(contextHidden)
        if c.shape[0] < totalCtx or c.shape[1] != p.shape[1]:
            raise IndexError("contextHidden must hold totalCtx rows of priceHidden's width.")
        out = np.zeros(totalCtx, np.float32)
        self._ck(self.lib.b200_ComputeMemoryAttentionScores(self.ctx, _pf(p), p.shape[0], p.shape[1], int(lastPos), _pf(c), int(totalCtx),
                                                            float(scale), _pf(out)))
        return out

    def ProjectGlobalFeatures(self, globalFeatures, projection, bias):
        g, P, b = _f(globalFeatures), _f(projection), _f(bias)
        ed, gd = P.shape
        if len(g) != gd:
            raise ValueError(f"Expected global feature length {gd}, got {len(g)}.")
        if len(b) != ed:
            raise ValueError(f"Expected bias length {ed}, got {len(b)}.")
        out = np.zeros(ed, np.float32)
        self._ck(self.lib.b200_ProjectGlobalFeatures(self.ctx, _pf(g), gd, _pf(P), _pf(b), ed, _pf(out)))
        return out

    def MeanPoolRows(self, matrix):
        m = _f(matrix)
        out = np.zeros(m.shape[1], np.float32)
        self._ck(self.lib.b200_MeanPoolRows(self.ctx, _pf(m), m.shape[0], m.shape[1], _pf(out)))
        return out

    def ExpandMeanPoolGradient(self, pooledGradient, rowIndex, rowCount, embeddingDim):
        g = _f(pooledGradient)
        out = np.zeros((max(int(rowCount), 0), embeddingDim), np.float32)
        self._ck(self.lib.b200_ExpandMeanPoolGradient(self.ctx, _pf(g), g.shape[0], g.shape[1], int(rowIndex), int(rowCount), int(embeddingDim),
                                                      _pf(out)))
        return out

    def SoftmaxVector(self, scores):
        s = _f(scores)
        out = np.zeros(len(s), np.float32)
        self._ck(self.lib.b200_SoftmaxVector(self.ctx, _pf(s), len(s), _pf(out)))
        return out

    def SigmoidInPlace(self, matrix):
        m = _inplace(matrix, "matrix")
        self._ck(self.lib.b200_SigmoidInPlace(self.ctx, _pf(m), m.size))

    def ZeroMatrixColumns(self, matrix, columnCount):
        m = _inplace(matrix, "matrix")
        self._ck(self.lib.b200_ZeroMatrixColumns(self.ctx, _pf(m), m.shape[0], m.shape[1], int(columnCount)))

    def VectorUpdateClamped(self, weights, gradients, learningRate, minValue, maxValue):
        w, g = _inplace(weights, "weights"), _f(gradients)
        if g.shape != w.shape:
            raise ValueError("weights and gradients must have the same length.")
        self._ck(self.lib.b200_VectorUpdateClamped(self.ctx, _pf(w), _pf(g), w.size, float(learningRate), float(minValue), float(maxValue)))

    def AccumulateGlobalProjectionGradients(self, dGlobalHidden, globalFeatures, projectionGrad, biasGrad):
        if dGlobalHidden is None or globalFeatures is None or projectionGrad is None or biasGrad is None:
            return  # the reference returns silently
        d, g = _f(dGlobalHidden), _f(globalFeatures)
        pg, bg = _inplace(projectionGrad, "projectionGrad"), _inplace(biasGrad, "biasGrad")
        if pg.shape != (len(d), len(g)) or bg.shape != (len(d),):
            raise IndexError("gradient shapes must be [len(dGlobalHidden), len(globalFeatures)] and [len(dGlobalHidden)].")
        self._ck(self.lib.b200_AccumulateGlobalProjectionGradients(self.ctx, _pf(d), len(d), _pf(g), len(g), _pf(pg), _pf(bg)))

    def Matrix3DScaleInPlace(self, matrix, scale):
        m = _inplace(matrix, "matrix")
        self._ck(self.lib.b200_Matrix3DScaleInPlace(self.ctx, _pf(m), m.size, float(scale)))

    def MatrixSquaredNorm3D(self, matrix):
        m = _f(matrix)
        out = C.c_float(0)
        self._ck(self.lib.b200_MatrixSquaredNorm3D(self.ctx, _pf(m), m.size, C.byref(out)))
        return np.float32(out.value)

    def Matrix3DAddInPlace(self, target, addend):
        t, a = _inplace(target, "target"), _f(addend)
        if a.shape != t.shape:
            raise ValueError("3D tensor shape mismatch.")
        self._ck(self.lib.b200_Matrix3DAddInPlace(self.ctx, _pf(t), _pf(a), t.size))

    def Matrix3DUpdate(self, weights, gradients, learningRate):
        w, g = _inplace(weights, "weights"), _f(gradients)
        if g.shape != w.shape:
            raise ValueError("3D tensor shape mismatch.")
        self._ck(self.lib.b200_Matrix3DUpdate(self.ctx, _pf(w), _pf(g), w.size, float(learningRate)))
