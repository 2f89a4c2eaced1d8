"""GPU parity of the sibling trainers' operators (IAccelerationManager.cs:251-361) through the C ABI against the CPU
oracle: the reference's own parity-test inputs (AccelerationManagerParityTests.cs:856-878, 967-993), larger ragged
shapes, -inf scores, empty inputs and the reference's argument errors.  FP32 kernels: |exp-act| <= 1e-5*max(1,|exp|)."""
import numpy as np
import pytest

from conftest import assert_close
from oracle import Oracle, pt_matrix, pt_tensor3, pt_vector

pytestmark = pytest.mark.gpu
TOL = 1e-5


@pytest.fixture(scope="module")
def mgr():
    from callaghandev.ml_b200 import GEMM_FP32_SIMT, CudaB200AccelerationManager

    m = CudaB200AccelerationManager(0, GEMM_FP32_SIMT)
    yield m
    m.Dispose()


@pytest.fixture(scope="module")
def oracle():
    return Oracle(threads=8)


@pytest.mark.parametrize("seq,ctx,ed,heads,seed", [(3, 4, 6, 2, 80), (37, 301, 64, 4, 5), (130, 77, 96, 3, 9), (1, 1, 8, 8, 2)])
def test_content_aware_cross_attention_forward(mgr, oracle, seq, ctx, ed, heads, seed):
    scale = 1.0 / np.sqrt(ed // heads)
    q, k, v, bias = pt_matrix(seq, ed, seed), pt_matrix(ctx, ed, seed + 1), pt_matrix(ctx, ed, seed + 2), pt_tensor3(seq, ctx, heads, seed + 3)
    for b in (bias, None):
        for e, a, n in zip(oracle.ContentAwareCrossAttentionForward(q, k, v, heads, scale, b),
                           mgr.ContentAwareCrossAttentionForward(q, k, v, heads, scale, b), ("output", "attentionWeights", "scoresPreSoftmax")):
            assert_close(e, a, TOL, "ContentAwareCrossAttentionForward." + n)
    out, w, s = mgr.ContentAwareCrossAttentionForward(q, k, v, heads, scale, bias, needBackwardCache=False)
    assert w is None and s is None
    assert_close(oracle.ContentAwareCrossAttentionForward(q, k, v, heads, scale, bias)[0], out, TOL, "output without cache")


def test_content_aware_cross_attention_masked_and_empty(mgr, oracle):
    seq, ctx, ed, heads = 5, 9, 8, 2
    q, k, v, bias = pt_matrix(seq, ed, 1), pt_matrix(ctx, ed, 2), pt_matrix(ctx, ed, 3), pt_tensor3(seq, ctx, heads, 4)
    bias[0, 1, :] = -np.inf   # one key removed for one query
    bias[2, :, 1] = -np.inf   # a row with nothing left in head 1: zero weights, zero output, scores stay -inf
    for e, a, n in zip(oracle.ContentAwareCrossAttentionForward(q, k, v, heads, 0.5, bias), mgr.ContentAwareCrossAttentionForward(q, k, v, heads, 0.5, bias), "OWS"):
        assert_close(e, a, TOL, "masked." + n)
    out, w, s = mgr.ContentAwareCrossAttentionForward(q, k, v, heads, 0.5, bias)
    assert np.all(w[1, 2] == 0) and np.all(out[2, 4:] == 0) and np.all(np.isneginf(s[1, 2]))
    out, w, s = mgr.ContentAwareCrossAttentionForward(q, np.zeros((0, ed), np.float32), np.zeros((0, ed), np.float32), heads, 0.5)
    assert out.shape == (seq, ed) and np.all(out == 0) and w.shape == (heads, seq, 0)
    assert mgr.ContentAwareCrossAttentionForward(np.zeros((0, ed), np.float32), k, v, heads, 0.5)[0].shape == (0, ed)
    with pytest.raises(ValueError):
        mgr.ContentAwareCrossAttentionForward(q, k, v, 3, 0.5)          # 8 columns, 3 heads
    with pytest.raises(ValueError):
        mgr.ContentAwareCrossAttentionForward(q, k, v[:, :4], heads, 0.5)


@pytest.mark.parametrize("seq,ctx,ed,heads,seed", [(3, 4, 6, 2, 91), (37, 301, 64, 4, 15), (130, 77, 96, 3, 19)])
def test_backprop_time_decayed_attention(mgr, oracle, seq, ctx, ed, heads, seed):
    scale = 1.0 / np.sqrt(ed // heads)
    q, k, v, decay = pt_matrix(seq, ed, seed), pt_matrix(ctx, ed, seed + 1), pt_matrix(ctx, ed, seed + 2), pt_tensor3(seq, ctx, heads, seed + 3)
    _, W, _ = oracle.ContentAwareCrossAttentionForward(q, k, v, heads, scale, decay)
    dO, td = pt_matrix(seq, ed, seed + 4), pt_matrix(seq, ctx, seed + 5)
    for e, a, n in zip(oracle.BackpropTimeDecayedAttention(q, k, v, dO, W, td, ed, heads),
                       mgr.BackpropTimeDecayedAttention(q, k, v, dO, W, td, ed, heads), ("dQ", "dK", "dV", "dDecayBias")):
        assert_close(e, a, TOL, "BackpropTimeDecayedAttention." + n)
    got = mgr.BackpropTimeDecayedAttention(q, k, v, dO, W, None, ed, heads)
    assert got[3] is None
    assert_close(oracle.BackpropTimeDecayedAttention(q, k, v, dO, W, None, ed, heads)[0], got[0], TOL, "dQ without time differences")
    with pytest.raises(ValueError):
        mgr.BackpropTimeDecayedAttention(q, k, v, dO, W[:, :, :-1], td, ed, heads)


def test_context_helpers(mgr, oracle):
    h, t, idx = pt_matrix(50, 64, 1), pt_matrix(3, 64, 2), (np.arange(50) % 3).astype(np.int32)
    he, ha = h.copy(), h.copy()
    oracle.ApplyContextTypeEmbedding(he, t, idx); mgr.ApplyContextTypeEmbedding(ha, t, idx)
    assert_close(he, ha, TOL, "ApplyContextTypeEmbedding")
    with pytest.raises(IndexError):
        mgr.ApplyContextTypeEmbedding(ha, t, np.full(50, 3, np.int32))
    with pytest.raises(ValueError):
        mgr.ApplyContextTypeEmbedding(ha, t, idx[:-1])
    times = pt_vector(33, 3) * 100
    assert np.array_equal(oracle.ComputeTimeDiffMatrix(17, times), mgr.ComputeTimeDiffMatrix(17, times))
    with pytest.raises(IndexError):
        mgr.ComputeTimeDiffMatrix(0, times)
    p, c = pt_matrix(40, 96, 4), pt_matrix(300, 96, 5)
    assert_close(oracle.ComputeMemoryAttentionScores(p, 39, c, 257, 0.1), mgr.ComputeMemoryAttentionScores(p, 39, c, 257, 0.1), TOL, "ComputeMemoryAttentionScores")
    g, P, b = pt_vector(23, 6), pt_matrix(64, 23, 7), pt_vector(64, 8)
    assert_close(oracle.ProjectGlobalFeatures(g, P, b), mgr.ProjectGlobalFeatures(g, P, b), TOL, "ProjectGlobalFeatures")
    with pytest.raises(ValueError):
        mgr.ProjectGlobalFeatures(g[:-1], P, b)
    m = pt_matrix(301, 70, 9)
    assert_close(oracle.MeanPoolRows(m), mgr.MeanPoolRows(m), TOL, "MeanPoolRows")
    assert np.all(mgr.MeanPoolRows(np.zeros((0, 5), np.float32)) == 0)
    assert np.array_equal(oracle.ExpandMeanPoolGradient(m, 7, 13, 64), mgr.ExpandMeanPoolGradient(m, 7, 13, 64))
    assert mgr.ExpandMeanPoolGradient(m, 7, 0, 64).shape == (0, 64)
    with pytest.raises(IndexError):
        mgr.ExpandMeanPoolGradient(m, 301, 2, 64)
    s = pt_vector(1000, 10) * 30
    assert_close(oracle.SoftmaxVector(s), mgr.SoftmaxVector(s), TOL, "SoftmaxVector")
    assert mgr.SoftmaxVector(np.zeros(0, np.float32)).shape == (0,)


def test_in_place_helpers(mgr, oracle):
    x = (pt_matrix(37, 53, 11) * 200).astype(np.float32)
    xe, xa = x.copy(), x.copy()
    oracle.SigmoidInPlace(xe); mgr.SigmoidInPlace(xa)
    assert_close(xe, xa, TOL, "SigmoidInPlace")
    z = pt_matrix(19, 31, 12)
    for count in (0, -3, 7, 31, 99):
        ze, za = z.copy(), z.copy()
        oracle.ZeroMatrixColumns(ze, count); mgr.ZeroMatrixColumns(za, count)
        assert np.array_equal(ze, za)
    w, gr = pt_vector(5000, 13), pt_vector(5000, 14)
    we, wa = w.copy(), w.copy()
    oracle.VectorUpdateClamped(we, gr, 0.5, -0.1, 0.15); mgr.VectorUpdateClamped(wa, gr, 0.5, -0.1, 0.15)
    assert_close(we, wa, TOL, "VectorUpdateClamped")
    with pytest.raises(ValueError):
        mgr.VectorUpdateClamped(wa, gr, 0.5, 1.0, -1.0)
    d, gf, pg, bg = pt_vector(64, 15), pt_vector(23, 16), pt_matrix(64, 23, 17), pt_vector(64, 18)
    pe, be, pa, ba = pg.copy(), bg.copy(), pg.copy(), bg.copy()
    oracle.AccumulateGlobalProjectionGradients(d, gf, pe, be); mgr.AccumulateGlobalProjectionGradients(d, gf, pa, ba)
    assert_close(pe, pa, TOL, "projectionGrad"); assert_close(be, ba, TOL, "biasGrad")
    mgr.AccumulateGlobalProjectionGradients(None, gf, pa, ba)  # silently ignored, as in the reference
    assert_close(pe, pa, TOL, "projectionGrad untouched")


def test_rank3_elementwise(mgr):
    t = pt_tensor3(7, 9, 5, 1)
    a = t.copy()
    mgr.Matrix3DScaleInPlace(a, 0.37)
    assert_close(t * np.float32(0.37), a, TOL, "Matrix3DScaleInPlace")
    assert_close(np.sum(t.astype(np.float64) ** 2), mgr.MatrixSquaredNorm3D(t), TOL, "MatrixSquaredNorm3D")
    b = pt_tensor3(7, 9, 5, 2)
    a = t.copy(); mgr.Matrix3DAddInPlace(a, b)
    assert_close(t + b, a, TOL, "Matrix3DAddInPlace")
    a = t.copy(); mgr.Matrix3DUpdate(a, b, 0.25)
    assert_close(t - np.float32(0.25) * b, a, TOL, "Matrix3DUpdate")
    with pytest.raises(ValueError):
        mgr.Matrix3DAddInPlace(a, b[:, :, :-1])
