"""The oracle's restatement of the sibling trainers' operators (IAccelerationManager.cs:251-361) against an independent
float64 numpy statement of the same mathematics, on the inputs of the reference's own parity tests
(AccelerationManagerParityTests.cs:856-878, 967-993) and on edge cases (-inf scores, empty inputs, clamps).
The reference holds no known-answer vectors for these operators (its tests compare back ends with each other), so
this independent statement is what pins the oracle here."""
import numpy as np
import pytest

from conftest import assert_close
from oracle import Oracle, pt_matrix, pt_tensor3, pt_vector

CPU_TOL = 1e-5


@pytest.fixture(scope="module")
def oracle():
    return Oracle()


def np_decay_attention(Q, K, V, H, scale, bias):
    Q, K, V = (x.astype(np.float64) for x in (Q, K, V))
    qn, e = Q.shape
    kn, hd = K.shape[0], e // H
    out, W, S = np.zeros((qn, e)), np.zeros((H, qn, kn)), np.zeros((H, qn, kn))
    for h in range(H):
        sl = slice(h * hd, (h + 1) * hd)
        s = Q[:, sl] @ K[:, sl].T * scale
        if bias is not None:
            s = s + bias[:, :, h].astype(np.float64)
        S[h] = s
        for q in range(qn):
            fin = ~np.isneginf(s[q])
            if not fin.any():
                continue
            w = np.where(fin, np.exp(np.where(fin, s[q], 0.0) - s[q][fin].max()), 0.0)
            W[h, q] = w / w.sum()
        out[:, sl] = W[h] @ V[:, sl]
    return out, W, S


def np_decay_attention_backward(q, k, v, dO, W, H):
    q, k, v, dO, W = (x.astype(np.float64) for x in (q, k, v, dO, W))
    e = q.shape[1]
    hd = e // H
    scale = 1.0 / np.sqrt(hd)
    dQ, dK, dV, dB = np.zeros_like(q), np.zeros_like(k), np.zeros_like(v), np.zeros((q.shape[0], k.shape[0], H))
    for h in range(H):
        sl = slice(h * hd, (h + 1) * hd)
        dW = dO[:, sl] @ v[:, sl].T
        dS = W[h] * (dW - (W[h] * dW).sum(1, keepdims=True))
        dB[:, :, h] = dS
        dQ[:, sl] = dS @ k[:, sl] * scale
        dK[:, sl] = dS.T @ q[:, sl] * scale
        dV[:, sl] = W[h].T @ dO[:, sl]
    return dQ, dK, dV, dB


def test_content_aware_cross_attention_forward(oracle):  # PT:856-878
    seq, ctx, ed, heads = 3, 4, 6, 2
    scale = 1.0 / np.sqrt(ed // heads)
    q, k, v, bias = pt_matrix(seq, ed, 80), pt_matrix(ctx, ed, 81), pt_matrix(ctx, ed, 82), pt_tensor3(seq, ctx, heads, 83)
    for b in (bias, None):
        out, W, S = oracle.ContentAwareCrossAttentionForward(q, k, v, heads, scale, b)
        eo, eW, eS = np_decay_attention(q, k, v, heads, scale, b)
        assert_close(eo, out, CPU_TOL, "output"); assert_close(eW, W, CPU_TOL, "weights"); assert_close(eS, S, CPU_TOL, "scores")
        out2, W2, S2 = oracle.ContentAwareCrossAttentionForward(q, k, v, heads, scale, b, needBackwardCache=False)
        assert W2 is None and S2 is None and np.array_equal(out, out2)
    # -inf entries of the bias remove keys; a row with no key left keeps zero weights and a zero output
    b = bias.copy()
    b[0, 1, :] = -np.inf
    b[2, :, 1] = -np.inf
    out, W, S = oracle.ContentAwareCrossAttentionForward(q, k, v, heads, scale, b)
    eo, eW, eS = np_decay_attention(q, k, v, heads, scale, b)
    assert_close(eo, out, CPU_TOL, "masked output"); assert_close(eW, W, CPU_TOL, "masked weights"); assert_close(eS, S, CPU_TOL, "masked scores")
    assert np.all(W[1, 2] == 0) and np.all(out[2, 3:] == 0) and np.all(W[:, 0, 1] == 0)


def test_backprop_time_decayed_attention(oracle):  # PT:967-993
    seq, ctx, ed, heads = 3, 4, 6, 2
    scale = 1.0 / np.sqrt(ed // heads)
    q, k, v, decay = pt_matrix(seq, ed, 91), pt_matrix(ctx, ed, 92), pt_matrix(ctx, ed, 93), pt_tensor3(seq, ctx, heads, 94)
    _, W, _ = oracle.ContentAwareCrossAttentionForward(q, k, v, heads, scale, decay)
    dO, td = pt_matrix(seq, ed, 95), pt_matrix(seq, ctx, 96)
    got = oracle.BackpropTimeDecayedAttention(q, k, v, dO, W, td, ed, heads)
    for e, a, n in zip(np_decay_attention_backward(q, k, v, dO, W, heads), got, ("dQ", "dK", "dV", "dDecayBias")):
        assert_close(e, a, CPU_TOL, n)
    assert oracle.BackpropTimeDecayedAttention(q, k, v, dO, W, None, ed, heads)[3] is None
    # finite differences of the forward's scalar <output, dO> with respect to the bias: dDecayBias is its gradient
    f = lambda b: float((np_decay_attention(q, k, v, heads, scale, b)[0] * dO).sum())
    eps, num = 1e-4, np.zeros_like(decay, dtype=np.float64)
    for idx in np.ndindex(*decay.shape):
        bp, bm = decay.astype(np.float64), decay.astype(np.float64)
        bp[idx] += eps; bm[idx] -= eps
        num[idx] = (f(bp) - f(bm)) / (2 * eps)
    assert np.max(np.abs(num - got[3])) < 1e-6


def test_small_context_operators(oracle):
    h, t, idx = pt_matrix(5, 6, 1), pt_matrix(3, 6, 2), np.array([2, 0, 1, 1, 2], np.int32)
    e = h.astype(np.float64) + t.astype(np.float64)[idx]
    oracle.ApplyContextTypeEmbedding(h, t, idx)
    assert_close(e, h, CPU_TOL, "type embedding")
    times = pt_vector(7, 3) * 10
    assert_close(np.arange(4)[:, None] - times.astype(np.float64)[None, :], oracle.ComputeTimeDiffMatrix(4, times), CPU_TOL, "time diffs")
    p, c = pt_matrix(4, 6, 4), pt_matrix(9, 6, 5)
    assert_close(c[:7].astype(np.float64) @ p[2].astype(np.float64) * 0.3, oracle.ComputeMemoryAttentionScores(p, 2, c, 7, 0.3), CPU_TOL, "memory scores")
    g, P, b = pt_vector(5, 6), pt_matrix(8, 5, 7), pt_vector(8, 8)
    assert_close(P.astype(np.float64) @ g + b, oracle.ProjectGlobalFeatures(g, P, b), CPU_TOL, "global features")
    m = pt_matrix(11, 6, 9)
    assert_close(m.astype(np.float64).mean(0), oracle.MeanPoolRows(m), CPU_TOL, "mean pool")
    assert np.all(oracle.MeanPoolRows(np.zeros((0, 4), np.float32)) == 0)
    assert_close(np.tile(m[3, :4].astype(np.float64) / 5, (5, 1)), oracle.ExpandMeanPoolGradient(m, 3, 5, 4), CPU_TOL, "expand mean pool")
    assert oracle.ExpandMeanPoolGradient(m, 3, 0, 4).shape == (0, 4)
    s = pt_vector(13, 10) * 8
    es = np.exp(s.astype(np.float64) - s.max())
    assert_close(es / es.sum(), oracle.SoftmaxVector(s), CPU_TOL, "softmax")
    x = (pt_matrix(4, 5, 11) * 200).astype(np.float32)  # +-50: both branches of the stable form, far into saturation
    ex = 1 / (1 + np.exp(-x.astype(np.float64)))
    oracle.SigmoidInPlace(x)
    assert_close(ex, x, CPU_TOL, "sigmoid")
    z = pt_matrix(4, 6, 12)
    ez = z.copy(); ez[:, :2] = 0
    oracle.ZeroMatrixColumns(z, 2)
    assert np.array_equal(ez, z)
    oracle.ZeroMatrixColumns(z, 0); assert np.array_equal(ez, z)
    oracle.ZeroMatrixColumns(z, 99); assert np.all(z == 0)
    w, gr = pt_vector(9, 13), pt_vector(9, 14)
    ew = np.clip(w.astype(np.float64) - 0.5 * gr, -0.1, 0.15)
    oracle.VectorUpdateClamped(w, gr, 0.5, -0.1, 0.15)
    assert_close(ew, w, CPU_TOL, "clamped update")
    d, gf, pg, bg = pt_vector(4, 15), pt_vector(3, 16), pt_matrix(4, 3, 17), pt_vector(4, 18)
    epg, ebg = pg.astype(np.float64) + np.outer(d, gf), bg.astype(np.float64) + d
    oracle.AccumulateGlobalProjectionGradients(d, gf, pg, bg)
    assert_close(epg, pg, CPU_TOL, "projection grad"); assert_close(ebg, bg, CPU_TOL, "bias grad")
