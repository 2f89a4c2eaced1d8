"""Pins the CPU oracle to every known-answer test the reference's own suites hold for the hot path, to independent
numpy restatements (float64), and to finite differences.  CPU only.

Reference test files (paths inside the reference project):
  PT  = CallaghanDev.ML.TestConsoleApp/Tests/AccelerationManagerParityTests.cs
  TTT = CallaghanDev.ML.TestConsoleApp/Tests/MultiTypeTransformerTests.cs
  RPT = CallaghanDev.ML.TestConsoleApp/Tests/RotaryPositionEmbeddingTests.cs
"""
import numpy as np
import pytest

from conftest import assert_close
from lmutil import init_params, lm_config, random_walk_batch, token_batch
from oracle import pt_matrix, pt_positive_vector, pt_vector

CPU_TOL = 1e-5  # PT:34


def _golden():
    import json
    from pathlib import Path

    return json.loads((Path(__file__).parent / "golden" / "reference_known_answers.json").read_text())


def check_known_answers(backend, tol_scale=1.0):
    """The reference's own known-answer vectors (tests/golden/reference_known_answers.json) against any object with the
    interface's method names: the CPU oracle here, the device manager in the GPU suite."""
    g = _golden()
    c = g["matmul_transpose"]
    out = backend.MatrixMultiplyTranspose(np.array(c["A"], np.float32), np.array(c["B"], np.float32))
    for i, j, v in c["expected_entries"]:
        assert abs(out[i, j] - v) <= c["tolerance"] * tol_scale, (i, j, out[i, j], v)
    c = g["layernorm_unit_gamma"]
    x = np.array(c["input"], np.float32)
    out = backend.LayerNormForward(x, np.ones(x.shape[1], np.float32), np.zeros(x.shape[1], np.float32))[0]
    assert np.all(np.abs(out.mean(axis=1) - c["row_mean"]) <= c["row_mean_tolerance"])
    assert np.all(np.abs(out.var(axis=1) - c["row_variance"]) <= c["row_variance_tolerance"])
    for name in ("rope_known_values", "rope_heads_independent"):
        c = g[name]
        x = np.array(c["input"], np.float32)
        backend.ApplyRotaryPositionEmbeddingInPlace(x, c["num_heads"])
        assert np.max(np.abs(x - np.array(c["expected"]))) <= c["tolerance"] * tol_scale, name


def test_reference_known_answer_vectors(oracle):
    check_known_answers(oracle)


def test_matmul_transpose_known_values(oracle):  # TTT:664-674
    c = oracle.MatrixMultiplyTranspose([[1, 2], [3, 4]], [[5, 6], [7, 8], [9, 10]])
    assert c.shape == (2, 3)
    assert abs(c[0, 0] - 17) < 1e-6 and abs(c[0, 1] - 23) < 1e-6 and abs(c[1, 2] - 67) < 1e-6


def test_matmul_against_numpy(oracle):  # PT:1146-1150 shapes
    a, b = pt_matrix(128, 128, 99), pt_matrix(128, 64, 100)
    assert_close(a.astype(np.float64) @ b.astype(np.float64), oracle.MatrixMultiply(a, b), CPU_TOL, "MatrixMultiply")


def test_layernorm_stats(oracle):  # TTT:676-701
    x = np.array([[1, 2, 3, 4], [-1, 0, 1, 2]], np.float32)
    out = oracle.LayerNormForward(x, np.ones(4), np.zeros(4))[0]
    assert np.all(np.abs(out.mean(axis=1)) < 1e-5)
    assert np.all(np.abs(out.var(axis=1) - 1) < 1e-3)


def _ln_numpy(x, g, b, eps=1e-5):
    x = x.astype(np.float64)
    m = x.mean(1, keepdims=True)
    v = ((x - m) ** 2).mean(1, keepdims=True)
    n = (x - m) / np.sqrt(v + eps)
    return n * g + b, m[:, 0], v[:, 0], n


def _ln_bwd_numpy(dout, x, g, eps=1e-5):
    """Textbook LayerNorm backward (independent of the reference's dVar/dMean formulation)."""
    dout, x, g = dout.astype(np.float64), x.astype(np.float64), g.astype(np.float64)
    _, m, v, n = _ln_numpy(x, g, 0)
    inv = 1 / np.sqrt(v + eps)
    dn = dout * g
    dx = inv[:, None] * (dn - dn.mean(1, keepdims=True) - n * (dn * n).mean(1, keepdims=True))
    return dx, (dout * n).sum(0), dout.sum(0)


@pytest.mark.parametrize("rows,cols,seeds", [(5, 6, (27, 28, 29, 30)), (512, 512, (106, 107, 108, 109))])  # PT:327-351, PT:1161-1186
def test_layernorm_forward_backward(oracle, rows, cols, seeds):
    x, g, b, dout = pt_matrix(rows, cols, seeds[0]), pt_positive_vector(cols, seeds[1]), pt_vector(cols, seeds[2]), pt_matrix(rows, cols, seeds[3])
    out, mean, var, norm = oracle.LayerNormForward(x, g, b)
    eo, em, ev, en = _ln_numpy(x, g, b)
    assert_close(eo, out, CPU_TOL, "LN out"); assert_close(em, mean, CPU_TOL, "LN mean")
    assert_close(ev, var, CPU_TOL, "LN var"); assert_close(en, norm, 2e-5, "LN normalized")
    dx, dg, db = oracle.LayerNormBackward(dout, norm, g, x, mean, var)
    ex, eg, eb = _ln_bwd_numpy(dout, x, g)
    assert_close(ex, dx, 5e-5, "LN dInput"); assert_close(eg, dg, 5e-5, "LN dGamma"); assert_close(eb, db, 5e-5, "LN dBeta")


def test_rope_known_values(oracle):  # RPT:156-196
    x = np.array([[1, 0], [1, 0], [0, 1]], np.float32)
    oracle.ApplyRotaryPositionEmbeddingInPlace(x, 1)
    exp = np.array([[1, 0], [np.cos(1.0), np.sin(1.0)], [-np.sin(2.0), np.cos(2.0)]])
    assert_close(exp, x, 1e-6, "rope known")
    y = np.array([[1, 2, 3, 4], [1, 0, 0, 1]], np.float32)
    oracle.ApplyRotaryPositionEmbeddingInPlace(y, 2)
    assert_close([1, 2, 3, 4], y[0], 1e-7, "rope position 0 unchanged")
    assert_close([np.cos(1.0), np.sin(1.0), -np.sin(1.0), np.cos(1.0)], y[1], 1e-6, "rope heads independent")


def test_rope_roundtrip_and_head(oracle):  # PT:1087-1112
    m = pt_matrix(4, 8, 97)
    r = m.copy()
    oracle.ApplyRotaryPositionEmbeddingInPlace(r, 2)
    assert not np.allclose(r[1:], m[1:])
    oracle.ApplyRotaryPositionEmbeddingInPlace(r, 2, inverse=True)
    assert_close(m, r, 5e-4, "rope round trip")
    h = m.copy()
    oracle.ApplyRotaryPositionEmbeddingHeadInPlace(h, 2, 4)
    assert np.array_equal(h[:, :2], m[:, :2]) and np.array_equal(h[:, 6:], m[:, 6:])
    # independent numpy formula
    pos = np.arange(4)[:, None]
    pair = np.arange(2)[None, :]
    th = pos / (10000.0 ** (2 * pair / 4))
    x0, x1 = m[:, 2:6:2].astype(np.float64), m[:, 3:6:2].astype(np.float64)
    assert_close(x0 * np.cos(th) - x1 * np.sin(th), h[:, 2:6:2], CPU_TOL, "rope head even")
    assert_close(x0 * np.sin(th) + x1 * np.cos(th), h[:, 3:6:2], CPU_TOL, "rope head odd")


def _sdpa_numpy(q, k, v, heads, mask=None, causal=False):
    q, k, v = (t.astype(np.float64) for t in (q, k, v))
    Tq, d = q.shape
    Tk = k.shape[0]
    hd = d // heads
    out = np.zeros((Tq, d))
    vis = np.ones((Tq, Tk), bool) if mask is None else np.asarray(mask, bool)
    if causal:
        vis = vis & (np.arange(Tk)[None, :] <= np.arange(Tq)[:, None])
    for h in range(heads):
        s = q[:, h * hd:(h + 1) * hd] @ k[:, h * hd:(h + 1) * hd].T / np.sqrt(hd)
        s = np.where(vis, s, -np.inf)
        for i in range(Tq):
            if not vis[i].any():
                continue
            e = np.exp(s[i] - s[i].max())
            out[i, h * hd:(h + 1) * hd] = (e / e.sum()) @ v[:, h * hd:(h + 1) * hd]
    return out


def test_sdpa_cases(oracle):  # PT:386-459
    q, k, v = pt_matrix(4, 8, 118), pt_matrix(4, 8, 119), pt_matrix(4, 8, 120)
    self_mask = np.array([[1, 0, 1, 0], [1, 1, 0, 0], [0, 1, 1, 0], [1, 1, 1, 1]], bool)
    assert_close(_sdpa_numpy(q, k, v, 2), oracle.ScaledDotProductAttention(q, k, v, 2), CPU_TOL, "self/no mask")
    assert_close(_sdpa_numpy(q, k, v, 2, self_mask), oracle.ScaledDotProductAttention(q, k, v, 2, self_mask), CPU_TOL, "self/mask")
    flag = oracle.ScaledDotProductAttention(q, k, v, 2, None, True)
    tril = np.tril(np.ones((4, 4), bool))
    assert_close(oracle.ScaledDotProductAttention(q, k, v, 2, tril, False), flag, CPU_TOL, "causal flag == causal mask")
    assert_close(_sdpa_numpy(q, k, v, 2, None, True), flag, CPU_TOL, "causal flag")
    qc, kc, vc = pt_matrix(4, 8, 121), pt_matrix(5, 8, 122), pt_matrix(5, 8, 123)
    cross = np.array([[1, 0, 1, 0, 1], [1, 1, 0, 1, 0], [0, 1, 1, 0, 1], [1, 0, 0, 1, 1]], bool)
    assert_close(_sdpa_numpy(qc, kc, vc, 2, cross), oracle.ScaledDotProductAttention(qc, kc, vc, 2, cross), CPU_TOL, "cross/mask")
    masked = cross.copy()
    masked[0] = False
    out = oracle.ScaledDotProductAttention(qc, kc, vc, 2, masked)
    assert np.all(out[0] == 0), "all-masked row must be zero"
    with pytest.raises(ValueError):
        oracle.ScaledDotProductAttention(qc, kc, vc, 2, None, True)


def _mha_bwd_numpy(q, k, v, do, heads, scale, vis):
    q, k, v, do = (t.astype(np.float64) for t in (q, k, v, do))
    d = q.shape[1]
    hd = d // heads
    dq, dk, dv = np.zeros_like(q), np.zeros_like(k), np.zeros_like(v)
    for h in range(heads):
        sl = slice(h * hd, (h + 1) * hd)
        s = np.where(vis, q[:, sl] @ k[:, sl].T * scale, -np.inf)
        p = np.zeros_like(s)
        for i in range(s.shape[0]):
            if vis[i].any():
                e = np.exp(s[i] - s[i].max())
                p[i] = e / e.sum()
        dv[:, sl] = p.T @ do[:, sl]
        dp = do[:, sl] @ v[:, sl].T
        ds = p * (dp - (p * dp).sum(1, keepdims=True)) * scale
        dq[:, sl] = ds @ k[:, sl]
        dk[:, sl] = ds.T @ q[:, sl]
    return dq, dk, dv


def test_mha_backward_cases(oracle):  # PT:355-381, PT:584-607
    q, k, v, do = pt_matrix(4, 6, 31), pt_matrix(4, 6, 32), pt_matrix(4, 6, 33), pt_matrix(4, 6, 34)
    scale = 1 / np.sqrt(3.0)
    tril = np.tril(np.ones((4, 4), bool))
    exp = _mha_bwd_numpy(q, k, v, do, 2, scale, tril)
    got_flag = oracle.MultiHeadAttentionBackward(q, k, v, do, 2, scale, useDecoderMask=True)
    got_mask = oracle.MultiHeadAttentionBackward(q, k, v, do, 2, scale, mask=tril)
    for e, a, b, n in zip(exp, got_flag, got_mask, "QKV"):
        assert_close(e, a, CPU_TOL, "mha bwd flag d" + n)
        assert_close(e, b, CPU_TOL, "mha bwd mask d" + n)
    q, k, v, do = pt_matrix(3, 4, 101), pt_matrix(5, 4, 102), pt_matrix(5, 4, 103), pt_matrix(3, 4, 104)
    cross = np.array([[1, 0, 1, 0, 1], [1, 1, 0, 1, 0], [0, 1, 1, 0, 1]], bool)
    exp = _mha_bwd_numpy(q, k, v, do, 2, 1 / np.sqrt(2.0), cross)
    got = oracle.MultiHeadAttentionBackward(q, k, v, do, 2, 1 / np.sqrt(2.0), mask=cross)
    for e, a, n in zip(exp, got, "QKV"):
        assert_close(e, a, CPU_TOL, "mha bwd non-square d" + n)


def test_segmented_attention_equals_per_sequence(oracle):
    L, S, d, H = 9, 3, 16, 2
    Q, K, V, dO = (pt_matrix(L * S, d, s) for s in (1, 2, 3, 4))
    out = oracle.SegmentedAttentionForward(Q, K, V, L, S, H, True)
    dQ, dK, dV = oracle.SegmentedAttentionBackward(Q, K, V, dO, L, S, H, 1 / np.sqrt(d / H), True)
    for s in range(S):
        r = slice(s * L, (s + 1) * L)
        assert_close(oracle.ScaledDotProductAttention(Q[r], K[r], V[r], H, None, True), out[r], CPU_TOL, "seg fwd")
        e = oracle.MultiHeadAttentionBackward(Q[r], K[r], V[r], dO[r], H, 1 / np.sqrt(d / H), useDecoderMask=True)
        for x, y in zip(e, (dQ[r], dK[r], dV[r])):
            assert_close(x, y, CPU_TOL, "seg bwd")


def test_qkv_forward_backward_against_independent_restatement(oracle):  # PT:461-562, PT:2057-2149
    rows, inp, out = 6, 5, 8
    x = pt_matrix(rows, inp, 124)
    wq, wk, wv = pt_matrix(out, inp, 125), pt_matrix(out, inp, 126), pt_matrix(out, inp, 127)
    bq, bk, bv = pt_vector(out, 128), pt_vector(out, 129), pt_vector(out, 130)
    Q, K, V = oracle.ProjectQKV(x, wq, bq, wk, bk, wv, bv)
    x64 = x.astype(np.float64)
    assert_close(x64 @ wq.T + bq, Q, CPU_TOL, "Q"); assert_close(x64 @ wk.T + bk, K, CPU_TOL, "K"); assert_close(x64 @ wv.T + bv, V, CPU_TOL, "V")
    dQ, dK, dV = pt_matrix(rows, out, 131), pt_matrix(rows, out, 132), pt_matrix(rows, out, 133)
    g0 = [pt_matrix(out, inp, 134), pt_vector(out, 137), pt_matrix(out, inp, 135), pt_vector(out, 138), pt_matrix(out, inp, 136), pt_vector(out, 139)]
    g = [t.copy() for t in g0]
    dIn = oracle.BackpropQKV(x, dQ, dK, dV, wq, wk, wv, *g)  # gradient buffers start NON-zero: accumulate semantics
    assert_close(dQ.astype(np.float64) @ wq + dK.astype(np.float64) @ wk + dV.astype(np.float64) @ wv, dIn, CPU_TOL, "dInput")
    for (w0, b0), (w1, b1), dY, n in zip(zip(g0[0::2], g0[1::2]), zip(g[0::2], g[1::2]), (dQ, dK, dV), "QKV"):
        assert_close(w0 + dY.astype(np.float64).T @ x64, w1, CPU_TOL, f"W{n}Grad")
        assert_close(b0 + dY.astype(np.float64).sum(0), b1, CPU_TOL, f"bias{n}Grad")


def test_kv_forward_backward_against_independent_restatement(oracle):  # IAccelerationManager.cs:329-331, AccelerationCPU.cs:4361-4560
    rows, inp, out = 7, 5, 6
    x = pt_matrix(rows, inp, 224)
    wk, wv = pt_matrix(out, inp, 225), pt_matrix(out, inp, 226)
    bk, bv = pt_vector(out, 227), pt_vector(out, 228)
    K, V = oracle.ProjectKV(x, wk, bk, wv, bv)
    x64 = x.astype(np.float64)
    assert_close(x64 @ wk.T + bk, K, CPU_TOL, "K"); assert_close(x64 @ wv.T + bv, V, CPU_TOL, "V")
    Kq, Vq = oracle.ProjectQKV(x, wk, bk, wk, bk, wv, bv)[1:]  # the two-output form agrees with the pinned three-output one
    assert np.array_equal(K, Kq) and np.array_equal(V, Vq)
    dK, dV = pt_matrix(rows, out, 229), pt_matrix(rows, out, 230)
    g0 = [pt_matrix(out, inp, 231), pt_vector(out, 233), pt_matrix(out, inp, 232), pt_vector(out, 234)]
    g = [t.copy() for t in g0]
    dIn = oracle.BackpropKV(x, dK, dV, wk, wv, *g)  # gradient buffers start NON-zero: accumulate semantics
    assert_close(dK.astype(np.float64) @ wk + dV.astype(np.float64) @ wv, dIn, CPU_TOL, "dInput")
    for (w0, b0), (w1, b1), dY, n in zip(zip(g0[0::2], g0[1::2]), zip(g[0::2], g[1::2]), (dK, dV), "KV"):
        assert_close(w0 + dY.astype(np.float64).T @ x64, w1, CPU_TOL, f"W{n}Grad")
        assert_close(b0 + dY.astype(np.float64).sum(0), b1, CPU_TOL, f"bias{n}Grad")


def test_training_ops_against_numpy(oracle):  # PT:610-737
    x, dY, W = pt_matrix(4, 5, 34), pt_matrix(4, 3, 35), pt_matrix(3, 5, 36)
    x64, dY64 = x.astype(np.float64), dY.astype(np.float64)
    wg, bg, di = np.zeros((3, 5), np.float32), np.zeros(3, np.float32), np.zeros((4, 5), np.float32)
    oracle.BackpropLinearProjection(x, dY, W, wg, bg, di)
    assert_close(dY64.T @ x64, wg, CPU_TOL, "lin Wg"); assert_close(dY64.sum(0), bg, CPU_TOL, "lin bg"); assert_close(dY64 @ W, di, CPU_TOL, "lin dIn")
    oracle.BackpropLinearProjection(x, dY, W, wg, bg, di)  # all three accumulate (CPU:2215-2226)
    assert_close(2 * dY64 @ W, di, CPU_TOL, "lin dIn accumulates")
    dL = pt_matrix(4, 3, 37)
    wg, bg = np.zeros((3, 5), np.float32), np.zeros(3, np.float32)
    dX = oracle.BackpropOutputProjection(dL, x, W, wg, bg, 4, 3, 5)
    assert_close(dL.astype(np.float64) @ W, dX, CPU_TOL, "out dX"); assert_close(dL.astype(np.float64).T @ x64, wg, CPU_TOL, "out Wg")
    cont, dXi = pt_matrix(4, 2, 38), pt_matrix(4, 5, 39)
    wg, bg = np.zeros((5, 2), np.float32), np.zeros(5, np.float32)
    oracle.BackpropInputProjection(dXi, cont, wg, bg, 4, 5, 2)
    assert_close(dXi.astype(np.float64).T @ cont, wg, CPU_TOL, "inp Wg"); assert_close(dXi.astype(np.float64).sum(0), bg, CPU_TOL, "inp bg")
    eg = np.zeros((8, 5), np.float32)
    oracle.AccumulateTokenEmbeddingGrad(eg, x, [1, 2, 2, 5], 4, 5)  # duplicate id
    exp = np.zeros((8, 5)); exp[1] = x[0]; exp[2] = x[1].astype(np.float64) + x[2]; exp[5] = x[3]
    assert_close(exp, eg, CPU_TOL, "embedding scatter")
    logits, tg = pt_matrix(4, 5, 40), [0, 2, 4, 1]
    loss, dl = oracle.CrossEntropyLossAndGradient(logits, tg, 4)
    l64 = logits.astype(np.float64)
    p = np.exp(l64 - l64.max(1, keepdims=True)); p /= p.sum(1, keepdims=True)
    oh = np.eye(5)[tg]
    assert_close(-np.log(p[np.arange(4), tg] + 1e-10).mean(), loss, CPU_TOL, "CE loss"); assert_close((p - oh) / 4, dl, CPU_TOL, "CE grad")
    pr, tm = pt_matrix(4, 3, 41), pt_matrix(4, 3, 42)
    loss, d = oracle.MSELossAndGradient(pr, tm, 4)
    diff = pr.astype(np.float64) - tm
    assert_close((diff ** 2).mean(), loss, CPU_TOL, "MSE loss"); assert_close(2 * diff / 12, d, CPU_TOL, "MSE grad")
    assert_close((x64 ** 2).sum(), oracle.MatrixSquaredNorm(x), CPU_TOL, "sqnorm")
    m = pt_matrix(4, 5, 44); oracle.MatrixScaleInPlace(m, -0.25); assert_close(pt_matrix(4, 5, 44) * -0.25, m, CPU_TOL, "scale")
    w = pt_matrix(4, 5, 46); oracle.MatrixUpdate(w, pt_matrix(4, 5, 47), 0.02)
    assert_close(pt_matrix(4, 5, 46) - 0.02 * pt_matrix(4, 5, 47).astype(np.float64), w, CPU_TOL, "update")
    ids = np.array([3, 0, 7], np.int32); E = pt_matrix(8, 5, 1)
    assert np.array_equal(oracle.EmbedTokenIds(ids, E, 5), E[ids])
    with pytest.raises(IndexError):
        oracle.EmbedTokenIds([8], E, 5)


def test_threaded_oracle_is_bit_identical(oracle):
    rng = np.random.default_rng(5)
    cfg = lm_config(vocab=50, d=32, H=4, L=2, f=64)
    P = init_params(oracle, cfg, 1)
    toks, off = token_batch(rng, 6, 50, 3, 20)
    res = []
    for th in (1, 4):
        oracle.set_threads(th)
        p, g = P.copy(), np.zeros_like(P)
        res.append((oracle.lm_train_step(cfg, p, g, off, tokens=toks), p, g))
    oracle.set_threads(1)
    assert res[0][0] == res[1][0] and np.array_equal(res[0][1], res[1][1]) and np.array_equal(res[0][2], res[1][2])


@pytest.mark.parametrize("kind", ["discrete", "continuous"])
def test_lm_gradients_match_finite_differences(oracle64, kind):
    """The trainer-level step has no stored results in the reference's tests; pin the analytic backward of the
    restated step against central differences of its own loss in float64."""
    rng = np.random.default_rng(11)
    if kind == "discrete":
        cfg = lm_config(vocab=13, d=8, H=2, L=2, f=16, act="Tanh", align=1)
        toks, off = token_batch(rng, 3, 13, fixed_len=6)
        kw = dict(tokens=toks)
    else:
        cfg = lm_config(F=3, O=1, d=8, H=2, L=1, f=16, act="Swish", discrete=False, loss="mse", align=1)
        x, t, off = random_walk_batch(rng, 2, 7, 3, 1)
        kw = dict(cont=x, reg_targets=t)
    P = init_params(oracle64, cfg, 3, np.float64)
    G = np.zeros_like(P)
    loss, norm, valid = oracle64.lm_train_step(cfg, P, G, off, use_clip=False, do_step=False, **kw)
    assert valid == len(off) - 1 and np.isfinite(loss)

    def f(p):
        return oracle64.lm_train_step(cfg, p, np.zeros_like(p), off, use_clip=False, do_step=False, **kw)[0]

    idx = rng.choice(P.size, 60, replace=False)
    for i in idx:
        p1, p2 = P.copy(), P.copy()
        p1[i] += 1e-5; p2[i] -= 1e-5
        fd = (f(p1) - f(p2)) / 2e-5
        assert abs(fd - G[i]) <= 1e-6 + 1e-5 * abs(fd), f"param {i}: fd {fd} vs analytic {G[i]}"


def test_lm_step_semantics(oracle):
    """Mixed lengths, an invalid sequence, clipping and the SGD update (TT:217-327)."""
    rng = np.random.default_rng(2)
    cfg = lm_config(vocab=30, d=16, H=2, L=1, f=32)
    P = init_params(oracle, cfg, 4)
    toks, off = token_batch(rng, 5, 30, 2, 12)
    toks = np.concatenate([toks, [1, 99, 2], [1]]).astype(np.int32)  # id >= vocab -> dropped; length 1 -> dropped
    off = np.concatenate([off, [off[-1] + 3, off[-1] + 4]]).astype(np.int32)
    p, g = P.copy(), np.zeros_like(P)
    loss, norm, valid = oracle.lm_train_step(cfg, p, g, off, tokens=toks, lr=0.1, use_clip=True, clip_thr=0.05)
    assert valid == 5 and norm > 0.05
    assert_close(0.05, np.sqrt((g.astype(np.float64) ** 2).sum()), 1e-4, "clipped norm")
    assert_close(P - 0.1 * g.astype(np.float64), p, 1e-6, "sgd update")
    emb_rows = g[:30 * 16].reshape(30, 16)
    used = set(int(t) for s in range(5) for t in toks[off[s]:off[s + 1] - 1])
    for r in range(30):
        assert (np.abs(emb_rows[r]).sum() > 0) == (r in used)  # TTT:287-304: unused rows stay untouched


def _mlp_numpy(widths, acts, W, B, X, Y, lr, lam, thr):
    X = X.astype(np.float64)
    A, D = [X], [None]
    for l in range(1, len(widths)):
        z = A[-1] @ W[l - 1].astype(np.float64).T + B[l - 1]
        if acts[l] == "Relu":
            a, d = np.maximum(z, 0), (z > 0) * 1.0
        elif acts[l] == "Sigmoid":
            a = 1 / (1 + np.exp(-z)); d = a * (1 - a)
        elif acts[l] == "Tanh":
            a = np.tanh(z); d = 1 - a * a
        else:
            a, d = z, np.ones_like(z)
        A.append(a); D.append(d)
    deltas = {len(widths) - 1: 2 * (A[-1] - Y) * D[-1]}
    for l in range(len(widths) - 2, 0, -1):
        deltas[l] = (deltas[l + 1] @ W[l].astype(np.float64)) * D[l]
    norm = np.sqrt(sum((v ** 2).sum() for v in deltas.values()))
    s = thr / norm if norm > thr else 1.0
    nb = X.shape[0]
    Wn = [W[l - 1] - lr / nb * (s * deltas[l].T @ A[l - 1] + lam * W[l - 1]) for l in range(1, len(widths))]
    Bn = [B[l - 1] - lr / nb * s * deltas[l].sum(0) for l in range(1, len(widths))]
    return Wn, Bn, norm


def test_mlp_learn_batch_against_numpy(oracle):  # NN:499-610, GPUB:251-358; MSE cost => delta = 2(a-y)act'
    rng = np.random.default_rng(0)
    widths, acts = [12, 9, 7, 3], ["Relu", "Relu", "Tanh", "Sigmoid"]
    W = [rng.normal(0, 0.4, (widths[l], widths[l - 1])).astype(np.float32) for l in range(1, 4)]
    B = [rng.normal(0, 0.1, widths[l]).astype(np.float32) for l in range(1, 4)]
    X = rng.uniform(0, 1, (16, 12)).astype(np.float32)
    Y = np.eye(3, dtype=np.float32)[rng.integers(0, 3, 16)]
    for thr in (1.0, 1e9):
        w, b = [t.copy() for t in W], [t.copy() for t in B]
        norm = oracle.mlp_learn_batch(widths, acts, w, b, X, Y, "mse", lr=0.3, lam=1e-2, clip_thr=thr)
        Wn, Bn, en = _mlp_numpy(widths, acts, W, B, X, Y, 0.3, 1e-2, thr)
        assert_close(en, norm, CPU_TOL, "delta norm")
        for a, e in zip(w + b, Wn + Bn):
            assert_close(e, a, CPU_TOL, "mlp weights")


def test_mlp_batch_of_one_equals_per_sample_rule(oracle):
    """Cross-check inside the reference: with B=1 the batch update equals the per-sample rule
    w - lr*(delta*a_prev + lambda*w) (AccelerationCPU.cs:674) for activations whose conventions coincide."""
    rng = np.random.default_rng(3)
    widths, acts = [5, 4, 2], ["None", "Tanh", "Sigmoid"]
    W = [rng.normal(0, 0.5, (4, 5)).astype(np.float32), rng.normal(0, 0.5, (2, 4)).astype(np.float32)]
    B = [np.zeros(4, np.float32), np.zeros(2, np.float32)]
    x, y = rng.uniform(0, 1, (1, 5)).astype(np.float32), np.array([[0.0, 1.0]], np.float32)
    w, b = [t.copy() for t in W], [t.copy() for t in B]
    oracle.mlp_learn_batch(widths, acts, w, b, x, y, "mse", lr=0.1, lam=0.01, clip_thr=1e9)
    a1 = np.tanh(x.astype(np.float64) @ W[0].T); a2 = 1 / (1 + np.exp(-(a1 @ W[1].T)))
    d2 = 2 * (a2 - y) * a2 * (1 - a2); d1 = (d2 @ W[1]) * (1 - a1 * a1)
    assert_close(W[1] - 0.1 * (d2.T @ a1 + 0.01 * W[1]), w[1], CPU_TOL, "W2")
    assert_close(W[0] - 0.1 * (d1.T @ x + 0.01 * W[0]), w[0], CPU_TOL, "W1")


def test_ffn_paths(oracle, oracle64):  # NN:629-716, NN:773-987 incl. the 0.1 LeakyReLU derivative and ReLU'(0)=1
    rng = np.random.default_rng(9)
    widths = [6, 10, 6]
    for act in ("Relu", "Leakyrelu", "Sigmoid", "Tanh", "Swish", "None"):
        acts = ["None", act, "None"]
        W = [rng.normal(0, 0.5, (10, 6)), rng.normal(0, 0.5, (6, 10))]
        B = [rng.normal(0, 0.1, 10), rng.normal(0, 0.1, 6)]
        x, dO = rng.normal(0, 1, (7, 6)), rng.normal(0, 1, (7, 6))
        z = x @ W[0].T + B[0]
        sig = 1 / (1 + np.exp(-z))
        a, d = {"Relu": (np.maximum(z, 0), (z >= 0) * 1.0), "Leakyrelu": (np.where(z > 0, z, 0.01 * z), np.where(z <= 0, 0.1, 1.0)),
                "Sigmoid": (sig, sig * (1 - sig)), "Tanh": (np.tanh(z), 1 - np.tanh(z) ** 2),
                "Swish": (z * sig, sig + z * sig * (1 - sig)), "None": (z, np.ones_like(z))}[act]
        assert_close(a @ W[1].T + B[1], oracle64.FFNForwardBatch(x, widths, acts, W, B), 1e-12, "ffn fwd " + act)
        wg = [np.ones((10, 6)), np.ones((6, 10))]; bg = [np.ones(10), np.ones(6)]
        dIn = oracle64.FFNInputGradientBatch(x, dO, widths, acts, W, B, wg, bg)
        d1 = (dO @ W[1]) * d
        assert_close(d1 @ W[0], dIn, 1e-12, "ffn dIn " + act)
        assert_close(1 + dO.T @ a, wg[1], 1e-12, "ffn W2g"); assert_close(1 + d1.T @ x, wg[0], 1e-12, "ffn W1g")
        assert_close(1 + dO.sum(0), bg[1], 1e-12, "ffn b2g"); assert_close(1 + d1.sum(0), bg[0], 1e-12, "ffn b1g")


def test_validate_agrees_with_the_train_step_loss_on_equal_lengths(oracle):
    """TransformerTrainer.Validate (TransformerTrainer.cs:1142-1184) weights every sequence's mean loss by its rows; for
    sequences of one length that is the bucket loss the train step reports (TransformerTrainer.cs:294, :326)."""
    import sys, os
    sys.path.insert(0, os.path.dirname(__file__))
    from lmutil import init_params, lm_config, token_batch

    rng = np.random.default_rng(0)
    cfg = lm_config(vocab=50, d=32, H=2, L=1, f=64)
    toks, off = token_batch(rng, 3, 50, 9, 9)
    P = init_params(oracle, cfg, 1)
    loss, _, valid = oracle.lm_train_step(cfg, P.copy(), np.zeros_like(P), off, tokens=toks, do_step=False)
    vloss, items = oracle.lm_validate(cfg, P, off, tokens=toks)
    assert valid == 3 and items == 3 * 8
    assert abs(loss - vloss) <= 1e-5 * max(1.0, abs(loss))


def test_incremental_decoding_agrees_with_the_batched_forward(oracle):
    """LanguageModel.cs:293-537 pushes tokens one at a time through a key/value cache with the rotary angle of the
    absolute position; the training forward (TransformerTrainer.cs:540-590) does the same sequence in one causal pass.
    Their next-token distributions must agree: the cross-entropy of the incremental logits equals the step's loss."""
    import sys, os
    sys.path.insert(0, os.path.dirname(__file__))
    from lmutil import init_params, lm_config, token_batch

    rng = np.random.default_rng(0)
    cfg = lm_config(vocab=50, d=32, H=2, L=2, f=64)
    toks, off = token_batch(rng, 1, 50, 12, 12)
    P = init_params(oracle, cfg, 1)
    lg = oracle.lm_decode_logits(cfg, P, toks[:-1]).astype(np.float64)
    tg = toks[1:]
    m = lg.max(1, keepdims=True)
    ce = -(lg - m - np.log(np.exp(lg - m).sum(1, keepdims=True)))[np.arange(len(tg)), tg]
    loss, _, valid = oracle.lm_train_step(cfg, P.copy(), np.zeros_like(P), off, tokens=toks, do_step=False)
    assert valid == 1
    assert abs(ce.mean() - loss) <= 1e-5 * max(1.0, abs(loss))
