"""Train-step parity on the GPU through the resident C-ABI entry points: gradients (tensor by tensor) and weight
updates of the language-model step and of the MLP batch step against the CPU oracle on identical seeded weights and
inputs.  FP32 SIMT path: RELATIVE error <= 1e-5, measured per tensor (max|diff| <= tol*max|ref| and the same in the
2-norm) on the gradient and on the weight update (after - before); scalars (loss, norm) and O(1) operator outputs keep
the reference's metric |exp-act| <= tol*max(1,|exp|).  Every whole-step comparison is followed by a negative control:
the same comparison against a zero gradient / un-stepped weights must fail.
"""
import numpy as np
import pytest

from conftest import assert_close, assert_tensor_close, ulp32
from lmutil import compare_gradients, compare_updates, expect_failure, unclip, init_params, lm_config, random_walk_batch, token_batch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mgr():
    from callaghandev.ml_b200 import GEMM_FP32_SIMT, CudaB200AccelerationManager

    m = CudaB200AccelerationManager(0, GEMM_FP32_SIMT)
    yield m
    m.Dispose()


def _b200_cfg(cfg):
    from callaghandev.ml_b200 import LMConfig

    c = LMConfig()
    for name, _ in LMConfig._fields_:
        setattr(c, name, getattr(cfg, name))
    return c


FP32_TOL = 1e-5


def _grads(oracle, cfg, exp, act, tol=FP32_TOL, what="grad", norms=None, thr=None):
    """norms = (oracle's, device's) pre-clip gradient norm and thr the clip threshold of a clipped step (see unclip)."""
    T = oracle.lm_tensors(cfg)
    es, as_ = (unclip(norms[0], thr), unclip(norms[1], thr)) if norms else (1.0, 1.0)
    compare_gradients(T, cfg, exp, act, tol, what, es, as_)
    expect_failure(compare_gradients, T, cfg, exp, np.zeros_like(act), tol, what, es, as_)  # a zero gradient must not pass


def _updates(oracle, cfg, exp_before, exp_after, act_before, act_after, tol=FP32_TOL, what="update", norms=None, thr=None):
    T = oracle.lm_tensors(cfg)
    es, as_ = (unclip(norms[0], thr), unclip(norms[1], thr)) if norms else (1.0, 1.0)
    compare_updates(T, cfg, exp_before, exp_after, act_before, act_after, tol, what, es, as_)
    expect_failure(compare_updates, T, cfg, exp_before, exp_after, act_before, act_before, tol, what, es, as_)  # un-stepped weights must not pass


def test_layout_matches_oracle(mgr, oracle):
    from callaghandev.ml_b200 import B200LanguageModelTrainer

    for cfg in (lm_config(vocab=200, d=64, H=4, L=2, f=128), lm_config(F=5, O=1, d=32, H=4, L=3, f=64, discrete=False, loss="mse"),
                lm_config(vocab=13, d=8, H=2, L=1, f=16, align=1)):
        t = B200LanguageModelTrainer(mgr, _b200_cfg(cfg), 64)
        assert t.param_count == oracle.lm_param_count(cfg)
        assert t.tensors() == oracle.lm_tensors(cfg)
        t.close()


@pytest.mark.parametrize("max_rows", [4096, 70])  # one packed pass, and several passes with gradient accumulation
def test_config1_discrete_step(mgr, oracle, max_rows):
    """BASELINE config 1: vocab 200, d 64, 4 heads, 2 layers, ffn 128, batch of 4 sequences of length 2..64,
    lr 1e-3, clipping at 1.0: one training step compared gradient by gradient and weight by weight."""
    from callaghandev.ml_b200 import B200LanguageModelTrainer

    rng = np.random.default_rng(1234)
    cfg = lm_config(vocab=200, d=64, H=4, L=2, f=128, act="Relu")
    toks, off = token_batch(rng, 32, 200, 2, 64)
    toks4, off4 = toks[:off[4]], off[:5]
    P = init_params(oracle, cfg, 7)
    t = B200LanguageModelTrainer(mgr, _b200_cfg(cfg), max_rows)
    # gradients only (no clipping, no update)
    pe, ge = P.copy(), np.zeros_like(P)
    el, en, ev = oracle.lm_train_step(cfg, pe, ge, off4, tokens=toks4, use_clip=False, do_step=False)
    t.upload_params(P)
    al, an, av = t.train_step_discrete(toks4, off4, 1e-3, use_clip=False, do_step=False)
    assert av == ev == 4
    assert_close(el, al, 1e-5, "loss"); assert_close(en, an, 2e-5, "grad norm")
    _grads(oracle, cfg, ge, t.download_grads())
    assert np.array_equal(t.download_params(), P), "do_step=0 must leave the weights untouched"
    # the full step
    pe, ge = P.copy(), np.zeros_like(P)
    el, en, ev = oracle.lm_train_step(cfg, pe, ge, off4, tokens=toks4, lr=1e-3, use_clip=True, clip_thr=1.0, do_step=True)
    al, an, av = t.train_step_discrete(toks4, off4, 1e-3, use_clip=True, clip_threshold=1.0, do_step=True)
    assert_close(el, al, 1e-5, "loss (step)"); assert_close(en, an, 2e-5, "grad norm (step)")
    _grads(oracle, cfg, ge, t.download_grads(), what="scaled and clipped grad", norms=(en, an), thr=1.0)
    a1 = t.download_params()
    _updates(oracle, cfg, P, pe, P, a1, norms=(en, an), thr=1.0)
    # all 32 sequences as one batch, second step on the updated weights (each side from its own step-1 weights)
    p1 = pe.copy()
    el, en, ev = oracle.lm_train_step(cfg, pe, ge, off, tokens=toks, lr=1e-3, use_clip=True, clip_thr=1.0, do_step=True)
    al, an, av = t.train_step_discrete(toks, off, 1e-3, use_clip=True, clip_threshold=1.0, do_step=True)
    assert av == ev == 32
    assert_close(el, al, 2e-5, "loss (32 sequences)")
    assert_close(en, an, 3e-5, "grad norm (32 sequences)")
    _grads(oracle, cfg, ge, t.download_grads(), what="grad (32 sequences)", norms=(en, an), thr=1.0)
    _updates(oracle, cfg, p1, pe, a1, t.download_params(), what="update (32 sequences)", norms=(en, an), thr=1.0)
    t.close()


def test_step_semantics_and_edge_batches(mgr, oracle):
    from callaghandev.ml_b200 import B200LanguageModelTrainer

    rng = np.random.default_rng(2)
    cfg = lm_config(vocab=30, d=16, H=2, L=1, f=32, act="Tanh")
    P = init_params(oracle, cfg, 4)
    toks, off = token_batch(rng, 5, 30, 2, 12)
    toks = np.concatenate([toks, [1, 99, 2], [1]]).astype(np.int32)  # out-of-vocabulary id and a length-1 sequence are skipped
    off = np.concatenate([off, [off[-1] + 3, off[-1] + 4]]).astype(np.int32)
    t = B200LanguageModelTrainer(mgr, _b200_cfg(cfg), 256)
    t.upload_params(P)
    pe, ge = P.copy(), np.zeros_like(P)
    el, en, ev = oracle.lm_train_step(cfg, pe, ge, off, tokens=toks, lr=0.1, use_clip=True, clip_thr=0.05)
    al, an, av = t.train_step_discrete(toks, off, 0.1, True, 0.05, True)
    assert av == ev == 5 and an > 0.05
    assert_close(el, al, 1e-5, "loss"); assert_close(en, an, 2e-5, "norm")
    g = t.download_grads()
    assert_close(0.05, np.sqrt((g.astype(np.float64) ** 2).sum()), 1e-4, "gradients are left scaled and clipped")
    _grads(oracle, cfg, ge, g, norms=(en, an), thr=0.05)
    _updates(oracle, cfg, P, pe, P, t.download_params(), norms=(en, an), thr=0.05)
    emb = g[:30 * 16].reshape(30, 16)
    used = set(int(x) for s in range(5) for x in toks[off[s]:off[s + 1] - 1])
    for r in range(30):
        assert (np.abs(emb[r]).sum() > 0) == (r in used), "only embedding rows of seen tokens receive gradient"
    # nothing valid: loss 0, weights untouched (TransformerTrainer.cs:309-310)
    before = t.download_params()
    assert t.train_step_discrete(np.array([1], np.int32), np.array([0, 1], np.int32), 0.1) == (0.0, 0.0, 0)
    assert t.train_step_discrete(np.zeros(0, np.int32), np.array([0], np.int32), 0.1) == (0.0, 0.0, 0)
    assert np.array_equal(before, t.download_params())
    # non-finite weights: the step is skipped and gradients are zeroed (TransformerTrainer.cs:271-272, :316-320)
    bad = before.copy(); bad[oracle.lm_tensors(cfg)[-1][0]] = np.inf  # first output bias
    t.upload_params(bad)
    l, n, v = t.train_step_discrete(toks, off, 0.1)
    assert v == 0 and l == 0.0
    assert np.array_equal(t.download_params(), bad)
    assert not t.download_grads().any()
    t.upload_params(before)
    with pytest.raises(IndexError):  # ClipGradients rejects a non-positive threshold (TransformerTrainer.cs:1313-1314)
        t.train_step_discrete(toks, off, 0.1, True, -1.0)
    t.close()


@pytest.mark.parametrize("act", ["Relu", "Leakyrelu", "Swish"])
def test_config3_continuous_regression_step(mgr, oracle, oracle64, act):
    """BASELINE config 3 shape family (features 5 -> d -> 1, MSE, one-step target shift) at a size the oracle finishes
    in seconds: d 64, 4 heads, 2 layers, ffn 256, 6 sequences of 40 steps."""
    from callaghandev.ml_b200 import B200LanguageModelTrainer

    rng = np.random.default_rng(5)
    cfg = lm_config(F=5, O=1, d=64, H=4, L=2, f=256, act=act, discrete=False, loss="mse")
    x, tg, off = random_walk_batch(rng, 6, 40, 5, 3)
    P = init_params(oracle, cfg, 9)
    t = B200LanguageModelTrainer(mgr, _b200_cfg(cfg), 100)  # 3 passes
    t.upload_params(P)
    pe, ge = P.copy(), np.zeros_like(P)
    el, en, ev = oracle.lm_train_step(cfg, pe, ge, off, cont=x, reg_targets=tg, lr=0.01, use_clip=True, clip_thr=1.0)
    al, an, av = t.train_step_continuous(x, off, reg_targets=tg, lr=0.01, use_clip=True, clip_threshold=1.0)
    assert av == ev == 6
    assert_close(el, al, 1e-5, "loss")
    # The norm here is ~128 and the float32 oracle adds 1.1 M squares serially, which alone costs ~3e-5 relative
    # (float32 oracle vs the same code in float64).  The device's tree sum is held to 1e-5 of the float64 value.
    p64, g64 = P.astype(np.float64), np.zeros(P.size, np.float64)
    n64 = oracle64.lm_train_step(cfg, p64, g64, off, cont=x, reg_targets=tg, lr=0.01, use_clip=True, clip_thr=1.0)[1]
    assert_close(n64, an, 1e-5, "norm vs float64 oracle"); assert_close(en, an, 1e-4, "norm vs float32 oracle")
    _grads(oracle, cfg, ge, t.download_grads(), norms=(en, an), thr=1.0)
    _updates(oracle, cfg, P, pe, P, t.download_params(), norms=(en, an), thr=1.0)
    t.close()


def test_continuous_classification_step(mgr, oracle):
    from callaghandev.ml_b200 import B200LanguageModelTrainer

    rng = np.random.default_rng(6)
    cfg = lm_config(F=3, O=4, d=32, H=2, L=1, f=64, act="Sigmoid", discrete=False, loss="ce", causal=True)
    x, _, off = random_walk_batch(rng, 4, 17, 3, 1)
    cls = rng.integers(0, 4, x.shape[0]).astype(np.int32)
    P = init_params(oracle, cfg, 10)
    t = B200LanguageModelTrainer(mgr, _b200_cfg(cfg), 512)
    t.upload_params(P)
    pe, ge = P.copy(), np.zeros_like(P)
    el, en, ev = oracle.lm_train_step(cfg, pe, ge, off, cont=x, cls_targets=cls, lr=0.01)
    al, an, av = t.train_step_continuous(x, off, class_targets=cls, lr=0.01)
    assert av == ev == 4
    assert_close(el, al, 1e-5, "loss")
    _grads(oracle, cfg, ge, t.download_grads(), norms=(en, an), thr=1.0)
    _updates(oracle, cfg, P, pe, P, t.download_params(), norms=(en, an), thr=1.0)
    t.close()


def test_padded_and_unpadded_arena_agree(mgr, oracle):
    """align_floats=1 (no padding, the three-GEMM Q/K/V path) and align_floats=64 (fused [3d,d] projection)."""
    from callaghandev.ml_b200 import B200LanguageModelTrainer

    rng = np.random.default_rng(8)
    toks, off = token_batch(rng, 3, 13, fixed_len=6)
    for align in (1, 64):
        cfg = lm_config(vocab=13, d=8, H=2, L=2, f=16, act="Tanh", align=align)
        P = init_params(oracle, cfg, 3)
        t = B200LanguageModelTrainer(mgr, _b200_cfg(cfg), 64)
        t.upload_params(P)
        pe, ge = P.copy(), np.zeros_like(P)
        en = oracle.lm_train_step(cfg, pe, ge, off, tokens=toks, lr=0.05)[1]
        an = t.train_step_discrete(toks, off, 0.05)[1]
        _grads(oracle, cfg, ge, t.download_grads(), what=f"align {align} grad", norms=(en, an), thr=1.0)
        _updates(oracle, cfg, P, pe, P, t.download_params(), what=f"align {align} update", norms=(en, an), thr=1.0)
        t.close()


def test_adam_extension_against_numpy(mgr, oracle):
    """Adam is an extension (the reference only has SGD).  Two separate checks per step, so that neither hides the
    other: the scaled-and-clipped gradient the step leaves behind against the oracle's (FP32 tolerance), and the
    weight update against a float64 numpy Adam applied to that very gradient from the device's own previous weights
    (the update is a smooth function of the gradient, so this isolates the optimiser arithmetic)."""
    from callaghandev.ml_b200 import B200LanguageModelTrainer

    rng = np.random.default_rng(3)
    cfg = lm_config(vocab=40, d=32, H=4, L=1, f=64)
    toks, off = token_batch(rng, 4, 40, 4, 20)
    P = init_params(oracle, cfg, 11)
    T = oracle.lm_tensors(cfg)
    t = B200LanguageModelTrainer(mgr, _b200_cfg(cfg), 256)
    t.set_optimizer("adam", 0.9, 0.999, 1e-8)
    t.upload_params(P)
    before = P.copy()
    m = np.zeros(P.size); v = np.zeros(P.size)
    for step in (1, 2, 3):
        ge = np.zeros_like(P)
        en = oracle.lm_train_step(cfg, before.copy(), ge, off, tokens=toks, use_clip=True, clip_thr=1.0, do_step=False)[1]
        an = t.train_step_discrete(toks, off, 3e-4, True, 1.0, True)[1]
        g = t.download_grads()
        _grads(oracle, cfg, ge, g, what=f"step {step} grad", norms=(en, an), thr=1.0)
        g = g.astype(np.float64)
        m = 0.9 * m + 0.1 * g; v = 0.999 * v + 0.001 * g * g
        want = before.astype(np.float64) - 3e-4 * (m / (1 - 0.9 ** step)) / (np.sqrt(v / (1 - 0.999 ** step)) + 1e-8)
        after = t.download_params()
        compare_updates(T, cfg, before, want, before, after, FP32_TOL, f"Adam step {step}")
        expect_failure(compare_updates, T, cfg, before, want, before, before, FP32_TOL)
        before = after
    t.close()


def test_step_when_the_last_pass_trains_nothing(mgr, oracle):
    """The parameter step reads the gradient once when every range of the arena was summed as it became final during
    the last pass's backward.  Here the last pass holds one sequence whose loss is not finite (its token's embedding row
    is +inf), so that pass runs no backward, nothing is announced, and the step falls back to its two-phase form (norm,
    grid barrier, update).  Reference rule: a non-finite loss drops the sequences of that length (TransformerTrainer.cs:271-272)."""
    from callaghandev.ml_b200 import B200LanguageModelTrainer

    rng = np.random.default_rng(21)
    cfg = lm_config(vocab=60, d=32, H=4, L=2, f=64, act="Tanh")
    toks, off = token_batch(rng, 5, 58, fixed_len=12)       # ids 4..57
    toks = np.concatenate([toks, [1, 59, 59, 59, 59, 59, 59, 59, 59, 2]]).astype(np.int32)  # a sixth sequence, of another length, on token 59 only
    off = np.concatenate([off, [off[-1] + 10]]).astype(np.int32)
    P = init_params(oracle, cfg, 3)
    P[59 * 32:59 * 32 + 32] = np.inf
    t = B200LanguageModelTrainer(mgr, _b200_cfg(cfg), 55)   # five sequences of 11 rows fill one pass; the sixth is alone in the last
    t.upload_params(P)
    pe, ge = P.copy(), np.zeros_like(P)
    el, en, ev = oracle.lm_train_step(cfg, pe, ge, off, tokens=toks, lr=0.05, use_clip=True, clip_thr=0.5)
    al, an, av = t.train_step_discrete(toks, off, 0.05, True, 0.5, True)
    assert av == ev == 5
    assert_close(el, al, 1e-5, "loss"); assert_close(en, an, 2e-5, "norm")
    finite = np.isfinite(P)
    ga, pa = t.download_grads(), t.download_params()
    assert np.array_equal(np.isfinite(pa), finite)
    T = oracle.lm_tensors(cfg)
    z = lambda a: np.where(finite, a, 0).astype(np.float32)
    es, as_ = (en / 0.5 if en > 0.5 else 1.0), (an / 0.5 if an > 0.5 else 1.0)
    compare_gradients(T, cfg, ge, ga, FP32_TOL, "grad", es, as_)
    compare_updates(T, cfg, z(P), z(pe), z(P), z(pa), FP32_TOL, "update", es, as_)
    expect_failure(compare_updates, T, cfg, z(P), z(pe), z(P), z(P), FP32_TOL, "update", es, as_)
    t.close()


def test_run_twice_bit_identical_step(mgr, oracle):
    from callaghandev.ml_b200 import B200LanguageModelTrainer

    rng = np.random.default_rng(12)
    cfg = lm_config(vocab=100, d=64, H=4, L=2, f=128)
    toks, off = token_batch(rng, 8, 100, 5, 50, zipf=1.1)
    P = init_params(oracle, cfg, 1)
    outs = []
    for _ in range(2):
        t = B200LanguageModelTrainer(mgr, _b200_cfg(cfg), 128)
        t.upload_params(P)
        r = t.train_step_discrete(toks, off, 1e-3)
        outs.append((r, t.download_params(), t.download_grads()))
        t.close()
    assert outs[0][0] == outs[1][0] and np.array_equal(outs[0][1], outs[1][1]) and np.array_equal(outs[0][2], outs[1][2])


# ------------------------------------------------------------------------------------------------ MLP batch trainer
def _mlp_setup(rng, widths):
    W = [rng.normal(0, np.sqrt(2.0 / widths[l - 1]), (widths[l], widths[l - 1])).astype(np.float32) for l in range(1, len(widths))]
    B = [rng.normal(0, 0.05, widths[l]).astype(np.float32) for l in range(1, len(widths))]
    return W, B


def _mlp_update_close(before, exp_after, act_after, tol, label):
    """Weight update of one MLP tensor, normalised by its own magnitude, with the un-stepped negative control."""
    b = before.astype(np.float64)
    q = ulp32(np.maximum(np.abs(exp_after), np.abs(before)))
    assert_tensor_close(exp_after - b, act_after - b, tol, label, quantum=q)
    expect_failure(assert_tensor_close, exp_after - b, np.zeros_like(b), tol, label, quantum=q)


def test_config2_mlp_batch_step(mgr, oracle):
    """BASELINE config 2: 784-512-256-10, ReLU hidden, Sigmoid output, MSE, L2 1e-4, batch 256, inputs U[0,1),
    one-hot targets: one LearnBatch compared weight by weight."""
    from callaghandev.ml_b200 import B200MlpBatchTrainer

    rng = np.random.default_rng(42)
    widths, acts = [784, 512, 256, 10], ["Relu", "Relu", "Relu", "Sigmoid"]
    W, B = _mlp_setup(rng, widths)
    X = rng.uniform(0, 1, (256, 784)).astype(np.float32)
    Y = np.eye(10, dtype=np.float32)[rng.integers(0, 10, 256)]
    for thr in (1.0, 1e9):
        we, be = [w.copy() for w in W], [b.copy() for b in B]
        en = oracle.mlp_learn_batch(widths, acts, we, be, X, Y, "mse", lr=0.1, lam=1e-4, clip_thr=thr)
        t = B200MlpBatchTrainer(mgr, widths, acts, "mse", 1.0, 1e-4, thr, 256)
        for l in range(1, 4):
            t.upload_layer(l, W[l - 1], B[l - 1])
        an = t.learn_batch(X, Y, 0.1)
        assert_close(en, an, 2e-5, "delta norm")
        # When the clip is active every delta carries the factor thr/norm, and the reference adds the squared deltas of
        # all layers and samples serially in FP32 (NeuralNetwork.cs:571-580): the two norms differ by up to 2e-5 (asserted
        # above), uniformly in every update.  That difference is added to the bound; without clipping it is plain 1e-5.
        tol = FP32_TOL + (abs(en - an) / en if en > thr else 0.0)
        for l in range(1, 4):
            w, b = t.download_layer(l)
            _mlp_update_close(W[l - 1], we[l - 1], w, tol, f"W{l} update (clip {thr})")
            _mlp_update_close(B[l - 1], be[l - 1], b, tol, f"b{l} update (clip {thr})")
        t.close()


@pytest.mark.parametrize("cost", ["mse", "ZeroWeightedMSE", "mae", "categoricalCrossEntropy", "huberLoss", "binaryCrossEntropy"])
@pytest.mark.parametrize("act", ["None", "Sigmoid", "Tanh", "Relu", "Leakyrelu"])
def test_mlp_costs_and_activations(mgr, oracle, cost, act):
    """The six cost derivatives and five activation derivatives of the batch path (conventions of
    BatchedAccelerationGPU.cs:262-287 and NeuralNetwork.cs:314-390), two steps, ragged batch, with input scaling."""
    from callaghandev.ml_b200 import B200MlpBatchTrainer

    rng = np.random.default_rng(sum(map(ord, cost + act)))
    widths, acts = [20, 33, 7], ["None", act, "Sigmoid"]
    W, B = _mlp_setup(rng, widths)
    X = rng.uniform(-2, 3, (37, 20)).astype(np.float32)
    Y = rng.uniform(0.05, 0.95, (37, 7)).astype(np.float32)  # strictly inside (0,1): BCE divides by y(1-y)
    if cost == "ZeroWeightedMSE":
        Y[:, 0] = 0
    mn, mx = X.min(0), X.max(0)
    mx[3] = mn[3]  # zero range -> scaled input 0 (NeuralNetwork.cs:131)
    Xs = oracle.mlp_scale_inputs(X, mn, mx)
    we, be = [w.copy() for w in W], [b.copy() for b in B]
    t = B200MlpBatchTrainer(mgr, widths, acts, cost, 0.3, 1e-3, 0.7, 64)
    for l in (1, 2):
        t.upload_layer(l, W[l - 1], B[l - 1])
    for _ in range(2):
        en = oracle.mlp_learn_batch(widths, acts, we, be, Xs, Y, cost, huber_delta=0.3, lr=0.2, lam=1e-3, clip_thr=0.7)
        an = t.learn_batch(X, Y, 0.2, mn, mx)
        assert_close(en, an, 2e-5, "delta norm")
    for l in (1, 2):
        w, b = t.download_layer(l)
        _mlp_update_close(W[l - 1], we[l - 1], w, 2e-5, f"W{l} update after two steps")
        _mlp_update_close(B[l - 1], be[l - 1], b, 2e-5, f"b{l} update after two steps")
    t.close()


def test_mlp_bce_with_one_hot_targets_is_nonfinite_like_the_reference(mgr, oracle):
    """binaryCrossEntropy divides by y(1-y) (NeuralNetwork.cs:348): one-hot targets give inf/NaN deltas in the reference;
    the device path reproduces that instead of hiding it."""
    from callaghandev.ml_b200 import B200MlpBatchTrainer

    rng = np.random.default_rng(1)
    widths, acts = [4, 3], ["None", "Sigmoid"]
    W, B = _mlp_setup(rng, widths)
    X, Y = rng.uniform(0, 1, (5, 4)).astype(np.float32), np.eye(3, dtype=np.float32)[rng.integers(0, 3, 5)]
    t = B200MlpBatchTrainer(mgr, widths, acts, "binaryCrossEntropy", 1.0, 0.0, 1.0, 8)
    t.upload_layer(1, W[0], B[0])
    assert not np.isfinite(t.learn_batch(X, Y, 0.1))
    we, be = [W[0].copy()], [B[0].copy()]
    assert not np.isfinite(oracle.mlp_learn_batch(widths, acts, we, be, X, Y, "binaryCrossEntropy", lr=0.1))
    t.close()


def test_prepared_batch_equals_host_path(mgr, oracle):
    """A batch copied to the device once (b200_lm_batch_*) trains bit-identically to the host-buffer entry point."""
    from callaghandev.ml_b200 import B200LanguageModelTrainer

    rng = np.random.default_rng(21)
    cfg = lm_config(vocab=120, d=64, H=4, L=2, f=128)
    toks, off = token_batch(rng, 9, 120, 2, 40, zipf=1.1)
    toks = np.concatenate([toks, [1]]).astype(np.int32); off = np.concatenate([off, [off[-1] + 1]]).astype(np.int32)  # one invalid sequence
    P = init_params(oracle, cfg, 2)
    a, b = B200LanguageModelTrainer(mgr, _b200_cfg(cfg), 96), B200LanguageModelTrainer(mgr, _b200_cfg(cfg), 96)
    a.upload_params(P); b.upload_params(P)
    h = b.prepare_discrete(toks, off)
    for _ in range(3):
        ra, rb = a.train_step_discrete(toks, off, 1e-2), b.train_step_batch(h, 1e-2)
        assert ra == rb and ra[2] == 9
    assert np.array_equal(a.download_params(), b.download_params())
    b.release_batch(h)
    a.close(); b.close()


def test_validate_discrete_and_continuous(mgr, oracle):
    """TransformerTrainer.Validate / ValidateContinuous on the device: row-weighted mean loss of the valid sequences,
    forward and loss only (weights and gradients untouched), packed into several passes."""
    from callaghandev.ml_b200 import B200LanguageModelTrainer

    rng = np.random.default_rng(21)
    cfg = lm_config(vocab=200, d=64, H=4, L=2, f=128, act="Relu")
    toks, off = token_batch(rng, 12, 200, 2, 48)
    toks = toks.copy()
    toks[off[3] + 1] = 999          # an id outside the vocabulary: the sequence is skipped (TokensAreValid)
    off = np.concatenate([off, [off[-1] + 1]]).astype(np.int32)  # and one sequence of a single token: too short
    toks = np.concatenate([toks, [5]]).astype(np.int32)
    P = init_params(oracle, cfg, 31)
    t = B200LanguageModelTrainer(mgr, _b200_cfg(cfg), 100)  # several passes
    t.upload_params(P)
    el, ei = oracle.lm_validate(cfg, P, off, tokens=toks)
    al, ai = t.validate_discrete(toks, off)
    assert ai == ei and ei > 0
    assert_close(el, al, 1e-5, "validation loss (discrete)")
    assert np.array_equal(t.download_params(), P), "validation must not touch the weights"
    t.close()

    cfg = lm_config(F=5, O=1, d=64, H=4, L=2, f=256, act="Tanh", discrete=False, loss="mse")
    x, tg, off = random_walk_batch(rng, 5, 30, 5, 3)
    P = init_params(oracle, cfg, 32)
    t = B200LanguageModelTrainer(mgr, _b200_cfg(cfg), 64)
    t.upload_params(P)
    el, ei = oracle.lm_validate(cfg, P, off, cont=x, reg_targets=tg)
    al, ai = t.validate_continuous(x, off, reg_targets=tg)
    assert ai == ei == 5 * 29
    assert_close(el, al, 1e-5, "validation loss (continuous regression)")
    t.close()


def test_checkpoint_with_optimizer_state_resumes_bit_identically(mgr, oracle, tmp_path):
    """Parameters (in the reference's own directory format: config.json, weights.bin, ffn/ffn_layer_i.json) + Adam
    moments + step index (optimizer.bin beside them) survive a save/load round trip: a run that is interrupted after
    two steps and resumed in a fresh trainer ends with exactly the weights of the uninterrupted run."""
    from callaghandev.ml_b200 import B200LanguageModelTrainer

    rng = np.random.default_rng(4)
    cfg = lm_config(vocab=40, d=32, H=4, L=1, f=64)
    toks, off = token_batch(rng, 4, 40, 4, 20)
    P = init_params(oracle, cfg, 12)
    a = B200LanguageModelTrainer(mgr, _b200_cfg(cfg), 256)
    a.set_optimizer("adam", 0.9, 0.999, 1e-8)
    a.upload_params(P)
    for _ in range(2):
        a.train_step_discrete(toks, off, 3e-4, True, 1.0, True)
    path = tmp_path / "model"
    a.save_checkpoint(path, max_sequence_length=32)
    assert sorted(p.name for p in path.iterdir()) == ["config.json", "ffn", "optimizer.bin", "weights.bin"]
    m, v, step = a.download_optimizer_state()
    assert step == 2 and np.any(m != 0) and np.all(v >= 0)
    for _ in range(2):
        a.train_step_discrete(toks, off, 3e-4, True, 1.0, True)
    want = a.download_params()
    a.close()
    b = B200LanguageModelTrainer(mgr, _b200_cfg(cfg), 256)
    b.set_optimizer("adam", 0.9, 0.999, 1e-8)
    b.load_checkpoint(path)
    for _ in range(2):
        b.train_step_discrete(toks, off, 3e-4, True, 1.0, True)
    assert np.array_equal(b.download_params(), want)
    b.close()


@pytest.mark.parametrize("single_kernel", [True, False])
def test_incremental_decoding_with_device_kv_cache(mgr, oracle, single_kernel):
    """LanguageModel.Generate's decoder path: every token goes through the model at its absolute position against the
    cached keys/values; the next-token logits after each token match the restated reference loop, and an arg-max
    continuation picks the tokens the oracle's logits pick."""
    from callaghandev.ml_b200 import B200LanguageModelTrainer

    rng = np.random.default_rng(8)
    cfg = lm_config(vocab=120, d=64, H=4, L=2, f=128, act="Relu")
    P = init_params(oracle, cfg, 41)
    t = B200LanguageModelTrainer(mgr, _b200_cfg(cfg), 64)
    t.upload_params(P)
    prompt = rng.integers(4, 120, 9).astype(np.int32)
    want = oracle.lm_decode_logits(cfg, P, prompt, max_len=32)
    g = t.generator(32)
    g.set_single_kernel(single_kernel)
    for i, tok in enumerate(prompt):
        assert_close(want[i], g.step(int(tok)), 1e-5, f"logits after token {i}")
    assert len(g) == len(prompt)
    if single_kernel:
        assert g.single_kernel(), "one cooperative kernel per token"
    else:
        assert not g.single_kernel() and g.graph_nodes() > 0, "from the second token on the launch sequence is replayed from a CUDA graph"
    # greedy continuation: device arg-max loop vs the oracle driven token by token
    seq = list(prompt)
    for _ in range(6):
        seq.append(int(np.argmax(oracle.lm_decode_logits(cfg, P, np.array(seq, np.int32), max_len=32)[-1])))
    got = g.greedy(prompt, 6)
    assert got.tolist() == seq
    # the cache is full after max_len tokens: generation stops there, a further step is an error
    got = g.greedy(prompt, 100)
    assert len(got) == 32
    g.reset()
    for tok in got:
        g.step(int(tok))
    with pytest.raises(Exception):
        g.step(5)
    with pytest.raises(Exception):
        g.step(9999)
    g.close(); t.close()


def test_handles_may_be_destroyed_in_any_order(oracle):
    """A garbage-collected host runs finalizers in no particular order: the context must stay usable until its last
    trainer / session has gone, and a trainer until its last generation session has."""
    import ctypes as C

    from callaghandev.ml_b200 import B200LanguageModelTrainer, B200MlpBatchTrainer, CudaB200AccelerationManager

    m = CudaB200AccelerationManager(0)
    lib, ctx = m.lib, m.ctx
    cfg = lm_config(vocab=50, d=32, H=2, L=1, f=64, act="Relu")
    t = B200LanguageModelTrainer(m, _b200_cfg(cfg), 32)
    t.upload_params(init_params(oracle, cfg, 3))
    g = t.generator(8)
    mlp = B200MlpBatchTrainer(m, [4, 3, 2], ["None", "Tanh", "Sigmoid"], max_batch=4)
    hg, ht, hm = g.h, t.h, mlp.h
    g.h = t.h = mlp.h = m.ctx = None  # the Python wrappers no longer own anything
    assert lib.b200_destroy(ctx) == 0        # context first ...
    assert lib.b200_lm_destroy(ht) == 0      # ... then the trainer under a live session ...
    out = np.zeros(50, np.float32)
    assert lib.b200_lm_gen_step(hg, 7, out.ctypes.data_as(C.POINTER(C.c_float))) == 0  # ... which still decodes
    assert np.isfinite(out).all()
    assert lib.b200_mlp_destroy(hm) == 0
    assert lib.b200_lm_gen_destroy(hg) == 0  # the last handle frees trainer and context


@pytest.mark.parametrize("act", ["Relu", "Leakyrelu"])
@pytest.mark.parametrize("engine", ["fp32", "tf32"])
def test_activation_derivative_at_and_below_zero(oracle, act, engine):
    """Only the activation output is cached for the backward pass.  The reference's FFN conventions make that lossy at
    one point -- ReLU'(0) is 1 (NeuralNetwork.cs:886-946) while ReLU(0) = ReLU(z<0) = 0 -- so hidden units are pinned
    to z == 0 exactly (zero weights, zero bias: gradient must flow) and to z < 0 (zero weights, negative bias: no
    gradient), at sizes the vectorised tcgen05 epilogues take, and the gradients are compared with the oracle."""
    from callaghandev.ml_b200 import GEMM_AUTO, GEMM_FP32_SIMT, B200LanguageModelTrainer, CudaB200AccelerationManager

    m = CudaB200AccelerationManager(0, GEMM_FP32_SIMT if engine == "fp32" else GEMM_AUTO)
    d, f = 128, 256
    cfg = lm_config(vocab=300, d=d, H=2, L=1, f=f, act=act)
    P = init_params(oracle, cfg, 5)
    tensors = oracle.lm_tensors(cfg)
    (w1, r1, c1), (b1, _, _) = tensors[1 + 12], tensors[1 + 13]
    W1 = P[w1:w1 + r1 * c1].reshape(r1, c1)
    assert (r1, c1) == (f, d)
    W1[:64] = 0; P[b1:b1 + 64] = 0          # z == 0 exactly
    W1[64:128] = 0; P[b1 + 64:b1 + 128] = -0.5  # z < 0
    rng = np.random.default_rng(3)
    toks, off = token_batch(rng, 4, 300, 130, 160)  # >= 128 rows per pass: the tensor-core GEMMs and their 128-bit epilogues run
    t = B200LanguageModelTrainer(m, _b200_cfg(cfg), 1024)
    t.upload_params(P)
    pe, ge = P.copy(), np.zeros_like(P)
    el, en, ev = oracle.lm_train_step(cfg, pe, ge, off, tokens=toks, use_clip=False, do_step=False)
    al, an, av = t.train_step_discrete(toks, off, 1e-3, use_clip=False, do_step=False)
    assert_close(el, al, FP32_TOL if engine == "fp32" else 2e-3, "loss")
    ga = t.download_grads()
    if engine == "fp32":
        _grads(oracle, cfg, ge, ga, FP32_TOL)
    else:
        # TF32 moves the other (unpinned) pre-activations by ~3e-4 of their spread and flips the few that sit closer to
        # zero than that, each by 100 % of its delta: a statistical bound in the 2-norm; the pinned units are checked exactly below
        for (o, r, c) in oracle.lm_tensors(cfg):
            e, a = ge[o:o + r * c].astype(np.float64), ga[o:o + r * c].astype(np.float64)
            assert np.linalg.norm(e - a) <= 0.1 * np.linalg.norm(e) + 1e-12
    gb1 = ga[b1:b1 + f]
    assert np.all(ge[b1:b1 + 64] != 0) and np.all(gb1[:64] != 0), "units at z == 0 receive gradient (ReLU'(0) = 1 / LeakyReLU'(0) = 0.1)"
    if act == "Relu":
        assert np.all(gb1[64:128] == 0), "units below zero receive none"
    t.close(); m.Dispose()
