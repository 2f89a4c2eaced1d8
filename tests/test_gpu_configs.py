"""Whole-step parity at the dimensions of the benchmark configurations, in the mode a user gets by default (AUTO).

One train step (forward, backward, scale, clip, update) on identical seeded weights and inputs against the CPU oracle
(restating TransformerTrainer.cs:217-327 / :337-486), compared tensor by tensor with a bound relative to each tensor's
own magnitude (max|diff| <= tol*max|ref| and ||diff||_2 <= tol*||ref||_2) on the gradient and on the weight update
(after - before), each followed by a negative control (zero gradient / un-stepped weights must fail).

  c1  V 200  d 64  H 4  L 2  f 128, 4 sequences of 2..64: every dimension below 128 -> FP32 engines, tol 1e-5
  c3  F 5 -> d 256, H 8 (head dim 32), L 4, f 1024 -> O 1, MSE, 4 sequences of 128 steps: TF32 GEMMs + mma.sync attention
  c4  V 8000 d 512 H 8 (head dim 64) L 6 f 2048, 4 sequences of 256: TF32 GEMMs (two-SM kernel) + tcgen05 attention
  c5  V 32000 d 1024 H 16 L 12 f 4096, 2 sequences of 258 tokens (every GEMM dimension >= 256): the benchmarked path

The batch is smaller than the benchmark's (the oracle has to finish in seconds) but every model dimension is the
configuration's, so the same kernels run with the same tile shapes; the launch counters prove which ones did.

TF32 tolerance.  Each TF32 product carries 2^-11 relative rounding per operand; a gradient that has passed through k
matrix products accumulates about sqrt(k) of those.  The bound is stated per configuration next to the measured error.
"""
import numpy as np
import pytest

from conftest import assert_close
from lmutil import compare_gradients, compare_updates, expect_failure, init_params, lm_config, random_walk_batch, token_batch

pytestmark = pytest.mark.gpu


def _b200_cfg(cfg):
    from callaghandev.ml_b200 import LMConfig

    c = LMConfig()
    for name, _ in LMConfig._fields_:
        setattr(c, name, getattr(cfg, name))
    return c


def _step_parity(oracle, cfg, batch, lr, tol, scalar_tol, max_rows, expect_engines, forbid_engines=(), threads=None):
    """Runs one step on both sides and compares; returns the engine counters of the device run."""
    from callaghandev.ml_b200 import GEMM_AUTO, B200LanguageModelTrainer, CudaB200AccelerationManager

    oracle.set_threads(threads or oracle.max_threads())
    try:
        P = init_params(oracle, cfg, 1)
        T = oracle.lm_tensors(cfg)
        m = CudaB200AccelerationManager(0, GEMM_AUTO)
        t = B200LanguageModelTrainer(m, _b200_cfg(cfg), max_rows)
        t.upload_params(P)
        pe, ge = P.copy(), np.zeros_like(P)
        if cfg.discrete:
            toks, off = batch
            el, en, ev = oracle.lm_train_step(cfg, pe, ge, off, tokens=toks, lr=lr, use_clip=True, clip_thr=1.0)
            al, an, av = t.train_step_discrete(toks, off, lr, True, 1.0, True)
        else:
            x, tg, off = batch
            el, en, ev = oracle.lm_train_step(cfg, pe, ge, off, cont=x, reg_targets=tg, lr=lr, use_clip=True, clip_thr=1.0)
            al, an, av = t.train_step_continuous(x, off, reg_targets=tg, lr=lr, use_clip=True, clip_threshold=1.0)
        eng = m.engine_launches()
        for name in expect_engines:
            assert eng[name] > 0, f"{name} did not run: {eng}"
        for name in forbid_engines:
            assert eng[name] == 0, f"{name} ran although the configuration is below its threshold: {eng}"
        assert av == ev and ev == len(off) - 1
        assert_close(el, al, scalar_tol, "loss")
        assert_close(en, an, scalar_tol, "gradient norm")
        ga, pa = t.download_grads(), t.download_params()
        worst_g = compare_gradients(T, cfg, ge, ga, tol)
        expect_failure(compare_gradients, T, cfg, ge, np.zeros_like(ga), tol)
        worst_u = compare_updates(T, cfg, P, pe, P, pa, tol)
        expect_failure(compare_updates, T, cfg, P, pe, P, P, tol)
        print(f"worst per-tensor relative error: gradient {worst_g:.2e}, update {worst_u:.2e}; loss {al:.6f} (oracle {el:.6f}); engines {eng}")
        t.close(); m.Dispose()
        return eng
    finally:
        oracle.set_threads(1)


def test_config1_default_mode_runs_fp32_engines(oracle):
    """BASELINE config 1 in AUTO mode: every dimension is below 128, so the FP32 SIMT GEMM and the FP32 attention run
    and the step holds the FP32 tolerance."""
    rng = np.random.default_rng(1234)
    cfg = lm_config(vocab=200, d=64, H=4, L=2, f=128, act="Relu")
    toks, off = token_batch(rng, 32, 200, 2, 64)
    batch = (toks[:off[4]], off[:5])
    _step_parity(oracle, cfg, batch, 1e-3, 1e-5, 1e-5, 512, ("gemm_simt", "attn_fp32"),
                 ("gemm_tile", "gemm_persistent", "gemm_pair", "attn_mma_sync", "attn_tcgen05"))


def test_config3_stated_size(oracle):
    """BASELINE config 3 at its stated size: 5 features -> d 256, 8 heads, 4 layers, ffn 1024 -> 1 output, MSE,
    sequences of 128 steps (4 of them), random-walk inputs."""
    rng = np.random.default_rng(33)
    cfg = lm_config(F=5, O=1, d=256, H=8, L=4, f=1024, act="Relu", discrete=False, loss="mse")
    batch = random_walk_batch(rng, 4, 128, 5, 3)
    _step_parity(oracle, cfg, batch, 1e-2, TF32_STEP_TOL["c3"], 2e-3, 4 * 127, ("gemm_simt", "attn_mma_sync"), ("attn_fp32",))


def test_config4_dimensions(oracle):
    """BASELINE config 4 dimensions: V 8000, d 512, 8 heads of 64, 6 layers, ffn 2048, sequences of 256 (4 of them),
    Zipf(1.1) ids."""
    rng = np.random.default_rng(44)
    cfg = lm_config(vocab=8000, d=512, H=8, L=6, f=2048, act="Relu")
    batch = token_batch(rng, 4, 8000, fixed_len=256, zipf=1.1)
    _step_parity(oracle, cfg, batch, 3e-3, TF32_STEP_TOL["c4"], 2e-3, 4 * 255, ("gemm_pair", "attn_tcgen05"), ("attn_fp32", "gemm_simt"))


def test_config5_dimensions(oracle):
    """BASELINE config 5 dimensions, the benchmarked model: V 32000, d 1024, 16 heads of 64, 12 layers, ffn 4096,
    2 sequences of 258 tokens (514 trained rows: every GEMM dimension is at least 256, so the two-SM GEMM, the tcgen05
    attention and the large-vocabulary cross-entropy all run)."""
    rng = np.random.default_rng(55)
    cfg = lm_config(vocab=32000, d=1024, H=16, L=12, f=4096, act="Relu")
    batch = token_batch(rng, 2, 32000, fixed_len=258, zipf=1.1)
    _step_parity(oracle, cfg, batch, 3e-3, TF32_STEP_TOL["c5"], 2e-3, 2 * 257, ("gemm_pair", "attn_tcgen05"), ("attn_fp32", "gemm_simt"))


# Per-tensor relative bounds of the TF32 configurations (see the module docstring); measured worst cases beside them.
TF32_STEP_TOL = {"c3": 2e-3, "c4": 2e-3, "c5": 2e-3}
