"""Multi-GPU data parallelism through the C ABI (needs >= 2 GPUs; skipped otherwise): bucketed NCCL gradient all-reduce
issued by the library on its own communication stream and overlapped with the backward, identical fused step on every
rank.  Two hosts are covered: one process per GPU (b200_dp_create_rank, launched with torch.distributed.run) and one
process for all GPUs (b200_dp_group_*, what a single-process host such as the reference's C# trainer calls).  The result
must equal single-GPU training of the same global batch; a rank whose pass fails must drop the step on every rank."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

from conftest import assert_close  # noqa: F401  (puts the repository root on sys.path)

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_data_parallel_equals_single_gpu():
    import torch

    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    world = 2 if n < 4 else 4
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29700 + os.getpid() % 200), str(ROOT / "tests" / "dp_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]


def _gpus():
    import torch

    return torch.cuda.device_count()


def test_single_process_group_equals_single_gpu(oracle):
    """b200_dp_group_*: two devices behind one handle against one GPU training the same batches: two SGD steps compared
    update by update (the only difference is the order in which the two shards' gradient sums are added), then Adam."""
    import sys

    import numpy as np

    sys.path.insert(0, str(ROOT / "tests"))
    from lmutil import init_params, token_batch

    from callaghandev.ml_b200 import (GEMM_FP32_SIMT, B200DataParallelGroup, B200LanguageModelTrainer, CudaB200AccelerationManager,
                                      make_config)

    if _gpus() < 2:
        pytest.skip("needs at least 2 GPUs")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    cfg = make_config(vocab_size=300, embedding_dim=64, num_heads=4, num_layers=2, ffn_dim=128)
    rng = np.random.default_rng(11)
    toks, off = token_batch(rng, 9, 300, 2, 50, zipf=1.1)
    mgr = CudaB200AccelerationManager(0, GEMM_FP32_SIMT)
    one = B200LanguageModelTrainer(mgr, cfg, 96)
    P = init_params(None, cfg, 4, tensors=one.tensors(), total=one.param_count)
    one.upload_params(P)
    g = B200DataParallelGroup([0, 1], cfg, 96, GEMM_FP32_SIMT)
    g.upload_params(P)
    for step in range(2):
        want = one.train_step_discrete(toks, off, 3e-3, True, 1.0, True)
        got = g.train_step_discrete(toks, off, 3e-3, True, 1.0, True)
        assert got[2] == want[2] and abs(got[0] - want[0]) <= 1e-5 * max(1, abs(want[0])) and abs(got[1] - want[1]) <= 2e-5 * want[1], (got, want)
    w0, w1, ref = g.download_params(0), g.download_params(1), one.download_params()
    assert np.array_equal(w0, w1), "both ranks must hold identical weights"
    delta = ref - P
    assert np.max(np.abs((w0 - P) - delta)) <= 1e-5 * np.max(np.abs(delta)) + 2e-7, "the update must equal the single-GPU update"
    # Adam on both sides (its first steps divide by |g|, so tiny gradients amplify the summation-order difference: 2-norm bound)
    one.set_optimizer("adam"); g.set_optimizer("adam")
    before = w0
    want = one.train_step_discrete(toks, off, 3e-3, True, 1.0, True)
    got = g.train_step_discrete(toks, off, 3e-3, True, 1.0, True)
    assert got[2] == want[2] and abs(got[0] - want[0]) <= 1e-5 * max(1, abs(want[0]))
    w0, w1, ref2 = g.download_params(0), g.download_params(1), one.download_params()
    assert np.array_equal(w0, w1)
    assert np.linalg.norm((w0 - before) - (ref2 - ref)) <= 1e-2 * np.linalg.norm(ref2 - ref)

    # a rank whose pass fails: the second sequence (rank 1's shard) is longer than a pass can hold
    long_toks = np.concatenate([toks[:off[1]], np.full(200, 7, np.int32)]).astype(np.int32)
    long_off = np.array([0, off[1], off[1] + 200], np.int32)
    before = g.download_params(0)
    with pytest.raises(IndexError, match="rank 1"):
        g.train_step_discrete(long_toks, long_off, 3e-3, True, 1.0, True)
    for r in (0, 1):
        assert np.array_equal(g.download_params(r), before), "a dropped step leaves the weights untouched on every rank"
        assert not g.download_grads(r).any(), "and zeroes the gradients (TransformerTrainer.cs:298-307)"
    # the group is still healthy
    got = g.train_step_discrete(toks, off, 3e-3, True, 1.0, True)
    want = one.train_step_discrete(toks, off, 3e-3, True, 1.0, True)
    assert got[2] == want[2] and abs(got[0] - want[0]) <= 1e-5 * max(1, abs(want[0]))
    g.close(); one.close(); mgr.Dispose()
