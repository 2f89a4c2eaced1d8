"""Data-parallel decomposition on CPU with two gloo ranks: the batch is split by sequence (b200_dp_shard, which needs no
GPU), each rank produces the unscaled gradient sum, loss sum and valid count of its shard (here with the CPU oracle
standing in for the device pass), the three are all-reduced, and every rank scales by the global valid count.  The
result must equal the single-process step on the whole batch -- also when a rank's shard is empty or holds only
sequences that are too short to train.  This is the arithmetic the library's data-parallel layer (b200_dp_*) performs
around b200_lm_accumulate_* / b200_lm_apply_step; its control flow and failure rules are tested in test_dp_protocol.py."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _batch(case):
    from lmutil import token_batch

    rng = np.random.default_rng(3)
    if case == "mixed":      # includes possibly invalid (length-1) sequences
        return token_batch(rng, 7, 40, 1, 12)
    if case == "one":        # fewer sequences than ranks: rank 1's shard is empty
        return token_batch(rng, 1, 40, 5, 12)
    toks, off = token_batch(rng, 3, 40, 5, 12)  # "invalid": rank 1's only sequence has a single token (skipped by the trainer)
    return np.concatenate([toks[:off[2]], [5]]).astype(np.int32), np.array([off[0], off[1], off[2], off[2] + 1], np.int32)


def _worker(rank, world, port, out_dir, case):
    sys.path.insert(0, str(ROOT)); sys.path.insert(0, str(ROOT / "tests"))
    import torch
    import torch.distributed as dist

    from lmutil import init_params, lm_config
    from oracle import Oracle

    from callaghandev.ml_b200.trainer import split_sequences

    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    orc = Oracle()
    cfg = lm_config(vocab=40, d=16, H=2, L=1, f=32)
    toks, off = _batch(case)
    P = init_params(orc, cfg, 2)
    lo, hi = split_sequences(len(off) - 1, rank, world)
    loc_off = (off[lo:hi + 1] - off[lo]).astype(np.int32)
    loc_tok = toks[off[lo]:off[hi]]
    g = np.zeros_like(P)
    loss, _, valid = orc.lm_train_step(cfg, P.copy(), g, loc_off, tokens=loc_tok, use_clip=False, do_step=False)
    gsum = torch.from_numpy(g.astype(np.float64) * valid)       # undo the local 1/valid scaling: unscaled gradient sum
    dist.all_reduce(gsum)
    scal = torch.tensor([loss * valid, float(valid)], dtype=torch.float64)
    dist.all_reduce(scal)
    ls, vc = float(scal[0]), int(round(float(scal[1])))
    G = (gsum.numpy() / max(vc, 1)).astype(np.float32)
    np.save(os.path.join(out_dir, f"g{rank}.npy"), G)
    np.save(os.path.join(out_dir, f"s{rank}.npy"), np.array([ls / max(vc, 1), vc]))
    dist.destroy_process_group()


@pytest.mark.parametrize("case", ["mixed", "one", "invalid"])
def test_two_rank_gradient_sum_equals_single_process(tmp_path, oracle, case):
    import torch.multiprocessing as mp

    sys.path.insert(0, str(ROOT / "tests"))
    from lmutil import init_params, lm_config

    port = 29600 + (os.getpid() + ["mixed", "one", "invalid"].index(case) * 7) % 300
    mp.spawn(_worker, args=(2, port, str(tmp_path), case), nprocs=2, join=True)
    cfg = lm_config(vocab=40, d=16, H=2, L=1, f=32)
    toks, off = _batch(case)
    P = init_params(oracle, cfg, 2)
    g = np.zeros_like(P)
    loss, _, valid = oracle.lm_train_step(cfg, P.copy(), g, off, tokens=toks, use_clip=False, do_step=False)
    for r in range(2):
        G = np.load(tmp_path / f"g{r}.npy"); s = np.load(tmp_path / f"s{r}.npy")
        assert int(s[1]) == valid
        assert abs(s[0] - loss) <= 1e-6 * max(1, abs(loss))
        assert np.max(np.abs(G - g)) <= 1e-6
    assert np.array_equal(np.load(tmp_path / "g0.npy"), np.load(tmp_path / "g1.npy")), "every rank must hold identical gradients"
