"""Worker of the multi-GPU data-parallel test: one process per GPU (launched by torch.distributed.run).  Every rank
trains the same global batches with DataParallelLMTrainer (the library's b200_dp_* entry points): a host batch, the same
batch prepared on the device, and a batch with fewer sequences than ranks (some shards are empty and still have to
issue every collective).  Rank 0 also trains them on one GPU alone and the weights must agree."""
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT)); sys.path.insert(0, str(ROOT / "tests"))


def main():
    import torch
    import torch.distributed as dist

    from lmutil import init_params, token_batch

    from callaghandev.ml_b200 import (GEMM_FP32_SIMT, B200LanguageModelTrainer, CudaB200AccelerationManager, DataParallelLMTrainer,
                                      make_config)

    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = make_config(vocab_size=300, embedding_dim=64, num_heads=4, num_layers=2, ffn_dim=128)
    rng = np.random.default_rng(11)
    toks, off = token_batch(rng, 13, 300, 2, 50, zipf=1.1)
    tr = DataParallelLMTrainer(cfg, 96, local, None, GEMM_FP32_SIMT)  # 96 rows per pass: several passes per rank
    P = init_params(None, cfg, 4, tensors=tr.lm.tensors(), total=tr.lm.param_count)
    tr.broadcast_params(P)
    res = [tr.train_step_discrete(toks, off, 1e-2, True, 1.0, True)]
    batch = tr.prepare_discrete(toks, off)
    res.append(tr.train_step_prepared(batch, 1e-2, True, 1.0, True))
    toks1, off1 = toks[:off[1]], off[:2]  # one sequence for the whole world: every rank but the first has nothing to train
    res.append(tr.train_step_discrete(toks1, off1, 1e-2, True, 1.0, True))
    exposed = tr.timings_ms()
    got = tr.lm.download_params()
    ok = True
    if rank == 0:
        mgr = CudaB200AccelerationManager(local, GEMM_FP32_SIMT)
        one = B200LanguageModelTrainer(mgr, cfg, 96)
        one.upload_params(P)
        ref = [one.train_step_discrete(toks, off, 1e-2, True, 1.0, True) for _ in range(2)] + [one.train_step_discrete(toks1, off1, 1e-2, True, 1.0, True)]
        exp = one.download_params()
        err = float(np.max(np.abs(exp - got) / np.maximum(1.0, np.abs(exp))))
        ok = err <= 1e-5 and all(abs(a[0] - b[0]) <= 1e-5 * max(1, abs(b[0])) and a[2] == b[2] for a, b in zip(res, ref))
        print(f"DP world {world}: max weight error {err:.3e}, losses {res} vs {ref}, timings {exposed}", flush=True)
        one.close(); mgr.Dispose()
    # all ranks must hold identical weights
    t = torch.from_numpy(got).cuda()
    lo, hi = t.clone(), t.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN); dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    same = bool(torch.equal(lo, hi))
    flag = torch.tensor([1 if (ok and same) else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    tr.close()  # release the device state before the process group goes away
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1 else 1)


if __name__ == "__main__":
    main()
