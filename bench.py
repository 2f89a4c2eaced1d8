#!/usr/bin/env python
"""Headline benchmark: train tokens/s (forward + backward + clipped Adam step) of the scaling decoder LM

    VocabSize 32000, sequence length 1024, EmbeddingDim 1024, 16 heads, 12 layers, FeedForwardDim 4096, FP32
    parameters, global batch 256 sequences, Adam lr 3e-4, global-norm clip 1.0, token ids Zipf(1.1), seeded

on N GPUs of one node (the batch is split by sequence: strong scaling).

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...
    python bench.py --impl reference ...     # the CPU restatement of the reference's multi-thread manager, on the host cores

One JSON line is printed by rank 0.  `value` is measured with the batch already resident in HBM; `e2e` goes through the
host-buffer entry point (token ids copied from pinned host memory and the loss read back every step).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

METRIC = "train tokens/sec (fwd+bwd+step)"
WORKLOADS = {
    # name: (vocab, seq_len, d, heads, layers, ffn, global_batch)
    "c5": dict(vocab=32000, seq=1024, d=1024, H=16, L=12, f=4096, batch=256, lr=3e-4,
               desc="decoder LM V32000 T1024 d1024 H16 L12 f4096, global batch 256, Adam+clip1.0, Zipf(1.1) ids"),
    "c4": dict(vocab=8000, seq=256, d=512, H=8, L=6, f=2048, batch=64, lr=3e-4,
               desc="decoder LM V8000 T256 d512 H8 L6 f2048, batch 64 per GPU, Adam+clip1.0, Zipf(1.1) ids"),
    "c1": dict(vocab=200, seq=64, d=64, H=4, L=2, f=128, batch=4, lr=1e-3,
               desc="decoder LM V200 T<=64 d64 H4 L2 f128, batch 4 (reference CPU-runnable case)"),
}


def zipf_batch(rng, n_seq, vocab, seq_len, s=1.1):
    """[START=1, Zipf(s) ids over [4, vocab), END=2], fixed length, by inverse CDF on the seeded generator."""
    ranks = np.arange(1, vocab - 4 + 1, dtype=np.float64)
    cdf = np.cumsum(ranks ** (-s))
    cdf /= cdf[-1]
    body = 4 + np.searchsorted(cdf, rng.random((n_seq, seq_len - 2)))
    toks = np.concatenate([np.ones((n_seq, 1), np.int64), body, np.full((n_seq, 1), 2, np.int64)], axis=1).astype(np.int32)
    return toks.reshape(-1), np.arange(0, (n_seq + 1) * seq_len, seq_len, dtype=np.int32)


def flops_per_token(w):
    """Algorithmic FLOPs per trained token: linear forward 2*P_mm, backward 4*P_mm, causal attention forward 2*T*d*L,
    backward 5*T*d*L, with P_mm = L(4d^2 + 2df) + d*V."""
    pmm = w["L"] * (4 * w["d"] ** 2 + 2 * w["d"] * w["f"]) + w["d"] * w["vocab"]
    T = w["seq"] - 1
    return 6 * pmm + 7 * T * w["d"] * w["L"]


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""

    FIELDS = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.samples, self.stop_flag, self.thread = index, [], threading.Event(), None

    def _run(self):
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([x.strip() for x in out.split(",")])
            except Exception:
                pass
            self.stop_flag.wait(0.2)

    def start(self):
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def stop(self):
        self.stop_flag.set()
        if self.thread:
            self.thread.join(timeout=6)
        sm = [float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit()]
        mx = [float(s[1]) for s in self.samples if s[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in self.samples for n, v in zip(names, s[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(sm)}


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    return json.loads(p.read_text()) if p.exists() else None


def cpu_reference_tokens_per_s(w, budget_s, threads=None):
    """Times the CPU oracle (restatement of the reference's multi-thread CPU manager loops) on a bounded sample of the
    same workload: one sequence truncated so that a full train step takes roughly budget_s seconds."""
    from lmutil import init_params, lm_config
    from oracle import Oracle

    orc = Oracle()
    # torch.distributed.run exports OMP_NUM_THREADS=1 to its workers: take the cores this process may run on, not OpenMP's default
    threads = threads or max(orc.max_threads(), len(os.sched_getaffinity(0)))
    orc.set_threads(threads)
    cfg = lm_config(vocab=w["vocab"], d=w["d"], H=w["H"], L=w["L"], f=w["f"], act="Relu")
    P = init_params(orc, cfg, 1)
    G = np.zeros_like(P)
    rng = np.random.default_rng(1234)
    toks, _ = zipf_batch(rng, 1, w["vocab"], w["seq"])

    def run(n_tok):
        t = np.concatenate([toks[:n_tok], [2]]).astype(np.int32)
        t0 = time.perf_counter()
        orc.lm_train_step(cfg, P, G, np.array([0, len(t)], np.int32), tokens=t, lr=w["lr"], use_clip=True, clip_thr=1.0, do_step=True)
        return time.perf_counter() - t0

    probe = min(16, w["seq"] - 1)
    dt = run(probe)
    n = int(max(probe, min(w["seq"] - 1, probe * budget_s / max(dt, 1e-6))))
    return orc, cfg, run, n, threads


def reference_arm(args, w):
    """--impl reference: the reference's own CPU implementation of the path (CPU oracle, all host threads)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    budget = 8.0
    orc, cfg, run, n, threads = cpu_reference_tokens_per_s(w, budget)
    for _ in range(args.warmup):
        run(n)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run(n)
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    value = n / dt
    sample = f"{n} trained tokens of one sequence per step (full workload: {w['batch']} sequences x {w['seq'] - 1})"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
            "config": {"workload": w["desc"], "sample": sample},
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c5", choices=sorted(WORKLOADS))
    ap.add_argument("--seqs-per-pass", type=int, default=128,
                    help="sequences packed into one forward/backward pass (activation cache ~0.8 GB per sequence at c5; 128 fits one B200)")
    ap.add_argument("--gemm", default="auto", choices=["auto", "simt", "tcgen05"])
    ap.add_argument("--cpu-budget", type=float, default=15.0, help="seconds of CPU work for the cpu_baseline sample (0 disables)")
    ap.add_argument("--batch", type=int, default=0, help="override the global batch (sequences)")
    ap.add_argument("--gemm-csv", default="", help="write the per-shape GEMM timing table of the timed region to this file")
    args = ap.parse_args()
    w = dict(WORKLOADS[args.workload])
    if args.batch:
        w["batch"] = args.batch
    if args.impl == "reference":
        return reference_arm(args, w)

    import torch
    import torch.distributed as dist

    from callaghandev.ml_b200 import GEMM_AUTO, GEMM_FP32_SIMT, GEMM_TF32_TCGEN05, DataParallelLMTrainer, make_config

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("gloo", rank=0, world_size=1)

    cfg = make_config(vocab_size=w["vocab"], embedding_dim=w["d"], num_heads=w["H"], num_layers=w["L"], ffn_dim=w["f"], ffn_activation="Relu")
    args.seqs_per_pass = max(1, min(args.seqs_per_pass, -(-w["batch"] // world)))  # never more than this rank trains per step
    max_rows = args.seqs_per_pass * (w["seq"] - 1)
    mode = {"auto": GEMM_AUTO, "simt": GEMM_FP32_SIMT, "tcgen05": GEMM_TF32_TCGEN05}[args.gemm]
    tr = DataParallelLMTrainer(cfg, max_rows, local, None, mode)
    tr.lm.set_optimizer("adam", 0.9, 0.999, 1e-8)

    # seeded weights (identical on every rank) and the seeded global batch
    from lmutil import init_params

    P = init_params(None, cfg, 1, tensors=tr.lm.tensors(), total=tr.lm.param_count)  # layout from the device library itself
    tr.broadcast_params(P)
    del P
    rng = np.random.default_rng(1234)
    toks, off = zipf_batch(rng, w["batch"], w["vocab"], w["seq"])
    tokens_per_step = w["batch"] * (w["seq"] - 1)
    pinned_toks = torch.from_numpy(toks).pin_memory().numpy()
    batch = tr.prepare_discrete(toks, off)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record(tr.compute)
        out = None
        for _ in range(steps):
            out = fn()
        e1.record(tr.compute)
        barrier()
        wall = time.perf_counter() - t0
        dev_ms = e0.elapsed_time(e1)
        t = torch.tensor([dev_ms, wall * 1e3], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t[0].item(), t[1].item(), out

    step_resident = lambda: tr.train_step_prepared(batch, w["lr"], True, 1.0, True)
    step_host = lambda: tr.train_step_discrete(pinned_toks, off, w["lr"], True, 1.0, True)

    for _ in range(args.warmup):
        step_resident()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    tr.mgr.profile_gemm(True)
    l0 = tr.mgr.kernel_launches()
    dev_ms, wall_ms, out = timed(step_resident, args.steps)
    launches = tr.mgr.kernel_launches() - l0
    prof = {e: tr.mgr.gemm_profile(e) for e in (0, 1)}
    if args.gemm_csv and rank == 0:
        Path(args.gemm_csv).write_text(tr.mgr.gemm_profile_csv())
    tr.mgr.profile_gemm(False)
    clocks = sampler.stop() if rank == 0 else None
    step_host()  # one untimed call so that the host path is warm as well
    e2e_dev_ms, e2e_wall_ms, out2 = timed(step_host, args.steps)

    if rank == 0:
        ms_per_step = max(dev_ms, 0.0) / args.steps
        value = tokens_per_step / (ms_per_step / 1e3)
        e2e_ms = e2e_wall_ms / args.steps
        rows_local = tokens_per_step // world
        n_pass = -(-(w["batch"] // world) // args.seqs_per_pass)
        h2d = rows_local * 4 * 7 + n_pass * 64  # ids, targets, positions, row scale, and the three sort arrays of the scatter
        d2h = rows_local * 8 + 8                # per-row loss and finite flag, then the gradient norm
        peaks = measured_peaks()
        # TF32 tensor-pipe denominator: cuBLAS TF32 8192^3, measured in this run the way MEASURED_PEAKS.json measured bf16
        torch.backends.cuda.matmul.allow_tf32 = True
        a = torch.randn(8192, 8192, device="cuda"); b = torch.randn(8192, 8192, device="cuda")
        for _ in range(3):
            a @ b
        best = 1e9
        for _ in range(10):
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record(); a @ b; s1.record(); torch.cuda.synchronize()
            best = min(best, s0.elapsed_time(s1))
        tf32_peak = 2 * 8192 ** 3 / (best / 1e3) / 1e12
        del a, b
        eng = 1 if prof[1][0] > prof[0][0] and prof[1][2] > 0 else 0
        n_l, fl, ms = prof[eng]
        achieved = fl / (ms / 1e3) / 1e12 if ms > 0 else 0.0
        # DRAM traffic per launch: ncu capture of the three GEMM layouts of one linear layer (8192 x 1024 x 4096, see
        # profiles/gemm_tcgen05_8192x4096x1024.md): 595.6 MB of dram read+write for 3 x 68.7 GFLOP, i.e. 2.89 bytes per
        # kFLOP (0.98-1.27 x the algorithmic bytes); traffic grows with the FLOPs of a launch, so it is scaled by them.
        traffic = (fl / n_l) * 2.89e-3 if (eng and n_l) else None
        roofline = {"bound": "tensor", "kernel": "gemm_tcgen05_tf32" if eng else "gemm_simt_fp32", "achieved": achieved, "peak": tf32_peak,
                    "unit": "TFLOP/s", "frac": achieved / tf32_peak if tf32_peak else None, "traffic": traffic,
                    "traffic_note": "bytes per average GEMM launch, scaled from an ncu capture of a smaller case by FLOPs",
                    "peak_source": "cuBLAS TF32 8192^3 measured in this run (of measured); bf16 peaks of MEASURED_PEAKS.json: "
                                   + (f"{peaks['bf16_tflops']:.0f} burst / {peaks['bf16_tflops_sustained']:.0f} sustained TFLOP/s" if peaks else "file absent"),
                    "launches": n_l, "gemm_ms_per_step": ms / args.steps,
                    "gemm_share_of_step": (ms / args.steps) / ms_per_step if ms_per_step else None}
        cpu = None
        if args.cpu_budget > 0 and world == 1:
            orc, ocfg2, run, n, threads = cpu_reference_tokens_per_s(w, args.cpu_budget)
            dt = run(n)
            cpu = {"value": n / dt, "unit": "tokens/s", "cores": threads, "kind": "port",
                   "sample": f"one train step on {n} tokens of one sequence ({dt:.1f} s of CPU work); full workload is {w['batch']} x {w['seq'] - 1} tokens"}
        line = {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "tf32" if eng else "fp32", "data": "synthetic",
                "config": {"workload": w["desc"], "global_batch": w["batch"], "seq_len": w["seq"], "parallelism": f"dp{world}",
                           "seqs_per_pass": args.seqs_per_pass, "l2_note": "inputs (activations ~1 GB per layer per pass) far exceed the 126 MB L2",
                           "algorithmic_tflop_per_step": flops_per_token(w) * tokens_per_step / 1e12,
                           "model_tflops": flops_per_token(w) * tokens_per_step / 1e12 / (ms_per_step / 1e3)},
                "clocks": clocks, "e2e": {"value": tokens_per_step / (e2e_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                                          "ms_per_step": e2e_ms},
                "gpu_launches": int(launches), "roofline": roofline, "cpu_baseline": cpu,
                "loss": out[0] if out else None, "grad_norm": out[1] if out else None, "phase_ms_last_step": tr.lm.timings_ms()}
        print(json.dumps(line), flush=True)
    barrier()
    tr.close()
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
