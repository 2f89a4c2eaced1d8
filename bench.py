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
    # BASELINE.json's five configurations.  kind: lm = decoder LM on token ids, ts = time-series regression transformer,
    # mlp = feed-forward batch trainer.  scaling: how the batch follows the GPU count.
    "c5": dict(kind="lm", vocab=32000, seq=1024, d=1024, H=16, L=12, f=4096, batch=256, lr=3e-4, opt="adam", scaling="strong",
               desc="decoder LM V32000 T1024 d1024 H16 L12 f4096, global batch 256, Adam+clip1.0, Zipf(1.1) ids"),
    "c4": dict(kind="lm", vocab=8000, seq=256, d=512, H=8, L=6, f=2048, batch=64, lr=3e-4, opt="adam", scaling="weak",
               desc="decoder LM V8000 T256 d512 H8 L6 f2048, batch 64 per GPU, Adam+clip1.0, Zipf(1.1) ids"),
    "c3": dict(kind="ts", F=5, O=1, seq=128, d=256, H=8, L=4, f=1024, batch=128, lr=1e-3, opt="sgd", scaling="weak",
               desc="time-series regression transformer F5 O1 T128 d256 H8 L4 f1024, batch 128 per GPU, SGD+clip1.0, random-walk inputs"),
    "c2": dict(kind="mlp", widths=[784, 512, 256, 10], batch=256, lr=0.1, scaling="weak",
               desc="MLP 784-512-256-10 ReLU/Sigmoid, MSE, L2 1e-4, batch 256, SGD step, inputs U[0,1), one-hot targets"),
    "c1": dict(kind="lm", vocab=200, seq=64, d=64, H=4, L=2, f=128, batch=4, lr=1e-3, opt="sgd", scaling="strong",
               desc="decoder LM V200 T<=64 d64 H4 L2 f128, batch 4, SGD+clip1.0 (the reference's CPU-runnable case)"),
}


def zipf_batch(rng, n_seq, vocab, seq_len, s=1.1):
    """[START=1, Zipf(s) ids over [4, vocab), END=2], fixed length, by inverse CDF on the seeded generator."""
    ranks = np.arange(1, vocab - 4 + 1, dtype=np.float64)
    cdf = np.cumsum(ranks ** (-s))
    cdf /= cdf[-1]
    body = 4 + np.searchsorted(cdf, rng.random((n_seq, seq_len - 2)))
    toks = np.concatenate([np.ones((n_seq, 1), np.int64), body, np.full((n_seq, 1), 2, np.int64)], axis=1).astype(np.int32)
    return toks.reshape(-1), np.arange(0, (n_seq + 1) * seq_len, seq_len, dtype=np.int32)


def c1_batch(rng, n_seq, vocab, max_len):
    """Config 1: sequences of length 2..max_len (uniform), token 1 = START, ids uniform in [4, vocab), token 2 = END."""
    toks, off = [], [0]
    for _ in range(n_seq):
        n = int(rng.integers(2, max_len + 1))
        toks += [1] + list(rng.integers(4, vocab, size=max(n - 2, 0))) + [2]
        off.append(len(toks))
    return np.asarray(toks, np.int32), np.asarray(off, np.int32)


def flops_per_token(w):
    """Algorithmic FLOPs per trained token: linear forward 2*P_mm, backward 4*P_mm, causal attention forward 2*T*d*L,
    backward 5*T*d*L, with P_mm = L(4d^2 + 2df) + d*V_out (+ d*F for a continuous input projection)."""
    out = w["vocab"] if w["kind"] == "lm" else w["O"]
    pmm = w["L"] * (4 * w["d"] ** 2 + 2 * w["d"] * w["f"]) + w["d"] * out + (w["d"] * w["F"] if w["kind"] == "ts" else 0)
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


def random_walks(rng, n_seq, seq_len, F, target_feature=3):
    """Config 3 inputs: per-feature Gaussian random walks (step sigma 0.01) min-max normalised to [0,1]; the regression
    target is the given feature (the trainer applies the one-step shift itself)."""
    x = np.cumsum(rng.normal(0, 0.01, (n_seq, seq_len, F)), axis=1)
    mn, mx = x.min(axis=1, keepdims=True), x.max(axis=1, keepdims=True)
    x = ((x - mn) / np.maximum(mx - mn, 1e-12)).astype(np.float32)
    tgt = x[:, :, target_feature:target_feature + 1].copy()
    return x.reshape(-1, F), tgt.reshape(-1, 1), np.arange(0, (n_seq + 1) * seq_len, seq_len, dtype=np.int32)


def host_threads():
    """Cores this process may run on.  torch.distributed.run exports OMP_NUM_THREADS=1 to its workers, so OpenMP's own
    default cannot be trusted there."""
    return len(os.sched_getaffinity(0))


def oracle_config(w):
    from lmutil import lm_config

    if w["kind"] == "lm":
        return lm_config(vocab=w["vocab"], d=w["d"], H=w["H"], L=w["L"], f=w["f"], act="Relu")
    return lm_config(F=w["F"], O=w["O"], d=w["d"], H=w["H"], L=w["L"], f=w["f"], act="Relu", discrete=False, loss="mse")


def cpu_reference(w, budget_s, threads=None):
    """The CPU oracle (restatement of the reference's multi-thread CPU manager loops) on a bounded sample of the same
    workload.  Returns (run, units, threads, sample): run() executes one train step on `units` trained tokens (samples
    for the MLP) and returns its seconds."""
    from lmutil import init_params
    from oracle import Oracle

    orc = Oracle()
    threads = threads or max(orc.max_threads(), host_threads())
    orc.set_threads(threads)
    rng = np.random.default_rng(1234)
    if w["kind"] == "mlp":
        widths, acts = w["widths"], ["Relu"] * (len(w["widths"]) - 1) + ["Sigmoid"]
        W = [rng.normal(0, np.sqrt(2.0 / widths[l - 1]), (widths[l], widths[l - 1])).astype(np.float32) for l in range(1, len(widths))]
        Bv = [np.zeros(widths[l], np.float32) for l in range(1, len(widths))]
        X = rng.uniform(0, 1, (w["batch"], widths[0])).astype(np.float32)
        Y = np.eye(widths[-1], dtype=np.float32)[rng.integers(0, widths[-1], w["batch"])]

        def run():
            t0 = time.perf_counter()
            orc.mlp_learn_batch(widths, acts, W, Bv, X, Y, "mse", lr=w["lr"], lam=1e-4, clip_thr=1.0)
            return time.perf_counter() - t0

        return run, w["batch"], threads, f"the full batch of {w['batch']} samples per step"
    cfg = oracle_config(w)
    P = init_params(orc, cfg, 1)
    G = np.zeros_like(P)
    T = w["seq"] - 1
    if w["kind"] == "lm":
        toks, _ = zipf_batch(rng, 1, w["vocab"], w["seq"]) if w["seq"] > 64 else c1_batch(rng, 1, w["vocab"], w["seq"])

        def step(n_tok):
            t = np.concatenate([toks[:n_tok], [2]]).astype(np.int32)
            t0 = time.perf_counter()
            orc.lm_train_step(cfg, P, G, np.array([0, len(t)], np.int32), tokens=t, lr=w["lr"], use_clip=True, clip_thr=1.0, do_step=True)
            return time.perf_counter() - t0
    else:
        x, tg, _ = random_walks(rng, 1, w["seq"], w["F"])

        def step(n_tok):
            t0 = time.perf_counter()
            orc.lm_train_step(cfg, P, G, np.array([0, n_tok + 1], np.int32), cont=x[:n_tok + 1], reg_targets=tg[:n_tok + 1], lr=w["lr"], use_clip=True, clip_thr=1.0)
            return time.perf_counter() - t0
    probe = min(16, T)
    dt = step(probe)
    n = int(max(probe, min(T, probe * budget_s / max(dt, 1e-6))))
    return (lambda: step(n)), n, threads, f"{n} trained tokens of one sequence per step (full workload: {w['batch']} sequences x {T})"


def unit_of(w):
    return "samples/s" if w["kind"] == "mlp" else "tokens/s"


def reference_arm(args, w):
    """--impl reference: the reference's own CPU implementation of the path (CPU oracle, all host threads).  Under
    torch.distributed.run rank 0 alone runs it."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    run, n, threads, sample = cpu_reference(w, 8.0)
    for _ in range(args.warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run()
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    value = n / dt
    line = {"impl": "reference", "metric": METRIC if w["kind"] != "mlp" else "train samples/sec (fwd+bwd+step)", "value": value, "unit": unit_of(w), "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": w["scaling"], "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
            "config": {"workload": w["desc"], "sample": sample},
            "cpu_baseline": {"value": value, "unit": unit_of(w), "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": unit_of(w), "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def tf32_peak_now(torch):
    """cuBLAS TF32 8192^3 in this process, the way MEASURED_PEAKS.json measured bf16: best of 10 (burst) and the mean of a
    back-to-back loop of about two seconds (sustained, under the power cap the timed steps run under)."""
    torch.backends.cuda.matmul.allow_tf32 = True
    a = torch.randn(8192, 8192, device="cuda"); b = torch.randn(8192, 8192, device="cuda")
    for _ in range(3):
        a @ b
    fl = 2 * 8192 ** 3
    best = 1e9
    for _ in range(10):
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record(); a @ b; s1.record(); torch.cuda.synchronize()
        best = min(best, s0.elapsed_time(s1))
    n = max(10, int(2000.0 / best))
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for _ in range(n):
        a @ b
    s1.record(); torch.cuda.synchronize()
    sustained = s0.elapsed_time(s1) / n
    return fl / (best / 1e3) / 1e12, fl / (sustained / 1e3) / 1e12


def gemm_bytes_per_launch(csv_text):
    """Algorithmic operand + output bytes of an average tensor-core GEMM launch, 4*(M*K + K*N + M*N), from the per-shape
    timing table of the timed region."""
    tot, n = 0.0, 0
    for line in csv_text.strip().splitlines()[1:]:
        f = line.split(",")
        if len(f) < 7 or f[0] != "1":
            continue
        M, N, K, k = int(f[1]), int(f[2]), int(f[3]), int(f[6])
        tot += 4.0 * (M * K + K * N + M * N) * k
        n += k
    return tot / n if n else None


def mlp_bench(args, w, torch):
    """Config 2: NeuralNetwork.TrainBatch on one GPU.  The batch trainer's interface takes the host batch every step (as the
    reference's does), so `value` and `e2e` are the same measurement."""
    from callaghandev.ml_b200 import GEMM_AUTO, B200MlpBatchTrainer, CudaB200AccelerationManager

    if args.gpus != 1:
        raise SystemExit("the MLP workload is single-GPU (replicas only)")
    rng = np.random.default_rng(1234)
    widths, acts = w["widths"], ["Relu"] * (len(w["widths"]) - 1) + ["Sigmoid"]
    mgr = CudaB200AccelerationManager(0, GEMM_AUTO)
    t = B200MlpBatchTrainer(mgr, widths, acts, "mse", 1.0, 1e-4, 1.0, w["batch"])
    for l in range(1, len(widths)):
        t.upload_layer(l, rng.normal(0, np.sqrt(2.0 / widths[l - 1]), (widths[l], widths[l - 1])).astype(np.float32), np.zeros(widths[l], np.float32))
    X = torch.from_numpy(rng.uniform(0, 1, (w["batch"], widths[0])).astype(np.float32)).pin_memory().numpy()
    Y = torch.from_numpy(np.eye(widths[-1], dtype=np.float32)[rng.integers(0, widths[-1], w["batch"])]).pin_memory().numpy()
    for _ in range(max(args.warmup, 3)):
        t.learn_batch(X, Y, w["lr"])
    sampler = ClockSampler(0); sampler.start()
    l0 = mgr.kernel_launches()
    steps = max(args.steps, 200)  # a step is tens of microseconds of device work: time many
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        t.learn_batch(X, Y, w["lr"])
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / steps
    launches = (mgr.kernel_launches() - l0) // steps
    clocks = sampler.stop()
    flops = sum(6.0 * widths[l] * widths[l - 1] for l in range(1, len(widths))) * w["batch"]
    run, n, threads, sample = cpu_reference(w, 0)
    cdt = min(run() for _ in range(3))
    value = w["batch"] / dt
    line = {"metric": "train samples/sec (fwd+bwd+step)", "value": value, "unit": "samples/s", "n_gpus": 1, "steps": steps, "warmup": max(args.warmup, 3),
            "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "tf32", "data": "synthetic",
            "config": {"workload": w["desc"], "l2_note": "the whole problem (2.2 MB of weights, 0.8 MB batch) lives in L2: latency-bound, not graded against a roofline"},
            "clocks": clocks, "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": int(X.nbytes + Y.nbytes), "d2h_bytes_per_step": 4, "ms_per_step": dt * 1e3},
            "gpu_launches": int(launches * steps),
            "roofline": {"bound": "latency", "achieved": flops / dt / 1e12, "unit": "TFLOP/s", "peak": None, "frac": None, "traffic": None,
                         "note": f"{launches} kernel launches and two host copies per step; 0.6 GFLOP per step"},
            "cpu_baseline": {"value": n / cdt, "unit": "samples/s", "cores": threads, "kind": "port", "sample": sample}}
    print(json.dumps(line), flush=True)
    t.close(); mgr.Dispose()


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
    ap.add_argument("--batch", type=int, default=0, help="override the batch (sequences; global for c5/c1, per GPU for c3/c4)")
    ap.add_argument("--nccl-ctas", type=int, default=-1, help="CTAs the data-parallel communicator may use (-1: the library's default of 16, 0: NCCL's own choice)")
    ap.add_argument("--gemm-csv", default="", help="write the per-shape GEMM timing table of the timed region to this file")
    args = ap.parse_args()
    w = dict(WORKLOADS[args.workload])
    if args.batch:
        w["batch"] = args.batch
    if args.impl == "reference":
        return reference_arm(args, w)

    import torch

    if w["kind"] == "mlp":
        return mlp_bench(args, w, torch)

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

    global_batch = w["batch"] * (world if w["scaling"] == "weak" else 1)
    T = w["seq"] - 1
    if w["kind"] == "lm":
        cfg = make_config(vocab_size=w["vocab"], embedding_dim=w["d"], num_heads=w["H"], num_layers=w["L"], ffn_dim=w["f"], ffn_activation="Relu")
    else:
        cfg = make_config(input_feature_dim=w["F"], output_dim=w["O"], embedding_dim=w["d"], num_heads=w["H"], num_layers=w["L"], ffn_dim=w["f"],
                          ffn_activation="Relu", discrete=False, loss="mse")
    args.seqs_per_pass = max(1, min(args.seqs_per_pass, -(-global_batch // world)))  # never more than this rank trains per step
    max_rows = args.seqs_per_pass * T
    mode = {"auto": GEMM_AUTO, "simt": GEMM_FP32_SIMT, "tcgen05": GEMM_TF32_TCGEN05}[args.gemm]
    if args.nccl_ctas >= 0:
        from callaghandev.ml_b200 import _lib as _b200lib
        _b200lib.load().b200_dp_set_nccl_max_ctas(args.nccl_ctas)
    tr = DataParallelLMTrainer(cfg, max_rows, local, None, mode)
    if w["opt"] == "adam":
        tr.lm.set_optimizer("adam", 0.9, 0.999, 1e-8)

    # seeded weights (identical on every rank) and the seeded global batch
    from lmutil import init_params

    P = init_params(None, cfg, 1, tensors=tr.lm.tensors(), total=tr.lm.param_count)  # layout from the device library itself
    tr.broadcast_params(P)
    del P
    rng = np.random.default_rng(1234)
    pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory().numpy()
    if w["kind"] == "lm":
        toks, off = zipf_batch(rng, global_batch, w["vocab"], w["seq"]) if w["seq"] > 64 else c1_batch(rng, global_batch, w["vocab"], w["seq"])
        tokens_per_step = int(off[-1]) - global_batch
        host = pin(toks)
        batch = tr.prepare_discrete(toks, off)
        step_host = lambda: tr.train_step_discrete(host, off, w["lr"], True, 1.0, True)
        h2d_row, d2h_row = 4 * 7, 8  # ids, targets, positions, row scale, three sort arrays of the scatter; per-row loss and finite flag
    else:
        x, tg, off = random_walks(rng, global_batch, w["seq"], w["F"])
        tokens_per_step = global_batch * T
        hx, ht = pin(x), pin(tg)
        batch = tr.prepare_continuous(x, off, reg_targets=tg)
        step_host = lambda: tr.train_step_continuous(hx, off, reg_targets=ht, lr=w["lr"], use_clip=True, clip_threshold=1.0, do_step=True)
        h2d_row, d2h_row = 4 * (w["F"] + w["O"] + 2), 8  # features, targets, positions, row scale
    step_resident = lambda: tr.train_step_prepared(batch, w["lr"], True, 1.0, True)

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

    for _ in range(args.warmup):
        step_resident()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    tr.mgr.profile_gemm(True)
    l0 = tr.mgr.kernel_launches()
    dev_ms, wall_ms, out = timed(step_resident, args.steps)
    launches = tr.mgr.kernel_launches() - l0
    phases = tr.timings_ms()
    prof = {e: tr.mgr.gemm_profile(e) for e in (0, 1)}
    csv_text = tr.mgr.gemm_profile_csv()
    if args.gemm_csv and rank == 0:
        Path(args.gemm_csv).write_text(csv_text)
    tr.mgr.profile_gemm(False)
    clocks = sampler.stop() if rank == 0 else None
    step_host()  # one untimed call so that the host path is warm as well
    e2e_dev_ms, e2e_wall_ms, out2 = timed(step_host, args.steps)

    if rank == 0:
        ms_per_step = max(dev_ms, 0.0) / args.steps
        value = tokens_per_step / (ms_per_step / 1e3)
        e2e_ms = e2e_wall_ms / args.steps
        rows_local = tokens_per_step // world
        n_pass = -(-(global_batch // world) // args.seqs_per_pass)
        h2d = rows_local * h2d_row + n_pass * 64
        d2h = rows_local * d2h_row + 8  # ... then the gradient norm
        peaks = measured_peaks()
        tf32_burst, tf32_sustained = tf32_peak_now(torch)
        eng = 1 if prof[1][0] > prof[0][0] and prof[1][2] > 0 else 0
        n_l, fl, ms = prof[eng]
        achieved = fl / (ms / 1e3) / 1e12 if ms > 0 else 0.0
        roofline = {"bound": "tensor", "kernel": "gemm_tcgen05_tf32" if eng else "gemm_simt_fp32", "achieved": achieved, "peak": tf32_burst,
                    "unit": "TFLOP/s", "frac": achieved / tf32_burst if tf32_burst else None,
                    "frac_of_sustained_peak": achieved / tf32_sustained if tf32_sustained else None,
                    "frac_of_half_bf16_sustained": achieved / (peaks["bf16_tflops_sustained"] / 2) if peaks else None,
                    "traffic": gemm_bytes_per_launch(csv_text) if eng else None,
                    "traffic_note": "algorithmic operand + output bytes of an average GEMM launch of the timed region, 4(MK+KN+MN); the launches are "
                                    "too large for a counter capture, which on a smaller case read 0.98-1.27x of this figure",
                    "peak_source": f"cuBLAS TF32 8192^3 measured in this run: best of 10 = {tf32_burst:.0f} (the peak used, of measured), a 2 s back-to-back "
                                   f"loop = {tf32_sustained:.0f} TFLOP/s; MEASURED_PEAKS.json has no TF32 entry, its bf16 figures are "
                                   + (f"{peaks['bf16_tflops']:.0f} burst / {peaks['bf16_tflops_sustained']:.0f} sustained" if peaks else "absent"),
                    "launches": n_l, "gemm_ms_per_step": ms / args.steps,
                    "gemm_share_of_step": (ms / args.steps) / ms_per_step if ms_per_step else None}
        cpu = None
        if args.cpu_budget > 0 and world == 1:
            run, n, threads, sample = cpu_reference(w, args.cpu_budget)
            dt = run()
            cpu = {"value": n / dt, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": f"{sample}; {dt:.1f} s of CPU work"}
        line = {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
                "higher_is_better": True, "scaling": w["scaling"], "vs_baseline": None,
                "dtype": "tf32" if eng else "fp32", "data": "synthetic",
                "config": {"workload": w["desc"], "global_batch": global_batch, "seq_len": w["seq"], "parallelism": f"dp{world}",
                           "seqs_per_pass": args.seqs_per_pass,
                           "l2_note": "inputs (activation caches of one pass) far exceed the 126 MB L2" if max_rows * w["d"] * 4 > 126e6 else
                                      "small workload: the activations of a pass fit in L2, so this is not a DRAM-bound measurement",
                           "algorithmic_tflop_per_step": flops_per_token(w) * tokens_per_step / 1e12,
                           "model_tflops": flops_per_token(w) * tokens_per_step / 1e12 / (ms_per_step / 1e3)},
                "clocks": clocks, "e2e": {"value": tokens_per_step / (e2e_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                                          "ms_per_step": e2e_ms},
                "gpu_launches": int(launches), "roofline": roofline, "cpu_baseline": cpu,
                "loss": out[0] if out else None, "grad_norm": out[1] if out else None, "phase_ms_last_step": phases}
        print(json.dumps(line), flush=True)
    barrier()
    tr.close()
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
