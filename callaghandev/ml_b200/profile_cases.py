"""Small, self-contained launches of the hot kernels, sized for a profiler capture (a few hundred MB on the device,
a handful of launches).  ``python -m callaghandev.ml_b200.profile_cases <case>`` with case one of

  attention   segmented causal attention forward + backward, 8 sequences x 1024 tokens, 16 heads of 64
  gemm        the three GEMM layouts of a linear layer (forward, dX, dW) at 8192 x 1024 x 4096
  wgrad       the weight-gradient layout alone (both operands row-contiguous along M / N, long K): 1024 x 4096 x 65536
  ffn         feed-forward block forward + input gradient (bias+activation and derivative-multiply GEMM epilogues),
              16384 rows, 1024 -> 4096 -> 1024, ReLU
  decayattention  cross-attention with a per-head decay bias, forward + backward over materialised weights:
              512 queries x 4096 keys, 8 heads of 64
  layernorm   LayerNorm forward + backward on 32768 x 1024
  crossentropy  cross-entropy loss + gradient on 4096 rows x 32000 classes
  generate    greedy decoding with the device key/value cache on the c5 model (V 32000, d 1024, 16 heads, 12 layers,
              f 4096): 16-token prompt + 240 generated tokens, prints tokens/s
"""
import sys

import numpy as np

from . import CudaB200AccelerationManager, GEMM_AUTO


def attention(m, rng):
    L, S, d, H = 1024, 8, 1024, 16
    Q, K, V, dO = (rng.normal(0, 1, (L * S, d)).astype(np.float32) for _ in range(4))
    out = None
    for _ in range(2):
        m.SegmentedAttentionForward(Q, K, V, L, S, H, True)
        out = m.SegmentedAttentionBackward(Q, K, V, dO, L, S, H, 0.125, True)
    return float(np.abs(out[0]).mean())


def gemm(m, rng):
    rows, inp, out = 8192, 1024, 4096
    x = rng.normal(0, 1, (rows, inp)).astype(np.float32)
    W = rng.normal(0, 0.02, (out, inp)).astype(np.float32)
    b = np.zeros(out, np.float32)
    dy = rng.normal(0, 1, (rows, out)).astype(np.float32)
    y = m.BatchDotProductAddBias(W, x, b)
    wg, bg, di = np.zeros_like(W), np.zeros_like(b), np.zeros_like(x)
    for _ in range(2):
        m.BackpropLinearProjection(x, dy, W, wg, bg, di)
    return float(np.abs(wg).mean()) + float(np.abs(y).mean())


def wgrad(m, rng):
    rows, inp, out = 65536, 1024, 4096
    x = rng.normal(0, 1, (rows, inp)).astype(np.float32)
    W = rng.normal(0, 0.02, (out, inp)).astype(np.float32)
    dy = rng.normal(0, 1, (rows, out)).astype(np.float32)
    wg, bg, di = np.zeros_like(W), np.zeros(out, np.float32), np.zeros_like(x)
    for _ in range(2):
        m.BackpropLinearProjection(x, dy, W, wg, bg, di)
    return float(np.abs(wg).mean())


def ffn(m, rng):
    rows, d, f = 16384, 1024, 4096
    x = rng.normal(0, 1, (rows, d)).astype(np.float32)
    dy = rng.normal(0, 1, (rows, d)).astype(np.float32)
    W = [rng.normal(0, 0.02, (f, d)).astype(np.float32), rng.normal(0, 0.02, (d, f)).astype(np.float32)]
    B = [np.zeros(f, np.float32), np.zeros(d, np.float32)]
    r = None
    for _ in range(2):
        y = m.FFNForwardBatch(x, [d, f, d], ["None", "Relu", "None"], W, B)
        r = m.FFNInputGradientBatch(x, dy, [d, f, d], ["None", "Relu", "None"], W, B)
    return float(np.abs(y).mean()) + float(np.abs(r).mean())


def decayattention(m, rng):
    import time

    qn, kn, e, h = 512, 4096, 512, 8
    q, do = (rng.normal(0, 1, (qn, e)).astype(np.float32) for _ in range(2))
    k, v = (rng.normal(0, 1, (kn, e)).astype(np.float32) for _ in range(2))
    bias = rng.normal(0, 1, (qn, kn, h)).astype(np.float32)
    r = None
    for _ in range(3):
        t0 = time.perf_counter()
        out, w, s = m.ContentAwareCrossAttentionForward(q, k, v, h, 0.125, bias)
        r = m.BackpropTimeDecayedAttention(q, k, v, do, w, bias, e, h)
        dt = time.perf_counter() - t0
    print(f"decay attention forward + backward through host arrays: {dt * 1e3:.2f} ms per call pair")
    return float(np.abs(r[0]).mean())


def layernorm(m, rng):
    rows, f = 32768, 1024
    x = rng.normal(0, 1, (rows, f)).astype(np.float32)
    g, b = np.ones(f, np.float32), np.zeros(f, np.float32)
    dOut = rng.normal(0, 1, (rows, f)).astype(np.float32)
    r = None
    for _ in range(2):
        out, mean, var, normalized = m.LayerNormForward(x, g, b)
        r = m.LayerNormBackward(dOut, normalized, g, x, mean, var)
    return float(np.abs(r[0]).mean())


def crossentropy(m, rng):
    rows, vocab = 4096, 32000
    logits = rng.normal(0, 1, (rows, vocab)).astype(np.float32)
    targets = rng.integers(0, vocab, rows).astype(np.int32)
    r = None
    for _ in range(2):
        r = m.CrossEntropyLossAndGradient(logits, targets, rows)
    return float(r[0])


def generate(m, rng):
    import time

    from . import B200LanguageModelTrainer, make_config

    cfg = make_config(vocab_size=32000, embedding_dim=1024, num_heads=16, num_layers=12, ffn_dim=4096, ffn_activation="Relu")
    t = B200LanguageModelTrainer(m, cfg, max_rows_per_pass=1024)
    n = t.param_count
    w = (rng.standard_normal(n, dtype=np.float32) * 0.02)
    t.upload_params(w)
    g = t.generator(256)
    prompt = rng.integers(4, 32000, 16).astype(np.int32)
    g.greedy(prompt, 8)  # warm-up (module load, first-launch effects)
    t0 = time.perf_counter()
    out = g.greedy(prompt, 240)
    dt = time.perf_counter() - t0
    print("decode: %d tokens in %.3f s = %.1f tokens/s (prompt included, one token per model pass)" % (len(out), dt, len(out) / dt))
    g.close(); t.close()
    return float(out[-1])


CASES = {"generate": generate, "attention": attention, "gemm": gemm, "wgrad": wgrad, "ffn": ffn, "decayattention": decayattention, "layernorm": layernorm, "crossentropy": crossentropy}


def main(argv):
    if len(argv) != 2 or argv[1] not in CASES:
        print(__doc__)
        return 2
    m = CudaB200AccelerationManager(0, GEMM_AUTO)
    print(argv[1], "ok", CASES[argv[1]](m, np.random.default_rng(0)))
    m.Dispose()
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
