"""Small, self-contained launches of the hot kernels, sized for a profiler capture (a few hundred MB on the device,
a handful of launches).  ``python -m callaghandev.profile_cases <case>`` with case one of

  attention   segmented causal attention forward + backward, 8 sequences x 1024 tokens, 16 heads of 64
  gemm        the three GEMM layouts of a linear layer (forward, dX, dW) at 8192 x 1024 x 4096
  wgrad       the weight-gradient layout alone (both operands row-contiguous along M / N, long K): 1024 x 4096 x 65536
  ffn         feed-forward block forward + input gradient (bias+activation and derivative-multiply GEMM epilogues),
              16384 rows, 1024 -> 4096 -> 1024, ReLU
  decayattention  cross-attention with a per-head decay bias, forward + backward over materialised weights:
              512 queries x 4096 keys, 8 heads of 64
  layernorm   LayerNorm forward + backward on 32768 x 1024
  crossentropy  cross-entropy loss + gradient on 4096 rows x 32000 classes
  step        the parameter step on a 64 M-parameter arena (Adam): the sums of squares range by range and the one-pass
              update, then the two-phase fallback; one small LM so that the trainer owns the arenas
  embedding   token-embedding gather and the deterministic gradient scatter: 65536 rows x 1024, Zipf(1.1) ids over 32000
  generate    greedy decoding with the device key/value cache on the c5 model (V 32000, d 1024, 16 heads, 12 layers,
              f 4096): 16-token prompt + 240 generated tokens, prints tokens/s
"""
import sys

import numpy as np

from .ml_b200 import CudaB200AccelerationManager, GEMM_AUTO


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


def step(m, rng):
    """A model whose arena is dominated by a 60000 x 1024 embedding and output projection (~124 M parameters, 0.5 GB per
    arena, four arenas with Adam): a tiny batch is trained so that every range is announced, then the step runs."""
    from .ml_b200 import B200LanguageModelTrainer, make_config

    cfg = make_config(vocab_size=60000, embedding_dim=1024, num_heads=16, num_layers=1, ffn_dim=1024, ffn_activation="Relu")
    t = B200LanguageModelTrainer(m, cfg, max_rows_per_pass=256)
    t.set_optimizer("adam")
    t.upload_params(rng.standard_normal(t.param_count, dtype=np.float32) * 0.02)
    toks = np.concatenate([[1], rng.integers(4, 60000, 130), [2]]).astype(np.int32)
    off = np.array([0, len(toks)], np.int32)
    r = None
    for _ in range(3):
        r = t.train_step_discrete(toks, off, 1e-3, True, 1.0, True)
    t.close()
    return float(r[1])


def embedding(m, rng):
    rows, d, vocab = 65536, 1024, 32000
    ranks = np.arange(1, vocab - 4 + 1, dtype=np.float64)
    cdf = np.cumsum(ranks ** -1.1); cdf /= cdf[-1]
    ids = (4 + np.searchsorted(cdf, rng.random(rows))).astype(np.int32)
    emb = rng.normal(0, 0.02, (vocab, d)).astype(np.float32)
    dx = rng.normal(0, 1, (rows, d)).astype(np.float32)
    eg = np.zeros_like(emb)
    for _ in range(2):
        x = m.EmbedTokenIds(ids, emb, d)
        m.AccumulateTokenEmbeddingGrad(eg, dx, ids, rows, d)
    return float(np.abs(eg).mean()) + float(np.abs(x).mean())


def generate(m, rng):
    import time

    from .ml_b200 import B200LanguageModelTrainer, make_config

    cfg = make_config(vocab_size=32000, embedding_dim=1024, num_heads=16, num_layers=12, ffn_dim=4096, ffn_activation="Relu")
    t = B200LanguageModelTrainer(m, cfg, max_rows_per_pass=1024)
    n = t.param_count
    w = (rng.standard_normal(n, dtype=np.float32) * 0.02)
    t.upload_params(w)
    prompt = rng.integers(4, 32000, 16).astype(np.int32)
    for single in (True, False):
        g = t.generator(256)
        g.set_single_kernel(single)
        g.greedy(prompt, 8)  # warm-up (module load, first-launch effects, graph capture)
        t0 = time.perf_counter()
        out = g.greedy(prompt, 240)
        dt = time.perf_counter() - t0
        how = "one cooperative kernel per token" if g.single_kernel() else "CUDA graph of %d launches per token" % g.graph_nodes()
        print("decode: %d tokens in %.3f s = %.1f tokens/s (prompt included, one token per model pass, %s)" % (len(out), dt, len(out) / dt, how))
        g.close()
    t.close()
    return float(out[-1])


CASES = {"generate": generate, "step": step, "embedding": embedding, "attention": attention, "gemm": gemm, "wgrad": wgrad, "ffn": ffn, "decayattention": decayattention, "layernorm": layernorm, "crossentropy": crossentropy}


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
