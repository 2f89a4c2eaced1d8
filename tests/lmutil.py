"""Shared helpers for the parity tests: model configs, seeded weights and synthetic batches.

Weights follow the reference's initial distributions (values only matter for being realistic):
token embedding N(0, 1/d) (LanguageModel.cs:44), projections N(0, 2/(rows+cols)) (LanguageModel.cs:53,93;
MultiHeadAttention.cs:75), FFN He-normal N(0, 2/fan_in) (Neural Network/Data.cs:135-143), LayerNorm gamma=1,
beta=0 (TransformerBlock.cs:88-92), biases 0.  Parity runs inject identical weights on both sides, so System.Random
is not reproduced; small random biases/gammas are added so that every gradient path carries signal.
"""
from __future__ import annotations

import numpy as np

from oracle import ACT, LMConfig


def lm_config(vocab=0, F=0, O=None, d=64, H=4, L=2, f=128, act="Relu", discrete=True, loss="ce", causal=True, align=64):
    c = LMConfig()
    c.vocab_size = vocab
    c.input_feature_dim = F
    c.output_dim = vocab if (discrete and O is None) else int(O)
    c.embedding_dim, c.num_heads, c.num_layers, c.ffn_dim = d, H, L, f
    c.ffn_activation = ACT[act]
    c.discrete = 1 if discrete else 0
    c.loss_kind = 0 if loss == "ce" else 1
    c.causal = 1 if causal else 0
    c.align_floats = align
    return c


def init_params(oracle, cfg, seed=0, dtype=np.float32, tensors=None, total=None):
    """Flat arena with seeded weights; padding between tensors stays zero.  The arena layout comes from the oracle, or
    from an explicit (tensors, total) pair (e.g. the device library's own b200_lm_tensor_info) when oracle is None."""
    rng = np.random.default_rng(seed)
    if tensors is None:
        total = oracle.lm_param_count(cfg)
        tensors = oracle.lm_tensors(cfg)
    P = np.zeros(total, dtype)
    d, f = cfg.embedding_dim, cfg.ffn_dim
    n0 = 1 if cfg.discrete else 2
    for idx, (off, r, c) in enumerate(tensors):
        n = r * c
        if idx < n0:
            if cfg.discrete:
                v = rng.normal(0, np.sqrt(1.0 / d), n)
            elif idx == 0:
                v = rng.normal(0, np.sqrt(2.0 / (cfg.input_feature_dim + d)), n)
            else:
                v = rng.normal(0, 0.02, n)
        elif idx < n0 + 16 * cfg.num_layers:
            t = (idx - n0) % 16
            if t < 4:
                v = rng.normal(0, np.sqrt(2.0 / (2 * d)), n)
            elif t < 8:
                v = rng.normal(0, 0.02, n)
            elif t in (8, 10):
                v = 1.0 + rng.normal(0, 0.05, n)
            elif t in (9, 11):
                v = rng.normal(0, 0.05, n)
            elif t == 12:
                v = rng.normal(0, np.sqrt(2.0 / d), n)
            elif t == 14:
                v = rng.normal(0, np.sqrt(2.0 / f), n)
            else:
                v = rng.normal(0, 0.02, n)
        elif idx == n0 + 16 * cfg.num_layers:
            v = rng.normal(0, np.sqrt(2.0 / (d + cfg.output_dim)), n)
        else:
            v = rng.normal(0, 0.02, n)
        P[off:off + n] = v.astype(dtype)
    return P


def token_batch(rng, n_seq, vocab, min_len=2, max_len=64, fixed_len=None, zipf=None):
    """Sequences [START=1, ids in [4, vocab), END=2] as (tokens, offsets)."""
    toks, off = [], [0]
    for _ in range(n_seq):
        n = fixed_len if fixed_len else int(rng.integers(min_len, max_len + 1))
        body = max(n - 2, 0)
        if zipf:
            ranks = np.arange(1, vocab - 4 + 1, dtype=np.float64)
            p = ranks ** (-zipf)
            p /= p.sum()
            ids = 4 + rng.choice(vocab - 4, size=body, p=p)
        else:
            ids = rng.integers(4, vocab, size=body)
        seq = [1] + list(ids) + [2]
        seq = seq[:max(n, 2)]
        toks += seq
        off.append(len(toks))
    return np.asarray(toks, np.int32), np.asarray(off, np.int32)


def random_walk_batch(rng, n_seq, seq_len, F, target_feature=3):
    """Per-feature Gaussian random walks (step sigma 0.01) min-max normalised to [0,1]; regression target is the
    given feature (the trainer itself applies the one-step shift)."""
    x = np.cumsum(rng.normal(0, 0.01, (n_seq, seq_len, F)), axis=1)
    mn, mx = x.min(axis=1, keepdims=True), x.max(axis=1, keepdims=True)
    x = ((x - mn) / np.maximum(mx - mn, 1e-12)).astype(np.float32)
    tgt = x[:, :, target_feature:target_feature + 1].copy()
    off = np.arange(0, (n_seq + 1) * seq_len, seq_len, dtype=np.int32)
    return x.reshape(-1, F), tgt.reshape(-1, 1), off


def tensor_names(cfg):
    return (["emb"] if cfg.discrete else ["inW", "inB"]) + [f"L{l}.{n}" for l in range(cfg.num_layers) for n in
            ("WQ", "WK", "WV", "WO", "bQ", "bK", "bV", "bO", "g1", "b1", "g2", "b2", "W1", "fb1", "W2", "fb2")] + ["Wout", "bout"]


def unclip(norm, clip_thr):
    """Factor that undoes global-norm clipping on one side: clipped = unclipped * thr/norm when norm > thr.

    Why it is needed: after clipping EVERY gradient element (and so every weight update) carries the factor thr/norm,
    and the reference adds the squares of all P gradient elements serially in FP32 (TransformerTrainer.cs:1319-1352,
    AccelerationCPU.cs:2493-2502).  That one sum is off by 1e-5..4e-5 relative at P = 1e5..1e6 (FP32 oracle against its
    float64 build), which would show up as a uniform relative error of all clipped gradients.  The norm is compared
    separately with a tolerance that says so; the element-wise comparisons multiply each side by its OWN norm/thr, so
    they measure the gradient itself at full sharpness."""
    return float(norm) / float(clip_thr) if (clip_thr is not None and norm > clip_thr) else 1.0


def _yardsticks(tensors, cfg, values, scale, key_bias_by_query_bias, score_path_by_value_path=False):
    """Per tensor (max|ref|, ||ref||_2).  With key_bias_by_query_bias the key-projection bias is measured against the
    query-projection bias of its layer: a bias added to every key moves all scores of a query by (almost) the same
    amount, which the soft-max ignores, so that gradient is the small remainder of contributions that cancel (10-100x
    below its sibling's) and its rounding error is set by the size of what cancels, not by what is left.
    score_path_by_value_path (statistical comparisons of steps with a discontinuous activation derivative only): the
    query/key projections' gradients pass through the soft-max Jacobian, which at initialisation (near-uniform
    attention) removes all but 1e-2..1e-4 of what comes in; the units flipped by TF32 rounding perturb what comes in by
    percents, so those gradients are measured against the value projection's of the same layer."""
    names = tensor_names(cfg)
    out = {}
    for (off, r, c), name in zip(tensors, names):
        v = np.asarray(values[off:off + r * c], np.float64) * scale
        out[name] = (float(np.max(np.abs(v))) if v.size else 0.0, float(np.sqrt((v * v).sum())))
    if key_bias_by_query_bias:
        for name in names:
            if name.endswith(".bK"):
                q = out[name[:-3] + ".bQ"]
                out[name] = (max(out[name][0], q[0]), max(out[name][1], q[1]))
    if score_path_by_value_path:
        for name in names:
            for mine, sibling in ((".WQ", ".WV"), (".WK", ".WV"), (".bQ", ".bV"), (".bK", ".bV")):
                if name.endswith(mine):
                    v = out[name[:-3] + sibling]
                    out[name] = (max(out[name][0], v[0]), max(out[name][1], v[1]))
    return out


def compare_gradients(tensors, cfg, exp, act, tol, what="grad", exp_scale=1.0, act_scale=1.0, key_bias_by_query_bias=False):
    """Every tensor of the gradient arena against the oracle's, each normalised by its own magnitude
    (max|diff| <= tol*max|ref| and ||diff||_2 <= tol*||ref||_2).  exp_scale / act_scale: see unclip;
    key_bias_by_query_bias: see _yardsticks (TF32 comparisons only).  Returns the worst relative max-error seen."""
    from conftest import assert_tensor_close

    ys = _yardsticks(tensors, cfg, exp, exp_scale, key_bias_by_query_bias)
    worst = 0.0
    for (off, r, c), name in zip(tensors, tensor_names(cfg)):
        e = np.asarray(exp[off:off + r * c], np.float64) * exp_scale
        a = np.asarray(act[off:off + r * c], np.float64) * act_scale
        assert_tensor_close(e, a, tol, f"{what} {name}", ref_max=ys[name][0], ref_l2=ys[name][1])
        worst = max(worst, float(np.max(np.abs(e - a))) / max(ys[name][0], 1e-300))
    return worst


def compare_updates(tensors, cfg, exp_before, exp_after, act_before, act_after, tol, what="update", exp_scale=1.0, act_scale=1.0,
                    key_bias_by_query_bias=False):
    """The weight UPDATE (after - before, each side from its own starting weights) of every tensor against the oracle's,
    normalised per tensor.  Each side rounds the stepped weight to FP32, so the observable update is quantised to the
    weight's last place: one unit of it is allowed per element on top of tol.  Comparing the weights themselves would
    hide the update (it is orders of magnitude smaller than the weight).  exp_scale / act_scale: see unclip."""
    from conftest import assert_tensor_close, ulp32

    ys = _yardsticks(tensors, cfg, np.asarray(exp_after, np.float64) - np.asarray(exp_before, np.float64), exp_scale, key_bias_by_query_bias)
    worst = 0.0
    for (off, r, c), name in zip(tensors, tensor_names(cfg)):
        s = slice(off, off + r * c)
        de = (np.asarray(exp_after[s], np.float64) - np.asarray(exp_before[s], np.float64)) * exp_scale
        da = (np.asarray(act_after[s], np.float64) - np.asarray(act_before[s], np.float64)) * act_scale
        q = ulp32(np.maximum(np.abs(exp_after[s]), np.abs(exp_before[s]))) * max(exp_scale, act_scale)
        assert_tensor_close(de, da, tol, f"{what} {name}", quantum=q, ref_max=ys[name][0], ref_l2=ys[name][1])
        worst = max(worst, float(np.max(np.maximum(np.abs(de - da) - q, 0.0))) / max(ys[name][0], 1e-300))
    return worst


def expect_failure(fn, *args, **kw):
    """Negative control: the comparison must reject this input."""
    try:
        fn(*args, **kw)
    except AssertionError:
        return
    raise AssertionError("negative control passed: the comparison cannot fail")
