// C ABI, part B: the resident language-model trainer.  Weights, gradients and activation caches stay in HBM; the
// host side below restates the orchestration of TransformerTrainer.TrainBatchDiscrete / TrainBatchContinuous
// (TransformerTrainer.cs:217-486), ForwardFromEmbeddingWithCache (:540-590) and BackpropFromOutput / BackpropBlock /
// BackpropAttention (:874-987) over PACKED passes: the valid sequences of a batch are concatenated (any mix of
// lengths) up to max_rows_per_pass rows, attention runs per sequence through a segment table, and the loss scale is
// per row (1/len of the row's sequence), which is exactly the reference's "mean over a bucket, times the bucket's
// sequence count".  Gradients accumulate across passes; one fused kernel then scales, clips and steps.
#include <algorithm>
#include <cmath>
#include <cstring>

#include "common.h"

using namespace b200;

namespace {

struct LayerOff { int64_t WQ, WK, WV, WO, bQ, bK, bV, bO, g1, b1n, g2, b2n, W1, fb1, W2, fb2; };
struct Layout {
    int64_t in0 = 0, in1 = -1;
    std::vector<LayerOff> layer;
    int64_t Wout = 0, bout = 0, total = 0;
};
int64_t al(int64_t x, int a) { return a <= 1 ? x : (x + a - 1) / a * a; }

Layout make_layout(const b200_lm_config& c) {
    Layout o;
    int a = c.align_floats < 1 ? 1 : c.align_floats, d = c.embedding_dim, f = c.ffn_dim;
    int64_t p = 0;
    if (c.discrete) { o.in0 = p; p = al(p + (int64_t)c.vocab_size * d, a); }
    else { o.in0 = p; p = al(p + (int64_t)d * c.input_feature_dim, a); o.in1 = p; p = al(p + d, a); }
    o.layer.resize((size_t)c.num_layers);
    for (auto& L : o.layer) {
        L.WQ = p; p = al(p + (int64_t)d * d, a);
        L.WK = p; p = al(p + (int64_t)d * d, a);
        L.WV = p; p = al(p + (int64_t)d * d, a);
        L.WO = p; p = al(p + (int64_t)d * d, a);
        L.bQ = p; p = al(p + d, a);
        L.bK = p; p = al(p + d, a);
        L.bV = p; p = al(p + d, a);
        L.bO = p; p = al(p + d, a);
        L.g1 = p; p = al(p + d, a);
        L.b1n = p; p = al(p + d, a);
        L.g2 = p; p = al(p + d, a);
        L.b2n = p; p = al(p + d, a);
        L.W1 = p; p = al(p + (int64_t)f * d, a);
        L.fb1 = p; p = al(p + f, a);
        L.W2 = p; p = al(p + (int64_t)d * f, a);
        L.fb2 = p; p = al(p + d, a);
    }
    o.Wout = p; p = al(p + (int64_t)c.output_dim * d, a);
    o.bout = p; p = al(p + c.output_dim, a);
    o.total = p;
    return o;
}

bool config_ok(const b200_lm_config* c) {
    if (!c) return false;
    if (c->embedding_dim <= 0 || c->num_heads <= 0 || c->num_layers < 0 || c->ffn_dim <= 0 || c->output_dim <= 0) return false;
    if (c->embedding_dim % c->num_heads) return false;
    int hd = c->embedding_dim / c->num_heads;
    if ((hd & 1) || hd > 128) return false;
    if (c->discrete ? c->vocab_size <= 0 : c->input_feature_dim <= 0) return false;
    if (c->ffn_activation < 0 || c->ffn_activation > 5) return false;
    if (c->loss_kind == 0 && c->discrete && c->output_dim != c->vocab_size) return false;
    return true;
}

struct LayerCache {
    float *x, *qkv, *attnO, *rowMax, *rowSum, *ln1In, *mean1, *var1, *n1, *z1, *a1, *ln2In, *mean2, *var2;
};

struct Seq { int index, start, len; };  // len = input length (sequence length - 1)

// Device-resident inputs of one packed pass.
struct PassDev {
    int32_t *ids = nullptr, *targets = nullptr, *pos = nullptr, *segId = nullptr, *segOff = nullptr, *perm = nullptr;
    AttnSeg* segs = nullptr;
    float *rowScale = nullptr, *contIn = nullptr, *regTgt = nullptr;
    size_t nDistinct = 0;  // distinct token ids of the pass (segments of the embedding-gradient scatter)
};
struct Pass {
    std::vector<Seq> seqs;
    int rows = 0, maxLen = 0;
};
struct Batch {  // host views of the caller's batch
    const int32_t* tokens = nullptr;
    const float* feats = nullptr;
    const float* regT = nullptr;
    const int32_t* clsT = nullptr;
    const int32_t* off = nullptr;
};

}  // namespace

struct b200_lm {
    b200_ctx* ctx = nullptr;
    std::atomic<int> refs{1};  // the owner's handle plus one per generation session
    b200_lm_config cfg{};
    Layout lay;
    float *P = nullptr, *G = nullptr, *M = nullptr, *V = nullptr;
    bool ownP = false, ownG = false;
    int opt = B200_OPT_SGD;
    float beta1 = 0.9f, beta2 = 0.999f, adam_eps = 1e-8f;
    int step_index = 0;
    int maxRows = 0, maxSeqs = 0;
    char* block = nullptr;
    std::vector<LayerCache> cache;
    float *xFinal = nullptr, *logits = nullptr, *proj = nullptr, *gbuf[4] = {nullptr, nullptr, nullptr, nullptr}, *dqkv = nullptr, *d1 = nullptr,
          *rowDot = nullptr, *rowLoss = nullptr, *stepOut = nullptr;
    int32_t* rowOk = nullptr;
    PassDev own;  // the trainer's own staging buffers (one pass)
    PassDev cur;  // inputs of the pass being processed: `own`, or a slice of a prepared batch
    // pinned host staging
    int32_t* h_int = nullptr;
    float* h_float = nullptr;
    std::vector<char> t_has_bwd;  // per group of four timing events: was the backward-end event recorded
    b200_grad_ready_fn cb = nullptr;
    void* cb_user = nullptr;
    std::vector<cudaEvent_t> cb_events;
    size_t cb_used = 0;
    std::vector<cudaEvent_t> t_events;
    size_t t_used = 0;
    float timings[4] = {0, 0, 0, 0};
    const float* rope = nullptr;
    // Sums of squares of the gradient ranges, taken as each range becomes final in the last pass (on a side stream, under
    // the remaining backward), so that the step reads the gradient once.  sumsq_done counts the ranges summed since
    // the last accumulation started; the step falls back to its two-phase form unless all of them are there.
    float* sumsq_partials = nullptr;  // [ranges][SUMSQ_BLOCKS], unused slots zero
    int n_ranges = 0, sumsq_next = 0, sumsq_done = 0;
    bool external_norm = false;       // a data-parallel layer sums after each range's all-reduce instead
    // The step does not write the scaled-and-clipped gradient back (4 bytes per parameter nobody reads in a training
    // loop, whose next step starts by zeroing the arena): the factor is kept here and applied the moment anything looks
    // at the gradient arena or adds to it, so the reference's observable state -- gradients left scaled and clipped -- holds.
    float g_pending = 1.f;
    cudaStream_t norm_stream = nullptr;
    cudaEvent_t norm_event = nullptr;
};

// A batch whose inputs have been planned, packed and copied to the device once; it can be trained on repeatedly
// (epochs over a resident dataset) without touching host memory again.
struct b200_lm_batch {
    b200_lm* lm = nullptr;
    std::vector<int32_t> tokens, off, clsT;  // host copies (needed only if a pass must be re-packed after a non-finite loss)
    std::vector<float> feats, regT;
    int n_seq = 0;
    char* block = nullptr;
    std::vector<PassDev> dev;
    void* plan = nullptr;  // Plan*
};

namespace {

int lm_fail(b200_lm* lm, int code, const char* msg) { return fail(lm->ctx, code, "%s", msg); }

cudaEvent_t next_event(std::vector<cudaEvent_t>& pool, size_t& used) {
    if (used == pool.size()) {
        cudaEvent_t e;
        cudaEventCreate(&e);
        pool.push_back(e);
    }
    return pool[used++];
}

constexpr int SUMSQ_BLOCKS = 592;  // partial sums per range (four blocks per SM of a B200)

void fire(b200_lm* lm, int64_t off, int64_t count) {
    if (!lm->cb || count <= 0) return;
    cudaEvent_t e = next_event(lm->cb_events, lm->cb_used);
    cudaEventRecord(e, lm->ctx->stream);
    lm->cb(lm->cb_user, off, count, (void*)e);
}

int settle_grads(b200_lm* lm) {
    if (lm->g_pending == 1.f) return B200_OK;
    const float f = lm->g_pending;
    lm->g_pending = 1.f;
    return k_scale_arena(lm->ctx, lm->G, lm->lay.total, f);
}

int sumsq_range(b200_lm* lm, int index, cudaStream_t stream) {
    if (index < 0 || index >= lm->n_ranges) return B200_OK;
    const auto r = lm_grad_ranges(lm)[(size_t)index];
    int blocks = 0;
    B200_TRY(k_sumsq_partials(lm->ctx, lm->G + r.first, r.second, lm->sumsq_partials + (size_t)index * SUMSQ_BLOCKS, SUMSQ_BLOCKS, stream, &blocks));
    lm->sumsq_done++;
    return B200_OK;
}

// A range of the gradient arena has received its final contribution of this step (ranges arrive in grad_ranges order):
// its sum of squares starts on the side stream, and a data-parallel caller is told.
int range_final(b200_lm* lm, int64_t off, int64_t count) {
    const int index = lm->sumsq_next++;
    if (!lm->external_norm && lm->norm_stream) {
        cudaEvent_t e = next_event(lm->cb_events, lm->cb_used);
        B200_CUDA(lm->ctx, cudaEventRecord(e, lm->ctx->stream));
        B200_CUDA(lm->ctx, cudaStreamWaitEvent(lm->norm_stream, e, 0));
        B200_TRY(sumsq_range(lm, index, lm->norm_stream));
        B200_CUDA(lm->ctx, cudaEventRecord(lm->norm_event, lm->norm_stream));
    }
    fire(lm, off, count);
    return B200_OK;
}

// The ranges of the gradient arena in the order the last pass's backward finishes them: output projection and bias,
// the blocks last to first, then the embedding / input projection.  Every rank of a data-parallel job must issue its
// collectives over exactly this list in exactly this order, whatever happened locally.
std::vector<std::pair<int64_t, int64_t>> grad_ranges(const b200_lm* lm) {
    std::vector<std::pair<int64_t, int64_t>> r;
    const Layout& o = lm->lay;
    r.emplace_back(o.Wout, o.total - o.Wout);
    for (int l = lm->cfg.num_layers - 1; l >= 0; l--) {
        const int64_t end = (l + 1 < lm->cfg.num_layers) ? o.layer[(size_t)l + 1].WQ : o.Wout;
        r.emplace_back(o.layer[(size_t)l].WQ, end - o.layer[(size_t)l].WQ);
    }
    r.emplace_back(0, lm->cfg.num_layers > 0 ? o.layer[0].WQ : o.Wout);
    return r;
}

// A rank whose last pass ran no backward (empty shard, every sequence too short or non-finite) still announces every
// range, one by one and in the same order, so that its peers' collectives find their counterparts.
void fire_all(b200_lm* lm) {
    if (!lm->cb) return;
    for (const auto& r : grad_ranges(lm)) fire(lm, r.first, r.second);
}

// ---- one packed pass ---------------------------------------------------------------------------------------------

int stage_pass(b200_lm* lm, const Batch& b, const Pass& p, PassDev& dst) {
    b200_ctx* ctx = lm->ctx;
    const b200_lm_config& c = lm->cfg;
    const int N = p.rows, S = (int)p.seqs.size(), F = c.input_feature_dim, O = c.output_dim;
    int32_t* hi = lm->h_int;
    int32_t *h_ids = hi, *h_tgt = hi + lm->maxRows, *h_pos = hi + 2 * (size_t)lm->maxRows;
    AttnSeg* h_segs = (AttnSeg*)(hi + 3 * (size_t)lm->maxRows);
    float* hf = lm->h_float;
    float* h_scale = hf;
    float* h_cont = hf + lm->maxRows;
    float* h_reg = h_cont + (size_t)lm->maxRows * (c.discrete ? 0 : F);
    int r = 0;
    for (int s = 0; s < S; s++) {
        const Seq& q = p.seqs[s];
        h_segs[s] = AttnSeg{r, q.len, r, q.len};
        float sc = c.loss_kind == 0 ? 1.0f / (float)q.len : 1.0f / ((float)q.len * O);
        for (int t = 0; t < q.len; t++, r++) {
            h_pos[r] = t;
            h_scale[r] = sc;
            if (c.discrete) {
                h_ids[r] = b.tokens[q.start + t];
                h_tgt[r] = b.tokens[q.start + t + 1];
            } else {
                memcpy(h_cont + (size_t)r * F, b.feats + (size_t)(q.start + t) * F, sizeof(float) * F);
                if (c.loss_kind == 1) memcpy(h_reg + (size_t)r * O, b.regT + (size_t)(q.start + t + 1) * O, sizeof(float) * O);
                else h_tgt[r] = b.clsT[q.start + t + 1];
            }
        }
    }
    cudaStream_t st = ctx->stream;
    B200_CUDA(ctx, cudaMemcpyAsync(dst.pos, h_pos, sizeof(int32_t) * N, cudaMemcpyHostToDevice, st));
    B200_CUDA(ctx, cudaMemcpyAsync(dst.segs, h_segs, sizeof(AttnSeg) * S, cudaMemcpyHostToDevice, st));
    B200_CUDA(ctx, cudaMemcpyAsync(dst.rowScale, h_scale, sizeof(float) * N, cudaMemcpyHostToDevice, st));
    if (c.discrete || c.loss_kind == 0) B200_CUDA(ctx, cudaMemcpyAsync(dst.targets, h_tgt, sizeof(int32_t) * N, cudaMemcpyHostToDevice, st));
    if (c.discrete) {
        B200_CUDA(ctx, cudaMemcpyAsync(dst.ids, h_ids, sizeof(int32_t) * N, cudaMemcpyHostToDevice, st));
        // rows grouped by token id for the deterministic embedding-gradient scatter
        std::vector<int32_t> sid, soff, perm;
        sort_rows_by_id(h_ids, N, c.vocab_size, sid, soff, perm);
        int32_t* h_sort = (int32_t*)(h_segs + lm->maxSeqs);
        memcpy(h_sort, sid.data(), sizeof(int32_t) * sid.size());
        memcpy(h_sort + lm->maxRows, soff.data(), sizeof(int32_t) * soff.size());
        memcpy(h_sort + 2 * (size_t)lm->maxRows + 1, perm.data(), sizeof(int32_t) * perm.size());
        B200_CUDA(ctx, cudaMemcpyAsync(dst.segId, h_sort, sizeof(int32_t) * sid.size(), cudaMemcpyHostToDevice, st));
        B200_CUDA(ctx, cudaMemcpyAsync(dst.segOff, h_sort + lm->maxRows, sizeof(int32_t) * soff.size(), cudaMemcpyHostToDevice, st));
        B200_CUDA(ctx, cudaMemcpyAsync(dst.perm, h_sort + 2 * (size_t)lm->maxRows + 1, sizeof(int32_t) * perm.size(), cudaMemcpyHostToDevice, st));
        dst.nDistinct = sid.size();
    } else {
        B200_CUDA(ctx, cudaMemcpyAsync(dst.contIn, h_cont, sizeof(float) * (size_t)N * F, cudaMemcpyHostToDevice, st));
        if (c.loss_kind == 1) B200_CUDA(ctx, cudaMemcpyAsync(dst.regTgt, h_reg, sizeof(float) * (size_t)N * O, cudaMemcpyHostToDevice, st));
    }
    return B200_OK;
}

// Three products against the per-layer Q/K/V weights.  When the arena places WQ|WK|WV (and the biases) back to back
// they are one [3d, d] matrix and one GEMM; otherwise (padding between tensors) three GEMMs into column blocks.
bool qkv_fused(const b200_lm* lm, const LayerOff& L) {
    int64_t d = lm->cfg.embedding_dim;
    return L.WK == L.WQ + d * d && L.WV == L.WK + d * d && L.bK == L.bQ + d && L.bV == L.bK + d;
}

// In TF32 mode the attention kernels run on tensor cores; their operands are rounded to TF32 where they are produced
// (Q/K/V projection epilogue, rotary kernel, attention-output dX epilogue) so that tiles can be copied as they are.
bool tf32_attention(const b200_lm* lm) {
    const b200_ctx* ctx = lm->ctx;
    const int hd = lm->cfg.embedding_dim / lm->cfg.num_heads;
    if (ctx->gemm_mode == B200_GEMM_FP32_SIMT || ctx->cc_major < 8 || hd < 8 || hd > 64) return false;
    return ctx->gemm_mode == B200_GEMM_TF32_TCGEN05 || lm->cfg.embedding_dim >= 128;  // same rule as attn_tc_eligible
}

int forward_pass(b200_lm* lm, const Pass& p) {
    b200_ctx* ctx = lm->ctx;
    const b200_lm_config& c = lm->cfg;
    const int N = p.rows, d = c.embedding_dim, H = c.num_heads, hd = d / H, f = c.ffn_dim, O = c.output_dim;
    const float* P = lm->P;
    float* x = c.num_layers > 0 ? lm->cache[0].x : lm->xFinal;
    if (c.discrete) B200_TRY(k_embed(ctx, lm->cur.ids, N, P + lm->lay.in0, d, x));
    else B200_TRY(linear_fwd(ctx, lm->cur.contIn, N, c.input_feature_dim, P + lm->lay.in0, P + lm->lay.in1, d, x, d));
    for (int l = 0; l < c.num_layers; l++) {
        const LayerOff& L = lm->lay.layer[(size_t)l];
        LayerCache& k = lm->cache[(size_t)l];
        const int rnd = tf32_attention(lm) ? 1 : 0;
        {
            const int nParts = qkv_fused(lm, L) ? 1 : 3;
            const int64_t Ws[3] = {L.WQ, L.WK, L.WV}, Bs[3] = {L.bQ, L.bK, L.bV};
            for (int i = 0; i < nParts; i++) {
                Gemm g;
                g.M = N; g.N = nParts == 1 ? 3 * d : d; g.K = d; g.A = k.x; g.lda = d; g.B = P + Ws[i]; g.ldb = d; g.transB = 1;
                g.C = k.qkv + i * d; g.ldc = 3 * d; g.bias = P + Bs[i]; g.round_tf32 = rnd;
                // rotary embedding of the Q and K column blocks, inside the epilogue where the engine allows
                g.rope_table = lm->rope; g.rope_pos = lm->cur.pos; g.rope_head_dim = hd;
                g.rope_cols = nParts == 1 ? 2 * d : (i < 2 ? d : 0);
                if (g.rope_cols == 0) g.rope_table = nullptr;
                B200_TRY(gemm(ctx, g));
            }
        }
        Attn a;
        a.Q = k.qkv; a.K = k.qkv + d; a.V = k.qkv + 2 * d; a.ldq = a.ldk = a.ldv = 3 * d;
        a.numHeads = H; a.headDim = hd; a.scale = 1.0f / sqrtf((float)hd); a.causal = c.causal;
        a.segs_dev = lm->cur.segs; a.nSeg = (int)p.seqs.size(); a.maxQLen = a.maxKLen = p.maxLen; a.totalQ = a.totalK = N;
        a.O = k.attnO; a.ldo = d; a.rowMax = k.rowMax; a.rowSum = k.rowSum; a.pre_rounded = rnd;
        B200_TRY(attn_forward(ctx, a));
        B200_TRY(linear_fwd(ctx, k.attnO, N, d, P + L.WO, P + L.bO, d, lm->proj, d));
        B200_TRY(k_ln_forward(ctx, k.x, lm->proj, P + L.g1, P + L.b1n, N, d, 1e-5f, k.n1, k.mean1, k.var1, nullptr, k.ln1In));
        {
            Gemm g;
            g.M = N; g.N = f; g.K = d; g.A = k.n1; g.lda = d; g.B = P + L.W1; g.ldb = d; g.transB = 1;
            // Only the activation is cached: the backward pass recovers act'(z) from it (a negative zero marks the
            // ReLU outputs that came from z < 0).  Swish is the one activation whose derivative needs z itself.
            g.C = k.a1; g.ldc = f; g.bias = P + L.fb1; g.act = c.ffn_activation; g.act_sign_zero = 1;
            if (c.ffn_activation == B200_ACT_SWISH) { g.zout = k.z1; g.ldz = f; }
            B200_TRY(gemm(ctx, g));
        }
        B200_TRY(linear_fwd(ctx, k.a1, N, f, P + L.W2, P + L.fb2, d, lm->proj, d));
        float* nx = (l + 1 < c.num_layers) ? lm->cache[(size_t)l + 1].x : lm->xFinal;
        B200_TRY(k_ln_forward(ctx, k.n1, lm->proj, P + L.g2, P + L.b2n, N, d, 1e-5f, nx, k.mean2, k.var2, nullptr, k.ln2In));
    }
    B200_TRY(linear_fwd(ctx, lm->xFinal, N, d, P + lm->lay.Wout, P + lm->lay.bout, O, lm->logits, O));
    return B200_OK;
}

int loss_pass(b200_lm* lm, const Pass& p) {
    const b200_lm_config& c = lm->cfg;
    if (c.loss_kind == 0)
        return k_cross_entropy(lm->ctx, lm->logits, p.rows, c.output_dim, lm->cur.targets, p.rows, lm->cur.rowScale, 0.f, lm->logits, lm->rowLoss, lm->rowOk);
    return k_mse(lm->ctx, lm->logits, p.rows, c.output_dim, lm->cur.regTgt, p.rows, lm->cur.rowScale, 0.f, lm->logits, lm->rowLoss, lm->rowOk);
}

int backward_pass(b200_lm* lm, const Pass& p, bool notify) {
    b200_ctx* ctx = lm->ctx;
    const b200_lm_config& c = lm->cfg;
    const int N = p.rows, d = c.embedding_dim, H = c.num_heads, hd = d / H, f = c.ffn_dim, O = c.output_dim;
    const float* P = lm->P;
    float* G = lm->G;
    float *dX = lm->gbuf[0], *t1 = lm->gbuf[1], *t2 = lm->gbuf[2], *t3 = lm->gbuf[3];
    // TransformerTrainer.cs:874-879: output projection.
    B200_TRY(wgrad(ctx, lm->logits, O, lm->xFinal, d, N, O, d, G + lm->lay.Wout, G + lm->lay.bout));
    B200_TRY(dgrad(ctx, lm->logits, O, P + lm->lay.Wout, N, O, d, dX, 0));
    if (notify) B200_TRY(range_final(lm, lm->lay.Wout, lm->lay.total - lm->lay.Wout));
    for (int l = c.num_layers - 1; l >= 0; l--) {
        const LayerOff& L = lm->lay.layer[(size_t)l];
        LayerCache& k = lm->cache[(size_t)l];
        // LN2 backward (:903-906): dFF -> t1, gamma/beta grads accumulate.
        // The column sums of dFF are the bias gradient of the FFN output layer: taken in the same pass.
        B200_TRY(k_ln_backward(ctx, dX, nullptr, k.ln2In, P + L.g2, k.mean2, k.var2, N, d, 1e-5f, t1, G + L.g2, G + L.b2n, 1, G + L.fb2));
        // FFN backward (NeuralNetwork.cs:773-884).  delta2 = dFF (output activation None).
        B200_TRY(wgrad(ctx, t1, d, k.a1, f, N, d, f, G + L.W2, nullptr));
        {
            Gemm g;  // delta1 = (delta2 * W2) o act'(z1)
            g.M = N; g.N = f; g.K = d; g.A = t1; g.lda = d; g.B = P + L.W2; g.ldb = f; g.C = lm->d1; g.ldc = f;
            if (c.ffn_activation == B200_ACT_SWISH) { g.mulz = k.z1; g.ldmulz = f; }
            else { g.mulz = k.a1; g.ldmulz = f; g.mulz_is_act = 1; }
            g.mulz_act = c.ffn_activation;
            B200_TRY(gemm(ctx, g));
        }
        B200_TRY(wgrad(ctx, lm->d1, f, k.n1, d, N, f, d, G + L.W1, G + L.fb1));
        {
            Gemm g;  // dNormed1 = delta1 * W1 + dFF  (:908-909, residual add fused)
            g.M = N; g.N = d; g.K = f; g.A = lm->d1; g.lda = f; g.B = P + L.W1; g.ldb = d; g.C = t2; g.ldc = d;
            g.addmat = t1; g.ldadd = d;
            B200_TRY(gemm(ctx, g));
        }
        // LN1 backward (:913-916): dAttnResidual -> t3.
        // Its column sums are the bias gradient of the attention output projection.
        B200_TRY(k_ln_backward(ctx, t2, nullptr, k.ln1In, P + L.g1, k.mean1, k.var1, N, d, 1e-5f, t3, G + L.g1, G + L.b1n, 1, G + L.bO));
        // BackpropAttention (:933-987): output projection, attention core, inverse rotary, Q/K/V projections.
        B200_TRY(wgrad(ctx, t3, d, k.attnO, d, N, d, d, G + L.WO, nullptr));
        {
            Gemm g;  // dConcatenated = dAttnResidual * WO (zero-initialised += in the reference)
            g.M = N; g.N = d; g.K = d; g.A = t3; g.lda = d; g.B = P + L.WO; g.ldb = d; g.C = t1; g.ldc = d;
            g.round_tf32 = tf32_attention(lm) ? 1 : 0;
            B200_TRY(gemm(ctx, g));
        }
        Attn a;
        a.Q = k.qkv; a.K = k.qkv + d; a.V = k.qkv + 2 * d; a.ldq = a.ldk = a.ldv = 3 * d;
        a.numHeads = H; a.headDim = hd; a.scale = 1.0f / sqrtf((float)hd); a.causal = c.causal;
        a.segs_dev = lm->cur.segs; a.nSeg = (int)p.seqs.size(); a.maxQLen = a.maxKLen = p.maxLen; a.totalQ = a.totalK = N;
        a.O = k.attnO; a.ldo = d; a.rowMax = k.rowMax; a.rowSum = k.rowSum; a.rowDot = lm->rowDot;
        a.dO = t1; a.lddo = d; a.dQ = lm->dqkv; a.dK = lm->dqkv + d; a.dV = lm->dqkv + 2 * d; a.lddq = a.lddk = a.lddv = 3 * d;
        a.pre_rounded = tf32_attention(lm) ? 1 : 0;
        a.rope_table = lm->rope; a.rope_pos = lm->cur.pos;  // inverse rotation of dQ and dK
        B200_TRY(attn_backward(ctx, a));
        float* out = t2;  // dX of the layer input = dQKV * Wqkv + dAttnResidual (:919, residual add fused)
        if (qkv_fused(lm, L)) {
            B200_TRY(wgrad(ctx, lm->dqkv, 3 * d, k.x, d, N, 3 * d, d, G + L.WQ, G + L.bQ));
            Gemm g;
            g.M = N; g.N = d; g.K = 3 * d; g.A = lm->dqkv; g.lda = 3 * d; g.B = P + L.WQ; g.ldb = d; g.C = out; g.ldc = d;
            g.addmat = t3; g.ldadd = d;
            B200_TRY(gemm(ctx, g));
        } else {
            const int64_t Ws[3] = {L.WQ, L.WK, L.WV}, Bs[3] = {L.bQ, L.bK, L.bV};
            for (int i = 0; i < 3; i++) {
                B200_TRY(wgrad(ctx, lm->dqkv + i * d, 3 * d, k.x, d, N, d, d, G + Ws[i], G + Bs[i]));
                Gemm g;
                g.M = N; g.N = d; g.K = d; g.A = lm->dqkv + i * d; g.lda = 3 * d; g.B = P + Ws[i]; g.ldb = d; g.C = out; g.ldc = d;
                if (i == 0) { g.addmat = t3; g.ldadd = d; } else g.accumulate = 1;
                B200_TRY(gemm(ctx, g));
            }
        }
        std::swap(dX, t2);
        if (notify) {
            int64_t end = (l + 1 < c.num_layers) ? lm->lay.layer[(size_t)l + 1].WQ : lm->lay.Wout;
            B200_TRY(range_final(lm, L.WQ, end - L.WQ));
        }
    }
    // BackpropInput (:887-896)
    if (c.discrete)
        B200_TRY(k_embed_scatter(ctx, G + lm->lay.in0, dX, nullptr, lm->cur.segId, lm->cur.segOff, lm->cur.perm, (int)lm->cur.nDistinct, d));
    else
        B200_TRY(wgrad(ctx, dX, d, lm->cur.contIn, c.input_feature_dim, N, d, c.input_feature_dim, G + lm->lay.in0, G + lm->lay.in1));
    if (notify) {
        int64_t end = c.num_layers > 0 ? lm->lay.layer[0].WQ : lm->lay.Wout;
        B200_TRY(range_final(lm, 0, end));
    }
    // the swap above rotates local names only; restore the canonical buffer order for the next pass
    return B200_OK;
}

// The plan of a batch: which sequences are trained, the distinct lengths in order of first appearance (the
// reference's buckets, TransformerTrainer.cs:229-245) and the packed passes.
struct Plan {
    std::vector<int> bucketLens;
    std::vector<Pass> passes;
};

int plan_batch(b200_lm* lm, const Batch& b, int n_seq, Plan& plan) {
    b200_ctx* ctx = lm->ctx;
    const b200_lm_config& c = lm->cfg;
    std::vector<Seq> seqs;
    for (int s = 0; s < n_seq; s++) {
        int start = b.off[s], n = b.off[s + 1] - b.off[s];
        if (n < 2) continue;
        bool ok = true;
        if (c.discrete) {  // TransformerTrainer.cs:1467-1478 TokensAreValid
            for (int t = 0; t < n && ok; t++) ok = (uint32_t)b.tokens[start + t] < (uint32_t)c.vocab_size;
        } else {
            for (int64_t i = 0; i < (int64_t)n * c.input_feature_dim && ok; i++) ok = std::isfinite(b.feats[(size_t)start * c.input_feature_dim + i]);
            if (ok && c.loss_kind == 1)
                for (int64_t i = 0; i < (int64_t)n * c.output_dim && ok; i++) ok = std::isfinite(b.regT[(size_t)start * c.output_dim + i]);
            if (ok && c.loss_kind == 0)
                for (int t = 0; t < n && ok; t++) ok = (uint32_t)b.clsT[start + t] < (uint32_t)c.output_dim;
        }
        if (!ok) continue;
        if (n - 1 > lm->maxRows) return fail(ctx, B200_ERR_OUT_OF_RANGE, "sequence %d has %d rows, above max_rows_per_pass %d", s, n - 1, lm->maxRows);
        seqs.push_back(Seq{s, start, n - 1});
        if (std::find(plan.bucketLens.begin(), plan.bucketLens.end(), n - 1) == plan.bucketLens.end()) plan.bucketLens.push_back(n - 1);
    }
    if (seqs.empty()) return B200_OK;
    Pass cur;
    for (int len : plan.bucketLens)
        for (const Seq& q : seqs) {
            if (q.len != len) continue;
            if (!cur.seqs.empty() && (cur.rows + q.len > lm->maxRows || (int)cur.seqs.size() >= lm->maxSeqs)) {
                plan.passes.push_back(cur);
                cur = Pass();
            }
            cur.seqs.push_back(q);
            cur.rows += q.len;
            cur.maxLen = std::max(cur.maxLen, q.len);
        }
    plan.passes.push_back(cur);
    return B200_OK;
}

// Accumulates gradients of all planned sequences.  loss_sum = sum over sequences of their mean loss (the reference's
// totalLoss), valid = number of contributing sequences.  `staged`, when given, holds the device-resident inputs of
// every pass (a prepared batch); otherwise each pass is staged from the host arrays in `b`.
int run_plan(b200_lm* lm, const Batch& b, const Plan& plan, const std::vector<PassDev>* staged, float* loss_sum, int32_t* valid_count) {
    b200_ctx* ctx = lm->ctx;
    const b200_lm_config& c = lm->cfg;
    *loss_sum = 0.f;
    *valid_count = 0;
    lm->cb_used = 0;
    lm->t_used = 0;
    B200_TRY(settle_grads(lm));  // adding to a gradient whose scaling is still owed
    lm->sumsq_next = lm->sumsq_done = 0;
    B200_CUDA(ctx, cudaMemsetAsync(lm->sumsq_partials, 0, sizeof(float) * (size_t)lm->n_ranges * SUMSQ_BLOCKS, ctx->stream));
    const std::vector<int>& bucketLens = plan.bucketLens;
    const std::vector<Pass>& passes = plan.passes;
    if (passes.empty()) {
        fire_all(lm);
        return B200_OK;
    }
    auto bucket_of = [&](int len) { return (size_t)(std::find(bucketLens.begin(), bucketLens.end(), len) - bucketLens.begin()); };
    // per-length running sums for the loss, in the reference's row order
    std::vector<float> bucketSum(bucketLens.size(), 0.f);
    std::vector<int> bucketCount(bucketLens.size(), 0);
    std::vector<float> rowLoss((size_t)lm->maxRows);
    std::vector<int32_t> rowOk((size_t)lm->maxRows);
    bool notified = false;
    for (size_t pi = 0; pi < passes.size(); pi++) {
        Pass p = passes[pi];
        const bool last = pi + 1 == passes.size();
        for (int attempt = 0; attempt < 64 && !p.seqs.empty(); attempt++) {
            cudaEvent_t e0 = next_event(lm->t_events, lm->t_used), e1 = next_event(lm->t_events, lm->t_used),
                        e2 = next_event(lm->t_events, lm->t_used), e3 = next_event(lm->t_events, lm->t_used);
            lm->t_has_bwd.resize(lm->t_used / 4, 0);
            lm->t_has_bwd[lm->t_used / 4 - 1] = 0;
            if (staged && attempt == 0) {
                lm->cur = (*staged)[pi];
            } else {
                B200_TRY(stage_pass(lm, b, p, lm->own));
                lm->cur = lm->own;
            }
            cudaEventRecord(e0, ctx->stream);
            B200_TRY(forward_pass(lm, p));
            cudaEventRecord(e1, ctx->stream);
            B200_TRY(loss_pass(lm, p));
            cudaEventRecord(e2, ctx->stream);
            B200_CUDA(ctx, cudaMemcpyAsync(rowLoss.data(), lm->rowLoss, sizeof(float) * p.rows, cudaMemcpyDeviceToHost, ctx->stream));
            B200_CUDA(ctx, cudaMemcpyAsync(rowOk.data(), lm->rowOk, sizeof(int32_t) * p.rows, cudaMemcpyDeviceToHost, ctx->stream));
            B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            // TransformerTrainer.cs:271-272 / :286-287: a non-finite loss or gradient drops the sequences of that length
            // (here: of that length within this pass).
            std::vector<char> lenBad(bucketLens.size(), 0);
            std::vector<float> passSum(bucketLens.size(), 0.f);
            int r = 0;
            for (const Seq& q : p.seqs) {
                size_t bi = bucket_of(q.len);
                for (int t = 0; t < q.len; t++, r++) {
                    passSum[bi] += rowLoss[(size_t)r];
                    if (!rowOk[(size_t)r]) lenBad[bi] = 1;
                }
            }
            for (size_t bi = 0; bi < bucketLens.size(); bi++)
                if (!std::isfinite(passSum[bi])) lenBad[bi] = 1;
            bool anyBad = false;
            Pass good;
            for (const Seq& q : p.seqs) {
                if (lenBad[bucket_of(q.len)]) { anyBad = true; continue; }
                good.seqs.push_back(q);
                good.rows += q.len;
                good.maxLen = std::max(good.maxLen, q.len);
            }
            float ms;
            if (cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess) lm->timings[0] += ms;
            if (cudaEventElapsedTime(&ms, e1, e2) == cudaSuccess) lm->timings[1] += ms;
            if (good.seqs.empty()) break;
            if (anyBad) {  // rerun the pass with the finite sequences only: their activations must not mix with the others'
                p = good;
                continue;
            }
            r = 0;
            for (const Seq& q : p.seqs) {
                size_t bi = bucket_of(q.len);
                for (int t = 0; t < q.len; t++, r++) bucketSum[bi] += rowLoss[(size_t)r];
                bucketCount[bi]++;
            }
            B200_TRY(backward_pass(lm, p, last));
            cudaEventRecord(e3, ctx->stream);
            lm->t_has_bwd[lm->t_used / 4 - 1] = 1;
            if (last && lm->cb) notified = true;
            break;
        }
    }
    if (lm->cb && !notified) fire_all(lm);
    float total = 0.f;
    int valid = 0;
    for (size_t bi = 0; bi < bucketLens.size(); bi++) {
        if (bucketCount[bi] == 0) continue;
        float denom = (float)bucketCount[bi] * bucketLens[bi] * (c.loss_kind == 1 ? c.output_dim : 1);
        float loss = bucketSum[bi] / denom;       // CPU:2438 / CPU:2489: mean over the bucket's rows
        total += loss * (float)bucketCount[bi];   // TransformerTrainer.cs:294
        valid += bucketCount[bi];
    }
    *loss_sum = total;
    *valid_count = valid;
    return B200_OK;
}

int accumulate(b200_lm* lm, const Batch& b, int n_seq, float* loss_sum, int32_t* valid_count) {
    b200_ctx* ctx = lm->ctx;
    std::lock_guard<std::mutex> lock(ctx->mu);
    B200_CUDA(ctx, cudaSetDevice(ctx->device));
    *loss_sum = 0.f;
    *valid_count = 0;
    Plan plan;
    B200_TRY(plan_batch(lm, b, n_seq, plan));
    return run_plan(lm, b, plan, nullptr, loss_sum, valid_count);
}

// TransformerTrainer.Validate / ValidateContinuous (TransformerTrainer.cs:1142-1268): forward and loss only.  Every
// valid sequence contributes (its mean loss) x (its trained rows); a sequence whose loss is not finite is skipped; the
// result is the sum divided by the contributing rows.  Sequences are packed into passes like in training.
int validate(b200_lm* lm, const Batch& b, int n_seq, float* mean_loss, int32_t* items) {
    b200_ctx* ctx = lm->ctx;
    const b200_lm_config& c = lm->cfg;
    std::lock_guard<std::mutex> lock(ctx->mu);
    B200_CUDA(ctx, cudaSetDevice(ctx->device));
    *mean_loss = 0.f;
    *items = 0;
    Plan plan;
    B200_TRY(plan_batch(lm, b, n_seq, plan));
    // per-sequence results in input order, so that the summation order is the reference's (sequence by sequence)
    std::vector<float> seqLoss((size_t)n_seq, 0.f);
    std::vector<char> seqUsed((size_t)n_seq, 0);
    std::vector<float> rowLoss((size_t)lm->maxRows);
    for (const Pass& p : plan.passes) {
        if (p.seqs.empty()) continue;
        B200_TRY(stage_pass(lm, b, p, lm->own));
        lm->cur = lm->own;
        B200_TRY(forward_pass(lm, p));
        B200_TRY(loss_pass(lm, p));  // also writes the loss gradient over the logits, which nobody reads here
        B200_CUDA(ctx, cudaMemcpyAsync(rowLoss.data(), lm->rowLoss, sizeof(float) * p.rows, cudaMemcpyDeviceToHost, ctx->stream));
        B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        int r = 0;
        for (const Seq& q : p.seqs) {
            float sum = 0.f;
            for (int t = 0; t < q.len; t++, r++) sum += rowLoss[(size_t)r];
            const float loss = sum / ((float)q.len * (c.loss_kind == 1 ? c.output_dim : 1));  // CPU:2438 / CPU:2489
            seqLoss[(size_t)q.index] = loss * (float)q.len;
            seqUsed[(size_t)q.index] = std::isfinite(loss) ? 1 : 0;
        }
    }
    B200_TRY(check_device_status(ctx));
    float total = 0.f;
    int32_t count = 0;
    for (int sidx = 0; sidx < n_seq; sidx++) {
        if (!seqUsed[(size_t)sidx]) continue;
        total += seqLoss[(size_t)sidx];
        count += b.off[sidx + 1] - b.off[sidx] - 1;
    }
    *items = count;
    *mean_loss = count > 0 ? total / (float)count : 0.f;
    return B200_OK;
}

int collect_backward_time(b200_lm* lm) {
    // events are laid out in groups of four per attempted pass: forward start, forward end, loss end, backward end
    for (size_t i = 0; i + 3 < lm->t_used; i += 4) {
        float ms;
        if (i / 4 < lm->t_has_bwd.size() && lm->t_has_bwd[i / 4] &&
            cudaEventElapsedTime(&ms, lm->t_events[i + 2], lm->t_events[i + 3]) == cudaSuccess)
            lm->timings[2] += ms;
    }
    return B200_OK;
}

int apply_step(b200_lm* lm, int valid, float lr, int use_clip, float thr, int do_step, float* grad_norm) {
    b200_ctx* ctx = lm->ctx;
    std::lock_guard<std::mutex> lock(ctx->mu);
    B200_CUDA(ctx, cudaSetDevice(ctx->device));
    if (grad_norm) *grad_norm = 0.f;
    if (valid <= 0) return B200_OK;  // TransformerTrainer.cs:309-310
    if (use_clip && !(thr > 0.f && std::isfinite(thr)))
        return fail(ctx, B200_ERR_OUT_OF_RANGE, "Gradient clip threshold must be finite and positive.");
    if (lm->opt == B200_OPT_ADAM && do_step) {
        if (!lm->M) {
            B200_CUDA(ctx, cudaMalloc(&lm->M, sizeof(float) * (size_t)lm->lay.total));
            B200_CUDA(ctx, cudaMalloc(&lm->V, sizeof(float) * (size_t)lm->lay.total));
            B200_CUDA(ctx, cudaMemsetAsync(lm->M, 0, sizeof(float) * (size_t)lm->lay.total, ctx->stream));
            B200_CUDA(ctx, cudaMemsetAsync(lm->V, 0, sizeof(float) * (size_t)lm->lay.total, ctx->stream));
        }
        lm->step_index++;
    }
    B200_TRY(settle_grads(lm));
    cudaEvent_t e0 = next_event(lm->t_events, lm->t_used), e1 = next_event(lm->t_events, lm->t_used);
    cudaEventRecord(e0, ctx->stream);
    if (lm->sumsq_done == lm->n_ranges && lm->n_ranges > 0) {  // every range was summed as it became final: one pass
        if (!lm->external_norm) B200_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, lm->norm_event, 0));
        B200_TRY(k_fused_step_presummed(ctx, lm->P, lm->G, lm->M, lm->V, lm->lay.total, lm->sumsq_partials, lm->n_ranges * SUMSQ_BLOCKS,
                                        1.0f / (float)valid, lr, use_clip, thr, do_step, lm->opt, lm->beta1, lm->beta2, lm->adam_eps, lm->step_index,
                                        lm->stepOut, 0));
    } else {
        B200_TRY(k_fused_step(ctx, lm->P, lm->G, lm->M, lm->V, lm->lay.total, 1.0f / (float)valid, lr, use_clip, thr, do_step, lm->opt, lm->beta1,
                              lm->beta2, lm->adam_eps, lm->step_index, lm->stepOut, 0));
    }
    lm->sumsq_done = 0;  // one step per set of sums
    cudaEventRecord(e1, ctx->stream);
    B200_CUDA(ctx, cudaMemcpyAsync(ctx->pinned, lm->stepOut, 2 * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    B200_TRY(check_device_status(ctx));
    if (grad_norm) *grad_norm = ctx->pinned[0];
    // the factor the kernel applied to every gradient element on its way into the update (a non-finite norm zeroed the arena instead)
    lm->g_pending = std::isfinite(ctx->pinned[0]) ? (1.0f / (float)valid) * ctx->pinned[1] : 1.f;
    float ms;
    if (cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess) lm->timings[3] += ms;
    lm->t_used -= 2;
    collect_backward_time(lm);
    return B200_OK;
}

int zero_grads(b200_lm* lm) {
    b200_ctx* ctx = lm->ctx;
    std::lock_guard<std::mutex> lock(ctx->mu);
    B200_CUDA(ctx, cudaSetDevice(ctx->device));
    for (int i = 0; i < 4; i++) lm->timings[i] = 0.f;
    lm->sumsq_next = lm->sumsq_done = 0;
    lm->g_pending = 1.f;
    B200_CUDA(ctx, cudaMemsetAsync(lm->sumsq_partials, 0, sizeof(float) * (size_t)lm->n_ranges * SUMSQ_BLOCKS, ctx->stream));
    B200_CUDA(ctx, cudaMemsetAsync(lm->G, 0, sizeof(float) * (size_t)lm->lay.total, ctx->stream));
    return B200_OK;
}

}  // namespace

namespace b200 {
b200_ctx* lm_context(b200_lm* lm) { return lm->ctx; }
void lm_retain(b200_lm* lm) { lm->refs.fetch_add(1); }
int64_t lm_param_total(const b200_lm* lm) { return lm->lay.total; }
const b200_lm_config& lm_config_of(const b200_lm* lm) { return lm->cfg; }
std::vector<std::pair<int64_t, int64_t>> lm_grad_ranges(const b200_lm* lm) { return grad_ranges(lm); }
void lm_set_external_norm(b200_lm* lm, bool on) { lm->external_norm = on; }
int lm_sumsq_range(b200_lm* lm, int index, cudaStream_t stream) { return sumsq_range(lm, index, stream); }
}  // namespace b200

extern "C" {

int64_t b200_lm_param_count(const b200_lm_config* cfg) { return config_ok(cfg) ? make_layout(*cfg).total : -1; }
int32_t b200_lm_tensor_count(const b200_lm_config* cfg) { return config_ok(cfg) ? (cfg->discrete ? 1 : 2) + 16 * cfg->num_layers + 2 : -1; }
int32_t b200_lm_tensor_info(const b200_lm_config* cfg, int32_t idx, int64_t* off, int32_t* rows, int32_t* cols) {
    if (!config_ok(cfg) || !off || !rows || !cols) return B200_ERR_INVALID_ARG;
    Layout o = make_layout(*cfg);
    int d = cfg->embedding_dim, f = cfg->ffn_dim, n0 = cfg->discrete ? 1 : 2;
    if (idx < 0) return B200_ERR_OUT_OF_RANGE;
    if (idx < n0) {
        if (cfg->discrete) { *off = o.in0; *rows = cfg->vocab_size; *cols = d; }
        else if (idx == 0) { *off = o.in0; *rows = d; *cols = cfg->input_feature_dim; }
        else { *off = o.in1; *rows = 1; *cols = d; }
        return B200_OK;
    }
    if (idx < n0 + 16 * cfg->num_layers) {
        const LayerOff& L = o.layer[(size_t)((idx - n0) / 16)];
        int t = (idx - n0) % 16;
        const int64_t offs[16] = {L.WQ, L.WK, L.WV, L.WO, L.bQ, L.bK, L.bV, L.bO, L.g1, L.b1n, L.g2, L.b2n, L.W1, L.fb1, L.W2, L.fb2};
        const int rws[16] = {d, d, d, d, 1, 1, 1, 1, 1, 1, 1, 1, f, 1, d, 1};
        const int cls[16] = {d, d, d, d, d, d, d, d, d, d, d, d, d, f, f, d};
        *off = offs[t]; *rows = rws[t]; *cols = cls[t];
        return B200_OK;
    }
    if (idx == n0 + 16 * cfg->num_layers) { *off = o.Wout; *rows = cfg->output_dim; *cols = d; return B200_OK; }
    if (idx == n0 + 16 * cfg->num_layers + 1) { *off = o.bout; *rows = 1; *cols = cfg->output_dim; return B200_OK; }
    return B200_ERR_OUT_OF_RANGE;
}

int32_t b200_lm_create(b200_ctx* ctx, const b200_lm_config* cfg, float* params_dev, float* grads_dev, int32_t max_rows, b200_lm** out) {
    if (!ctx || !out) return B200_ERR_INVALID_ARG;
    *out = nullptr;
    if (!config_ok(cfg)) return fail(ctx, B200_ERR_INVALID_ARG, "invalid model configuration");
    if (max_rows <= 0) return fail(ctx, B200_ERR_INVALID_ARG, "max_rows_per_pass must be positive");
    std::lock_guard<std::mutex> lock(ctx->mu);
    B200_CUDA(ctx, cudaSetDevice(ctx->device));
    b200_lm* lm = new b200_lm();
    lm->ctx = ctx;
    ctx_retain(ctx);
    lm->cfg = *cfg;
    if (lm->cfg.align_floats < 1) lm->cfg.align_floats = 1;
    lm->lay = make_layout(lm->cfg);
    lm->maxRows = max_rows;
    lm->maxSeqs = std::min(max_rows, 65535);
    const b200_lm_config& c = lm->cfg;
    const size_t N = (size_t)max_rows, d = (size_t)c.embedding_dim, f = (size_t)c.ffn_dim, H = (size_t)c.num_heads, O = (size_t)c.output_dim,
                 F = (size_t)c.input_feature_dim, Lc = (size_t)c.num_layers;
    auto rnd = [](size_t n) { return (n + 63) & ~(size_t)63; };  // keep every buffer 256-byte aligned
    size_t perLayer = rnd(N * d) * 5 + rnd(N * 3 * d) + rnd(N * H) * 2 + rnd(N) * 4 + rnd(N * f) * 2;
    size_t floats = perLayer * Lc + rnd(N * d) /*xFinal*/ + rnd(N * O) /*logits*/ + rnd(N * d) * 5 /*proj, gbuf*/ + rnd(N * 3 * d) + rnd(N * f) +
                    rnd(N * H) + rnd(N * std::max<size_t>(F, 1)) + rnd(N * O) + rnd(N) * 2 + 64;
    size_t ints = rnd(N) * 7 + rnd(4 * (size_t)lm->maxSeqs) + 64;
    auto cleanup = [&](int rc) { b200_lm_destroy(lm); return rc; };
    cudaError_t e;
    if (!params_dev) {
        if ((e = cudaMalloc(&lm->P, sizeof(float) * (size_t)lm->lay.total)) != cudaSuccess)
            return cleanup(fail(ctx, B200_ERR_CUDA, "parameter arena allocation failed: %s", cudaGetErrorString(e)));
        lm->ownP = true;
        cudaMemsetAsync(lm->P, 0, sizeof(float) * (size_t)lm->lay.total, ctx->stream);
    } else lm->P = params_dev;
    if (!grads_dev) {
        if ((e = cudaMalloc(&lm->G, sizeof(float) * (size_t)lm->lay.total)) != cudaSuccess)
            return cleanup(fail(ctx, B200_ERR_CUDA, "gradient arena allocation failed: %s", cudaGetErrorString(e)));
        lm->ownG = true;
    } else lm->G = grads_dev;
    cudaMemsetAsync(lm->G, 0, sizeof(float) * (size_t)lm->lay.total, ctx->stream);
    if ((e = cudaMalloc((void**)&lm->block, sizeof(float) * floats + sizeof(int32_t) * ints)) != cudaSuccess)
        return cleanup(fail(ctx, B200_ERR_CUDA, "activation cache allocation of %.2f GiB failed: %s",
                            (sizeof(float) * floats + sizeof(int32_t) * ints) / 1073741824.0, cudaGetErrorString(e)));
    float* q = (float*)lm->block;
    auto take = [&](size_t n) { float* r = q; q += rnd(n); return r; };
    lm->cache.resize(Lc);
    for (auto& k : lm->cache) {
        k.x = take(N * d); k.qkv = take(N * 3 * d); k.attnO = take(N * d); k.rowMax = take(N * H); k.rowSum = take(N * H);
        k.ln1In = take(N * d); k.mean1 = take(N); k.var1 = take(N); k.n1 = take(N * d); k.z1 = take(N * f); k.a1 = take(N * f);
        k.ln2In = take(N * d); k.mean2 = take(N); k.var2 = take(N);
    }
    lm->xFinal = take(N * d); lm->logits = take(N * O); lm->proj = take(N * d);
    for (int i = 0; i < 4; i++) lm->gbuf[i] = take(N * d);
    lm->dqkv = take(N * 3 * d); lm->d1 = take(N * f); lm->rowDot = take(N * H);
    lm->own.contIn = take(N * std::max<size_t>(F, 1)); lm->own.regTgt = take(N * O); lm->own.rowScale = take(N); lm->rowLoss = take(N);
    lm->stepOut = take(64);
    int32_t* qi = (int32_t*)q;
    auto takei = [&](size_t n) { int32_t* r = qi; qi += rnd(n); return r; };
    lm->rowOk = takei(N); lm->own.ids = takei(N); lm->own.targets = takei(N); lm->own.pos = takei(N); lm->own.segId = takei(N); lm->own.segOff = takei(N + 1);
    lm->own.perm = takei(N);
    lm->own.segs = (AttnSeg*)takei(4 * (size_t)lm->maxSeqs);
    size_t hInts = 3 * N + 4 * (size_t)lm->maxSeqs + 3 * N + 8;
    size_t hFloats = N + N * F + N * O + 8;
    if (cudaMallocHost((void**)&lm->h_int, sizeof(int32_t) * hInts) != cudaSuccess || cudaMallocHost((void**)&lm->h_float, sizeof(float) * hFloats) != cudaSuccess)
        return cleanup(fail(ctx, B200_ERR_CUDA, "pinned staging allocation failed"));
    lm->n_ranges = c.num_layers + 2;
    if (cudaMalloc((void**)&lm->sumsq_partials, sizeof(float) * (size_t)lm->n_ranges * SUMSQ_BLOCKS) != cudaSuccess ||
        cudaStreamCreateWithFlags(&lm->norm_stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&lm->norm_event, cudaEventDisableTiming) != cudaSuccess)
        return cleanup(fail(ctx, B200_ERR_CUDA, "could not set up the gradient-norm side stream"));
    cudaMemsetAsync(lm->sumsq_partials, 0, sizeof(float) * (size_t)lm->n_ranges * SUMSQ_BLOCKS, ctx->stream);
    int rc = rope_table(ctx, c.embedding_dim / c.num_heads, 10000.0f, max_rows, &lm->rope);
    if (rc != B200_OK) return cleanup(rc);
    *out = lm;
    return B200_OK;
}

int32_t b200_lm_destroy(b200_lm* lm) {
    if (!lm || lm->refs.fetch_sub(1) != 1) return B200_OK;  // a generation session still reads the weights: it frees them
    cudaSetDevice(lm->ctx->device);
    cudaStreamSynchronize(lm->ctx->stream);
    if (lm->ownP && lm->P) cudaFree(lm->P);
    if (lm->ownG && lm->G) cudaFree(lm->G);
    if (lm->M) cudaFree(lm->M);
    if (lm->V) cudaFree(lm->V);
    if (lm->block) cudaFree(lm->block);
    if (lm->h_int) cudaFreeHost(lm->h_int);
    if (lm->h_float) cudaFreeHost(lm->h_float);
    if (lm->norm_stream) { cudaStreamSynchronize(lm->norm_stream); cudaStreamDestroy(lm->norm_stream); }
    if (lm->norm_event) cudaEventDestroy(lm->norm_event);
    if (lm->sumsq_partials) cudaFree(lm->sumsq_partials);
    for (cudaEvent_t e : lm->cb_events) cudaEventDestroy(e);
    for (cudaEvent_t e : lm->t_events) cudaEventDestroy(e);
    b200_ctx* ctx = lm->ctx;
    delete lm;
    ctx_release(ctx);
    return B200_OK;
}

static int lm_copy(b200_lm* lm, float* host, const float* chost, float* dev, int64_t offset, int64_t count, bool up) {
    if (!lm) return B200_ERR_INVALID_ARG;
    b200_ctx* ctx = lm->ctx;
    if ((!host && !chost) || offset < 0 || count < 0 || offset + count > lm->lay.total)
        return fail(ctx, B200_ERR_OUT_OF_RANGE, "arena range [%lld,%lld) outside [0,%lld)", (long long)offset, (long long)(offset + count), (long long)lm->lay.total);
    std::lock_guard<std::mutex> lock(ctx->mu);
    B200_CUDA(ctx, cudaSetDevice(ctx->device));
    if (up) B200_CUDA(ctx, cudaMemcpyAsync(dev + offset, chost, sizeof(float) * (size_t)count, cudaMemcpyHostToDevice, ctx->stream));
    else B200_CUDA(ctx, cudaMemcpyAsync(host, dev + offset, sizeof(float) * (size_t)count, cudaMemcpyDeviceToHost, ctx->stream));
    B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return B200_OK;
}
int32_t b200_lm_upload_params(b200_lm* lm, const float* host, int64_t offset, int64_t count) { return lm_copy(lm, nullptr, host, lm ? lm->P : nullptr, offset, count, true); }
int32_t b200_lm_download_params(b200_lm* lm, float* host, int64_t offset, int64_t count) { return lm_copy(lm, host, nullptr, lm ? lm->P : nullptr, offset, count, false); }
static int settle_locked(b200_lm* lm) {
    std::lock_guard<std::mutex> lock(lm->ctx->mu);
    B200_CUDA(lm->ctx, cudaSetDevice(lm->ctx->device));
    return settle_grads(lm);
}
int32_t b200_lm_download_grads(b200_lm* lm, float* host, int64_t offset, int64_t count) {
    if (!lm) return B200_ERR_INVALID_ARG;
    B200_TRY(settle_locked(lm));
    return lm_copy(lm, host, nullptr, lm->G, offset, count, false);
}
float* b200_lm_params_device(b200_lm* lm) { return lm ? lm->P : nullptr; }
float* b200_lm_grads_device(b200_lm* lm) {
    if (!lm) return nullptr;
    if (lm->g_pending != 1.f && settle_locked(lm) != B200_OK) return nullptr;  // enqueued on the context's stream, like every other write to the arena
    return lm->G;
}

int32_t b200_lm_set_optimizer(b200_lm* lm, int32_t kind, float beta1, float beta2, float eps) {
    if (!lm) return B200_ERR_INVALID_ARG;
    if (kind != B200_OPT_SGD && kind != B200_OPT_ADAM) return lm_fail(lm, B200_ERR_INVALID_ARG, "unknown optimizer");
    lm->opt = kind;
    if (kind == B200_OPT_ADAM) {
        if (!(beta1 >= 0.f && beta1 < 1.f && beta2 >= 0.f && beta2 < 1.f && eps > 0.f)) return lm_fail(lm, B200_ERR_INVALID_ARG, "bad Adam hyper-parameters");
        lm->beta1 = beta1; lm->beta2 = beta2; lm->adam_eps = eps;
    }
    return B200_OK;
}

int32_t b200_lm_set_grad_ready_callback(b200_lm* lm, b200_grad_ready_fn fn, void* user) {
    if (!lm) return B200_ERR_INVALID_ARG;
    lm->cb = fn;
    lm->cb_user = user;
    return B200_OK;
}

int32_t b200_lm_zero_grads(b200_lm* lm) { return lm ? zero_grads(lm) : B200_ERR_INVALID_ARG; }

int32_t b200_lm_accumulate_discrete(b200_lm* lm, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq, float* loss_sum, int32_t* valid_count) {
    if (!lm) return B200_ERR_INVALID_ARG;
    if (!lm->cfg.discrete) return lm_fail(lm, B200_ERR_INVALID_ARG, "model takes continuous inputs");
    if (!tokens || !seq_offsets || !loss_sum || !valid_count || n_seq < 0) return lm_fail(lm, B200_ERR_INVALID_ARG, "null batch argument");
    Batch b;
    b.tokens = tokens; b.off = seq_offsets;
    return accumulate(lm, b, n_seq, loss_sum, valid_count);
}

int32_t b200_lm_accumulate_continuous(b200_lm* lm, const float* features, const float* reg_targets, const int32_t* class_targets,
                                      const int32_t* seq_offsets, int32_t n_seq, float* loss_sum, int32_t* valid_count) {
    if (!lm) return B200_ERR_INVALID_ARG;
    if (lm->cfg.discrete) return lm_fail(lm, B200_ERR_INVALID_ARG, "model takes token ids");
    if (!features || !seq_offsets || !loss_sum || !valid_count || n_seq < 0) return lm_fail(lm, B200_ERR_INVALID_ARG, "null batch argument");
    if (lm->cfg.loss_kind == 1 ? !reg_targets : !class_targets) return lm_fail(lm, B200_ERR_INVALID_ARG, "targets missing for the configured loss");
    Batch b;
    b.feats = features; b.regT = reg_targets; b.clsT = class_targets; b.off = seq_offsets;
    return accumulate(lm, b, n_seq, loss_sum, valid_count);
}

int32_t b200_lm_validate_discrete(b200_lm* lm, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq, float* mean_loss, int32_t* items) {
    if (!lm) return B200_ERR_INVALID_ARG;
    if (!lm->cfg.discrete) return lm_fail(lm, B200_ERR_INVALID_ARG, "model takes continuous inputs");
    if (!tokens || !seq_offsets || !mean_loss || !items || n_seq < 0) return lm_fail(lm, B200_ERR_INVALID_ARG, "null batch argument");
    Batch b;
    b.tokens = tokens; b.off = seq_offsets;
    return validate(lm, b, n_seq, mean_loss, items);
}

int32_t b200_lm_validate_continuous(b200_lm* lm, const float* features, const float* reg_targets, const int32_t* class_targets,
                                    const int32_t* seq_offsets, int32_t n_seq, float* mean_loss, int32_t* items) {
    if (!lm) return B200_ERR_INVALID_ARG;
    if (lm->cfg.discrete) return lm_fail(lm, B200_ERR_INVALID_ARG, "model takes token ids");
    if (!features || !seq_offsets || !mean_loss || !items || n_seq < 0) return lm_fail(lm, B200_ERR_INVALID_ARG, "null batch argument");
    if (lm->cfg.loss_kind == 1 ? !reg_targets : !class_targets) return lm_fail(lm, B200_ERR_INVALID_ARG, "targets missing for the configured loss");
    Batch b;
    b.feats = features; b.regT = reg_targets; b.clsT = class_targets; b.off = seq_offsets;
    return validate(lm, b, n_seq, mean_loss, items);
}

// Optimiser state for checkpoints: kind 0 = first moments, 1 = second moments (same layout as the parameter arena).
static int32_t opt_state_copy(b200_lm* lm, int32_t which, float* host_out, const float* host_in, int64_t offset, int64_t count, bool upload) {
    if (!lm) return B200_ERR_INVALID_ARG;
    if (which != 0 && which != 1) return lm_fail(lm, B200_ERR_INVALID_ARG, "optimizer state index must be 0 (first moments) or 1 (second moments)");
    if (lm->opt != B200_OPT_ADAM) return lm_fail(lm, B200_ERR_INVALID_ARG, "the configured optimizer keeps no state");
    b200_ctx* ctx = lm->ctx;
    {
        std::lock_guard<std::mutex> lock(ctx->mu);
        B200_CUDA(ctx, cudaSetDevice(ctx->device));
        if (!lm->M) {  // not stepped yet: the moments are zero
            B200_CUDA(ctx, cudaMalloc(&lm->M, sizeof(float) * (size_t)lm->lay.total));
            B200_CUDA(ctx, cudaMalloc(&lm->V, sizeof(float) * (size_t)lm->lay.total));
            B200_CUDA(ctx, cudaMemsetAsync(lm->M, 0, sizeof(float) * (size_t)lm->lay.total, ctx->stream));
            B200_CUDA(ctx, cudaMemsetAsync(lm->V, 0, sizeof(float) * (size_t)lm->lay.total, ctx->stream));
        }
    }
    return lm_copy(lm, host_out, host_in, which == 0 ? lm->M : lm->V, offset, count, upload);
}
int32_t b200_lm_download_optimizer_state(b200_lm* lm, int32_t which, float* host, int64_t offset, int64_t count) {
    return opt_state_copy(lm, which, host, nullptr, offset, count, false);
}
int32_t b200_lm_upload_optimizer_state(b200_lm* lm, int32_t which, const float* host, int64_t offset, int64_t count) {
    return opt_state_copy(lm, which, nullptr, host, offset, count, true);
}
int32_t b200_lm_get_step_index(b200_lm* lm, int32_t* step_index) {
    if (!lm || !step_index) return B200_ERR_INVALID_ARG;
    *step_index = lm->step_index;
    return B200_OK;
}
int32_t b200_lm_set_step_index(b200_lm* lm, int32_t step_index) {
    if (!lm) return B200_ERR_INVALID_ARG;
    if (step_index < 0) return lm_fail(lm, B200_ERR_INVALID_ARG, "step index must not be negative");
    lm->step_index = step_index;
    return B200_OK;
}

int32_t b200_lm_apply_step(b200_lm* lm, int32_t global_valid_count, float lr, int32_t use_clip, float clip_threshold, int32_t do_step, float* grad_norm) {
    if (!lm) return B200_ERR_INVALID_ARG;
    return apply_step(lm, global_valid_count, lr, use_clip, clip_threshold, do_step, grad_norm);
}

int32_t b200_lm_train_step_discrete(b200_lm* lm, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq, float lr, int32_t use_clip,
                                    float clip_threshold, int32_t do_step, float* loss, float* grad_norm, int32_t* valid_count) {
    if (!lm) return B200_ERR_INVALID_ARG;
    float ls = 0.f, gn = 0.f;
    int32_t vc = 0;
    B200_TRY(b200_lm_zero_grads(lm));
    B200_TRY(b200_lm_accumulate_discrete(lm, tokens, seq_offsets, n_seq, &ls, &vc));
    B200_TRY(b200_lm_apply_step(lm, vc, lr, use_clip, clip_threshold, do_step, &gn));
    if (loss) *loss = vc > 0 ? ls / (float)vc : 0.f;
    if (grad_norm) *grad_norm = gn;
    if (valid_count) *valid_count = vc;
    return B200_OK;
}

int32_t b200_lm_train_step_continuous(b200_lm* lm, const float* features, const float* reg_targets, const int32_t* class_targets,
                                      const int32_t* seq_offsets, int32_t n_seq, float lr, int32_t use_clip, float clip_threshold, int32_t do_step,
                                      float* loss, float* grad_norm, int32_t* valid_count) {
    if (!lm) return B200_ERR_INVALID_ARG;
    float ls = 0.f, gn = 0.f;
    int32_t vc = 0;
    B200_TRY(b200_lm_zero_grads(lm));
    B200_TRY(b200_lm_accumulate_continuous(lm, features, reg_targets, class_targets, seq_offsets, n_seq, &ls, &vc));
    B200_TRY(b200_lm_apply_step(lm, vc, lr, use_clip, clip_threshold, do_step, &gn));
    if (loss) *loss = vc > 0 ? ls / (float)vc : 0.f;
    if (grad_norm) *grad_norm = gn;
    if (valid_count) *valid_count = vc;
    return B200_OK;
}

static int batch_finish(b200_lm* lm, b200_lm_batch* bt, b200_lm_batch** out) {
    b200_ctx* ctx = lm->ctx;
    const b200_lm_config& c = lm->cfg;
    std::lock_guard<std::mutex> lock(ctx->mu);
    B200_CUDA(ctx, cudaSetDevice(ctx->device));
    Batch hb;
    hb.tokens = bt->tokens.data(); hb.feats = bt->feats.data(); hb.regT = bt->regT.data(); hb.clsT = bt->clsT.data(); hb.off = bt->off.data();
    Plan* plan = new Plan();
    bt->plan = plan;
    int rc = plan_batch(lm, hb, bt->n_seq, *plan);
    if (rc != B200_OK) return rc;
    auto rnd = [](size_t n) { return (n + 63) & ~(size_t)63; };
    const size_t F = (size_t)c.input_feature_dim, O = (size_t)c.output_dim;
    size_t words = 64;
    for (const Pass& p : plan->passes) {
        size_t N = (size_t)p.rows, S = p.seqs.size();
        words += rnd(N) * 6 + rnd(N + 1) + rnd(4 * S) + rnd(N * std::max<size_t>(F, 1)) + rnd(N * O);
    }
    if (!plan->passes.empty()) {
        cudaError_t e = cudaMalloc((void**)&bt->block, words * 4);
        if (e != cudaSuccess) return fail(ctx, B200_ERR_CUDA, "prepared batch allocation of %zu bytes failed: %s", words * 4, cudaGetErrorString(e));
    }
    int32_t* q = (int32_t*)bt->block;
    auto take = [&](size_t n) { int32_t* r = q; q += rnd(n); return r; };
    for (const Pass& p : plan->passes) {
        size_t N = (size_t)p.rows, S = p.seqs.size();
        PassDev d;
        d.ids = take(N); d.targets = take(N); d.pos = take(N); d.segId = take(N); d.segOff = take(N + 1); d.perm = take(N);
        d.segs = (AttnSeg*)take(4 * S);
        d.rowScale = (float*)take(N); d.contIn = (float*)take(N * std::max<size_t>(F, 1)); d.regTgt = (float*)take(N * O);
        rc = stage_pass(lm, hb, p, d);
        if (rc != B200_OK) return rc;
        B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // the pinned staging area is reused by the next pass
        bt->dev.push_back(d);
    }
    *out = bt;
    return B200_OK;
}

int32_t b200_lm_batch_create_discrete(b200_lm* lm, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq, b200_lm_batch** out) {
    if (!lm || !out) return B200_ERR_INVALID_ARG;
    *out = nullptr;
    if (!lm->cfg.discrete) return lm_fail(lm, B200_ERR_INVALID_ARG, "model takes continuous inputs");
    if (!tokens || !seq_offsets || n_seq < 0) return lm_fail(lm, B200_ERR_INVALID_ARG, "null batch argument");
    b200_lm_batch* bt = new b200_lm_batch();
    bt->lm = lm; bt->n_seq = n_seq;
    bt->off.assign(seq_offsets, seq_offsets + n_seq + 1);
    bt->tokens.assign(tokens, tokens + seq_offsets[n_seq]);
    int rc = batch_finish(lm, bt, out);
    if (rc != B200_OK) b200_lm_batch_destroy(bt);
    return rc;
}

int32_t b200_lm_batch_create_continuous(b200_lm* lm, const float* features, const float* reg_targets, const int32_t* class_targets,
                                        const int32_t* seq_offsets, int32_t n_seq, b200_lm_batch** out) {
    if (!lm || !out) return B200_ERR_INVALID_ARG;
    *out = nullptr;
    if (lm->cfg.discrete) return lm_fail(lm, B200_ERR_INVALID_ARG, "model takes token ids");
    if (!features || !seq_offsets || n_seq < 0) return lm_fail(lm, B200_ERR_INVALID_ARG, "null batch argument");
    if (lm->cfg.loss_kind == 1 ? !reg_targets : !class_targets) return lm_fail(lm, B200_ERR_INVALID_ARG, "targets missing for the configured loss");
    b200_lm_batch* bt = new b200_lm_batch();
    bt->lm = lm; bt->n_seq = n_seq;
    bt->off.assign(seq_offsets, seq_offsets + n_seq + 1);
    size_t rows = (size_t)seq_offsets[n_seq];
    bt->feats.assign(features, features + rows * lm->cfg.input_feature_dim);
    if (reg_targets && lm->cfg.loss_kind == 1) bt->regT.assign(reg_targets, reg_targets + rows * lm->cfg.output_dim);
    if (class_targets && lm->cfg.loss_kind == 0) bt->clsT.assign(class_targets, class_targets + rows);
    int rc = batch_finish(lm, bt, out);
    if (rc != B200_OK) b200_lm_batch_destroy(bt);
    return rc;
}

int32_t b200_lm_batch_destroy(b200_lm_batch* bt) {
    if (!bt) return B200_OK;
    if (bt->lm) {
        cudaSetDevice(bt->lm->ctx->device);
        cudaStreamSynchronize(bt->lm->ctx->stream);
    }
    if (bt->block) cudaFree(bt->block);
    delete (Plan*)bt->plan;
    delete bt;
    return B200_OK;
}

int32_t b200_lm_accumulate_batch(b200_lm* lm, b200_lm_batch* bt, float* loss_sum, int32_t* valid_count) {
    if (!lm || !bt || bt->lm != lm || !loss_sum || !valid_count) return B200_ERR_INVALID_ARG;
    b200_ctx* ctx = lm->ctx;
    std::lock_guard<std::mutex> lock(ctx->mu);
    B200_CUDA(ctx, cudaSetDevice(ctx->device));
    Batch hb;
    hb.tokens = bt->tokens.data(); hb.feats = bt->feats.data(); hb.regT = bt->regT.data(); hb.clsT = bt->clsT.data(); hb.off = bt->off.data();
    return run_plan(lm, hb, *(Plan*)bt->plan, &bt->dev, loss_sum, valid_count);
}

int32_t b200_lm_train_step_batch(b200_lm* lm, b200_lm_batch* bt, float lr, int32_t use_clip, float clip_threshold, int32_t do_step, float* loss,
                                 float* grad_norm, int32_t* valid_count) {
    if (!lm) return B200_ERR_INVALID_ARG;
    float ls = 0.f, gn = 0.f;
    int32_t vc = 0;
    B200_TRY(b200_lm_zero_grads(lm));
    B200_TRY(b200_lm_accumulate_batch(lm, bt, &ls, &vc));
    B200_TRY(b200_lm_apply_step(lm, vc, lr, use_clip, clip_threshold, do_step, &gn));
    if (loss) *loss = vc > 0 ? ls / (float)vc : 0.f;
    if (grad_norm) *grad_norm = gn;
    if (valid_count) *valid_count = vc;
    return B200_OK;
}

int32_t b200_lm_get_timings(b200_lm* lm, float* ms4) {
    if (!lm || !ms4) return B200_ERR_INVALID_ARG;
    for (int i = 0; i < 4; i++) ms4[i] = lm->timings[i];
    return B200_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------ incremental decoding
// LanguageModel.Generate's decoder path (LanguageModel.cs:270-537) with the key/value cache in device memory: every
// token is pushed through the blocks at its absolute position (ForwardDecoderTokenFromId), its rotated K and its V rows
// are appended to the per-layer cache, attention runs over the cached rows (all in the past, so no mask), and
// ProjectLastTokenOnly gives the next-token logits.  Sampling stays with the caller (the reference draws from its own
// System.Random); b200_lm_gen_greedy is the arg-max special case that never leaves the device.
struct b200_lm_gen {
    b200_lm* lm = nullptr;
    int maxLen = 0, len = 0;
    char* block = nullptr;
    float *K = nullptr, *V = nullptr;  // [layers][maxLen][d]
    float *x = nullptr, *xn = nullptr, *qkv = nullptr, *attnO = nullptr, *proj = nullptr, *proj2 = nullptr, *n1 = nullptr, *z1 = nullptr, *a1 = nullptr,
          *lnIn = nullptr, *stat = nullptr, *logits = nullptr;
    int32_t* tokens = nullptr;  // device: token ids by position
    int32_t* d_pos = nullptr;   // device: position of the token the next forward processes (always equal to len)
    const float* rope = nullptr;
    // The launch sequence of one token has no host-dependent argument (the position is read from d_pos), so it is
    // captured once into a CUDA graph: the first token runs eagerly (first-use set-up), the second is captured.
    int forwards = 0;
    bool graph_failed = false;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t graph_exec = nullptr;
    // Preferred path: the whole token as one cooperative kernel (k_decode_token); the graph of separate launches above
    // serves arenas it cannot take (unaligned tensors, Q/K/V weights not back to back) or devices without cooperative launch.
    DecodeLayer* dec_layers = nullptr;  // device array, one entry per block
    int coop_blocks = 0;                // 0 not tried yet, -1 unavailable, else the grid size
    int use_single_kernel = 1;
};

namespace {

// The same sequence with the general-purpose kernels (one launch per LayerNorm and per product): arenas whose tensors
// are not 16-byte aligned, or widths that are not multiples of 4.
int gen_forward_plain(b200_lm_gen* g) {
    b200_lm* lm = g->lm;
    b200_ctx* ctx = lm->ctx;
    const b200_lm_config& c = lm->cfg;
    const int d = c.embedding_dim, H = c.num_heads, hd = d / H, f = c.ffn_dim, O = c.output_dim;
    const float* P = lm->P;
    B200_TRY(k_decode_embed(ctx, g->tokens, g->d_pos, P + lm->lay.in0, d, g->x));
    for (int l = 0; l < c.num_layers; l++) {
        const LayerOff& L = lm->lay.layer[(size_t)l];
        float* Kc = g->K + (size_t)l * g->maxLen * d;
        float* Vc = g->V + (size_t)l * g->maxLen * d;
        if (qkv_fused(lm, L)) {
            B200_TRY(linear_fwd(ctx, g->x, 1, d, P + L.WQ, P + L.bQ, 3 * d, g->qkv, 3 * d));
        } else {
            const int64_t Ws[3] = {L.WQ, L.WK, L.WV}, Bs[3] = {L.bQ, L.bK, L.bV};
            for (int i = 0; i < 3; i++) B200_TRY(linear_fwd(ctx, g->x, 1, d, P + Ws[i], P + Bs[i], d, g->qkv + i * d, d));
        }
        B200_TRY(k_decode_rope_scatter(ctx, g->qkv, g->d_pos, g->rope, d, hd, Kc, Vc));
        B200_TRY(k_decode_attn(ctx, g->qkv, Kc, Vc, g->d_pos, H, hd, 1.0f / sqrtf((float)hd), g->attnO));
        B200_TRY(linear_fwd(ctx, g->attnO, 1, d, P + L.WO, P + L.bO, d, g->proj, d));
        B200_TRY(k_ln_forward(ctx, g->x, g->proj, P + L.g1, P + L.b1n, 1, d, 1e-5f, g->n1, g->stat, g->stat + 1, nullptr, g->lnIn));
        {
            Gemm gm;
            gm.M = 1; gm.N = f; gm.K = d; gm.A = g->n1; gm.lda = d; gm.B = P + L.W1; gm.ldb = d; gm.transB = 1;
            gm.C = g->a1; gm.ldc = f; gm.bias = P + L.fb1; gm.zout = g->z1; gm.ldz = f; gm.act = c.ffn_activation;
            B200_TRY(gemm(ctx, gm));
        }
        B200_TRY(linear_fwd(ctx, g->a1, 1, f, P + L.W2, P + L.fb2, d, g->proj, d));
        B200_TRY(k_ln_forward(ctx, g->n1, g->proj, P + L.g2, P + L.b2n, 1, d, 1e-5f, g->x, g->stat, g->stat + 1, nullptr, g->lnIn));
    }
    return linear_fwd(ctx, g->x, 1, d, P + lm->lay.Wout, P + lm->lay.bout, O, g->logits, O);
}

// One token through the model: the token at position *d_pos (id read from gen->tokens on the device); its rotated key
// and its value go into row *d_pos of every layer's cache; logits land in gen->logits.  Six launches per layer: the two
// LayerNorms ride in the prologue of the product that consumes them (k_decode_gemv).
int gen_forward(b200_lm_gen* g) {
    b200_lm* lm = g->lm;
    b200_ctx* ctx = lm->ctx;
    const b200_lm_config& c = lm->cfg;
    const int d = c.embedding_dim, H = c.num_heads, hd = d / H, f = c.ffn_dim, O = c.output_dim, Lc = c.num_layers;
    const float* P = lm->P;
    const bool fast = d % 4 == 0 && f % 4 == 0 && c.align_floats % 4 == 0 && d <= 12288 && f <= 12288 && (((uintptr_t)P) & 15) == 0;
    if (!fast) return gen_forward_plain(g);
    B200_TRY(k_decode_embed(ctx, g->tokens, g->d_pos, P + lm->lay.in0, d, g->x));
    // input of the next product that follows a LayerNorm: LN(res + sub) with these parameters; none before the first layer
    const float *res = nullptr, *sub = nullptr, *gam = nullptr, *bet = nullptr;
    for (int l = 0; l < Lc; l++) {
        const LayerOff& L = lm->lay.layer[(size_t)l];
        float* Kc = g->K + (size_t)l * g->maxLen * d;
        float* Vc = g->V + (size_t)l * g->maxLen * d;
        // x_l = embedding (first layer) or LN2 of the previous block, formed inside the Q/K/V product and stored to g->x
        if (qkv_fused(lm, L)) {
            B200_TRY(k_decode_gemv(ctx, sub ? res : g->x, sub, gam, bet, 1e-5f, g->x, P + L.WQ, P + L.bQ, 3 * d, d, B200_ACT_NONE, g->qkv));
        } else {
            const int64_t Ws[3] = {L.WQ, L.WK, L.WV}, Bs[3] = {L.bQ, L.bK, L.bV};
            for (int i = 0; i < 3; i++)  // the first product stores x_l; the other two recompute it from the same inputs (g->n1, g->proj are still intact)
                B200_TRY(k_decode_gemv(ctx, sub ? res : g->x, sub, gam, bet, 1e-5f, i == 0 ? g->xn : nullptr, P + Ws[i], P + Bs[i], d, d, B200_ACT_NONE, g->qkv + i * d));
            if (sub) B200_CUDA(ctx, cudaMemcpyAsync(g->x, g->xn, sizeof(float) * (size_t)d, cudaMemcpyDeviceToDevice, ctx->stream));
        }
        B200_TRY(k_decode_rope_scatter(ctx, g->qkv, g->d_pos, g->rope, d, hd, Kc, Vc));
        B200_TRY(k_decode_attn(ctx, g->qkv, Kc, Vc, g->d_pos, H, hd, 1.0f / sqrtf((float)hd), g->attnO));
        B200_TRY(k_decode_gemv(ctx, g->attnO, nullptr, nullptr, nullptr, 0.f, nullptr, P + L.WO, P + L.bO, d, d, B200_ACT_NONE, g->proj));
        // n1 = LN1(x_l + attention projection), formed inside the first FFN product and stored to g->n1
        B200_TRY(k_decode_gemv(ctx, g->x, g->proj, P + L.g1, P + L.b1n, 1e-5f, g->n1, P + L.W1, P + L.fb1, f, d, c.ffn_activation, g->a1));
        B200_TRY(k_decode_gemv(ctx, g->a1, nullptr, nullptr, nullptr, 0.f, nullptr, P + L.W2, P + L.fb2, d, f, B200_ACT_NONE, g->proj2));
        res = g->n1; sub = g->proj2; gam = P + L.g2; bet = P + L.b2n;  // LN2(n1 + FFN output) is formed by whoever consumes it
    }
    return k_decode_gemv(ctx, sub ? res : g->x, sub, gam, bet, 1e-5f, nullptr, P + lm->lay.Wout, P + lm->lay.bout, O, d, B200_ACT_NONE, g->logits);
}

// One token, position advanced, next token picked when asked: a single cooperative launch when possible.
int gen_run(b200_lm_gen* g);
int gen_token(b200_lm_gen* g, int pick) {
    b200_lm* lm = g->lm;
    b200_ctx* ctx = lm->ctx;
    const b200_lm_config& c = lm->cfg;
    if (g->dec_layers && g->use_single_kernel && g->coop_blocks >= 0) {
        DecodeArgs a;
        a.layers = g->dec_layers; a.L = c.num_layers; a.d = c.embedding_dim; a.f = c.ffn_dim; a.H = c.num_heads; a.hd = c.embedding_dim / c.num_heads;
        a.V = c.output_dim; a.act = c.ffn_activation; a.pick = pick; a.scale = 1.0f / sqrtf((float)a.hd);
        a.emb = lm->P + lm->lay.in0; a.Wout = lm->P + lm->lay.Wout; a.bout = lm->P + lm->lay.bout; a.rope = g->rope;
        a.tokens = g->tokens; a.pos = g->d_pos;
        a.x = g->x; a.qkv = g->qkv; a.attnO = g->attnO; a.proj = g->proj; a.proj2 = g->proj2; a.n1 = g->n1; a.a1 = g->a1; a.logits = g->logits;
        const int rc = k_decode_token(ctx, a, &g->coop_blocks);
        if (rc != B200_ERR_UNSUPPORTED) return rc;
    }
    B200_TRY(gen_run(g));
    return k_decode_advance(ctx, g->logits, c.output_dim, g->tokens, g->d_pos, pick);
}

// The same through the captured graph once it exists.  Anything that prevents the capture (a legacy default stream, a
// driver that refuses) leaves the session on plain launches of the very same kernels.
int gen_run(b200_lm_gen* g) {
    b200_ctx* ctx = g->lm->ctx;
    g->forwards++;
    if (g->graph_exec) {
        B200_CUDA(ctx, cudaGraphLaunch(g->graph_exec, ctx->stream));
        ctx->launches++;
        return B200_OK;
    }
    if (g->forwards < 2 || g->graph_failed || ctx->stream == nullptr) return gen_forward(g);
    const int profile = ctx->profile;
    ctx->profile = 0;  // no event pairs inside a capture
    int rc = B200_OK;
    if (cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
        (void)cudaGetLastError();
        g->graph_failed = true;
        ctx->profile = profile;
        return gen_forward(g);
    }
    rc = gen_forward(g);
    cudaGraph_t graph = nullptr;
    const cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
    ctx->profile = profile;
    if (rc != B200_OK || e != cudaSuccess || !graph || cudaGraphInstantiate(&g->graph_exec, graph, 0) != cudaSuccess) {
        (void)cudaGetLastError();
        if (graph) cudaGraphDestroy(graph);
        g->graph_exec = nullptr;
        g->graph_failed = true;
        return rc != B200_OK ? rc : gen_forward(g);  // nothing ran during the capture: do the work now
    }
    g->graph = graph;
    B200_CUDA(ctx, cudaGraphLaunch(g->graph_exec, ctx->stream));
    ctx->launches++;
    return B200_OK;
}

}  // namespace

extern "C" {

int32_t b200_lm_gen_create(b200_lm* lm, int32_t max_len, b200_lm_gen** out) {
    if (!lm || !out) return B200_ERR_INVALID_ARG;
    *out = nullptr;
    b200_ctx* ctx = lm->ctx;
    const b200_lm_config& c = lm->cfg;
    if (!c.discrete) return lm_fail(lm, B200_ERR_UNSUPPORTED, "Generate is only supported for discrete token data types.");
    if (max_len <= 0) return lm_fail(lm, B200_ERR_INVALID_ARG, "max_len must be positive");
    std::lock_guard<std::mutex> lock(ctx->mu);
    B200_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t d = (size_t)c.embedding_dim, f = (size_t)c.ffn_dim, O = (size_t)c.output_dim, Lc = (size_t)c.num_layers, T = (size_t)max_len;
    auto rnd = [](size_t n) { return (n + 63) & ~(size_t)63; };
    const size_t floats = 2 * rnd(Lc * T * d) + 7 * rnd(d) + rnd(3 * d) + 2 * rnd(f) + rnd(O) + rnd(64);
    const size_t ints = rnd(T + 1) + rnd(1);
    const size_t bytes = floats * 4 + ints * 4;
    b200_lm_gen* g = new b200_lm_gen();
    g->lm = lm; g->maxLen = max_len;
    if (cudaMalloc(&g->block, bytes) != cudaSuccess) {
        delete g;
        return lm_fail(lm, B200_ERR_CUDA, "out of device memory for the key/value cache");
    }
    char* cur = g->block;
    auto takef = [&](size_t n) { float* r = reinterpret_cast<float*>(cur); cur += rnd(n) * 4; return r; };
    g->K = takef(Lc * T * d); g->V = takef(Lc * T * d);
    g->x = takef(d); g->xn = takef(d); g->qkv = takef(3 * d); g->attnO = takef(d); g->proj = takef(d); g->proj2 = takef(d); g->n1 = takef(d); g->lnIn = takef(d);
    g->z1 = takef(f); g->a1 = takef(f); g->logits = takef(O); g->stat = takef(64);
    g->tokens = reinterpret_cast<int32_t*>(cur); cur += rnd(T + 1) * 4;
    g->d_pos = reinterpret_cast<int32_t*>(cur); cur += rnd(1) * 4;
    int rc = B200_OK;
    if (cudaMemsetAsync(g->d_pos, 0, sizeof(int32_t), ctx->stream) != cudaSuccess || cudaStreamSynchronize(ctx->stream) != cudaSuccess)
        rc = lm_fail(lm, B200_ERR_CUDA, "could not initialise the generation session");
    if (rc == B200_OK) rc = rope_table(ctx, c.embedding_dim / c.num_heads, 10000.0f, max_len, &g->rope);
    if (rc == B200_OK) {
        bool ok = c.num_layers > 0 && d % 4 == 0 && f % 4 == 0 && c.align_floats % 4 == 0 && d <= 12288 && f <= 12288 && (((uintptr_t)lm->P) & 15) == 0;
        for (int l = 0; l < c.num_layers && ok; l++) ok = qkv_fused(lm, lm->lay.layer[(size_t)l]);
        if (ok) {
            std::vector<DecodeLayer> host((size_t)c.num_layers);
            const float* P = lm->P;
            for (int l = 0; l < c.num_layers; l++) {
                const LayerOff& L = lm->lay.layer[(size_t)l];
                host[(size_t)l] = DecodeLayer{P + L.WQ, P + L.bQ, P + L.WO, P + L.bO, P + L.g1, P + L.b1n, P + L.W1, P + L.fb1, P + L.W2, P + L.fb2,
                                              P + L.g2, P + L.b2n, g->K + (size_t)l * T * d, g->V + (size_t)l * T * d};
            }
            if (cudaMalloc((void**)&g->dec_layers, sizeof(DecodeLayer) * host.size()) != cudaSuccess ||
                cudaMemcpy(g->dec_layers, host.data(), sizeof(DecodeLayer) * host.size(), cudaMemcpyHostToDevice) != cudaSuccess) {
                (void)cudaGetLastError();
                if (g->dec_layers) cudaFree(g->dec_layers);
                g->dec_layers = nullptr;  // the separate-launch path needs no table
            }
        }
    }
    if (rc != B200_OK) { cudaFree(g->block); delete g; return rc; }
    lm->refs.fetch_add(1);
    *out = g;
    return B200_OK;
}

int32_t b200_lm_gen_destroy(b200_lm_gen* g) {
    if (!g) return B200_OK;
    cudaSetDevice(g->lm->ctx->device);
    cudaStreamSynchronize(g->lm->ctx->stream);
    if (g->graph_exec) cudaGraphExecDestroy(g->graph_exec);
    if (g->graph) cudaGraphDestroy(g->graph);
    if (g->dec_layers) cudaFree(g->dec_layers);
    cudaFree(g->block);
    b200_lm* lm = g->lm;
    delete g;
    return b200_lm_destroy(lm);
}

int32_t b200_lm_gen_reset(b200_lm_gen* g) {
    if (!g) return B200_ERR_INVALID_ARG;
    b200_ctx* ctx = g->lm->ctx;
    std::lock_guard<std::mutex> lock(ctx->mu);
    B200_CUDA(ctx, cudaSetDevice(ctx->device));
    B200_CUDA(ctx, cudaMemsetAsync(g->d_pos, 0, sizeof(int32_t), ctx->stream));
    g->len = 0;
    return B200_OK;
}

// Number of kernel launches replayed per token from the captured graph (0: the session issues plain launches, either
// because fewer than two tokens have been processed or because the capture was refused).
int32_t b200_lm_gen_graph_nodes(b200_lm_gen* g, int32_t* nodes) {
    if (!g || !nodes) return B200_ERR_INVALID_ARG;
    *nodes = 0;
    if (g->graph) {
        size_t n = 0;
        if (cudaGraphGetNodes(g->graph, nullptr, &n) == cudaSuccess) *nodes = (int32_t)n;
    }
    return B200_OK;
}

// 1 when the session runs each token as one cooperative kernel, 0 when it issues the phases as separate launches (through
// the captured graph from the second token on).  b200_lm_gen_set_single_kernel(g, 0) selects the latter on purpose.
int32_t b200_lm_gen_single_kernel(b200_lm_gen* g) { return (g && g->dec_layers && g->use_single_kernel && g->coop_blocks >= 0) ? 1 : 0; }
int32_t b200_lm_gen_set_single_kernel(b200_lm_gen* g, int32_t on) {
    if (!g) return B200_ERR_INVALID_ARG;
    g->use_single_kernel = on ? 1 : 0;
    return B200_OK;
}

int32_t b200_lm_gen_length(b200_lm_gen* g, int32_t* len) {
    if (!g || !len) return B200_ERR_INVALID_ARG;
    *len = g->len;
    return B200_OK;
}

// ForwardDecoderTokenFromId at position = current length, then ProjectLastTokenOnly; logits (host, [output_dim]) may be null.
int32_t b200_lm_gen_step(b200_lm_gen* g, int32_t token_id, float* logits) {
    if (!g) return B200_ERR_INVALID_ARG;
    b200_lm* lm = g->lm;
    b200_ctx* ctx = lm->ctx;
    if ((uint32_t)token_id >= (uint32_t)lm->cfg.vocab_size) return fail(ctx, B200_ERR_OUT_OF_RANGE, "token id %d outside the vocabulary", token_id);
    if (g->len >= g->maxLen) return lm_fail(lm, B200_ERR_OUT_OF_RANGE, "Decoder KV cache is full.");
    std::lock_guard<std::mutex> lock(ctx->mu);
    B200_CUDA(ctx, cudaSetDevice(ctx->device));
    B200_CUDA(ctx, cudaMemcpyAsync(g->tokens + g->len, &token_id, 4, cudaMemcpyHostToDevice, ctx->stream));
    B200_TRY(gen_token(g, 0));
    g->len++;
    if (logits) B200_CUDA(ctx, cudaMemcpyAsync(logits, g->logits, sizeof(float) * (size_t)lm->cfg.output_dim, cudaMemcpyDeviceToHost, ctx->stream));
    B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return check_device_status(ctx);
}

// Prompt then arg-max continuation, all launches enqueued without a host round trip per token.  out_tokens receives the
// prompt followed by the generated ids (at most n_prompt + max_new, never beyond the cache); *n_out their number.
int32_t b200_lm_gen_greedy(b200_lm_gen* g, const int32_t* prompt, int32_t n_prompt, int32_t max_new, int32_t* out_tokens, int32_t* n_out) {
    if (!g || !prompt || !out_tokens || !n_out || n_prompt <= 0 || max_new < 0) return B200_ERR_INVALID_ARG;
    b200_lm* lm = g->lm;
    b200_ctx* ctx = lm->ctx;
    for (int i = 0; i < n_prompt; i++)
        if ((uint32_t)prompt[i] >= (uint32_t)lm->cfg.vocab_size) return fail(ctx, B200_ERR_OUT_OF_RANGE, "token id %d outside the vocabulary", prompt[i]);
    if (n_prompt > g->maxLen) return lm_fail(lm, B200_ERR_OUT_OF_RANGE, "prompt longer than the key/value cache");
    std::lock_guard<std::mutex> lock(ctx->mu);
    B200_CUDA(ctx, cudaSetDevice(ctx->device));
    g->len = 0;
    B200_CUDA(ctx, cudaMemsetAsync(g->d_pos, 0, sizeof(int32_t), ctx->stream));
    B200_CUDA(ctx, cudaMemcpyAsync(g->tokens, prompt, 4 * (size_t)n_prompt, cudaMemcpyHostToDevice, ctx->stream));
    int total = n_prompt;
    for (int pos = 0; pos < n_prompt; pos++) {  // LanguageModel.cs:517-520: the prompt token by token
        // after the last prompt token the first new token is chosen (it lands in tokens[n_prompt]); every token moves d_pos on
        B200_TRY(gen_token(g, (pos == n_prompt - 1 && max_new > 0 && total < g->maxLen) ? 1 : 0));
    }
    g->len = n_prompt;
    for (int gen = 0; gen < max_new && total < g->maxLen; gen++) {  // LanguageModel.cs:522-535 with arg-max in place of sampling
        total++;  // the token chosen by the previous advance
        if (total < g->maxLen && gen + 1 < max_new) {
            B200_TRY(gen_token(g, 1));
            g->len = total;
        }
    }
    B200_CUDA(ctx, cudaMemcpyAsync(out_tokens, g->tokens, 4 * (size_t)total, cudaMemcpyDeviceToHost, ctx->stream));
    B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    *n_out = total;
    return check_device_status(ctx);
}

}  // extern "C"
