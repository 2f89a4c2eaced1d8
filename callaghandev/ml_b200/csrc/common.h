// Shared host-side definitions of libcallaghan_b200: the context object, status helpers and the launcher
// prototypes of every kernel family.  All launchers take DEVICE pointers and enqueue on ctx->stream.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <map>
#include <set>
#include <mutex>
#include <atomic>
#include <string>
#include <vector>

#include "../../../include/callaghan_b200.h"

struct RopeTable {
    float* dev = nullptr;  // [rows][headDim/2][2] = (cos, sin), computed on the host with the oracle's libm calls
    int rows = 0;
};

struct b200_ctx {
    // The context outlives every trainer / session created on it, whatever order the caller destroys them in
    // (finalizers of a garbage-collected host language run in no particular order): each child holds one reference
    // and b200_destroy only drops the owner's.
    std::atomic<int> refs{1};
    int device = 0;
    cudaStream_t stream = nullptr;
    cudaStream_t own_stream = nullptr;
    std::string err;
    std::mutex mu;
    int gemm_mode = B200_GEMM_AUTO;
    int cc_major = 0, sm_count = 0;
    int64_t launches = 0;
    // grow-only scratch for the per-op (host pointer) API
    char* pool = nullptr;
    size_t pool_bytes = 0, pool_used = 0;
    // small grow-only device workspace for reductions / split-K partials owned by kernels
    float* ws = nullptr;
    size_t ws_floats = 0;
    float* pinned = nullptr;  // 4 KiB pinned staging for scalars
    std::map<std::pair<int, uint32_t>, RopeTable> rope;  // key: (headDim, bits of baseTheta)
    std::vector<float*> rope_retired;  // smaller tables replaced by larger ones: trainers may still point at them, freed with the context
    void* tmap_encode = nullptr;                          // cuTensorMapEncodeTiled entry point (resolved lazily)
    int* status_host = nullptr;  // host-mapped word raised by a kernel whose bounded wait gave up (0 = healthy)
    int* status_dev = nullptr;
    int gemm_tc_configured = 0, attn_umma_configured = 0;
    // cudaFuncSetAttribute applies to the current device only: which launch sites have configured their kernels on THIS
    // context's device (a process-wide flag would leave the second GPU of a single-process job unconfigured)
    std::set<const void*> configured_sites;
    int gemm_tile_n = 0;  // 0 = choose by shape; 1 / 128 / 256 / 512 force one tcgen05 GEMM kernel (b200_set_gemm_kernel)
    int gemm_box3d = 1;  // M/N-contiguous GEMM operands fetched as one three-dimensional TMA box per stage (0: one box per 32 columns)
    int clock_khz = 0;   // SM clock the bounded-wait budget is converted with
    // launches per engine since the context was created (b200_engine_launches): which code path a call really took
    int64_t engine_launches[B200_ENGINE_COUNT] = {0};
    // optional per-launch GEMM timing (b200_profile_gemm): event pairs recorded around every GEMM launch
    int profile = 0;
    std::vector<cudaEvent_t> prof_events;
    size_t prof_used = 0;
    std::vector<double> prof_flops;   // per launch
    std::vector<int> prof_engine;     // per launch: 0 SIMT, 1 tcgen05
    struct ProfShape { int M, N, K, tA, tB; };
    std::vector<ProfShape> prof_shape;  // per launch
};

namespace b200 {

int fail(b200_ctx* ctx, int code, const char* fmt, ...);
inline void ctx_retain(b200_ctx* ctx) { ctx->refs.fetch_add(1); }
// True the first time a launch site (identified by the address of a static tag) is reached on this context.
inline bool first_use(b200_ctx* ctx, const void* site) { return ctx->configured_sites.insert(site).second; }
void ctx_release(b200_ctx* ctx);  // frees the context when the last reference goes

#define B200_CUDA(ctx, expr)                                                                               \
    do {                                                                                                   \
        cudaError_t e__ = (expr);                                                                          \
        if (e__ != cudaSuccess)                                                                            \
            return b200::fail(ctx, B200_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), \
                              __FILE__, __LINE__);                                                         \
    } while (0)
#define B200_TRY(expr)              \
    do {                            \
        int rc__ = (expr);          \
        if (rc__ != B200_OK) return rc__; \
    } while (0)
#define B200_LAUNCH_CHECK(ctx)                                                                                  \
    do {                                                                                                        \
        (ctx)->launches++;                                                                                      \
        cudaError_t e__ = cudaGetLastError();                                                                   \
        if (e__ != cudaSuccess)                                                                                 \
            return b200::fail(ctx, B200_ERR_CUDA, "kernel launch failed: %s (%s:%d)", cudaGetErrorString(e__), \
                              __FILE__, __LINE__);                                                              \
    } while (0)

// B200_ERR_TIMEOUT if a kernel of this context reported that a bounded device-side wait expired (call after a sync).
int check_device_status(b200_ctx* ctx);
// Ensure ctx->ws holds at least n floats (contents are not preserved).
int ensure_ws(b200_ctx* ctx, size_t n);
// cos/sin table for rotary embeddings covering positions [0, rows).
int rope_table(b200_ctx* ctx, int headDim, float baseTheta, int rows, const float** out);

// ------------------------------------------------------------------------------------------------ GEMM
// C[M,N] = epilogue(alpha * op(A) * op(B)).  op(A) is [M,K]: stored [M,K] row-major (transA=0, leading dim lda) or
// [K,M] row-major (transA=1).  op(B) is [K,N]: stored [K,N] row-major (transB=0) or [N,K] row-major (transB=1).
// Epilogue, in order, for element (m,n) with v = alpha * acc (times *alpha_dev when given):
//   v += bias[n]; zout[m,n] = v; (act != NONE or dout) -> a = act(v), dout[m,n] = act'(v), v = a;
//   v *= act'(mulz[m,n]) (FFN derivative conventions); v *= mulmat[m,n]; v += addmat[m,n];
//   sgd_lr != 0 -> C = C - sgd_lr * (v + sgd_lambda * C); else accumulate ? C += v : C = v.
struct Gemm {
    int M = 0, N = 0, K = 0;
    const float* A = nullptr; int lda = 0; int transA = 0;
    const float* B = nullptr; int ldb = 0; int transB = 0;
    float* C = nullptr; int ldc = 0;
    float alpha = 1.f; const float* alpha_dev = nullptr;
    int accumulate = 0;
    const float* bias = nullptr;
    float* zout = nullptr; int ldz = 0;
    int act = B200_ACT_NONE; int act_conv = 0;  // 0: transformer-FFN conventions, 1: batch-MLP conventions
    float* dout = nullptr; int lddo = 0;
    const float* mulz = nullptr; int ldmulz = 0; int mulz_act = B200_ACT_NONE;
    int act_sign_zero = 0;  // activation outputs that are 0 because z < 0 are stored as -0.0 (lets ReLU'(z) be recovered from a)
    int mulz_is_act = 0;    // mulz holds the activation OUTPUT (stored with act_sign_zero); its derivative is computed from that
    const float* mulmat = nullptr; int ldmul = 0;
    const float* addmat = nullptr; int ldadd = 0;
    float sgd_lr = 0.f, sgd_lambda = 0.f;
    int round_tf32 = 0;  // store the result rounded to TF32 (round-to-nearest): its only consumer is a TF32 tensor-core kernel
    // Rotary position embedding applied to the result (after the bias) for columns [0, rope_cols): column pair
    // (2i, 2i+1) of every head of width rope_head_dim is rotated by table[pos[row]][i] = (cos, sin).  Fused into the
    // tcgen05 epilogue when the shape allows, otherwise run as a separate kernel after the GEMM.
    const float* rope_table = nullptr; const int32_t* rope_pos = nullptr; int rope_cols = 0, rope_head_dim = 0;
};
int gemm(b200_ctx* ctx, const Gemm& g);            // picks the engine from ctx->gemm_mode and the shape
int gemm_simt(b200_ctx* ctx, const Gemm& g);       // FP32 SIMT, any shape
int gemm_tcgen05_set_wait_budget(b200_ctx* ctx, long long clocks);
int attn_umma_set_wait_budget(b200_ctx* ctx, long long clocks);
int gemm_tcgen05_probe_wait(b200_ctx* ctx);
int gemm_tcgen05(b200_ctx* ctx, const Gemm& g);    // TF32 tcgen05/TMEM/TMA; B200_ERR_UNSUPPORTED if the shape does not qualify
bool gemm_tcgen05_eligible(b200_ctx* ctx, const Gemm& g);
bool gemm_tcgen05_fuses_rope(b200_ctx* ctx, const Gemm& g);  // the rope_* fields would be applied inside the tcgen05 epilogue
// Y[rows,outDim] (leading dim ldy) = X[rows,inDim] * W[outDim,inDim]^T + bias
int linear_fwd(b200_ctx* ctx, const float* X, int rows, int inDim, const float* W, const float* bias, int outDim, float* Y, int ldy);
// Wg[outDim,inDim] += dY^T X ; bg[outDim] += column sums of dY (bg may be null when the producer of dY already summed its columns)
int wgrad(b200_ctx* ctx, const float* dY, int lddy, const float* X, int ldx, int rows, int outDim, int inDim, float* Wg, float* bg);
// dX[rows,inDim] (+)= dY[rows,outDim] * W[outDim,inDim]
int dgrad(b200_ctx* ctx, const float* dY, int lddy, const float* W, int rows, int outDim, int inDim, float* dX, int accumulate);
// Stable counting sort of rows by token id (host): seg_id = distinct ids ascending, seg_off = start of each id's run in
// perm (plus the end), perm = row indices grouped by id with ascending row order inside a group.
void sort_rows_by_id(const int32_t* ids, int n, int vocab, std::vector<int32_t>& seg_id, std::vector<int32_t>& seg_off, std::vector<int32_t>& perm);

// ------------------------------------------------------------------------------------------------ elementwise / reductions
int k_add_inplace(b200_ctx*, float* target, const float* addend, int64_t n);
int k_scale_inplace(b200_ctx*, float* x, int64_t n, float scale);
int k_sgd_update(b200_ctx*, float* w, const float* g, int64_t n, float lr);
// x[i] *= act'(z[i]) with the transformer-FFN derivative conventions.
int k_mul_act_deriv(b200_ctx*, float* x, const float* z, int act, int64_t n);
int k_sqnorm(b200_ctx*, const float* x, int64_t n, float* out_dev);  // out_dev[0] = sum x^2 (deterministic two-stage)
// out[j] (+)= sum_i x[i, j] over rows; x has leading dimension ld.
int k_colsum(b200_ctx*, const float* x, int rows, int cols, int ld, float* out, int accumulate);
int k_embed(b200_ctx*, const int32_t* ids_dev, int count, const float* emb, int embDim, float* out);
int k_argmax(b200_ctx*, const float* x, int n, int32_t* out_dev);  // index of the maximum (lowest index among equals)
// Single-token decoding with the position in device memory (decode.cu): graph-capturable, no host-dependent argument.
int k_decode_embed(b200_ctx*, const int32_t* tokens, const int32_t* pos, const float* emb, int d, float* x);
int k_decode_rope_scatter(b200_ctx*, float* qkv, const int32_t* pos, const float* table, int d, int headDim, float* Kc, float* Vc);
int k_decode_attn(b200_ctx*, const float* q, const float* Kc, const float* Vc, const int32_t* pos, int numHeads, int headDim, float scale, float* out);
int k_decode_advance(b200_ctx*, const float* logits, int n, int32_t* tokens, int32_t* pos, int pick);
// One token through the whole model as one cooperative kernel (decode.cu).
struct DecodeLayer {
    const float *Wqkv, *bqkv, *WO, *bO, *g1, *b1n, *W1, *fb1, *W2, *fb2, *g2, *b2n;
    float *Kc, *Vc;  // this layer's key / value cache, [maxLen][d]
};
struct DecodeArgs {
    const DecodeLayer* layers;  // device array
    int L, d, f, H, hd, V, act, pick;
    float scale;
    const float *emb, *Wout, *bout, *rope;
    int32_t *tokens, *pos;
    float *x, *qkv, *attnO, *proj, *proj2, *n1, *a1, *logits;
};
int k_decode_token(b200_ctx*, const DecodeArgs& args, int* blocks_cache);
// y = act(W v + bias) for one token; with sub != NULL v = LayerNorm(x + sub) * gamma + beta, also stored to v_out.  K a
// multiple of 4 and at most 12288, all pointers 16-byte aligned, W rows K floats apart.
int k_decode_gemv(b200_ctx*, const float* x, const float* sub, const float* gamma, const float* beta, float eps, float* v_out, const float* W,
                  const float* bias, int N, int K, int act, float* y);
// Deterministic scatter-add: rows of (dXa [+ dXb]) sorted by id on the host.  seg_id[s] = vocabulary row, rows of
// segment s are perm[seg_off[s] .. seg_off[s+1]) in ascending original order.
int k_embed_scatter(b200_ctx*, float* eg, const float* dXa, const float* dXb, const int32_t* seg_id, const int32_t* seg_off,
                    const int32_t* perm, int nSeg, int embDim);
// Rotary embedding in place on `count` row-major matrices sharing one launch: matrix m = base + m*matStride, rows x ld,
// heads are numHeads slices of headDim columns starting at startCol.  pos_dev (per row) or row index when NULL.
int k_rope(b200_ctx*, float* base, int64_t matStride, int count, int rows, int ld, int startCol, int numHeads, int headDim,
           const float* table, const int32_t* pos_dev, int inverse, int round_tf32 = 0);
// Residual + LayerNorm forward.  sub, mean, var, normalized, residual may be null.
int k_ln_forward(b200_ctx*, const float* x, const float* sub, const float* gamma, const float* beta, int rows, int d, float eps,
                 float* out, float* mean, float* var, float* normalized, float* residual);
// LayerNorm backward on dOut = dOutA (+ dOutB).  dGamma/dBeta: accumulate ? += : =.
int k_ln_backward(b200_ctx*, const float* dOutA, const float* dOutB, const float* x, const float* gamma, const float* mean,
                  const float* var, int rows, int d, float eps, float* dx, float* dGamma, float* dBeta, int accumulate,
                  float* dxColSum = nullptr);  // dxColSum (optional): += column sums of dx, computed in the same pass
// Softmax cross-entropy, in place capable (dLogits may alias logits).  Per row i < effRows:
//   row_loss[i] = -log(p_t + 1e-10), row_ok[i] = all gradient entries finite, dLogits = (p - onehot) * row_scale[i]
// (row_scale_dev per row, or the constant row_scale when null).  Rows >= effRows are zeroed.
int k_cross_entropy(b200_ctx*, const float* logits, int rows, int V, const int32_t* targets_dev, int effRows, const float* row_scale_dev,
                    float row_scale, float* dLogits, float* row_loss, int32_t* row_ok);
// MSE: dOut = 2*(pred - target)*row_scale; row_loss[i] = sum_j diff^2.
int k_mse(b200_ctx*, const float* pred, int rows, int O, const float* targets_dev, int effRows, const float* row_scale_dev, float row_scale,
          float* dOut, float* row_loss, int32_t* row_ok);
// Batch-MLP output delta (GPUB:315-322 with the six cost derivatives of NN:314-390): delta = -costDeriv(a, y) * D.
int k_mlp_output_delta(b200_ctx*, const float* A, const float* D, const float* Y, int64_t n, int cost, float huberDelta, float* delta);
int k_mlp_scale_inputs(b200_ctx*, const float* X, int B, int F, const float* mn, const float* mx, float* out);
int k_mlp_clip_scale(b200_ctx*, const float* sumsq_dev, int nParts, float thr, float* scale_norm_dev);  // [0]=scale, [1]=norm
int k_bias_update(b200_ctx*, float* b, const float* delta, int rows, int cols, float slr, const float* scale_dev);

// ------------------------------------------------------------------------------------------------ attention
// Segment table: segment s covers query rows [qStart, qStart+qLen) and key rows [kStart, kStart+kLen).
struct AttnSeg { int qStart, qLen, kStart, kLen; };
struct Attn {
    const float *Q = nullptr, *K = nullptr, *V = nullptr;  // heads are column slices h*headDim..; leading dims below
    int ldq = 0, ldk = 0, ldv = 0;
    int numHeads = 0, headDim = 0;
    float scale = 1.f;
    int causal = 0;
    const uint8_t* mask = nullptr;  // only with a single segment: [qLen, kLen]
    const AttnSeg* segs_dev = nullptr; int nSeg = 0; int maxQLen = 0, maxKLen = 0;
    int totalQ = 0, totalK = 0;
    float* O = nullptr; int ldo = 0;
    float* rowMax = nullptr; float* rowSum = nullptr;  // [totalQ, numHeads]
    // backward
    const float* dO = nullptr; int lddo = 0;
    float *dQ = nullptr, *dK = nullptr, *dV = nullptr; int lddq = 0, lddk = 0, lddv = 0;
    float* rowDot = nullptr;  // [totalQ, numHeads] scratch: sum_k dO*O
    int pre_rounded = 0;      // Q, K, V (and dO) already hold TF32-rounded values: tiles can be copied asynchronously as they are
    // backward only: inverse rotary rotation of dQ and dK (table[pos[row]][i] = (cos, sin)), fused into the stores of
    // the tcgen05 engine, a separate kernel behind the other engines
    const float* rope_table = nullptr; const int32_t* rope_pos = nullptr;
};
int attn_forward(b200_ctx*, const Attn& a);   // dispatches to the TF32 tensor-core kernels when attn_tc_eligible
// TF32 mma.sync engine (head dimension <= 64, context not in FP32 mode)
bool attn_tc_eligible(b200_ctx*, const Attn& a);
int attn_forward_tc(b200_ctx*, const Attn& a);
int attn_backward_tc(b200_ctx*, const Attn& a);
// tcgen05 engine (head dimension 64, no explicit mask, sm_100a, context not in FP32 mode)
bool attn_umma_eligible(b200_ctx*, const Attn& a);
int attn_forward_umma(b200_ctx*, const Attn& a);
bool attn_umma_bwd_eligible(b200_ctx*, const Attn& a);
int attn_backward_umma(b200_ctx*, const Attn& a);
int attn_backward(b200_ctx*, const Attn& a);  // needs O, rowMax, rowSum from the forward

// ------------------------------------------------------------------------------------------------ parameter step
// One cooperative kernel: sumsq of (g*gscale) -> clip factor -> SGD or Adam update.  out_dev[0] = grad norm,
// out_dev[1] = applied clip factor.  A non-finite norm zeroes g and leaves w untouched.
int k_fused_step(b200_ctx*, float* w, float* g, float* m, float* v, int64_t n, float gscale, float lr, int use_clip, float clip_thr,
                 int do_step, int optimizer, float beta1, float beta2, float eps, int step_index, float* out_dev, int write_g = 1);
// The same step in one pass over HBM, for a gradient whose sums of squares were taken beforehand: partials[0, n_partials)
// hold sums of UNSCALED squares (unused slots zero); they are added in index order.
int k_fused_step_presummed(b200_ctx*, float* w, float* g, float* m, float* v, int64_t n, const float* partials, int n_partials, float gscale,
                           float lr, int use_clip, float clip_thr, int do_step, int optimizer, float beta1, float beta2, float eps, int step_index,
                           float* out_dev, int write_g = 1);
// g[0, n) *= factor (the scaling a step launched with write_g = 0 still owes the gradient arena).
int k_scale_arena(b200_ctx*, float* g, int64_t n, float factor);
// Sums of squares of g[0, n) into partials[0, *blocks) on `stream`, one partial per block, fixed order (deterministic).
int k_sumsq_partials(b200_ctx*, const float* g, int64_t n, float* partials, int max_blocks, cudaStream_t stream, int* blocks);


// ------------------------------------------------------------------------------------------------ resident trainer, as seen by the data-parallel layer
b200_ctx* lm_context(b200_lm* lm);
void lm_retain(b200_lm* lm);  // released with b200_lm_destroy
int64_t lm_param_total(const b200_lm* lm);
const b200_lm_config& lm_config_of(const b200_lm* lm);
// Ranges of the gradient arena in the order the last pass's backward completes them (and announces them to the callback).
std::vector<std::pair<int64_t, int64_t>> lm_grad_ranges(const b200_lm* lm);
// Data-parallel jobs take the sums of squares for the one-pass step themselves, after each range's all-reduce:
// lm_set_external_norm(true) stops the trainer from summing its local gradient, lm_sumsq_range enqueues the sum of range
// `index` (in lm_grad_ranges order) on `stream`.
void lm_set_external_norm(b200_lm* lm, bool on);
int lm_sumsq_range(b200_lm* lm, int index, cudaStream_t stream);

}  // namespace b200
