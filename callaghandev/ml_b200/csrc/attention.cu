// Multi-head scaled-dot-product attention, forward and backward, over a table of independent segments (one segment
// per sequence of a packed batch; heads are column slices of the [rows, embeddingDim] matrices).
//
// Forward: 64-query x 64-key tiles, online softmax, saves the row maximum and row sum of exponentials per
// (row, head) instead of the probability matrix.
// Backward: probabilities are recomputed tile by tile from the saved row max / sum.  Two passes, each owning its
// outputs exclusively (no atomics, deterministic):
//   pass dKV: a block owns 64 keys and walks the query tiles that can see them: dV += P^T dO, dK += dS^T Q;
//   pass dQ : a block owns 64 queries and walks the visible key tiles:          dQ += dS K,
// with dP = dO V^T, dS = P o (dP - rowDot) * scale and rowDot[i] = sum_c dO[i,c] O[i,c] (equal to the reference's
// sum_j w_j dA_j).  FP32 throughout.  Head dimensions up to 128 (padded to a multiple of 16 in shared memory).
#include "common.h"
#include "device_math.cuh"

namespace b200 {

constexpr int TQ = 64, TK = 64, ATT_THREADS = 256, PS = TK + 1;

struct AttnArgs {
    const float *Q, *K, *V, *dO, *O;
    int ldq, ldk, ldv, lddo, ldo;
    float *Oout, *dQ, *dK, *dV;
    int lddq, lddk, lddv;
    float *rowMax, *rowSum, *rowDot;
    const AttnSeg* segs;
    const uint8_t* mask;
    int numHeads, headDim, causal;
    float scale;
};

template <int HD>
__device__ __forceinline__ void load_tile(float* __restrict__ dst, const float* __restrict__ src, int ld, int rowStart, int nValid,
                                          int colOff, int hd) {
    constexpr int HS = HD + 1;
    for (int idx = threadIdx.x; idx < 64 * HD; idx += ATT_THREADS) {
        int r = idx / HD, c = idx - r * HD;
        float v = 0.f;
        if (r < nValid && c < hd) v = src[(size_t)(rowStart + r) * ld + colOff + c];
        dst[r * HS + c] = v;
    }
}

__device__ __forceinline__ bool visible(const AttnArgs& a, const AttnSeg& sg, int qi, int kj) {
    if (qi >= sg.qLen || kj >= sg.kLen) return false;
    if (a.causal && kj > qi) return false;
    if (a.mask && !a.mask[(size_t)qi * sg.kLen + kj]) return false;
    return true;
}

// s[i][j] = sum_c X[(ty*4+i)][c] * Y[(tx+16j)][c]
template <int HD>
__device__ __forceinline__ void tile_dot(const float* __restrict__ X, const float* __restrict__ Y, int ty, int tx, float s[4][4]) {
    constexpr int HS = HD + 1;
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) s[i][j] = 0.f;
#pragma unroll 8
    for (int c = 0; c < HD; c++) {
        float x[4], y[4];
#pragma unroll
        for (int i = 0; i < 4; i++) x[i] = X[(ty * 4 + i) * HS + c];
#pragma unroll
        for (int j = 0; j < 4; j++) y[j] = Y[(tx + 16 * j) * HS + c];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) s[i][j] = fmaf(x[i], y[j], s[i][j]);
    }
}

template <int HD>
__global__ void __launch_bounds__(ATT_THREADS) attn_fwd_kernel(AttnArgs a) {
    constexpr int HS = HD + 1, NC = HD / 16;
    extern __shared__ float sm[];
    float* Qs = sm;
    float* Ks = Qs + 64 * HS;
    float* Vs = Ks + 64 * HS;
    float* Ps = Vs + 64 * HS;
    const AttnSeg sg = a.segs[blockIdx.z];
    const int q0 = blockIdx.x * TQ;
    if (q0 >= sg.qLen) return;
    const int head = blockIdx.y, colOff = head * a.headDim, hd = a.headDim;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    load_tile<HD>(Qs, a.Q, a.ldq, sg.qStart + q0, min(TQ, sg.qLen - q0), colOff, hd);
    float m_i[4], l_i[4], o[4][NC];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        m_i[i] = -INFINITY;
        l_i[i] = 0.f;
#pragma unroll
        for (int j = 0; j < NC; j++) o[i][j] = 0.f;
    }
    const int kEnd = a.causal ? min(sg.kLen, q0 + TQ) : sg.kLen;
    for (int k0 = 0; k0 < kEnd; k0 += TK) {
        __syncthreads();  // previous tile fully consumed (also orders the Q load before first use)
        load_tile<HD>(Ks, a.K, a.ldk, sg.kStart + k0, min(TK, sg.kLen - k0), colOff, hd);
        load_tile<HD>(Vs, a.V, a.ldv, sg.kStart + k0, min(TK, sg.kLen - k0), colOff, hd);
        __syncthreads();
        float s[4][4];
        tile_dot<HD>(Qs, Ks, ty, tx, s);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int qi = q0 + ty * 4 + i;
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                int kj = k0 + tx + 16 * j;
                s[i][j] = visible(a, sg, qi, kj) ? s[i][j] * a.scale : -INFINITY;
                mx = fmaxf(mx, s[i][j]);
            }
#pragma unroll
            for (int o2 = 8; o2 > 0; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o2));
            float m_new = fmaxf(m_i[i], mx);
            float corr = (m_i[i] == -INFINITY) ? 0.f : expf(m_i[i] - m_new);
            float rs = 0.f;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float p = (s[i][j] == -INFINITY) ? 0.f : expf(s[i][j] - m_new);
                rs += p;
                Ps[(ty * 4 + i) * PS + tx + 16 * j] = p;
            }
#pragma unroll
            for (int o2 = 8; o2 > 0; o2 >>= 1) rs += __shfl_xor_sync(0xffffffffu, rs, o2);
            l_i[i] = l_i[i] * corr + rs;
            m_i[i] = m_new;
#pragma unroll
            for (int j = 0; j < NC; j++) o[i][j] *= corr;
        }
        __syncthreads();
#pragma unroll 4
        for (int n = 0; n < TK; n++) {
            float p[4], v[NC];
#pragma unroll
            for (int i = 0; i < 4; i++) p[i] = Ps[(ty * 4 + i) * PS + n];
#pragma unroll
            for (int j = 0; j < NC; j++) v[j] = Vs[n * HS + tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < NC; j++) o[i][j] = fmaf(p[i], v[j], o[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int qi = q0 + ty * 4 + i;
        if (qi >= sg.qLen) continue;
        float inv = l_i[i] > 0.f ? 1.0f / l_i[i] : 0.f;
        size_t row = (size_t)(sg.qStart + qi);
#pragma unroll
        for (int j = 0; j < NC; j++) {
            int c = tx + 16 * j;
            if (c < hd) a.Oout[row * a.ldo + colOff + c] = o[i][j] * inv;
        }
        if (tx == 0 && a.rowMax) {
            a.rowMax[row * a.numHeads + head] = m_i[i];
            a.rowSum[row * a.numHeads + head] = l_i[i];
        }
    }
}

// rowDot[row, head] = sum_c dO[row, head*hd + c] * O[row, head*hd + c]; one warp per (row, head).
__global__ void attn_rowdot_kernel(const float* __restrict__ dO, int lddo, const float* __restrict__ O, int ldo, int rows, int numHeads,
                                   int hd, float* __restrict__ rowDot) {
    int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (w >= rows * numHeads) return;
    int row = w / numHeads, head = w - row * numHeads;
    float s = 0.f;
    for (int c = lane; c < hd; c += 32) s += dO[(size_t)row * lddo + head * hd + c] * O[(size_t)row * ldo + head * hd + c];
    s = warp_sum(s);
    if (lane == 0) rowDot[w] = s;
}

// Recompute P and dS for the (q tile, k tile) pair held in shared memory; results go to Ps / dSs.
template <int HD>
__device__ __forceinline__ void recompute_p_ds(const AttnArgs& a, const AttnSeg& sg, const float* Qs, const float* Ks, const float* Vs,
                                               const float* dOs, const float* s_m, const float* s_il, const float* s_D, int q0, int k0,
                                               int ty, int tx, float* Ps, float* dSs) {
    float s[4][4], dp[4][4];
    tile_dot<HD>(Qs, Ks, ty, tx, s);
    tile_dot<HD>(dOs, Vs, ty, tx, dp);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int r = ty * 4 + i, qi = q0 + r;
        float m = s_m[r], il = s_il[r], D = s_D[r];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int kj = k0 + tx + 16 * j;
            float p = 0.f;
            if (il > 0.f && visible(a, sg, qi, kj)) p = expf(s[i][j] * a.scale - m) * il;
            Ps[r * PS + tx + 16 * j] = p;
            if (dSs) dSs[r * PS + tx + 16 * j] = p * (dp[i][j] - D) * a.scale;
        }
    }
}

template <int HD>
__device__ __forceinline__ void load_row_stats(const AttnArgs& a, const AttnSeg& sg, int q0, int head, float* s_m, float* s_il, float* s_D) {
    if (threadIdx.x < 64) {
        int qi = q0 + threadIdx.x;
        float m = 0.f, il = 0.f, D = 0.f;
        if (qi < sg.qLen) {
            size_t idx = (size_t)(sg.qStart + qi) * a.numHeads + head;
            m = a.rowMax[idx];
            float l = a.rowSum[idx];
            il = (l > 0.f && m != -INFINITY) ? 1.0f / l : 0.f;
            D = a.rowDot[idx];
        }
        s_m[threadIdx.x] = m;
        s_il[threadIdx.x] = il;
        s_D[threadIdx.x] = D;
    }
}

template <int HD>
__global__ void __launch_bounds__(ATT_THREADS) attn_bwd_dkv_kernel(AttnArgs a) {
    constexpr int HS = HD + 1, NC = HD / 16;
    extern __shared__ float sm[];
    float* Ks = sm;
    float* Vs = Ks + 64 * HS;
    float* Qs = Vs + 64 * HS;
    float* dOs = Qs + 64 * HS;
    float* Ps = dOs + 64 * HS;
    float* dSs = Ps + 64 * PS;
    float* s_m = dSs + 64 * PS;
    float* s_il = s_m + 64;
    float* s_D = s_il + 64;
    const AttnSeg sg = a.segs[blockIdx.z];
    const int k0 = blockIdx.x * TK;
    if (k0 >= sg.kLen) return;
    const int head = blockIdx.y, colOff = head * a.headDim, hd = a.headDim;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    load_tile<HD>(Ks, a.K, a.ldk, sg.kStart + k0, min(TK, sg.kLen - k0), colOff, hd);
    load_tile<HD>(Vs, a.V, a.ldv, sg.kStart + k0, min(TK, sg.kLen - k0), colOff, hd);
    float dk[4][NC], dv[4][NC];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < NC; j++) { dk[i][j] = 0.f; dv[i][j] = 0.f; }
    const int qBegin = a.causal ? k0 : 0;  // queries before the tile's first key cannot see any of its keys
    for (int q0 = qBegin; q0 < sg.qLen; q0 += TQ) {
        __syncthreads();
        load_tile<HD>(Qs, a.Q, a.ldq, sg.qStart + q0, min(TQ, sg.qLen - q0), colOff, hd);
        load_tile<HD>(dOs, a.dO, a.lddo, sg.qStart + q0, min(TQ, sg.qLen - q0), colOff, hd);
        load_row_stats<HD>(a, sg, q0, head, s_m, s_il, s_D);
        __syncthreads();
        recompute_p_ds<HD>(a, sg, Qs, Ks, Vs, dOs, s_m, s_il, s_D, q0, k0, ty, tx, Ps, dSs);
        __syncthreads();
#pragma unroll 4
        for (int q = 0; q < TQ; q++) {
            float p[4], ds[4], dov[NC], qv[NC];
#pragma unroll
            for (int i = 0; i < 4; i++) { p[i] = Ps[q * PS + ty * 4 + i]; ds[i] = dSs[q * PS + ty * 4 + i]; }
#pragma unroll
            for (int j = 0; j < NC; j++) { dov[j] = dOs[q * HS + tx + 16 * j]; qv[j] = Qs[q * HS + tx + 16 * j]; }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < NC; j++) {
                    dv[i][j] = fmaf(p[i], dov[j], dv[i][j]);
                    dk[i][j] = fmaf(ds[i], qv[j], dk[i][j]);
                }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int kj = k0 + ty * 4 + i;
        if (kj >= sg.kLen) continue;
        size_t row = (size_t)(sg.kStart + kj);
#pragma unroll
        for (int j = 0; j < NC; j++) {
            int c = tx + 16 * j;
            if (c < hd) {
                a.dK[row * a.lddk + colOff + c] = dk[i][j];
                a.dV[row * a.lddv + colOff + c] = dv[i][j];
            }
        }
    }
}

template <int HD>
__global__ void __launch_bounds__(ATT_THREADS) attn_bwd_dq_kernel(AttnArgs a) {
    constexpr int HS = HD + 1, NC = HD / 16;
    extern __shared__ float sm[];
    float* Ks = sm;
    float* Vs = Ks + 64 * HS;
    float* Qs = Vs + 64 * HS;
    float* dOs = Qs + 64 * HS;
    float* Ps = dOs + 64 * HS;
    float* dSs = Ps + 64 * PS;
    float* s_m = dSs + 64 * PS;
    float* s_il = s_m + 64;
    float* s_D = s_il + 64;
    const AttnSeg sg = a.segs[blockIdx.z];
    const int q0 = blockIdx.x * TQ;
    if (q0 >= sg.qLen) return;
    const int head = blockIdx.y, colOff = head * a.headDim, hd = a.headDim;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    load_tile<HD>(Qs, a.Q, a.ldq, sg.qStart + q0, min(TQ, sg.qLen - q0), colOff, hd);
    load_tile<HD>(dOs, a.dO, a.lddo, sg.qStart + q0, min(TQ, sg.qLen - q0), colOff, hd);
    load_row_stats<HD>(a, sg, q0, head, s_m, s_il, s_D);
    float dq[4][NC];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < NC; j++) dq[i][j] = 0.f;
    const int kEnd = a.causal ? min(sg.kLen, q0 + TQ) : sg.kLen;
    for (int k0 = 0; k0 < kEnd; k0 += TK) {
        __syncthreads();
        load_tile<HD>(Ks, a.K, a.ldk, sg.kStart + k0, min(TK, sg.kLen - k0), colOff, hd);
        load_tile<HD>(Vs, a.V, a.ldv, sg.kStart + k0, min(TK, sg.kLen - k0), colOff, hd);
        __syncthreads();
        recompute_p_ds<HD>(a, sg, Qs, Ks, Vs, dOs, s_m, s_il, s_D, q0, k0, ty, tx, Ps, dSs);
        __syncthreads();
#pragma unroll 4
        for (int n = 0; n < TK; n++) {
            float ds[4], kv[NC];
#pragma unroll
            for (int i = 0; i < 4; i++) ds[i] = dSs[(ty * 4 + i) * PS + n];
#pragma unroll
            for (int j = 0; j < NC; j++) kv[j] = Ks[n * HS + tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < NC; j++) dq[i][j] = fmaf(ds[i], kv[j], dq[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int qi = q0 + ty * 4 + i;
        if (qi >= sg.qLen) continue;
        size_t row = (size_t)(sg.qStart + qi);
#pragma unroll
        for (int j = 0; j < NC; j++) {
            int c = tx + 16 * j;
            if (c < hd) a.dQ[row * a.lddq + colOff + c] = dq[i][j];
        }
    }
}

static AttnArgs make_args(const Attn& t) {
    AttnArgs a;
    a.Q = t.Q; a.K = t.K; a.V = t.V; a.dO = t.dO; a.O = t.O;
    a.ldq = t.ldq; a.ldk = t.ldk; a.ldv = t.ldv; a.lddo = t.lddo; a.ldo = t.ldo;
    a.Oout = t.O; a.dQ = t.dQ; a.dK = t.dK; a.dV = t.dV; a.lddq = t.lddq; a.lddk = t.lddk; a.lddv = t.lddv;
    a.rowMax = t.rowMax; a.rowSum = t.rowSum; a.rowDot = t.rowDot;
    a.segs = t.segs_dev; a.mask = t.mask; a.numHeads = t.numHeads; a.headDim = t.headDim; a.causal = t.causal; a.scale = t.scale;
    return a;
}

static size_t fwd_smem(int HD) { return (size_t)(3 * 64 * (HD + 1) + 64 * PS) * sizeof(float); }
static size_t bwd_smem(int HD) { return (size_t)(4 * 64 * (HD + 1) + 2 * 64 * PS + 3 * 64) * sizeof(float); }

template <int HD>
static int launch_fwd(b200_ctx* ctx, const Attn& t) {
    static char configured_site;
    if (first_use(ctx, &configured_site)) {
        B200_CUDA(ctx, cudaFuncSetAttribute(attn_fwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fwd_smem(HD)));
    }
    dim3 grid((t.maxQLen + TQ - 1) / TQ, t.numHeads, t.nSeg);
    attn_fwd_kernel<HD><<<grid, ATT_THREADS, fwd_smem(HD), ctx->stream>>>(make_args(t));
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}
template <int HD>
static int launch_bwd(b200_ctx* ctx, const Attn& t) {
    static char configured_site;
    if (first_use(ctx, &configured_site)) {
        B200_CUDA(ctx, cudaFuncSetAttribute(attn_bwd_dkv_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bwd_smem(HD)));
        B200_CUDA(ctx, cudaFuncSetAttribute(attn_bwd_dq_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bwd_smem(HD)));
    }
    AttnArgs a = make_args(t);
    int warps = t.totalQ * t.numHeads;
    attn_rowdot_kernel<<<(warps * 32 + 255) / 256, 256, 0, ctx->stream>>>(t.dO, t.lddo, t.O, t.ldo, t.totalQ, t.numHeads, t.headDim, t.rowDot);
    B200_LAUNCH_CHECK(ctx);
    dim3 gk((t.maxKLen + TK - 1) / TK, t.numHeads, t.nSeg);
    attn_bwd_dkv_kernel<HD><<<gk, ATT_THREADS, bwd_smem(HD), ctx->stream>>>(a);
    B200_LAUNCH_CHECK(ctx);
    dim3 gq((t.maxQLen + TQ - 1) / TQ, t.numHeads, t.nSeg);
    attn_bwd_dq_kernel<HD><<<gq, ATT_THREADS, bwd_smem(HD), ctx->stream>>>(a);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

int attn_forward(b200_ctx* ctx, const Attn& t) {
    if (t.nSeg <= 0 || t.maxQLen <= 0 || t.numHeads <= 0) return B200_OK;
    if (attn_tc_eligible(ctx, t)) return attn_forward_tc(ctx, t);
    ctx->engine_launches[B200_ENGINE_ATTN_FP32]++;
    if (t.headDim <= 16) return launch_fwd<16>(ctx, t);
    if (t.headDim <= 32) return launch_fwd<32>(ctx, t);
    if (t.headDim <= 64) return launch_fwd<64>(ctx, t);
    if (t.headDim <= 128) return launch_fwd<128>(ctx, t);
    return fail(ctx, B200_ERR_UNSUPPORTED, "attention head dimension %d exceeds 128", t.headDim);
}
static int attn_backward_engine(b200_ctx* ctx, const Attn& t) {
    if (attn_tc_eligible(ctx, t)) return attn_backward_tc(ctx, t);
    ctx->engine_launches[B200_ENGINE_ATTN_FP32]++;
    if (t.headDim <= 16) return launch_bwd<16>(ctx, t);
    if (t.headDim <= 32) return launch_bwd<32>(ctx, t);
    if (t.headDim <= 64) return launch_bwd<64>(ctx, t);
    if (t.headDim <= 128) return launch_bwd<128>(ctx, t);
    return fail(ctx, B200_ERR_UNSUPPORTED, "attention head dimension %d exceeds 128", t.headDim);
}
int attn_backward(b200_ctx* ctx, const Attn& t) {
    if (t.nSeg <= 0 || t.numHeads <= 0) return B200_OK;
    if (!t.rope_table || (attn_tc_eligible(ctx, t) && attn_umma_bwd_eligible(ctx, t))) return attn_backward_engine(ctx, t);  // fused, or nothing to rotate
    Attn u = t;
    u.rope_table = nullptr;
    B200_TRY(attn_backward_engine(ctx, u));
    B200_TRY(k_rope(ctx, t.dQ, 0, 1, t.totalQ, t.lddq, 0, t.numHeads, t.headDim, t.rope_table, t.rope_pos, 1, 0));
    return k_rope(ctx, t.dK, 0, 1, t.totalK, t.lddk, 0, t.numHeads, t.headDim, t.rope_table, t.rope_pos, 1, 0);
}

}  // namespace b200
