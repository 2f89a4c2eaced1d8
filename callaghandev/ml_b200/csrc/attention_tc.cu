// Tensor-core attention (TF32 mma.sync m16n8k8, FP32 accumulate) for head dimensions up to 64: the engine used when
// the context runs in TF32 mode.  Same algorithm and the same saved statistics as the FP32 kernels in attention.cu
// (online-softmax forward that stores row max / row sum; backward that recomputes P tile by tile; two deterministic
// passes, no atomics), with every 64x64xhd contraction issued as warp-level tensor-core MMAs.
//
// A block is 4 warps and owns 64 rows (queries in forward / dQ pass, keys in dK,dV pass); a warp owns 16 of them.
// Fragment conventions of mma.m16n8k8 (g = lane/4, t = lane%4):
//   A 16x8: a0=(g,t) a1=(g+8,t) a2=(g,t+4) a3=(g+8,t+4);  B 8x8: b0=(k=t,n=g) b1=(k=t+4,n=g);
//   C 16x8: c0=(g,2t) c1=(g,2t+1) c2=(g+8,2t) c3=(g+8,2t+1).
// Where a C fragment (probabilities, dS) feeds the next product as the A operand, the contraction index is taken in
// the order (2t, 2t+1) instead of (t, t+4) on both operands, so the accumulator registers are used in place.
// Operands are rounded to TF32 (cvt.rna) when they are staged in shared memory.
#include "common.h"
#include "device_math.cuh"

namespace b200 {

namespace {

constexpr int TC_THREADS = 128;

struct TcAttnArgs {
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

__device__ __forceinline__ uint32_t to_tf32(float x) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
    return u;
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float fast_exp2(float x) {  // 2^x; -inf gives +0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Four 8x4-word blocks of a row-major tile in one instruction: lane l supplies the address of row (l%8) of block (l/8);
// every lane receives word (l%4) of row (l/4) of each block, which is exactly the B fragment (k = l%4, n = l/4) of a
// tile stored [n][k].
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const uint32_t* p) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// Stage rows [rowStart, rowStart+64) x columns [colOff, colOff+hd) of a [rows, ld] matrix as TF32 words, zero-padded to
// 64 x HD, with row stride STRIDE.
template <int HD, int STRIDE>
__device__ __forceinline__ void stage_tile(uint32_t* __restrict__ dst, const float* __restrict__ src, int ld, int rowStart, int nValid, int colOff,
                                           int hd, bool vec) {
    if (vec) {
        for (int idx = threadIdx.x; idx < 64 * (HD / 4); idx += TC_THREADS) {
            int r = idx / (HD / 4), c = (idx - r * (HD / 4)) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (r < nValid && c < hd) v = *reinterpret_cast<const float4*>(src + (size_t)(rowStart + r) * ld + colOff + c);
            uint4 u = make_uint4(to_tf32(v.x), to_tf32(v.y), to_tf32(v.z), to_tf32(v.w));
            *reinterpret_cast<uint4*>(dst + r * STRIDE + c) = u;
        }
    } else {
        for (int idx = threadIdx.x; idx < 64 * HD; idx += TC_THREADS) {
            int r = idx / HD, c = idx - r * HD;
            float v = 0.f;
            if (r < nValid && c < hd) v = src[(size_t)(rowStart + r) * ld + colOff + c];
            dst[r * STRIDE + c] = to_tf32(v);
        }
    }
}

__device__ __forceinline__ bool tc_visible(const TcAttnArgs& a, const AttnSeg& sg, int qi, int kj) {
    if (qi >= sg.qLen || kj >= sg.kLen) return false;
    if (a.causal && kj > qi) return false;
    if (a.mask && !a.mask[(size_t)qi * sg.kLen + kj]) return false;
    return true;
}

// A fragments of a warp's 16 rows (rows w16.. of a staged tile) over the whole head dimension.
template <int HD, int STRIDE>
__device__ __forceinline__ void load_a_frags(const uint32_t* __restrict__ tile, int row0, int g, int t, uint32_t (&a)[HD / 8][4]) {
#pragma unroll
    for (int ks = 0; ks < HD / 8; ks++) {
        a[ks][0] = tile[(row0 + g) * STRIDE + ks * 8 + t];
        a[ks][1] = tile[(row0 + g + 8) * STRIDE + ks * 8 + t];
        a[ks][2] = tile[(row0 + g) * STRIDE + ks * 8 + t + 4];
        a[ks][3] = tile[(row0 + g + 8) * STRIDE + ks * 8 + t + 4];
    }
}

// c[nt] (16 rows x 64 staged rows of Bt) += A(16 x HD) * Bt(64 x HD)^T.  B fragments come four at a time (two K steps).
template <int HD, int STRIDE>
__device__ __forceinline__ void mma_a_bt(const uint32_t (&a)[HD / 8][4], const uint32_t* __restrict__ Bt, int g, int t, float (&c)[8][4]) {
    const int lane = g * 4 + t;
    const uint32_t* base = Bt + (lane & 7) * STRIDE + 4 * (lane >> 3);
#pragma unroll
    for (int nt = 0; nt < 8; nt++) {
#pragma unroll
        for (int ks = 0; ks < HD / 8; ks += 2) {
            uint32_t b[4];
            ldsm_x4(b, base + nt * 8 * STRIDE + ks * 8);
            mma_tf32(c[nt], a[ks][0], a[ks][1], a[ks][2], a[ks][3], b[0], b[1]);
            mma_tf32(c[nt], a[ks + 1][0], a[ks + 1][1], a[ks + 1][2], a[ks + 1][3], b[2], b[3]);
        }
    }
}

// o[nt2] (16 x HD) += P(16 x 64, held as C fragments p[nt]) * B(64 x HD); contraction order (2t, 2t+1) per 8-block.
template <int HD, int STRIDE>
__device__ __forceinline__ void mma_c_b(const uint32_t (&p)[8][4], const uint32_t* __restrict__ B, int g, int t, float (&o)[HD / 8][4]) {
#pragma unroll
    for (int nt = 0; nt < 8; nt++) {
#pragma unroll
        for (int n2 = 0; n2 < HD / 8; n2++) {
            uint32_t b0 = B[(nt * 8 + 2 * t) * STRIDE + n2 * 8 + g], b1 = B[(nt * 8 + 2 * t + 1) * STRIDE + n2 * 8 + g];
            mma_tf32(o[n2], p[nt][0], p[nt][2], p[nt][1], p[nt][3], b0, b1);
        }
    }
}

constexpr float LOG2E = 1.4426950408889634f;

template <int HD>
__global__ void __launch_bounds__(TC_THREADS) attn_fwd_tc_kernel(TcAttnArgs a, int vec) {
    constexpr int ST = HD + 4;
    extern __shared__ __align__(16) uint32_t smu[];
    uint32_t* Qs = smu;
    uint32_t* Ks = Qs + 64 * ST;
    uint32_t* Vs = Ks + 64 * ST;
    const AttnSeg sg = a.segs[blockIdx.z];
    const int q0 = blockIdx.x * 64;
    if (q0 >= sg.qLen) return;
    const int head = blockIdx.y, colOff = head * a.headDim, hd = a.headDim;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    stage_tile<HD, ST>(Qs, a.Q, a.ldq, sg.qStart + q0, min(64, sg.qLen - q0), colOff, hd, vec);
    __syncthreads();
    uint32_t qa[HD / 8][4];
    load_a_frags<HD, ST>(Qs, warp * 16, g, t, qa);
    float m_i[2] = {-INFINITY, -INFINITY}, l_i[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    const int kEnd = a.causal ? min(sg.kLen, q0 + 64) : sg.kLen;
    const float sl2 = a.scale * LOG2E;
    for (int k0 = 0; k0 < kEnd; k0 += 64) {
        __syncthreads();
        stage_tile<HD, ST>(Ks, a.K, a.ldk, sg.kStart + k0, min(64, sg.kLen - k0), colOff, hd, vec);
        stage_tile<HD, ST>(Vs, a.V, a.ldv, sg.kStart + k0, min(64, sg.kLen - k0), colOff, hd, vec);
        __syncthreads();
        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; nt++) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
        mma_a_bt<HD, ST>(qa, Ks, g, t, s);
        uint32_t p[8][4];
        // a tile that no mask, sequence end or causal diagonal touches needs no per-element visibility test (warp-uniform)
        const bool full = !a.mask && k0 + 64 <= sg.kLen && q0 + warp * 16 + 16 <= sg.qLen && (!a.causal || k0 + 63 <= q0 + warp * 16);
#pragma unroll
        for (int h = 0; h < 2; h++) {  // the two rows (g, g+8) this thread holds
            const int qi = q0 + warp * 16 + g + 8 * h;
            float mx = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 8; nt++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int kj = k0 + nt * 8 + 2 * t + e;
                    float v = (full || tc_visible(a, sg, qi, kj)) ? s[nt][2 * h + e] * sl2 : -INFINITY;  // scores in log2 units
                    s[nt][2 * h + e] = v;
                    mx = fmaxf(mx, v);
                }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_i[h], mx);
            const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;  // keeps (-inf) - (-inf) out of the exponent
            const float corr = fast_exp2(m_i[h] - m_safe);
            float rs = 0.f;
#pragma unroll
            for (int nt = 0; nt < 8; nt++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const float v = s[nt][2 * h + e];
                    const float pv = fast_exp2(v - m_safe);
                    rs += pv;
                    p[nt][2 * h + e] = to_tf32(pv);
                }
            rs += __shfl_xor_sync(0xffffffffu, rs, 1);
            rs += __shfl_xor_sync(0xffffffffu, rs, 2);
            l_i[h] = l_i[h] * corr + rs;
            m_i[h] = m_new;
#pragma unroll
            for (int i = 0; i < HD / 8; i++) { o[i][2 * h] *= corr; o[i][2 * h + 1] *= corr; }
        }
        mma_c_b<HD, ST>(p, Vs, g, t, o);
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int qi = q0 + warp * 16 + g + 8 * h;
        if (qi >= sg.qLen) continue;
        const float inv = l_i[h] > 0.f ? 1.0f / l_i[h] : 0.f;
        const size_t row = (size_t)(sg.qStart + qi);
#pragma unroll
        for (int i = 0; i < HD / 8; i++) {
            const int c = i * 8 + 2 * t;
            if (c < hd) a.Oout[row * a.ldo + colOff + c] = o[i][2 * h] * inv;
            if (c + 1 < hd) a.Oout[row * a.ldo + colOff + c + 1] = o[i][2 * h + 1] * inv;
        }
        if (t == 0 && a.rowMax) {  // stored in natural-log units, the convention of the FP32 kernels
            a.rowMax[row * a.numHeads + head] = m_i[h] == -INFINITY ? -INFINITY : m_i[h] / LOG2E;
            a.rowSum[row * a.numHeads + head] = l_i[h];
        }
    }
}

// Recompute P and dS fragments of this warp's 16 query rows against the staged 64 keys.
//   s = (q.k)*scale; P = exp(s - m)/l; dP = dO.V^T; dS = P*(dP - D)*scale
template <int HD, int STK>
__device__ __forceinline__ void recompute_tc(const TcAttnArgs& a, const AttnSeg& sg, const uint32_t (&qa)[HD / 8][4], const uint32_t (&da)[HD / 8][4],
                                             const uint32_t* Ks, const uint32_t* Vs, const float (&mrow)[2], const float (&ilrow)[2],
                                             const float (&drow)[2], int qbase, int k0, int g, int t, float (&s)[8][4], float (&dp)[8][4]) {
#pragma unroll
    for (int nt = 0; nt < 8; nt++) {
        s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
        dp[nt][0] = dp[nt][1] = dp[nt][2] = dp[nt][3] = 0.f;
    }
    mma_a_bt<HD, STK>(qa, Ks, g, t, s);
    mma_a_bt<HD, STK>(da, Vs, g, t, dp);
    const float sl2 = a.scale * LOG2E;
    const bool full = !a.mask && k0 + 64 <= sg.kLen && qbase + 16 <= sg.qLen && (!a.causal || k0 + 63 <= qbase);
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int qi = qbase + g + 8 * h;
        const float m2 = mrow[h] * LOG2E;
#pragma unroll
        for (int nt = 0; nt < 8; nt++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int kj = k0 + nt * 8 + 2 * t + e;
                float pv = 0.f;
                if (full || tc_visible(a, sg, qi, kj)) pv = fast_exp2(s[nt][2 * h + e] * sl2 - m2) * ilrow[h];  // ilrow = 0 for rows with no visible key
                s[nt][2 * h + e] = pv;                                              // P
                dp[nt][2 * h + e] = pv * (dp[nt][2 * h + e] - drow[h]) * a.scale;  // dS
            }
    }
}

__device__ __forceinline__ void row_stats(const TcAttnArgs& a, const AttnSeg& sg, int qi, int head, float& m, float& il, float& D) {
    m = 0.f; il = 0.f; D = 0.f;
    if (qi < sg.qLen) {
        const size_t idx = (size_t)(sg.qStart + qi) * a.numHeads + head;
        m = a.rowMax[idx];
        const float l = a.rowSum[idx];
        il = (l > 0.f && m != -INFINITY) ? 1.0f / l : 0.f;
        if (il == 0.f) m = 0.f;
        D = a.rowDot[idx];
    }
}

template <int HD>
__global__ void __launch_bounds__(TC_THREADS) attn_bwd_dq_tc_kernel(TcAttnArgs a, int vec) {
    constexpr int ST = HD + 4;
    extern __shared__ __align__(16) uint32_t smu[];
    uint32_t* Qs = smu;           // Q then dO staging (reused), later K
    uint32_t* Ks = Qs + 64 * ST;
    uint32_t* Vs = Ks + 64 * ST;
    const AttnSeg sg = a.segs[blockIdx.z];
    const int q0 = blockIdx.x * 64;
    if (q0 >= sg.qLen) return;
    const int head = blockIdx.y, colOff = head * a.headDim, hd = a.headDim;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    uint32_t qa[HD / 8][4], da[HD / 8][4];
    stage_tile<HD, ST>(Qs, a.Q, a.ldq, sg.qStart + q0, min(64, sg.qLen - q0), colOff, hd, vec);
    __syncthreads();
    load_a_frags<HD, ST>(Qs, warp * 16, g, t, qa);
    __syncthreads();
    stage_tile<HD, ST>(Qs, a.dO, a.lddo, sg.qStart + q0, min(64, sg.qLen - q0), colOff, hd, vec);
    __syncthreads();
    load_a_frags<HD, ST>(Qs, warp * 16, g, t, da);
    float mrow[2], ilrow[2], drow[2];
#pragma unroll
    for (int h = 0; h < 2; h++) row_stats(a, sg, q0 + warp * 16 + g + 8 * h, head, mrow[h], ilrow[h], drow[h]);
    float dq[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; i++) dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f;
    const int kEnd = a.causal ? min(sg.kLen, q0 + 64) : sg.kLen;
    for (int k0 = 0; k0 < kEnd; k0 += 64) {
        __syncthreads();
        stage_tile<HD, ST>(Ks, a.K, a.ldk, sg.kStart + k0, min(64, sg.kLen - k0), colOff, hd, vec);
        stage_tile<HD, ST>(Vs, a.V, a.ldv, sg.kStart + k0, min(64, sg.kLen - k0), colOff, hd, vec);
        __syncthreads();
        float s[8][4], ds[8][4];
        recompute_tc<HD, ST>(a, sg, qa, da, Ks, Vs, mrow, ilrow, drow, q0 + warp * 16, k0, g, t, s, ds);
        uint32_t dsu[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) dsu[nt][e] = to_tf32(ds[nt][e]);
        mma_c_b<HD, ST>(dsu, Ks, g, t, dq);  // dQ += dS * K
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int qi = q0 + warp * 16 + g + 8 * h;
        if (qi >= sg.qLen) continue;
        const size_t row = (size_t)(sg.qStart + qi);
#pragma unroll
        for (int i = 0; i < HD / 8; i++) {
            const int c = i * 8 + 2 * t;
            if (c < hd) a.dQ[row * a.lddq + colOff + c] = dq[i][2 * h];
            if (c + 1 < hd) a.dQ[row * a.lddq + colOff + c + 1] = dq[i][2 * h + 1];
        }
    }
}

template <int HD>
__global__ void __launch_bounds__(TC_THREADS) attn_bwd_dkv_tc_kernel(TcAttnArgs a, int vec) {
    constexpr int STK = HD + 4;  // K, V: B operands indexed [key][hd]
    constexpr int STQ = HD + 8;  // Q, dO: A operands of the score products and B operands [q][hd] of the dK/dV products
    constexpr int STP = 72;      // P, dS [q][key], read transposed as A operands
    extern __shared__ __align__(16) uint32_t smu[];
    uint32_t* Ks = smu;
    uint32_t* Vs = Ks + 64 * STK;
    uint32_t* Qs = Vs + 64 * STK;
    uint32_t* dOs = Qs + 64 * STQ;
    uint32_t* Ps = dOs + 64 * STQ;
    uint32_t* dSs = Ps + 64 * STP;
    const AttnSeg sg = a.segs[blockIdx.z];
    const int k0 = blockIdx.x * 64;
    if (k0 >= sg.kLen) return;
    const int head = blockIdx.y, colOff = head * a.headDim, hd = a.headDim;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    stage_tile<HD, STK>(Ks, a.K, a.ldk, sg.kStart + k0, min(64, sg.kLen - k0), colOff, hd, vec);
    stage_tile<HD, STK>(Vs, a.V, a.ldv, sg.kStart + k0, min(64, sg.kLen - k0), colOff, hd, vec);
    float dk[HD / 8][4], dv[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; i++) {
        dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.f;
        dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.f;
    }
    const int qBegin = a.causal ? k0 : 0;
    for (int q0 = qBegin; q0 < sg.qLen; q0 += 64) {
        __syncthreads();
        stage_tile<HD, STQ>(Qs, a.Q, a.ldq, sg.qStart + q0, min(64, sg.qLen - q0), colOff, hd, vec);
        stage_tile<HD, STQ>(dOs, a.dO, a.lddo, sg.qStart + q0, min(64, sg.qLen - q0), colOff, hd, vec);
        __syncthreads();
        {
            uint32_t qa[HD / 8][4], da[HD / 8][4];
            load_a_frags<HD, STQ>(Qs, warp * 16, g, t, qa);
            load_a_frags<HD, STQ>(dOs, warp * 16, g, t, da);
            float mrow[2], ilrow[2], drow[2];
#pragma unroll
            for (int h = 0; h < 2; h++) row_stats(a, sg, q0 + warp * 16 + g + 8 * h, head, mrow[h], ilrow[h], drow[h]);
            float s[8][4], ds[8][4];
            recompute_tc<HD, STK>(a, sg, qa, da, Ks, Vs, mrow, ilrow, drow, q0 + warp * 16, k0, g, t, s, ds);
#pragma unroll
            for (int nt = 0; nt < 8; nt++)
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int r = warp * 16 + g + 8 * h, c = nt * 8 + 2 * t;
                    *reinterpret_cast<uint2*>(Ps + r * STP + c) = make_uint2(to_tf32(s[nt][2 * h]), to_tf32(s[nt][2 * h + 1]));
                    *reinterpret_cast<uint2*>(dSs + r * STP + c) = make_uint2(to_tf32(ds[nt][2 * h]), to_tf32(ds[nt][2 * h + 1]));
                }
        }
        __syncthreads();
        // dV[key, :] += sum_q P[q,key] dO[q,:]   and   dK[key, :] += sum_q dS[q,key] Q[q,:]   for this warp's 16 keys
        const int key0 = warp * 16;
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {  // 8 queries per step
            const uint32_t* pr = Ps + (ks * 8 + t) * STP + key0 + g;
            const uint32_t* sr = dSs + (ks * 8 + t) * STP + key0 + g;
            const uint32_t pa0 = pr[0], pa1 = pr[8], pa2 = pr[4 * STP], pa3 = pr[4 * STP + 8];
            const uint32_t sa0 = sr[0], sa1 = sr[8], sa2 = sr[4 * STP], sa3 = sr[4 * STP + 8];
#pragma unroll
            for (int n2 = 0; n2 < HD / 8; n2++) {
                const uint32_t b0 = dOs[(ks * 8 + t) * STQ + n2 * 8 + g], b1 = dOs[(ks * 8 + t + 4) * STQ + n2 * 8 + g];
                mma_tf32(dv[n2], pa0, pa1, pa2, pa3, b0, b1);
                const uint32_t c0 = Qs[(ks * 8 + t) * STQ + n2 * 8 + g], c1 = Qs[(ks * 8 + t + 4) * STQ + n2 * 8 + g];
                mma_tf32(dk[n2], sa0, sa1, sa2, sa3, c0, c1);
            }
        }
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int kj = k0 + warp * 16 + g + 8 * h;
        if (kj >= sg.kLen) continue;
        const size_t row = (size_t)(sg.kStart + kj);
#pragma unroll
        for (int i = 0; i < HD / 8; i++) {
            const int c = i * 8 + 2 * t;
            if (c < hd) { a.dK[row * a.lddk + colOff + c] = dk[i][2 * h]; a.dV[row * a.lddv + colOff + c] = dv[i][2 * h]; }
            if (c + 1 < hd) { a.dK[row * a.lddk + colOff + c + 1] = dk[i][2 * h + 1]; a.dV[row * a.lddv + colOff + c + 1] = dv[i][2 * h + 1]; }
        }
    }
}

// ------------------------------------------------------------------------------------------------ pipelined variants
// When the producer of Q, K, V and dO has already rounded them to TF32 (the resident trainer does: the Q/K/V projection
// and rotary kernels and the attention-output dX GEMM round on store), tiles need no conversion and are copied with
// cp.async into a two-deep ring, so the copy of tile i+1 overlaps the MMAs on tile i.
__device__ __forceinline__ void cp16(uint32_t* dst, const float* src, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int HD, int STRIDE>
__device__ __forceinline__ void copy_tile_async(uint32_t* __restrict__ dst, const float* __restrict__ src, int ld, int rowStart, int nValid,
                                                int colOff, int hd) {
    for (int idx = threadIdx.x; idx < 64 * (HD / 4); idx += TC_THREADS) {
        const int r = idx / (HD / 4), c = (idx - r * (HD / 4)) * 4;
        const bool ok = r < nValid && c < hd;
        cp16(dst + r * STRIDE + c, ok ? src + (size_t)(rowStart + r) * ld + colOff + c : src, ok);
    }
}

template <int HD>
__global__ void __launch_bounds__(TC_THREADS) attn_fwd_tc_pipe_kernel(TcAttnArgs a) {
    constexpr int ST = HD + 4, TILE = 64 * ST;
    extern __shared__ __align__(16) uint32_t smu[];
    uint32_t* Qs = smu;
    uint32_t* KV = Qs + TILE;  // ring: [buf][K | V]
    const AttnSeg sg = a.segs[blockIdx.z];
    const int q0 = blockIdx.x * 64;
    if (q0 >= sg.qLen) return;
    const int head = blockIdx.y, colOff = head * a.headDim, hd = a.headDim;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int kEnd = a.causal ? min(sg.kLen, q0 + 64) : sg.kLen;
    const int nTiles = (kEnd + 63) / 64;
    copy_tile_async<HD, ST>(Qs, a.Q, a.ldq, sg.qStart + q0, min(64, sg.qLen - q0), colOff, hd);
    if (nTiles > 0) {
        copy_tile_async<HD, ST>(KV, a.K, a.ldk, sg.kStart, min(64, sg.kLen), colOff, hd);
        copy_tile_async<HD, ST>(KV + TILE, a.V, a.ldv, sg.kStart, min(64, sg.kLen), colOff, hd);
    }
    cp_commit();
    float m_i[2] = {-INFINITY, -INFINITY}, l_i[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    uint32_t qa[HD / 8][4];
    const float sl2 = a.scale * LOG2E;
    for (int it = 0; it < nTiles; it++) {
        const int k0 = it * 64;
        uint32_t* Ks = KV + (it & 1) * 2 * TILE;
        uint32_t* Vs = Ks + TILE;
        if (it + 1 < nTiles) {  // prefetch the next tile into the other buffer (its last readers passed the barrier below)
            uint32_t* Kn = KV + ((it + 1) & 1) * 2 * TILE;
            copy_tile_async<HD, ST>(Kn, a.K, a.ldk, sg.kStart + k0 + 64, min(64, sg.kLen - k0 - 64), colOff, hd);
            copy_tile_async<HD, ST>(Kn + TILE, a.V, a.ldv, sg.kStart + k0 + 64, min(64, sg.kLen - k0 - 64), colOff, hd);
            cp_commit();
            cp_wait<1>();
        } else {
            cp_wait<0>();
        }
        __syncthreads();
        if (it == 0) load_a_frags<HD, ST>(Qs, warp * 16, g, t, qa);
        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; nt++) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
        mma_a_bt<HD, ST>(qa, Ks, g, t, s);
        uint32_t p[8][4];
        // a tile that no mask, sequence end or causal diagonal touches needs no per-element visibility test (warp-uniform)
        const bool full = !a.mask && k0 + 64 <= sg.kLen && q0 + warp * 16 + 16 <= sg.qLen && (!a.causal || k0 + 63 <= q0 + warp * 16);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int qi = q0 + warp * 16 + g + 8 * h;
            float mx = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 8; nt++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int kj = k0 + nt * 8 + 2 * t + e;
                    float v = (full || tc_visible(a, sg, qi, kj)) ? s[nt][2 * h + e] * sl2 : -INFINITY;  // scores in log2 units
                    s[nt][2 * h + e] = v;
                    mx = fmaxf(mx, v);
                }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_i[h], mx);
            const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;  // keeps (-inf) - (-inf) out of the exponent
            const float corr = fast_exp2(m_i[h] - m_safe);
            float rs = 0.f;
#pragma unroll
            for (int nt = 0; nt < 8; nt++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const float v = s[nt][2 * h + e];
                    const float pv = fast_exp2(v - m_safe);
                    rs += pv;
                    p[nt][2 * h + e] = to_tf32(pv);
                }
            rs += __shfl_xor_sync(0xffffffffu, rs, 1);
            rs += __shfl_xor_sync(0xffffffffu, rs, 2);
            l_i[h] = l_i[h] * corr + rs;
            m_i[h] = m_new;
#pragma unroll
            for (int i = 0; i < HD / 8; i++) { o[i][2 * h] *= corr; o[i][2 * h + 1] *= corr; }
        }
        mma_c_b<HD, ST>(p, Vs, g, t, o);
        __syncthreads();  // everyone is done with this buffer before the next iteration's prefetch overwrites it
    }
    cp_wait<0>();
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int qi = q0 + warp * 16 + g + 8 * h;
        if (qi >= sg.qLen) continue;
        const float inv = l_i[h] > 0.f ? 1.0f / l_i[h] : 0.f;
        const size_t row = (size_t)(sg.qStart + qi);
#pragma unroll
        for (int i = 0; i < HD / 8; i++) {
            const int c = i * 8 + 2 * t;  // hd is a multiple of 4 on this path, so c+1 < hd whenever c < hd
            if (c < hd) *reinterpret_cast<float2*>(a.Oout + row * a.ldo + colOff + c) = make_float2(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
        }
        if (t == 0 && a.rowMax) {
            a.rowMax[row * a.numHeads + head] = m_i[h] == -INFINITY ? -INFINITY : m_i[h] / LOG2E;
            a.rowSum[row * a.numHeads + head] = l_i[h];
        }
    }
}

template <int HD>
__global__ void __launch_bounds__(TC_THREADS) attn_bwd_dq_tc_pipe_kernel(TcAttnArgs a) {
    constexpr int ST = HD + 4, TILE = 64 * ST;
    extern __shared__ __align__(16) uint32_t smu[];
    uint32_t* Qs = smu;
    uint32_t* dOs = Qs + TILE;
    uint32_t* KV = dOs + TILE;
    const AttnSeg sg = a.segs[blockIdx.z];
    const int q0 = blockIdx.x * 64;
    if (q0 >= sg.qLen) return;
    const int head = blockIdx.y, colOff = head * a.headDim, hd = a.headDim;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int kEnd = a.causal ? min(sg.kLen, q0 + 64) : sg.kLen;
    const int nTiles = (kEnd + 63) / 64;
    copy_tile_async<HD, ST>(Qs, a.Q, a.ldq, sg.qStart + q0, min(64, sg.qLen - q0), colOff, hd);
    copy_tile_async<HD, ST>(dOs, a.dO, a.lddo, sg.qStart + q0, min(64, sg.qLen - q0), colOff, hd);
    if (nTiles > 0) {
        copy_tile_async<HD, ST>(KV, a.K, a.ldk, sg.kStart, min(64, sg.kLen), colOff, hd);
        copy_tile_async<HD, ST>(KV + TILE, a.V, a.ldv, sg.kStart, min(64, sg.kLen), colOff, hd);
    }
    cp_commit();
    float mrow[2], ilrow[2], drow[2];
#pragma unroll
    for (int h = 0; h < 2; h++) row_stats(a, sg, q0 + warp * 16 + g + 8 * h, head, mrow[h], ilrow[h], drow[h]);
    float dq[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; i++) dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f;
    uint32_t qa[HD / 8][4], da[HD / 8][4];
    for (int it = 0; it < nTiles; it++) {
        const int k0 = it * 64;
        uint32_t* Ks = KV + (it & 1) * 2 * TILE;
        uint32_t* Vs = Ks + TILE;
        if (it + 1 < nTiles) {
            uint32_t* Kn = KV + ((it + 1) & 1) * 2 * TILE;
            copy_tile_async<HD, ST>(Kn, a.K, a.ldk, sg.kStart + k0 + 64, min(64, sg.kLen - k0 - 64), colOff, hd);
            copy_tile_async<HD, ST>(Kn + TILE, a.V, a.ldv, sg.kStart + k0 + 64, min(64, sg.kLen - k0 - 64), colOff, hd);
            cp_commit();
            cp_wait<1>();
        } else {
            cp_wait<0>();
        }
        __syncthreads();
        if (it == 0) {
            load_a_frags<HD, ST>(Qs, warp * 16, g, t, qa);
            load_a_frags<HD, ST>(dOs, warp * 16, g, t, da);
        }
        float s[8][4], ds[8][4];
        recompute_tc<HD, ST>(a, sg, qa, da, Ks, Vs, mrow, ilrow, drow, q0 + warp * 16, k0, g, t, s, ds);
        uint32_t dsu[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) dsu[nt][e] = to_tf32(ds[nt][e]);
        mma_c_b<HD, ST>(dsu, Ks, g, t, dq);
        __syncthreads();
    }
    cp_wait<0>();
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int qi = q0 + warp * 16 + g + 8 * h;
        if (qi >= sg.qLen) continue;
        const size_t row = (size_t)(sg.qStart + qi);
#pragma unroll
        for (int i = 0; i < HD / 8; i++) {
            const int c = i * 8 + 2 * t;
            if (c < hd) *reinterpret_cast<float2*>(a.dQ + row * a.lddq + colOff + c) = make_float2(dq[i][2 * h], dq[i][2 * h + 1]);
        }
    }
}

__global__ void attn_rowdot_tc_kernel(const float* __restrict__ dO, int lddo, const float* __restrict__ O, int ldo, int rows, int numHeads, int hd,
                                      float* __restrict__ rowDot) {
    int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (w >= rows * numHeads) return;
    int row = w / numHeads, head = w - row * numHeads;
    float s = 0.f;
    for (int c = lane; c < hd; c += 32) s += dO[(size_t)row * lddo + head * hd + c] * O[(size_t)row * ldo + head * hd + c];
    s = warp_sum(s);
    if (lane == 0) rowDot[w] = s;
}

TcAttnArgs make_tc_args(const Attn& t) {
    TcAttnArgs a;
    a.Q = t.Q; a.K = t.K; a.V = t.V; a.dO = t.dO; a.O = t.O;
    a.ldq = t.ldq; a.ldk = t.ldk; a.ldv = t.ldv; a.lddo = t.lddo; a.ldo = t.ldo;
    a.Oout = t.O; a.dQ = t.dQ; a.dK = t.dK; a.dV = t.dV; a.lddq = t.lddq; a.lddk = t.lddk; a.lddv = t.lddv;
    a.rowMax = t.rowMax; a.rowSum = t.rowSum; a.rowDot = t.rowDot;
    a.segs = t.segs_dev; a.mask = t.mask; a.numHeads = t.numHeads; a.headDim = t.headDim; a.causal = t.causal; a.scale = t.scale;
    return a;
}

bool vec_ok(const Attn& t, bool bwd) {
    auto ok = [](const void* p, int ld) { return (((uintptr_t)p) & 15) == 0 && (ld & 3) == 0; };
    bool v = (t.headDim % 4 == 0) && ok(t.Q, t.ldq) && ok(t.K, t.ldk) && ok(t.V, t.ldv);
    if (bwd) v = v && ok(t.dO, t.lddo);
    return v;
}

template <int HD>
int launch_fwd_tc(b200_ctx* ctx, const Attn& t) {
    constexpr size_t smem = (size_t)3 * 64 * (HD + 4) * 4;
    static char configured_site;
    if (first_use(ctx, &configured_site)) {
        B200_CUDA(ctx, cudaFuncSetAttribute(attn_fwd_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    }
    dim3 grid((t.maxQLen + 63) / 64, t.numHeads, t.nSeg);
    if (t.pre_rounded && vec_ok(t, false) && (t.ldo % 2 == 0) && (((uintptr_t)t.O & 7) == 0)) {
        constexpr size_t smem_pipe = (size_t)5 * 64 * (HD + 4) * 4;
        static char configured_pipe_site;
        if (first_use(ctx, &configured_pipe_site)) {
            B200_CUDA(ctx, cudaFuncSetAttribute(attn_fwd_tc_pipe_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_pipe));
        }
        attn_fwd_tc_pipe_kernel<HD><<<grid, TC_THREADS, smem_pipe, ctx->stream>>>(make_tc_args(t));
        B200_LAUNCH_CHECK(ctx);
        return B200_OK;
    }
    attn_fwd_tc_kernel<HD><<<grid, TC_THREADS, smem, ctx->stream>>>(make_tc_args(t), vec_ok(t, false) ? 1 : 0);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

template <int HD>
int launch_bwd_tc(b200_ctx* ctx, const Attn& t) {
    constexpr size_t smem_dq = (size_t)3 * 64 * (HD + 4) * 4;
    constexpr size_t smem_dkv = (size_t)(2 * 64 * (HD + 4) + 2 * 64 * (HD + 8) + 2 * 64 * 72) * 4;
    static char configured_site;
    if (first_use(ctx, &configured_site)) {
        B200_CUDA(ctx, cudaFuncSetAttribute(attn_bwd_dq_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dq));
        B200_CUDA(ctx, cudaFuncSetAttribute(attn_bwd_dkv_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dkv));
    }
    TcAttnArgs a = make_tc_args(t);
    const int vec = vec_ok(t, true) ? 1 : 0;
    int warps = t.totalQ * t.numHeads;
    attn_rowdot_tc_kernel<<<(warps * 32 + 255) / 256, 256, 0, ctx->stream>>>(t.dO, t.lddo, t.O, t.ldo, t.totalQ, t.numHeads, t.headDim, t.rowDot);
    B200_LAUNCH_CHECK(ctx);
    dim3 gk((t.maxKLen + 63) / 64, t.numHeads, t.nSeg);
    attn_bwd_dkv_tc_kernel<HD><<<gk, TC_THREADS, smem_dkv, ctx->stream>>>(a, vec);
    B200_LAUNCH_CHECK(ctx);
    dim3 gq((t.maxQLen + 63) / 64, t.numHeads, t.nSeg);
    if (t.pre_rounded && vec && (t.lddq % 2 == 0) && (((uintptr_t)t.dQ & 7) == 0)) {
        constexpr size_t smem_pipe = (size_t)6 * 64 * (HD + 4) * 4;
        static char configured_pipe_site;
        if (first_use(ctx, &configured_pipe_site)) {
            B200_CUDA(ctx, cudaFuncSetAttribute(attn_bwd_dq_tc_pipe_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_pipe));
        }
        attn_bwd_dq_tc_pipe_kernel<HD><<<gq, TC_THREADS, smem_pipe, ctx->stream>>>(a);
        B200_LAUNCH_CHECK(ctx);
        return B200_OK;
    }
    attn_bwd_dq_tc_kernel<HD><<<gq, TC_THREADS, smem_dq, ctx->stream>>>(a, vec);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

}  // namespace

// The automatic mode keeps models narrower than 128 on the FP32 kernels (their projections run on the FP32 SIMT GEMM
// as well, so the whole step holds the FP32 tolerance); forcing the tensor-core mode takes every head dim 8..64.
bool attn_tc_eligible(b200_ctx* ctx, const Attn& t) {
    if (ctx->gemm_mode == B200_GEMM_FP32_SIMT || ctx->cc_major < 8 || t.headDim < 8 || t.headDim > 64 || t.maxQLen < 32) return false;
    return ctx->gemm_mode == B200_GEMM_TF32_TCGEN05 || t.numHeads * t.headDim >= 128;
}

int attn_forward_tc(b200_ctx* ctx, const Attn& t) {
    if (attn_umma_eligible(ctx, t)) { ctx->engine_launches[B200_ENGINE_ATTN_TCGEN05]++; return attn_forward_umma(ctx, t); }
    ctx->engine_launches[B200_ENGINE_ATTN_MMA_SYNC]++;
    if (t.headDim <= 16) return launch_fwd_tc<16>(ctx, t);
    if (t.headDim <= 32) return launch_fwd_tc<32>(ctx, t);
    return launch_fwd_tc<64>(ctx, t);
}
int attn_backward_tc(b200_ctx* ctx, const Attn& t) {
    if (attn_umma_bwd_eligible(ctx, t)) { ctx->engine_launches[B200_ENGINE_ATTN_TCGEN05]++; return attn_backward_umma(ctx, t); }
    ctx->engine_launches[B200_ENGINE_ATTN_MMA_SYNC]++;
    if (t.headDim <= 16) return launch_bwd_tc<16>(ctx, t);
    if (t.headDim <= 32) return launch_bwd_tc<32>(ctx, t);
    return launch_bwd_tc<64>(ctx, t);
}

}  // namespace b200
