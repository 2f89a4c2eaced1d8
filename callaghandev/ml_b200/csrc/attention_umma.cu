// Attention on the fifth-generation tensor cores (tcgen05.mma.kind::tf32, accumulators in tensor memory) for head
// dimension 64: the engine the TF32 mode uses on sm_100a when no explicit mask is given.  Same algorithm and the
// same saved statistics (row max in natural-log units, row sum) as the other attention engines.
//
// Forward.  A CTA owns 128 query rows of one (segment, head) and walks the key tiles (128 keys each) it can see:
//   S  = Q K^T          tcgen05.mma, both operands K-major in shared memory (TMA, 128-byte swizzle), S in TMEM columns 0..127
//   P  = softmax tile   128 threads, one query row each: tcgen05.ld -> max / exp2 / sum -> tcgen05.st back over S
//   O += P V            tcgen05.mma with the A operand read from TMEM (P) and V as an N-contiguous shared-memory
//                       operand (TMA, 128-byte swizzle with 32-byte atoms), O in TMEM columns 128..191
// Warp roles: warp 0 = TMA producer, warp 1 = TMEM allocator and MMA issuer, warps 2..5 = softmax / output.  K and V
// are single-buffered with separate barriers, so the load of K(j+1) overlaps softmax(j) and P V(j), and V(j+1)
// overlaps S(j+1); two CTAs share an SM (96 KiB of tiles, 256 TMEM columns each) and fill each other's gaps.
// Rows of a packed batch that lie outside the segment are loaded (they are finite: other segments' rows, or zeros
// beyond the tensor) and masked to -inf before the exponent; they are never stored.
//
// Every mbarrier wait is bounded (see mbar_wait); on expiry the roles stop, the status word is raised, and the CTA
// frees its TMEM and returns.
#include <cstdlib>

#include "device_math.cuh"
#include "tcgen05.cuh"

namespace b200 {

namespace {

constexpr int UQ = 128, UK = 128, UHD = 64;
constexpr int U_ATOM = 128 * 128;     // bytes of one 128-row x 32-float swizzle atom column
constexpr int U_TILE = 2 * U_ATOM;    // a 128 x 64 operand tile
constexpr int U_THREADS = 192;
constexpr int S_COL = 0, O_COL = 128, FWD_TMEM_COLS = 256;
constexpr int FWD_SMEM = 3 * U_TILE + 1024 + 256;
constexpr int OUT_STRIDE = 68;        // floats per staged output row (16-byte aligned, conflict-free 128-bit accesses)
constexpr float LOG2E_F = 1.4426950408889634f;

struct UArgs {
    float* O; int ldo;
    float *rowMax, *rowSum;
    const AttnSeg* segs;
    int numHeads, causal;
    float scale;
    int* status;
};

__device__ __forceinline__ uint32_t idesc_tf32(uint32_t M, uint32_t N, uint32_t a_mn, uint32_t b_mn) {
    return (1u << 4) | (2u << 7) | (2u << 10) | (a_mn << 15) | (b_mn << 16) | ((N >> 3) << 17) | ((M >> 4) << 24);
}
// K-contiguous 128 x 64 tile (two swizzle atoms side by side): descriptor of K step kk (8 floats = 32 bytes)
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t tile, int kk) { return umma_desc(tile + (kk >> 2) * U_ATOM + (kk & 3) * 32, 16, 1024, 2); }
// N-contiguous [128 K rows][64 N] tile stored as two 32-column chunks: descriptor of K step kk (8 rows = 1024 bytes)
__device__ __forceinline__ uint64_t nmajor_desc(uint32_t tile, int kk) { return umma_desc(tile + kk * 1024, U_ATOM, 512, 1); }

__device__ __forceinline__ float ex2(float x) {  // 2^x; -inf gives +0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t rna_tf32(float x) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
    return u;
}

__global__ void __launch_bounds__(U_THREADS) attn_fwd_umma_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                                                                 const __grid_constant__ CUtensorMap mapV, UArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const AttnSeg sg = a.segs[blockIdx.z];
    const int head = blockIdx.y;
    const int q0 = (gridDim.x - 1 - blockIdx.x) * UQ;  // longest causal rows first
    if (q0 >= sg.qLen) return;
    const int kEnd = a.causal ? min(sg.kLen, q0 + UQ) : sg.kLen;
    const int nkt = (kEnd + UK - 1) / UK;
    if (nkt == 0) {  // no keys at all: zero output, empty statistics
        for (int idx = threadIdx.x; idx < UQ * (UHD / 4); idx += U_THREADS) {
            const int r = idx / (UHD / 4), c = (idx % (UHD / 4)) * 4;
            if (q0 + r < sg.qLen) *reinterpret_cast<float4*>(a.O + (size_t)(sg.qStart + q0 + r) * a.ldo + head * UHD + c) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (threadIdx.x < UQ && q0 + threadIdx.x < sg.qLen) {
            const size_t idx = (size_t)(sg.qStart + q0 + threadIdx.x) * a.numHeads + head;
            a.rowMax[idx] = -INFINITY;
            a.rowSum[idx] = 0.f;
        }
        return;
    }
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(tiles + 3 * U_TILE);
    uint32_t* tmem_slot = (uint32_t*)(bars + 8);
    const uint32_t Qs = smem_u32(tiles), Ks = Qs + U_TILE, Vs = Ks + U_TILE;
    const uint32_t bar0 = smem_u32(bars);
    const uint32_t q_full = bar0, k_full = bar0 + 8, k_empty = bar0 + 16, v_full = bar0 + 24, v_empty = bar0 + 32, s_full = bar0 + 40,
                   p_full = bar0 + 48, o_full = bar0 + 56;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* status = a.status;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 8; i++) mbar_init(bar0 + 8 * i, i == 6 ? 128 : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(FWD_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ---------------------------------------------------------------------------------- TMA producer
            const int col = head * UHD;
            mbar_expect_tx(q_full, U_TILE);
            tma_load_2d(Qs, &mapQ, q_full, col, sg.qStart + q0);
            tma_load_2d(Qs + U_ATOM, &mapQ, q_full, col + 32, sg.qStart + q0);
            bool ok = true;
            int kIssued = 0, vIssued = 0;
            for (int j = 0; j < nkt; j++) {
                const int row = sg.kStart + j * UK;
                ok = mbar_wait(k_empty, (j & 1) ^ 1, status, 11);
                if (!ok) break;
                mbar_expect_tx(k_full, U_TILE);
                tma_load_2d(Ks, &mapK, k_full, col, row);
                tma_load_2d(Ks + U_ATOM, &mapK, k_full, col + 32, row);
                kIssued = j + 1;
                ok = mbar_wait(v_empty, (j & 1) ^ 1, status, 12);
                if (!ok) break;
                mbar_expect_tx(v_full, U_TILE);
                tma_load_2d(Vs, &mapV, v_full, col, row);
                tma_load_2d(Vs + U_ATOM, &mapV, v_full, col + 32, row);
                vIssued = j + 1;
            }
            if (!ok) {  // failure path: let the copies already issued land (bounded) before the CTA may exit
                const long long t0 = clock64();
                while (!mbar_test(q_full, 0) && clock64() - t0 < WAIT_BUDGET_CLOCKS) __nanosleep(64);
                while (kIssued > 0 && !mbar_test(k_full, (kIssued - 1) & 1) && clock64() - t0 < WAIT_BUDGET_CLOCKS) __nanosleep(64);
                while (vIssued > 0 && !mbar_test(v_full, (vIssued - 1) & 1) && clock64() - t0 < WAIT_BUDGET_CLOCKS) __nanosleep(64);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------------------------------------------------------------------------- MMA issuer
            const uint32_t idS = idesc_tf32(UQ, UK, 0, 0), idO = idesc_tf32(UQ, UHD, 0, 1);
            bool ok = mbar_wait(q_full, 0, status, 13);
            for (int j = 0; j < nkt && ok; j++) {
                ok = mbar_wait(k_full, j & 1, status, 14);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < UHD / 8; kk++) umma_tf32(tmem_base + S_COL, kmajor_desc(Qs, kk), kmajor_desc(Ks, kk), idS, kk > 0 ? 1u : 0u);
                umma_commit(k_empty);
                umma_commit(s_full);
                ok = mbar_wait(p_full, j & 1, status, 15);
                if (!ok) break;
                ok = mbar_wait(v_full, j & 1, status, 16);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < UK / 8; kk++)
                    umma_tf32_ta(tmem_base + O_COL, tmem_base + S_COL + kk * 8, nmajor_desc(Vs, kk), idO, (j > 0 || kk > 0) ? 1u : 0u);
                umma_commit(v_empty);
            }
            umma_commit(o_full);
        }
    } else {
        // -------------------------------------------------------------------------------------- softmax and output
        const int quarter = warp & 3;  // TMEM lanes [32*quarter, +32)
        const int row = 32 * quarter + lane, qi = q0 + row;
        const uint32_t tlane = tmem_base + ((uint32_t)(32 * quarter) << 16);
        const float sl2 = a.scale * LOG2E_F;
        const int lim = a.causal ? min(sg.kLen, qi + 1) : sg.kLen;  // keys [0, lim) are visible to this row
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < nkt; j++) {
            ok = mbar_wait(s_full, j & 1, status, 17);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int k0 = j * UK;
            const bool full = k0 + UK <= sg.kLen && (!a.causal || k0 + UK - 1 <= q0 + 32 * quarter);  // warp-uniform
            const int nvis = lim - k0;  // columns [0, nvis) of this tile are visible
            float mx = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < UK; c += 32) {
                uint32_t r[32];
                tmem_ld32(tlane + S_COL + c, r);
                if (full) {
#pragma unroll
                    for (int i = 0; i < 32; i++) mx = fmaxf(mx, __uint_as_float(r[i]));
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++) mx = fmaxf(mx, (c + i < nvis) ? __uint_as_float(r[i]) : -INFINITY);
                }
            }
            const float m_new = fmaxf(m, mx * sl2);  // scale > 0, so the maximum commutes with the scaling
            const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
            const float corr = ex2(m - m_safe);
            float rs = 0.f;
#pragma unroll 1
            for (int c = 0; c < UK; c += 32) {
                uint32_t r[32];
                tmem_ld32(tlane + S_COL + c, r);
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    float v = fmaf(__uint_as_float(r[i]), sl2, -m_safe);
                    if (!full && c + i >= nvis) v = -INFINITY;
                    const float p = ex2(v);
                    rs += p;
                    r[i] = rna_tf32(p);
                }
                tmem_st32(tlane + S_COL + c, r);
            }
            l = l * corr + rs;
            m = m_new;
            if (j > 0 && __any_sync(0xffffffffu, corr != 1.f)) {  // S(j) complete implies P V(j-1) complete: O is stable
#pragma unroll 1
                for (int c = 0; c < UHD; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(tlane + O_COL + c, r);
#pragma unroll
                    for (int i = 0; i < 32; i++) r[i] = __float_as_uint(__uint_as_float(r[i]) * corr);
                    tmem_st32(tlane + O_COL + c, r);
                }
            }
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(p_full);
        }
        if (ok) {
            ok = mbar_wait(o_full, 0, status, 18);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok) {
            tc_fence_after();
            // every MMA has completed, so the operand tiles are free: stage this warp's 32 rows and store whole rows
            float* stage = reinterpret_cast<float*>(tiles) + quarter * (32 * OUT_STRIDE);
            const float il = l > 0.f ? 1.f / l : 0.f;
#pragma unroll 1
            for (int c = 0; c < UHD; c += 32) {
                uint32_t r[32];
                tmem_ld32(tlane + O_COL + c, r);
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                    *reinterpret_cast<float4*>(stage + lane * OUT_STRIDE + c + i) =
                        make_float4(__uint_as_float(r[i]) * il, __uint_as_float(r[i + 1]) * il, __uint_as_float(r[i + 2]) * il, __uint_as_float(r[i + 3]) * il);
            }
            if (qi < sg.qLen) {
                const size_t idx = (size_t)(sg.qStart + qi) * a.numHeads + head;
                a.rowMax[idx] = (m == -INFINITY) ? -INFINITY : m / LOG2E_F;
                a.rowSum[idx] = l;
            }
            __syncwarp();
            const int sub = lane >> 4, c4 = (lane & 15) * 4;
#pragma unroll 4
            for (int rr = 0; rr < 32; rr += 2) {
                const int r = rr + sub;
                if (q0 + 32 * quarter + r < sg.qLen)
                    *reinterpret_cast<float4*>(a.O + (size_t)(sg.qStart + q0 + 32 * quarter + r) * a.ldo + head * UHD + c4) =
                        *reinterpret_cast<const float4*>(stage + r * OUT_STRIDE + c4);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(FWD_TMEM_COLS) : "memory");
    }
}

bool umma_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("B200_ATTN_UMMA");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

}  // namespace

bool attn_umma_eligible(b200_ctx* ctx, const Attn& t) {
    auto ok = [](const void* p, int ld) { return (((uintptr_t)p) & 15) == 0 && (ld & 3) == 0; };
    return umma_enabled() && ctx->cc_major == 10 && ctx->gemm_mode != B200_GEMM_FP32_SIMT && t.headDim == UHD && !t.mask && t.rowMax && t.rowSum && t.scale > 0.f &&
           t.maxQLen >= 128 && t.totalQ >= 128 && t.totalK >= 128 && ok(t.Q, t.ldq) && ok(t.K, t.ldk) && ok(t.V, t.ldv) && ok(t.O, t.ldo);
}

int attn_forward_umma(b200_ctx* ctx, const Attn& t) {
    B200_TRY(resolve_encode(ctx));
    B200_TRY(ensure_status(ctx));
    if (!ctx->attn_umma_configured) {
        B200_CUDA(ctx, cudaFuncSetAttribute(attn_fwd_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM));
        ctx->attn_umma_configured = 1;
    }
    const uint64_t cols = (uint64_t)t.numHeads * UHD;
    CUtensorMap mq, mk, mv;
    B200_TRY(make_map(ctx, &mq, t.Q, cols, (uint64_t)t.totalQ, (uint64_t)t.ldq, 128, false));
    B200_TRY(make_map(ctx, &mk, t.K, cols, (uint64_t)t.totalK, (uint64_t)t.ldk, 128, false));
    B200_TRY(make_map(ctx, &mv, t.V, cols, (uint64_t)t.totalK, (uint64_t)t.ldv, 128, true));
    UArgs a;
    a.O = t.O; a.ldo = t.ldo; a.rowMax = t.rowMax; a.rowSum = t.rowSum; a.segs = t.segs_dev; a.numHeads = t.numHeads; a.causal = t.causal;
    a.scale = t.scale; a.status = ctx->status_dev;
    dim3 grid((t.maxQLen + UQ - 1) / UQ, t.numHeads, t.nSeg);
    attn_fwd_umma_kernel<<<grid, U_THREADS, FWD_SMEM, ctx->stream>>>(mq, mk, mv, a);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

}  // namespace b200
