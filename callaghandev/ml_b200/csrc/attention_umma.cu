// Attention on the fifth-generation tensor cores (tcgen05.mma.kind::tf32, accumulators in tensor memory) for head
// dimension 64: the engine the TF32 mode uses on sm_100a when no explicit mask is given.  Same algorithm and the
// same saved statistics (row max in natural-log units, row sum) as the other attention engines.
//
// Forward.  A CTA owns 128 query rows of one (segment, head) and walks the key tiles (128 keys each) it can see:
//   S  = Q K^T          tcgen05.mma, both operands K-major in shared memory (TMA, 128-byte swizzle), S in TMEM columns 0..127
//   P  = softmax tile   256 threads, two per query row (64 columns each; the row maximum crosses through shared memory, the row
//                       sum stays split until the end): tcgen05.ld -> max / exp2 / sum -> tcgen05.st back over S
//   O += P V            tcgen05.mma with the A operand read from TMEM (P) and V as an N-contiguous shared-memory
//                       operand (TMA, 128-byte swizzle with 32-byte atoms), O in TMEM columns 128..191
// Warp roles: warp 0 = TMA producer, warp 1 = TMEM allocator and MMA issuer, warps 2..9 = softmax / output.  K and V
// are single-buffered with separate barriers, so the load of K(j+1) overlaps softmax(j) and P V(j), and V(j+1)
// overlaps S(j+1); two CTAs share an SM (96 KiB of tiles, 256 TMEM columns each) and fill each other's gaps.
// Rows of a packed batch that lie outside the segment are loaded (they are finite: other segments' rows, or zeros
// beyond the tensor) and masked to -inf before the exponent; they are never stored.
//
// Every mbarrier wait is bounded (see mbar_wait); on expiry the roles stop, the status word is raised, and the CTA
// frees its TMEM and returns.
#include <algorithm>
#include <cstdlib>
#include <type_traits>

#include "device_math.cuh"
#include "tcgen05.cuh"

namespace b200 {

namespace {

constexpr int UQ = 128, UK = 128, UHD = 64;
constexpr int U_ATOM = 128 * 128;     // bytes of one 128-row x 32-float swizzle atom column
constexpr int U_TILE = 2 * U_ATOM;    // a 128 x 64 operand tile
constexpr int U_THREADS = 64 + 256;  // producer warp, MMA warp, eight softmax warps (lane quarter x column half)
constexpr int S_COL = 0, O_COL = 128, FWD_TMEM_COLS = 256;
constexpr int FWD_SMEM = 3 * U_TILE + 1024 + 256 + 3 * 2 * 128 * 4;  // + row statistics exchanged between the two halves of a row
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
// Descriptors are built once per kernel; inside the loops a K step or a ring slot is a constant added to the address
// field (the MMA warp is a single thread, so every instruction it spends on descriptor arithmetic delays the pipe).
__host__ __device__ constexpr uint64_t koff(int kk, int atom) { return (uint64_t)(((kk >> 2) * atom + (kk & 3) * 32) >> 4); }
__host__ __device__ constexpr uint64_t noff(int kk) { return (uint64_t)((kk * 1024) >> 4); }
// K-contiguous 128 x 64 tile (two swizzle atoms side by side): descriptor of K step kk (8 floats = 32 bytes)
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t tile, int kk) { return umma_desc(tile + (kk >> 2) * U_ATOM + (kk & 3) * 32, 16, 1024, 2); }
// N-contiguous [128 K rows][64 N] tile stored as two 32-column chunks: descriptor of K step kk (8 rows = 1024 bytes)
__device__ __forceinline__ uint64_t nmajor_desc(uint32_t tile, int kk) { return umma_desc(tile + kk * 1024, U_ATOM, 512, 1); }

__device__ __forceinline__ float ex2(float x) {  // 2^x; -inf gives +0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Packed FP32 pairs (one instruction for two lanes of arithmetic): the element-wise step is bound by instruction issue.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\tfma.rn.f32x2 rd, ra, rb, rc;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tadd.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmul.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}
// Round-to-nearest into the TF32 mantissa by adding half an ulp; the MMA ignores the 13 low bits that remain.
__device__ __forceinline__ uint32_t rna_tf32_add(float x) { return __float_as_uint(x) + 0x1000u; }

// Round to TF32 (nearest, ties away from zero) with integer instructions: the conversion instruction shares the
// transcendental pipe with ex2, which is the scarce resource of the element-wise step.
__device__ __forceinline__ uint32_t rna_tf32(float x) { return (__float_as_uint(x) + 0x1000u) & 0xffffe000u; }

// Copy half a row of a K-contiguous swizzle atom (16 floats, already TF32; h = which half) into TMEM columns [col, col+16)
// of the calling thread's lane, so the tile can serve as the A operand of tcgen05.mma from tensor memory: an A operand
// read from shared memory costs 4 KiB of shared-memory bandwidth per K step, which is what bounds TF32 MMAs with a narrow N.
__device__ __forceinline__ void half_row_to_tmem(const uint8_t* atom, int row, int h, uint32_t taddr) {
    uint32_t r[16];
#pragma unroll
    for (int c = 0; c < 4; c++) {
        const uint4 v = *reinterpret_cast<const uint4*>(atom + row * 128 + (((4 * h + c) ^ (row & 7)) << 4));
        r[4 * c] = v.x; r[4 * c + 1] = v.y; r[4 * c + 2] = v.z; r[4 * c + 3] = v.w;
    }
    tmem_st16(taddr, r);
}

// Named barrier of the forward kernel's 256 softmax threads, plain and with an OR vote.
__device__ __forceinline__ void sm_barrier() { asm volatile("bar.sync 2, 256;" ::: "memory"); }
__device__ __forceinline__ bool sm_barrier_or(bool pred) {
    uint32_t r;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %1, 0;\n\tbar.red.or.pred q, 2, 256, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                 : "=r"(r)
                 : "r"((uint32_t)pred)
                 : "memory");
    return r != 0;
}

__global__ void __launch_bounds__(U_THREADS, 2) attn_fwd_umma_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
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
    float* xch = reinterpret_cast<float*>(bars + 16);  // [3][2 halves][128 rows]: tile maxima (two buffers, alternating) and final sums
    const uint32_t Qs = smem_u32(tiles), Ks = Qs + U_TILE, Vs = Ks + U_TILE;
    const uint32_t bar0 = smem_u32(bars);
    const uint32_t q_full = bar0, k_full = bar0 + 8, k_empty = bar0 + 16, v_full = bar0 + 24, v_empty = bar0 + 32, s_full = bar0 + 40,
                   p_full = bar0 + 48, o_full = bar0 + 56;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* status = a.status;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 8; i++) mbar_init(bar0 + 8 * i, i == 6 ? 8 : 1);  // p_full: one arrival per softmax warp
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // Q is requested right away: its latency overlaps the TMEM allocation and the first sync.
        mbar_expect_tx(q_full, U_TILE);
        tma_load_3d(Qs, &mapQ, q_full, 0, sg.qStart + q0, head * (UHD / 32));
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
            bool ok = true;
            int kIssued = 0, vIssued = 0;
            for (int j = 0; j < nkt; j++) {
                const int row = sg.kStart + j * UK;
                ok = mbar_wait(k_empty, (j & 1) ^ 1, status, 11);
                if (!ok) break;
                mbar_expect_tx(k_full, U_TILE);
                tma_load_3d(Ks, &mapK, k_full, 0, row, col >> 5);
                kIssued = j + 1;
                ok = mbar_wait(v_empty, (j & 1) ^ 1, status, 12);
                if (!ok) break;
                mbar_expect_tx(v_full, U_TILE);
                tma_load_3d(Vs, &mapV, v_full, 0, row, col >> 5);
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
            const uint64_t dQ0 = kmajor_desc(Qs, 0), dK0 = kmajor_desc(Ks, 0), dV0 = nmajor_desc(Vs, 0);
            bool ok = mbar_wait(q_full, 0, status, 13);
            for (int j = 0; j < nkt && ok; j++) {
                ok = mbar_wait(k_full, j & 1, status, 14);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < UHD / 8; kk++) umma_tf32(tmem_base + S_COL, dQ0 + koff(kk, U_ATOM), dK0 + koff(kk, U_ATOM), idS, kk > 0 ? 1u : 0u);
                umma_commit(k_empty);
                umma_commit(s_full);
                ok = mbar_wait(p_full, j & 1, status, 15);
                if (!ok) break;
                ok = mbar_wait(v_full, j & 1, status, 16);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < UK / 8; kk++)
                    umma_tf32_ta(tmem_base + O_COL, tmem_base + S_COL + kk * 8, dV0 + noff(kk), idO, (j > 0 || kk > 0) ? 1u : 0u);
                umma_commit(v_empty);
            }
            umma_commit(o_full);
        }
    } else {
        // -------------------------------------------------------------------------------------- softmax and output
        // Two threads per query row, 64 score columns each (a thread alone walks a chain of 128 max / exp / add steps per
        // tile, and with one warp per scheduler nothing hides it).  The halves agree on the row maximum through shared
        // memory once per tile; each keeps its own partial row sum, which the correction factor scales alike.
        const int quarter = warp & 3, half = (warp - 2) >> 2, c0 = 64 * half;  // TMEM lanes [32*quarter, +32), columns [c0, +64)
        const int row = 32 * quarter + lane, qi = q0 + row;
        const uint32_t tlane = tmem_base + ((uint32_t)(32 * quarter) << 16);
        const float sl2 = a.scale * LOG2E_F;
        const int lim = a.causal ? min(sg.kLen, qi + 1) : sg.kLen;  // keys [0, lim) are visible to this row
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < nkt; j++) {
            ok = mbar_wait_warp(s_full, j & 1, status, 17);
            ok = __all_sync(0xffffffffu, ok);
            if (sm_barrier_or(!ok)) {  // also orders the previous tile's reads of the exchange buffer before its reuse two tiles on
                ok = false;
                break;
            }
            tc_fence_after();
            const int k0 = j * UK + c0;
            const bool full = k0 + 64 <= sg.kLen && (!a.causal || k0 + 63 <= q0 + 32 * quarter);  // warp-uniform
            const int nvis = lim - k0;  // columns [0, nvis) of this half are visible
            uint32_t r[2][32];
#pragma unroll
            for (int c = 0; c < 2; c++) tmem_ld32_nowait(tlane + S_COL + c0 + 32 * c, r[c]);
            tmem_ld_wait();
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (full) {
#pragma unroll
                for (int c = 0; c < 2; c++)
#pragma unroll
                    for (int i = 0; i < 32; i++) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(r[c][i]));
            } else {
#pragma unroll
                for (int c = 0; c < 2; c++)
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        if (32 * c + i >= nvis) r[c][i] = 0xff800000u;  // -inf
                        mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(r[c][i]));
                    }
            }
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            float* xm = xch + (j & 1) * 256;
            xm[half * 128 + row] = mx;
            sm_barrier();
            mx = fmaxf(mx, xm[(half ^ 1) * 128 + row]);
            const float m_new = fmaxf(m, mx * sl2);  // scale > 0, so the maximum commutes with the scaling
            const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
            const float corr = ex2(m - m_safe);
            float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < 2; c++) {
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    const float p = ex2(fmaf(__uint_as_float(r[c][i]), sl2, -m_safe));  // masked entries are -inf: p = 0
                    rs4[i & 3] += p;
                    r[c][i] = rna_tf32(p);
                }
                tmem_st32(tlane + S_COL + c0 + 32 * c, r[c]);
            }
            const float rs = (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
            l = l * corr + rs;  // this half's share of the row sum
            m = m_new;
            if (j > 0 && __any_sync(0xffffffffu, corr != 1.f)) {  // S(j) complete implies P V(j-1) complete: O is stable; this half's 32 columns
                uint32_t o[32];
                tmem_ld32(tlane + O_COL + 32 * half, o);
#pragma unroll
                for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                tmem_st32(tlane + O_COL + 32 * half, o);
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
        }
        if (ok) {
            ok = mbar_wait_warp(o_full, 0, status, 18);
            ok = __all_sync(0xffffffffu, ok);
        }
        float* xl = xch + 512;
        xl[half * 128 + row] = l;
        if (sm_barrier_or(!ok)) ok = false;  // the partial sums cross; a failed wait anywhere stops every softmax warp together
        if (ok) {
            tc_fence_after();
            l += xl[(half ^ 1) * 128 + row];
            // every MMA has completed, so the operand tiles are free: stage this quarter's 32 rows and store whole rows
            float* stage = reinterpret_cast<float*>(tiles) + quarter * (32 * OUT_STRIDE);
            const float il = l > 0.f ? 1.f / l : 0.f;
            uint32_t o[32];
            tmem_ld32(tlane + O_COL + 32 * half, o);
#pragma unroll
            for (int i = 0; i < 32; i += 4)
                *reinterpret_cast<float4*>(stage + lane * OUT_STRIDE + 32 * half + i) =
                    make_float4(__uint_as_float(o[i]) * il, __uint_as_float(o[i + 1]) * il, __uint_as_float(o[i + 2]) * il, __uint_as_float(o[i + 3]) * il);
            if (half == 0 && qi < sg.qLen) {
                const size_t idx = (size_t)(sg.qStart + qi) * a.numHeads + head;
                a.rowMax[idx] = (m == -INFINITY) ? -INFINITY : m / LOG2E_F;
                a.rowSum[idx] = l;
            }
        }
        sm_barrier();  // both halves of every row are staged
        if (ok) {
            const float* stage = reinterpret_cast<const float*>(tiles) + quarter * (32 * OUT_STRIDE);
            const int sub = lane >> 4, c4 = (lane & 15) * 4;
#pragma unroll 4
            for (int rr = 16 * half; rr < 16 * half + 16; rr += 2) {  // each warp of the pair stores half of the quarter's rows
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

// ------------------------------------------------------------------------------------------------------ backward
// Two deterministic passes, as in the other engines (dQ per query tile, dK/dV per key tile; no atomics), each a
// persistent kernel: one CTA per SM walks a static list of (segment, head, tile) items (see ItemWalk).
// The inner tiles are 64 wide and S/dP are double-buffered in TMEM.  Roles: one TMA producer thread; two threads that issue
// MMAs -- one the S and dP products, the other the products that consume P and dS (a single thread issues a narrow TF32
// MMA every ~55-65 cycles, the tensor pipe executes one in 32, so two issuers are what keeps it fed); sixteen
// element-wise warps (the softmax statistics are known, so this step has no row reduction and is split lane quarter x
// column quarter); four re-swizzle warps.  An operand that is needed both K-contiguous (for S / dP) and N-contiguous (for
// dQ, dK, dV) is loaded once, K-contiguous, and the re-swizzle warps rewrite it into the N-contiguous image inside
// shared memory (FP32 storage and 64-wide heads make the L2 -> shared-memory traffic of the streamed tiles the scarce
// resource after the element-wise step).
// What bounds them, from per-role wait counters of a development build (c5 shapes, 32 sequences of 1024): the element-wise
// warps are busy ~80 % of the time -- ex2 throughput (16 per cycle per SM) and packed FP32 arithmetic, ~800 cycles per
// 128 x 64 tile in the dQ pass -- and the first issuer needs ~1100 cycles per tile to issue its 16 MMAs; loads and the
// tensor pipe (768-1024 cycles of work per tile) wait for them.
constexpr int EW_THREADS = 512;                          // 16 element-wise warps: lane quarter (= warp % 4, the TMEM lanes a warp may touch) x column quarter
constexpr int B_THREADS = 64 + EW_THREADS + 128 + 32;    // producer, first MMA issuer, element-wise warps, 4 re-swizzle warps, second MMA issuer
constexpr int RESWIZZLE_T0 = 64 + EW_THREADS, ISSUER2_WARP = (64 + EW_THREADS + 128) / 32;
constexpr int A128 = 128 * 128, T128 = 2 * A128;  // atom column / tile with 128 rows
constexpr int A64 = 64 * 128, T64 = 2 * A64;      // atom column / tile with 64 rows
// Streamed operands live in two rings per kernel, because their consumers differ: the K-contiguous images feed the
// S / dP products and are free as soon as those complete, the N-contiguous images feed the products that follow the
// element-wise step.  Three slots let the loads run two to three tiles ahead of the MMA warp.
constexpr int RING_K = 3;                                      // slots of {two K-contiguous 64-row tiles} (32 KiB each)
constexpr int DQ_RING_N = 3, DKV_RING_N = 2;                   // slots of N-contiguous tiles: 16 KiB (dQ) / 32 KiB (dK,dV)
constexpr int DQ_SMEM = 2 * T128 + RING_K * 2 * T64 + DQ_RING_N * T64 + 1024 + 256;
constexpr int DKV_SMEM = 2 * T128 + RING_K * 2 * T64 + DKV_RING_N * 2 * T64 + 1024 + 256 + 2 * 3 * 64 * 4;
constexpr int BWD_TMEM_COLS = 512;

__device__ __forceinline__ uint64_t kdesc(uint32_t tile, int kk, int atom) { return umma_desc(tile + (kk >> 2) * atom + (kk & 3) * 32, 16, 1024, 2); }
__device__ __forceinline__ uint64_t ndesc(uint32_t tile, int kk, int atom) { return umma_desc(tile + kk * 1024, atom, 512, 1); }
// One arrival per warp: 32 lanes arriving on the same mbarrier are 32 serialised shared-memory atomics, and with every
// element-wise thread arriving the phase completes hundreds of cycles after the first of them.  Each lane has made its own
// accesses complete (tcgen05.wait, proxy fence) before this call; __syncwarp orders them before lane 0's arrival.
__device__ __forceinline__ void warp_arrive(uint32_t bar) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}
// Named barrier of the element-wise threads with an OR vote (true when any thread passes true).
__device__ __forceinline__ bool ew_barrier_or(bool pred) {
    uint32_t r;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %1, 0;\n\tbar.red.or.pred q, 1, 512, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                 : "=r"(r)
                 : "r"((uint32_t)pred)
                 : "memory");
    return r != 0;
}

// Copy a [64 x 64] FP32 tile (two 32-column atoms of 64 rows x 128 bytes) from the K-contiguous image (16-byte chunks
// XOR row%8, what TMA SWIZZLE_128B writes) to the N-contiguous image (32-byte chunks XOR row%4, what the UMMA layout
// "128-byte swizzle, 32-byte atoms" reads).  128 threads, eight 16-byte chunks each, conflict-free on both sides.
__device__ __forceinline__ void reswizzle_tile(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int t) {
#pragma unroll
    for (int it = 0; it < 8; it++) {
        const int idx = it * 128 + t;
        const int atom = idx >> 9, r = (idx >> 3) & 63, q = idx & 7;
        const uint4 v = *reinterpret_cast<const uint4*>(src + atom * A64 + r * 128 + ((q ^ (r & 7)) << 4));
        *reinterpret_cast<uint4*>(dst + atom * A64 + r * 128 + ((((q >> 1) ^ (r & 3)) << 5) | ((q & 1) << 4))) = v;
    }
}

struct UBwdArgs {
    float *dQ, *dK, *dV;
    int lddq, lddk, lddv;
    const float *rowMax, *rowSum, *rowDot;
    const AttnSeg* segs;
    int numHeads, causal;
    float scale;
    int* status;
    const float* rope_table; const int32_t* rope_pos;  // inverse rotary rotation of dQ and dK on the way out (or null)
};

// ---- work items of the persistent backward kernels.  A CTA stays on its SM and walks a static list of (segment, head,
// tile) items, so an item's fixed cost (resident operands -> shared memory -> TMEM, pipeline fill, output) runs under
// the tiles of its neighbours instead of standing alone: the loads of item n+1 are requested while item n streams,
// its first S / dP products are issued while the element-wise warps still write item n's result.
// Under a causal mask the work of tile t of n grows (dQ) or shrinks (dK/dV) linearly with t, so the list pairs tile p
// with tile n-1-p of the same (segment, head): every pair costs the same, a plain round-robin over the pairs balances
// the CTAs, and the CTAs that run at the same time work on the same few (segment, head) slices, which stay in L2.
struct ItemWalk {
    int u, second, nTiles, pairsPerGroup, nPairs, stride;
    __device__ ItemWalk(int nTiles_, int nGroups)
        : u(blockIdx.x), second(0), nTiles(nTiles_), pairsPerGroup((nTiles_ + 1) >> 1), nPairs(nGroups * ((nTiles_ + 1) >> 1)), stride(gridDim.x) {}
    // next (group, tile); `longFirstHigh`: the high tile of a pair is the long one (dQ) and goes first
    __device__ bool next(int& group, int& tile, bool longFirstHigh) {
        while (u < nPairs) {
            group = u / pairsPerGroup;
            const int p = u - group * pairsPerGroup, hi = nTiles - 1 - p;
            if (!second) {
                second = 1;
                tile = longFirstHigh ? hi : p;
                return true;
            }
            second = 0;
            u += stride;
            if (p != hi) {
                tile = longFirstHigh ? p : hi;
                return true;
            }
        }
        return false;
    }
};
// A segment descriptor through the read-only path: every role of a CTA reads the same few entries for each of its items,
// and after the first time they come from L1 instead of L2.
__device__ __forceinline__ AttnSeg load_seg(const AttnSeg* p) {
    const int4 v = __ldg(reinterpret_cast<const int4*>(p));
    AttnSeg s;
    s.qStart = v.x; s.qLen = v.y; s.kStart = v.z; s.kLen = v.w;
    return s;
}
struct BwdItem { AttnSeg sg; int head, t0, n, aux; };  // t0: first row of the resident tile; n: streamed tiles; aux: first streamed tile

// dQ items: 128 query rows against the 64-key tiles they can see.  Items without rows are skipped by every role alike;
// rows without any key get zeros from the caller of this function when `zeroFillTid` >= 0 (the element-wise threads).
__device__ __forceinline__ bool next_dq_item(ItemWalk& w, const UBwdArgs& a, BwdItem& it, int zeroFillTid) {
    int group, tile;
    while (w.next(group, tile, true)) {
        const int seg = group / a.numHeads, head = group - seg * a.numHeads;
        const AttnSeg sg = load_seg(a.segs + seg);
        const int q0 = tile * 128;
        if (q0 >= sg.qLen) continue;
        const int kEnd = a.causal ? min(sg.kLen, q0 + 128) : sg.kLen;
        const int nkt = (kEnd + 63) / 64;
        if (nkt == 0) {
            if (zeroFillTid >= 0)
                for (int idx = zeroFillTid; idx < 128 * 16; idx += EW_THREADS) {
                    const int r = idx >> 4, c = (idx & 15) * 4;
                    if (q0 + r < sg.qLen) *reinterpret_cast<float4*>(a.dQ + (size_t)(sg.qStart + q0 + r) * a.lddq + head * UHD + c) = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            continue;
        }
        it.sg = sg; it.head = head; it.t0 = q0; it.n = nkt;
        return true;
    }
    return false;
}

// One thread's 16 consecutive result columns of one row, scaled, optionally rotated back (gradient of a rotary rotation =
// rotation by the opposite angle; cs = the row's (cos, sin) pairs for these columns), written with 128-bit stores: the
// thread covers half a 128-byte line.
__device__ __forceinline__ void store_row_slice(const uint32_t (&r)[16], float scale, float* dst, const float4* cs) {
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
        float4 v = make_float4(__uint_as_float(r[i]) * scale, __uint_as_float(r[i + 1]) * scale, __uint_as_float(r[i + 2]) * scale,
                               __uint_as_float(r[i + 3]) * scale);
        if (cs) {
            const float4 c = cs[i >> 2];
            const float x0 = v.x, x1 = v.y, x2 = v.z, x3 = v.w;
            v.x = x0 * c.x + x1 * c.y; v.y = x1 * c.x - x0 * c.y;
            v.z = x2 * c.z + x3 * c.w; v.w = x3 * c.z - x2 * c.w;
        }
        *reinterpret_cast<float4*>(dst + i) = v;
    }
}

__global__ void __launch_bounds__(B_THREADS) attn_dq_umma_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapdO,
                                                                const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV,
                                                                UBwdArgs a, int nTiles, int nGroups) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(tiles + 2 * T128 + RING_K * 2 * T64 + DQ_RING_N * T64);
    uint32_t* tmem_slot = (uint32_t*)(bars + 23);
    const uint32_t Qs = smem_u32(tiles), dOs = Qs + T128;
    const uint32_t ringK = dOs + T128;                 // slot: K tile then V tile, both K-contiguous
    const uint32_t ringN = ringK + RING_K * 2 * T64;   // slot: K tile, N-contiguous
    const uint32_t bar0 = smem_u32(bars);
    // per item: qdo_full, a_ready, dq_full, acc_free; per streamed tile (counted across items): the rest
    const uint32_t qdo_full = bar0, kk_full = bar0 + 8, kk_empty = bar0 + 32, kn_full = bar0 + 56, kn_empty = bar0 + 80, sdp_full = bar0 + 104,
                   ds_full = bar0 + 120, dq_full = bar0 + 136, a_ready = bar0 + 144, buf_free = bar0 + 152, acc_free = bar0 + 168, ds_free = bar0 + 176;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* status = a.status;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 23; i++)  // ds_full (15; 16 unused), a_ready, buf_free, acc_free: one arrival per element-wise warp; kk_empty: MMA commit + 4 re-swizzle warps; kn_full: 4 re-swizzle warps
            mbar_init(bar0 + 8 * i, (i == 15 || i == 16 || (i >= 18 && i <= 21)) ? EW_THREADS / 32 : (i >= 4 && i <= 6) ? 5 : (i >= 7 && i <= 9) ? 4 : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(BWD_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm = *tmem_slot;
    // S / dP: two buffers of 128 columns from 0; Q and dO live in TMEM as A operands; dS has a buffer of its own, so an
    // S / dP buffer is free again as soon as the element-wise warps have read it (not only after the dQ product that
    // consumes dS), and the first issuer runs ahead of the rest of the pipeline instead of in lockstep with it
    constexpr uint32_t DQ_COL = 256, QA_COL = 320, DOA_COL = 384, DS_COL = 448;

    if (warp == 0) {
        if (lane == 0) {
            // ---------------------------------------------------------------- TMA producer
            ItemWalk w(nTiles, nGroups);
            BwdItem it;
            bool ok = true;
            int n = 0;
            uint32_t g = 0;
            while (ok && next_dq_item(w, a, it, -1)) {
                if (n > 0) {  // the element-wise threads have copied the previous item's Q and dO out of shared memory
                    ok = mbar_wait(a_ready, (n - 1) & 1, status, 20);
                    if (!ok) break;
                }
                mbar_expect_tx(qdo_full, 2 * T128);
                tma_load_3d(Qs, &mapQ, qdo_full, 0, it.sg.qStart + it.t0, it.head * (UHD / 32));
                tma_load_3d(dOs, &mapdO, qdo_full, 0, it.sg.qStart + it.t0, it.head * (UHD / 32));
                n++;
                for (int j = 0; j < it.n; j++) {
                    const int s = g % RING_K, row = it.sg.kStart + j * 64;
                    ok = mbar_wait(kk_empty + 8 * s, ((g / RING_K) & 1) ^ 1, status, 21);
                    if (!ok) break;
                    const uint32_t base = ringK + s * 2 * T64, bar = kk_full + 8 * s;
                    mbar_expect_tx(bar, 2 * T64);
                    tma_load_3d(base, &mapK, bar, 0, row, it.head * (UHD / 32));
                    tma_load_3d(base + T64, &mapV, bar, 0, row, it.head * (UHD / 32));
                    g++;
                }
            }
            if (!ok) {  // failure path: let the copies already issued land (bounded) before the CTA may exit
                const long long t0 = clock64();
                while (n > 0 && !mbar_test(qdo_full, (n - 1) & 1) && clock64() - t0 < WAIT_BUDGET_CLOCKS) __nanosleep(64);
                for (uint32_t j = g > RING_K ? g - RING_K : 0; j < g; j++)
                    while (!mbar_test(kk_full + 8 * (j % RING_K), (j / RING_K) & 1) && clock64() - t0 < WAIT_BUDGET_CLOCKS) __nanosleep(64);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------------------------------------------------------- first issuer: S(j) and dP(j) into TMEM buffer g&1
            const uint32_t idS = idesc_tf32(128, 64, 0, 0);
            const uint64_t dRK0 = kdesc(ringK, 0, A64);
            ItemWalk w(nTiles, nGroups);
            BwdItem it;
            bool ok = true;
            int n = 0;
            uint32_t g = 0;
            while (ok && next_dq_item(w, a, it, -1)) {
                ok = mbar_wait(a_ready, n & 1, status, 22);  // this item's Q and dO are in TMEM
                if (!ok) break;
                n++;
                for (int j = 0; j < it.n; j++) {
                    const int s = g % RING_K, b = g & 1;
                    ok = mbar_wait(kk_full + 8 * s, (g / RING_K) & 1, status, 23);
                    if (!ok) break;
                    ok = mbar_wait(buf_free + 8 * b, ((g >> 1) & 1) ^ 1, status, 24);  // the element-wise warps have read the tile two back out of the buffer
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t dk = dRK0 + (uint64_t)(s * ((2 * T64) >> 4)), dv = dk + (uint64_t)(T64 >> 4);
#pragma unroll
                    for (int kk = 0; kk < 8; kk++) umma_tf32_ta(tm + b * 128, tm + QA_COL + kk * 8, dk + koff(kk, A64), idS, kk > 0 ? 1u : 0u);
#pragma unroll
                    for (int kk = 0; kk < 8; kk++) umma_tf32_ta(tm + b * 128 + 64, tm + DOA_COL + kk * 8, dv + koff(kk, A64), idS, kk > 0 ? 1u : 0u);
                    umma_commit(kk_empty + 8 * s);
                    umma_commit(sdp_full + 8 * b);
                    g++;
                }
            }
        }
    } else if (warp == ISSUER2_WARP) {
        if (lane == 0) {
            // ---------------------------------------------------------------- second issuer: dQ += dS(j) K(j)
            const uint32_t idN = idesc_tf32(128, 64, 0, 1);
            const uint64_t dRN0 = ndesc(ringN, 0, A64);
            ItemWalk w(nTiles, nGroups);
            BwdItem it;
            bool ok = true;
            int n = 0;
            uint32_t g = 0;
            while (ok && next_dq_item(w, a, it, -1)) {
                for (int j = 0; j < it.n; j++) {
                    const int s = g % DQ_RING_N;
                    ok = mbar_wait(kn_full + 8 * s, (g / DQ_RING_N) & 1, status, 25);
                    if (!ok) break;
                    ok = mbar_wait(ds_full, g & 1, status, 25);
                    if (!ok) break;
                    if (j == 0 && n > 0) {  // the previous item's dQ has been read out of the accumulator
                        ok = mbar_wait(acc_free, (n - 1) & 1, status, 28);
                        if (!ok) break;
                    }
                    tc_fence_after();
                    const uint64_t dn = dRN0 + (uint64_t)(s * (T64 >> 4));
#pragma unroll
                    for (int kk = 0; kk < 8; kk++) umma_tf32_ta(tm + DQ_COL, tm + DS_COL + kk * 8, dn + noff(kk), idN, (j > 0 || kk > 0) ? 1u : 0u);
                    umma_commit(kn_empty + 8 * s);
                    umma_commit(ds_free);
                    g++;
                }
                if (!ok) break;
                umma_commit(dq_full);
                n++;
            }
        }
    } else if (warp < 2 + EW_THREADS / 32) {
        // ------------------------------------------------------------------------------ element-wise warps and output
        const int quarter = warp & 3, colq = (warp - 2) >> 2, c0 = 16 * colq;
        const int row = 32 * quarter + lane;
        const uint32_t tlane = tm + ((uint32_t)(32 * quarter) << 16);
        const float sl2 = a.scale * LOG2E_F;
        const float2 sl22 = make_float2(sl2, sl2);
        // P = 2^(s*sl2 - m2l) with m2l = rowMax*log2(e) + log2(rowSum): the normalisation rides in the exponent.
        // Rows without any visible key (or outside the segment) get m2l = +inf, i.e. P = 0.
        float m2l = INFINITY, D = 0.f;
        bool live = false;
        // A row's statistics are requested one item ahead (raw values in registers) and turned into (m2l, D) at the boundary.
        float rm = -INFINITY, rl = 0.f, rD = 0.f;
        int rpos = 0, pos = 0;  // rotary position of this thread's row (next item / current item)
        auto request_stats = [&](const BwdItem& it) {
            rm = -INFINITY; rl = 0.f; rD = 0.f; rpos = 0;
            const int qi = it.t0 + row;
            if (qi < it.sg.qLen) {
                const size_t idx = (size_t)(it.sg.qStart + qi) * a.numHeads + it.head;
                rm = a.rowMax[idx]; rl = a.rowSum[idx]; rD = a.rowDot[idx];
                if (a.rope_table) rpos = a.rope_pos ? a.rope_pos[it.sg.qStart + qi] : it.sg.qStart + qi;
            }
        };
        auto take_stats = [&]() {
            live = rl > 0.f && rm != -INFINITY;
            m2l = live ? fmaf(rm, LOG2E_F, log2f(rl)) : INFINITY;
            D = rD;
            pos = rpos;
        };
        auto operands_to_tmem = [&](int n) -> bool {  // this thread's quarter rows of Q and dO: shared memory -> TMEM
            const bool ok = __all_sync(0xffffffffu, mbar_wait_warp(qdo_full, n & 1, status, 20));
            if (!ok) return false;
            half_row_to_tmem(tiles + (colq >> 1) * A128, row, colq & 1, tlane + QA_COL + c0);
            half_row_to_tmem(tiles + T128 + (colq >> 1) * A128, row, colq & 1, tlane + DOA_COL + c0);
            tmem_st_wait();
            tc_fence_before();
            warp_arrive(a_ready);
            return true;
        };
        ItemWalk w(nTiles, nGroups);
        BwdItem cur, nxt;
        const int tid = threadIdx.x - 64;
        bool have = next_dq_item(w, a, cur, tid);
        bool ok = true;
        int n = 0;
        uint32_t g = 0;
        if (have) {
            request_stats(cur);
            ok = operands_to_tmem(0);
        }
        while (have && ok) {
            take_stats();
            const bool haveN = next_dq_item(w, a, nxt, tid);
            if (haveN) request_stats(nxt);
            const int qi = cur.t0 + row;
            const int lim = live ? (a.causal ? min(cur.sg.kLen, qi + 1) : cur.sg.kLen) : 0;  // keys [0, lim) are visible to this row
            const float2 nm2 = make_float2(-m2l, -m2l), nD2 = make_float2(-D, -D);
            for (int j = 0; j < cur.n; j++, g++) {
                const int s = g & 1;
                ok = mbar_wait_warp(sdp_full + 8 * s, (g >> 1) & 1, status, 26);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const int nvis = lim - j * 64 - c0;  // columns [0, nvis) of this warp's 16 are visible
                uint32_t sr[16], pr[16];
                tmem_ld16_nowait(tlane + s * 128 + c0, sr);
                tmem_ld16_nowait(tlane + s * 128 + 64 + c0, pr);
                tmem_ld_wait();
                tc_fence_before();
                warp_arrive(buf_free + 8 * s);  // S and dP are in registers: the buffer may be refilled
                // Two copies of the loop, chosen once per tile: a branch inside the unrolled body would fence the scheduling
                // of everything around it, and only the tiles on the diagonal (or at a segment's end) need the masks.
                auto tile_math = [&](auto masked) {
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {
                        float2 v = fma2(make_float2(__uint_as_float(sr[i]), __uint_as_float(sr[i + 1])), sl22, nm2);
                        if (decltype(masked)::value) {
                            if (i >= nvis) v.x = -INFINITY;
                            if (i + 1 >= nvis) v.y = -INFINITY;
                        }
                        const float2 pp = make_float2(ex2(v.x), ex2(v.y));
                        const float2 ds = mul2(pp, add2(make_float2(__uint_as_float(pr[i]), __uint_as_float(pr[i + 1])), nD2));
                        sr[i] = rna_tf32_add(ds.x);
                        sr[i + 1] = rna_tf32_add(ds.y);
                    }
                };
                if (__all_sync(0xffffffffu, nvis >= 16)) tile_math(std::false_type());  // no masking anywhere in this warp's slice
                else tile_math(std::true_type());
                ok = __all_sync(0xffffffffu, mbar_wait_warp(ds_free, (g & 1) ^ 1, status, 31));  // the previous dQ product has read dS
                if (!ok) break;
                tc_fence_after();
                tmem_st16(tlane + DS_COL + c0, sr);
                tmem_st_wait();
                tc_fence_before();
                warp_arrive(ds_full);
            }
            if (!ok) break;
            // The S / dP products of this item are complete (its last sdp_full was seen), so the next item's Q and dO may
            // replace it in TMEM right away: the first issuer starts on the next item while this one's result is written.
            // this row's rotation factors (its position came with the statistics) are requested before the next item's operands
            // are moved and the accumulator is waited for, which hides their latency
            const bool rot = a.rope_table != nullptr && qi < cur.sg.qLen;
            float4 cs[4];
            if (rot) {
                const float4* cs4 = reinterpret_cast<const float4*>(a.rope_table + ((size_t)pos * (UHD / 2) + (c0 >> 1)) * 2);
#pragma unroll
                for (int i = 0; i < 4; i++) cs[i] = cs4[i];
            }
            if (haveN) {
                ok = operands_to_tmem(n + 1);
                if (!ok) break;
            }
            ok = __all_sync(0xffffffffu, mbar_wait_warp(dq_full, n & 1, status, 27));
            if (!ok) break;
            tc_fence_after();
            uint32_t r[16];
            tmem_ld16_nowait(tlane + DQ_COL + c0, r);
            tmem_ld_wait();
            tc_fence_before();
            warp_arrive(acc_free);
            // a lane writes its own row slice: the stores retire in the background while the next item's tiles are worked on
            if (qi < cur.sg.qLen) store_row_slice(r, a.scale, a.dQ + (size_t)(cur.sg.qStart + qi) * a.lddq + cur.head * UHD + c0, rot ? cs : nullptr);
            cur = nxt;
            have = haveN;
            n++;
        }
    } else if (warp < ISSUER2_WARP) {
        // ------------------------------------------------------------------------------ re-swizzle warps: K -> N-contiguous image
        const int t = threadIdx.x - RESWIZZLE_T0;
        uint8_t* ringK_p = tiles + 2 * T128;
        uint8_t* ringN_p = ringK_p + RING_K * 2 * T64;
        ItemWalk w(nTiles, nGroups);
        BwdItem it;
        bool ok = true;
        uint32_t g = 0;
        while (ok && next_dq_item(w, a, it, -1)) {
            for (int j = 0; j < it.n; j++, g++) {
                const int sk = g % RING_K, sn = g % DQ_RING_N;
                ok = mbar_wait_warp(kk_full + 8 * sk, (g / RING_K) & 1, status, 29) && mbar_wait_warp(kn_empty + 8 * sn, ((g / DQ_RING_N) & 1) ^ 1, status, 30);
                if (!ok) break;
                reswizzle_tile(ringK_p + sk * 2 * T64, ringN_p + sn * T64, t);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the MMA's reads
                warp_arrive(kn_full + 8 * sn);
                warp_arrive(kk_empty + 8 * sk);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tm), "r"(BWD_TMEM_COLS) : "memory");
    }
}

// dK / dV items: 128 keys (one per TMEM lane) against the 64-row query tiles that can see them; aux = first such tile.
__device__ __forceinline__ bool next_dkv_item(ItemWalk& w, const UBwdArgs& a, BwdItem& it, int zeroFillTid) {
    int group, tile;
    while (w.next(group, tile, false)) {
        const int seg = group / a.numHeads, head = group - seg * a.numHeads;
        const AttnSeg sg = load_seg(a.segs + seg);
        const int k0 = tile * 128;  // under a causal mask the first key tiles see the most queries
        if (k0 >= sg.kLen) continue;
        const int qtBegin = a.causal ? k0 / 64 : 0, nqt = (sg.qLen + 63) / 64 - qtBegin;
        if (nqt <= 0) {  // keys no query can see
            if (zeroFillTid >= 0)
                for (int idx = zeroFillTid; idx < 128 * 16; idx += EW_THREADS) {
                    const int r = idx >> 4, c = (idx & 15) * 4;
                    if (k0 + r < sg.kLen) {
                        *reinterpret_cast<float4*>(a.dK + (size_t)(sg.kStart + k0 + r) * a.lddk + head * UHD + c) = make_float4(0.f, 0.f, 0.f, 0.f);
                        *reinterpret_cast<float4*>(a.dV + (size_t)(sg.kStart + k0 + r) * a.lddv + head * UHD + c) = make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
            continue;
        }
        it.sg = sg; it.head = head; it.t0 = k0; it.n = nqt; it.aux = qtBegin;
        return true;
    }
    return false;
}

// dK / dV for 128 keys (one key per TMEM lane) against the query tiles (64 rows each) that can see them:
//   S^T = K Q^T, dP^T = V dO^T  ->  P^T, dS^T (element-wise, per-column statistics from shared memory)
//   dV += P^T dO,  dK += dS^T Q   (A from TMEM, Q / dO as N-contiguous shared-memory operands)
__global__ void __launch_bounds__(B_THREADS) attn_dkv_umma_kernel(const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV,
                                                                 const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapdO,
                                                                 UBwdArgs a, int nTiles, int nGroups) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(tiles + 2 * T128 + RING_K * 2 * T64 + DKV_RING_N * 2 * T64);
    uint32_t* tmem_slot = (uint32_t*)(bars + 21);
    float* stats = reinterpret_cast<float*>(bars + 24);  // [2 buffers][-(m2 + log2 l) | -D][64] (stride 192 floats)
    const uint32_t Ks = smem_u32(tiles), Vs = Ks + T128;
    const uint32_t ringK = Vs + T128;                  // slot: Q tile then dO tile, both K-contiguous
    const uint32_t ringN = ringK + RING_K * 2 * T64;   // slot: Q tile then dO tile, both N-contiguous
    const uint32_t bar0 = smem_u32(bars);
    // per item: kv_full, a_ready, acc_full, acc_free; per streamed tile (counted across items): the rest
    const uint32_t kv_full = bar0, qk_full = bar0 + 8, qk_empty = bar0 + 32, qn_full = bar0 + 56, qn_empty = bar0 + 72, sdp_full = bar0 + 88,
                   ds_full = bar0 + 104, acc_full = bar0 + 120, a_ready = bar0 + 128, buf_free = bar0 + 136, acc_free = bar0 + 152;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* status = a.status;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 20; i++)  // a_ready, ds_full, acc_free: one arrival per element-wise warp; qk_empty: MMA commit + 4 re-swizzle warps; qn_full: 4 re-swizzle warps
            mbar_init(bar0 + 8 * i, (i == 13 || i == 14 || i == 16 || i == 19) ? EW_THREADS / 32 : (i >= 4 && i <= 6) ? 5 : (i == 7 || i == 8) ? 4 : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(BWD_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm = *tmem_slot;
    constexpr uint32_t DV_COL = 256, DK_COL = 320, KA_COL = 384, VA_COL = 448;  // K and V live in TMEM as A operands

    if (warp == 0) {
        if (lane == 0) {
            // ---------------------------------------------------------------- TMA producer
            ItemWalk w(nTiles, nGroups);
            BwdItem it;
            bool ok = true;
            int n = 0;
            uint32_t g = 0;
            while (ok && next_dkv_item(w, a, it, -1)) {
                if (n > 0) {  // the element-wise threads have copied the previous item's K and V out of shared memory
                    ok = mbar_wait(a_ready, (n - 1) & 1, status, 30);
                    if (!ok) break;
                }
                mbar_expect_tx(kv_full, 2 * T128);
                tma_load_3d(Ks, &mapK, kv_full, 0, it.sg.kStart + it.t0, it.head * (UHD / 32));
                tma_load_3d(Vs, &mapV, kv_full, 0, it.sg.kStart + it.t0, it.head * (UHD / 32));
                n++;
                for (int i = 0; i < it.n; i++) {
                    const int s = g % RING_K, row = it.sg.qStart + (it.aux + i) * 64;
                    ok = mbar_wait(qk_empty + 8 * s, ((g / RING_K) & 1) ^ 1, status, 31);
                    if (!ok) break;
                    const uint32_t base = ringK + s * 2 * T64, bar = qk_full + 8 * s;
                    mbar_expect_tx(bar, 2 * T64);
                    tma_load_3d(base, &mapQ, bar, 0, row, it.head * (UHD / 32));
                    tma_load_3d(base + T64, &mapdO, bar, 0, row, it.head * (UHD / 32));
                    g++;
                }
            }
            if (!ok) {  // failure path: let the copies already issued land (bounded) before the CTA may exit
                const long long t0 = clock64();
                while (n > 0 && !mbar_test(kv_full, (n - 1) & 1) && clock64() - t0 < WAIT_BUDGET_CLOCKS) __nanosleep(64);
                for (uint32_t j = g > RING_K ? g - RING_K : 0; j < g; j++)
                    while (!mbar_test(qk_full + 8 * (j % RING_K), (j / RING_K) & 1) && clock64() - t0 < WAIT_BUDGET_CLOCKS) __nanosleep(64);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------------------------------------------------------- first issuer: S^T(i) and dP^T(i) into TMEM buffer g&1
            const uint32_t idS = idesc_tf32(128, 64, 0, 0);
            const uint64_t dRK0 = kdesc(ringK, 0, A64);
            ItemWalk w(nTiles, nGroups);
            BwdItem it;
            bool ok = true;
            int n = 0;
            uint32_t g = 0;
            while (ok && next_dkv_item(w, a, it, -1)) {
                ok = mbar_wait(a_ready, n & 1, status, 32);  // this item's K and V are in TMEM
                if (!ok) break;
                n++;
                for (int i = 0; i < it.n; i++) {
                    const int s = g % RING_K, b = g & 1;
                    ok = mbar_wait(qk_full + 8 * s, (g / RING_K) & 1, status, 33);
                    if (!ok) break;
                    ok = mbar_wait(buf_free + 8 * b, ((g >> 1) & 1) ^ 1, status, 34);  // the dV, dK products two tiles back have consumed the buffer
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t dq = dRK0 + (uint64_t)(s * ((2 * T64) >> 4)), dd = dq + (uint64_t)(T64 >> 4);
#pragma unroll
                    for (int kk = 0; kk < 8; kk++) umma_tf32_ta(tm + b * 128, tm + KA_COL + kk * 8, dq + koff(kk, A64), idS, kk > 0 ? 1u : 0u);
#pragma unroll
                    for (int kk = 0; kk < 8; kk++) umma_tf32_ta(tm + b * 128 + 64, tm + VA_COL + kk * 8, dd + koff(kk, A64), idS, kk > 0 ? 1u : 0u);
                    umma_commit(qk_empty + 8 * s);
                    umma_commit(sdp_full + 8 * b);
                    g++;
                }
            }
        }
    } else if (warp == ISSUER2_WARP) {
        if (lane == 0) {
            // ---------------------------------------------------------------- second issuer: dV += P^T dO, dK += dS^T Q
            const uint32_t idN = idesc_tf32(128, 64, 0, 1);
            const uint64_t dRN0 = ndesc(ringN, 0, A64);
            ItemWalk w(nTiles, nGroups);
            BwdItem it;
            bool ok = true;
            int n = 0;
            uint32_t g = 0;
            while (ok && next_dkv_item(w, a, it, -1)) {
                for (int i = 0; i < it.n; i++) {
                    const int s = g % DKV_RING_N, b = g & 1;
                    ok = mbar_wait(qn_full + 8 * s, (g / DKV_RING_N) & 1, status, 35);
                    if (!ok) break;
                    ok = mbar_wait(ds_full + 8 * b, (g >> 1) & 1, status, 35);
                    if (!ok) break;
                    if (i == 0 && n > 0) {  // the previous item's dV and dK have been read out of the accumulators
                        ok = mbar_wait(acc_free, (n - 1) & 1, status, 38);
                        if (!ok) break;
                    }
                    tc_fence_after();
                    const uint64_t dqn = dRN0 + (uint64_t)(s * ((2 * T64) >> 4)), ddn = dqn + (uint64_t)(T64 >> 4);
#pragma unroll
                    for (int kk = 0; kk < 8; kk++) umma_tf32_ta(tm + DV_COL, tm + b * 128 + kk * 8, ddn + noff(kk), idN, (i > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
                    for (int kk = 0; kk < 8; kk++) umma_tf32_ta(tm + DK_COL, tm + b * 128 + 64 + kk * 8, dqn + noff(kk), idN, (i > 0 || kk > 0) ? 1u : 0u);
                    umma_commit(qn_empty + 8 * s);
                    umma_commit(buf_free + 8 * b);
                    g++;
                }
                if (!ok) break;
                umma_commit(acc_full);
                n++;
            }
        }
    } else if (warp < 2 + EW_THREADS / 32) {
        // ------------------------------------------------------------------------------ element-wise warps and output
        const int quarter = warp & 3, colq = (warp - 2) >> 2, c0 = 16 * colq, tid = threadIdx.x - 64;
        const int row = 32 * quarter + lane;
        const uint32_t tlane = tm + ((uint32_t)(32 * quarter) << 16);
        const float sl2 = a.scale * LOG2E_F;
        const float2 sl22 = make_float2(sl2, sl2);
        auto operands_to_tmem = [&](int n) -> bool {  // this thread's quarter rows of K and V: shared memory -> TMEM
            const bool ok = __all_sync(0xffffffffu, mbar_wait_warp(kv_full, n & 1, status, 30));
            if (!ok) return false;
            half_row_to_tmem(tiles + (colq >> 1) * A128, row, colq & 1, tlane + KA_COL + c0);
            half_row_to_tmem(tiles + T128 + (colq >> 1) * A128, row, colq & 1, tlane + VA_COL + c0);
            tmem_st_wait();
            tc_fence_before();
            warp_arrive(a_ready);
            return true;
        };
        // Statistics of a tile's 64 query rows: fetched one tile ahead into registers (threads 0..63), across item
        // boundaries too, so their global latency overlaps the previous tile instead of sitting in front of every tile.
        float pm = -INFINITY, pl = 0.f, pD = 0.f;
        auto fetch_stats = [&](const BwdItem& it, int i) {
            pm = -INFINITY; pl = 0.f; pD = 0.f;
            const int q = (it.aux + i) * 64 + tid;
            if (tid < 64 && q < it.sg.qLen) {
                const size_t idx = (size_t)(it.sg.qStart + q) * a.numHeads + it.head;
                pm = a.rowMax[idx]; pl = a.rowSum[idx]; pD = a.rowDot[idx];
            }
        };
        ItemWalk w(nTiles, nGroups);
        BwdItem cur, nxt;
        bool have = next_dkv_item(w, a, cur, tid);
        bool ok = true;
        int n = 0;
        uint32_t g = 0;
        if (have) {
            fetch_stats(cur, 0);
            ok = !ew_barrier_or(!operands_to_tmem(0));
        }
        while (have && ok) {
            const bool haveN = next_dkv_item(w, a, nxt, tid);
            const int kj = cur.t0 + row;
            int kpos = cur.sg.kStart + kj;  // rotary position of this thread's key, requested a whole item before its use
            if (a.rope_table && a.rope_pos && kj < cur.sg.kLen) kpos = a.rope_pos[kpos];
            for (int i = 0; i < cur.n; i++, g++) {
                const int s = g & 1, qbase = (cur.aux + i) * 64;
                float* st = stats + s * 192;
                if (tid < 64) {
                    // +inf: P = 0 for query rows outside the segment or without a visible key
                    const float m2l = (pl > 0.f && pm != -INFINITY) ? fmaf(pm, LOG2E_F, log2f(pl)) : INFINITY;
                    st[tid] = -m2l; st[64 + tid] = -pD;
                }
                if (i + 1 < cur.n) fetch_stats(cur, i + 1);
                else if (haveN) fetch_stats(nxt, 0);
                ok = mbar_wait_warp(sdp_full + 8 * s, (g >> 1) & 1, status, 36);
                if (ew_barrier_or(!ok)) {  // publishes the statistics; a failed wait anywhere stops all 256 threads together
                    ok = false;
                    break;
                }
                tc_fence_after();
                // visible columns of this warp's 16: query index >= key index (causal), query inside the segment, key inside it
                int cmin = a.causal ? kj - qbase - c0 : 0, cmax = cur.sg.qLen - qbase - c0;
                if (kj >= cur.sg.kLen) cmax = 0;
                uint32_t sr[16], pr[16];
                tmem_ld16_nowait(tlane + s * 128 + c0, sr);
                tmem_ld16_nowait(tlane + s * 128 + 64 + c0, pr);
                tmem_ld_wait();
                // Two copies of the loop, chosen once per tile: a branch inside the unrolled body would keep the loads of the
                // per-column statistics from moving ahead of the arithmetic that precedes them.
                auto tile_math = [&](auto masked) {
#pragma unroll
                    for (int c = 0; c < 16; c += 4) {
                        const float4 m4 = *reinterpret_cast<const float4*>(st + c0 + c), d4 = *reinterpret_cast<const float4*>(st + 64 + c0 + c);
                        const float2 nm[2] = {make_float2(m4.x, m4.y), make_float2(m4.z, m4.w)}, nd[2] = {make_float2(d4.x, d4.y), make_float2(d4.z, d4.w)};
#pragma unroll
                        for (int e = 0; e < 2; e++) {
                            const int ii = c + 2 * e;
                            float2 v = fma2(make_float2(__uint_as_float(sr[ii]), __uint_as_float(sr[ii + 1])), sl22, nm[e]);
                            if (decltype(masked)::value) {
                                if (ii < cmin || ii >= cmax) v.x = -INFINITY;
                                if (ii + 1 < cmin || ii + 1 >= cmax) v.y = -INFINITY;
                            }
                            const float2 pp = make_float2(ex2(v.x), ex2(v.y));
                            const float2 ds = mul2(pp, add2(make_float2(__uint_as_float(pr[ii]), __uint_as_float(pr[ii + 1])), nd[e]));
                            sr[ii] = rna_tf32_add(pp.x); sr[ii + 1] = rna_tf32_add(pp.y);
                            pr[ii] = rna_tf32_add(ds.x); pr[ii + 1] = rna_tf32_add(ds.y);
                        }
                    }
                };
                if (__all_sync(0xffffffffu, cmin <= 0 && cmax >= 16)) tile_math(std::false_type());  // no masking anywhere in this warp's slice
                else tile_math(std::true_type());
                tmem_st16(tlane + s * 128 + c0, sr);
                tmem_st16(tlane + s * 128 + 64 + c0, pr);
                tmem_st_wait();
                tc_fence_before();
                warp_arrive(ds_full + 8 * s);
            }
            if (!ok) break;
            // The S^T / dP^T products of this item are complete (its last sdp_full was seen), so the next item's K and V may
            // replace it in TMEM right away: the first issuer starts on the next item while this one's results are written.
            bool okb = true;
            if (haveN) okb = operands_to_tmem(n + 1);
            if (okb) okb = __all_sync(0xffffffffu, mbar_wait_warp(acc_full, n & 1, status, 37));
            if (okb) {
                tc_fence_after();
                uint32_t rv[16], rk[16];
                tmem_ld16_nowait(tlane + DV_COL + c0, rv);
                tmem_ld16_nowait(tlane + DK_COL + c0, rk);
                tmem_ld_wait();
                tc_fence_before();
                warp_arrive(acc_free);
                if (kj < cur.sg.kLen) {  // a lane writes its own row slices: the stores retire in the background while the next item's tiles are worked on
                    const size_t grow = (size_t)(cur.sg.kStart + kj);
                    store_row_slice(rv, 1.f, a.dV + grow * a.lddv + cur.head * UHD + c0, nullptr);
                    store_row_slice(rk, a.scale, a.dK + grow * a.lddk + cur.head * UHD + c0,
                                    a.rope_table ? reinterpret_cast<const float4*>(a.rope_table + ((size_t)kpos * (UHD / 2) + (c0 >> 1)) * 2) : nullptr);
                }
            }
            if (ew_barrier_or(!okb)) {  // every element-wise thread votes once per item, whatever its status
                ok = false;
                break;
            }
            cur = nxt;
            have = haveN;
            n++;
        }
    } else if (warp < ISSUER2_WARP) {
        // ------------------------------------------------------------------------------ re-swizzle warps: Q, dO -> N-contiguous images
        const int t = threadIdx.x - RESWIZZLE_T0;
        uint8_t* ringK_p = tiles + 2 * T128;
        uint8_t* ringN_p = ringK_p + RING_K * 2 * T64;
        ItemWalk w(nTiles, nGroups);
        BwdItem it;
        bool ok = true;
        uint32_t g = 0;
        while (ok && next_dkv_item(w, a, it, -1)) {
            for (int i = 0; i < it.n; i++, g++) {
                const int sk = g % RING_K, sn = g % DKV_RING_N;
                ok = mbar_wait_warp(qk_full + 8 * sk, (g / RING_K) & 1, status, 39) && mbar_wait_warp(qn_empty + 8 * sn, ((g / DKV_RING_N) & 1) ^ 1, status, 40);
                if (!ok) break;
                reswizzle_tile(ringK_p + sk * 2 * T64, ringN_p + sn * 2 * T64, t);
                reswizzle_tile(ringK_p + sk * 2 * T64 + T64, ringN_p + sn * 2 * T64 + T64, t);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the MMA's reads
                warp_arrive(qn_full + 8 * sn);
                warp_arrive(qk_empty + 8 * sk);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tm), "r"(BWD_TMEM_COLS) : "memory");
    }
}

// rowDot[row, head] = sum_c dO[row, head*64 + c] * O[row, head*64 + c].  One warp per row: a lane owns one 16-byte piece of
// each 512-byte stretch of the row (two heads), so all its loads are issued before the first product, and the 16 lanes
// that share a head add up with four shuffles.
__global__ void __launch_bounds__(256) attn_rowdot_umma_kernel(const float* __restrict__ dO, int lddo, const float* __restrict__ O, int ldo, int rows,
                                                               int numHeads, float* __restrict__ rowDot) {
    const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float4* a = reinterpret_cast<const float4*>(dO + (size_t)row * lddo) + lane;
    const float4* b = reinterpret_cast<const float4*>(O + (size_t)row * ldo) + lane;
    for (int h0 = 0; h0 < numHeads; h0 += 16) {  // 16 heads (eight stretches of two) per round
        float4 x[8], y[8];
#pragma unroll
        for (int i = 0; i < 8; i++)
            if (h0 + 2 * i + (lane >> 4) < numHeads) { x[i] = a[(h0 / 2 + i) * 32]; y[i] = b[(h0 / 2 + i) * 32]; }  // an odd head count ends in half a stretch
#pragma unroll
        for (int i = 0; i < 8; i++) {
            if (h0 + 2 * i >= numHeads) break;  // warp-uniform
            const int head = h0 + 2 * i + (lane >> 4);
            float s = head < numHeads ? (x[i].x * y[i].x + x[i].y * y[i].y) + (x[i].z * y[i].z + x[i].w * y[i].w) : 0.f;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if ((lane & 15) == 0 && head < numHeads) rowDot[(size_t)row * numHeads + head] = s;
        }
    }
}

}  // namespace

int attn_umma_set_wait_budget(b200_ctx* ctx, long long clocks) {
    B200_CUDA(ctx, cudaMemcpyToSymbol(g_wait_budget_clocks, &clocks, sizeof(clocks)));
    return B200_OK;
}

bool attn_umma_eligible(b200_ctx* ctx, const Attn& t) {
    auto ok = [](const void* p, int ld) { return (((uintptr_t)p) & 15) == 0 && (ld & 3) == 0; };
    return ctx->cc_major == 10 && ctx->gemm_mode != B200_GEMM_FP32_SIMT && t.headDim == UHD && !t.mask && t.rowMax && t.rowSum && t.scale > 0.f &&
           t.maxQLen >= 128 && t.totalQ >= 128 && t.totalK >= 128 && ok(t.Q, t.ldq) && ok(t.K, t.ldk) && ok(t.V, t.ldv) && ok(t.O, t.ldo);
}

namespace {
int configure(b200_ctx* ctx) {
    B200_TRY(resolve_encode(ctx));
    B200_TRY(ensure_status(ctx));
    if (!ctx->attn_umma_configured) {
        B200_CUDA(ctx, cudaFuncSetAttribute(attn_fwd_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM));
        B200_CUDA(ctx, cudaFuncSetAttribute(attn_dq_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DQ_SMEM));
        B200_CUDA(ctx, cudaFuncSetAttribute(attn_dkv_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DKV_SMEM));
        ctx->attn_umma_configured = 1;
    }
    return B200_OK;
}
}  // namespace

// A head's 64 columns are two 32-column swizzle rows: one three-dimensional box brings both in one copy.
static int map2(b200_ctx* ctx, CUtensorMap* map, const float* base, uint64_t cols, uint64_t rows, uint64_t ld, uint32_t boxRows, bool mn_major) {
    if (make_map_chunked(ctx, map, base, cols, rows, ld, boxRows, 2, mn_major) != B200_OK)
        return fail(ctx, B200_ERR_CUDA, "cuTensorMapEncodeTiled refused the attention operand map (cols %llu rows %llu ld %llu)",
                    (unsigned long long)cols, (unsigned long long)rows, (unsigned long long)ld);
    return B200_OK;
}

bool attn_umma_bwd_eligible(b200_ctx* ctx, const Attn& t) {
    auto ok = [](const void* p, int ld) { return p && (((uintptr_t)p) & 15) == 0 && (ld & 3) == 0; };
    return attn_umma_eligible(ctx, t) && t.maxKLen >= 128 && t.rowDot && ok(t.dO, t.lddo) && ok(t.dQ, t.lddq) && ok(t.dK, t.lddk) && ok(t.dV, t.lddv);
}

int attn_backward_umma(b200_ctx* ctx, const Attn& t) {
    B200_TRY(configure(ctx));
    const uint64_t cols = (uint64_t)t.numHeads * UHD;
    const uint64_t nq = (uint64_t)t.totalQ, nk = (uint64_t)t.totalK;
    CUtensorMap q128, do128, k128, v128, q64, do64, k64, v64;
    B200_TRY(map2(ctx, &q128, t.Q, cols, nq, (uint64_t)t.ldq, 128, false));
    B200_TRY(map2(ctx, &do128, t.dO, cols, nq, (uint64_t)t.lddo, 128, false));
    B200_TRY(map2(ctx, &k128, t.K, cols, nk, (uint64_t)t.ldk, 128, false));
    B200_TRY(map2(ctx, &v128, t.V, cols, nk, (uint64_t)t.ldv, 128, false));
    B200_TRY(map2(ctx, &q64, t.Q, cols, nq, (uint64_t)t.ldq, 64, false));
    B200_TRY(map2(ctx, &do64, t.dO, cols, nq, (uint64_t)t.lddo, 64, false));
    B200_TRY(map2(ctx, &k64, t.K, cols, nk, (uint64_t)t.ldk, 64, false));
    B200_TRY(map2(ctx, &v64, t.V, cols, nk, (uint64_t)t.ldv, 64, false));
    UBwdArgs a;
    a.dQ = t.dQ; a.dK = t.dK; a.dV = t.dV; a.lddq = t.lddq; a.lddk = t.lddk; a.lddv = t.lddv;
    a.rowMax = t.rowMax; a.rowSum = t.rowSum; a.rowDot = t.rowDot; a.segs = t.segs_dev; a.numHeads = t.numHeads; a.causal = t.causal;
    a.scale = t.scale; a.status = ctx->status_dev; a.rope_table = t.rope_table; a.rope_pos = t.rope_pos;
    attn_rowdot_umma_kernel<<<(t.totalQ * 32 + 255) / 256, 256, 0, ctx->stream>>>(t.dO, t.lddo, t.O, t.ldo, t.totalQ, t.numHeads, t.rowDot);
    B200_LAUNCH_CHECK(ctx);
    // persistent kernels: one CTA per SM walks its share of the (segment, head, tile) pairs
    const int nGroups = t.numHeads * t.nSeg, sms = ctx->sm_count > 0 ? ctx->sm_count : 148;
    const int kTiles = (t.maxKLen + 127) / 128, qTiles = (t.maxQLen + 127) / 128;
    attn_dkv_umma_kernel<<<std::min(sms, nGroups * ((kTiles + 1) / 2)), B_THREADS, DKV_SMEM, ctx->stream>>>(k128, v128, q64, do64, a, kTiles, nGroups);
    B200_LAUNCH_CHECK(ctx);
    attn_dq_umma_kernel<<<std::min(sms, nGroups * ((qTiles + 1) / 2)), B_THREADS, DQ_SMEM, ctx->stream>>>(q128, do128, k64, v64, a, qTiles, nGroups);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

int attn_forward_umma(b200_ctx* ctx, const Attn& t) {
    B200_TRY(configure(ctx));
    const uint64_t cols = (uint64_t)t.numHeads * UHD;
    CUtensorMap mq, mk, mv;
    B200_TRY(map2(ctx, &mq, t.Q, cols, (uint64_t)t.totalQ, (uint64_t)t.ldq, 128, false));
    B200_TRY(map2(ctx, &mk, t.K, cols, (uint64_t)t.totalK, (uint64_t)t.ldk, 128, false));
    B200_TRY(map2(ctx, &mv, t.V, cols, (uint64_t)t.totalK, (uint64_t)t.ldv, 128, true));
    UArgs a;
    a.O = t.O; a.ldo = t.ldo; a.rowMax = t.rowMax; a.rowSum = t.rowSum; a.segs = t.segs_dev; a.numHeads = t.numHeads; a.causal = t.causal;
    a.scale = t.scale; a.status = ctx->status_dev;
    dim3 grid((t.maxQLen + UQ - 1) / UQ, t.numHeads, t.nSeg);
    attn_fwd_umma_kernel<<<grid, U_THREADS, FWD_SMEM, ctx->stream>>>(mq, mk, mv, a);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

}  // namespace b200
