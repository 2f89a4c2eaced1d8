// TF32 tensor-core GEMM for sm_100a: tcgen05.mma with the accumulator in tensor memory (TMEM), operands staged in
// shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle, every CTA loads its own tiles), an mbarrier pipeline, and the fused
// epilogue read back from TMEM with tcgen05.ld.
//
//   CTA tile 128 x BN (BN = 128), K step 32 floats (= one 128-byte swizzle row) per pipeline stage, 4 UMMAs
//   (M128 x N128 x K8) per stage.  192 threads: warp 0 = TMA producer (one elected lane), warp 1 = TMEM allocator and
//   MMA issuer (one elected lane), warps 2-5 = epilogue (each owns the 32 TMEM lanes its warp id modulo 4 selects).
//   Three stages of 32 KiB keep a CTA under 100 KiB so two CTAs share an SM: one runs its epilogue while the other
//   keeps the tensor pipe busy.
//
// All four operand layouts are supported without a transpose pass: a K-contiguous operand is one TMA box per stage
// and a K-major UMMA descriptor; an M/N-contiguous operand (dX = dY W uses W as [K,N]; dW = dY^T X uses both
// operands as [K,M] / [K,N]) is loaded as 32-column boxes and described as MN-major.  TMA converts FP32 to TF32 with
// round-to-nearest on the way in (tensor-map data type TFLOAT32); accumulation is FP32.
//
// Every wait on an mbarrier is bounded by a clock budget: on expiry the kernel raises a status word in host-mapped
// memory, drains the copies it still has in flight (bounded again), frees its TMEM and returns.
#include <cstdlib>

#include <type_traits>

#include "tcgen05.cuh"
#include "gemm_epilogue.cuh"

namespace b200 {

namespace {

constexpr int BM = 128, BK = 32;
constexpr int A_BYTES = BM * BK * 4;
constexpr int EPI_STRIDE64 = 68;                        // floats per staged row of 64 columns: 16-byte aligned, conflict-free 128-bit accesses
constexpr int EPI_STAGE_BYTES = 8 * 32 * EPI_STRIDE64 * 4;  // persistent kernel: up to 8 epilogue warps x 32 rows x 64 columns
// Tile configurations: 128 x 128 with three stages (two CTAs per SM), or 128 x 256 with four stages (one CTA per SM).
// A TF32 MMA with operands in shared memory reads (128 + N) x 32 bytes per K step of 8; at N = 128 that already equals
// the shared-memory bandwidth of the SM, and the TMA writes of the next stage come on top, so the wide tile (which
// reads 25% less shared memory per flop) is preferred whenever N allows it.
template <int BN_> struct TileCfg {
    static constexpr int STAGES = BN_ == 256 ? 3 : 4;
    static constexpr int EPI_WARPS = BN_ / 32;                 // one warp per (lane quarter, 128-column half)
    static constexpr int THREADS = 64 + 32 * EPI_WARPS;
    static constexpr int B_BYTES = BN_ * BK * 4, STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};
constexpr int THREADS = 192;
constexpr int GROUP_M = 16;

struct TcParams {
    int M, N, K;
    int a_mn_major, b_mn_major;  // 0: K contiguous (one box per stage); 1: M/N contiguous (32-column boxes)
    int a_box3d, b_box3d;        // M/N-contiguous operand fetched as ONE three-dimensional box (32 columns x BK rows x chunks)
    int* status;                 // host-mapped status word
    int kb_per_split;            // K blocks handled by one work item (split-K); all of them without a split
    long long split_stride;      // elements between the partial outputs of consecutive splits
    int items;                   // work items of the persistent schedule: C tiles x K splits
};

// Epilogue kinds.  GENERIC handles every field of Epilogue element by element.  The other three are the shapes the
// transformer step uses, written as 128-bit row operations (requirements checked on the host: N and every leading
// dimension a multiple of 4, 16-byte aligned bases):
//   LINEAR: v = alpha*acc (+bias) (+addmat); C = v or C += v
//   ACT   : z = acc + bias -> zout; C = act(z)                       (FFN hidden layer forward)
//   MULZ  : C = acc * act'(mulz)                                     (FFN hidden delta)
enum { EPI_GENERIC = 0, EPI_LINEAR = 1, EPI_ACT = 2, EPI_MULZ = 3 };
constexpr int EPI_STRIDE = 132;  // floats per staged row: 16-byte aligned and conflict-free for 128-bit accesses

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }

// Epilogue of one accumulator tile for one warp: 32 rows (TMEM lanes of quarter q) x 128 columns starting at colBase,
// read from TMEM at `acc`, transposed through the warp's staging slice, combined with the fused operands and stored.
// `release` is called (by every lane, after a warp-level sync) as soon as the warp has read its part of the accumulator.
template <int EPI, typename Release>
__device__ __forceinline__ void epilogue_tile(const Epilogue& ep, const TcParams& p, uint32_t acc, float* stage, int lane, int q, int colBase, int m0,
                                              int n0, int split, float alpha, Release release) {
    // Each warp transposes its accumulator rows through its own padded staging slice, which turns "one row per
    // thread" (the TMEM load shape) into "one row per half warp" and makes every global access of the epilogue
    // a full line.  The accumulator is handed back to the MMA warp as soon as this warp has read its part.
    if (EPI == EPI_GENERIC) {
#pragma unroll 1
        for (int c0 = 0; c0 < 128; c0 += 32) {
            const bool live = n0 + colBase + c0 < p.N;  // warp-uniform
            if (live) {
                uint32_t r[32];
                tmem_ld32(acc + (uint32_t)c0, r);
#pragma unroll
                for (int j = 0; j < 32; j++) stage[lane * 33 + j] = __uint_as_float(r[j]);
            }
            if (c0 == 96) {  // last chunk read: release the accumulator
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                release();
            }
            __syncwarp();
            const int n = n0 + colBase + c0 + lane;
            if (live && n < p.N) {
#pragma unroll 4
                for (int rr = 0; rr < 32; rr++) {
                    const int m = m0 + 32 * q + rr;
                    if (m < p.M) epilogue_store(ep, m, n, stage[rr * 33 + lane], alpha);
                }
            }
            __syncwarp();
        }
    } else {
        const int rsub = lane >> 4, l16 = lane & 15;
#pragma unroll 1
        for (int c0 = 0; c0 < 128; c0 += 64) {  // 64 accumulator columns per pass
            const bool live = n0 + colBase + c0 < p.N;  // warp-uniform (N is a multiple of 4, tiles start at multiples of 128)
            __syncwarp();
            if (live) {
                uint32_t r0[32], r1[32];
                tmem_ld32_nowait(acc + (uint32_t)c0, r0);
                tmem_ld32_nowait(acc + (uint32_t)(c0 + 32), r1);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    st4(stage + lane * EPI_STRIDE64 + j,
                        make_float4(__uint_as_float(r0[j]), __uint_as_float(r0[j + 1]), __uint_as_float(r0[j + 2]), __uint_as_float(r0[j + 3])));
                    st4(stage + lane * EPI_STRIDE64 + 32 + j,
                        make_float4(__uint_as_float(r1[j]), __uint_as_float(r1[j + 1]), __uint_as_float(r1[j + 2]), __uint_as_float(r1[j + 3])));
                }
            }
            if (c0 == 64) {  // last columns read: release the accumulator
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                release();
            }
            __syncwarp();
            const int n = n0 + colBase + c0 + 4 * l16;  // this lane's four columns; lanes 16..31 take the odd rows
            if (live && n < p.N) {
                float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
                if (EPI != EPI_MULZ && ep.bias) b4 = ld4(ep.bias + n);
                const bool rope = EPI == EPI_LINEAR && ep.rope_table && n < ep.rope_cols;
                const int rows = min(32, p.M - (m0 + 32 * q));
                if (EPI == EPI_ACT) {
                    // No operand loads to overlap here, so a rolled loop with ONE activation switch per row keeps the
                    // code small: the unrolled form below inlines every activation's code 32 times and ran out of
                    // the instruction cache (the warps spent more time waiting for instructions than storing).
#pragma unroll 2
                    for (int rr = rsub; rr < rows; rr += 2) {
                        const size_t m = (size_t)(m0 + 32 * q + rr);
                        float4 z = ld4(stage + rr * EPI_STRIDE64 + 4 * l16);
                        z.x += b4.x; z.y += b4.y; z.z += b4.z; z.w += b4.w;
                        if (ep.zout) st4(ep.zout + m * ep.ldz + n, z);
                        float4 a = z;
                        switch (ep.act) {
                            case B200_ACT_RELU: a.x = z.x > 0.f ? z.x : 0.f; a.y = z.y > 0.f ? z.y : 0.f; a.z = z.z > 0.f ? z.z : 0.f; a.w = z.w > 0.f ? z.w : 0.f; break;
                            case B200_ACT_NONE: break;
                            default: {
                                float d;
                                ffn_act_der(z.x, ep.act, a.x, d); ffn_act_der(z.y, ep.act, a.y, d);
                                ffn_act_der(z.z, ep.act, a.z, d); ffn_act_der(z.w, ep.act, a.w, d);
                            }
                        }
                        if (ep.act_sign_zero) { a.x = act_sign_zero(z.x, a.x); a.y = act_sign_zero(z.y, a.y); a.z = act_sign_zero(z.z, a.z); a.w = act_sign_zero(z.w, a.w); }
                        st4(ep.C + m * ep.ldc + n, a);
                    }
                    continue;
                }
                if (EPI == EPI_MULZ) {
                    // One copy of the batched row loop per derivative form, chosen once per pass: with the switch inside
                    // the unrolled loop every activation's code (exp, tanh) was inlined 32 times and the warps waited on
                    // instruction fetch.  MODE >= 0: derivative from the cached activation of that kind; -1: from z.
                    auto run = [&](auto MODE) {
                        constexpr int mode = decltype(MODE)::value;
#pragma unroll 1
                        for (int rb = 0; rb < rows; rb += 16) {
                            float4 ext[8];
#pragma unroll
                            for (int i = 0; i < 8; i++) {
                                const int rr = rb + 2 * i + rsub;
                                ext[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                                if (rr < rows) ext[i] = ld4(ep.mulz + (size_t)(m0 + 32 * q + rr) * ep.ldmulz + n);
                            }
#pragma unroll
                            for (int i = 0; i < 8; i++) {
                                const int rr = rb + 2 * i + rsub;
                                if (rr >= rows) continue;
                                float4 v = ld4(stage + rr * EPI_STRIDE64 + 4 * l16);
                                float a, dx, dy, dz, dw;
                                if (mode >= 0) {
                                    dx = ffn_der_from_act(ext[i].x, mode); dy = ffn_der_from_act(ext[i].y, mode);
                                    dz = ffn_der_from_act(ext[i].z, mode); dw = ffn_der_from_act(ext[i].w, mode);
                                } else {
                                    ffn_act_der(ext[i].x, ep.mulz_act, a, dx); ffn_act_der(ext[i].y, ep.mulz_act, a, dy);
                                    ffn_act_der(ext[i].z, ep.mulz_act, a, dz); ffn_act_der(ext[i].w, ep.mulz_act, a, dw);
                                }
                                v.x *= dx; v.y *= dy; v.z *= dz; v.w *= dw;
                                st4(ep.C + (size_t)(m0 + 32 * q + rr) * ep.ldc + n, v);
                            }
                        }
                    };
                    if (!ep.mulz_is_act) run(std::integral_constant<int, -1>{});
                    else switch (ep.mulz_act) {
                        case B200_ACT_RELU: run(std::integral_constant<int, B200_ACT_RELU>{}); break;
                        case B200_ACT_SIGMOID: run(std::integral_constant<int, B200_ACT_SIGMOID>{}); break;
                        case B200_ACT_TANH: run(std::integral_constant<int, B200_ACT_TANH>{}); break;
                        case B200_ACT_LEAKYRELU: run(std::integral_constant<int, B200_ACT_LEAKYRELU>{}); break;
                        default: run(std::integral_constant<int, B200_ACT_NONE>{}); break;
                    }
                    continue;
                }
                if (EPI == EPI_LINEAR && !ep.accumulate && !ep.addmat && !rope) {  // nothing to fetch: the same compact loop
#pragma unroll 2
                    for (int rr = rsub; rr < rows; rr += 2) {
                        const size_t m = (size_t)(m0 + 32 * q + rr);
                        float4 v = ld4(stage + rr * EPI_STRIDE64 + 4 * l16);
                        v.x = alpha * v.x + b4.x; v.y = alpha * v.y + b4.y; v.z = alpha * v.z + b4.z; v.w = alpha * v.w + b4.w;
                        if (ep.round_tf32) { v.x = tf32_round(v.x); v.y = tf32_round(v.y); v.z = tf32_round(v.z); v.w = tf32_round(v.w); }
                        st4(ep.C + (size_t)split * p.split_stride + m * ep.ldc + n, v);
                    }
                    continue;
                }
                // 16 rows (8 per half warp) per batch: all global loads of the batch are issued before any is consumed
#pragma unroll 1
                for (int rb = 0; rb < rows; rb += 16) {
                    float4 ext[8], ext2[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const int rr = rb + 2 * i + rsub;
                        const size_t m = (size_t)(m0 + 32 * q + rr);
                        ext[i] = ext2[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (rr < rows) {
                            if (EPI == EPI_LINEAR) {
                                if (ep.accumulate) ext[i] = ld4(ep.C + m * ep.ldc + n);
                                if (ep.addmat) ext2[i] = ld4(ep.addmat + m * ep.ldadd + n);
                                else if (rope) ext2[i] = rope_cs(ep, (int)m, n);  // (cos, sin) of this lane's two column pairs
                            } else if (EPI == EPI_MULZ) {
                                ext[i] = ld4(ep.mulz + m * ep.ldmulz + n);
                            }
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const int rr = rb + 2 * i + rsub;
                        if (rr >= rows) continue;
                        const size_t m = (size_t)(m0 + 32 * q + rr);
                        float4 v = ld4(stage + rr * EPI_STRIDE64 + 4 * l16);
                        if (EPI == EPI_LINEAR) {
                            v.x = alpha * v.x + b4.x + ext[i].x; v.y = alpha * v.y + b4.y + ext[i].y;
                            v.z = alpha * v.z + b4.z + ext[i].z; v.w = alpha * v.w + b4.w + ext[i].w;
                            if (rope) rope_rotate(ext2[i], v);
                            else { v.x += ext2[i].x; v.y += ext2[i].y; v.z += ext2[i].z; v.w += ext2[i].w; }
                            if (ep.round_tf32) { v.x = tf32_round(v.x); v.y = tf32_round(v.y); v.z = tf32_round(v.z); v.w = tf32_round(v.w); }
                            st4(ep.C + (size_t)split * p.split_stride + m * ep.ldc + n, v);
                        } else {  // EPI_MULZ
                            float a, dx, dy, dz, dw;
                            if (ep.mulz_is_act) {
                                dx = ffn_der_from_act(ext[i].x, ep.mulz_act); dy = ffn_der_from_act(ext[i].y, ep.mulz_act);
                                dz = ffn_der_from_act(ext[i].z, ep.mulz_act); dw = ffn_der_from_act(ext[i].w, ep.mulz_act);
                            } else {
                                ffn_act_der(ext[i].x, ep.mulz_act, a, dx); ffn_act_der(ext[i].y, ep.mulz_act, a, dy);
                                ffn_act_der(ext[i].z, ep.mulz_act, a, dz); ffn_act_der(ext[i].w, ep.mulz_act, a, dw);
                            }
                            v.x *= dx; v.y *= dy; v.z *= dz; v.w *= dw;
                            st4(ep.C + m * ep.ldc + n, v);
                        }
                    }
                }
            }
        }
    }
}

// Decode a work item (tile of C, K split) of the persistent schedule.  Tiles: bands of GROUP_M row-tiles are walked
// column by column, so the CTAs working at one time share a few A bands and B panels through L2 instead of streaming
// the whole B operand once per row-tile.
template <int BN>
__device__ __forceinline__ void decode_item(const TcParams& p, int item, int& m0, int& n0, int& split) {
    const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
    const int tiles = tiles_m * tiles_n;
    split = item / tiles;
    const int tile = item - split * tiles;
    const int per_group = GROUP_M * tiles_n;
    const int group = tile / per_group, first_m = group * GROUP_M;
    const int gm = min(tiles_m - first_m, GROUP_M);
    const int r = tile - group * per_group;
    m0 = (first_m + r % gm) * BM;
    n0 = (r / gm) * BN;
}

// Persistent kernel: one CTA per SM walks work items blockIdx.x, blockIdx.x + gridDim.x, ...  The operand ring and
// the two TMEM accumulators are shared by consecutive items, so the producer keeps loading and the MMA warp keeps
// issuing across item boundaries while the epilogue warps drain the previous accumulator.
template <int EPI, int BN>
__global__ void __launch_bounds__(TileCfg<BN>::THREADS) gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                                                               TcParams p, Epilogue ep) {
    constexpr int STAGES = TileCfg<BN>::STAGES, STAGE_BYTES = TileCfg<BN>::STAGE_BYTES;
    extern __shared__ uint8_t smem_raw[];
    // 128-byte swizzled tiles must start on 1024-byte boundaries
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    float* epi_stage = reinterpret_cast<float*>(tiles + STAGES * STAGE_BYTES);  // one 32 x 64 staging slice per epilogue warp
    uint64_t* bars = (uint64_t*)(tiles + STAGES * STAGE_BYTES + EPI_STAGE_BYTES);
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
    const uint32_t tiles_s = smem_u32(tiles);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES), acc_full0 = smem_u32(bars + 2 * STAGES),
                   acc_empty0 = smem_u32(bars + 2 * STAGES + 2);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kblocks_total = (p.K + BK - 1) / BK;
    const int n_items = p.items;
    volatile int* status = p.status;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full0 + 8 * b, 1);
            mbar_init(acc_empty0 + 8 * b, TileCfg<BN>::EPI_WARPS);  // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {  // TMEM: two accumulators of BN fp32 columns x 128 lanes
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ------------------------------------------------------------------ TMA producer
            int kc = 0;  // K blocks loaded so far, over all items: ring position and phase
            bool ok = true;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                int m0, n0, split;
                decode_item<BN>(p, item, m0, n0, split);
                const int kb_begin = split * p.kb_per_split;
                const int kblocks = min(kblocks_total - kb_begin, p.kb_per_split);
                for (int kb = 0; kb < kblocks; kb++, kc++) {
                    const int s = kc % STAGES;
                    ok = mbar_wait(empty0 + 8 * s, ((kc / STAGES) & 1) ^ 1, status, 1);  // first pass over the ring finds every slot empty
                    if (!ok) break;
                    const uint32_t a_dst = tiles_s + s * STAGE_BYTES, b_dst = a_dst + A_BYTES, bar = full0 + 8 * s;
                    mbar_expect_tx(bar, STAGE_BYTES);
                    const int k0 = (kb_begin + kb) * BK;
                    if (!p.a_mn_major) tma_load_2d(a_dst, &mapA, bar, k0, m0);
                    else
                        for (int c = 0; c < BM / 32; c++) tma_load_2d(a_dst + c * (BK * 128), &mapA, bar, m0 + 32 * c, k0);
                    if (!p.b_mn_major) tma_load_2d(b_dst, &mapB, bar, k0, n0);
                    else
                        for (int c = 0; c < BN / 32; c++) tma_load_2d(b_dst + c * (BK * 128), &mapB, bar, n0 + 32 * c, k0);
                }
            }
            if (!ok) {
                // failure path: wait (bounded) until the copies already issued have landed before the CTA may exit
                for (int k = (kc > STAGES ? kc - STAGES : 0); k < kc; k++) {
                    const long long t0 = clock64();
                    while (!mbar_test(full0 + 8 * (k % STAGES), (k / STAGES) & 1) && clock64() - t0 < WAIT_BUDGET_CLOCKS) __nanosleep(64);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ------------------------------------------------------------------ MMA issuer
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((p.a_mn_major ? 1u : 0u) << 15) | ((p.b_mn_major ? 1u : 0u) << 16) |
                                   ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            // K-major: rows 128 B apart, 8-row groups 1024 B apart (SBO), 32 B per K=8 step inside the swizzle row.
            // MN-major: 32-column chunks BK*128 B apart (LBO), K rows 128 B apart in groups of 4 rows, groups 512 B
            //           apart (SBO); one K=8 step is two groups = 1024 B.
            // The descriptors of stage 0 are built once; a stage or a K step only adds to the address field.
            const uint64_t a_d0 = umma_desc(tiles_s, p.a_mn_major ? BK * 128 : 16, p.a_mn_major ? 512 : 1024, p.a_mn_major ? 1 : 2);
            const uint64_t b_d0 = umma_desc(tiles_s + A_BYTES, p.b_mn_major ? BK * 128 : 16, p.b_mn_major ? 512 : 1024, p.b_mn_major ? 1 : 2);
            const uint64_t a_step = p.a_mn_major ? (1024 >> 4) : (32 >> 4), b_step = p.b_mn_major ? (1024 >> 4) : (32 >> 4);
            int kc = 0, it = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, it++) {
                int m0, n0, split;
                decode_item<BN>(p, item, m0, n0, split);
                const int kblocks = min(kblocks_total - split * p.kb_per_split, p.kb_per_split);
                const int buf = it & 1;
                ok = mbar_wait(acc_empty0 + 8 * buf, ((it >> 1) & 1) ^ 1, status, 4);  // the epilogue has drained this accumulator
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem_base + (uint32_t)(buf * BN);
                for (int kb = 0; kb < kblocks; kb++, kc++) {
                    const int s = kc % STAGES;
                    ok = mbar_wait(full0 + 8 * s, (kc / STAGES) & 1, status, 2);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t so = (uint64_t)(s * (STAGE_BYTES >> 4));
#pragma unroll
                    for (int kk = 0; kk < BK / 8; kk++) umma_tf32(acc, a_d0 + so + kk * a_step, b_d0 + so + kk * b_step, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                    umma_commit(empty0 + 8 * s);  // frees the stage once these MMAs have read it
                }
                umma_commit(acc_full0 + 8 * buf);  // accumulator complete (also issued on the failure path so nobody waits forever)
            }
        }
    } else {
        // ---------------------------------------------------------------------- epilogue (warps 2 .. 2+EW-1)
        // A warp owns 32 accumulator rows (the TMEM lanes its warp id modulo 4 selects) and 128 of the tile's columns:
        // with the wide tile two warps share a lane quarter, one per column half.
        const int q = warp & 3, ew = warp - 2;
        const int colBase = (ew >> 2) * 128;
        float alpha = ep.alpha;
        if (ep.alpha_dev) alpha *= ep.alpha_dev[0];
        float* stage = epi_stage + ew * (32 * EPI_STRIDE64);
        int it = 0;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x, it++) {
            int m0, n0, split;
            decode_item<BN>(p, item, m0, n0, split);
            const int buf = it & 1;
            const uint32_t acc = tmem_base + (uint32_t)(buf * BN + colBase) + ((uint32_t)(32 * q) << 16);
            if (!mbar_wait_warp(acc_full0 + 8 * buf, (it >> 1) & 1, status, 3)) break;  // tcgen05.ld is warp-collective: the warp decides together
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            epilogue_tile<EPI>(ep, p, acc, stage, lane, q, colBase, m0, n0, split, alpha, [&] {
                if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
            });
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------ two SMs per tile
// Persistent kernel on clusters of two CTAs: a pair works on a 256 x 256 tile of C with tcgen05.mma.cta_group::2.  Each
// CTA loads its own 128 rows of A and half of the tile's B rows (128 of the 256 N), so per K step of 8 an SM reads
// 8 KiB of shared memory for twice the flops of the one-CTA 128 x 128 MMA -- the one-CTA kernels are bound by exactly
// that shared-memory traffic.  The leader CTA (cluster rank 0) issues the MMAs; the TMA loads of both CTAs signal the
// leader's "full" barrier; tcgen05.commit arrives on the "empty" / "accumulator full" barriers of both CTAs; the
// epilogue warps of both CTAs hand an accumulator back by arriving on the leader's "accumulator empty" barrier.
constexpr int PAIR_BN = 256, PAIR_STAGES = 4, PAIR_EPI_WARPS = 8, PAIR_THREADS = 64 + 32 * PAIR_EPI_WARPS;
constexpr int PAIR_B_BYTES = 128 * BK * 4, PAIR_STAGE_BYTES = A_BYTES + PAIR_B_BYTES;
constexpr int PAIR_SMEM_BYTES = PAIR_STAGES * PAIR_STAGE_BYTES + EPI_STAGE_BYTES + 1024 + 256;

__device__ __forceinline__ void decode_pair_item(const TcParams& p, int item, int& m0, int& n0, int& split) {
    const int tiles_m = (p.M + 255) / 256, tiles_n = (p.N + PAIR_BN - 1) / PAIR_BN;
    const int tiles = tiles_m * tiles_n;
    split = item / tiles;
    const int tile = item - split * tiles;
    const int per_group = (GROUP_M / 2) * tiles_n;
    const int group = tile / per_group, first_m = group * (GROUP_M / 2);
    const int gm = min(tiles_m - first_m, GROUP_M / 2);
    const int r = tile - group * per_group;
    m0 = (first_m + r % gm) * 256;
    n0 = (r / gm) * PAIR_BN;
}

template <int EPI>
__global__ void __launch_bounds__(PAIR_THREADS) gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                                                                        TcParams p, Epilogue ep) {
    constexpr int STAGES = PAIR_STAGES, STAGE_BYTES = PAIR_STAGE_BYTES, BN = PAIR_BN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    float* epi_stage = reinterpret_cast<float*>(tiles + STAGES * STAGE_BYTES);
    uint64_t* bars = (uint64_t*)(tiles + STAGES * STAGE_BYTES + EPI_STAGE_BYTES);
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
    const uint32_t tiles_s = smem_u32(tiles);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES), acc_full0 = smem_u32(bars + 2 * STAGES),
                   acc_empty0 = smem_u32(bars + 2 * STAGES + 2);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0 = leader
    const int cluster = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    const int kblocks_total = (p.K + BK - 1) / BK;
    const int n_items = p.items;
    volatile int* status = p.status;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);   // used in the leader: its own arrive.expect_tx; bytes arrive from both CTAs
            mbar_init(empty0 + 8 * s, 1);  // one multicast commit per phase, in both CTAs
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full0 + 8 * b, 1);                    // multicast commit, in both CTAs
            mbar_init(acc_empty0 + 8 * b, 2 * PAIR_EPI_WARPS);  // used in the leader: the epilogue warps of both CTAs
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {  // TMEM of the pair: two accumulators of 256 fp32 columns x 128 lanes in each CTA
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs, whole warp: one copy per lane)
        const int nA = (p.a_mn_major && !p.a_box3d) ? 4 : 1, nB = (p.b_mn_major && !p.b_box3d) ? 4 : 1;
        int kc = 0;
        bool ok = true;
        for (int item = cluster; item < n_items && ok; item += n_clusters) {
            int m0, n0, split;
            decode_pair_item(p, item, m0, n0, split);
            const int my_m = m0 + 128 * (int)rank, my_n = n0 + 128 * (int)rank;
            const int kb_begin = split * p.kb_per_split;
            const int kblocks = min(kblocks_total - kb_begin, p.kb_per_split);
            for (int kb = 0; kb < kblocks; kb++, kc++) {
                const int s = kc % STAGES;
                ok = mbar_wait_warp(empty0 + 8 * s, ((kc / STAGES) & 1) ^ 1, status, 41);
                if (!ok) break;
                const uint32_t a_dst = tiles_s + s * STAGE_BYTES, b_dst = a_dst + A_BYTES;
                const uint32_t bar = mapa_cluster(full0 + 8 * s, 0);  // the leader's barrier
                if (rank == 0 && lane == 0) mbar_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);
                __syncwarp();
                const int k0 = (kb_begin + kb) * BK;
                if (lane < nA) {
                    if (!p.a_mn_major) tma_load_2d_pair(a_dst, &mapA, bar, k0, my_m);
                    else if (p.a_box3d) tma_load_3d_pair(a_dst, &mapA, bar, 0, k0, my_m >> 5);
                    else tma_load_2d_pair(a_dst + lane * (BK * 128), &mapA, bar, my_m + 32 * lane, k0);
                } else if (lane < nA + nB) {
                    const int c = lane - nA;
                    if (!p.b_mn_major) tma_load_2d_pair(b_dst, &mapB, bar, k0, my_n);
                    else if (p.b_box3d) tma_load_3d_pair(b_dst, &mapB, bar, 0, k0, my_n >> 5);
                    else tma_load_2d_pair(b_dst + c * (BK * 128), &mapB, bar, my_n + 32 * c, k0);
                }
            }
        }
        if (!ok) {  // failure path: give the copies already issued time to land before the CTA may exit
            const long long t0 = clock64();
            while (clock64() - t0 < 4000000LL) __nanosleep(256);
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ------------------------------------------------------------------ MMA issuer (leader CTA only)
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((p.a_mn_major ? 1u : 0u) << 15) | ((p.b_mn_major ? 1u : 0u) << 16) |
                                   ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
            const uint64_t a_d0 = umma_desc(tiles_s, p.a_mn_major ? BK * 128 : 16, p.a_mn_major ? 512 : 1024, p.a_mn_major ? 1 : 2);
            const uint64_t b_d0 = umma_desc(tiles_s + A_BYTES, p.b_mn_major ? BK * 128 : 16, p.b_mn_major ? 512 : 1024, p.b_mn_major ? 1 : 2);
            const uint64_t a_step = p.a_mn_major ? (1024 >> 4) : (32 >> 4), b_step = p.b_mn_major ? (1024 >> 4) : (32 >> 4);
            int kc = 0, it = 0;
            bool ok = true;
            for (int item = cluster; item < n_items && ok; item += n_clusters, it++) {
                int m0, n0, split;
                decode_pair_item(p, item, m0, n0, split);
                const int kblocks = min(kblocks_total - split * p.kb_per_split, p.kb_per_split);
                const int buf = it & 1;
                ok = mbar_wait(acc_empty0 + 8 * buf, ((it >> 1) & 1) ^ 1, status, 44);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem_base + (uint32_t)(buf * BN);
                for (int kb = 0; kb < kblocks; kb++, kc++) {
                    const int s = kc % STAGES;
                    ok = mbar_wait(full0 + 8 * s, (kc / STAGES) & 1, status, 42);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t so = (uint64_t)(s * (STAGE_BYTES >> 4));
#pragma unroll
                    for (int kk = 0; kk < BK / 8; kk++)
                        umma_tf32_pair(acc, a_d0 + so + kk * a_step, b_d0 + so + kk * b_step, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                    umma_commit_pair(empty0 + 8 * s);
                }
                umma_commit_pair(acc_full0 + 8 * buf);
            }
        }
    } else {
        // ---------------------------------------------------------------------- epilogue (both CTAs, warps 2..9)
        const int q = warp & 3, ew = warp - 2;
        const int colBase = (ew >> 2) * 128;
        float alpha = ep.alpha;
        if (ep.alpha_dev) alpha *= ep.alpha_dev[0];
        float* stage = epi_stage + ew * (32 * EPI_STRIDE64);
        int it = 0;
        for (int item = cluster; item < n_items; item += n_clusters, it++) {
            int m0, n0, split;
            decode_pair_item(p, item, m0, n0, split);
            const int buf = it & 1;
            const uint32_t acc = tmem_base + (uint32_t)(buf * BN + colBase) + ((uint32_t)(32 * q) << 16);
            if (!mbar_wait_warp(acc_full0 + 8 * buf, (it >> 1) & 1, status, 43)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t release_bar = mapa_cluster(acc_empty0 + 8 * buf, 0);
            epilogue_tile<EPI>(ep, p, acc, stage, lane, q, colBase, m0 + 128 * (int)rank, n0, split, alpha, [&] {
                if (lane == 0) mbar_arrive_cluster(release_bar);
            });
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();  // nobody leaves while the peer may still read its shared memory or arrive on its barriers
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------ one tile per CTA
// 128 x 128 tile, three stages of 32 KiB, two CTAs per SM (one runs its epilogue while the other keeps the tensor pipe
// busy).  Used for split-K and for long K, where it measures faster than the persistent kernel above.
constexpr int T_BN = 128, T_STAGES = 3;
constexpr int T_B_BYTES = T_BN * BK * 4, T_STAGE_BYTES = A_BYTES + T_B_BYTES;
constexpr int T_SMEM_BYTES = T_STAGES * T_STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;

template <int EPI>
__global__ void __launch_bounds__(THREADS) gemm_tcgen05_tile_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                                                               TcParams p, Epilogue ep) {
    extern __shared__ uint8_t smem_raw[];
    // 128-byte swizzled tiles must start on 1024-byte boundaries
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(tiles + T_STAGES * T_STAGE_BYTES);
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * T_STAGES + 1);
    const uint32_t tiles_s = smem_u32(tiles);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + T_STAGES), accum_bar = smem_u32(bars + 2 * T_STAGES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Tile order: bands of GROUP_M row-tiles are walked column by column, so the CTAs resident at one time share a few
    // A bands and B panels through L2 instead of streaming the whole B operand once per row-tile.
    int m0, n0;
    {
        const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + T_BN - 1) / T_BN;
        const int per_group = GROUP_M * tiles_n;
        const int group = blockIdx.x / per_group, first_m = group * GROUP_M;
        const int gm = min(tiles_m - first_m, GROUP_M);
        const int r = blockIdx.x - group * per_group;
        m0 = (first_m + r % gm) * BM;
        n0 = (r / gm) * T_BN;
    }
    const int kb_begin = blockIdx.y * p.kb_per_split;
    const int kblocks = min((p.K + BK - 1) / BK - kb_begin, p.kb_per_split);  // K blocks of this split
    volatile int* status = p.status;

    if (threadIdx.x == 0) {
        for (int s = 0; s < T_STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {  // TMEM: T_BN fp32 accumulator columns x 128 lanes
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(T_BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (whole warp)
        // Lane 0 waits for the slot and posts the byte count; then every copy of the stage is issued by its own lane in
        // one warp instruction -- an M/N-contiguous operand is four 32-column boxes, and a single thread issuing eight
        // copies per stage was slower than the MMAs that consume them.
        const int nA = (p.a_mn_major && !p.a_box3d) ? BM / 32 : 1, nB = (p.b_mn_major && !p.b_box3d) ? T_BN / 32 : 1;
        int issued = 0;
        bool ok = true;
        for (int kb = 0; kb < kblocks && ok; kb++) {
            const int s = kb % T_STAGES;
            const uint32_t par = ((kb / T_STAGES) & 1) ^ 1;  // first pass over the ring finds every slot empty
            ok = mbar_wait_warp(empty0 + 8 * s, par, status, 1);
            if (!ok) break;
            const uint32_t a_dst = tiles_s + s * T_STAGE_BYTES, b_dst = a_dst + A_BYTES, bar = full0 + 8 * s;
            if (lane == 0) mbar_expect_tx(bar, T_STAGE_BYTES);
            __syncwarp();
            const int k0 = (kb_begin + kb) * BK;
            if (lane < nA) {
                if (!p.a_mn_major) tma_load_2d(a_dst, &mapA, bar, k0, m0);
                else if (p.a_box3d) tma_load_3d(a_dst, &mapA, bar, 0, k0, m0 >> 5);
                else tma_load_2d(a_dst + lane * (BK * 128), &mapA, bar, m0 + 32 * lane, k0);
            } else if (lane < nA + nB) {
                const int c = lane - nA;
                if (!p.b_mn_major) tma_load_2d(b_dst, &mapB, bar, k0, n0);
                else if (p.b_box3d) tma_load_3d(b_dst, &mapB, bar, 0, k0, n0 >> 5);
                else tma_load_2d(b_dst + c * (BK * 128), &mapB, bar, n0 + 32 * c, k0);
            }
            issued = kb + 1;
        }
        if (!ok && lane == 0) {
            // failure path: wait (bounded) until the copies already issued have landed before the CTA may exit
            for (int kb = (issued > T_STAGES ? issued - T_STAGES : 0); kb < issued; kb++) {
                const long long t0 = clock64();
                while (!mbar_test(full0 + 8 * (kb % T_STAGES), (kb / T_STAGES) & 1) && clock64() - t0 < WAIT_BUDGET_CLOCKS) __nanosleep(64);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ------------------------------------------------------------------ MMA issuer
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((p.a_mn_major ? 1u : 0u) << 15) | ((p.b_mn_major ? 1u : 0u) << 16) |
                                   ((uint32_t)(T_BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            // K-major: rows 128 B apart, 8-row groups 1024 B apart (SBO), 32 B per K=8 step inside the swizzle row.
            // MN-major: 32-column chunks BK*128 B apart (LBO), K rows 128 B apart in groups of 4 rows, groups 512 B
            //           apart (SBO); one K=8 step is two groups = 1024 B.
            const uint32_t a_lbo = p.a_mn_major ? BK * 128 : 16, b_lbo = p.b_mn_major ? BK * 128 : 16;
            const uint32_t a_sbo = p.a_mn_major ? 512 : 1024, b_sbo = p.b_mn_major ? 512 : 1024;
            const uint32_t a_lay = p.a_mn_major ? 1 : 2, b_lay = p.b_mn_major ? 1 : 2;
            const uint32_t a_step = p.a_mn_major ? 1024 : 32, b_step = p.b_mn_major ? 1024 : 32;
            bool ok = true;
            for (int kb = 0; kb < kblocks; kb++) {
                const int s = kb % T_STAGES;
                ok = mbar_wait(full0 + 8 * s, (kb / T_STAGES) & 1, status, 2);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_s = tiles_s + s * T_STAGE_BYTES, b_s = a_s + A_BYTES;
#pragma unroll
                for (int kk = 0; kk < BK / 8; kk++) {
                    const uint64_t ad = umma_desc(a_s + kk * a_step, a_lbo, a_sbo, a_lay);
                    const uint64_t bd = umma_desc(b_s + kk * b_step, b_lbo, b_sbo, b_lay);
                    umma_tf32(tmem_base, ad, bd, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(empty0 + 8 * s);  // frees the stage once these MMAs have read it
            }
            umma_commit(accum_bar);  // accumulator complete (also issued on the failure path so nobody waits forever)
        }
    } else {
        // ---------------------------------------------------------------------- epilogue (warps 2..5)
        const bool ok = mbar_wait_warp(accum_bar, 0, status, 3);  // one polling lane per warp; tcgen05.ld is warp-collective, so the warp decides together
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            const int q = warp & 3;  // this warp may touch TMEM lanes [32q, 32q+32)
            float alpha = ep.alpha;
            if (ep.alpha_dev) alpha *= ep.alpha_dev[0];
            // All MMAs have completed, so the operand stages are free: each warp transposes its accumulator rows
            // through a padded slice of them, which turns "one row per thread" (the TMEM load shape) into "one row
            // per warp instruction" and makes every global access of the epilogue a full line.
            if (EPI == EPI_GENERIC) {
                float* stage = reinterpret_cast<float*>(tiles) + q * (32 * 33);
#pragma unroll 1
                for (int c0 = 0; c0 < T_BN; c0 += 32) {
                    if (n0 + c0 >= p.N) break;
                    uint32_t r[32];
                    tmem_ld32(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)c0, r);
#pragma unroll
                    for (int j = 0; j < 32; j++) stage[lane * 33 + j] = __uint_as_float(r[j]);
                    __syncwarp();
                    const int n = n0 + c0 + lane;
                    if (n < p.N) {
#pragma unroll 4
                        for (int rr = 0; rr < 32; rr++) {
                            const int m = m0 + 32 * q + rr;
                            if (m < p.M) epilogue_store(ep, m, n, stage[rr * 33 + lane], alpha);
                        }
                    }
                    __syncwarp();
                }
            } else {
                float* stage = reinterpret_cast<float*>(tiles) + q * (32 * EPI_STRIDE);
#pragma unroll 1
                for (int c0 = 0; c0 < T_BN; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld32(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)c0, r);
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        st4(stage + lane * EPI_STRIDE + c0 + j,
                            make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])));
                }
                __syncwarp();
                const int n = n0 + 4 * lane;  // this lane's four columns of every row
                if (n < p.N) {                // N is a multiple of 4 on this path
                    float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (EPI != EPI_MULZ && ep.bias) b4 = ld4(ep.bias + n);
                    const bool rope = EPI == EPI_LINEAR && ep.rope_table && n < ep.rope_cols;
                    const int rows = min(32, p.M - (m0 + 32 * q));
                    // 8 rows per batch: all global loads of the batch are issued before any of them is consumed
#pragma unroll 1
                    for (int r0 = 0; r0 < rows; r0 += 8) {
                        float4 ext[8], ext2[8];
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            const size_t m = (size_t)(m0 + 32 * q + r0 + i);
                            ext[i] = ext2[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                            if (r0 + i < rows) {
                                if (EPI == EPI_LINEAR) {
                                    if (ep.accumulate) ext[i] = ld4(ep.C + m * ep.ldc + n);
                                    if (ep.addmat) ext2[i] = ld4(ep.addmat + m * ep.ldadd + n);
                                    else if (rope) ext2[i] = rope_cs(ep, (int)m, n);  // (cos, sin) of this lane's two column pairs
                                } else if (EPI == EPI_MULZ) {
                                    ext[i] = ld4(ep.mulz + m * ep.ldmulz + n);
                                }
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            if (r0 + i >= rows) break;
                            const size_t m = (size_t)(m0 + 32 * q + r0 + i);
                            float4 v = ld4(stage + (r0 + i) * EPI_STRIDE + 4 * lane);
                            if (EPI == EPI_LINEAR) {
                                v.x = alpha * v.x + b4.x + ext[i].x; v.y = alpha * v.y + b4.y + ext[i].y;
                                v.z = alpha * v.z + b4.z + ext[i].z; v.w = alpha * v.w + b4.w + ext[i].w;
                                if (rope) rope_rotate(ext2[i], v);
                                else { v.x += ext2[i].x; v.y += ext2[i].y; v.z += ext2[i].z; v.w += ext2[i].w; }
                                if (ep.round_tf32) { v.x = tf32_round(v.x); v.y = tf32_round(v.y); v.z = tf32_round(v.z); v.w = tf32_round(v.w); }
                                st4(ep.C + (size_t)blockIdx.y * p.split_stride + m * ep.ldc + n, v);
                            } else if (EPI == EPI_ACT) {
                                v.x += b4.x; v.y += b4.y; v.z += b4.z; v.w += b4.w;
                                if (ep.zout) st4(ep.zout + m * ep.ldz + n, v);
                                const float4 z = v;
                                float d;
                                ffn_act_der(v.x, ep.act, v.x, d); ffn_act_der(v.y, ep.act, v.y, d);
                                ffn_act_der(v.z, ep.act, v.z, d); ffn_act_der(v.w, ep.act, v.w, d);
                                if (ep.act_sign_zero) { v.x = act_sign_zero(z.x, v.x); v.y = act_sign_zero(z.y, v.y); v.z = act_sign_zero(z.z, v.z); v.w = act_sign_zero(z.w, v.w); }
                                st4(ep.C + m * ep.ldc + n, v);
                            } else {  // EPI_MULZ
                                float a, dx, dy, dz, dw;
                                if (ep.mulz_is_act) {
                                    dx = ffn_der_from_act(ext[i].x, ep.mulz_act); dy = ffn_der_from_act(ext[i].y, ep.mulz_act);
                                    dz = ffn_der_from_act(ext[i].z, ep.mulz_act); dw = ffn_der_from_act(ext[i].w, ep.mulz_act);
                                } else {
                                    ffn_act_der(ext[i].x, ep.mulz_act, a, dx); ffn_act_der(ext[i].y, ep.mulz_act, a, dy);
                                    ffn_act_der(ext[i].z, ep.mulz_act, a, dz); ffn_act_der(ext[i].w, ep.mulz_act, a, dw);
                                }
                                v.x *= dx; v.y *= dy; v.z *= dz; v.w *= dw;
                                st4(ep.C + m * ep.ldc + n, v);
                            }
                        }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(T_BN) : "memory");
    }
}

// C[m,n] (+)= alpha * sum_s partial[s][m,n], splits added in index order (N a multiple of 4).
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int splits, int M, int N, float* __restrict__ C, int ldc, float alpha,
                                     const float* __restrict__ alpha_dev, int accumulate) {
    const int64_t n4 = (int64_t)M * N / 4, plane = (int64_t)M * N;
    if (alpha_dev) alpha *= alpha_dev[0];
    const bool vecC = (ldc % 4 == 0) && (((uintptr_t)C & 15) == 0);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
        float4 s = ld4(partial + 4 * i);
        for (int k = 1; k < splits; k++) {
            const float4 v = ld4(partial + k * plane + 4 * i);
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        const int64_t e = 4 * i;
        const int m = (int)(e / N), n = (int)(e - (int64_t)m * N);
        float* c = C + (size_t)m * ldc + n;
        if (vecC) {
            float4 o = accumulate ? ld4(c) : make_float4(0.f, 0.f, 0.f, 0.f);
            o.x += alpha * s.x; o.y += alpha * s.y; o.z += alpha * s.z; o.w += alpha * s.w;
            st4(c, o);
        } else {
            c[0] = (accumulate ? c[0] : 0.f) + alpha * s.x; c[1] = (accumulate ? c[1] : 0.f) + alpha * s.y;
            c[2] = (accumulate ? c[2] : 0.f) + alpha * s.z; c[3] = (accumulate ? c[3] : 0.f) + alpha * s.w;
        }
    }
}

}  // namespace

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int resolve_encode(b200_ctx* ctx) {
    if (ctx->tmap_encode) return B200_OK;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    B200_CUDA(ctx, cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    if (!fn || q != cudaDriverEntryPointSuccess) return fail(ctx, B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    ctx->tmap_encode = fn;
    return B200_OK;
}

int make_map(b200_ctx* ctx, CUtensorMap* map, const float* base, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t boxOuter, bool mn_major) {
    cuuint64_t gdim[2] = {inner, outer};
    cuuint64_t gstride[1] = {ld * sizeof(float)};
    cuuint32_t box[2] = {32, boxOuter};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = ((EncodeTiledFn)ctx->tmap_encode)(map, CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 2, (void*)base, gdim, gstride, box, estr,
                                                   CU_TENSOR_MAP_INTERLEAVE_NONE, mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ctx, B200_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d (inner %llu outer %llu ld %llu)", (int)r,
                                       (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)ld);
    return B200_OK;
}

// Several 32-column chunks of a row-major matrix as one three-dimensional box (used for M/N-contiguous GEMM operands
// and for the 64-wide head slices of attention): dimension 0 = 32 contiguous elements (one 128-byte swizzle
// row), dimension 1 = the K rows (stride ld), dimension 2 = the 32-column chunks of the row (stride 128 bytes).  A box
// of 32 x boxK x chunks lands in shared memory as [chunk][k][32], the layout the M/N-major UMMA descriptors read, with
// one copy instruction instead of one per chunk.  The chunks are synthetic, so the extent along M/N must be a
// multiple of 32 (nothing else keeps the last chunk inside the row); rows beyond K are zero-filled by the copy.
int make_map_chunked(b200_ctx* ctx, CUtensorMap* map, const float* base, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t boxOuter,
                     uint32_t chunks, bool mn_major) {
    cuuint64_t gdim[3] = {32, outer, inner / 32};
    cuuint64_t gstride[2] = {ld * sizeof(float), 32 * sizeof(float)};
    cuuint32_t box[3] = {32, boxOuter, chunks};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = ((EncodeTiledFn)ctx->tmap_encode)(map, CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 3, (void*)base, gdim, gstride, box, estr,
                                                   CU_TENSOR_MAP_INTERLEAVE_NONE, mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? B200_OK : B200_ERR_UNSUPPORTED;
}
int make_map_mn3d(b200_ctx* ctx, CUtensorMap* map, const float* base, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t boxK, uint32_t chunks) {
    return make_map_chunked(ctx, map, base, inner, outer, ld, boxK, chunks, true);  // the caller falls back to 32-column boxes
}

int ensure_status(b200_ctx* ctx) {
    if (ctx->status_host) return B200_OK;
    B200_CUDA(ctx, cudaHostAlloc((void**)&ctx->status_host, sizeof(int), cudaHostAllocMapped));
    *ctx->status_host = 0;
    B200_CUDA(ctx, cudaHostGetDevicePointer((void**)&ctx->status_dev, ctx->status_host, 0));
    return B200_OK;
}

int gemm_tcgen05_set_wait_budget(b200_ctx* ctx, long long clocks) {
    B200_CUDA(ctx, cudaMemcpyToSymbol(g_wait_budget_clocks, &clocks, sizeof(clocks)));
    return B200_OK;
}

namespace {
// The expiry path of the bounded waits, without any real failure: one thread initialises a barrier that expects one
// arrival and waits for a phase nobody completes.  mbar_wait gives up after the budget, raises the status word and
// returns false; the kernel then simply ends (it holds no tensor memory and has no copy in flight).
__global__ void bounded_wait_probe_kernel(volatile int* status, int* gave_up) {
    __shared__ __align__(8) unsigned long long bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const bool ok = mbar_wait(smem_u32(&bar), 0, status, 9);
        *gave_up = ok ? 0 : 1;
    }
}
}  // namespace

int gemm_tcgen05_probe_wait(b200_ctx* ctx) {
    B200_TRY(ensure_status(ctx));
    B200_TRY(ensure_ws(ctx, 64));
    int* flag = (int*)ctx->ws;
    B200_CUDA(ctx, cudaMemsetAsync(flag, 0, sizeof(int), ctx->stream));
    bounded_wait_probe_kernel<<<1, 32, 0, ctx->stream>>>(ctx->status_dev, flag);
    B200_LAUNCH_CHECK(ctx);
    int gave_up = 0;
    B200_CUDA(ctx, cudaMemcpyAsync(ctx->pinned, flag, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    gave_up = *(int*)ctx->pinned;
    int rc = check_device_status(ctx);
    if (rc == B200_OK && gave_up) return fail(ctx, B200_ERR_CUDA, "the wait expired but the status word was not raised");
    return rc;
}

bool gemm_tcgen05_eligible(b200_ctx* ctx, const Gemm& g) {
    if (ctx->cc_major != 10) return false;
    if (g.M < 128 || g.N < 128 || g.K < 128) return false;
    if ((g.lda & 3) || (g.ldb & 3)) return false;
    if (((uintptr_t)g.A | (uintptr_t)g.B) & 15) return false;
    return true;
}

namespace {
template <int BN>
int gemm_tcgen05_persistent(b200_ctx* ctx, const Gemm& g) {
    ctx->engine_launches[B200_ENGINE_GEMM_PERSISTENT]++;
    constexpr int SMEM_BYTES = TileCfg<BN>::SMEM_BYTES;
    static char configured_site;  // one per tile width (template instantiation); remembered per context, i.e. per device
    if (first_use(ctx, &configured_site)) {
        B200_CUDA(ctx, cudaFuncSetAttribute(gemm_tcgen05_persistent_kernel<EPI_GENERIC, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        B200_CUDA(ctx, cudaFuncSetAttribute(gemm_tcgen05_persistent_kernel<EPI_LINEAR, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        B200_CUDA(ctx, cudaFuncSetAttribute(gemm_tcgen05_persistent_kernel<EPI_ACT, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        B200_CUDA(ctx, cudaFuncSetAttribute(gemm_tcgen05_persistent_kernel<EPI_MULZ, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    }
    CUtensorMap mapA, mapB;
    // A: stored [M,K] (K contiguous) or [K,M] (M contiguous).  B: stored [N,K] (transB, K contiguous) or [K,N].
    if (!g.transA) B200_TRY(make_map(ctx, &mapA, g.A, (uint64_t)g.K, (uint64_t)g.M, (uint64_t)g.lda, BM, false));
    else B200_TRY(make_map(ctx, &mapA, g.A, (uint64_t)g.M, (uint64_t)g.K, (uint64_t)g.lda, BK, true));
    if (g.transB) B200_TRY(make_map(ctx, &mapB, g.B, (uint64_t)g.K, (uint64_t)g.N, (uint64_t)g.ldb, BN, false));
    else B200_TRY(make_map(ctx, &mapB, g.B, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.ldb, BK, true));
    TcParams p;
    p.M = g.M; p.N = g.N; p.K = g.K;
    p.a_mn_major = g.transA ? 1 : 0;
    p.b_mn_major = g.transB ? 0 : 1;
    p.a_box3d = p.b_box3d = 0;  // this kernel keeps one box per 32 columns
    p.status = ctx->status_dev;
    const int tiles = ((g.N + BN - 1) / BN) * ((g.M + BM - 1) / BM);
    const int kblocks_total = (g.K + BK - 1) / BK;
    p.kb_per_split = kblocks_total;
    p.split_stride = 0;
    // Split-K for the weight-gradient shape (few output tiles, very long K): partial products go to a workspace and a
    // second kernel adds them to C in split order, so the result does not depend on scheduling.
    int splits = 1;
    const bool plain = g.act == B200_ACT_NONE && !g.dout && !g.zout && !g.mulz && !g.mulmat && !g.addmat && !g.bias && g.sgd_lr == 0.f && !g.round_tf32;
    if (plain && tiles < 2 * ctx->sm_count && kblocks_total >= 256 && (g.N % 4 == 0)) {
        splits = (2 * ctx->sm_count + tiles - 1) / tiles;
        if (splits > 8) splits = 8;
        while (splits > 1 && (kblocks_total + splits - 1) / splits < 64) splits--;
        p.kb_per_split = (kblocks_total + splits - 1) / splits;
        splits = (kblocks_total + p.kb_per_split - 1) / p.kb_per_split;  // every split owns at least one K block
    }
    Epilogue e;
    e.C = g.C; e.ldc = g.ldc; e.alpha = g.alpha; e.alpha_dev = g.alpha_dev; e.accumulate = g.accumulate; e.bias = g.bias;
    e.zout = g.zout; e.ldz = g.ldz; e.act = g.act; e.act_conv = g.act_conv; e.dout = g.dout; e.lddo = g.lddo;
    e.mulz = g.mulz; e.ldmulz = g.ldmulz; e.mulz_act = g.mulz_act; e.mulmat = g.mulmat; e.ldmul = g.ldmul;
    e.act_sign_zero = g.act_sign_zero; e.mulz_is_act = g.mulz_is_act;
    e.addmat = g.addmat; e.ldadd = g.ldadd; e.sgd_lr = g.sgd_lr; e.sgd_lambda = g.sgd_lambda; e.round_tf32 = g.round_tf32;
    e.rope_table = g.rope_table; e.rope_pos = g.rope_pos; e.rope_cols = g.rope_cols; e.rope_hd = g.rope_head_dim;
    p.items = tiles * splits;
    const unsigned grid = (unsigned)(p.items < ctx->sm_count ? p.items : ctx->sm_count);  // persistent: one CTA per SM
    if (splits > 1) {
        B200_TRY(ensure_ws(ctx, (size_t)splits * g.M * g.N));
        p.split_stride = (long long)g.M * g.N;
        e.C = ctx->ws; e.ldc = g.N; e.accumulate = 0; e.alpha = 1.f; e.alpha_dev = nullptr;
        gemm_tcgen05_persistent_kernel<EPI_LINEAR, BN><<<grid, TileCfg<BN>::THREADS, SMEM_BYTES, ctx->stream>>>(mapA, mapB, p, e);
        B200_LAUNCH_CHECK(ctx);
        const int64_t count = (int64_t)g.M * g.N;
        int blocks = (int)((count / 4 + 255) / 256);
        if (blocks > ctx->sm_count * 8) blocks = ctx->sm_count * 8;
        splitk_reduce_kernel<<<blocks, 256, 0, ctx->stream>>>(ctx->ws, splits, g.M, g.N, g.C, g.ldc, g.alpha, g.alpha_dev, g.accumulate);
        B200_LAUNCH_CHECK(ctx);
        return B200_OK;
    }
    // pick the epilogue kind
    auto a16 = [](const void* q) { return ((uintptr_t)q & 15) == 0; };
    const bool plain_act = g.act == B200_ACT_NONE && !g.dout && !g.zout;
    const bool no_sgd = g.sgd_lr == 0.f && !g.mulmat;
    const bool vec_c = (g.N % 4 == 0) && (g.ldc % 4 == 0) && a16(g.C) && (!g.bias || a16(g.bias));
    int kind = EPI_GENERIC;
    if (vec_c && no_sgd) {
        if (plain_act && !g.mulz && (!g.addmat || (g.ldadd % 4 == 0 && a16(g.addmat)))) kind = EPI_LINEAR;
        else if (g.act != B200_ACT_NONE && !g.dout && g.act_conv == 0 && !g.mulz && !g.addmat && !g.accumulate && g.alpha == 1.f && !g.alpha_dev &&
                 (!g.zout || (g.ldz % 4 == 0 && a16(g.zout))))
            kind = EPI_ACT;
        else if (g.mulz && plain_act && !g.addmat && !g.accumulate && !g.bias && g.alpha == 1.f && !g.alpha_dev && g.ldmulz % 4 == 0 && a16(g.mulz))
            kind = EPI_MULZ;
    }
    switch (kind) {
        case EPI_LINEAR: gemm_tcgen05_persistent_kernel<EPI_LINEAR, BN><<<grid, TileCfg<BN>::THREADS, SMEM_BYTES, ctx->stream>>>(mapA, mapB, p, e); break;
        case EPI_ACT: gemm_tcgen05_persistent_kernel<EPI_ACT, BN><<<grid, TileCfg<BN>::THREADS, SMEM_BYTES, ctx->stream>>>(mapA, mapB, p, e); break;
        case EPI_MULZ: gemm_tcgen05_persistent_kernel<EPI_MULZ, BN><<<grid, TileCfg<BN>::THREADS, SMEM_BYTES, ctx->stream>>>(mapA, mapB, p, e); break;
        default: gemm_tcgen05_persistent_kernel<EPI_GENERIC, BN><<<grid, TileCfg<BN>::THREADS, SMEM_BYTES, ctx->stream>>>(mapA, mapB, p, e); break;
    }
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}
int gemm_tcgen05_tile(b200_ctx* ctx, const Gemm& g) {
    ctx->engine_launches[B200_ENGINE_GEMM_TILE]++;
    constexpr int BN = T_BN, SMEM_BYTES = T_SMEM_BYTES;
    if (!ctx->gemm_tc_configured) {
        ctx->gemm_tc_configured = 1;
        B200_CUDA(ctx, cudaFuncSetAttribute(gemm_tcgen05_tile_kernel<EPI_GENERIC>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        B200_CUDA(ctx, cudaFuncSetAttribute(gemm_tcgen05_tile_kernel<EPI_LINEAR>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        B200_CUDA(ctx, cudaFuncSetAttribute(gemm_tcgen05_tile_kernel<EPI_ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        B200_CUDA(ctx, cudaFuncSetAttribute(gemm_tcgen05_tile_kernel<EPI_MULZ>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    }
    CUtensorMap mapA, mapB;
    // A: stored [M,K] (K contiguous) or [K,M] (M contiguous).  B: stored [N,K] (transB, K contiguous) or [K,N].
    TcParams p;
    p.M = g.M; p.N = g.N; p.K = g.K;
    p.a_mn_major = g.transA ? 1 : 0;
    p.b_mn_major = g.transB ? 0 : 1;
    p.a_box3d = p.b_box3d = 0;
    if (!g.transA) B200_TRY(make_map(ctx, &mapA, g.A, (uint64_t)g.K, (uint64_t)g.M, (uint64_t)g.lda, BM, false));
    else if (ctx->gemm_box3d && g.M % 32 == 0 && make_map_mn3d(ctx, &mapA, g.A, (uint64_t)g.M, (uint64_t)g.K, (uint64_t)g.lda, BK, BM / 32) == B200_OK) p.a_box3d = 1;
    else B200_TRY(make_map(ctx, &mapA, g.A, (uint64_t)g.M, (uint64_t)g.K, (uint64_t)g.lda, BK, true));
    if (g.transB) B200_TRY(make_map(ctx, &mapB, g.B, (uint64_t)g.K, (uint64_t)g.N, (uint64_t)g.ldb, BN, false));
    else if (ctx->gemm_box3d && g.N % 32 == 0 && make_map_mn3d(ctx, &mapB, g.B, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.ldb, BK, BN / 32) == B200_OK) p.b_box3d = 1;
    else B200_TRY(make_map(ctx, &mapB, g.B, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.ldb, BK, true));
    p.status = ctx->status_dev;
    const int tiles = ((g.N + BN - 1) / BN) * ((g.M + BM - 1) / BM);
    const int kblocks_total = (g.K + BK - 1) / BK;
    p.kb_per_split = kblocks_total;
    p.split_stride = 0;
    // Split-K for the weight-gradient shape (few output tiles, very long K): partial products go to a workspace and a
    // second kernel adds them to C in split order, so the result does not depend on scheduling.
    int splits = 1;
    const bool plain = g.act == B200_ACT_NONE && !g.dout && !g.zout && !g.mulz && !g.mulmat && !g.addmat && !g.bias && g.sgd_lr == 0.f && !g.round_tf32;
    if (plain && tiles < 4 * ctx->sm_count && kblocks_total >= 256 && (g.N % 4 == 0)) {
        // Cost model in units of one K block on one SM: the SM that receives the most work items sets the time
        // (items are spread evenly over SMs, two resident at a time), every item pays a fixed fill + epilogue cost,
        // and every split adds one more pass over the output in the reduction.
        const double fixed = 16.0, reduce_per_split = (double)g.M * g.N * 8.0 / 5.0e12 / 0.26e-6;
        double best = 1e30;
        for (int sp = 1; sp <= 12; sp++) {
            const int kbs = (kblocks_total + sp - 1) / sp;
            if (sp > 1 && kbs < 48) break;
            const int per_sm = (tiles * sp + ctx->sm_count - 1) / ctx->sm_count;
            // items run two at a time on an SM and share its tensor pipe; an item that runs alone reaches about 65%
            const double item = kbs + fixed;
            const double cost = (per_sm / 2) * 2 * item + (per_sm & 1 ? item / 0.65 : 0.0) + (sp > 1 ? (sp + 0.5) * reduce_per_split : 0.0);
            if (cost < best) { best = cost; splits = sp; }
        }
        p.kb_per_split = (kblocks_total + splits - 1) / splits;
        splits = (kblocks_total + p.kb_per_split - 1) / p.kb_per_split;  // every split owns at least one K block
    }
    Epilogue e;
    e.C = g.C; e.ldc = g.ldc; e.alpha = g.alpha; e.alpha_dev = g.alpha_dev; e.accumulate = g.accumulate; e.bias = g.bias;
    e.zout = g.zout; e.ldz = g.ldz; e.act = g.act; e.act_conv = g.act_conv; e.dout = g.dout; e.lddo = g.lddo;
    e.mulz = g.mulz; e.ldmulz = g.ldmulz; e.mulz_act = g.mulz_act; e.mulmat = g.mulmat; e.ldmul = g.ldmul;
    e.act_sign_zero = g.act_sign_zero; e.mulz_is_act = g.mulz_is_act;
    e.addmat = g.addmat; e.ldadd = g.ldadd; e.sgd_lr = g.sgd_lr; e.sgd_lambda = g.sgd_lambda; e.round_tf32 = g.round_tf32;
    e.rope_table = g.rope_table; e.rope_pos = g.rope_pos; e.rope_cols = g.rope_cols; e.rope_hd = g.rope_head_dim;
    dim3 grid((unsigned)tiles, (unsigned)splits);
    if (splits > 1) {
        B200_TRY(ensure_ws(ctx, (size_t)splits * g.M * g.N));
        p.split_stride = (long long)g.M * g.N;
        e.C = ctx->ws; e.ldc = g.N; e.accumulate = 0; e.alpha = 1.f; e.alpha_dev = nullptr;
        gemm_tcgen05_tile_kernel<EPI_LINEAR><<<grid, THREADS, SMEM_BYTES, ctx->stream>>>(mapA, mapB, p, e);
        B200_LAUNCH_CHECK(ctx);
        const int64_t count = (int64_t)g.M * g.N;
        int blocks = (int)((count / 4 + 255) / 256);
        if (blocks > ctx->sm_count * 8) blocks = ctx->sm_count * 8;
        splitk_reduce_kernel<<<blocks, 256, 0, ctx->stream>>>(ctx->ws, splits, g.M, g.N, g.C, g.ldc, g.alpha, g.alpha_dev, g.accumulate);
        B200_LAUNCH_CHECK(ctx);
        return B200_OK;
    }
    // pick the epilogue kind
    auto a16 = [](const void* q) { return ((uintptr_t)q & 15) == 0; };
    const bool plain_act = g.act == B200_ACT_NONE && !g.dout && !g.zout;
    const bool no_sgd = g.sgd_lr == 0.f && !g.mulmat;
    const bool vec_c = (g.N % 4 == 0) && (g.ldc % 4 == 0) && a16(g.C) && (!g.bias || a16(g.bias));
    int kind = EPI_GENERIC;
    if (vec_c && no_sgd) {
        if (plain_act && !g.mulz && (!g.addmat || (g.ldadd % 4 == 0 && a16(g.addmat)))) kind = EPI_LINEAR;
        else if (g.act != B200_ACT_NONE && !g.dout && g.act_conv == 0 && !g.mulz && !g.addmat && !g.accumulate && g.alpha == 1.f && !g.alpha_dev &&
                 (!g.zout || (g.ldz % 4 == 0 && a16(g.zout))))
            kind = EPI_ACT;
        else if (g.mulz && plain_act && !g.addmat && !g.accumulate && !g.bias && g.alpha == 1.f && !g.alpha_dev && g.ldmulz % 4 == 0 && a16(g.mulz))
            kind = EPI_MULZ;
    }
    switch (kind) {
        case EPI_LINEAR: gemm_tcgen05_tile_kernel<EPI_LINEAR><<<grid, THREADS, SMEM_BYTES, ctx->stream>>>(mapA, mapB, p, e); break;
        case EPI_ACT: gemm_tcgen05_tile_kernel<EPI_ACT><<<grid, THREADS, SMEM_BYTES, ctx->stream>>>(mapA, mapB, p, e); break;
        case EPI_MULZ: gemm_tcgen05_tile_kernel<EPI_MULZ><<<grid, THREADS, SMEM_BYTES, ctx->stream>>>(mapA, mapB, p, e); break;
        default: gemm_tcgen05_tile_kernel<EPI_GENERIC><<<grid, THREADS, SMEM_BYTES, ctx->stream>>>(mapA, mapB, p, e); break;
    }
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}


// Two-SM kernel launcher: no split-K; M and N at least 256.
int gemm_tcgen05_pair(b200_ctx* ctx, const Gemm& g) {
    ctx->engine_launches[B200_ENGINE_GEMM_PAIR]++;
    static char configured_site;
    if (first_use(ctx, &configured_site)) {
        B200_CUDA(ctx, cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<EPI_GENERIC>, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_BYTES));
        B200_CUDA(ctx, cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<EPI_LINEAR>, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_BYTES));
        B200_CUDA(ctx, cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<EPI_ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_BYTES));
        B200_CUDA(ctx, cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<EPI_MULZ>, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_BYTES));
    }
    CUtensorMap mapA, mapB;
    // every CTA loads 128 rows of A and 128 of the tile's 256 B rows per stage
    TcParams p;
    p.M = g.M; p.N = g.N; p.K = g.K;
    p.a_mn_major = g.transA ? 1 : 0;
    p.b_mn_major = g.transB ? 0 : 1;
    p.a_box3d = p.b_box3d = 0;
    if (!g.transA) B200_TRY(make_map(ctx, &mapA, g.A, (uint64_t)g.K, (uint64_t)g.M, (uint64_t)g.lda, 128, false));
    else if (ctx->gemm_box3d && g.M % 32 == 0 && make_map_mn3d(ctx, &mapA, g.A, (uint64_t)g.M, (uint64_t)g.K, (uint64_t)g.lda, BK, 4) == B200_OK) p.a_box3d = 1;
    else B200_TRY(make_map(ctx, &mapA, g.A, (uint64_t)g.M, (uint64_t)g.K, (uint64_t)g.lda, BK, true));
    if (g.transB) B200_TRY(make_map(ctx, &mapB, g.B, (uint64_t)g.K, (uint64_t)g.N, (uint64_t)g.ldb, 128, false));
    else if (ctx->gemm_box3d && g.N % 32 == 0 && make_map_mn3d(ctx, &mapB, g.B, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.ldb, BK, 4) == B200_OK) p.b_box3d = 1;
    else B200_TRY(make_map(ctx, &mapB, g.B, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.ldb, BK, true));
    p.status = ctx->status_dev;
    const int kblocks_total = (g.K + BK - 1) / BK;
    const int tiles = ((g.M + 255) / 256) * ((g.N + PAIR_BN - 1) / PAIR_BN);
    const int n_pairs = ctx->sm_count / 2;
    p.kb_per_split = kblocks_total;
    p.split_stride = 0;
    // Split-K for the weight-gradient shape (few output tiles, very long K), as in the one-tile kernel: partial products
    // go to a workspace and a second kernel adds them in split order.  The pair that receives the most items sets the time.
    int splits = 1;
    const bool plain = g.act == B200_ACT_NONE && !g.dout && !g.zout && !g.mulz && !g.mulmat && !g.addmat && !g.bias && g.sgd_lr == 0.f && !g.round_tf32;
    if (plain && tiles < 4 * n_pairs && kblocks_total >= 256 && (g.N % 4 == 0)) {
        const double fixed = 24.0, reduce_per_split = (double)g.M * g.N * 8.0 / 5.0e12 / 0.1e-6;  // units: one K block of a 256 x 256 tile (~0.1 us)
        double best = 1e30;
        for (int sp = 1; sp <= 16; sp++) {
            const int kbs = (kblocks_total + sp - 1) / sp;
            if (sp > 1 && kbs < 48) break;
            const int per_pair = (tiles * sp + n_pairs - 1) / n_pairs;
            const double cost = per_pair * (kbs + fixed) + (sp > 1 ? (sp + 0.5) * reduce_per_split : 0.0);
            if (cost < best) { best = cost; splits = sp; }
        }
        p.kb_per_split = (kblocks_total + splits - 1) / splits;
        splits = (kblocks_total + p.kb_per_split - 1) / p.kb_per_split;
    }
    p.items = tiles * splits;
    Epilogue e;
    e.C = g.C; e.ldc = g.ldc; e.alpha = g.alpha; e.alpha_dev = g.alpha_dev; e.accumulate = g.accumulate; e.bias = g.bias;
    e.zout = g.zout; e.ldz = g.ldz; e.act = g.act; e.act_conv = g.act_conv; e.dout = g.dout; e.lddo = g.lddo;
    e.mulz = g.mulz; e.ldmulz = g.ldmulz; e.mulz_act = g.mulz_act; e.mulmat = g.mulmat; e.ldmul = g.ldmul;
    e.act_sign_zero = g.act_sign_zero; e.mulz_is_act = g.mulz_is_act;
    e.addmat = g.addmat; e.ldadd = g.ldadd; e.sgd_lr = g.sgd_lr; e.sgd_lambda = g.sgd_lambda; e.round_tf32 = g.round_tf32;
    e.rope_table = g.rope_table; e.rope_pos = g.rope_pos; e.rope_cols = g.rope_cols; e.rope_hd = g.rope_head_dim;
    int clusters = n_pairs;
    if (clusters > p.items) clusters = p.items;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * clusters));
    cfg.blockDim = dim3(PAIR_THREADS);
    cfg.dynamicSmemBytes = PAIR_SMEM_BYTES;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (splits > 1) {
        B200_TRY(ensure_ws(ctx, (size_t)splits * g.M * g.N));
        p.split_stride = (long long)g.M * g.N;
        e.C = ctx->ws; e.ldc = g.N; e.accumulate = 0; e.alpha = 1.f; e.alpha_dev = nullptr;
        B200_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel<EPI_LINEAR>, mapA, mapB, p, e));
        B200_LAUNCH_CHECK(ctx);
        const int64_t count = (int64_t)g.M * g.N;
        int blocks = (int)((count / 4 + 255) / 256);
        if (blocks > ctx->sm_count * 8) blocks = ctx->sm_count * 8;
        splitk_reduce_kernel<<<blocks, 256, 0, ctx->stream>>>(ctx->ws, splits, g.M, g.N, g.C, g.ldc, g.alpha, g.alpha_dev, g.accumulate);
        B200_LAUNCH_CHECK(ctx);
        return B200_OK;
    }
    auto a16 = [](const void* q) { return ((uintptr_t)q & 15) == 0; };
    const bool plain_act = g.act == B200_ACT_NONE && !g.dout && !g.zout;
    const bool no_sgd = g.sgd_lr == 0.f && !g.mulmat;
    const bool vec_c = (g.N % 4 == 0) && (g.ldc % 4 == 0) && a16(g.C) && (!g.bias || a16(g.bias));
    int kind = EPI_GENERIC;
    if (vec_c && no_sgd) {
        if (plain_act && !g.mulz && (!g.addmat || (g.ldadd % 4 == 0 && a16(g.addmat)))) kind = EPI_LINEAR;
        else if (g.act != B200_ACT_NONE && !g.dout && g.act_conv == 0 && !g.mulz && !g.addmat && !g.accumulate && g.alpha == 1.f && !g.alpha_dev &&
                 (!g.zout || (g.ldz % 4 == 0 && a16(g.zout))))
            kind = EPI_ACT;
        else if (g.mulz && plain_act && !g.addmat && !g.accumulate && !g.bias && g.alpha == 1.f && !g.alpha_dev && g.ldmulz % 4 == 0 && a16(g.mulz))
            kind = EPI_MULZ;
    }
    switch (kind) {
        case EPI_LINEAR: B200_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel<EPI_LINEAR>, mapA, mapB, p, e)); break;
        case EPI_ACT: B200_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel<EPI_ACT>, mapA, mapB, p, e)); break;
        case EPI_MULZ: B200_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel<EPI_MULZ>, mapA, mapB, p, e)); break;
        default: B200_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel<EPI_GENERIC>, mapA, mapB, p, e)); break;
    }
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

}  // namespace

// The rotation is part of the 128-bit LINEAR epilogue only, and never of a split-K launch (a bias keeps the split off).
bool gemm_tcgen05_fuses_rope(b200_ctx* ctx, const Gemm& g) {
    auto a16 = [](const void* q) { return ((uintptr_t)q & 15) == 0; };
    return gemm_tcgen05_eligible(ctx, g) && g.rope_table && g.bias && a16(g.bias) && a16(g.rope_table) && g.rope_head_dim % 4 == 0 &&
           g.rope_cols % g.rope_head_dim == 0 && g.N % 4 == 0 && g.ldc % 4 == 0 && a16(g.C) && g.act == B200_ACT_NONE && !g.dout && !g.zout &&
           !g.mulz && !g.mulmat && g.sgd_lr == 0.f && !g.accumulate && !g.addmat;
}

int gemm_tcgen05(b200_ctx* ctx, const Gemm& g) {
    if (!gemm_tcgen05_eligible(ctx, g)) return fail(ctx, B200_ERR_UNSUPPORTED, "shape does not qualify for the tcgen05 GEMM");
    B200_TRY(resolve_encode(ctx));
    B200_TRY(ensure_status(ctx));
    // M, N >= 256: the two-SM kernel (256 x 256 tiles, with split-K for weight gradients).  Narrower problems: the
    // one-CTA persistent kernel for short K (where the epilogue and the pipeline fill are a large share of a tile),
    // one tile per CTA otherwise.
    const int mode = ctx->gemm_tile_n;  // 0 = choose; 1 = always one tile per CTA; 128 / 256 = always one-CTA persistent with that width
    // Weight gradients (both operands M/N-contiguous, very long K) go to the two-SM kernel too when each operand stage
    // can be fetched as one three-dimensional box (4-8 % faster there than one tile per CTA); with one box per 32
    // columns the one-tile kernel was the faster of the two.
    const bool wgrad_pair = ctx->gemm_box3d && g.M % 32 == 0 && g.N % 32 == 0;
    if (g.M >= 256 && g.N >= 256 && (mode == 512 || (mode == 0 && (!g.transA || wgrad_pair)))) return gemm_tcgen05_pair(ctx, g);  // two SMs per 256 x 256 tile
    if (mode == 128) return gemm_tcgen05_persistent<128>(ctx, g);
    if (mode == 256 && g.N >= 256) return gemm_tcgen05_persistent<256>(ctx, g);
    if (mode == 0 && g.K <= 1024) return g.N >= 256 ? gemm_tcgen05_persistent<256>(ctx, g) : gemm_tcgen05_persistent<128>(ctx, g);
    return gemm_tcgen05_tile(ctx, g);
}

}  // namespace b200
