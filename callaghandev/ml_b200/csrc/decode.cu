// Single-token decoding kernels for the generation session (LanguageModel.Generate's decoder path,
// LanguageModel.cs:270-537).  Every kernel here takes the token's position from DEVICE memory, so the launch sequence
// of one token has no host-dependent argument: it is captured once into a CUDA graph and replayed for every token
// (decoding one token is ~100 launches of a few microseconds each, i.e. launch-bound when issued one by one).
#include <cooperative_groups.h>

#include "common.h"
#include "device_math.cuh"

namespace cg = cooperative_groups;

namespace b200 {

// x[0, d) = embedding row of tokens[*pos]   (EmbedTokenIds for one id, AccelerationCPU.cs:3473-3515)
__global__ void decode_embed_kernel(const int32_t* __restrict__ tokens, const int32_t* __restrict__ pos, const float* __restrict__ emb, int d,
                                    float* __restrict__ x) {
    const int id = tokens[*pos];
    for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < d; j += gridDim.x * blockDim.x) x[j] = emb[(size_t)id * d + j];
}

// qkv = [q | k | v] of the current token (3d floats, biases added).  Rotates q and k by the position's angles
// (pairs (2p, 2p+1) within each head, AccelerationCPU.cs:4855-4982), leaves q in place and appends the rotated k and the
// v to row *pos of the layer's key / value cache.
__global__ void decode_rope_scatter_kernel(float* __restrict__ qkv, const int32_t* __restrict__ pos, const float2* __restrict__ table, int d,
                                           int headDim, float* __restrict__ Kc, float* __restrict__ Vc) {
    const int p = *pos, pairs = headDim >> 1, total = d >> 1;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const float2 cs = table[(size_t)p * pairs + (i % pairs)];
        float2 q = reinterpret_cast<float2*>(qkv)[i];
        const float2 k = reinterpret_cast<const float2*>(qkv + d)[i];
        const float2 v = reinterpret_cast<const float2*>(qkv + 2 * d)[i];
        reinterpret_cast<float2*>(qkv)[i] = make_float2(q.x * cs.x - q.y * cs.y, q.x * cs.y + q.y * cs.x);
        reinterpret_cast<float2*>(Kc + (size_t)p * d)[i] = make_float2(k.x * cs.x - k.y * cs.y, k.x * cs.y + k.y * cs.x);
        reinterpret_cast<float2*>(Vc + (size_t)p * d)[i] = v;
    }
}

// One query row against the cached rows 0..*pos of one layer; a block per head, a warp per key (strided), lanes over
// the head's columns.  Soft-max with the running-maximum form of AccelerationCPU.cs:1874-1946; every cached row is in
// the past, so there is no mask.
template <int MAXHD>  // head dimension hd <= MAXHD
__global__ void __launch_bounds__(128) decode_attn_kernel(const float* __restrict__ q, const float* __restrict__ Kc, const float* __restrict__ Vc,
                                                          const int32_t* __restrict__ pos, int d, int HD, float scale, float* __restrict__ out) {
    constexpr int PER = (MAXHD + 31) / 32;
    __shared__ float s_m[4], s_l[4], s_o[4][MAXHD];
    const int head = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nKeys = *pos + 1;
    float qr[PER], acc[PER];
#pragma unroll
    for (int i = 0; i < PER; i++) {
        const int c = lane + 32 * i;
        qr[i] = c < HD ? q[head * HD + c] : 0.f;
        acc[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    for (int j = warp; j < nKeys; j += 4) {
        const float* kr = Kc + (size_t)j * d + head * HD;
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < PER; i++) {
            const int c = lane + 32 * i;
            if (c < HD) s += qr[i] * kr[c];
        }
        s = warp_sum(s) * scale;
        const float mn = fmaxf(m, s);
        const float corr = (m == -INFINITY) ? 0.f : expf(m - mn), w = expf(s - mn);
        const float* vr = Vc + (size_t)j * d + head * HD;
        l = l * corr + w;
#pragma unroll
        for (int i = 0; i < PER; i++) {
            const int c = lane + 32 * i;
            acc[i] = acc[i] * corr + (c < HD ? w * vr[c] : 0.f);
        }
        m = mn;
    }
    if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
    for (int i = 0; i < PER; i++) {
        const int c = lane + 32 * i;
        if (c < HD) s_o[warp][c] = acc[i];
    }
    __syncthreads();
    if (warp == 0) {
        float M = fmaxf(fmaxf(s_m[0], s_m[1]), fmaxf(s_m[2], s_m[3]));
        float L = 0.f;
        float f[4];
#pragma unroll
        for (int w = 0; w < 4; w++) {
            f[w] = (s_m[w] == -INFINITY) ? 0.f : expf(s_m[w] - M);
            L += s_l[w] * f[w];
        }
#pragma unroll
        for (int i = 0; i < PER; i++) {
            const int c = lane + 32 * i;
            if (c < HD) {
                const float o = (s_o[0][c] * f[0] + s_o[1][c] * f[1]) + (s_o[2][c] * f[2] + s_o[3][c] * f[3]);
                out[head * HD + c] = L > 0.f ? o / L : 0.f;
            }
        }
    }
}

// Arg-max of the logits into tokens[*pos + 1] (when pick != 0: the greedy choice of the next token, lowest index among
// equals), then the position moves on by one.  One block.
__global__ void __launch_bounds__(1024) decode_advance_kernel(const float* __restrict__ logits, int n, int32_t* __restrict__ tokens,
                                                              int32_t* __restrict__ pos, int pick) {
    __shared__ float sv[32];
    __shared__ int si[32];
    const int p = *pos;
    if (pick) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const float v = logits[i];
            if (bi == 0x7fffffff || v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
        }
        if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
        __syncthreads();
        if (threadIdx.x < 32) {
            bv = sv[threadIdx.x]; bi = si[threadIdx.x];
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
            }
            if (threadIdx.x == 0) tokens[p + 1] = bi == 0x7fffffff ? 0 : bi;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) *pos = p + 1;
}

// y[n] = act(W[n,:] . v + bias[n]) for one token, v of length K.  With LN the input is v = LayerNorm(x + sub) * gamma + beta
// (ResidualLayerNormForward for one row, AccelerationCPU.cs:1440-1514: biased variance, eps inside the root), computed
// by every block into shared memory -- 8 KB of reads that hit L2 -- so that the normalisation costs no launch of its own;
// block 0 stores v to v_out, where the next residual addition finds it.  Without LN v = x.  As in the few-row product
// of the trainer, `wpc` warps share an output column and every lane keeps four 128-bit weight loads in flight.
template <bool LN>
__global__ void __launch_bounds__(256) decode_gemv_kernel(const float* __restrict__ x, const float* __restrict__ sub, const float* __restrict__ gamma,
                                                          const float* __restrict__ beta, float eps, float* __restrict__ v_out,
                                                          const float* __restrict__ W, const float* __restrict__ bias, int N, int K, int wpc, int act,
                                                          float* __restrict__ y) {
    extern __shared__ float sv[];  // the input vector
    __shared__ float red[32];
    __shared__ float part[8];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, K4 = K >> 2;
    float4* sv4 = reinterpret_cast<float4*>(sv);
    if (LN) {
        float s = 0.f;
        for (int i = tid; i < K4; i += 256) {
            float4 a = reinterpret_cast<const float4*>(x)[i];
            const float4 b = reinterpret_cast<const float4*>(sub)[i];
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
            sv4[i] = a;
            s += (a.x + a.y) + (a.z + a.w);
        }
        const float mu = block_sum(s, red) / (float)K;
        float q = 0.f;
        for (int i = tid; i < K4; i += 256) {
            const float4 a = sv4[i];
            const float d0 = a.x - mu, d1 = a.y - mu, d2 = a.z - mu, d3 = a.w - mu;
            q += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
        }
        const float inv = 1.0f / sqrtf(block_sum(q, red) / (float)K + eps);
        for (int i = tid; i < K4; i += 256) {
            const float4 a = sv4[i], g = reinterpret_cast<const float4*>(gamma)[i], b = reinterpret_cast<const float4*>(beta)[i];
            float4 o;
            o.x = g.x * ((a.x - mu) * inv) + b.x; o.y = g.y * ((a.y - mu) * inv) + b.y;
            o.z = g.z * ((a.z - mu) * inv) + b.z; o.w = g.w * ((a.w - mu) * inv) + b.w;
            sv4[i] = o;
            if (blockIdx.x == 0 && v_out) reinterpret_cast<float4*>(v_out)[i] = o;
        }
    } else {
        for (int i = tid; i < K4; i += 256) sv4[i] = reinterpret_cast<const float4*>(x)[i];
    }
    __syncthreads();
    const int n = blockIdx.x * (8 / wpc) + warp / wpc, seg = warp % wpc;
    float acc = 0.f;
    if (n < N) {
        const float* w = W + (size_t)n * K;
        int chunk = (K + wpc - 1) / wpc;
        chunk = (chunk + 127) & ~127;
        const int k0 = seg * chunk, k1 = min(K, k0 + chunk);
        int k = k0 + lane * 4;
        for (; k + 384 < k1; k += 512) {
            float4 wv[4];
#pragma unroll
            for (int u = 0; u < 4; u++) wv[u] = *reinterpret_cast<const float4*>(w + k + 128 * u);
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const float4 xv = *reinterpret_cast<const float4*>(sv + k + 128 * u);
                acc += (wv[u].x * xv.x + wv[u].y * xv.y) + (wv[u].z * xv.z + wv[u].w * xv.w);
            }
        }
        for (; k < k1; k += 128) {
            const float4 wv = *reinterpret_cast<const float4*>(w + k);
            const float4 xv = *reinterpret_cast<const float4*>(sv + k);
            acc += (wv.x * xv.x + wv.y * xv.y) + (wv.z * xv.z + wv.w * xv.w);
        }
    }
    acc = warp_sum(acc);
    if (lane == 0) part[warp] = acc;
    __syncthreads();
    if (n < N && seg == 0 && lane == 0) {
        float v = part[warp];
        for (int s2 = 1; s2 < wpc; s2++) v += part[warp + s2];
        v += bias[n];
        if (act != B200_ACT_NONE) {
            float a, dd;
            ffn_act_der(v, act, a, dd);
            v = a;
        }
        y[n] = v;
    }
}

int k_decode_gemv(b200_ctx* ctx, const float* x, const float* sub, const float* gamma, const float* beta, float eps, float* v_out, const float* W,
                  const float* bias, int N, int K, int act, float* y) {
    int wpc = 1;  // warps per output column: a few thousand warps in the grid, never less than 256 elements of K per warp
    while (wpc < 8 && (int64_t)N * wpc < 8192 && K / (2 * wpc) >= 256) wpc *= 2;
    const int cols = 8 / wpc, blocks = (N + cols - 1) / cols;
    const size_t smem = sizeof(float) * (size_t)K;
    if (sub) decode_gemv_kernel<true><<<blocks, 256, smem, ctx->stream>>>(x, sub, gamma, beta, eps, v_out, W, bias, N, K, wpc, act, y);
    else decode_gemv_kernel<false><<<blocks, 256, smem, ctx->stream>>>(x, nullptr, nullptr, nullptr, eps, nullptr, W, bias, N, K, wpc, act, y);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

int k_decode_embed(b200_ctx* ctx, const int32_t* tokens, const int32_t* pos, const float* emb, int d, float* x) {
    decode_embed_kernel<<<(d + 255) / 256, 256, 0, ctx->stream>>>(tokens, pos, emb, d, x);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

int k_decode_rope_scatter(b200_ctx* ctx, float* qkv, const int32_t* pos, const float* table, int d, int headDim, float* Kc, float* Vc) {
    decode_rope_scatter_kernel<<<(d / 2 + 255) / 256, 256, 0, ctx->stream>>>(qkv, pos, reinterpret_cast<const float2*>(table), d, headDim, Kc, Vc);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

int k_decode_attn(b200_ctx* ctx, const float* q, const float* Kc, const float* Vc, const int32_t* pos, int numHeads, int headDim, float scale, float* out) {
    const int d = numHeads * headDim;
    if (headDim <= 32) decode_attn_kernel<32><<<numHeads, 128, 0, ctx->stream>>>(q, Kc, Vc, pos, d, headDim, scale, out);
    else if (headDim <= 64) decode_attn_kernel<64><<<numHeads, 128, 0, ctx->stream>>>(q, Kc, Vc, pos, d, headDim, scale, out);
    else if (headDim <= 128) decode_attn_kernel<128><<<numHeads, 128, 0, ctx->stream>>>(q, Kc, Vc, pos, d, headDim, scale, out);
    else return fail(ctx, B200_ERR_UNSUPPORTED, "attention head dimension %d exceeds 128", headDim);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

int k_decode_advance(b200_ctx* ctx, const float* logits, int n, int32_t* tokens, int32_t* pos, int pick) {
    decode_advance_kernel<<<1, 1024, 0, ctx->stream>>>(logits, n, tokens, pos, pick);
    B200_LAUNCH_CHECK(ctx);
    return B200_OK;
}

// ------------------------------------------------------------------------------------------------ one token, one launch
// The whole model for one token as ONE cooperative kernel: the phases of a block (Q/K/V product with the previous
// LayerNorm in its prologue; rotation + cache append + attention; output projection; first FFN product with LayerNorm 1
// in its prologue and the activation in its epilogue; second FFN product) are separated by grid barriers instead of
// kernel boundaries.  A launch of a few microseconds of work costs ~6-7 us of fixed latency (launch, prologue, tail);
// a grid barrier costs about one.  The blocks stay resident, every product is a grid-stride loop over its output
// columns, and the position is read from device memory, so the launch arguments never change from token to token.
__device__ __forceinline__ int decode_wpc(int N, int K) {
    int wpc = 1;
    while (wpc < 8 && (long long)N * wpc < 8192 && K / (2 * wpc) >= 256) wpc *= 2;
    return wpc;
}

// y = act(W v + bias) with v staged in shared memory by stage_vector(); grid-stride over groups of 8 / wpc columns.
__device__ void product_phase(const float* __restrict__ sv, float* part, const float* __restrict__ W, const float* __restrict__ bias, int N, int K,
                              int act, float* __restrict__ y) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wpc = decode_wpc(N, K), cols = 8 / wpc, items = (N + cols - 1) / cols;
    int chunk = (K + wpc - 1) / wpc;
    chunk = (chunk + 127) & ~127;
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int n = item * cols + warp / wpc, seg = warp % wpc;
        float acc = 0.f;
        if (n < N) {
            const float* w = W + (size_t)n * K;
            const int k0 = seg * chunk, k1 = min(K, k0 + chunk);
            int k = k0 + lane * 4;
            for (; k + 384 < k1; k += 512) {
                float4 wv[4];
#pragma unroll
                for (int u = 0; u < 4; u++) wv[u] = *reinterpret_cast<const float4*>(w + k + 128 * u);
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const float4 xv = *reinterpret_cast<const float4*>(sv + k + 128 * u);
                    acc += (wv[u].x * xv.x + wv[u].y * xv.y) + (wv[u].z * xv.z + wv[u].w * xv.w);
                }
            }
            for (; k < k1; k += 128) {
                const float4 wv = *reinterpret_cast<const float4*>(w + k);
                const float4 xv = *reinterpret_cast<const float4*>(sv + k);
                acc += (wv.x * xv.x + wv.y * xv.y) + (wv.z * xv.z + wv.w * xv.w);
            }
        }
        acc = warp_sum(acc);
        if (lane == 0) part[warp] = acc;
        __syncthreads();
        if (n < N && seg == 0 && lane == 0) {
            float v = part[warp];
            for (int s2 = 1; s2 < wpc; s2++) v += part[warp + s2];
            v += bias[n];
            if (act != B200_ACT_NONE) {
                float a, dd;
                ffn_act_der(v, act, a, dd);
                v = a;
            }
            y[n] = v;
        }
        __syncthreads();  // part is reused by the next item
    }
}

// sv = x (sub == NULL) or LayerNorm(x + sub) * gamma + beta; block 0 stores the latter to v_out.
__device__ void stage_vector(float* sv, float* red, const float* __restrict__ x, const float* __restrict__ sub, const float* __restrict__ gamma,
                             const float* __restrict__ beta, float eps, float* __restrict__ v_out, int K) {
    const int tid = threadIdx.x, K4 = K >> 2;
    float4* sv4 = reinterpret_cast<float4*>(sv);
    if (sub) {
        float s = 0.f;
        for (int i = tid; i < K4; i += blockDim.x) {
            float4 a = reinterpret_cast<const float4*>(x)[i];
            const float4 b = reinterpret_cast<const float4*>(sub)[i];
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
            sv4[i] = a;
            s += (a.x + a.y) + (a.z + a.w);
        }
        const float mu = block_sum(s, red) / (float)K;
        float q = 0.f;
        for (int i = tid; i < K4; i += blockDim.x) {
            const float4 a = sv4[i];
            const float d0 = a.x - mu, d1 = a.y - mu, d2 = a.z - mu, d3 = a.w - mu;
            q += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
        }
        const float inv = 1.0f / sqrtf(block_sum(q, red) / (float)K + eps);
        for (int i = tid; i < K4; i += blockDim.x) {
            const float4 a = sv4[i], g = reinterpret_cast<const float4*>(gamma)[i], b = reinterpret_cast<const float4*>(beta)[i];
            float4 o;
            o.x = g.x * ((a.x - mu) * inv) + b.x; o.y = g.y * ((a.y - mu) * inv) + b.y;
            o.z = g.z * ((a.z - mu) * inv) + b.z; o.w = g.w * ((a.w - mu) * inv) + b.w;
            sv4[i] = o;
            if (blockIdx.x == 0 && v_out) reinterpret_cast<float4*>(v_out)[i] = o;
        }
    } else {
        for (int i = tid; i < K4; i += blockDim.x) sv4[i] = reinterpret_cast<const float4*>(x)[i];
    }
    __syncthreads();
}

// Rotation of the token's query / key head slices, append of key and value to the cache, and the token's attention over
// rows 0..p of the cache, one head per block iteration (8 warps: a warp per key, strided).
__device__ void attention_phase(float* sq, float* s_m, float* s_l, float* s_o /*[8][128]*/, const float* __restrict__ qkv, const float2* __restrict__ rope,
                                int p, int d, int H, int hd, float scale, float* __restrict__ Kc, float* __restrict__ Vc, float* __restrict__ out) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, pairs = hd >> 1;
    for (int head = blockIdx.x; head < H; head += gridDim.x) {
        if (tid < pairs) {
            const float2 cs = rope[(size_t)p * pairs + tid];
            const int c = head * hd + 2 * tid;
            const float2 q = *reinterpret_cast<const float2*>(qkv + c), k = *reinterpret_cast<const float2*>(qkv + d + c);
            sq[2 * tid] = q.x * cs.x - q.y * cs.y;
            sq[2 * tid + 1] = q.x * cs.y + q.y * cs.x;
            *reinterpret_cast<float2*>(Kc + (size_t)p * d + c) = make_float2(k.x * cs.x - k.y * cs.y, k.x * cs.y + k.y * cs.x);
            *reinterpret_cast<float2*>(Vc + (size_t)p * d + c) = *reinterpret_cast<const float2*>(qkv + 2 * d + c);
        }
        __syncthreads();  // the block's own global writes (row p of the cache) are visible to all its threads after this
        float qr[4], acc[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int c = lane + 32 * i;
            qr[i] = c < hd ? sq[c] : 0.f;
            acc[i] = 0.f;
        }
        float m = -INFINITY, l = 0.f;
        for (int j = warp; j <= p; j += 8) {
            const float* kr = Kc + (size_t)j * d + head * hd;
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int c = lane + 32 * i;
                if (c < hd) s += qr[i] * kr[c];
            }
            s = warp_sum(s) * scale;
            const float mn = fmaxf(m, s);
            const float corr = (m == -INFINITY) ? 0.f : expf(m - mn), w = expf(s - mn);
            const float* vr = Vc + (size_t)j * d + head * hd;
            l = l * corr + w;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int c = lane + 32 * i;
                acc[i] = acc[i] * corr + (c < hd ? w * vr[c] : 0.f);
            }
            m = mn;
        }
        if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int c = lane + 32 * i;
            if (c < hd) s_o[warp * 128 + c] = acc[i];
        }
        __syncthreads();
        if (warp == 0) {
            float M = -INFINITY;
            for (int w = 0; w < 8; w++) M = fmaxf(M, s_m[w]);
            float L = 0.f, f[8];
            for (int w = 0; w < 8; w++) {
                f[w] = (s_m[w] == -INFINITY) ? 0.f : expf(s_m[w] - M);
                L += s_l[w] * f[w];
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int c = lane + 32 * i;
                if (c < hd) {
                    float o = 0.f;
                    for (int w = 0; w < 8; w++) o += s_o[w * 128 + c] * f[w];
                    out[head * hd + c] = L > 0.f ? o / L : 0.f;
                }
            }
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(256) decode_token_kernel(DecodeArgs a) {
    extern __shared__ float sv[];  // max(d, f) floats
    __shared__ float red[32], part[8], sq[128], s_m[8], s_l[8], s_o[8 * 128];
    cg::grid_group grid = cg::this_grid();
    const int p = *a.pos;            // read by every block before the first barrier; block 0 moves it on after the last
    const int id = a.tokens[p];
    const float* x_in = a.emb + (size_t)id * a.d;  // input of the first block: the token's embedding row
    const float *res = nullptr, *sub = nullptr, *gam = nullptr, *bet = nullptr;
    for (int l = 0; l < a.L; l++) {
        const DecodeLayer& Ly = a.layers[l];
        // x_l = embedding row, or LayerNorm 2 of the previous block (stored to a.x by block 0 for the residual of LayerNorm 1)
        stage_vector(sv, red, sub ? res : x_in, sub, gam, bet, 1e-5f, a.x, a.d);
        if (!sub && blockIdx.x == 0)
            for (int i = threadIdx.x; i < a.d; i += blockDim.x) a.x[i] = sv[i];
        product_phase(sv, part, Ly.Wqkv, Ly.bqkv, 3 * a.d, a.d, B200_ACT_NONE, a.qkv);
        grid.sync();
        attention_phase(sq, s_m, s_l, s_o, a.qkv, reinterpret_cast<const float2*>(a.rope), p, a.d, a.H, a.hd, a.scale, Ly.Kc, Ly.Vc, a.attnO);
        grid.sync();
        stage_vector(sv, red, a.attnO, nullptr, nullptr, nullptr, 0.f, nullptr, a.d);
        product_phase(sv, part, Ly.WO, Ly.bO, a.d, a.d, B200_ACT_NONE, a.proj);
        grid.sync();
        stage_vector(sv, red, a.x, a.proj, Ly.g1, Ly.b1n, 1e-5f, a.n1, a.d);  // n1 = LayerNorm 1 (x_l + attention projection)
        product_phase(sv, part, Ly.W1, Ly.fb1, a.f, a.d, a.act, a.a1);
        grid.sync();
        stage_vector(sv, red, a.a1, nullptr, nullptr, nullptr, 0.f, nullptr, a.f);
        product_phase(sv, part, Ly.W2, Ly.fb2, a.d, a.f, B200_ACT_NONE, a.proj2);
        grid.sync();
        res = a.n1; sub = a.proj2; gam = Ly.g2; bet = Ly.b2n;
    }
    stage_vector(sv, red, sub ? res : x_in, sub, gam, bet, 1e-5f, nullptr, a.d);
    product_phase(sv, part, a.Wout, a.bout, a.V, a.d, B200_ACT_NONE, a.logits);
    grid.sync();
    if (blockIdx.x == 0) {
        if (a.pick) {  // arg-max of the logits (lowest index among equals) is the next token
            __shared__ float bvs[8];
            __shared__ int bis[8];
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            for (int i = threadIdx.x; i < a.V; i += blockDim.x) {
                const float v = a.logits[i];
                if (bi == 0x7fffffff || v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
            }
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
            }
            if ((threadIdx.x & 31) == 0) { bvs[threadIdx.x >> 5] = bv; bis[threadIdx.x >> 5] = bi; }
            __syncthreads();
            if (threadIdx.x == 0) {
                for (int w = 1; w < 8; w++)
                    if (bis[w] != 0x7fffffff && (bi == 0x7fffffff || bvs[w] > bv || (bvs[w] == bv && bis[w] < bi))) { bv = bvs[w]; bi = bis[w]; }
                a.tokens[p + 1] = bi == 0x7fffffff ? 0 : bi;
            }
        }
        if (threadIdx.x == 0) *a.pos = p + 1;
    }
}

// Launches the one-token kernel; *blocks_cache keeps the grid size between calls (0 = not computed yet).  Returns
// B200_ERR_UNSUPPORTED when the device cannot hold a cooperative grid of it (the caller then issues the phases as
// separate launches).
int k_decode_token(b200_ctx* ctx, const DecodeArgs& args, int* blocks_cache) {
    const size_t smem = sizeof(float) * (size_t)(args.d > args.f ? args.d : args.f);
    if (*blocks_cache == 0) {
        int coop = 0, per_sm = 0;
        if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, ctx->device) != cudaSuccess || !coop) { *blocks_cache = -1; }
        else if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_token_kernel, 256, smem) != cudaSuccess || per_sm < 1) { *blocks_cache = -1; }
        else *blocks_cache = ctx->sm_count * (per_sm > 4 ? 4 : per_sm);
        (void)cudaGetLastError();
    }
    if (*blocks_cache < 0) return B200_ERR_UNSUPPORTED;
    DecodeArgs a = args;
    void* params[] = {&a};
    B200_CUDA(ctx, cudaLaunchCooperativeKernel((void*)decode_token_kernel, dim3(*blocks_cache), dim3(256), params, smem, ctx->stream));
    ctx->launches++;
    return B200_OK;
}

}  // namespace b200
