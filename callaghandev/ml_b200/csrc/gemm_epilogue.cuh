// The fused GEMM epilogue shared by the FP32 SIMT kernel and the TF32 tcgen05 kernel (see struct Gemm in common.h
// for the order of operations).  Passed to kernels by value.
#pragma once
#include "device_math.cuh"

namespace b200 {

struct Epilogue {
    float* C; int ldc;
    float alpha; const float* alpha_dev;
    int accumulate;
    const float* bias;
    float* zout; int ldz;
    int act, act_conv;
    float* dout; int lddo;
    const float* mulz; int ldmulz; int mulz_act;
    const float* mulmat; int ldmul;
    const float* addmat; int ldadd;
    float sgd_lr, sgd_lambda;
    int round_tf32;
    int act_sign_zero, mulz_is_act;
    const float* rope_table; const int32_t* rope_pos; int rope_cols, rope_hd;
};

__device__ __forceinline__ float tf32_round(float x) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
    return __uint_as_float(u);
}

// Rotary embedding in the 128-bit epilogue: a lane owns columns n..n+3 (two pairs inside one head) of row m.
// rope_cs fetches (cos0, sin0, cos1, sin1) for them -- issued with the other operand loads of a row batch, so its
// latency is overlapped -- and rope_rotate applies the rotation.
__device__ __forceinline__ float4 rope_cs(const Epilogue& e, int m, int n) {
    const int pos = e.rope_pos ? e.rope_pos[m] : m;
    return *reinterpret_cast<const float4*>(e.rope_table + ((size_t)pos * (e.rope_hd >> 1) + ((n % e.rope_hd) >> 1)) * 2);
}
__device__ __forceinline__ void rope_rotate(const float4& cs, float4& v) {
    const float x0 = v.x, x1 = v.y, x2 = v.z, x3 = v.w;
    v.x = x0 * cs.x - x1 * cs.y; v.y = x0 * cs.y + x1 * cs.x;
    v.z = x2 * cs.z - x3 * cs.w; v.w = x2 * cs.w + x3 * cs.z;
}

__device__ __forceinline__ void epilogue_store(const Epilogue& e, int m, int n, float acc, float alpha) {
    float v = alpha * acc;
    if (e.bias) v += e.bias[n];
    if (e.zout) e.zout[(size_t)m * e.ldz + n] = v;
    if (e.act != B200_ACT_NONE || e.dout) {
        float a, d;
        if (e.act_conv) mlp_act_der(v, e.act, a, d);
        else ffn_act_der(v, e.act, a, d);
        if (e.dout) e.dout[(size_t)m * e.lddo + n] = d;
        v = e.act_sign_zero ? act_sign_zero(v, a) : a;
    }
    if (e.mulz) {
        float a, d;
        const float zv = e.mulz[(size_t)m * e.ldmulz + n];
        if (e.mulz_is_act) d = ffn_der_from_act(zv, e.mulz_act);
        else ffn_act_der(zv, e.mulz_act, a, d);
        v *= d;
    }
    if (e.mulmat) v *= e.mulmat[(size_t)m * e.ldmul + n];
    if (e.addmat) v += e.addmat[(size_t)m * e.ldadd + n];
    float* c = e.C + (size_t)m * e.ldc + n;
    if (e.sgd_lr != 0.f) {
        float w = *c;
        *c = w - e.sgd_lr * (v + e.sgd_lambda * w);
    } else if (e.accumulate) {
        v += *c;
        *c = e.round_tf32 ? tf32_round(v) : v;
    } else {
        *c = e.round_tf32 ? tf32_round(v) : v;
    }
}

}  // namespace b200
