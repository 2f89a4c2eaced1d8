// Device-side helpers shared by the kernels: warp/block reductions and the activation / cost conventions of the
// reference's different code paths.
#pragma once
#include <cuda_runtime.h>
#include <math.h>

#include "../../../include/callaghan_b200.h"

namespace b200 {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Block-wide reductions; `red` is a 32-float shared array; the result is returned to every thread.
__device__ __forceinline__ float block_sum(float v, float* red) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x * blockDim.y + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < nw; i++) t += red[i];
    return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x * blockDim.y + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float t = -INFINITY;
    for (int i = 0; i < nw; i++) t = fmaxf(t, red[i]);
    return t;
}

// NeuralNetwork.cs:704-716 StableSigmoidLocal.
__device__ __forceinline__ float stable_sigmoid(float x) {
    if (x >= 0.f) { float z = expf(-x); return 1.0f / (1.0f + z); }
    float z = expf(x);
    return z / (1.0f + z);
}
// The same derivative computed from the stored activation instead of the pre-activation, so that the forward pass
// need not keep both.  It returns exactly what ffn_act_der returns for every activation whose derivative is a function
// of its output -- all but Swish -- PROVIDED the forward pass marks "z < 0 (or NaN) gave a == 0" with a negative zero
// (act_sign_zero below): ReLU'(z) is 1 for z >= 0, and +0 / -0 is the one bit that a = max(z, 0) loses.
__device__ __forceinline__ float ffn_der_from_act(float a, int t) {
    switch (t) {
        case B200_ACT_SIGMOID: return a * (1.0f - a);
        case B200_ACT_TANH: return 1.0f - a * a;
        case B200_ACT_RELU: return signbit(a) ? 0.f : 1.f;
        case B200_ACT_LEAKYRELU: return a > 0.f ? 1.f : 0.1f;
        default: return 1.f;
    }
}
__device__ __forceinline__ float act_sign_zero(float z, float a) { return (a == 0.f && !(z >= 0.f)) ? -0.0f : a; }
// Transformer-FFN conventions: forward NeuralNetwork.cs:670-702, derivative NeuralNetwork.cs:886-946
// (ReLU'(0) = 1; LeakyReLU slope 0.01 forward but derivative 0.1 for z <= 0).
__device__ __forceinline__ void ffn_act_der(float z, int t, float& a, float& d) {
    switch (t) {
        case B200_ACT_SIGMOID: { float s = stable_sigmoid(z); a = s; d = s * (1.0f - s); break; }
        case B200_ACT_TANH: { float th = tanhf(z); a = th; d = 1.0f - th * th; break; }
        case B200_ACT_RELU: a = z > 0.f ? z : 0.f; d = z >= 0.f ? 1.f : 0.f; break;
        case B200_ACT_LEAKYRELU: a = z > 0.f ? z : 0.01f * z; d = z <= 0.f ? 0.1f : 1.f; break;
        case B200_ACT_SWISH: { float s = stable_sigmoid(z); a = z * s; d = s + z * s * (1.0f - s); break; }
        default: a = z; d = 1.f; break;
    }
}
// Batch-MLP conventions (BatchedAccelerationGPU.cs:262-287): sigmoid as e^z/(1+e^z), ReLU'(0) = 0,
// LeakyReLU' = 0.01, anything else (Swish) gives a = d = 0.
__device__ __forceinline__ void mlp_act_der(float z, int t, float& a, float& d) {
    switch (t) {
        case B200_ACT_NONE: a = z; d = 1.f; break;
        case B200_ACT_SIGMOID: { float e = expf(z); a = e / (1.0f + e); d = a * (1.0f - a); break; }
        case B200_ACT_TANH: a = tanhf(z); d = 1.0f - a * a; break;
        case B200_ACT_RELU: a = z > 0.f ? z : 0.f; d = z > 0.f ? 1.f : 0.f; break;
        case B200_ACT_LEAKYRELU: a = z > 0.f ? z : 0.01f * z; d = z > 0.f ? 1.f : 0.01f; break;
        default: a = 0.f; d = 0.f; break;
    }
}
// NeuralNetwork.cs:314-390 CostFunctionDeriv called as (ActualValue := activation a, predicted := target y) at
// NeuralNetwork.cs:514; the caller negates it (BatchedAccelerationGPU.cs:321).
__device__ __forceinline__ float mlp_cost_deriv(int kind, float a, float y, float huberDelta) {
    switch (kind) {
        case B200_COST_MSE: return 2.0f * (y - a);
        case B200_COST_ZERO_WEIGHTED_MSE: return 2.0f * (a == 0.f ? 0.25f : 1.0f) * (y - a);
        case B200_COST_BCE: return (y - a) / (y * (1.0f - y));
        case B200_COST_MAE: return a > y ? -1.0f : 1.0f;
        case B200_COST_CCE: return y - a;
        default: {
            float diff = a - y;
            if (fabsf(diff) <= huberDelta) return diff;
            return huberDelta * (float)((diff > 0.f) - (diff < 0.f));
        }
    }
}

}  // namespace b200
