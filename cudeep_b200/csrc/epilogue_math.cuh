// Activation functions applied in GEMM / conv epilogues.
//
// The definitions follow the reference's device math
// (include/cudeep/ptx_intrinsics.cuh:531-554): sigmoid through the SFU
// ex2/rcp approximations, tanh(x) = 2*sigmoid(2x) - 1, GELU in its tanh form
// (not erf), SiLU = x*sigmoid(x).
#pragma once

#include <cuda_runtime.h>

namespace cudeep_b200 {

// Epilogue codes; the numeric values equal cudeep::kernels::GemmEpilogue
// (include/cudeep/kernels/matmul.cuh:32-38 in the reference).
enum Epilogue : int { EPI_NONE = 0, EPI_RELU = 1, EPI_GELU = 2, EPI_SILU = 3, EPI_SIGMOID = 4 };

__device__ __forceinline__ float sfu_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float sfu_rcp(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float act_sigmoid(float x) {
    return sfu_rcp(1.0f + sfu_ex2(-1.4426950408889634f * x));
}
__device__ __forceinline__ float act_tanh(float x) { return 2.0f * act_sigmoid(2.0f * x) - 1.0f; }
__device__ __forceinline__ float act_gelu(float x) {
    const float inner = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.0f + act_tanh(inner));
}
__device__ __forceinline__ float act_silu(float x) { return x * act_sigmoid(x); }

template <int N>
__device__ __forceinline__ void apply_activation(float (&v)[N], int act) {
    switch (act) {
        case EPI_RELU:
#pragma unroll
            for (int j = 0; j < N; ++j) v[j] = fmaxf(v[j], 0.0f);
            break;
        case EPI_GELU:
#pragma unroll
            for (int j = 0; j < N; ++j) v[j] = act_gelu(v[j]);
            break;
        case EPI_SILU:
#pragma unroll
            for (int j = 0; j < N; ++j) v[j] = act_silu(v[j]);
            break;
        case EPI_SIGMOID:
#pragma unroll
            for (int j = 0; j < N; ++j) v[j] = act_sigmoid(v[j]);
            break;
        default:
            break;
    }
}

__device__ __forceinline__ float apply_activation1(float x, int act) {
    switch (act) {
        case EPI_RELU: return fmaxf(x, 0.0f);
        case EPI_GELU: return act_gelu(x);
        case EPI_SILU: return act_silu(x);
        case EPI_SIGMOID: return act_sigmoid(x);
        default: return x;
    }
}

}  // namespace cudeep_b200
