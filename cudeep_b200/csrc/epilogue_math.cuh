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

// Four values through one of the transcendental activations, out of line.  An epilogue handles 32
// values per thread and per step and has several store paths; with the activations inlined each
// path carried about 700 instructions of them (12 per GELU), the tensor-core kernels grew to many
// times the instruction cache, and a launch whose epilogue runs once per CTA spent hundreds of
// cycles fetching code it then jumped over (608 cycles in a bias- and activation-free `finish`
// were measured).  A call per four values costs the activated epilogues a few per cent.
static __device__ __noinline__ float4 activate4(float4 x, int act) {
    switch (act) {
        case EPI_GELU:
            return make_float4(act_gelu(x.x), act_gelu(x.y), act_gelu(x.z), act_gelu(x.w));
        case EPI_SILU:
            return make_float4(act_silu(x.x), act_silu(x.y), act_silu(x.z), act_silu(x.w));
        case EPI_SIGMOID:
            return make_float4(act_sigmoid(x.x), act_sigmoid(x.y), act_sigmoid(x.z), act_sigmoid(x.w));
        default:
            return x;
    }
}

template <int N>
__device__ __forceinline__ void apply_activation(float (&v)[N], int act) {
    static_assert(N % 4 == 0, "activations are applied four values at a time");
    if (__builtin_expect(act == EPI_NONE, 1)) return;      // the plain epilogue falls straight through
    if (act == EPI_RELU) {
#pragma unroll
        for (int j = 0; j < N; ++j) v[j] = fmaxf(v[j], 0.0f);
        return;
    }
#pragma unroll
    for (int j = 0; j < N; j += 4) {
        const float4 y = activate4(make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]), act);
        v[j] = y.x;
        v[j + 1] = y.y;
        v[j + 2] = y.z;
        v[j + 3] = y.w;
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
