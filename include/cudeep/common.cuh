// Shared enums, launch constants and small device helpers of the C++ surface.
//
// Everything declared by the reference's include/cudeep/common.cuh is declared here under the
// same name and with the same meaning, so the reference's kernels that are outside the
// dense-contraction path (elementwise, reduce, loss, norm, pool, optimiser, unary, activation)
// compile against this header unchanged:
//   * DType / Layout (include/cudeep/common.cuh:10-19): enumerator order is part of the ABI of
//     cudeep::Tensor and of the Python module;
//   * WARP_SIZE, MAX_THREADS_PER_BLOCK, DEFAULT_BLOCK_SIZE, DTypeTraits, ceil_div, ceil_div64
//     (:21-52);
//   * warp and block reductions, Vec4, cp.async wrappers, SFU math wrappers (:57-298), device
//     code only.
// The reductions are written as xor butterflies, so every lane of a warp ends up with the warp's
// result; the block reductions deliver the block's result to warp 0 (callers read it in thread 0).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cstddef>
#include <cstdint>
#include <cstdio>

namespace cudeep {

enum class DType { Float16, Float32, Float64 };
enum class Layout { NCHW, NHWC };

constexpr int WARP_SIZE = 32;
constexpr int MAX_THREADS_PER_BLOCK = 1024;
constexpr int DEFAULT_BLOCK_SIZE = 256;

inline size_t dtype_size(DType t) { return t == DType::Float16 ? 2 : t == DType::Float32 ? 4 : 8; }

template <DType D> struct DTypeTraits;
template <> struct DTypeTraits<DType::Float16> { using type = __half; static constexpr size_t size = sizeof(__half); };
template <> struct DTypeTraits<DType::Float32> { using type = float;  static constexpr size_t size = sizeof(float); };
template <> struct DTypeTraits<DType::Float64> { using type = double; static constexpr size_t size = sizeof(double); };

inline int ceil_div(int value, int unit) { return (value + unit - 1) / unit; }
inline int64_t ceil_div64(int64_t value, int64_t unit) { return (value + unit - 1) / unit; }

#ifdef __CUDACC__

// ---- warp reductions -----------------------------------------------------------------------

// Maps a float to an unsigned integer whose unsigned order is the float order (negative values
// are bit-flipped, non-negative ones get the sign bit set), and back.
__device__ __forceinline__ unsigned int float_to_ordered_uint(float v) {
    const unsigned int bits = __float_as_uint(v);
    return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}
__device__ __forceinline__ float ordered_uint_to_float(unsigned int key) {
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

// 64-bit shuffle built from two 32-bit ones (kept for the kernels that call it by name).
__device__ __forceinline__ double shfl_down_double(double v, int delta) {
    const int hi = __shfl_down_sync(0xffffffffu, __double2hiint(v), delta);
    const int lo = __shfl_down_sync(0xffffffffu, __double2loint(v), delta);
    return __hiloint2double(hi, lo);
}

namespace detail {
__device__ __forceinline__ float lane_xor(float v, int mask) { return __shfl_xor_sync(0xffffffffu, v, mask); }
__device__ __forceinline__ double lane_xor(double v, int mask) {
    const int hi = __shfl_xor_sync(0xffffffffu, __double2hiint(v), mask);
    const int lo = __shfl_xor_sync(0xffffffffu, __double2loint(v), mask);
    return __hiloint2double(hi, lo);
}
struct AddOp { template <typename T> __device__ __forceinline__ T operator()(T a, T b) const { return a + b; } };
struct MaxOp {
    __device__ __forceinline__ float operator()(float a, float b) const { return fmaxf(a, b); }
    __device__ __forceinline__ double operator()(double a, double b) const { return fmax(a, b); }
};
struct MinOp {
    __device__ __forceinline__ float operator()(float a, float b) const { return fminf(a, b); }
    __device__ __forceinline__ double operator()(double a, double b) const { return fmin(a, b); }
};
template <typename T, typename Op>
__device__ __forceinline__ T warp_butterfly(T v, Op op) {
#pragma unroll
    for (int mask = WARP_SIZE >> 1; mask >= 1; mask >>= 1) v = op(v, lane_xor(v, mask));
    return v;
}
// Block-wide combine: one partial per warp through shared memory, combined again by warp 0.
// The leading barrier lets a kernel call this more than once.
template <typename T, typename Op>
__device__ __forceinline__ T block_combine(T v, Op op, T neutral) {
    __shared__ T partial[WARP_SIZE];
    const int lane = threadIdx.x % WARP_SIZE;
    const int warp = threadIdx.x / WARP_SIZE;
    const int warps = (blockDim.x + WARP_SIZE - 1) / WARP_SIZE;
    v = warp_butterfly(v, op);
    __syncthreads();
    if (lane == 0) partial[warp] = v;
    __syncthreads();
    v = (static_cast<int>(threadIdx.x) < warps) ? partial[threadIdx.x] : neutral;
    if (warp == 0) v = warp_butterfly(v, op);
    return v;
}
}  // namespace detail

__device__ __forceinline__ float warp_reduce_sum(float v) { return detail::warp_butterfly(v, detail::AddOp{}); }
__device__ __forceinline__ double warp_reduce_sum(double v) { return detail::warp_butterfly(v, detail::AddOp{}); }
__device__ __forceinline__ float warp_reduce_max(float v) {
    return ordered_uint_to_float(__reduce_max_sync(0xffffffffu, float_to_ordered_uint(v)));
}
__device__ __forceinline__ float warp_reduce_min(float v) {
    return ordered_uint_to_float(__reduce_min_sync(0xffffffffu, float_to_ordered_uint(v)));
}
__device__ __forceinline__ double warp_reduce_max(double v) { return detail::warp_butterfly(v, detail::MaxOp{}); }
__device__ __forceinline__ double warp_reduce_min(double v) { return detail::warp_butterfly(v, detail::MinOp{}); }

// ---- block reductions (blockDim.x <= 1024; result valid in warp 0) ---------------------------

template <typename T>
__device__ __forceinline__ T block_reduce_sum(T v) { return detail::block_combine(v, detail::AddOp{}, T(0)); }
template <typename T>
__device__ __forceinline__ T block_reduce_max(T v) { return detail::block_combine(v, detail::MaxOp{}, T(-1e38)); }
template <typename T>
__device__ __forceinline__ T block_reduce_min(T v) { return detail::block_combine(v, detail::MinOp{}, T(1e38)); }

// ---- 128-bit accesses ------------------------------------------------------------------------

template <typename T> struct Vec4;
template <> struct Vec4<float> {
    using type = float4;
    static constexpr int width = 4;
    static __device__ __forceinline__ type load(const float* p) { return *reinterpret_cast<const type*>(p); }
    static __device__ __forceinline__ void store(float* p, type v) { *reinterpret_cast<type*>(p) = v; }
};
template <> struct Vec4<double> {
    using type = double2;
    static constexpr int width = 2;
    static __device__ __forceinline__ type load(const double* p) { return *reinterpret_cast<const type*>(p); }
    static __device__ __forceinline__ void store(double* p, type v) { *reinterpret_cast<type*>(p) = v; }
};

// ---- cp.async (global -> shared, 16 bytes, bypassing registers) ------------------------------

__device__ __forceinline__ void cp_async_f4(void* shared_dst, const void* global_src) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(shared_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(global_src) : "memory");
}
// Copies 16 bytes when `valid`, otherwise fills the destination with zeros (src-size operand 0).
__device__ __forceinline__ void cp_async_f4_zfill(void* shared_dst, const void* global_src, bool valid) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(shared_dst));
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(global_src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// ---- SFU math --------------------------------------------------------------------------------

__device__ __forceinline__ float fast_exp(float x) { return __expf(x); }
__device__ __forceinline__ float fast_tanh(float x) { return tanhf(x); }
__device__ __forceinline__ float fast_sigmoid(float x) { return __frcp_rn(1.0f + __expf(-x)); }
__device__ __forceinline__ float fast_rsqrt(float x) { return rsqrtf(x); }

#endif  // __CUDACC__

}  // namespace cudeep
