// Data-movement helpers of the Tensor host type (see tensor_ops.cu).
#pragma once

#include "runtime.h"

namespace cudeep_b200 {

struct StridedView {
    static constexpr int kMaxDims = 8;
    int ndim;
    long long shape[kMaxDims];
    long long strides[kMaxDims];   // in elements
};

// dst (contiguous, row-major over view.shape) = src read through view.strides.
template <typename T>
void strided_copy(const T* src, T* dst, const StridedView& view, cudaStream_t stream);

template <typename T>
void fill(T* dst, T value, long long total, cudaStream_t stream);

// out[i, j] = m[i, j] + row[j]   (reference: broadcast_add_row_kernel, elementwise_kernel.cu:187-204)
template <typename T>
void add_row(const T* m, const T* row, T* out, long long rows, int cols, cudaStream_t stream);

// y = act(x), the epilogue activations as a standalone pass.
void activation(const float* x, float* y, long long total, int act, cudaStream_t stream);

}  // namespace cudeep_b200
