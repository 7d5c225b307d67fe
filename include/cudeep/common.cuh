// Enums shared by the C++ surface; values match the reference's include/cudeep/common.cuh:10-19
// (they are part of the ABI of the Tensor class and of the Python module).
#pragma once

#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>

namespace cudeep {

enum class DType { Float16, Float32, Float64 };
enum class Layout { NCHW, NHWC };

inline size_t dtype_size(DType t) { return t == DType::Float16 ? 2 : t == DType::Float32 ? 4 : 8; }

}  // namespace cudeep
