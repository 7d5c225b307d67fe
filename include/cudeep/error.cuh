// Error convention of the C++ surface: every failure is a std::runtime_error (pybind11 turns it
// into a Python RuntimeError).  The three macros carry the names and meaning of the reference's
// include/cudeep/error.cuh:11-40, so sources written against that header compile against this one:
//
//   CUDEEP_CHECK_CUDA(expr)     throws when a CUDA runtime call does not return cudaSuccess
//   CUDEEP_CHECK_LAST_KERNEL()  throws when the launch just made was rejected (cudaGetLastError;
//                               asynchronous execution errors surface at the next synchronising call)
//   CUDEEP_ASSERT(cond, msg)    throws when a shape / dtype / contiguity precondition fails
#pragma once

#include <cuda_runtime.h>
#include <stdexcept>
#include <string>

namespace cudeep {
namespace detail {

[[noreturn]] inline void raise_at(const char* what, const char* detail, const char* file, int line) {
    std::string text(what);
    text += file;
    text += ':';
    text += std::to_string(line);
    text += " — ";
    text += detail;
    throw std::runtime_error(text);
}

inline void require_cuda_ok(cudaError_t status, const char* what, const char* file, int line) {
    if (status != cudaSuccess) raise_at(what, cudaGetErrorString(status), file, line);
}

}  // namespace detail
}  // namespace cudeep

#define CUDEEP_CHECK_CUDA(call) \
    ::cudeep::detail::require_cuda_ok((call), "CUDA error at ", __FILE__, __LINE__)

#define CUDEEP_CHECK_LAST_KERNEL() \
    ::cudeep::detail::require_cuda_ok(cudaGetLastError(), "Kernel launch error at ", __FILE__, __LINE__)

#define CUDEEP_ASSERT(cond, msg)                                                                     \
    do {                                                                                             \
        if (!(cond)) {                                                                               \
            throw std::runtime_error(std::string("cuDeep assertion failed: ") + (msg) + " at " +     \
                                     __FILE__ + ":" + std::to_string(__LINE__));                     \
        }                                                                                            \
    } while (0)
