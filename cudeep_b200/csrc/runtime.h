// Host-side plumbing shared by all launchers: error convention, per-device
// state (SM count, status word, opt-in shared memory), TMA descriptor encoding.
#pragma once

#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>
#include <stdexcept>
#include <string>

namespace cudeep_b200 {

// Errors are C++ exceptions (std::runtime_error), the convention of the
// reference's CUDEEP_CHECK_CUDA / CUDEEP_ASSERT (include/cudeep/error.cuh:11-40).
// The C ABI converts them to status codes.
[[noreturn]] void throw_cuda(cudaError_t err, const char* what, const char* file, int line);
[[noreturn]] void throw_msg(const std::string& msg, const char* file, int line);

#define CB200_CUDA(call)                                                        \
    do {                                                                        \
        cudaError_t cb200_err_ = (call);                                        \
        if (cb200_err_ != cudaSuccess)                                          \
            ::cudeep_b200::throw_cuda(cb200_err_, #call, __FILE__, __LINE__);   \
    } while (0)

#define CB200_REQUIRE(cond, msg)                                                \
    do {                                                                        \
        if (!(cond)) ::cudeep_b200::throw_msg((msg), __FILE__, __LINE__);       \
    } while (0)

#define CB200_CHECK_LAUNCH() CB200_CUDA(cudaGetLastError())

// Dispatch trace: with CUDEEP_LOG=1 in the environment (read once) every launcher writes one line
// to stderr saying which kernel a call took and with what tile / cluster / pipeline shape - the way
// to see that a shape went to the strict-precision or the direct kernel instead of the tensor cores.
bool trace_enabled();
void trace(const char* format, ...) __attribute__((format(printf, 1, 2)));
#define CB200_TRACE(...)                                                        \
    do {                                                                        \
        if (::cudeep_b200::trace_enabled()) ::cudeep_b200::trace(__VA_ARGS__);  \
    } while (0)

struct DeviceInfo {
    int device = -1;
    int num_sms = 0;
    int cc_major = 0, cc_minor = 0;
    size_t smem_optin = 0;
    uint32_t* status_word = nullptr;   // device address of this device's status word
};

// State of the current device, created on first use (thread-safe).
const DeviceInfo& device_info();

// Raise the dynamic shared-memory limit of `func` on the current device once.
void ensure_dynamic_smem(const void* func, size_t bytes);

// Stream-ordered scratch (cudaMallocFromPoolAsync / cudaFreeAsync on `stream`) from a memory pool
// of the library's own on the current device; freed scratch stays cached in that pool instead of
// going back to the driver at every synchronisation.  scratch_trim returns all but `keep_bytes` of
// the cached memory to the driver (memory in use is not touched).
void* scratch_alloc(size_t bytes, cudaStream_t stream);
void scratch_free(void* ptr, cudaStream_t stream) noexcept;
void scratch_trim(size_t keep_bytes);

// Read-and-clear the current device's kernel status word (synchronises the device).
uint32_t read_device_status(bool clear);

enum class TmaSwizzle {
    None,
    B128,          // 16-byte chunks XOR-ed within each 128-byte row, period 8 rows
    B128Atom32,    // 32-byte chunks XOR-ed within each 128-byte row, period 4 rows
};

// 64-byte aligned TMA descriptor for an fp32 tensor of rank <= 5.
// dims[0] is the contiguous dimension; strides_bytes[i] is the stride of
// dims[i+1].  Out-of-range elements read as zero.  With a swizzle the inner
// box must span exactly 128 bytes (narrower boxes are not packed densely in
// shared memory: measured, a {8, 4, 128} box did not land as 128-byte rows).
// The same for 2-byte (FP16) elements: dims, boxes and coordinates count elements.
void encode_tensor_map_f16(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                           const uint64_t* strides_bytes, const uint32_t* box, TmaSwizzle swizzle);
// element_strides (optional, one per dimension): traverse dimension i in steps of that many
// elements; box[i] then is the extent traversed (a multiple of the step) and box[i] / step
// elements are loaded.
void encode_tensor_map(CUtensorMap* map, const float* base, int rank, const uint64_t* dims,
                       const uint64_t* strides_bytes, const uint32_t* box, TmaSwizzle swizzle,
                       const uint32_t* element_strides = nullptr);

}  // namespace cudeep_b200
