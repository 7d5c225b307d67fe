// Conv2d forward for callers that must not allocate device memory.
//
// Some users of this library run with a fixed device-memory plan: a serving process
// that has handed every free byte to its own allocator, or a control loop that cannot
// afford the failure modes and the implicit synchronisation of an allocation in the
// middle of a step.  The regular convolution entry points take their scratch (the NHWC
// copy of the input and the packed filters) from the stream-ordered allocator; this
// entry point takes it from a fixed array that is part of the library image instead.
//
// The array is a file-scope __device__ object: every GPU that loads this part of the library
// holds its 32 MiB until the process exits.  In host code the array's name is only a handle;
// the device address is looked up once per device with cudaGetSymbolAddress, with that
// device current, and that address is what the kernels receive.
//
// "Loads" is literal: with CUDA's default lazy module loading the array's module is loaded -
// and its 32 MiB taken from the device - by that first look-up, and each kernel variant
// (tile shape, re-layout kernel) is loaded and has its shared-memory limit raised at its first
// launch.  So the calls that must not allocate are the second and later ones of a shape class.
// A caller with a fixed memory plan warms up at start-up, before it hands the free memory to
// its own allocator and before any stream capture: cudeep_b200_conv2d_noalloc_capacity() on
// each device resolves the array, one call per layer shape it will use loads the kernels
// (or the process runs with CUDA_MODULE_LOADING=EAGER).
#include "cudeep_b200.h"

#include "abi_error.h"
#include "conv_igemm.h"

#include <mutex>

namespace {

constexpr size_t kStaticScratchBytes = size_t(32) << 20;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_conv_scratch[kStaticScratchBytes];

std::mutex g_mu;
void* g_scratch_addr[kMaxDevices] = {};

// Device address of the scratch array on the calling thread's current device.
void* static_scratch() {
    int dev = 0;
    CB200_CUDA(cudaGetDevice(&dev));
    CB200_REQUIRE(dev >= 0 && dev < kMaxDevices, "conv2d (no-alloc): device index out of range");
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        CB200_CUDA(cudaGetSymbolAddress(&p, g_conv_scratch));
        CB200_REQUIRE(p != nullptr, "conv2d (no-alloc): scratch symbol has no device address");
        g_scratch_addr[dev] = p;
    }
    return g_scratch_addr[dev];
}

}  // namespace

// Also the warm-up for the current device: resolving the array here loads its module, so the
// 32 MiB are taken now and not inside the first convolution.  Without a usable device it only
// reports the size.
extern "C" size_t cudeep_b200_conv2d_noalloc_capacity(void) {
    try {
        static_scratch();
    } catch (...) {
        cudaGetLastError();
    }
    return kStaticScratchBytes;
}

extern "C" int cudeep_b200_conv2d_forward_noalloc_f32(const float* input, const float* weight,
                                                      const float* bias, float* output, int batch,
                                                      int in_channels, int out_channels, int in_h,
                                                      int in_w, int kernel_h, int kernel_w, int stride_h,
                                                      int stride_w, int pad_h, int pad_w, int epilogue,
                                                      cudeep_b200_stream_t stream) {
    try {
        CB200_REQUIRE(input != nullptr && weight != nullptr && output != nullptr,
                      "conv2d (no-alloc): null tensor pointer");
        CB200_REQUIRE(epilogue >= 0 && epilogue <= 4, "conv2d (no-alloc): unknown epilogue code");
        const cudeep_b200::ConvShape shape{batch, in_channels, out_channels, in_h, in_w, kernel_h,
                                           kernel_w, stride_h, stride_w, pad_h, pad_w};
        cudeep_b200::check_conv_shape(shape);
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        if (!cudeep_b200::conv2d_igemm_supported(shape)) {
            // Shapes the tensor-core path does not take (under 32 output channels or 64 output
            // pixels, strides above 8) run the direct kernel, which needs no scratch.
            cudeep_b200::conv2d_direct<float>(input, weight, bias, output, shape, epilogue, s);
            return CUDEEP_B200_OK;
        }
        const size_t need = cudeep_b200::conv2d_igemm_scratch_bytes(shape, nullptr, nullptr);
        CB200_REQUIRE(need <= kStaticScratchBytes,
                      "conv2d (no-alloc): this shape needs " + std::to_string(need) +
                          " bytes of scratch, the built-in scratch holds " +
                          std::to_string(kStaticScratchBytes) +
                          "; split the batch or use cudeep_b200_conv2d_forward_fused_f32");
        cudeep_b200::conv2d_igemm_with_scratch(input, weight, bias, output, shape, epilogue,
                                               static_scratch(), 0, s);
        return CUDEEP_B200_OK;
    } catch (const std::exception& e) {
        cudeep_b200::set_last_error(e.what());
    } catch (...) {
        cudeep_b200::set_last_error("unknown C++ exception");
    }
    return CUDEEP_B200_ERROR;
}
