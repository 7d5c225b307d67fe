#include "runtime.h"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <unordered_set>
#include <vector>
#include <memory>

namespace cudeep_b200 {

// One status word per device image of this library.  Kernels write a non-zero
// code here when a bounded wait gives up; the host reads it on request.
__device__ uint32_t g_status_word[4];

static const char* base_name(const char* path) {
    const char* base = path;
    for (const char* p = path; *p; ++p)
        if (*p == '/') base = p + 1;
    return base;
}

void throw_cuda(cudaError_t err, const char* what, const char* file, int line) {
    cudaGetLastError();      // reported here: a later launch check must not find it again
    throw std::runtime_error(std::string("CUDA error: ") + cudaGetErrorString(err) + " in " + what +
                             " (" + base_name(file) + ":" + std::to_string(line) + ")");
}
void throw_msg(const std::string& msg, const char* file, int line) {
    throw std::runtime_error("cudeep_b200: " + msg + " (" + base_name(file) + ":" +
                             std::to_string(line) + ")");
}

namespace {

struct DeviceState {
    DeviceInfo info;
    std::mutex mu;
    std::unordered_set<const void*> smem_done;
    cudaMemPool_t scratch_pool = nullptr;      // created on first scratch_alloc
};

std::mutex g_mu;
std::vector<std::unique_ptr<DeviceState>> g_devices;

DeviceState& state() {
    int dev = 0;
    CB200_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(g_mu);
    if (dev >= static_cast<int>(g_devices.size())) g_devices.resize(dev + 1);
    if (!g_devices[dev]) {
        auto st = std::make_unique<DeviceState>();
        cudaDeviceProp prop{};
        CB200_CUDA(cudaGetDeviceProperties(&prop, dev));
        st->info.device = dev;
        st->info.num_sms = prop.multiProcessorCount;
        st->info.cc_major = prop.major;
        st->info.cc_minor = prop.minor;
        st->info.smem_optin = prop.sharedMemPerBlockOptin;
        void* p = nullptr;
        CB200_CUDA(cudaGetSymbolAddress(&p, g_status_word));
        st->info.status_word = static_cast<uint32_t*>(p);
        CB200_CUDA(cudaMemset(p, 0, sizeof(uint32_t) * 4));
        g_devices[dev] = std::move(st);
    }
    return *g_devices[dev];
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q{};
        CB200_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
        CB200_REQUIRE(p != nullptr && q == cudaDriverEntryPointSuccess,
                      "driver does not provide cuTensorMapEncodeTiled");
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

}  // namespace

const DeviceInfo& device_info() { return state().info; }

void ensure_dynamic_smem(const void* func, size_t bytes) {
    DeviceState& st = state();
    std::lock_guard<std::mutex> lock(st.mu);
    if (st.smem_done.count(func)) return;
    CB200_REQUIRE(bytes <= st.info.smem_optin, "kernel needs more shared memory than the device offers");
    CB200_CUDA(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(bytes)));
    st.smem_done.insert(func);
}

bool trace_enabled() {
    static const bool on = [] {
        const char* v = std::getenv("CUDEEP_LOG");
        return v != nullptr && v[0] != '\0' && v[0] != '0';
    }();
    return on;
}

void trace(const char* format, ...) {
    char line[512];
    va_list args;
    va_start(args, format);
    std::vsnprintf(line, sizeof(line), format, args);
    va_end(args);
    std::fprintf(stderr, "[cudeep_b200] %s\n", line);
}

bool programmatic_launch_enabled() {
    static const bool on = [] {
        const char* v = std::getenv("CUDEEP_B200_PDL");
        return !(v != nullptr && v[0] == '0');
    }();
    return on;
}

namespace {
// The library's own stream-ordered pool on the current device.  It is private so that its release
// threshold (keep freed scratch cached across synchronisations) does not change how the device's
// default pool behaves for other cudaMallocAsync users in the process.
cudaMemPool_t scratch_pool() {
    DeviceState& st = state();
    std::lock_guard<std::mutex> lock(st.mu);
    if (st.scratch_pool == nullptr) {
        cudaMemPoolProps props{};
        props.allocType = cudaMemAllocationTypePinned;
        props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice;
        props.location.id = st.info.device;
        cudaMemPool_t pool = nullptr;
        CB200_CUDA(cudaMemPoolCreate(&pool, &props));
        uint64_t keep = UINT64_MAX;
        CB200_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
        st.scratch_pool = pool;
    }
    return st.scratch_pool;
}
}  // namespace

void* scratch_alloc(size_t bytes, cudaStream_t stream) {
    void* ptr = nullptr;
    CB200_CUDA(cudaMallocFromPoolAsync(&ptr, bytes, scratch_pool(), stream));
    return ptr;
}

void scratch_trim(size_t keep_bytes) {
    DeviceState& st = state();
    cudaMemPool_t pool = nullptr;
    {
        std::lock_guard<std::mutex> lock(st.mu);
        pool = st.scratch_pool;
    }
    if (pool != nullptr) CB200_CUDA(cudaMemPoolTrimTo(pool, keep_bytes));
}

void scratch_free(void* ptr, cudaStream_t stream) noexcept {
    if (ptr != nullptr) cudaFreeAsync(ptr, stream);
}

uint32_t read_device_status(bool clear) {
    const DeviceInfo& info = device_info();
    CB200_CUDA(cudaDeviceSynchronize());
    uint32_t v = 0;
    CB200_CUDA(cudaMemcpy(&v, info.status_word, sizeof(v), cudaMemcpyDeviceToHost));
    if (clear && v != 0) CB200_CUDA(cudaMemset(info.status_word, 0, sizeof(uint32_t)));
    return v;
}

namespace {
void encode_map(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, uint32_t elem_bytes, int rank,
                const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box, TmaSwizzle swizzle,
                const uint32_t* element_strides) {
    CB200_REQUIRE(rank >= 1 && rank <= 5, "tensor map rank must be 1..5");
    CB200_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15u) == 0, "TMA base address must be 16-byte aligned");
    cuuint64_t gdim[5];
    cuuint64_t gstride[4];
    cuuint32_t gbox[5];
    cuuint32_t estride[5];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        gbox[i] = box[i];
        estride[i] = element_strides ? element_strides[i] : 1;
        CB200_REQUIRE(box[i] >= 1 && box[i] <= 256, "TMA box extent must be 1..256");
        CB200_REQUIRE(estride[i] >= 1 && estride[i] <= 8 && box[i] % estride[i] == 0,
                      "TMA element stride must be 1..8 and divide the box extent");
    }
    for (int i = 0; i + 1 < rank; ++i) {
        gstride[i] = strides_bytes[i];
        CB200_REQUIRE((strides_bytes[i] & 15u) == 0, "TMA strides must be multiples of 16 bytes");
    }
    if (swizzle != TmaSwizzle::None)
        CB200_REQUIRE(box[0] * elem_bytes == 128, "128-byte swizzle needs a 128-byte inner box");
    const CUtensorMapSwizzle sw = swizzle == TmaSwizzle::B128         ? CU_TENSOR_MAP_SWIZZLE_128B
                                  : swizzle == TmaSwizzle::B128Atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                                                      : CU_TENSOR_MAP_SWIZZLE_NONE;
    CUresult r = encode_fn()(map, dtype, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim, gstride,
                             gbox, estride, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    CB200_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
}
}  // namespace

void encode_tensor_map(CUtensorMap* map, const float* base, int rank, const uint64_t* dims,
                       const uint64_t* strides_bytes, const uint32_t* box, TmaSwizzle swizzle,
                       const uint32_t* element_strides) {
    encode_map(map, base, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, rank, dims, strides_bytes, box, swizzle,
               element_strides);
}

void encode_tensor_map_f16(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                           const uint64_t* strides_bytes, const uint32_t* box, TmaSwizzle swizzle) {
    encode_map(map, base, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, rank, dims, strides_bytes, box, swizzle, nullptr);
}

}  // namespace cudeep_b200
