// Multicast memory over NVSwitch (see multicast.h).
#include "multicast.h"

#include <mutex>

namespace cudeep_b200 {

namespace {

struct DriverApi {
    decltype(&cuDeviceGet) DeviceGet = nullptr;
    decltype(&cuDeviceGetAttribute) DeviceGetAttribute = nullptr;
    decltype(&cuMemGetAllocationGranularity) MemGetAllocationGranularity = nullptr;
    decltype(&cuMemCreate) MemCreate = nullptr;
    decltype(&cuMemRelease) MemRelease = nullptr;
    decltype(&cuMemAddressReserve) MemAddressReserve = nullptr;
    decltype(&cuMemAddressFree) MemAddressFree = nullptr;
    decltype(&cuMemMap) MemMap = nullptr;
    decltype(&cuMemUnmap) MemUnmap = nullptr;
    decltype(&cuMemSetAccess) MemSetAccess = nullptr;
    decltype(&cuMemExportToShareableHandle) MemExportToShareableHandle = nullptr;
    decltype(&cuMemImportFromShareableHandle) MemImportFromShareableHandle = nullptr;
    decltype(&cuMulticastCreate) MulticastCreate = nullptr;
    decltype(&cuMulticastAddDevice) MulticastAddDevice = nullptr;
    decltype(&cuMulticastBindMem) MulticastBindMem = nullptr;
    decltype(&cuMulticastUnbind) MulticastUnbind = nullptr;
    decltype(&cuMulticastGetGranularity) MulticastGetGranularity = nullptr;
};

const DriverApi& driver() {
    static DriverApi api;
    static std::once_flag once;
    static std::string failure;
    std::call_once(once, [] {
        CB200_CUDA(cudaFree(nullptr));      // a context, so that the driver entry points resolve
        auto bind = [&](auto& slot, const char* name) {
            void* p = nullptr;
            cudaDriverEntryPointQueryResult q{};
            const cudaError_t err = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
            if (err != cudaSuccess || p == nullptr || q != cudaDriverEntryPointSuccess) {
                cudaGetLastError();
                if (failure.empty()) failure = std::string("the driver does not provide ") + name;
                return;
            }
            slot = reinterpret_cast<std::remove_reference_t<decltype(slot)>>(p);
        };
        bind(api.DeviceGet, "cuDeviceGet");
        bind(api.DeviceGetAttribute, "cuDeviceGetAttribute");
        bind(api.MemGetAllocationGranularity, "cuMemGetAllocationGranularity");
        bind(api.MemCreate, "cuMemCreate");
        bind(api.MemRelease, "cuMemRelease");
        bind(api.MemAddressReserve, "cuMemAddressReserve");
        bind(api.MemAddressFree, "cuMemAddressFree");
        bind(api.MemMap, "cuMemMap");
        bind(api.MemUnmap, "cuMemUnmap");
        bind(api.MemSetAccess, "cuMemSetAccess");
        bind(api.MemExportToShareableHandle, "cuMemExportToShareableHandle");
        bind(api.MemImportFromShareableHandle, "cuMemImportFromShareableHandle");
        bind(api.MulticastCreate, "cuMulticastCreate");
        bind(api.MulticastAddDevice, "cuMulticastAddDevice");
        bind(api.MulticastBindMem, "cuMulticastBindMem");
        bind(api.MulticastUnbind, "cuMulticastUnbind");
        bind(api.MulticastGetGranularity, "cuMulticastGetGranularity");
    });
    if (!failure.empty()) throw std::runtime_error("cudeep_b200: " + failure);
    return api;
}

void drv_ok(CUresult r, const char* what) {
    if (r != CUDA_SUCCESS)
        throw std::runtime_error(std::string("cudeep_b200: ") + what + " failed with driver error " +
                                 std::to_string(int(r)));
}

constexpr CUmemAllocationHandleType kHandleType = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;

CUmemAllocationProp share_prop(int device) {
    CUmemAllocationProp prop{};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device;
    prop.requestedHandleTypes = kHandleType;
    return prop;
}

CUmulticastObjectProp group_prop(int world, size_t size) {
    CUmulticastObjectProp prop{};
    prop.numDevices = static_cast<unsigned int>(world);
    prop.size = size;
    prop.handleTypes = kHandleType;
    prop.flags = 0;
    return prop;
}

void map_for_device(CUdeviceptr* va, size_t size, size_t align, unsigned long long handle, int device,
                    const char* what) {
    const DriverApi& d = driver();
    drv_ok(d.MemAddressReserve(va, size, align, 0, 0), "cuMemAddressReserve");
    CUresult r = d.MemMap(*va, size, 0, handle, 0);
    if (r == CUDA_SUCCESS) {
        CUmemAccessDesc access{};
        access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        access.location.id = device;
        access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
        r = d.MemSetAccess(*va, size, &access, 1);
        if (r != CUDA_SUCCESS) d.MemUnmap(*va, size);
    }
    if (r != CUDA_SUCCESS) {
        d.MemAddressFree(*va, size);
        *va = 0;
        drv_ok(r, what);
    }
}

}  // namespace

bool multicast_supported() {
    try {
        const DriverApi& d = driver();
        int dev = 0;
        CB200_CUDA(cudaGetDevice(&dev));
        CUdevice cu = 0;
        if (d.DeviceGet(&cu, dev) != CUDA_SUCCESS) return false;
        int yes = 0;
        if (d.DeviceGetAttribute(&yes, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cu) != CUDA_SUCCESS) return false;
        return yes != 0;
    } catch (...) {
        return false;
    }
}

size_t multicast_round_size(int world, size_t bytes) {
    const DriverApi& d = driver();
    int dev = 0;
    CB200_CUDA(cudaGetDevice(&dev));
    size_t alloc_gran = 0, mc_gran = 0;
    const CUmemAllocationProp aprop = share_prop(dev);
    drv_ok(d.MemGetAllocationGranularity(&alloc_gran, &aprop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED),
           "cuMemGetAllocationGranularity");
    const CUmulticastObjectProp mprop = group_prop(world < 2 ? 2 : world, bytes);
    drv_ok(d.MulticastGetGranularity(&mc_gran, &mprop, CU_MULTICAST_GRANULARITY_RECOMMENDED),
           "cuMulticastGetGranularity");
    const size_t gran = alloc_gran > mc_gran ? alloc_gran : mc_gran;
    return (bytes + gran - 1) / gran * gran;
}

MulticastGroup multicast_create(int world, size_t size) {
    CB200_REQUIRE(world >= 2, "a multicast group needs at least two GPUs");
    MulticastGroup g;
    g.size = size;
    g.world = world;
    const CUmulticastObjectProp prop = group_prop(world, size);
    CUmemGenericAllocationHandle h = 0;
    drv_ok(driver().MulticastCreate(&h, &prop), "cuMulticastCreate");
    g.handle = h;
    return g;
}

int multicast_export_fd(const MulticastGroup& group) {
    int fd = -1;
    drv_ok(driver().MemExportToShareableHandle(&fd, group.handle, kHandleType, 0), "cuMemExportToShareableHandle");
    return fd;
}

MulticastGroup multicast_import_fd(int fd, int world, size_t size) {
    MulticastGroup g;
    g.size = size;
    g.world = world;
    CUmemGenericAllocationHandle h = 0;
    drv_ok(driver().MemImportFromShareableHandle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), kHandleType),
           "cuMemImportFromShareableHandle");
    g.handle = h;
    return g;
}

void multicast_add_device(const MulticastGroup& group, int device) {
    CUdevice cu = 0;
    drv_ok(driver().DeviceGet(&cu, device), "cuDeviceGet");
    drv_ok(driver().MulticastAddDevice(group.handle, cu), "cuMulticastAddDevice");
}

void multicast_allocate(MulticastShare& share, int device, size_t size) {
    const DriverApi& d = driver();
    share.device = device;
    share.size = size;
    const CUmemAllocationProp prop = share_prop(device);
    CUmemGenericAllocationHandle h = 0;
    drv_ok(d.MemCreate(&h, size, &prop, 0), "cuMemCreate");
    share.memory = h;
    CUdeviceptr va = 0;
    try {
        map_for_device(&va, size, multicast_round_size(2, 1), share.memory, device, "mapping the GPU's share");
    } catch (...) {
        d.MemRelease(share.memory);
        share.memory = 0;
        throw;
    }
    share.local = reinterpret_cast<void*>(va);
}

void multicast_bind(const MulticastGroup& group, MulticastShare& share) {
    const DriverApi& d = driver();
    CB200_REQUIRE(share.memory != 0 && share.size == group.size, "multicast_bind: share and group sizes differ");
    drv_ok(d.MulticastBindMem(group.handle, 0, share.memory, 0, share.size, 0), "cuMulticastBindMem");
    share.bound = true;
    CUdeviceptr va = 0;
    map_for_device(&va, share.size, multicast_round_size(group.world, 1), group.handle, share.device,
                   "mapping the multicast object");
    share.group = reinterpret_cast<void*>(va);
}

void multicast_release(const MulticastGroup& group, MulticastShare& share) noexcept {
    try {
        const DriverApi& d = driver();
        if (share.group != nullptr) {
            d.MemUnmap(reinterpret_cast<CUdeviceptr>(share.group), share.size);
            d.MemAddressFree(reinterpret_cast<CUdeviceptr>(share.group), share.size);
            share.group = nullptr;
        }
        if (share.bound && group.handle != 0) {
            CUdevice cu = 0;
            if (d.DeviceGet(&cu, share.device) == CUDA_SUCCESS) d.MulticastUnbind(group.handle, cu, 0, share.size);
            share.bound = false;
        }
        if (share.local != nullptr) {
            d.MemUnmap(reinterpret_cast<CUdeviceptr>(share.local), share.size);
            d.MemAddressFree(reinterpret_cast<CUdeviceptr>(share.local), share.size);
            share.local = nullptr;
        }
        if (share.memory != 0) {
            d.MemRelease(share.memory);
            share.memory = 0;
        }
    } catch (...) {
    }
}

void multicast_destroy(MulticastGroup& group) noexcept {
    try {
        if (group.handle != 0) driver().MemRelease(group.handle);
    } catch (...) {
    }
    group.handle = 0;
}

}  // namespace cudeep_b200
