// Device memory that several GPUs of one NVSwitch domain can all be written through at once.
//
// A multicast object groups one equally sized physical allocation per GPU.  Mapped into a GPU's
// address space it gives a second address for that memory: a store to it (multimem.st) is carried
// once over NVLink and replicated by the switch into every GPU's allocation, the writer's own
// included.  The row-sharded GEMM uses it so that a rank sends each tile of C once instead of once
// per peer (cudeep::dist::Gather::Multimem).
//
// Built on the driver's virtual-memory API (cuMemCreate / cuMemMap / cuMulticast*), reached through
// cudaGetDriverEntryPoint so that the library still loads on machines without a driver.
#pragma once

#include "runtime.h"

namespace cudeep_b200 {

// True when the current device can take part in a multicast object.
bool multicast_supported();

// Size a buffer of `bytes` must be rounded up to for `world` GPUs (allocation and multicast granularity).
size_t multicast_round_size(int world, size_t bytes);

// One GPU's share: its physical memory, where that is mapped, and where the whole group is mapped.
struct MulticastShare {
    int device = -1;
    size_t size = 0;
    unsigned long long memory = 0;      // CUmemGenericAllocationHandle of this GPU's physical memory
    void* local = nullptr;              // ordinary address of that memory on `device`
    void* group = nullptr;              // address through which a store reaches every GPU's memory
    bool bound = false;
};

// The multicast object as one process sees it.
struct MulticastGroup {
    unsigned long long handle = 0;      // CUmemGenericAllocationHandle of the multicast object
    size_t size = 0;
    int world = 0;
};

// Creates the object for `world` GPUs (exportable to other processes as a file descriptor).
MulticastGroup multicast_create(int world, size_t size);
// A file descriptor another process can turn into the same object; the caller closes it.
int multicast_export_fd(const MulticastGroup& group);
MulticastGroup multicast_import_fd(int fd, int world, size_t size);
// Every participating device is added once, by whichever process drives it, before any binding.
void multicast_add_device(const MulticastGroup& group, int device);

// This GPU's physical memory, mapped at an ordinary address (usable at once, also without a group).
void multicast_allocate(MulticastShare& share, int device, size_t size);
// Binds the share into the group (all devices must have been added) and maps the group address.
void multicast_bind(const MulticastGroup& group, MulticastShare& share);
// Undoes bind and allocate; safe on a half-built share.  Never throws.
void multicast_release(const MulticastGroup& group, MulticastShare& share) noexcept;
void multicast_destroy(MulticastGroup& group) noexcept;

}  // namespace cudeep_b200
