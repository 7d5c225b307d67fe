// Device memory pool and copy helpers.
//
// Same public surface as the reference's include/cudeep/memory.cuh:13-46
// (MemoryPool::instance / allocate / deallocate / release_cached /
// allocated_bytes / cached_bytes, device_malloc / device_free, memcpy_h2d /
// d2h / d2d) so code written against it recompiles unchanged.  Differences in
// behaviour, all invisible to a single-GPU caller:
//   * one pool per CUDA device (the reference keeps a single device-agnostic
//     pool), selected by the calling thread's current device;
//   * requests are rounded up to size classes (256 B below 1 MiB, 2 MiB above)
//     so near-equal sizes reuse each other's blocks;
//   * a block is returned to the pool of the device that allocated it;
//   * the pool is stream-aware: a block freed with deallocate(ptr, stream) carries an event
//     recorded on that stream, and allocate(nbytes, stream) hands it out at once to the same
//     stream but to another stream only when that event has completed, so work still queued
//     on the freeing stream can never be overtaken by the block's next user.  The two calls
//     without a stream mean the legacy default stream.
#pragma once

#include "common.cuh"
#include "error.cuh"

#include <cuda_runtime.h>
#include <cstddef>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace cudeep {

class MemoryPool {
public:
    // Pool of the calling thread's current device.
    static MemoryPool& instance();

    void* allocate(size_t nbytes);
    void deallocate(void* ptr);
    void* allocate(size_t nbytes, cudaStream_t stream);
    void deallocate(void* ptr, cudaStream_t stream);
    void release_cached();
    size_t allocated_bytes() const { return allocated_bytes_; }
    size_t cached_bytes() const { return cached_bytes_; }

    MemoryPool(const MemoryPool&) = delete;
    MemoryPool& operator=(const MemoryPool&) = delete;
    explicit MemoryPool(int device) : device_(device) {}
    ~MemoryPool();

    static size_t size_class(size_t nbytes);

private:
    int device_;
    struct FreeBlock {
        void* ptr;
        cudaStream_t stream;     // stream the block's last use was queued on
        cudaEvent_t ready;       // recorded on that stream when the block was freed
    };
    std::unordered_map<size_t, std::vector<FreeBlock>> free_blocks_;   // size class -> cached blocks
    std::vector<cudaEvent_t> spare_events_;
    std::unordered_map<void*, size_t> live_blocks_;                // block -> size class
    mutable std::mutex mutex_;
    size_t allocated_bytes_ = 0;
    size_t cached_bytes_ = 0;
};

void* device_malloc(size_t nbytes);
void device_free(void* ptr);
void* device_malloc(size_t nbytes, cudaStream_t stream);    // additions: see MemoryPool
void device_free(void* ptr, cudaStream_t stream);
void memcpy_h2d(void* dst, const void* src, size_t nbytes, cudaStream_t stream = nullptr);
void memcpy_d2h(void* dst, const void* src, size_t nbytes, cudaStream_t stream = nullptr);
void memcpy_d2d(void* dst, const void* src, size_t nbytes, cudaStream_t stream = nullptr);

}  // namespace cudeep
