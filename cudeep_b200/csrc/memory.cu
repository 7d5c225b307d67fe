#include "cudeep/memory.cuh"
#include "cudeep/stream.cuh"
#include "runtime.h"

#include <memory>

namespace cudeep {

namespace {
std::mutex g_pools_mu;
std::vector<std::unique_ptr<MemoryPool>> g_pools;
// Which pool owns a live block (blocks may be freed while another device is current).
std::mutex g_owner_mu;
std::unordered_map<void*, MemoryPool*> g_owner;
}  // namespace

size_t MemoryPool::size_class(size_t nbytes) {
    if (nbytes == 0) nbytes = 1;
    const size_t gran = nbytes < (size_t(1) << 20) ? size_t(256) : (size_t(2) << 20);
    return (nbytes + gran - 1) / gran * gran;
}

MemoryPool& MemoryPool::instance() {
    int dev = 0;
    CB200_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(g_pools_mu);
    if (dev >= static_cast<int>(g_pools.size())) g_pools.resize(dev + 1);
    if (!g_pools[dev]) g_pools[dev] = std::make_unique<MemoryPool>(dev);
    return *g_pools[dev];
}

MemoryPool::~MemoryPool() {
    // The CUDA context may already be gone at process exit; ignore errors.
    for (auto& kv : free_blocks_)
        for (void* p : kv.second) cudaFree(p);
    for (auto& kv : live_blocks_) cudaFree(kv.first);
}

void* MemoryPool::allocate(size_t nbytes) {
    const size_t bin = size_class(nbytes);
    void* ptr = nullptr;
    {
        std::lock_guard<std::mutex> lock(mutex_);
        auto it = free_blocks_.find(bin);
        if (it != free_blocks_.end() && !it->second.empty()) {
            ptr = it->second.back();
            it->second.pop_back();
            cached_bytes_ -= bin;
        }
    }
    if (ptr == nullptr) {
        int prev = 0;
        CB200_CUDA(cudaGetDevice(&prev));
        if (prev != device_) CB200_CUDA(cudaSetDevice(device_));
        cudaError_t err = cudaMalloc(&ptr, bin);
        if (err == cudaErrorMemoryAllocation) {
            cudaGetLastError();
            release_cached();                 // give cached blocks back and retry once
            err = cudaMalloc(&ptr, bin);
        }
        if (prev != device_) cudaSetDevice(prev);
        if (err != cudaSuccess) cudeep_b200::throw_cuda(err, "cudaMalloc", __FILE__, __LINE__);
    }
    {
        std::lock_guard<std::mutex> lock(mutex_);
        live_blocks_[ptr] = bin;
        allocated_bytes_ += bin;
    }
    {
        std::lock_guard<std::mutex> lock(g_owner_mu);
        g_owner[ptr] = this;
    }
    return ptr;
}

void MemoryPool::deallocate(void* ptr) {
    if (ptr == nullptr) return;
    std::lock_guard<std::mutex> lock(mutex_);
    auto it = live_blocks_.find(ptr);
    if (it == live_blocks_.end()) return;     // not ours: ignore, as the reference does
    const size_t bin = it->second;
    live_blocks_.erase(it);
    allocated_bytes_ -= bin;
    free_blocks_[bin].push_back(ptr);
    cached_bytes_ += bin;
}

void MemoryPool::release_cached() {
    std::vector<void*> doomed;
    {
        std::lock_guard<std::mutex> lock(mutex_);
        for (auto& kv : free_blocks_)
            for (void* p : kv.second) doomed.push_back(p);
        free_blocks_.clear();
        cached_bytes_ = 0;
    }
    {
        std::lock_guard<std::mutex> lock(g_owner_mu);
        for (void* p : doomed) g_owner.erase(p);
    }
    for (void* p : doomed) cudaFree(p);
}

void* device_malloc(size_t nbytes) { return MemoryPool::instance().allocate(nbytes); }

void device_free(void* ptr) {
    if (ptr == nullptr) return;
    MemoryPool* owner = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_owner_mu);
        auto it = g_owner.find(ptr);
        if (it != g_owner.end()) owner = it->second;
    }
    if (owner != nullptr) owner->deallocate(ptr);
}

static void copy(void* dst, const void* src, size_t nbytes, cudaMemcpyKind kind, cudaStream_t stream) {
    if (nbytes == 0) return;
    if (stream) CB200_CUDA(cudaMemcpyAsync(dst, src, nbytes, kind, stream));
    else CB200_CUDA(cudaMemcpy(dst, src, nbytes, kind));
}
void memcpy_h2d(void* dst, const void* src, size_t nbytes, cudaStream_t stream) {
    copy(dst, src, nbytes, cudaMemcpyHostToDevice, stream);
}
void memcpy_d2h(void* dst, const void* src, size_t nbytes, cudaStream_t stream) {
    copy(dst, src, nbytes, cudaMemcpyDeviceToHost, stream);
}
void memcpy_d2d(void* dst, const void* src, size_t nbytes, cudaStream_t stream) {
    copy(dst, src, nbytes, cudaMemcpyDeviceToDevice, stream);
}

// ------------------------------------------------------------------ Stream / Event
Stream::Stream() { CB200_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking)); }
Stream::~Stream() { if (stream_) cudaStreamDestroy(stream_); }
Stream::Stream(Stream&& other) noexcept : stream_(other.stream_) { other.stream_ = nullptr; }
Stream& Stream::operator=(Stream&& other) noexcept {
    if (this != &other) {
        if (stream_) cudaStreamDestroy(stream_);
        stream_ = other.stream_;
        other.stream_ = nullptr;
    }
    return *this;
}
void Stream::synchronize() const { CB200_CUDA(cudaStreamSynchronize(stream_)); }

Event::Event() { CB200_CUDA(cudaEventCreate(&event_)); }
Event::~Event() { if (event_) cudaEventDestroy(event_); }
Event::Event(Event&& other) noexcept : event_(other.event_) { other.event_ = nullptr; }
Event& Event::operator=(Event&& other) noexcept {
    if (this != &other) {
        if (event_) cudaEventDestroy(event_);
        event_ = other.event_;
        other.event_ = nullptr;
    }
    return *this;
}
void Event::record(cudaStream_t stream) { CB200_CUDA(cudaEventRecord(event_, stream)); }
void Event::synchronize() const { CB200_CUDA(cudaEventSynchronize(event_)); }
float Event::elapsed_ms(const Event& start) const {
    float ms = 0.0f;
    CB200_CUDA(cudaEventElapsedTime(&ms, start.event_, event_));
    return ms;
}

}  // namespace cudeep
