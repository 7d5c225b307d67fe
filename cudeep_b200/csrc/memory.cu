#include "cudeep/memory.cuh"

#include <new>
#include "cudeep/stream.cuh"
#include "runtime.h"

#include <memory>
#include <unordered_set>

namespace cudeep {

namespace {
// Streams created and destroyed through this library.  A tensor may outlive the stream it worked
// on; the pool must then not hand that stream to the CUDA runtime again.  Streams are drained
// before they are destroyed, so storage last used on a destroyed stream has no work pending.
std::mutex g_streams_mu;
std::unordered_set<cudaStream_t> g_dead_streams;

cudaStream_t create_tracked_stream() {
    cudaStream_t s = nullptr;
    CB200_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    std::lock_guard<std::mutex> lock(g_streams_mu);
    g_dead_streams.erase(s);           // the driver may reuse a handle value
    return s;
}

void destroy_tracked_stream(cudaStream_t s) noexcept {
    if (s == nullptr) return;
    cudaStreamSynchronize(s);
    {
        std::lock_guard<std::mutex> lock(g_streams_mu);
        g_dead_streams.insert(s);
    }
    cudaStreamDestroy(s);
}

bool stream_is_dead(cudaStream_t s) {
    if (s == nullptr) return false;
    std::lock_guard<std::mutex> lock(g_streams_mu);
    return g_dead_streams.count(s) != 0;
}

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

namespace {
// Makes `device` current for the lifetime of the guard.
struct DeviceGuard {
    int prev = 0;
    bool switched = false;
    explicit DeviceGuard(int device) {
        CB200_CUDA(cudaGetDevice(&prev));
        if (prev != device) {
            CB200_CUDA(cudaSetDevice(device));
            switched = true;
        }
    }
    // Non-throwing form for release paths: on failure the current device is left as it is.
    DeviceGuard(int device, std::nothrow_t) noexcept {
        if (cudaGetDevice(&prev) == cudaSuccess && prev != device) switched = cudaSetDevice(device) == cudaSuccess;
    }
    ~DeviceGuard() {
        if (switched) cudaSetDevice(prev);
    }
};
}  // namespace

MemoryPool::~MemoryPool() {
    // The CUDA context may already be gone at process exit; ignore errors.
    for (auto& kv : free_blocks_)
        for (FreeBlock& b : kv.second) {
            cudaFree(b.ptr);
            cudaEventDestroy(b.ready);
        }
    for (cudaEvent_t e : spare_events_) cudaEventDestroy(e);
    for (auto& kv : live_blocks_) cudaFree(kv.first);
}

void* MemoryPool::allocate(size_t nbytes) { return allocate(nbytes, nullptr); }
void MemoryPool::deallocate(void* ptr) { deallocate(ptr, nullptr); }

void* MemoryPool::allocate(size_t nbytes, cudaStream_t stream) {
    const size_t bin = size_class(nbytes);
    void* ptr = nullptr;
    {
        std::lock_guard<std::mutex> lock(mutex_);
        auto it = free_blocks_.find(bin);
        if (it != free_blocks_.end()) {
            std::vector<FreeBlock>& blocks = it->second;
            int pick = -1;
            // A block last used on the same stream is ordered behind that use by the stream
            // itself; any other block only once the work queued before its release has drained.
            for (int i = static_cast<int>(blocks.size()) - 1; i >= 0 && pick < 0; --i)
                if (blocks[i].stream == stream) pick = i;
            for (int i = static_cast<int>(blocks.size()) - 1; i >= 0 && pick < 0; --i)
                if (cudaEventQuery(blocks[i].ready) == cudaSuccess) pick = i;
            cudaGetLastError();      // cudaErrorNotReady from the queries is not an error
            if (pick >= 0) {
                ptr = blocks[pick].ptr;
                spare_events_.push_back(blocks[pick].ready);
                blocks.erase(blocks.begin() + pick);
                cached_bytes_ -= bin;
            }
        }
    }
    if (ptr == nullptr) {
        DeviceGuard guard(device_);
        cudaError_t err = cudaMalloc(&ptr, bin);
        if (err == cudaErrorMemoryAllocation) {
            cudaGetLastError();
            release_cached();                 // give cached blocks back and retry once
            err = cudaMalloc(&ptr, bin);
        }
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

// Never throws: it runs from destructors (Tensor storage), possibly while another exception
// unwinds.  When the release event cannot be created or recorded (a context already in error)
// the block goes straight back to the driver, which waits for the device itself.
void MemoryPool::deallocate(void* ptr, cudaStream_t stream) {
    if (ptr == nullptr) return;
    std::lock_guard<std::mutex> lock(mutex_);
    auto it = live_blocks_.find(ptr);
    if (it == live_blocks_.end()) return;     // not ours: ignore, as the reference does
    const size_t bin = it->second;
    live_blocks_.erase(it);
    allocated_bytes_ -= bin;
    cudaEvent_t ready = nullptr;
    cudaError_t err = cudaSuccess;
    {
        DeviceGuard guard(device_, std::nothrow);
        if (!spare_events_.empty()) {
            ready = spare_events_.back();
            spare_events_.pop_back();
        } else {
            err = cudaEventCreateWithFlags(&ready, cudaEventDisableTiming);
            if (err != cudaSuccess) ready = nullptr;
        }
        // A stream of this library that is gone was drained when it was destroyed: nothing is
        // pending on the block.  (Streams created elsewhere must outlive the storage used on them.)
        if (stream_is_dead(stream)) stream = nullptr;
        if (err == cudaSuccess) err = cudaEventRecord(ready, stream);
        if (err != cudaSuccess) {
            cudaGetLastError();
            if (ready != nullptr) spare_events_.push_back(ready);
            cudaFree(ptr);
            std::lock_guard<std::mutex> owner_lock(g_owner_mu);
            g_owner.erase(ptr);
            return;
        }
    }
    free_blocks_[bin].push_back(FreeBlock{ptr, stream, ready});
    cached_bytes_ += bin;
}

void MemoryPool::release_cached() {
    std::vector<FreeBlock> doomed;
    {
        std::lock_guard<std::mutex> lock(mutex_);
        for (auto& kv : free_blocks_)
            for (FreeBlock& b : kv.second) doomed.push_back(b);
        free_blocks_.clear();
        cached_bytes_ = 0;
    }
    {
        std::lock_guard<std::mutex> lock(g_owner_mu);
        for (FreeBlock& b : doomed) g_owner.erase(b.ptr);
    }
    for (FreeBlock& b : doomed) {
        cudaFree(b.ptr);                      // waits for the device, so pending uses are over
        std::lock_guard<std::mutex> lock(mutex_);
        spare_events_.push_back(b.ready);
    }
}

void* device_malloc(size_t nbytes) { return MemoryPool::instance().allocate(nbytes); }
void* device_malloc(size_t nbytes, cudaStream_t stream) { return MemoryPool::instance().allocate(nbytes, stream); }

void device_free(void* ptr, cudaStream_t stream) {
    if (ptr == nullptr) return;
    MemoryPool* owner = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_owner_mu);
        auto it = g_owner.find(ptr);
        if (it != g_owner.end()) owner = it->second;
    }
    if (owner != nullptr) owner->deallocate(ptr, stream);
}
void device_free(void* ptr) { device_free(ptr, nullptr); }

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
Stream::Stream() : stream_(create_tracked_stream()) {}
Stream::~Stream() { destroy_tracked_stream(stream_); }
Stream::Stream(Stream&& other) noexcept : stream_(other.stream_) { other.stream_ = nullptr; }
Stream& Stream::operator=(Stream&& other) noexcept {
    if (this != &other) {
        destroy_tracked_stream(stream_);
        stream_ = other.stream_;
        other.stream_ = nullptr;
    }
    return *this;
}
void Stream::synchronize() const { CB200_CUDA(cudaStreamSynchronize(stream_)); }
cudaStream_t Stream::release() noexcept {
    cudaStream_t s = stream_;
    stream_ = nullptr;
    return s;
}
void Stream::destroy_handle(cudaStream_t stream) noexcept { destroy_tracked_stream(stream); }

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
