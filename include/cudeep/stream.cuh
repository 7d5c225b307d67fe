// RAII stream and event wrappers; public surface of the reference's
// include/cudeep/stream.cuh:8-44 (Stream: get/synchronize, Event:
// record/synchronize/elapsed_ms).  Streams here are created non-blocking so
// work on them overlaps the legacy default stream.  A Stream is drained before it is
// destroyed, and the memory pool knows which of these streams are gone, so tensors may
// outlive the stream they worked on.
#pragma once

#include "common.cuh"
#include "error.cuh"

#include <cuda_runtime.h>

namespace cudeep {

class Stream {
public:
    Stream();
    ~Stream();
    Stream(const Stream&) = delete;
    Stream& operator=(const Stream&) = delete;
    Stream(Stream&& other) noexcept;
    Stream& operator=(Stream&& other) noexcept;

    cudaStream_t get() const { return stream_; }
    void synchronize() const;
    // Additions for callers that hold raw handles (the C ABI): give up ownership of the handle /
    // drain and destroy a handle obtained that way.
    cudaStream_t release() noexcept;
    static void destroy_handle(cudaStream_t stream) noexcept;

private:
    cudaStream_t stream_ = nullptr;
};

class Event {
public:
    Event();
    ~Event();
    Event(const Event&) = delete;
    Event& operator=(const Event&) = delete;
    Event(Event&& other) noexcept;
    Event& operator=(Event&& other) noexcept;

    void record(cudaStream_t stream = nullptr);
    void synchronize() const;
    // Milliseconds between `start` and this event (both must have completed).
    float elapsed_ms(const Event& start) const;
    cudaEvent_t get() const { return event_; }

private:
    cudaEvent_t event_ = nullptr;
};

}  // namespace cudeep
