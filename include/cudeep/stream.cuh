// RAII stream and event wrappers; public surface of the reference's
// include/cudeep/stream.cuh:8-44 (Stream: get/synchronize, Event:
// record/synchronize/elapsed_ms).  Streams here are created non-blocking so
// work on them overlaps the legacy default stream.
#pragma once

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
