// cudeep::dist::ShardedGemm - C[M,N] = A[M,K] * B[K,N] (float32 storage, TF32 multiply, FP32
// accumulate) with A and C split by rows over the GPUs of one node and B replicated.
//
// The reference has no counterpart: it is single-device (its capability queries hard-code device 0,
// src/kernels/matmul_kernel.cu:1745, and its lazy kernel set-up is per process, :1769-1783).  This is
// the multi-GPU form of its launch_matmul_kernel<float> (include/cudeep/kernels/matmul.cuh:8-12);
// the product each rank computes is exactly that launcher's.
//
// Rows are independent, so computing needs no exchange.  The only communication is the optional
// all-gather of C for callers that need the whole product on every GPU, offered in these forms:
//
//   Gather::AfterGemm   the GEMM, then one in-place ncclAllGather on the same stream (the baseline);
//   Gather::Banded      the shard is cut into row bands; the NCCL transfer of band i runs on a second
//                       stream behind an event recorded after band i's GEMM, so it overlaps the GEMM of
//                       band i+1 (the GEMM leaves `comm_sms` SMs to NCCL's kernels);
//   Gather::CopyEngine  row bands again, but band i travels as one device-to-device copy per peer on the
//                       GPU's copy engines (peer-mapped memory, a stream per peer): no SM is taken from
//                       band i+1's GEMM and the links carry large contiguous blocks;
//   Gather::Multimem    one kernel does both, through the switch: C lives in memory bound to an NVLink
//                       multicast object, and the GEMM's epilogue writes every tile with multimem.st, which
//                       crosses NVLink once and is replicated into every GPU's C by the NVSwitch - the
//                       rank sends its rows once instead of once per peer (objects made with
//                       ShardedGemmOptions::multicast);
//   Gather::PeerStore   one kernel does both: the GEMM's epilogue stores every finished tile into all
//                       GPUs' copies of C through peer-mapped memory (bulk tensor stores; nothing is
//                       ever loaded from a peer), so the transfer overlaps the math tile by tile and no
//                       collective is called.
//
// Two ways to drive it:
//   * one process for all GPUs (`ShardedGemm(devices, ...)`): one host thread and one compute/comm
//     stream pair per device, NCCL communicators from ncclCommInitAll, peer access enabled between
//     all pairs;
//   * one process per GPU (`ShardedGemm(rank, world, device, ...)`): the caller carries the NCCL id
//     and the 64-byte memory handles of C between the processes (any transport will do).
//
// Failure handling is host-side only.  A step has two phases: every rank first completes its host-side
// preparation; only when all of them have succeeded is anything that waits on another GPU enqueued.
// A rank that fails therefore never leaves a collective in flight on the others; the step throws
// PeerFailure naming the rank, and the object refuses further steps.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace cudeep {
namespace dist {

enum class Gather : int {
    None = 0,            // C stays sharded: every GPU holds only the rows it computed
    AfterGemm = 1,
    Banded = 2,
    PeerStore = 3,
    CollectiveOnly = 4,  // only the all-gather of whatever C holds (to time the collective by itself)
    CopyEngine = 5,
    CopyOnly = 6,        // only the copy-engine pushes of whatever C holds (to time them by themselves)
    Multimem = 7,
};

struct RowRange {
    int64_t row0 = 0;
    int64_t rows = 0;
};

// A rank's host-side preparation failed (or was made to fail by inject_failure); raised on the
// thread that called run() before anything was enqueued on any GPU for that step.
class PeerFailure : public std::runtime_error {
public:
    using std::runtime_error::runtime_error;
};

struct ShardedGemmOptions {
    int bands = 4;         // row bands per shard in Gather::Banded
    int comm_sms = 20;     // SMs the banded GEMM leaves to the collective's kernels
    bool dry_run = false;  // host logic only: no CUDA or NCCL call is made (plan and failure-path tests)
    // C is allocated through the virtual-memory API and bound to an NVLink multicast object, which
    // Gather::Multimem writes through (needs GPUs behind one NVSwitch and at least two of them).  Such
    // an object offers None, AfterGemm, Banded and Multimem; the peer-mapped forms need the default.
    // Every rank must be idle (a barrier after the last step) before any rank destroys its object.
    bool multicast = false;
};

class ShardedGemm {
public:
    static constexpr int kIdBytes = 128;        // an NCCL unique id
    static constexpr int kHandleBytes = 64;     // a CUDA inter-process memory handle

    // One process drives all of `devices`; rank i runs on devices[i].
    ShardedGemm(const std::vector<int>& devices, int64_t m, int n, int k, const ShardedGemmOptions& options = {});
    // This process is rank `rank` of `world` and drives `device`.
    ShardedGemm(int rank, int world, int device, int64_t m, int n, int k, const ShardedGemmOptions& options = {});
    ~ShardedGemm();
    ShardedGemm(const ShardedGemm&) = delete;
    ShardedGemm& operator=(const ShardedGemm&) = delete;

    int world() const;
    int local_ranks() const;                    // ranks this object drives (world, or 1)
    int rank_of(int local) const;
    // Rows of A and C owned by `rank`: shares differ by at most 128 rows, later ranks get the shorter ones.
    RowRange rows_of(int rank) const;
    // Band `band` (0 <= band < bands) of that share, relative to the whole matrix.
    RowRange band_of(int rank, int band) const;

    // Device buffers of local rank `local`, allocated by the constructor: this rank's rows of A
    // [rows, K], the replica of B [K, N] and the whole C [M, N] (the rank's own rows lie at row0).
    float* a_shard(int local) const;
    float* b(int local) const;
    float* c(int local) const;
    void set_a(int local, const float* host_rows);      // blocking copies from host memory
    void set_b(const float* host_b);                    // into every local replica
    // Rows [row0, row0 + rows) of local rank `local`'s copy of C into host memory (blocking).
    void read_c(int local, int64_t row0, int64_t rows, float* host_dst) const;

    // One-process-per-GPU plumbing.  new_comm_id: rank 0 makes the id and ships it to the others;
    // init_comm: all ranks, collectively.  export_c / open_peers: every rank publishes the handle of
    // its C and opens the others' (`handles` = world handles in rank order; the own slot is ignored).
    static void new_comm_id(void* id_out);
    void init_comm(const void* id);
    void export_c(void* handle_out) const;
    void open_peers(const void* handles);

    // The same for an object made with the multicast option: rank 0 makes the multicast object and
    // gets a file descriptor for it, which the caller hands to the other processes (SCM_RIGHTS over a
    // unix socket, or pidfd_getfd) and closes; every rank joins (rank 0 passes -1); after a barrier
    // between the processes - every device must have joined - every rank binds its C.
    int multicast_create_fd();
    void multicast_join(int fd);
    void multicast_bind();

    // Enqueues one step on every local rank and returns without waiting.  With one process for all
    // GPUs the work goes on the object's own streams; with one process per GPU on `stream` (nullptr:
    // the object's compute stream), and the collective's stream is joined back into it, so events
    // recorded on `stream` around run() bracket the whole step.
    void run(Gather gather, cudaStream_t stream = nullptr);
    void synchronize();
    // Mean milliseconds per step over `steps` steps after `warmup`, device-timed on every local rank
    // between host barriers; the slowest rank's figure.
    float time_steps(Gather gather, int steps, int warmup);

    // Steps enqueued so far on local rank `local` (a step abandoned in its first phase counts nowhere).
    int64_t steps_enqueued(int local) const;
    // Test hook: the named rank's host-side preparation fails at the next step.
    void inject_failure(int rank);

private:
    struct Impl;
    std::unique_ptr<Impl> impl_;
};

}  // namespace dist
}  // namespace cudeep
