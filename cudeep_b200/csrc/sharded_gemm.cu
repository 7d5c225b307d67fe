// cudeep::dist::ShardedGemm (see include/cudeep/dist/sharded_gemm.cuh).
//
// NCCL is bound at run time (dlopen of libnccl.so.2, or of the path in CUDEEP_B200_NCCL_LIB) so that
// the library itself does not depend on it: single-GPU users never load it, and a process that
// already holds an NCCL (a framework's) shares that copy.
#include "cudeep/dist/sharded_gemm.cuh"

#include "cudeep/kernels/matmul.cuh"
#include "gemm_tf32.h"
#include "multicast.h"
#include "runtime.h"

#include <dlfcn.h>

#include <atomic>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <mutex>
#include <thread>

namespace cudeep {
namespace dist {

namespace {

// ---------------------------------------------------------------- NCCL, bound by name

struct NcclId { char bytes[ShardedGemm::kIdBytes]; };
using NcclComm = void*;
constexpr int kNcclFloat32 = 7;     // ncclFloat32 in nccl.h's ncclDataType_t

struct NcclApi {
    int (*GetUniqueId)(NcclId*) = nullptr;
    int (*CommInitRank)(NcclComm*, int, NcclId, int) = nullptr;
    int (*CommInitAll)(NcclComm*, int, const int*) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, NcclComm, cudaStream_t) = nullptr;
    int (*Broadcast)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    int (*CommDestroy)(NcclComm) = nullptr;
    int (*CommAbort)(NcclComm) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
};

const NcclApi& nccl() {
    static NcclApi api;
    static std::once_flag once;
    static std::string failure;
    std::call_once(once, [] {
        const char* named = std::getenv("CUDEEP_B200_NCCL_LIB");
        void* lib = nullptr;
        if (named != nullptr && named[0] != '\0') lib = dlopen(named, RTLD_NOW | RTLD_GLOBAL);
        if (lib == nullptr) lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (lib == nullptr) {
            failure = std::string("cannot load NCCL (libnccl.so.2; set CUDEEP_B200_NCCL_LIB): ") + dlerror();
            return;
        }
        auto bind = [&](auto& slot, const char* name) {
            slot = reinterpret_cast<std::remove_reference_t<decltype(slot)>>(dlsym(lib, name));
            if (slot == nullptr && failure.empty()) failure = std::string("NCCL lacks symbol ") + name;
        };
        bind(api.GetUniqueId, "ncclGetUniqueId");
        bind(api.CommInitRank, "ncclCommInitRank");
        bind(api.CommInitAll, "ncclCommInitAll");
        bind(api.AllGather, "ncclAllGather");
        bind(api.Broadcast, "ncclBroadcast");
        bind(api.GroupStart, "ncclGroupStart");
        bind(api.GroupEnd, "ncclGroupEnd");
        bind(api.CommDestroy, "ncclCommDestroy");
        bind(api.CommAbort, "ncclCommAbort");
        bind(api.GetErrorString, "ncclGetErrorString");
    });
    if (!failure.empty()) throw std::runtime_error(failure);
    return api;
}

void nccl_ok(int status, const char* what) {
    if (status != 0)
        throw std::runtime_error(std::string("NCCL ") + what + ": " + nccl().GetErrorString(status));
}

// ---------------------------------------------------------------- one host thread per device

// Runs closures one at a time on a thread of its own; wait() rethrows what the closure threw.
class Worker {
public:
    Worker() : thread_([this] { loop(); }) {}
    ~Worker() {
        {
            std::lock_guard<std::mutex> lock(mu_);
            stop_ = true;
        }
        cv_.notify_all();
        thread_.join();
    }
    void post(std::function<void()> task) {
        std::lock_guard<std::mutex> lock(mu_);
        task_ = std::move(task);
        pending_ = true;
        error_ = nullptr;
        cv_.notify_all();
    }
    void wait() {
        std::unique_lock<std::mutex> lock(mu_);
        cv_.wait(lock, [this] { return !pending_; });
        if (error_) std::rethrow_exception(error_);
    }

private:
    void loop() {
        std::unique_lock<std::mutex> lock(mu_);
        for (;;) {
            cv_.wait(lock, [this] { return pending_ || stop_; });
            if (stop_) return;
            std::function<void()> task = std::move(task_);
            lock.unlock();
            std::exception_ptr err;
            try {
                task();
            } catch (...) {
                err = std::current_exception();
            }
            lock.lock();
            error_ = err;
            pending_ = false;
            cv_.notify_all();
        }
    }
    std::mutex mu_;
    std::condition_variable cv_;
    std::function<void()> task_;
    bool pending_ = false;
    bool stop_ = false;
    std::exception_ptr error_;
    std::thread thread_;      // last: the members above exist before the thread starts
};

struct RankState {
    int rank = 0;
    int device = 0;
    float* a = nullptr;
    float* b = nullptr;
    float* c = nullptr;
    cudaStream_t compute = nullptr;
    cudaStream_t comm = nullptr;
    std::vector<cudaEvent_t> band_done;
    cudaEvent_t comm_done = nullptr;
    std::vector<cudaStream_t> copy_streams;    // Gather::CopyEngine: one per peer, made on first use
    std::vector<cudaEvent_t> copy_done;
    cudaEvent_t t0 = nullptr, t1 = nullptr;
    NcclComm nccl_comm = nullptr;
    std::vector<float*> peer_c;        // every rank's C as seen from this device (own slot: c)
    std::vector<void*> opened;         // inter-process mappings to close
    int num_sms = 0;
    int64_t steps_enqueued = 0;
    cudeep_b200::MulticastShare share;  // C when the object was made with the multicast option
};

}  // namespace

struct ShardedGemm::Impl {
    int world = 1;
    bool in_process = true;
    int64_t m = 0;
    int n = 0, k = 0;
    ShardedGemmOptions opt;
    std::vector<RankState> ranks;                      // local ranks
    std::vector<std::unique_ptr<Worker>> workers;      // one per local rank (in-process mode)
    bool comm_ready = false;
    bool peers_ready = false;
    cudeep_b200::MulticastGroup group;                 // multicast option: the object all ranks' C is bound to
    bool group_bound = false;
    bool broken = false;
    std::atomic<int> fail_rank{-1};

    RankState& at(int local) {
        CB200_REQUIRE(local >= 0 && local < int(ranks.size()), "local rank index out of range");
        return ranks[size_t(local)];
    }

    RowRange rows_of(int rank) const {
        const int64_t units = (m + 127) / 128;
        const int64_t base = units / world, extra = units % world;
        int64_t row0 = 0;
        RowRange out;
        for (int r = 0; r <= rank; ++r) {
            int64_t rows = (base + (r < extra ? 1 : 0)) * 128;
            if (rows > m - row0) rows = m - row0;
            if (rows < 0) rows = 0;
            out.row0 = row0;
            out.rows = rows;
            row0 += rows;
        }
        return out;
    }
    RowRange band_of(int rank, int band) const {
        const RowRange own = rows_of(rank);
        const int64_t units = (own.rows + 255) / 256;
        const int64_t per = (units + opt.bands - 1) / opt.bands * 256;
        RowRange out;
        out.row0 = own.row0 + (per * band < own.rows ? per * band : own.rows);
        const int64_t end = per * (band + 1) < own.rows ? per * (band + 1) : own.rows;
        out.rows = own.row0 + end - out.row0;
        return out;
    }
    bool equal_shares() const {
        for (int r = 1; r < world; ++r)
            if (rows_of(r).rows != rows_of(0).rows) return false;
        return true;
    }

    template <class F>
    void for_each_rank(F fn) {
        if (!in_process || workers.empty()) {
            for (size_t i = 0; i < ranks.size(); ++i) fn(ranks[i]);
            return;
        }
        for (size_t i = 0; i < ranks.size(); ++i) workers[i]->post([this, i, fn] { fn(ranks[i]); });
        std::exception_ptr first;
        for (auto& w : workers) {
            try {
                w->wait();
            } catch (...) {
                if (!first) first = std::current_exception();
            }
        }
        if (first) std::rethrow_exception(first);
    }

    void gemm(RankState& r, const float* a, float* c, int64_t rows, int max_ctas, cudaStream_t s) const {
        if (rows <= 0) return;
        if (max_ctas > 0 && cudeep_b200::gemm_tf32_supported(a, r.b, c, int(rows), n, k, false) && rows >= 64 &&
            n >= 64 && k >= 32) {
            cudeep_b200::GemmTuning tune;
            tune.max_ctas = max_ctas;
            cudeep_b200::gemm_tf32(a, r.b, false, c, int(rows), n, k, nullptr, false, 0, tune, s);
        } else {
            kernels::launch_matmul_kernel<float>(a, r.b, c, int(rows), n, k, s);
        }
    }

    // All ranks' rows of C, in place, on stream `s` (every rank calls this with the same arguments).
    void all_gather(RankState& r, int band, cudaStream_t s) const {
        const NcclApi& api = nccl();
        if (band < 0 && equal_shares()) {
            const RowRange own = rows_of(r.rank);
            nccl_ok(api.AllGather(r.c + own.row0 * n, r.c, size_t(own.rows) * n, kNcclFloat32, r.nccl_comm, s),
                    "ncclAllGather");
            return;
        }
        nccl_ok(api.GroupStart(), "ncclGroupStart");
        for (int root = 0; root < world; ++root) {
            const RowRange part = band < 0 ? rows_of(root) : band_of(root, band);
            if (part.rows <= 0) continue;
            float* at = r.c + part.row0 * n;
            nccl_ok(api.Broadcast(at, at, size_t(part.rows) * n, kNcclFloat32, root, r.nccl_comm, s), "ncclBroadcast");
        }
        nccl_ok(api.GroupEnd(), "ncclGroupEnd");
    }

    void enqueue(RankState& r, Gather gather, cudaStream_t s) {
        ++r.steps_enqueued;
        if (opt.dry_run) return;
        const RowRange own = rows_of(r.rank);
        float* c_own = r.c + own.row0 * n;
        switch (gather) {
        case Gather::None:
            gemm(r, r.a, c_own, own.rows, 0, s);
            break;
        case Gather::AfterGemm:
            gemm(r, r.a, c_own, own.rows, 0, s);
            all_gather(r, -1, s);
            break;
        case Gather::CollectiveOnly:
            all_gather(r, -1, s);
            break;
        case Gather::Banded: {
            const int gemm_ctas = r.num_sms - opt.comm_sms > 2 ? r.num_sms - opt.comm_sms : 2;
            for (int band = 0; band < opt.bands; ++band) {
                const RowRange part = band_of(r.rank, band);
                gemm(r, r.a + (part.row0 - own.row0) * k, r.c + part.row0 * n, part.rows, gemm_ctas, s);
                CB200_CUDA(cudaEventRecord(r.band_done[band], s));
                CB200_CUDA(cudaStreamWaitEvent(r.comm, r.band_done[band], 0));
                all_gather(r, band, r.comm);
            }
            // The step ends on `s` when its last transfer has: the next step's GEMM must not
            // overwrite rows a transfer still reads.
            CB200_CUDA(cudaEventRecord(r.comm_done, r.comm));
            CB200_CUDA(cudaStreamWaitEvent(s, r.comm_done, 0));
            break;
        }
        case Gather::CopyOnly:
        case Gather::CopyEngine: {
            // Band by band: the GEMM of a band, then one device-to-device copy of that band into every
            // peer's C, each on a stream of its own.  The copies run on the copy engines, so they take
            // no SM from the next band's GEMM, and they move large contiguous blocks at link rate.
            if (r.copy_streams.empty()) {
                r.copy_streams.resize(size_t(world));
                r.copy_done.resize(size_t(world));
                for (int p = 0; p < world; ++p) {
                    if (p == r.rank) continue;
                    CB200_CUDA(cudaStreamCreateWithFlags(&r.copy_streams[size_t(p)], cudaStreamNonBlocking));
                    CB200_CUDA(cudaEventCreateWithFlags(&r.copy_done[size_t(p)], cudaEventDisableTiming));
                }
            }
            for (int band = 0; band < opt.bands; ++band) {
                const RowRange part = band_of(r.rank, band);
                if (part.rows <= 0) continue;
                if (gather == Gather::CopyEngine)
                    gemm(r, r.a + (part.row0 - own.row0) * k, r.c + part.row0 * n, part.rows, 0, s);
                CB200_CUDA(cudaEventRecord(r.band_done[band], s));
                for (int p = 0; p < world; ++p) {
                    if (p == r.rank) continue;
                    cudaStream_t cs = r.copy_streams[size_t(p)];
                    CB200_CUDA(cudaStreamWaitEvent(cs, r.band_done[band], 0));
                    CB200_CUDA(cudaMemcpyAsync(r.peer_c[size_t(p)] + part.row0 * n, r.c + part.row0 * n,
                                               size_t(part.rows) * n * sizeof(float), cudaMemcpyDeviceToDevice, cs));
                }
            }
            for (int p = 0; p < world; ++p) {
                if (p == r.rank) continue;
                CB200_CUDA(cudaEventRecord(r.copy_done[size_t(p)], r.copy_streams[size_t(p)]));
                CB200_CUDA(cudaStreamWaitEvent(s, r.copy_done[size_t(p)], 0));
            }
            break;
        }
        case Gather::Multimem: {
            if (own.rows > 0) {
                float* through_switch = static_cast<float*>(r.share.group) + own.row0 * n;
                cudeep_b200::GemmTuning tune;
                cudeep_b200::gemm_tf32_multimem(r.a, r.b, false, c_own, through_switch, int(own.rows), n, k, tune, s);
            }
            break;
        }
        case Gather::PeerStore: {
            cudeep_b200::GemmPeerOutputs peers;
            for (int p = 0; p < world; ++p) {
                if (p == r.rank) continue;
                peers.c[peers.count++] = r.peer_c[p] + own.row0 * n;
            }
            if (own.rows > 0) {
                cudeep_b200::GemmTuning tune;
                cudeep_b200::gemm_tf32_push(r.a, r.b, false, c_own, int(own.rows), n, k, peers, tune, s);
            }
            break;
        }
        }
    }

    void ensure_comm() {
        if (comm_ready || opt.dry_run) return;
        CB200_REQUIRE(in_process, "init_comm() must be called before a step that uses NCCL");
        std::vector<NcclComm> comms(ranks.size());
        std::vector<int> devices;
        for (const RankState& r : ranks) devices.push_back(r.device);
        nccl_ok(nccl().CommInitAll(comms.data(), int(ranks.size()), devices.data()), "ncclCommInitAll");
        for (size_t i = 0; i < ranks.size(); ++i) ranks[i].nccl_comm = comms[i];
        comm_ready = true;
    }

    void ensure_peers() {
        if (peers_ready || opt.dry_run) return;
        CB200_REQUIRE(in_process, "open_peers() must be called before a step with Gather::PeerStore");
        CB200_REQUIRE(world - 1 <= cudeep_b200::kMaxGemmPeers, "Gather::PeerStore supports at most 8 ranks");
        int prev = 0;
        CB200_CUDA(cudaGetDevice(&prev));
        struct Restore {
            int device;
            ~Restore() { cudaSetDevice(device); }
        } restore{prev};
        for (RankState& r : ranks) {
            CB200_CUDA(cudaSetDevice(r.device));
            r.peer_c.assign(size_t(world), nullptr);
            for (const RankState& p : ranks) {
                r.peer_c[size_t(p.rank)] = p.c;
                if (p.device == r.device) continue;
                int can = 0;
                CB200_CUDA(cudaDeviceCanAccessPeer(&can, r.device, p.device));
                CB200_REQUIRE(can != 0, "Gather::PeerStore needs peer access between all GPUs of the job");
                const cudaError_t err = cudaDeviceEnablePeerAccess(p.device, 0);
                if (err == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
                else CB200_CUDA(err);
            }
        }
        peers_ready = true;
    }

    void check_mode(Gather gather) {
        CB200_REQUIRE(!broken, "this ShardedGemm had a failed step; make a new one");
        const int g = int(gather);
        CB200_REQUIRE(g >= 0 && g <= 7, "unknown gather mode");
        const bool peer_mapped = gather == Gather::PeerStore || gather == Gather::CopyEngine || gather == Gather::CopyOnly;
        CB200_REQUIRE(!(peer_mapped && opt.multicast && !opt.dry_run),
                      "an object made with the multicast option holds C in virtual-memory allocations, which the "
                      "peer-mapped gather forms do not reach; use Gather::Multimem");
        if (gather == Gather::Multimem)
            CB200_REQUIRE(opt.dry_run || (opt.multicast && group_bound && n % 4 == 0),
                          "Gather::Multimem needs an object made with the multicast option, bound (multicast_bind), and "
                          "N % 4 == 0");
        if (gather == Gather::AfterGemm || gather == Gather::Banded || gather == Gather::CollectiveOnly) ensure_comm();
        if (gather == Gather::CopyEngine || gather == Gather::CopyOnly) ensure_peers();
        if (gather == Gather::PeerStore) {
            ensure_peers();
            CB200_REQUIRE(opt.dry_run || n % 4 == 0, "Gather::PeerStore needs N % 4 == 0");
        }
    }

    // Phase one of a step: host-side preparation of every local rank; nothing is enqueued.
    void prepare_all() {
        std::vector<std::string> failures(ranks.size());
        for_each_rank([&](RankState& r) {
            const size_t slot = size_t(&r - ranks.data());
            try {
                if (fail_rank.load() == r.rank) throw std::runtime_error("failure injected on the host");
                if (!opt.dry_run) {
                    CB200_CUDA(cudaSetDevice(r.device));
                    CB200_REQUIRE(r.a != nullptr && r.b != nullptr && r.c != nullptr, "device buffers are missing");
                }
            } catch (const std::exception& e) {
                failures[slot] = e.what();
            }
        });
        std::string report;
        for (size_t i = 0; i < failures.size(); ++i)
            if (!failures[i].empty())
                report += (report.empty() ? "" : "; ") + ("rank " + std::to_string(ranks[i].rank) + ": " + failures[i]);
        if (!report.empty()) {
            broken = true;
            throw PeerFailure("step abandoned before anything was enqueued: " + report);
        }
    }
};

// ---------------------------------------------------------------- construction

namespace {
void allocate_rank(RankState& r, int64_t rows, int64_t m, int n, int k, int bands, int world, bool multicast) {
    CB200_CUDA(cudaSetDevice(r.device));
    cudaDeviceProp prop{};
    CB200_CUDA(cudaGetDeviceProperties(&prop, r.device));
    r.num_sms = prop.multiProcessorCount;
    CB200_CUDA(cudaMalloc(&r.a, size_t(rows > 0 ? rows : 1) * k * sizeof(float)));
    CB200_CUDA(cudaMalloc(&r.b, size_t(k) * n * sizeof(float)));
    if (multicast) {
        // C comes from the virtual-memory API so that it can be bound into a multicast object.
        CB200_REQUIRE(cudeep_b200::multicast_supported(), "this GPU cannot take part in a multicast object");
        cudeep_b200::multicast_allocate(r.share, r.device,
                                        cudeep_b200::multicast_round_size(world, size_t(m) * n * sizeof(float)));
        r.c = static_cast<float*>(r.share.local);
    } else {
        CB200_CUDA(cudaMalloc(&r.c, size_t(m) * n * sizeof(float)));
    }
    int least = 0, greatest = 0;
    CB200_CUDA(cudaDeviceGetStreamPriorityRange(&least, &greatest));
    CB200_CUDA(cudaStreamCreateWithFlags(&r.compute, cudaStreamNonBlocking));
    // The collective's kernels are few and short-lived next to the GEMM's persistent CTAs: give
    // them the first free SM.
    CB200_CUDA(cudaStreamCreateWithPriority(&r.comm, cudaStreamNonBlocking, greatest));
    r.band_done.resize(size_t(bands));
    for (cudaEvent_t& e : r.band_done) CB200_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    CB200_CUDA(cudaEventCreateWithFlags(&r.comm_done, cudaEventDisableTiming));
    CB200_CUDA(cudaEventCreate(&r.t0));
    CB200_CUDA(cudaEventCreate(&r.t1));
}

void check_extents(int world, int64_t m, int n, int k, const ShardedGemmOptions& opt) {
    CB200_REQUIRE(world >= 1 && world <= 64, "world size must be between 1 and 64");
    CB200_REQUIRE(m > 0 && n > 0 && k > 0, "ShardedGemm: extents must be positive");
    CB200_REQUIRE(m <= (int64_t(1) << 31) - 1, "ShardedGemm: M must fit 32 bits");
    CB200_REQUIRE(opt.bands >= 1 && opt.bands <= 64, "ShardedGemm: bands must be between 1 and 64");
    CB200_REQUIRE(opt.comm_sms >= 0, "ShardedGemm: comm_sms must not be negative");
}
}  // namespace

ShardedGemm::ShardedGemm(const std::vector<int>& devices, int64_t m, int n, int k, const ShardedGemmOptions& options)
    : impl_(new Impl) {
    check_extents(int(devices.size()), m, n, k, options);
    Impl& s = *impl_;
    s.world = int(devices.size());
    s.in_process = true;
    s.m = m; s.n = n; s.k = k;
    s.opt = options;
    s.ranks.resize(devices.size());
    for (size_t i = 0; i < devices.size(); ++i) {
        s.ranks[i].rank = int(i);
        s.ranks[i].device = devices[i];
    }
    if (!options.dry_run) {
        int prev = 0;
        CB200_CUDA(cudaGetDevice(&prev));
        for (RankState& r : s.ranks)
            allocate_rank(r, s.rows_of(r.rank).rows, m, n, k, options.bands, s.world, options.multicast);
        if (options.multicast) {
            // One process: make the object, add every device, then bind every share.
            CB200_REQUIRE(s.world >= 2, "the multicast option needs at least two GPUs");
            s.group = cudeep_b200::multicast_create(s.world, s.ranks[0].share.size);
            for (RankState& r : s.ranks) cudeep_b200::multicast_add_device(s.group, r.device);
            for (RankState& r : s.ranks) {
                CB200_CUDA(cudaSetDevice(r.device));
                cudeep_b200::multicast_bind(s.group, r.share);
            }
            s.group_bound = true;
        }
        CB200_CUDA(cudaSetDevice(prev));
    }
    for (size_t i = 0; i < devices.size(); ++i) s.workers.emplace_back(new Worker);
    if (!options.dry_run)
        s.for_each_rank([](RankState& r) { CB200_CUDA(cudaSetDevice(r.device)); });     // each worker keeps its device
}

ShardedGemm::ShardedGemm(int rank, int world, int device, int64_t m, int n, int k, const ShardedGemmOptions& options)
    : impl_(new Impl) {
    check_extents(world, m, n, k, options);
    CB200_REQUIRE(rank >= 0 && rank < world, "ShardedGemm: rank out of range");
    Impl& s = *impl_;
    s.world = world;
    s.in_process = false;
    s.m = m; s.n = n; s.k = k;
    s.opt = options;
    s.ranks.resize(1);
    s.ranks[0].rank = rank;
    s.ranks[0].device = device;
    if (!options.dry_run)
        allocate_rank(s.ranks[0], s.rows_of(rank).rows, m, n, k, options.bands, world, options.multicast);
}

ShardedGemm::~ShardedGemm() {
    Impl& s = *impl_;
    s.workers.clear();                       // joins the threads
    if (s.opt.dry_run) return;
    int prev = 0;
    cudaGetDevice(&prev);
    for (RankState& r : s.ranks) {
        cudaSetDevice(r.device);
        cudaDeviceSynchronize();
    }
    for (RankState& r : s.ranks) {
        cudaSetDevice(r.device);
        if (r.nccl_comm != nullptr) {
            try {
                nccl().CommDestroy(r.nccl_comm);
            } catch (...) {
            }
        }
        for (void* p : r.opened) cudaIpcCloseMemHandle(p);
        for (cudaEvent_t e : r.band_done) cudaEventDestroy(e);
        for (cudaEvent_t e : r.copy_done) if (e) cudaEventDestroy(e);
        for (cudaStream_t cs : r.copy_streams) if (cs) cudaStreamDestroy(cs);
        if (r.comm_done) cudaEventDestroy(r.comm_done);
        if (r.t0) cudaEventDestroy(r.t0);
        if (r.t1) cudaEventDestroy(r.t1);
        if (r.compute) cudaStreamDestroy(r.compute);
        if (r.comm) cudaStreamDestroy(r.comm);
        cudaFree(r.a);
        cudaFree(r.b);
        if (r.share.memory != 0) cudeep_b200::multicast_release(s.group, r.share);
        else cudaFree(r.c);
    }
    cudeep_b200::multicast_destroy(s.group);
    cudaSetDevice(prev);
    cudaGetLastError();
}

// ---------------------------------------------------------------- queries and buffers

int ShardedGemm::world() const { return impl_->world; }
int ShardedGemm::local_ranks() const { return int(impl_->ranks.size()); }
int ShardedGemm::rank_of(int local) const { return impl_->at(local).rank; }
int64_t ShardedGemm::steps_enqueued(int local) const { return impl_->at(local).steps_enqueued; }
RowRange ShardedGemm::rows_of(int rank) const {
    CB200_REQUIRE(rank >= 0 && rank < impl_->world, "rank out of range");
    return impl_->rows_of(rank);
}
RowRange ShardedGemm::band_of(int rank, int band) const {
    CB200_REQUIRE(rank >= 0 && rank < impl_->world, "rank out of range");
    CB200_REQUIRE(band >= 0 && band < impl_->opt.bands, "band out of range");
    return impl_->band_of(rank, band);
}
float* ShardedGemm::a_shard(int local) const { return impl_->at(local).a; }
float* ShardedGemm::b(int local) const { return impl_->at(local).b; }
float* ShardedGemm::c(int local) const { return impl_->at(local).c; }

void ShardedGemm::set_a(int local, const float* host_rows) {
    CB200_REQUIRE(host_rows != nullptr && !impl_->opt.dry_run, "set_a: null pointer or dry run");
    RankState& r = impl_->at(local);
    int prev = 0;
    CB200_CUDA(cudaGetDevice(&prev));
    CB200_CUDA(cudaSetDevice(r.device));
    CB200_CUDA(cudaMemcpy(r.a, host_rows, size_t(impl_->rows_of(r.rank).rows) * impl_->k * sizeof(float),
                          cudaMemcpyHostToDevice));
    CB200_CUDA(cudaSetDevice(prev));
}

void ShardedGemm::read_c(int local, int64_t row0, int64_t rows, float* host_dst) const {
    CB200_REQUIRE(host_dst != nullptr && !impl_->opt.dry_run, "read_c: null pointer or dry run");
    CB200_REQUIRE(row0 >= 0 && rows >= 0 && row0 + rows <= impl_->m, "read_c: rows out of range");
    const RankState& r = impl_->at(local);
    if (rows == 0) return;
    int prev = 0;
    CB200_CUDA(cudaGetDevice(&prev));
    CB200_CUDA(cudaSetDevice(r.device));         // memory from the virtual-memory API is reachable from its own device only
    const cudaError_t err = cudaMemcpy(host_dst, r.c + row0 * impl_->n, size_t(rows) * impl_->n * sizeof(float),
                                       cudaMemcpyDeviceToHost);
    cudaSetDevice(prev);
    CB200_CUDA(err);
}

void ShardedGemm::set_b(const float* host_b) {
    CB200_REQUIRE(host_b != nullptr && !impl_->opt.dry_run, "set_b: null pointer or dry run");
    int prev = 0;
    CB200_CUDA(cudaGetDevice(&prev));
    for (RankState& r : impl_->ranks) {
        CB200_CUDA(cudaSetDevice(r.device));
        CB200_CUDA(cudaMemcpy(r.b, host_b, size_t(impl_->k) * impl_->n * sizeof(float), cudaMemcpyHostToDevice));
    }
    CB200_CUDA(cudaSetDevice(prev));
}

// ---------------------------------------------------------------- one process per GPU

void ShardedGemm::new_comm_id(void* id_out) {
    CB200_REQUIRE(id_out != nullptr, "new_comm_id: null pointer");
    NcclId id{};
    nccl_ok(nccl().GetUniqueId(&id), "ncclGetUniqueId");
    std::memcpy(id_out, id.bytes, kIdBytes);
}

void ShardedGemm::init_comm(const void* id_bytes) {
    Impl& s = *impl_;
    CB200_REQUIRE(!s.in_process, "init_comm is for the one-process-per-GPU form");
    CB200_REQUIRE(id_bytes != nullptr && !s.comm_ready && !s.opt.dry_run, "init_comm: null id, repeated call or dry run");
    NcclId id{};
    std::memcpy(id.bytes, id_bytes, kIdBytes);
    RankState& r = s.ranks[0];
    CB200_CUDA(cudaSetDevice(r.device));
    nccl_ok(nccl().CommInitRank(&r.nccl_comm, s.world, id, r.rank), "ncclCommInitRank");
    s.comm_ready = true;
}

void ShardedGemm::export_c(void* handle_out) const {
    const Impl& s = *impl_;
    CB200_REQUIRE(!s.in_process && handle_out != nullptr && !s.opt.dry_run, "export_c: one-process-per-GPU form only");
    CB200_REQUIRE(!s.opt.multicast, "export_c: an object made with the multicast option shares C through multicast_join");
    static_assert(sizeof(cudaIpcMemHandle_t) == kHandleBytes, "unexpected handle size");
    cudaIpcMemHandle_t h{};
    CB200_CUDA(cudaSetDevice(s.ranks[0].device));
    CB200_CUDA(cudaIpcGetMemHandle(&h, s.ranks[0].c));
    std::memcpy(handle_out, &h, kHandleBytes);
}

void ShardedGemm::open_peers(const void* handles) {
    Impl& s = *impl_;
    CB200_REQUIRE(!s.in_process && handles != nullptr && !s.peers_ready && !s.opt.dry_run,
                  "open_peers: one-process-per-GPU form, once");
    CB200_REQUIRE(s.world - 1 <= cudeep_b200::kMaxGemmPeers, "Gather::PeerStore supports at most 8 ranks");
    RankState& r = s.ranks[0];
    CB200_CUDA(cudaSetDevice(r.device));
    r.peer_c.assign(size_t(s.world), nullptr);
    for (int p = 0; p < s.world; ++p) {
        if (p == r.rank) {
            r.peer_c[size_t(p)] = r.c;
            continue;
        }
        cudaIpcMemHandle_t h{};
        std::memcpy(&h, static_cast<const char*>(handles) + size_t(p) * kHandleBytes, kHandleBytes);
        void* mapped = nullptr;
        CB200_CUDA(cudaIpcOpenMemHandle(&mapped, h, cudaIpcMemLazyEnablePeerAccess));
        r.opened.push_back(mapped);
        r.peer_c[size_t(p)] = static_cast<float*>(mapped);
    }
    s.peers_ready = true;
}

int ShardedGemm::multicast_create_fd() {
    Impl& s = *impl_;
    CB200_REQUIRE(!s.in_process && s.opt.multicast && !s.opt.dry_run && s.ranks[0].rank == 0 && s.group.handle == 0,
                  "multicast_create_fd: rank 0 of a one-process-per-GPU object made with the multicast option, once");
    CB200_CUDA(cudaSetDevice(s.ranks[0].device));
    s.group = cudeep_b200::multicast_create(s.world, s.ranks[0].share.size);
    return cudeep_b200::multicast_export_fd(s.group);
}

void ShardedGemm::multicast_join(int fd) {
    Impl& s = *impl_;
    CB200_REQUIRE(!s.in_process && s.opt.multicast && !s.opt.dry_run, "multicast_join: one-process-per-GPU form with the multicast option");
    RankState& r = s.ranks[0];
    CB200_CUDA(cudaSetDevice(r.device));
    if (r.rank != 0) {
        CB200_REQUIRE(fd >= 0 && s.group.handle == 0, "multicast_join: a file descriptor from rank 0, once");
        s.group = cudeep_b200::multicast_import_fd(fd, s.world, r.share.size);
    }
    CB200_REQUIRE(s.group.handle != 0, "multicast_join: rank 0 calls multicast_create_fd first");
    cudeep_b200::multicast_add_device(s.group, r.device);
}

void ShardedGemm::multicast_bind() {
    Impl& s = *impl_;
    CB200_REQUIRE(!s.in_process && s.opt.multicast && !s.opt.dry_run && s.group.handle != 0 && !s.group_bound,
                  "multicast_bind: after multicast_join on every rank, once");
    CB200_CUDA(cudaSetDevice(s.ranks[0].device));
    cudeep_b200::multicast_bind(s.group, s.ranks[0].share);
    s.group_bound = true;
}

// ---------------------------------------------------------------- steps

void ShardedGemm::run(Gather gather, cudaStream_t stream) {
    Impl& s = *impl_;
    s.check_mode(gather);
    s.prepare_all();
    if (s.in_process) {
        s.for_each_rank([&s, gather](RankState& r) { s.enqueue(r, gather, r.compute); });
    } else {
        RankState& r = s.ranks[0];
        if (!s.opt.dry_run) CB200_CUDA(cudaSetDevice(r.device));
        s.enqueue(r, gather, stream != nullptr ? stream : r.compute);
    }
}

void ShardedGemm::synchronize() {
    Impl& s = *impl_;
    if (s.opt.dry_run) return;
    s.for_each_rank([](RankState& r) {
        CB200_CUDA(cudaSetDevice(r.device));
        CB200_CUDA(cudaStreamSynchronize(r.compute));
        CB200_CUDA(cudaStreamSynchronize(r.comm));
        for (cudaStream_t cs : r.copy_streams) if (cs) CB200_CUDA(cudaStreamSynchronize(cs));
    });
}

float ShardedGemm::time_steps(Gather gather, int steps, int warmup) {
    Impl& s = *impl_;
    CB200_REQUIRE(steps > 0 && warmup >= 0, "time_steps: steps must be positive");
    s.check_mode(gather);
    s.prepare_all();
    if (s.opt.dry_run) {
        s.for_each_rank([&](RankState& r) {
            for (int i = 0; i < warmup + steps; ++i) s.enqueue(r, gather, nullptr);
        });
        return 0.0f;
    }
    s.for_each_rank([&](RankState& r) {
        for (int i = 0; i < warmup; ++i) s.enqueue(r, gather, r.compute);
    });
    synchronize();                                   // host barrier: every rank is idle
    s.for_each_rank([&](RankState& r) {
        CB200_CUDA(cudaEventRecord(r.t0, r.compute));
        for (int i = 0; i < steps; ++i) s.enqueue(r, gather, r.compute);
        CB200_CUDA(cudaEventRecord(r.t1, r.compute));
    });
    synchronize();
    float slowest = 0.0f;
    for (RankState& r : s.ranks) {
        float ms = 0.0f;
        CB200_CUDA(cudaSetDevice(r.device));
        CB200_CUDA(cudaEventElapsedTime(&ms, r.t0, r.t1));
        if (ms > slowest) slowest = ms;
    }
    return slowest / float(steps);
}

void ShardedGemm::inject_failure(int rank) { impl_->fail_rank.store(rank); }

}  // namespace dist
}  // namespace cudeep
