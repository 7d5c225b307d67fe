// cudeep::dist::ShardedGemm as a C++ caller uses it: one process, every visible GPU (a world of one on
// a single-GPU machine), every gather mode checked against a float64 host loop on sampled elements;
// then the failure path - a rank whose host-side preparation fails stops the step before anything is
// enqueued anywhere, as a PeerFailure naming the rank.  Exits 0 and prints ALL PASSED when every check
// holds.  `--dry` runs only the parts that need no GPU.
#include "cudeep/dist/sharded_gemm.cuh"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <vector>

using namespace cudeep::dist;

#define CHECK(cond)                                                              \
    do {                                                                         \
        if (!(cond)) {                                                           \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);        \
            std::exit(1);                                                        \
        }                                                                        \
    } while (0)

static void test_plan_and_failure_path_without_a_gpu() {
    ShardedGemmOptions opt;
    opt.dry_run = true;
    opt.bands = 4;
    ShardedGemm g({0, 1, 2, 3, 4, 5, 6, 7}, 65536, 8192, 8192, opt);
    CHECK(g.world() == 8 && g.local_ranks() == 8);
    for (int r = 0; r < 8; ++r) {
        CHECK(g.rows_of(r).row0 == 8192 * r && g.rows_of(r).rows == 8192);
        CHECK(g.band_of(r, 3).row0 == 8192 * r + 3 * 2048 && g.band_of(r, 3).rows == 2048);
    }
    g.run(Gather::Banded);
    g.run(Gather::PeerStore);
    for (int i = 0; i < 8; ++i) CHECK(g.steps_enqueued(i) == 2);
    g.inject_failure(5);
    bool threw = false;
    try {
        g.run(Gather::AfterGemm);
    } catch (const PeerFailure& e) {
        threw = true;
        CHECK(std::strstr(e.what(), "rank 5") != nullptr && std::strstr(e.what(), "before anything was enqueued") != nullptr);
    }
    CHECK(threw);
    for (int i = 0; i < 8; ++i) CHECK(g.steps_enqueued(i) == 2);      // nobody started the failed step
    threw = false;
    try {
        g.run(Gather::None);
    } catch (const std::runtime_error&) {
        threw = true;
    }
    CHECK(threw);
    std::printf("[PASS] plan and failure path (dry run)\n");
}

static void test_every_gather_mode(int world, bool multicast = false) {
    const int64_t m = 1536 + 128;       // ragged over two or four ranks
    const int n = 768, k = 320;
    std::vector<int> devices(world);
    for (int i = 0; i < world; ++i) devices[i] = i;
    ShardedGemmOptions opt;
    opt.bands = 2;
    opt.multicast = multicast;          // C bound to an NVLink multicast object: Gather::Multimem
    ShardedGemm g(devices, m, n, k, opt);
    std::mt19937 gen(3);
    std::normal_distribution<float> dist(0.0f, 1.0f);
    std::vector<float> a(size_t(m) * k), b(size_t(k) * n);
    for (float& v : a) v = dist(gen);
    for (float& v : b) v = dist(gen);
    g.set_b(b.data());
    int64_t covered = 0;
    for (int i = 0; i < world; ++i) {
        const RowRange own = g.rows_of(i);
        CHECK(own.row0 == covered);
        covered += own.rows;
        g.set_a(i, a.data() + own.row0 * k);
    }
    CHECK(covered == m);
    const std::vector<Gather> modes = multicast
        ? std::vector<Gather>{Gather::Multimem, Gather::AfterGemm, Gather::Multimem}
        : std::vector<Gather>{Gather::AfterGemm, Gather::Banded, Gather::PeerStore, Gather::CopyEngine};
    std::vector<float> host(size_t(m) * n);
    for (Gather mode : modes) {
        for (int i = 0; i < world; ++i) {
            cudaSetDevice(devices[i]);
            cudaMemset(g.c(i), 0xff, size_t(m) * n * sizeof(float));     // NaN
            cudaDeviceSynchronize();
        }
        g.run(mode);
        g.synchronize();
        for (int i = 0; i < world; ++i) {
            g.read_c(i, 0, m, host.data());
            for (int s = 0; s < 400; ++s) {
                const int64_t row = (int64_t(s) * 7919 + i * 13) % m;
                const int col = (s * 104729) % n;
                double want = 0.0;
                for (int q = 0; q < k; ++q) want += double(a[row * k + q]) * double(b[size_t(q) * n + col]);
                const float got = host[row * n + col];
                CHECK(got == got);                                                   // not NaN: the row arrived
                CHECK(std::fabs(got - want) <= 2e-2 * (1.0 + std::fabs(want)));     // TF32 operands
            }
        }
    }
    const float ms = g.time_steps(multicast ? Gather::Multimem : Gather::PeerStore, 3, 1);
    CHECK(ms > 0.0f);
    std::printf("[PASS] every gather mode on %d GPU(s)%s, %.3f ms per fused step\n", world,
                multicast ? " through the switch" : "", ms);
}

int main(int argc, char** argv) {
    std::setvbuf(stdout, nullptr, _IONBF, 0);
    try {
        test_plan_and_failure_path_without_a_gpu();
        if (argc > 1 && std::string(argv[1]) == "--dry") {
            std::printf("ALL PASSED\n");
            return 0;
        }
        int count = 0;
        CHECK(cudaGetDeviceCount(&count) == cudaSuccess && count >= 1);
        test_every_gather_mode(1);
        if (count >= 2) {
            test_every_gather_mode(count >= 4 ? 4 : 2);
            test_every_gather_mode(count >= 4 ? 4 : 2, /*multicast=*/true);
        }
    } catch (const std::exception& e) {
        std::printf("FAILED with exception: %s\n", e.what());
        return 1;
    }
    std::printf("ALL PASSED\n");
    return 0;
}
