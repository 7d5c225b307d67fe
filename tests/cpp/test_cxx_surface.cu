// C++ callers' view of the library: cudeep::Tensor, MemoryPool, Stream/Event and the launchers in
// cudeep::kernels, exercised the way the reference's own C++ unit tests do
// (tests/unit/test_tensor.cu:189-248,368-381, tests/unit/test_matmul.cu:13-68,
// tests/unit/test_kernels.cu:324-425 in the cuDeep tree), plus one TF32-sized product checked
// against a float64 host loop.  Exits 0 when every check holds, prints the first failure otherwise.
#include "cudeep/kernels/conv.cuh"
#include "cudeep/kernels/matmul.cuh"
#include "cudeep/memory.cuh"
#include "cudeep/stream.cuh"
#include "cudeep/tensor.cuh"

#include <cuda_fp16.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <numeric>
#include <stdexcept>
#include <vector>

using namespace cudeep;

#define CHECK(cond)                                                              \
    do {                                                                         \
        if (!(cond)) {                                                           \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);        \
            std::exit(1);                                                        \
        }                                                                        \
    } while (0)

static std::vector<float> host_of(const Tensor& t) {
    std::vector<float> v(static_cast<size_t>(t.numel()));
    t.to_host(v.data());
    return v;
}

static void test_tensor_basics() {
    Tensor t({2, 3, 4});
    CHECK(t.ndim() == 3 && t.numel() == 24 && t.nbytes() == 96 && t.dtype() == DType::Float32);
    CHECK((t.strides() == std::vector<int64_t>{12, 4, 1}) && t.is_contiguous());
    t.fill_(2.5f);
    for (float v : host_of(t)) CHECK(v == 2.5f);
    Tensor copy = t;                          // deep copy
    CHECK(copy.data() != t.data());
    t.zero_();
    for (float v : host_of(copy)) CHECK(v == 2.5f);
    for (float v : host_of(t)) CHECK(v == 0.0f);
    Tensor moved = std::move(copy);
    CHECK(moved.numel() == 24);
    std::vector<float> iota(24);
    std::iota(iota.begin(), iota.end(), 0.0f);
    Tensor a = Tensor::from_host(iota.data(), {4, 6});
    Tensor r = a.reshape({3, -1});
    CHECK((r.shape() == std::vector<int64_t>{3, 8}) && r.data() == a.data());
    Tensor tr = a.transpose(0, 1);
    CHECK((tr.shape() == std::vector<int64_t>{6, 4}) && !tr.is_contiguous() && tr.data() == a.data());
    Tensor tc = tr.contiguous();
    CHECK(tc.is_contiguous() && tc.data() != a.data());
    std::vector<float> got = host_of(tc);
    for (int i = 0; i < 6; ++i)
        for (int j = 0; j < 4; ++j) CHECK(got[i * 4 + j] == iota[j * 6 + i]);
    Tensor s = a + a, d = a - a, p = a * a;
    std::vector<float> hs = host_of(s), hd = host_of(d), hp = host_of(p);
    for (int i = 0; i < 24; ++i) CHECK(hs[i] == 2 * iota[i] && hd[i] == 0.0f && hp[i] == iota[i] * iota[i]);
    for (float v : host_of(Tensor::ones({5}))) CHECK(v == 1.0f);
    Tensor z = Tensor::randn_seeded({1000}, DType::Float32, 7), z2 = Tensor::randn_seeded({1000}, DType::Float32, 7);
    CHECK(host_of(z) == host_of(z2));
    std::printf("[PASS] tensor basics\n");
}

static void test_tensor_matmul() {
    std::vector<float> a = {1, 2, 3, 4}, b = {5, 6, 7, 8};
    std::vector<float> c = host_of(Tensor::from_host(a.data(), {2, 2}).matmul(Tensor::from_host(b.data(), {2, 2})));
    CHECK(std::fabs(c[0] - 19) < 1e-5f && std::fabs(c[1] - 22) < 1e-5f && std::fabs(c[2] - 43) < 1e-5f &&
          std::fabs(c[3] - 50) < 1e-5f);
    // [2,3] x [3,4] with B = [I | 0]
    std::vector<float> a23 = {1, 2, 3, 4, 5, 6}, b34(12, 0.0f);
    b34[0] = b34[5] = b34[10] = 1.0f;
    std::vector<float> c24 = host_of(Tensor::from_host(a23.data(), {2, 3}).matmul(Tensor::from_host(b34.data(), {3, 4})));
    CHECK(c24[0] == 1 && c24[1] == 2 && c24[2] == 3 && c24[3] == 0 && c24[4] == 4 && c24[6] == 6 && c24[7] == 0);
    // 8x8 times identity
    Tensor r = Tensor::randn_seeded({8, 8}, DType::Float32, 3);
    std::vector<float> eye(64, 0.0f);
    for (int i = 0; i < 8; ++i) eye[i * 9] = 1.0f;
    std::vector<float> hr = host_of(r), hri = host_of(r.matmul(Tensor::from_host(eye.data(), {8, 8})));
    for (int i = 0; i < 64; ++i) CHECK(std::fabs(hr[i] - hri[i]) < 1e-5f);
    // float64 2x2
    std::vector<double> ad = {1.5, 2.5, 3.5, 4.5}, bd = {0.5, 1.5, 2.5, 3.5}, cd(4);
    Tensor::from_host(ad.data(), {2, 2}, DType::Float64).matmul(Tensor::from_host(bd.data(), {2, 2}, DType::Float64)).to_host(cd.data());
    CHECK(std::fabs(cd[0] - (1.5 * 0.5 + 2.5 * 2.5)) < 1e-10 && std::fabs(cd[3] - (3.5 * 1.5 + 4.5 * 3.5)) < 1e-10);
    // what the reference rejects
    bool threw = false;
    try { Tensor({4, 6}).matmul(Tensor({5, 3})); } catch (const std::runtime_error&) { threw = true; }
    CHECK(threw);
    threw = false;
    try { Tensor({4, 6}).matmul(Tensor({3, 6}).transpose(0, 1)); } catch (const std::runtime_error&) { threw = true; }
    CHECK(threw);
    std::printf("[PASS] Tensor::matmul\n");
}

static void test_tf32_product_against_host() {
    const int m = 384, n = 512, k = 256;
    Tensor a = Tensor::randn_seeded({m, k}, DType::Float32, 11), b = Tensor::randn_seeded({k, n}, DType::Float32, 12);
    std::vector<float> ha = host_of(a), hb = host_of(b), hc = host_of(a.matmul(b));
    double num = 0.0, den = 0.0;
    for (int i = 0; i < m; i += 7) {
        for (int j = 0; j < n; ++j) {
            double s = 0.0;
            for (int p = 0; p < k; ++p) s += double(ha[i * k + p]) * double(hb[p * n + j]);
            num += (hc[i * n + j] - s) * (hc[i * n + j] - s);
            den += s * s;
        }
    }
    const double rel = std::sqrt(num / den);
    CHECK(rel <= 5e-3 && rel > 1e-6);           // TF32 accuracy: the tensor-core path ran
    // the strict launcher on the same data is FP32-accurate
    Tensor c32({m, n});
    kernels::launch_matmul_kernel_fp32<float>(static_cast<const float*>(a.data()), static_cast<const float*>(b.data()),
                                              static_cast<float*>(c32.data()), m, n, k);
    std::vector<float> h32 = host_of(c32);
    num = den = 0.0;
    for (int j = 0; j < n; ++j) {
        double s = 0.0;
        for (int p = 0; p < k; ++p) s += double(ha[p]) * double(hb[p * n + j]);
        num += (h32[j] - s) * (h32[j] - s);
        den += s * s;
    }
    CHECK(std::sqrt(num / den) <= 1e-5);
    std::printf("[PASS] TF32 and strict FP32 products\n");
}

static void test_conv_launcher() {
    std::vector<float> ones(9, 1.0f), bias = {10.0f}, out(9);
    Tensor x = Tensor::from_host(ones.data(), {1, 1, 3, 3}), w = Tensor::from_host(ones.data(), {1, 1, 3, 3});
    Tensor b = Tensor::from_host(bias.data(), {1});
    Tensor y({1, 1, 1, 1});
    kernels::launch_conv2d_forward_kernel<float>(static_cast<const float*>(x.data()), static_cast<const float*>(w.data()),
                                                 static_cast<const float*>(b.data()), static_cast<float*>(y.data()),
                                                 1, 1, 1, 3, 3, 3, 3, 1, 1, 0, 0);
    CHECK(std::fabs(host_of(y)[0] - 19.0f) < 1e-4f);
    Tensor yp({1, 1, 3, 3});
    kernels::launch_conv2d_forward_kernel<float>(static_cast<const float*>(x.data()), static_cast<const float*>(w.data()),
                                                 nullptr, static_cast<float*>(yp.data()), 1, 1, 1, 3, 3, 3, 3, 1, 1, 1, 1);
    std::vector<float> hp = host_of(yp);
    CHECK(std::fabs(hp[4] - 9) < 1e-4f && std::fabs(hp[0] - 4) < 1e-4f && std::fabs(hp[1] - 6) < 1e-4f);
    std::printf("[PASS] conv2d launcher\n");
}

static void test_pool_and_events() {
    MemoryPool& pool = MemoryPool::instance();
    const size_t before = pool.allocated_bytes();
    void* p = device_malloc(1 << 20);
    CHECK(pool.allocated_bytes() == before + (2u << 20));      // 1 MiB requests take the 2 MiB class
    device_free(p);
    CHECK(pool.allocated_bytes() == before && pool.cached_bytes() >= (2u << 20));
    void* q = device_malloc(1 << 20);
    CHECK(q == p);                                             // the cached block is reused
    device_free(q);
    Stream s;
    Event e0, e1;
    Tensor a = Tensor::randn_seeded({512, 512}, DType::Float32, 1);
    a.set_stream(s.get());
    e0.record(s.get());
    Tensor c = a.matmul(a);
    e1.record(s.get());
    e1.synchronize();
    CHECK(e1.elapsed_ms(e0) >= 0.0f);
    s.synchronize();
    std::printf("[PASS] pool, stream, event\n");
}

static void test_stream_aware_pool() {
    MemoryPool& pool = MemoryPool::instance();
    pool.release_cached();
    Stream s1, s2;
    const size_t bytes = (4u << 20) + 512;                      // a size class of its own
    void* p = pool.allocate(bytes, s1.get());
    // A few milliseconds of work on s1, then the block is released behind it.
    Tensor a = Tensor::randn_seeded({4096, 4096}, DType::Float32, 3);
    a.set_stream(s1.get());
    Tensor c1 = a.matmul(a), c2 = a.matmul(a), c3 = a.matmul(a), c4 = a.matmul(a);
    pool.deallocate(p, s1.get());
    void* same = pool.allocate(bytes, s1.get());
    CHECK(same == p);                                           // same stream: reused at once
    pool.deallocate(same, s1.get());
    void* other = pool.allocate(bytes, s2.get());
    if (cudaStreamQuery(s1.get()) == cudaErrorNotReady) CHECK(other != p);   // s1 still busy: a fresh block
    cudaGetLastError();
    s1.synchronize();
    pool.deallocate(other, s2.get());
    // A tensor may outlive the stream it worked on.
    Tensor survivor;
    {
        Stream inner;
        Tensor t = Tensor::ones({256, 256});
        t.set_stream(inner.get());
        survivor = t.matmul(t);
    }
    survivor.set_stream(nullptr);                               // its stream is gone: further work goes elsewhere
    CHECK(std::fabs(host_of(survivor)[0] - 256.0f) < 1e-2f);
    survivor = Tensor();
    Tensor orphan;
    {
        Stream inner;
        Tensor t = Tensor::ones({128, 128});
        t.set_stream(inner.get());
        orphan = t.matmul(t);
    }
    orphan = Tensor();                                          // storage released on a stream that no longer exists
    pool.release_cached();
    std::printf("[PASS] stream-aware pool\n");
}

static void test_fp16_launcher() {
    const int m = 256, n = 192, k = 128;
    std::vector<__half> ha(m * k), hb(k * n);
    std::vector<float> fa(m * k), fb(k * n);
    for (int i = 0; i < m * k; ++i) { fa[i] = float((i * 7) % 13 - 6) / 8.0f; ha[i] = __float2half(fa[i]); }
    for (int i = 0; i < k * n; ++i) { fb[i] = float((i * 5) % 11 - 5) / 4.0f; hb[i] = __float2half(fb[i]); }
    __half* da = static_cast<__half*>(device_malloc(ha.size() * 2));
    __half* db = static_cast<__half*>(device_malloc(hb.size() * 2));
    float* dc = static_cast<float*>(device_malloc(size_t(m) * n * 4));
    memcpy_h2d(da, ha.data(), ha.size() * 2);
    memcpy_h2d(db, hb.data(), hb.size() * 2);
    kernels::launch_matmul_kernel_fp16(da, db, dc, m, n, k);
    std::vector<float> hc(size_t(m) * n);
    memcpy_d2h(hc.data(), dc, hc.size() * 4);
    for (int i : {0, 17, 255}) {
        for (int j : {0, 63, 191}) {
            double want = 0.0;
            for (int q = 0; q < k; ++q) want += double(fa[i * k + q]) * double(fb[q * n + j]);
            CHECK(std::fabs(hc[size_t(i) * n + j] - want) <= 1e-4 * (1.0 + std::fabs(want)));   // the inputs are exact in FP16
        }
    }
    device_free(da);
    device_free(db);
    device_free(dc);
    std::printf("[PASS] fp16 launcher\n");
}

int main() {
    std::setvbuf(stdout, nullptr, _IONBF, 0);
    try {
        test_tensor_basics();
        test_tensor_matmul();
        test_tf32_product_against_host();
        test_conv_launcher();
        test_pool_and_events();
        test_stream_aware_pool();
        test_fp16_launcher();
    } catch (const std::exception& e) {
        std::printf("FAILED with exception: %s\n", e.what());
        return 1;
    }
    std::printf("ALL PASSED\n");
    return 0;
}
