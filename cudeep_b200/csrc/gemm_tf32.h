// Host entry of the tcgen05 TF32 GEMM (see gemm_tf32.cu).
#pragma once

#include "runtime.h"

namespace cudeep_b200 {

// Optional overrides; zero means "let the launcher choose".
struct GemmTuning {
    int ctas = 0;            // 1 or 2 CTAs per MMA
    int bn = 0;              // tile columns: 64, 128 or 256
    int raster_group = 0;    // tile rows walked together
    int max_ctas = 0;        // cap on resident CTAs (default: one per SM)
    uint32_t b_lbo = 0;      // B shared-memory descriptor overrides (bring-up aid)
    uint32_t b_sbo = 0;
    int stages = 0;          // pipeline stages to use (default: all that fit)
    int split_k = 0;         // K ranges per tile of the ragged last wave: 0 = choose, 1 = never split
    int katoms = 0;          // 32-wide K blocks per pipeline stage: 1 or 2
    int cluster_split = 0;   // K ranges per tile reduced inside a thread-block cluster (2, 4, 8):
                             // 0 = choose, 1 = never
    int ring_staging = 0;    // -1: flip the default of staging a CTA's last tile in the idle stage ring
    int tma_store = 0;       // -1: write C from registers even where bulk tensor stores are possible
    int b_chunked = 0;       // -1: load B[K,N] as separate 32-column boxes even when N % 32 == 0
    uint32_t debug = 0;      // diagnostics, see UmmaSchedule::debug
    uint32_t wait_limit_ms = 0;   // limit of every in-kernel wait (0 = the default of 2000 ms)
};

// True when the tensor-core path can take this problem (sm_100 device,
// 16-byte aligned bases, K % 4 == 0, and N % 4 == 0 for B[K,N]).
bool gemm_tf32_supported(const float* a, const float* b, const float* c, int m, int n, int k,
                         bool b_is_nk);

// C[M,N] = act(A[M,K] * B + bias), TF32 multiply, FP32 accumulate.
//   b_is_nk == false: B is [K,N] row-major;  true: B is [N,K] row-major (y = x W^T).
//   bias: nullptr, or N values (bias_per_row == false), or M values (bias_per_row == true).
// Asynchronous on `stream`.  Throws std::runtime_error on bad arguments or launch failure.
void gemm_tf32(const float* a, const float* b, bool b_is_nk, float* c, int m, int n, int k,
               const float* bias, bool bias_per_row, int act, const GemmTuning& tune,
               cudaStream_t stream);

// One rank's share of a row-sharded product, written into this GPU's C and, by the same kernel,
// into the other GPUs' copies of C: c[i] are peer-mapped device pointers to the place this rank's
// rows have in peer i's C (same row pitch N).  Tile by tile the epilogue repeats its bulk tensor
// store once per peer, so the all-gather of C overlaps the GEMM instead of following it.  The
// caller makes the result visible across ranks (this launch must have completed on every rank
// before any rank reads rows it did not compute).  No activation, no bias, whole tiles only.
constexpr int kMaxGemmPeers = 7;
struct GemmPeerOutputs {
    int count = 0;
    float* c[kMaxGemmPeers] = {};
};
void gemm_tf32_push(const float* a, const float* b, bool b_is_nk, float* c, int m, int n, int k,
                    const GemmPeerOutputs& peers, const GemmTuning& tune, cudaStream_t stream);

// The same product with C behind a multicast address (GPUs of one NVSwitch domain, multicast.h):
// `c_multicast` is the address of this rank's rows of C through which a store reaches every GPU's
// copy, this GPU's included; `c_local` is their ordinary address on this GPU (used for alignment
// checks only: the kernel writes through `c_multicast` alone).  The epilogue reads each staged block
// back and writes it with multimem.st, so a tile crosses NVLink once however many GPUs receive it.
void gemm_tf32_multimem(const float* a, const float* b, bool b_is_nk, float* c_local, float* c_multicast, int m, int n,
                        int k, const GemmTuning& tune, cudaStream_t stream);

// The tile shape the launcher would pick for a problem on a device with `num_sms` SMs (host
// arithmetic only: no device is touched): CTAs per MMA, tile columns, K ranges per cluster,
// K blocks per stage, and the estimated time in microseconds.
struct GemmPlan {
    int ctas, bn, cluster_split, katoms;
    double estimate_us;
};
GemmPlan gemm_tf32_plan(int m, int n, int k, int act, int num_sms);

// C[M,N] = A^T * B with A stored [K,M] and B stored [K,N] (both row-major): the weight-gradient
// product dW = X^T dY of a Linear layer, and a^T @ grad of matmul's backward, without a transposed
// copy of the left operand (reference python/cuDeep/tensor.py:430-443 makes that copy).
bool gemm_tf32_tn_supported(const float* a, const float* b, int m, int n, int k);
void gemm_tf32_tn(const float* a, const float* b, float* c, int m, int n, int k, const GemmTuning& tune,
                  cudaStream_t stream);

}  // namespace cudeep_b200
