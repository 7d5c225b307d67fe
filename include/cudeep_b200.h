/* C ABI of libcudeep_b200.so: the dense-contraction hot path of cuDeep
 * (matmul, Linear forward, Conv2d forward) for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain pointers and sizes, returns 0 on success and a
 * non-zero code on failure; cudeep_b200_last_error() then describes the
 * failure for the calling thread.  Device-pointer entry points are
 * asynchronous on `stream` (NULL = the legacy default stream) and never
 * synchronise.  All matrices are row-major and contiguous, images are NCHW,
 * filters OIHW, as in the reference.
 *
 * Each declaration names the reference interface it stands in for
 * (paths are relative to the cuDeep source tree).
 */
#ifndef CUDEEP_B200_H
#define CUDEEP_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Return codes. */
#define CUDEEP_B200_OK 0
#define CUDEEP_B200_ERROR 1          /* bad argument or CUDA failure; see cudeep_b200_last_error() */

/* Epilogue codes; values equal cudeep::kernels::GemmEpilogue
 * (include/cudeep/kernels/matmul.cuh:32-38). */
#define CUDEEP_B200_EPI_NONE 0
#define CUDEEP_B200_EPI_RELU 1
#define CUDEEP_B200_EPI_GELU 2       /* tanh form, include/cudeep/ptx_intrinsics.cuh:545-549 */
#define CUDEEP_B200_EPI_SILU 3
#define CUDEEP_B200_EPI_SIGMOID 4

typedef void* cudeep_b200_stream_t;  /* a cudaStream_t */

/* ---- library ---------------------------------------------------------------------- */

/* Library version, major*100 + minor. */
int cudeep_b200_version(void);

/* Message of the last failure on this thread ("" if none).  The pointer stays
 * valid until the next failing call on the same thread. */
const char* cudeep_b200_last_error(void);

/* Reads the current device's kernel status word into *status (0 = no kernel
 * abandoned a wait; 1..4 name the pipeline role that timed out) and clears it
 * when `clear` is non-zero.  Synchronises the device. */
int cudeep_b200_device_status(int clear, uint32_t* status);

/* ---- matmul (device pointers) -------------------------------------------------------- */

/* C[M,N] = A[M,K] * B[K,N], float.  TF32 tensor cores (FP32 accumulate) for
 * M,N >= 64, K >= 32 with K % 4 == 0, N % 4 == 0 and 16-byte aligned A, B;
 * strict FP32 otherwise.
 * Replaces cudeep::kernels::launch_matmul_kernel<float>
 * (include/cudeep/kernels/matmul.cuh:8-12, src/kernels/matmul_kernel.cu:1785-1841). */
int cudeep_b200_matmul_f32(const float* A, const float* B, float* C, int M, int N, int K,
                           cudeep_b200_stream_t stream);

/* Same product, always strict FP32 (fused multiply-add, no tensor cores).
 * Replaces launch_matmul_kernel_fp32<float>
 * (matmul.cuh:14-18, matmul_kernel.cu:1851-1863). */
int cudeep_b200_matmul_f32_strict(const float* A, const float* B, float* C, int M, int N, int K,
                                  cudeep_b200_stream_t stream);

/* FP64 product.  Replaces launch_matmul_kernel<double> (matmul_kernel.cu:1843-1849). */
int cudeep_b200_matmul_f64(const double* A, const double* B, double* C, int M, int N, int K,
                           cudeep_b200_stream_t stream);

/* C = act(A * B).  Replaces launch_matmul_fused_act
 * (matmul.cuh:40-44, matmul_kernel.cu:1884-1924). */
int cudeep_b200_matmul_fused_act(const float* A, const float* B, float* C, int M, int N, int K,
                                 int epilogue, cudeep_b200_stream_t stream);

/* y[M,N] = act(x[M,K] * W[N,K]^T + bias[N]); bias may be NULL.  One kernel for
 * what nn.Linear.forward runs as transpose-copy + GEMM + broadcast_add (+ a
 * separate activation): python/cuDeep/nn.py:110-115,
 * src/bindings/module.cpp:664-694, src/tensor.cu:256-281. */
int cudeep_b200_linear_forward_f32(const float* x, const float* W, const float* bias, float* y,
                                   int M, int N, int K, int epilogue,
                                   cudeep_b200_stream_t stream);
int cudeep_b200_linear_forward_f64(const double* x, const double* W, const double* bias, double* y,
                                   int M, int N, int K, int epilogue,
                                   cudeep_b200_stream_t stream);

/* The two products of matmul's backward pass, computed without the transposed copies the
 * reference makes first (MatMulOp.backward, python/cuDeep/tensor.py:430-443):
 *   nt: C[M,N] = A[M,K] * B[N,K]^T   (grad_a = grad * b^T; also x * W^T of Linear)
 *   tn: C[M,N] = A[K,M]^T * B[K,N]   (grad_b = a^T * grad; also dW^T = x^T * dy of Linear)
 * Precision rule as cudeep_b200_matmul_f32 (tn needs M % 4 == 0 and N % 4 == 0 for TF32). */
int cudeep_b200_matmul_nt_f32(const float* A, const float* B, float* C, int M, int N, int K,
                              cudeep_b200_stream_t stream);
int cudeep_b200_matmul_tn_f32(const float* A, const float* B, float* C, int M, int N, int K,
                              cudeep_b200_stream_t stream);

/* What the launcher would choose for C[M,N] = A[M,K] * B on a device with num_sms SMs: CTAs per
 * MMA (1 | 2), tile columns, K ranges reduced inside a cluster (1 = none), K blocks per pipeline
 * stage, and its time estimate in microseconds.  Host arithmetic only: works without a GPU.  No
 * reference counterpart (the reference dispatches on cc and size thresholds, matmul_kernel.cu:1785-1841). */
int cudeep_b200_gemm_tf32_plan(int M, int N, int K, int epilogue, int num_sms, int* ctas, int* bn,
                               int* cluster_split, int* katoms, double* estimate_us);

/* C[M,N] (float) = A[M,K] * B[K,N] with IEEE half operands (passed as const void*) and FP32
 * accumulation: launch_matmul_kernel_fp16 (matmul.cuh:27-30).  Tensor cores (kind::f16) when A and
 * B are 16-byte aligned, K and N are multiples of 8 and M, N, K >= 64; a SIMT kernel otherwise. */
int cudeep_b200_matmul_f16(const void* A, const void* B, float* C, int M, int N, int K,
                           cudeep_b200_stream_t stream);
/* The same on the tensor-core path only (fails instead of falling back), for benchmarks and
 * bring-up: ctas 0 | 1 | 2; b_lbo / b_sbo as in cudeep_b200_gemm_tf32_tuned (bits 0-15 only). */
/* The same with BF16 operands (an addition: the reference has FP16 only). */
int cudeep_b200_matmul_bf16(const void* A, const void* B, float* C, int M, int N, int K,
                            cudeep_b200_stream_t stream);
int cudeep_b200_matmul_f16_tuned(const void* A, const void* B, float* C, int M, int N, int K, int ctas,
                                 uint32_t b_lbo, uint32_t b_sbo, cudeep_b200_stream_t stream);

/* The TF32 tensor-core GEMM with explicit tile choices, for benchmarks and
 * bring-up.  b_is_nk: 0 = B is [K,N], 1 = B is [N,K].  bias: NULL, N values, or
 * M values when bias_per_row != 0.  ctas (1|2), bn (64|128|256), raster_group,
 * max_ctas: 0 selects the default.  max_ctas is a packed field: bits 0-15 cap
 * the resident CTAs, bits 16-23 limit the pipeline stages (0 = all that fit),
 * bits 24-27 are performance diagnostics that make the result meaningless
 * (1: stop loading operands once the stage ring is full, 2: skip the MMAs,
 * 4: issue MMAs without the stage ring, 8: skip the epilogue's loads and stores);
 * bit 28 loads B[K,N] as separate 32-column boxes instead of one chunked box;
 * bits 29-30 set the 32-wide K blocks per pipeline stage (1 or 2, 0 = default).
 * b_lbo / b_sbo: 0, or a byte offset that overrides the B shared-memory
 * descriptor fields (b_lbo bits 0-15); bits 16-23 of b_lbo set the split-K factor
 * of the ragged last wave of tiles (0 = choose, 1 = never split); bits 24-27 of
 * b_lbo set the K ranges per tile that a thread-block cluster reduces through
 * distributed shared memory (0 = choose, 1 = never, else 2, 4 or 8); bit 28 of
 * b_lbo writes C from registers instead of through bulk tensor stores; bits
 * 29-30 of b_lbo are two more diagnostics (29: stage the results but issue no
 * bulk store, 30: skip the accumulator loads); bit 31 of b_lbo flips whether a
 * CTA's last tile stages its results in the idle stage ring.  b_sbo: bits 0-15
 * the descriptor override, bits 16-30 a limit in milliseconds for every wait
 * inside the kernel (0 = 2000 ms), bit 31 a diagnostic in which no operand is
 * ever loaded, so that the wait for operands runs out and the kernel returns with
 * cudeep_b200_device_status() = 2 (the bounded-wait path, testable without a fault).  Fails
 * instead of falling back when the tensor-core path cannot take the problem. */
int cudeep_b200_gemm_tf32_tuned(const float* A, const float* B, int b_is_nk, float* C, int M, int N,
                                int K, const float* bias, int bias_per_row, int epilogue, int ctas,
                                int bn, int raster_group, int max_ctas, uint32_t b_lbo,
                                uint32_t b_sbo, cudeep_b200_stream_t stream);

/* ---- conv2d forward (device pointers) -------------------------------------------------- */

/* output[N,OC,OH,OW] = conv(input[N,C,H,W], weight[OC,C,KH,KW]) + bias[OC]
 * (cross-correlation, zero padding, no dilation or groups; bias may be NULL),
 * OH = (H + 2*pad_h - KH) / stride_h + 1.  Replaces
 * launch_conv2d_forward_kernel<float> (include/cudeep/kernels/conv.cuh:8-16,
 * src/kernels/conv_kernel.cu:225-335). */
int cudeep_b200_conv2d_forward_f32(const float* input, const float* weight, const float* bias,
                                   float* output, int batch, int in_channels, int out_channels,
                                   int in_h, int in_w, int kernel_h, int kernel_w, int stride_h,
                                   int stride_w, int pad_h, int pad_w,
                                   cudeep_b200_stream_t stream);

/* Same with an activation applied to conv + bias in the epilogue. */
int cudeep_b200_conv2d_forward_fused_f32(const float* input, const float* weight, const float* bias,
                                         float* output, int batch, int in_channels,
                                         int out_channels, int in_h, int in_w, int kernel_h,
                                         int kernel_w, int stride_h, int stride_w, int pad_h,
                                         int pad_w, int epilogue, cudeep_b200_stream_t stream);

/* The same for an input already stored channels-last, input[N,H,W,C] (Layout::NHWC of
 * include/cudeep/common.cuh:10-19; the reference declares the enum and has no kernel for it): the
 * tensor-core kernel gathers from that layout, so the re-layout pass of the NCHW form is skipped.
 * Filters stay OIHW, the output stays NCHW.  Needs C % 4 == 0, a 16-byte aligned input and a shape
 * on the tensor-core path; fails otherwise (no fallback). */
int cudeep_b200_conv2d_forward_fused_nhwc_f32(const float* input_nhwc, const float* weight,
                                              const float* bias, float* output, int batch,
                                              int in_channels, int out_channels, int in_h, int in_w,
                                              int kernel_h, int kernel_w, int stride_h, int stride_w,
                                              int pad_h, int pad_w, int epilogue,
                                              cudeep_b200_stream_t stream);

/* Conv2d forward (+ bias + activation) that allocates nothing.  No counterpart in the
 * reference: it exists for callers with a fixed device-memory plan - a serving process
 * whose own allocator owns all free memory, or a loop that cannot take an allocation's
 * implicit synchronisation or its failure mid-step.  Same arguments and results as
 * cudeep_b200_conv2d_forward_fused_f32; the scratch (NHWC copy of the input + packed
 * filters) lives in a 32 MiB array built into the library, which every GPU that loads
 * the library holds until the process exits.
 *   - Shapes whose scratch exceeds cudeep_b200_conv2d_noalloc_capacity() are refused
 *     with an error that states both sizes (C*H*(W + 2*pad_w)*batch*4 bytes, channels
 *     rounded up to 4, plus the filters with channels rounded up to 32).  Shapes the
 *     tensor-core path does not take (tiny, stride > 8) run the direct kernel and need no scratch.
 *   - "Allocates nothing" holds from the second call of a shape class on.  With CUDA's lazy
 *     module loading the first look-up of the array on a device loads it (that is when the
 *     32 MiB are taken), and the first launch of each kernel variant loads that kernel and
 *     raises its shared-memory limit.  Warm up at start-up, before giving the free memory
 *     away and before any stream capture: cudeep_b200_conv2d_noalloc_capacity() on each device
 *     resolves the array, one call per layer shape loads the kernels (or run the process with
 *     CUDA_MODULE_LOADING=EAGER).
 *   - All calls on a device share the one array and it keeps the previous call's
 *     contents; each call rewrites every byte it later reads, so nothing needs
 *     clearing, but two calls that overlap on the GPU (different streams, no
 *     dependency) race on it.  Serialise them. */
int cudeep_b200_conv2d_forward_noalloc_f32(const float* input, const float* weight, const float* bias,
                                           float* output, int batch, int in_channels,
                                           int out_channels, int in_h, int in_w, int kernel_h,
                                           int kernel_w, int stride_h, int stride_w, int pad_h,
                                           int pad_w, int epilogue, cudeep_b200_stream_t stream);

/* Bytes of built-in scratch behind cudeep_b200_conv2d_forward_noalloc_f32.  On a machine with a
 * GPU it also resolves the array on the current device (the per-device warm-up, see above). */
size_t cudeep_b200_conv2d_noalloc_capacity(void);

/* FP64 convolution.  Replaces launch_conv2d_forward_kernel<double>. */
int cudeep_b200_conv2d_forward_f64(const double* input, const double* weight, const double* bias,
                                   double* output, int batch, int in_channels, int out_channels,
                                   int in_h, int in_w, int kernel_h, int kernel_w, int stride_h,
                                   int stride_w, int pad_h, int pad_w,
                                   cudeep_b200_stream_t stream);

/* Gradients of the convolution.  Replace launch_conv2d_backward_data_kernel<float> and
 * launch_conv2d_backward_weight_kernel<float> (include/cudeep/kernels/conv.cuh:18-36,
 * src/kernels/conv_kernel.cu:417-545).  in_h / in_w are the forward input's size.
 * Both run on the tensor cores (TF32) for layers with at least 32 output channels: grad_input
 * with at least 32 input channels (strided layers, strides up to 8, in sub-pixel form: one
 * stride-1 implicit GEMM over grad_output for all parity classes of the input pixels, no zeros
 * inserted), grad_weight with at least 256 output pixels and strides up to 8; strict FP32 kernels
 * otherwise. */
int cudeep_b200_conv2d_backward_data_f32(const float* grad_output, const float* weight, float* grad_input,
                                         int batch, int in_channels, int out_channels, int in_h, int in_w,
                                         int kernel_h, int kernel_w, int stride_h, int stride_w, int pad_h,
                                         int pad_w, cudeep_b200_stream_t stream);
int cudeep_b200_conv2d_backward_weight_f32(const float* grad_output, const float* input, float* grad_weight,
                                           int batch, int in_channels, int out_channels, int in_h, int in_w,
                                           int kernel_h, int kernel_w, int stride_h, int stride_w, int pad_h,
                                           int pad_w, cudeep_b200_stream_t stream);

/* ---- host-buffer entry points ---------------------------------------------------------- */

/* The reference's Python call sequence Tensor.from_numpy(a).matmul(
 * Tensor.from_numpy(b)).numpy() as one call on host memory: copies A and B to
 * the device, multiplies, copies C back and waits for it
 * (src/bindings/module.cpp:106,116-146; src/tensor.cu:208-223,384-420).
 * strict != 0 selects the strict FP32 kernel.  Device buffers come from the
 * library's memory pool and are reused by later calls of the same sizes. */
int cudeep_b200_matmul_host_f32(const float* A, const float* B, float* C, int M, int N, int K,
                                int strict);

/* nn.Linear forward on host memory (x, W, bias in; y out). */
int cudeep_b200_linear_forward_host_f32(const float* x, const float* W, const float* bias, float* y,
                                        int M, int N, int K, int epilogue);

/* conv2d forward on host memory. */
int cudeep_b200_conv2d_forward_host_f32(const float* input, const float* weight, const float* bias,
                                        float* output, int batch, int in_channels, int out_channels,
                                        int in_h, int in_w, int kernel_h, int kernel_w, int stride_h,
                                        int stride_w, int pad_h, int pad_w, int epilogue);

/* ---- tensor plumbing ------------------------------------------------------------------- */

/* Copies; asynchronous on `stream`, blocking when stream is NULL
 * (memcpy_h2d / d2h / d2d, include/cudeep/memory.cuh:41-45, src/memory.cu:75-97). */
int cudeep_b200_memcpy_h2d(void* dst, const void* src, size_t nbytes, cudeep_b200_stream_t stream);
int cudeep_b200_memcpy_d2h(void* dst, const void* src, size_t nbytes, cudeep_b200_stream_t stream);
int cudeep_b200_memcpy_d2d(void* dst, const void* src, size_t nbytes, cudeep_b200_stream_t stream);
int cudeep_b200_stream_synchronize(cudeep_b200_stream_t stream);   /* Stream::synchronize, stream.cuh:18 */
int cudeep_b200_device_synchronize(void);

/* dst (contiguous over `shape`) = src read through `strides` (in elements); rank 1..8,
 * elem_size 4 or 8.  Replaces Tensor::contiguous / launch_strided_copy
 * (src/tensor.cu:47-68,256-281) without its device allocations and stream synchronisation. */
int cudeep_b200_strided_copy(const void* src, void* dst, int ndim, const long long* shape,
                             const long long* strides, int elem_size, cudeep_b200_stream_t stream);

/* Tensor::fill_ (src/tensor.cu:422-446). */
int cudeep_b200_fill_f32(float* dst, float value, long long count, cudeep_b200_stream_t stream);
int cudeep_b200_fill_f64(double* dst, double value, long long count, cudeep_b200_stream_t stream);

/* out[i, j] = matrix[i, j] + row[j]: broadcast_add
 * (src/bindings/module.cpp:664-694, src/kernels/elementwise_kernel.cu:187-204). */
int cudeep_b200_broadcast_add_f32(const float* matrix, const float* row, float* out, long long rows,
                                  int cols, cudeep_b200_stream_t stream);
int cudeep_b200_broadcast_add_f64(const double* matrix, const double* row, double* out, long long rows,
                                  int cols, cudeep_b200_stream_t stream);

/* y = act(x) as a separate pass, for an activation module that does not follow a Linear or
 * Conv2d it could be fused into (activation_fwd kernels, src/kernels/activation_kernel.cu:70-95). */
int cudeep_b200_activation_f32(const float* x, float* y, long long count, int epilogue,
                               cudeep_b200_stream_t stream);

/* ---- streams, events, device (include/cudeep/stream.cuh:8-44, module.cpp:642-658) ------- */

int cudeep_b200_stream_create(cudeep_b200_stream_t* stream);
int cudeep_b200_stream_destroy(cudeep_b200_stream_t stream);
int cudeep_b200_event_create(void** event);
int cudeep_b200_event_destroy(void* event);
int cudeep_b200_event_record(void* event, cudeep_b200_stream_t stream);
int cudeep_b200_event_synchronize(void* event);
int cudeep_b200_event_elapsed_ms(void* start, void* end, float* ms);
int cudeep_b200_device_info(int* device, int* sm_count, int* cc_major, int* cc_minor, size_t* total_mem);

/* ---- memory pool (cudeep::MemoryPool, include/cudeep/memory.cuh:13-46) ------------------- */

int cudeep_b200_pool_alloc(size_t nbytes, void** ptr);     /* MemoryPool::allocate   */
int cudeep_b200_pool_free(void* ptr);                      /* MemoryPool::deallocate */
/* Stream-aware forms (additions): a block freed on a stream serves that stream again at once, any
 * other stream only after the work queued before the free has drained. */
int cudeep_b200_pool_alloc_on_stream(size_t nbytes, cudeep_b200_stream_t stream, void** ptr);
int cudeep_b200_pool_free_on_stream(void* ptr, cudeep_b200_stream_t stream);
int cudeep_b200_pool_release_cached(void);                 /* MemoryPool::release_cached */
int cudeep_b200_pool_stats(size_t* allocated_bytes, size_t* cached_bytes);
/* The launchers' temporaries (conv re-layouts, packed filters, split-K partial sums) come from a
 * stream-ordered pool of the library's own on each device, as the reference takes its temporaries
 * from cudaMallocAsync (src/kernels/conv_kernel.cu:282,314,748-754); unlike the reference it leaves
 * the device's default pool untouched and keeps freed scratch cached.  This call gives all but
 * `keep_bytes` of that cache on the current device back to the driver. */
int cudeep_b200_scratch_trim(size_t keep_bytes);

/* ---- row-sharded GEMM over the GPUs of one node (cudeep::dist::ShardedGemm) ---------------- */

/* C[M,N] = A[M,K] * B[K,N] with A and C split by rows over `world` GPUs and B replicated; each
 * rank's product is cudeep_b200_matmul_f32's.  No counterpart in the reference, which is
 * single-device (src/kernels/matmul_kernel.cu:1745 queries device 0 only): this is the multi-GPU
 * form of launch_matmul_kernel<float> (include/cudeep/kernels/matmul.cuh:8-12).  The object owns
 * its device buffers (per rank: its rows of A, a replica of B, the whole C).
 *
 * gather modes (what happens to C after / while it is computed):
 *   0 none            every GPU keeps only the rows it computed
 *   1 after GEMM      one in-place ncclAllGather behind the GEMM, same stream
 *   2 banded          row bands; band i's NCCL transfer on a second stream overlaps band i+1's GEMM
 *   3 peer store      the GEMM's epilogue stores each tile into every GPU's C (peer-mapped memory,
 *                     bulk tensor stores; no load ever touches a peer, no collective is called)
 *   4 collective only the all-gather alone (for timing)
 *   5 copy engine     row bands; band i goes to every peer as a device-to-device copy on the copy
 *                     engines (peer-mapped memory) while band i+1 is computed
 *   6 copy only       those copies alone (for timing)
 *   7 multimem        the GEMM's epilogue writes each tile with multimem.st through an NVLink multicast
 *                     object that all GPUs' C is bound to: the tile crosses NVLink once and the NVSwitch
 *                     replicates it (objects created with the multicast flag)
 * A step whose host-side preparation fails on any rank enqueues nothing on any GPU, returns an
 * error naming the rank, and the object refuses further steps. */
typedef struct cudeep_b200_sharded_gemm* cudeep_b200_sharded_gemm_t;

#define CUDEEP_B200_GATHER_NONE 0
#define CUDEEP_B200_GATHER_AFTER_GEMM 1
#define CUDEEP_B200_GATHER_BANDED 2
#define CUDEEP_B200_GATHER_PEER_STORE 3
#define CUDEEP_B200_GATHER_COLLECTIVE_ONLY 4
#define CUDEEP_B200_GATHER_COPY_ENGINE 5
#define CUDEEP_B200_GATHER_COPY_ONLY 6
#define CUDEEP_B200_GATHER_MULTIMEM 7
#define CUDEEP_B200_SHARDED_DRY_RUN 1        /* flag bits of the `dry_run` argument of the two create calls */
#define CUDEEP_B200_SHARDED_MULTICAST 2
#define CUDEEP_B200_COMM_ID_BYTES 128
#define CUDEEP_B200_MEM_HANDLE_BYTES 64

/* One process drives all of devices[0..n_devices): one host thread and stream pair per device,
 * communicators from ncclCommInitAll.  `dry_run` is a flag word: CUDEEP_B200_SHARDED_DRY_RUN = host logic
 * only, no CUDA or NCCL call; CUDEEP_B200_SHARDED_MULTICAST = C is bound to an NVLink multicast object
 * (gather mode 7; the peer-mapped modes 3, 5 and 6 are then unavailable). */
int cudeep_b200_sharded_gemm_create_local(const int* devices, int n_devices, long long M, int N, int K,
                                          int bands, int comm_sms, int dry_run,
                                          cudeep_b200_sharded_gemm_t* out);
/* This process is rank `rank` of `world` (one process per GPU) and drives `device`. */
int cudeep_b200_sharded_gemm_create_rank(int rank, int world, int device, long long M, int N, int K,
                                         int bands, int comm_sms, int dry_run,
                                         cudeep_b200_sharded_gemm_t* out);
int cudeep_b200_sharded_gemm_destroy(cudeep_b200_sharded_gemm_t g);
/* Rows of A and C owned by `rank`; band `band` of them (band < 0: the whole share). */
int cudeep_b200_sharded_gemm_rows(cudeep_b200_sharded_gemm_t g, int rank, int band, long long* row0,
                                  long long* rows);
/* Device buffers of local rank `local` (0 in the one-process-per-GPU form). */
int cudeep_b200_sharded_gemm_buffers(cudeep_b200_sharded_gemm_t g, int local, float** a_shard, float** b,
                                     float** c);
/* Rows [row0, row0 + rows) of local rank `local`'s copy of C into host memory (blocking). */
int cudeep_b200_sharded_gemm_read_c(cudeep_b200_sharded_gemm_t g, int local, long long row0, long long rows,
                                    float* host_dst);
/* One process per GPU: rank 0 makes a communicator id (128 bytes) and ships it; every rank then
 * calls init_comm with it.  export_c writes the 64-byte handle of this rank's C; open_peers takes
 * all ranks' handles in rank order (world * 64 bytes) and maps the others' C for peer stores. */
int cudeep_b200_sharded_gemm_comm_id(void* id_out);
int cudeep_b200_sharded_gemm_init_comm(cudeep_b200_sharded_gemm_t g, const void* id);
int cudeep_b200_sharded_gemm_export_c(cudeep_b200_sharded_gemm_t g, void* handle_out);
int cudeep_b200_sharded_gemm_open_peers(cudeep_b200_sharded_gemm_t g, const void* handles);
/* One process per GPU with the multicast flag: rank 0 creates the multicast object and receives a file
 * descriptor for it (multicast_fd), hands it to the other processes and closes it; every rank joins
 * (rank 0 with fd = -1); after a barrier between the processes every rank binds.  Before any rank
 * destroys its object all ranks must be idle (a barrier after the last step). */
int cudeep_b200_sharded_gemm_multicast_fd(cudeep_b200_sharded_gemm_t g, int* fd);
int cudeep_b200_sharded_gemm_multicast_join(cudeep_b200_sharded_gemm_t g, int fd);
int cudeep_b200_sharded_gemm_multicast_bind(cudeep_b200_sharded_gemm_t g);
/* Enqueue one step (asynchronous).  One process per GPU: on `stream` (NULL: the object's own);
 * the collective's stream is joined back into it.  One process for all GPUs: `stream` is ignored. */
int cudeep_b200_sharded_gemm_run(cudeep_b200_sharded_gemm_t g, int gather, cudeep_b200_stream_t stream);
int cudeep_b200_sharded_gemm_synchronize(cudeep_b200_sharded_gemm_t g);
/* Mean device time of a step in milliseconds, the slowest local rank's, over `steps` after `warmup`. */
int cudeep_b200_sharded_gemm_time(cudeep_b200_sharded_gemm_t g, int gather, int steps, int warmup,
                                  float* ms_per_step);
/* Steps enqueued so far on local rank `local`; and a test hook that makes `rank`'s host-side
 * preparation fail at the next step. */
int cudeep_b200_sharded_gemm_steps(cudeep_b200_sharded_gemm_t g, int local, long long* steps);
int cudeep_b200_sharded_gemm_inject_failure(cudeep_b200_sharded_gemm_t g, int rank);

#ifdef __cplusplus
}
#endif

#endif /* CUDEEP_B200_H */
