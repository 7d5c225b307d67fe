/* TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * CPU restatement of the arithmetic on cuDeep's dense-contraction path, used
 * only as the checker in tests/, in the smoke test and as the timed CPU
 * baseline of bench.py.  Nothing the library ships may call it.
 *
 * The reference (KevinWeiss1995/cuDeep) has no CPU implementation of this
 * path; each function below restates what the cited CUDA code computes:
 *   gemm        C = A*B, row-major            src/tensor.cu:384-420 (Tensor::matmul),
 *                                             src/kernels/matmul_kernel.cu:1785-1841
 *   linear      y = x*W^T + b                 python/cuDeep/nn.py:110-115
 *   conv2d      NCHW x OIHW cross-correlation src/kernels/conv_kernel.cu:113-159
 *               zero padding, bias once,      (conv2d_forward_naive_kernel), out size
 *               out = (in + 2p - k)/s + 1     src/bindings/module.cpp:326-381
 *   activations sigmoid/tanh-GELU/SiLU        include/cudeep/ptx_intrinsics.cuh:531-554
 *   tf32 input  FP32 words fed to the TF32    src/kernels/matmul_kernel.cu:186-201
 *   truncation  MMA: low 13 mantissa bits     (__float_as_uint of the shared-memory word,
 *               ignored                        no cvt.rna.tf32)
 *
 * Parity pin: the known-answer cases of the reference's own tests
 * (tests/unit/test_matmul.cu:13-68, tests/unit/test_tensor.cu:189-248,
 * tests/unit/test_kernels.cu:324-425, tests/unit/test_tensor_ops.py:210-262,
 * tests/unit/test_nn.py:50-76) are replayed against this file by
 * tests/test_oracle_pins.py.  The reference holds no golden vectors at
 * benchmark sizes; there parity rests on these functions and on the
 * reference's own kernels rebuilt for sm_100 (oracle/Makefile, target ref).
 *
 * Sums are accumulated in double from float inputs, so the result is the
 * exactly rounded product to ~1e-16 relative: the yardstick both the FP32 and
 * the TF32 device paths are measured against.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Value the TF32 tensor-core datapath sees for an FP32 word: mantissa cut to 10 bits. */
static inline float tf32_truncate(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    u &= 0xffffe000u;
    memcpy(&x, &u, 4);
    return x;
}

/* Round-to-nearest-even to 10 mantissa bits (what cvt.rna-style conversion would give;
 * kept to tell the two behaviours apart in tests). */
static inline float tf32_round(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7f800000u) == 0x7f800000u) return x;
    u += 0x00000fffu + ((u >> 13) & 1u);
    u &= 0xffffe000u;
    memcpy(&x, &u, 4);
    return x;
}

void oracle_tf32_truncate(const float* in, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = tf32_truncate(in[i]);
}
void oracle_tf32_round(const float* in, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = tf32_round(in[i]);
}

double oracle_activation(double x, int act) {
    switch (act) {
        case 1: return x > 0.0 ? x : 0.0;                                            /* ReLU */
        case 2: return 0.5 * x * (1.0 + tanh(0.7978845608028654 * (x + 0.044715 * x * x * x))); /* GELU */
        case 3: return x / (1.0 + exp(-x));                                           /* SiLU */
        case 4: return 1.0 / (1.0 + exp(-x));                                         /* sigmoid */
        default: return x;
    }
}

/* C[M,N] (double) = act(A[M,K] * B + bias).  b_is_nk: 0 -> B[K,N], 1 -> B[N,K].
 * bias: NULL, per column (bias_per_row = 0) or per row.  input_mode: 0 exact FP32
 * inputs, 1 inputs truncated to TF32, 2 inputs rounded to TF32. */
void oracle_gemm_f64(const float* a, const float* b, int b_is_nk, double* c, int m, int n, int k,
                     const float* bias, int bias_per_row, int act, int input_mode) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < m; ++i) {
        double* crow = c + (size_t)i * n;
        for (int j = 0; j < n; ++j) crow[j] = 0.0;
        if (!b_is_nk) {
            for (int p = 0; p < k; ++p) {
                float av = a[(size_t)i * k + p];
                if (input_mode == 1) av = tf32_truncate(av); else if (input_mode == 2) av = tf32_round(av);
                const double ad = av;
                const float* brow = b + (size_t)p * n;
                if (input_mode == 0) {
                    for (int j = 0; j < n; ++j) crow[j] += ad * (double)brow[j];
                } else if (input_mode == 1) {
                    for (int j = 0; j < n; ++j) crow[j] += ad * (double)tf32_truncate(brow[j]);
                } else {
                    for (int j = 0; j < n; ++j) crow[j] += ad * (double)tf32_round(brow[j]);
                }
            }
        } else {
            for (int j = 0; j < n; ++j) {
                const float* brow = b + (size_t)j * k;
                const float* arow = a + (size_t)i * k;
                double s = 0.0;
                for (int p = 0; p < k; ++p) {
                    float av = arow[p], bv = brow[p];
                    if (input_mode == 1) { av = tf32_truncate(av); bv = tf32_truncate(bv); }
                    else if (input_mode == 2) { av = tf32_round(av); bv = tf32_round(bv); }
                    s += (double)av * (double)bv;
                }
                crow[j] = s;
            }
        }
        for (int j = 0; j < n; ++j) {
            double v = crow[j];
            if (bias) v += bias_per_row ? (double)bias[i] : (double)bias[j];
            crow[j] = oracle_activation(v, act);
        }
    }
}

/* FP64 inputs (the reference's double path, matmul_kernel.cu:1843-1849). */
void oracle_gemm_f64_in64(const double* a, const double* b, int b_is_nk, double* c, int m, int n, int k,
                          const double* bias, int act) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < m; ++i) {
        for (int j = 0; j < n; ++j) {
            double s = 0.0;
            for (int p = 0; p < k; ++p)
                s += a[(size_t)i * k + p] * (b_is_nk ? b[(size_t)j * k + p] : b[(size_t)p * n + j]);
            if (bias) s += bias[j];
            c[(size_t)i * n + j] = oracle_activation(s, act);
        }
    }
}

/* out[N,OC,OH,OW] (double) = act(conv(x[N,C,H,W], w[OC,C,KH,KW]) + bias[OC]). */
void oracle_conv2d_f64(const float* x, const float* w, const float* bias, double* out, int batch, int c_in,
                       int c_out, int h, int wd, int kh, int kw, int sh, int sw, int ph, int pw, int act,
                       int input_mode) {
    const int oh = (h + 2 * ph - kh) / sh + 1;
    const int ow = (wd + 2 * pw - kw) / sw + 1;
#pragma omp parallel for collapse(2) schedule(static)
    for (int n = 0; n < batch; ++n) {
        for (int oc = 0; oc < c_out; ++oc) {
            double* plane = out + ((size_t)n * c_out + oc) * oh * ow;
            for (int i = 0; i < oh * ow; ++i) plane[i] = 0.0;
            for (int c = 0; c < c_in; ++c) {
                const float* xc = x + ((size_t)n * c_in + c) * h * wd;
                const float* wc = w + ((size_t)oc * c_in + c) * kh * kw;
                for (int r = 0; r < kh; ++r) {
                    for (int s = 0; s < kw; ++s) {
                        float wv = wc[r * kw + s];
                        if (input_mode == 1) wv = tf32_truncate(wv); else if (input_mode == 2) wv = tf32_round(wv);
                        const double wdv = wv;
                        for (int y = 0; y < oh; ++y) {
                            const int iy = y * sh - ph + r;
                            if (iy < 0 || iy >= h) continue;
                            for (int xo = 0; xo < ow; ++xo) {
                                const int ix = xo * sw - pw + s;
                                if (ix < 0 || ix >= wd) continue;
                                float xv = xc[iy * wd + ix];
                                if (input_mode == 1) xv = tf32_truncate(xv); else if (input_mode == 2) xv = tf32_round(xv);
                                plane[y * ow + xo] += wdv * (double)xv;
                            }
                        }
                    }
                }
            }
            const double bv = bias ? (double)bias[oc] : 0.0;
            for (int i = 0; i < oh * ow; ++i) plane[i] = oracle_activation(plane[i] + bv, act);
        }
    }
}

/* ---- float32 CPU baseline (timed by bench.py as the host comparison) -------------------
 * A cache-blocked, multi-threaded FP32 GEMM with FP32 accumulation: the same
 * arithmetic as the device's strict FP32 path, on host cores. */
void oracle_sgemm_f32(const float* a, const float* b, float* c, int m, int n, int k) {
    enum { BI = 64, BP = 256 };
#pragma omp parallel for schedule(dynamic)
    for (int i0 = 0; i0 < m; i0 += BI) {
        const int i1 = i0 + BI < m ? i0 + BI : m;
        for (int i = i0; i < i1; ++i) memset(c + (size_t)i * n, 0, (size_t)n * sizeof(float));
        for (int p0 = 0; p0 < k; p0 += BP) {
            const int p1 = p0 + BP < k ? p0 + BP : k;
            for (int i = i0; i < i1; ++i) {
                float* crow = c + (size_t)i * n;
                for (int p = p0; p < p1; ++p) {
                    const float av = a[(size_t)i * k + p];
                    const float* brow = b + (size_t)p * n;
                    for (int j = 0; j < n; ++j) crow[j] += av * brow[j];
                }
            }
        }
    }
}
