"""Seeded synthetic inputs for the benchmark configurations.

The reference measures on synthetic random matrices (benchmarks/bench_sgemm.cu:24-29);
these generators fix seeds, shapes and distributions so that the GPU path, the
CPU oracle and the rebuilt reference all see the same bytes.

  C1  FP32 SGEMM 512^3, Uniform(-1, 1), seed 0
  C2  TF32 GEMM N^3 for N in {1024, 2048, 4096, 8192}, N(0, 1), seed N
  C3  Linear(4096 -> 16384, GELU) -> Linear(16384 -> 4096) on X[8192, 4096], seed 3;
      weights Kaiming-uniform (bound sqrt(6 / fan_in), python/cuDeep/init.py:44-51),
      biases Uniform(-0.01, 0.01)
  C4  Conv2d 3x3 s1 p1, x[64, 256, 56, 56] ~ N(0, 1), weights Kaiming-normal
      (std sqrt(2 / fan_in), python/cuDeep/init.py:54-61), bias Uniform(-0.01, 0.01), seed 4
  C5  row-sharded GEMM (65536 x 8192 x 8192 and 16384^3), N(0, 1); A is generated per
      row band with seed [5, band] so every rank can make its own shard
"""
from __future__ import annotations

import math

import numpy as np

C2_SIZES = (1024, 2048, 4096, 8192)
C5_SHAPES = ((65536, 8192, 8192), (16384, 16384, 16384))
C5_BAND_ROWS = 1024


def c1_sgemm(n: int = 512):
    rng = np.random.default_rng(0)
    a = rng.uniform(-1.0, 1.0, (n, n)).astype(np.float32)
    b = rng.uniform(-1.0, 1.0, (n, n)).astype(np.float32)
    return a, b


def c2_gemm(n: int):
    rng = np.random.default_rng(n)
    a = rng.standard_normal((n, n), dtype=np.float32)
    b = rng.standard_normal((n, n), dtype=np.float32)
    return a, b


def c3_linear_stack(batch: int = 8192, d_in: int = 4096, d_hidden: int = 16384, d_out: int = 4096):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((batch, d_in), dtype=np.float32)
    bound1 = math.sqrt(6.0 / d_in)
    w1 = rng.uniform(-bound1, bound1, (d_hidden, d_in)).astype(np.float32)
    b1 = rng.uniform(-0.01, 0.01, d_hidden).astype(np.float32)
    bound2 = math.sqrt(6.0 / d_hidden)
    w2 = rng.uniform(-bound2, bound2, (d_out, d_hidden)).astype(np.float32)
    b2 = rng.uniform(-0.01, 0.01, d_out).astype(np.float32)
    return x, w1, b1, w2, b2


def c4_conv(batch: int = 64, channels: int = 256, size: int = 56, out_channels: int = 256, k: int = 3):
    rng = np.random.default_rng(4)
    x = rng.standard_normal((batch, channels, size, size), dtype=np.float32)
    std = math.sqrt(2.0 / (channels * k * k))
    w = (rng.standard_normal((out_channels, channels, k, k), dtype=np.float32) * np.float32(std))
    bias = rng.uniform(-0.01, 0.01, out_channels).astype(np.float32)
    return x, w, bias


def c5_b(n: int, k: int):
    rng = np.random.default_rng([5, 1 << 20])
    return rng.standard_normal((k, n), dtype=np.float32)


def c5_a_band(band: int, k: int, rows: int = C5_BAND_ROWS):
    """Rows [band*rows, (band+1)*rows) of the sharded A."""
    rng = np.random.default_rng([5, band])
    return rng.standard_normal((rows, k), dtype=np.float32)


def c5_a_rows(row0: int, nrows: int, k: int):
    """Rows [row0, row0+nrows) of A; row0 and nrows must be multiples of C5_BAND_ROWS."""
    assert row0 % C5_BAND_ROWS == 0 and nrows % C5_BAND_ROWS == 0
    bands = [c5_a_band(row0 // C5_BAND_ROWS + i, k) for i in range(nrows // C5_BAND_ROWS)]
    return np.concatenate(bands, axis=0)


def gemm_flops(m: int, n: int, k: int) -> float:
    return 2.0 * m * n * k


def conv_flops(batch: int, c_in: int, c_out: int, oh: int, ow: int, kh: int, kw: int) -> float:
    """Direct-convolution work, also when a comparator uses Winograd."""
    return 2.0 * batch * oh * ow * c_out * c_in * kh * kw
