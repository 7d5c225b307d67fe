#!/usr/bin/env python
"""Headline benchmark: TF32 GEMM TFLOP/s at 8192^3, on 1..8 B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one C = A @ B with A[8192, 8192], B[8192, 8192] float32 (N(0,1), seeded),
TF32 tensor-core multiply, FP32 accumulate, through the library's C ABI.  With N > 1
(launched under torchrun, one rank per GPU) the job is the row-sharded GEMM
C[N*8192, 8192] = A[N*8192, 8192] @ B: every rank owns 8192 rows of A and C and a
replica of B, so per-GPU work is fixed (weak scaling) and no collective is on the
data path.  At N = 8 that is the 65536 x 8192 x 8192 sharded configuration.

Prints one JSON line (rank 0).  `value` is device-resident throughput (CUDA events,
max over ranks); `e2e` is the same product through the host-buffer entry point with
pinned host inputs and outputs, copies inside the timed region.  Timed after the headline and
reported in the same line:
  * `value_burst` / `value_sustained`: the headline over a 20-step and a 200-step region (the
    GPU settles under its power cap within a few hundred milliseconds);
  * `parity`: every rank checks sampled rows of its own C against a float64 product on the
    host (the run fails above 5e-3);
  * `c5_strong`: the sharded configurations at FIXED total size - 65536 x 8192 x 8192 and
    16384^3, rows split evenly over the N ranks (cudeep::dist::ShardedGemm, one process per GPU);
  * `with_gather` (N > 1): the optional all-gather of C on 65536 x 8192 x 8192 - compute alone,
    the collective alone, GEMM followed by ncclAllGather, the band-pipelined NCCL form, and the
    fused form in which the GEMM's epilogue stores every tile into all ranks' C.

--impl reference times the reference's own CUDA kernels (cuDeep's matmul sources
rebuilt unmodified for sm_100, oracle/_ref) on the same GPU, inputs and protocol; the
reference has no CPU implementation of this path.  If that library is absent the arm
falls back to the CPU oracle port and says so.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SIZE = 8192
METRIC = "TF32 GEMM TFLOP/s at 8192^3"
FALLBACK_BF16_TFLOPS = 1590.0       # earlier measurement on this pool, used only without MEASURED_PEAKS.json
FALLBACK_BF16_SUSTAINED_TFLOPS = 1400.0
# A timed region longer than this runs under the power cap: its roofline uses the sustained peak.
SUSTAINED_REGION_MS = 100.0
NOMINAL_TF32_TFLOPS = 1125.0        # half the nominal dense bf16 rate of a B200

# DRAM bytes one 8192^3 launch moves (dram__bytes_read.sum + dram__bytes_write.sum from the
# ncu capture summarised in profiles/); None until a capture exists.
NCU_DRAM_BYTES_PER_LAUNCH = 2.54e9
NCU_DRAM_SOURCE = ("a constant, not re-measured by this run: one ncu capture of the 8192^3 launch on 1 GPU "
                   "(profiles/gemm_tf32_8192_umma_kernel.md)")
PARITY_TOL = 5e-3                   # relative Frobenius error of the TF32 path against float64
PARITY_ROWS = 16


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gather", action="store_true",
                    help="with --gpus N > 1: skip the timings of the optional all-gather of C (\"with_gather\")")
    ap.add_argument("--no-c5", action="store_true", help="skip the fixed-size sharded configurations (\"c5_strong\")")
    ap.add_argument("--c5-steps", type=int, default=10)
    ap.add_argument("--suite", action="store_true",
                    help="instead of the headline line, time every benchmark configuration next to "
                         "cuBLAS / cuDNN (through torch) and the reference's kernels; one JSON line each")
    ap.add_argument("--only", default="", help="with --suite: run only the configurations whose name starts "
                                               "with one of these comma-separated tags (C1, C2, C3, C4; "
                                               "B1 matmul backward, B2 conv backward, V1 other conv layers, S1 small-batch Linear, H1 FP16 GEMM; "
                                               "G1, only when named: small GEMMs timed inside a CUDA graph)")
    ap.add_argument("--no-comparators", action="store_true",
                    help="with --suite: time only this library (short runs for profiling)")
    return ap.parse_args()


# ---------------------------------------------------------------------------- clocks

class ClockSampler:
    """Samples SM clock, power and throttle reasons through NVML (read-only) while timing runs."""

    def __init__(self, index: int, period_s: float = 0.01):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---------------------------------------------------------------------------- helpers

def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            d = json.loads(path.read_text())
            return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
        except Exception:
            pass
    return FALLBACK_BF16_TFLOPS, FALLBACK_BF16_SUSTAINED_TFLOPS, "fallback"


def dist_setup(n_gpus: int):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist = dist_mod
    return rank, world, local, dist


def barrier_sync(dist):
    import torch
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(dist, value: float) -> float:
    import torch
    if dist is None:
        return value
    t = torch.tensor([value], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def shard_inputs(rank: int):
    """This rank's 8192 rows of A (seeded per rank) and the replicated B."""
    from cudeep_b200 import workloads
    a, b = workloads.c2_gemm(SIZE)                 # rank 0 runs exactly the 8192^3 benchmark configuration
    if rank != 0:
        a = np.random.default_rng([SIZE, rank]).standard_normal((SIZE, SIZE), dtype=np.float32)
    return a, b


def time_device_steps(launch, steps: int, warmup: int, dist, sampler_index: int):
    """K launches timed with CUDA events on the current stream; returns (seconds, per-launch ms, clocks)."""
    import torch
    for _ in range(warmup):
        launch()
    barrier_sync(dist)
    events = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    with ClockSampler(sampler_index) as clocks:
        events[0].record()
        for i in range(steps):
            launch()
            events[i + 1].record()
        barrier_sync(dist)
    total_ms = events[0].elapsed_time(events[-1])
    per_launch = [events[i].elapsed_time(events[i + 1]) for i in range(steps)]
    return total_ms / 1e3, per_launch, clocks.summary()


def time_e2e_steps(step, steps: int, dist):
    """Host-to-host steps; wall-clock per step is taken between device-synchronised points."""
    import torch
    step()
    barrier_sync(dist)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    barrier_sync(dist)
    wall = time.perf_counter() - t0
    return max(wall, e0.elapsed_time(e1) / 1e3)


def cpu_baseline_leg():
    """The oracle port's host GEMM (NumPy / OpenBLAS sgemm, FP32) on a bounded sample."""
    from oracle import oracle as o
    rows = 2048
    rng = np.random.default_rng(SIZE)
    a = rng.standard_normal((rows, SIZE), dtype=np.float32)
    b = rng.standard_normal((SIZE, SIZE), dtype=np.float32)
    o.cpu_sgemm(a[:256], b)
    best = float("inf")
    spent = 0.0
    while spent < 12.0:
        t0 = time.perf_counter()
        o.cpu_sgemm(a, b)
        dt = time.perf_counter() - t0
        best = min(best, dt)
        spent += dt
    return {"value": 2.0 * rows * SIZE * SIZE / best / 1e12, "unit": "TFLOP/s", "cores": o.cpu_threads(),
            "kind": "port",
            "sample": f"rows 0..{rows - 1} of the 8192^3 product, FP32 sgemm (NumPy/OpenBLAS), best of ~12 s"}



# ---------------------------------------------------------------------------- parity

def all_reduce_max(dist, value: float) -> float:
    return max_over_ranks(dist, value)


def headline_parity(a_np, b_np, c, dist):
    """Every rank: PARITY_ROWS sampled rows (all columns) of its own C against the float64 product of
    its own A rows and B, on the host, outside any timed region.  The worst rank's figures."""
    import torch
    from oracle import oracle as o
    rank = dist.get_rank() if dist is not None else 0
    rows = np.sort(np.random.default_rng([77, rank]).choice(a_np.shape[0], size=PARITY_ROWS, replace=False))
    got = c[torch.from_numpy(rows).cuda()].cpu().numpy()
    err = o.rel_frobenius(got, o.gemm(a_np[rows], b_np))
    model = o.rel_frobenius(got, o.gemm(a_np[rows], b_np, input_mode=o.INPUT_TF32_TRUNC))
    err, model = all_reduce_max(dist, float(err)), all_reduce_max(dist, float(model))
    if not (err <= PARITY_TOL):
        raise RuntimeError(f"parity: relative error {err} of the 8192^3 product exceeds {PARITY_TOL}")
    return {"max_rel_err": err, "max_rel_err_vs_tf32_truncated_operands": model, "rows_per_rank": PARITY_ROWS,
            "tolerance": PARITY_TOL, "checked": "sampled rows of every rank's C against a float64 host product"}


# ---------------------------------------------------------------------------- C5: fixed-size sharded GEMM

def run_c5(args, rank, world, local, dist, gather: bool):
    """65536 x 8192 x 8192 and 16384^3 with the rows split evenly over the ranks (strong scaling),
    through cudeep::dist::ShardedGemm in its one-process-per-GPU form; on the first shape also the
    optional all-gather of C in all its forms."""
    import torch
    from cudeep_b200 import workloads
    from cudeep_b200 import sharded as sh
    from oracle import oracle as o
    # A stream of its own (not the legacy default stream): the steps are enqueued on it, the
    # collective's stream is joined back into it, and the timing events are recorded on it.
    side = torch.cuda.Stream()
    stream = side.cuda_stream
    out = {"strong": [], "with_gather": None}

    def exchange_id(x):
        box = [x]
        dist.broadcast_object_list(box, src=0)
        return box[0]

    def exchange_handles(x):
        box = [None] * world
        dist.all_gather_object(box, x)
        return box

    def timed(g, mode, steps):
        with torch.cuda.stream(side):
            seconds, _, _ = time_device_steps(lambda: g.run(mode, stream), steps, 3, dist, local)
        return max_over_ranks(dist, seconds) / steps * 1e3

    def check_rows(g, rows_global, b_np, k, what):
        """float64 check of the given global rows of this rank's copy of C."""
        worst = 0.0
        for r in rows_global:
            band = int(r) // workloads.C5_BAND_ROWS
            a_row = workloads.c5_a_band(band, k)[int(r) % workloads.C5_BAND_ROWS][None, :]
            got = g.read_c(0, int(r), 1)
            worst = max(worst, float(o.rel_frobenius(got, o.gemm(a_row, b_np))))
        worst = all_reduce_max(dist, worst)
        if not (worst <= PARITY_TOL):
            raise RuntimeError(f"parity ({what}): relative error {worst} exceeds {PARITY_TOL}")
        return worst

    for m, n, k in workloads.C5_SHAPES:
        if m % (world * workloads.C5_BAND_ROWS) != 0:
            continue
        # Row bands of the pipelined gather forms: eight where a band still holds several waves of tiles
        # (2048 rows or more), else four.
        bands = 8 if m // world // 8 >= 2048 else 4
        g = sh.ShardedGemm.rank(rank, world, local, m, n, k, bands=bands)
        try:
            if world > 1:
                g.connect(exchange_id, exchange_handles)
            mine = g.rows_of(rank)
            b_np = workloads.c5_b(n, k)

            def load_operands(obj):
                obj.set_b(b_np)
                a_ptr = obj.buffers(0)[0]
                for i in range(mine.rows // workloads.C5_BAND_ROWS):   # band by band: no multi-GB host copy of A
                    band = workloads.c5_a_band(mine.row0 // workloads.C5_BAND_ROWS + i, k)
                    obj._h2d(a_ptr + i * workloads.C5_BAND_ROWS * k * 4, band)

            load_operands(g)
            ms = timed(g, sh.GATHER_NONE, args.c5_steps)
            flops = 2.0 * m * n * k
            rng = np.random.default_rng([55, rank, m])
            own = mine.row0 + np.sort(rng.choice(mine.rows, size=min(PARITY_ROWS, mine.rows), replace=False))
            err = check_rows(g, own, b_np, k, f"C5 {m}x{n}x{k}, own rows")
            out["strong"].append({
                "workload": f"C[{m},{n}] = A[{m},{k}] @ B[{k},{n}], {mine.rows} rows per GPU", "flop_per_step": flops,
                "rows_per_gpu": mine.rows, "ms_per_step": ms, "tflops": flops / (ms * 1e-3) / 1e12,
                "tflops_per_gpu": flops / (ms * 1e-3) / 1e12 / world, "steps": args.c5_steps,
                "scaling": "strong", "parity_max_rel_err": err})
            if gather and out["with_gather"] is None:
                t_compute = ms
                t_gather = timed(g, sh.GATHER_COLLECTIVE_ONLY, args.c5_steps)
                t_after = timed(g, sh.GATHER_AFTER_GEMM, args.c5_steps)
                t_banded = timed(g, sh.GATHER_BANDED, args.c5_steps)
                t_fused = timed(g, sh.GATHER_PEER_STORE, args.c5_steps)
                t_copy = timed(g, sh.GATHER_COPY_ENGINE, args.c5_steps)
                # the fused form's result, checked on rows this rank did NOT compute
                barrier_sync(dist)
                others = [r for r in range(world) if r != rank]
                foreign = []
                for j in range(PARITY_ROWS):
                    s_ = g.rows_of(others[j % len(others)])
                    foreign.append(s_.row0 + int(rng.integers(s_.rows)))
                err_fused = check_rows(g, foreign, b_np, k, "gathered C, peer-store form, rows of other ranks")
                barrier_sync(dist)
                g.run(sh.GATHER_BANDED, stream)
                barrier_sync(dist)
                err_banded = check_rows(g, foreign, b_np, k, "gathered C, banded NCCL form, rows of other ranks")
                barrier_sync(dist)
                g.run(sh.GATHER_COPY_ENGINE, stream)
                barrier_sync(dist)
                err_copy = check_rows(g, foreign, b_np, k, "gathered C, copy-engine form, rows of other ranks")
                # The same product with C bound to an NVLink multicast object: the epilogue writes each tile
                # once with multimem.st and the switch replicates it.
                t_multimem, err_multimem, multimem_note = None, None, None
                try:
                    gm = sh.ShardedGemm.rank(rank, world, local, m, n, k, bands=bands, multicast=True)
                except Exception as e:                      # no multicast support: the same on every rank
                    gm, multimem_note = None, str(e)
                if gm is not None:
                    try:
                        import tempfile
                        path = exchange_id(os.path.join(tempfile.gettempdir(), f"cudeep_mc_{os.getpid()}.sock")
                                           if rank == 0 else None)
                        gm.connect_multicast(sh.unix_socket_fd_sharing(rank, world, path), lambda: barrier_sync(dist))
                        load_operands(gm)
                        t_multimem = timed(gm, sh.GATHER_MULTIMEM, args.c5_steps)
                        barrier_sync(dist)
                        err_multimem = check_rows(gm, foreign, b_np, k, "gathered C, multimem form, rows of other ranks")
                    finally:
                        barrier_sync(dist)        # nobody unbinds while another rank may still write through the switch
                        gm.close()
                longer = max(t_compute, t_gather)
                forms = {"fused peer-store epilogue": t_fused, "banded NCCL": t_banded,
                         "banded copy-engine pushes": t_copy}
                if t_multimem is not None:
                    forms["fused multimem epilogue (NVSwitch multicast)"] = t_multimem
                best_form = min(forms, key=forms.get)
                best = forms[best_form]
                out["with_gather"] = {
                    "workload": f"C[{m},{n}] gathered on every GPU ({(world - 1) * mine.rows * n * 4} bytes received per GPU)",
                    "t_compute_ms": t_compute, "t_gather_alone_ms": t_gather,
                    "t_gemm_then_ncclAllGather_ms": t_after, "t_banded_nccl_ms": t_banded,
                    "t_fused_peer_store_ms": t_fused, "t_banded_copy_engine_ms": t_copy,
                    "t_fused_multimem_ms": t_multimem, "t_both_ms": best,
                    "form": best_form,
                    "overlap": best / longer, "overlap_banded_nccl": t_banded / longer,
                    "overlap_fused_peer_store": t_fused / longer, "overlap_banded_copy_engine": t_copy / longer,
                    "overlap_fused_multimem": (t_multimem / longer) if t_multimem is not None else None,
                    "multimem_unavailable": multimem_note,
                    "plain_sum_ms": t_compute + t_gather,
                    "tflops_with_gather": flops / (best * 1e-3) / 1e12,
                    "parity_max_rel_err_fused": err_fused, "parity_max_rel_err_banded": err_banded,
                    "parity_max_rel_err_copy_engine": err_copy, "parity_max_rel_err_multimem": err_multimem,
                    "steps": args.c5_steps, "bands": bands,
                    "note": "overlap = step time / max(compute alone, collective alone); 1.0 = the shorter leg is fully hidden"}
            barrier_sync(dist)
        finally:
            g.close()
    return out

# ---------------------------------------------------------------------------- arms

def run_ours(args):
    import torch
    from cudeep_b200 import _lib
    lib = _lib.load()
    rank, world, local, dist = dist_setup(args.gpus)
    a_np, b_np = shard_inputs(rank)
    a = torch.from_numpy(a_np).cuda()
    b = torch.from_numpy(b_np).cuda()
    c = torch.empty((SIZE, SIZE), device="cuda", dtype=torch.float32)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    pa, pb, pc = (ctypes.c_void_p(t.data_ptr()) for t in (a, b, c))

    def launch():
        rc = lib.cudeep_b200_matmul_f32(pa, pb, pc, SIZE, SIZE, SIZE, stream)
        if rc != 0:
            raise RuntimeError(lib.cudeep_b200_last_error().decode())

    seconds, per_launch, clocks = time_device_steps(launch, args.steps, args.warmup, dist, local)
    status = _lib.device_status(True)
    if status != 0:
        raise RuntimeError(f"kernel status word {status}: a pipeline wait was abandoned")
    seconds = max_over_ranks(dist, seconds)
    flops_step = 2.0 * SIZE ** 3 * world
    value = flops_step * args.steps / seconds / 1e12

    # end to end: pinned host buffers in, pinned host buffer out, through the host entry point.
    # The buffers are allocated (and the copies enqueued) from a thread that runs on the GPU's NUMA
    # node, so their pages sit on the socket the GPU's host link hangs off (a thread's CPU affinity,
    # restored afterwards; nothing about the GPU changes).
    from cudeep_b200 import hostmem
    with hostmem.near_gpu(local) as placement:
        ha = torch.from_numpy(a_np).pin_memory()
        hb = torch.from_numpy(b_np).pin_memory()
        hc = torch.empty((SIZE, SIZE), dtype=torch.float32).pin_memory()
        pha, phb, phc = (ctypes.c_void_p(t.data_ptr()) for t in (ha, hb, hc))

        def e2e_step():
            rc = lib.cudeep_b200_matmul_host_f32(pha, phb, phc, SIZE, SIZE, SIZE, 0)
            if rc != 0:
                raise RuntimeError(lib.cudeep_b200_last_error().decode())

        e2e_seconds = max_over_ranks(dist, time_e2e_steps(e2e_step, args.e2e_steps, dist))
    e2e_value = flops_step * args.e2e_steps / e2e_seconds / 1e12
    checksum = float(hc[0, :8].sum())      # the step's result is read on the host

    # the headline again over a short and a long region: burst and power-capped figures side by side
    other_steps = 200 if args.steps < 100 else 20
    other_seconds, _, _ = time_device_steps(launch, other_steps, 3, dist, local)
    other_seconds = max_over_ranks(dist, other_seconds)
    other_value = flops_step * other_steps / other_seconds / 1e12
    burst, sustained = (value, other_value) if args.steps < 100 else (other_value, value)

    parity = headline_parity(a_np, b_np, c, dist)
    del a, b, c, ha, hb, hc
    torch.cuda.empty_cache()

    c5 = None if args.no_c5 else run_c5(args, rank, world, local, dist, gather=(world > 1 and not args.no_gather))
    status = _lib.device_status(True)
    if status != 0:
        raise RuntimeError(f"kernel status word {status}: a pipeline wait was abandoned")
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    bf16_burst, bf16_sustained, peak_kind = measured_peaks()
    kernel_ms = float(np.mean(per_launch))
    achieved = 2.0 * SIZE ** 3 / (kernel_ms * 1e-3) / 1e12
    long_region = seconds * 1e3 >= SUSTAINED_REGION_MS
    bf16_peak = bf16_sustained if long_region else bf16_burst
    peak = bf16_peak / 2.0
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": seconds / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "tf32 multiply, f32 accumulate", "data": "synthetic",
        "config": {"workload": f"C = A[{SIZE * world},{SIZE}] @ B[{SIZE},{SIZE}] float32 N(0,1), "
                               f"{SIZE} rows of A and C per GPU, B replicated",
                   "flop_per_step": flops_step, "l2": "operands and result (805 MB per GPU) exceed the 126 MB L2; no flush",
                   "parallelism": f"rows sharded over {world} GPU(s), no data-path collective"},
        "pct_of_nominal_tf32_peak": 100.0 * value / world / NOMINAL_TF32_TFLOPS,
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": 2 * SIZE * SIZE * 4 * world,
                "d2h_bytes_per_step": SIZE * SIZE * 4 * world, "steps": args.e2e_steps,
                "host_placement": {"numa_node": placement["numa_node"], "bound": placement["bound"],
                                   "cpus": placement["cpus"]},
                "result_probe": checksum},
        "value_burst": burst, "value_sustained": sustained,
        "burst_sustained_note": "same launch over a 20-step region and a 200-step region; `value` is the one with --steps",
        "parity": parity,
        "gpu_launches": args.steps,
        "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                     "frac": achieved / peak,
                     "traffic": NCU_DRAM_BYTES_PER_LAUNCH,
                     "traffic_source": NCU_DRAM_SOURCE,
                     "peak_source": f"{peak_kind} dense bf16 cuBLAS {'sustained' if long_region else 'burst'} "
                                    f"({bf16_peak} TFLOP/s) / 2: TF32 issues at half the bf16 rate; the timed "
                                    f"region lasted {seconds * 1e3:.0f} ms (sustained figure from {SUSTAINED_REGION_MS:.0f} ms on)",
                     "frac_of_burst_peak": achieved / (bf16_burst / 2.0),
                     "kernel": "umma_tf32_kernel", "kernel_ms": kernel_ms},
    }
    if c5 is not None:
        line["c5_strong"] = c5["strong"]
        if c5.get("with_gather") is not None:
            line["with_gather"] = c5["with_gather"]
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_leg()
    print(json.dumps(line), flush=True)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return                                   # the reference is single-device: rank 0 alone measures
    from oracle import oracle as o
    flops_step = 2.0 * SIZE ** 3
    base = {"impl": "reference", "metric": METRIC, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "data": "synthetic"}
    use_gpu = o.REF_LIB_PATH.exists()
    if use_gpu:
        try:
            import torch
            use_gpu = torch.cuda.is_available()
        except Exception:
            use_gpu = False
    if use_gpu:
        import torch
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        ref = ctypes.CDLL(str(o.REF_LIB_PATH))
        a_np, b_np = shard_inputs(0)
        a, b = torch.from_numpy(a_np).cuda(), torch.from_numpy(b_np).cuda()
        c = torch.empty((SIZE, SIZE), device="cuda", dtype=torch.float32)
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        pa, pb, pc = (ctypes.c_void_p(t.data_ptr()) for t in (a, b, c))

        def launch():
            if ref.cudeep_ref_matmul_f32(pa, pb, pc, SIZE, SIZE, SIZE, stream) != 0:
                raise RuntimeError("reference launcher failed")

        steps = min(args.steps, 50)
        seconds, per_launch, clocks = time_device_steps(launch, steps, min(args.warmup, 5), None, 0)
        value = flops_step * steps / seconds / 1e12
        ha, hb = torch.from_numpy(a_np).pin_memory(), torch.from_numpy(b_np).pin_memory()
        hc = torch.empty((SIZE, SIZE), dtype=torch.float32).pin_memory()

        def e2e_step():                            # from_numpy -> matmul -> numpy, as the reference's Python API does
            a.copy_(ha, non_blocking=True)
            b.copy_(hb, non_blocking=True)
            launch()
            hc.copy_(c, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        e2e_seconds = time_e2e_steps(e2e_step, args.e2e_steps, None)
        line = dict(base, steps=steps, value=value, ms_per_step=seconds / steps * 1e3,
                    dtype="tf32 multiply, f32 accumulate",
                    config={"workload": f"C = A[{SIZE},{SIZE}] @ B[{SIZE},{SIZE}] float32 N(0,1)",
                            "device": "the reference's CUDA kernels (mma.sync TF32) on the same B200",
                            "flop_per_step": flops_step},
                    e2e={"value": flops_step * args.e2e_steps / e2e_seconds / 1e12, "unit": "TFLOP/s",
                         "h2d_bytes_per_step": 2 * SIZE * SIZE * 4, "d2h_bytes_per_step": SIZE * SIZE * 4},
                    cpu_baseline={"value": value, "unit": "TFLOP/s", "cores": 0, "kind": "reference",
                                  "sample": "not a CPU run: the reference has no CPU implementation of this path; "
                                            "its own GPU kernels were timed on the full workload"},
                    gpu_launches=steps, clocks=clocks)
    else:
        cpu = cpu_baseline_leg()
        line = dict(base, value=cpu["value"], ms_per_step=flops_step / (cpu["value"] * 1e12) * 1e3,
                    dtype="f32", config={"workload": f"C = A[{SIZE},{SIZE}] @ B[{SIZE},{SIZE}] float32 N(0,1)",
                                         "device": "host CPU (oracle port); reference kernels not built",
                                         "flop_per_step": flops_step},
                    cpu_baseline=cpu,
                    e2e={"value": cpu["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------- suite

def run_suite(args):
    """All single-GPU configurations side by side.  Device-resident inputs, CUDA events, an L2
    flush before every timed launch (several inputs are smaller than the 126 MB L2)."""
    import torch
    import torch.nn.functional as F
    from cudeep_b200 import _lib, workloads
    from oracle import oracle as o
    lib = _lib.load()
    torch.cuda.set_device(0)
    ref = ctypes.CDLL(str(o.REF_LIB_PATH)) if o.REF_LIB_PATH.exists() else None
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    flush = torch.empty(256 * 1024 * 1024 // 4, device="cuda")
    P = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())

    def timed(fn, iters, cmp=False):
        if cmp and args.no_comparators:
            return None
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return float(np.median(ts)), float(np.min(ts))

    def emit(name, flops, rows, **extra):
        line = {"suite": name, "gflop": flops / 1e9}
        for key, (med, mn) in rows.items():
            line[key] = {"ms_median": med, "ms_min": mn, "tflops": flops / (med * 1e-3) / 1e12}
        for key in rows:
            if key != "ours":
                line[f"ours_over_{key}"] = rows[key][0] / rows["ours"][0]
        rows = dict(rows)
        line.update(extra)
        print(json.dumps(line), flush=True)

    def ok(rc):
        if rc != 0:
            raise RuntimeError(lib.cudeep_b200_last_error().decode())

    only = [t.strip() for t in args.only.split(",") if t.strip()]
    want = lambda tag: not only or tag in only
    if args.no_comparators:
        ref = None

    def trim(rows):
        return {k: v for k, v in rows.items() if v is not None}

    # C1: strict FP32 512^3
    if want("C1"):
        run_c1(lib, ref, timed, emit, ok, P, stream, trim)
    if want("C2"):
        run_c2(lib, ref, timed, emit, ok, P, stream, trim)
    if want("C3"):
        run_c3(lib, ref, timed, emit, ok, P, stream, trim)
    if want("C4"):
        run_c4(lib, ref, timed, emit, ok, P, stream, trim)
    if want("B1"):
        run_b1(lib, ref, timed, emit, ok, P, stream, trim)
    if want("B2"):
        run_b2(lib, ref, timed, emit, ok, P, stream, trim)
    if want("V1"):
        run_v1(lib, timed, emit, ok, P, stream, trim)
    if want("S1"):
        run_s1(lib, ref, timed, emit, ok, P, stream, trim)
    if want("H1"):
        run_h1(lib, timed, emit, ok, P, stream, trim)
    if "G1" in only:            # only on request: a different timing protocol
        run_g1(lib, emit, ok, P)
    status = _lib.device_status(True)
    if status != 0:
        raise RuntimeError(f"kernel status word {status}")


def run_c1(lib, ref, timed, emit, ok, P, stream, trim):
    import torch
    from cudeep_b200 import workloads
    a_np, b_np = workloads.c1_sgemm()
    a, b = torch.from_numpy(a_np).cuda(), torch.from_numpy(b_np).cuda()
    c = torch.empty((512, 512), device="cuda")
    rows = {"ours": timed(lambda: ok(lib.cudeep_b200_matmul_f32_strict(P(a), P(b), P(c), 512, 512, 512, stream)), 50)}
    torch.backends.cuda.matmul.allow_tf32 = False
    rows["cublas_fp32"] = timed(lambda: torch.matmul(a, b, out=c), 50, cmp=True)
    if ref is not None:
        rows["reference"] = timed(lambda: ref.cudeep_ref_matmul_f32_strict(P(a), P(b), P(c), 512, 512, 512, stream), 50, cmp=True)
    emit("C1 FP32 SGEMM 512^3", 2.0 * 512 ** 3, trim(rows))


def run_c2(lib, ref, timed, emit, ok, P, stream, trim):
    import torch
    from cudeep_b200 import workloads
    torch.backends.cuda.matmul.allow_tf32 = True
    for n in workloads.C2_SIZES:
        a = torch.randn((n, n), device="cuda")
        b = torch.randn((n, n), device="cuda")
        c = torch.empty((n, n), device="cuda")
        iters = 30 if n <= 4096 else 15
        rows = {"ours": timed(lambda: ok(lib.cudeep_b200_matmul_f32(P(a), P(b), P(c), n, n, n, stream)), iters),
                "cublas_tf32": timed(lambda: torch.matmul(a, b, out=c), iters, cmp=True)}
        if ref is not None:
            rows["reference"] = timed(lambda: ref.cudeep_ref_matmul_f32(P(a), P(b), P(c), n, n, n, stream), max(3, iters // 5), cmp=True)
        emit(f"C2 TF32 GEMM {n}^3", 2.0 * n ** 3, trim(rows))


def run_c3(lib, ref, timed, emit, ok, P, stream, trim):
    """Linear(4096 -> 16384, GELU) -> Linear(16384 -> 4096), batch 8192."""
    import torch
    import torch.nn.functional as F
    torch.backends.cuda.matmul.allow_tf32 = True
    m, d_in, d_h, d_out = 8192, 4096, 16384, 4096
    x = torch.randn((m, d_in), device="cuda")
    w1 = (torch.rand((d_h, d_in), device="cuda") * 2 - 1) * (6.0 / d_in) ** 0.5
    b1 = (torch.rand(d_h, device="cuda") * 2 - 1) * 0.01
    w2 = (torch.rand((d_out, d_h), device="cuda") * 2 - 1) * (6.0 / d_h) ** 0.5
    b2 = (torch.rand(d_out, device="cuda") * 2 - 1) * 0.01
    h = torch.empty((m, d_h), device="cuda")
    y = torch.empty((m, d_out), device="cuda")

    def ours_c3():
        ok(lib.cudeep_b200_linear_forward_f32(P(x), P(w1), P(b1), P(h), m, d_h, d_in, 2, stream))
        ok(lib.cudeep_b200_linear_forward_f32(P(h), P(w2), P(b2), P(y), m, d_out, d_h, 0, stream))

    def torch_c3():
        F.linear(F.gelu(F.linear(x, w1, b1), approximate="tanh"), w2, b2)

    def lt_c3():        # cuBLASLt with the bias + GELU epilogue fused into the first GEMM
        torch.addmm(b2, torch._addmm_activation(b1, x, w1.t(), use_gelu=True), w2.t())

    rows = {"ours": timed(ours_c3, 8), "cublas_tf32_torch": timed(torch_c3, 8, cmp=True)}
    if hasattr(torch, "_addmm_activation"):
        rows["cublaslt_fused_epilogue_torch"] = timed(lt_c3, 8, cmp=True)
    if ref is not None:
        w1t, w2t = w1.t().contiguous(), w2.t().contiguous()

        def ref_c3():       # the reference's two GEMMs only: its transpose copies, bias and GELU passes are not counted
            ref.cudeep_ref_matmul_f32(P(x), P(w1t), P(h), m, d_h, d_in, stream)
            ref.cudeep_ref_matmul_f32(P(h), P(w2t), P(y), m, d_out, d_h, stream)

        rows["reference_gemms_only"] = timed(ref_c3, 3, cmp=True)
    emit("C3 Linear 8192x4096 -> 16384 (GELU) -> 4096", 2.0 * m * d_in * d_h * 2, trim(rows))


def run_c4(lib, ref, timed, emit, ok, P, stream, trim):
    """conv 3x3, 64 x 256 x 56 x 56 -> 256, bias + ReLU."""
    import torch
    import torch.nn.functional as F
    from cudeep_b200 import workloads
    nb, ch, size, oc = 64, 256, 56, 256
    xc = torch.randn((nb, ch, size, size), device="cuda")
    wc = torch.randn((oc, ch, 3, 3), device="cuda") * (2.0 / (ch * 9)) ** 0.5
    bc = (torch.rand(oc, device="cuda") * 2 - 1) * 0.01
    yc = torch.empty((nb, oc, size, size), device="cuda")
    torch.backends.cudnn.allow_tf32 = True
    torch.backends.cudnn.benchmark = True
    rows = {"ours": timed(lambda: ok(lib.cudeep_b200_conv2d_forward_fused_f32(
        P(xc), P(wc), P(bc), P(yc), nb, ch, oc, size, size, 3, 3, 1, 1, 1, 1, 1, stream)), 15),
            "cudnn_tf32_torch": timed(lambda: F.relu(F.conv2d(xc, wc, bc, padding=1)), 15, cmp=True)}
    xl = xc.contiguous(memory_format=torch.channels_last)
    rows["cudnn_tf32_torch_nhwc_input"] = timed(lambda: F.relu(F.conv2d(xl, wc, bc, padding=1)), 15, cmp=True)
    xh = xc.permute(0, 2, 3, 1).contiguous()           # [N, H, W, C] for the channels-last entry point
    rows["ours_nhwc_input"] = timed(lambda: ok(lib.cudeep_b200_conv2d_forward_fused_nhwc_f32(
        P(xh), P(wc), P(bc), P(yc), nb, ch, oc, size, size, 3, 3, 1, 1, 1, 1, 1, stream)), 15)
    if ref is not None:
        rows["reference_no_relu"] = timed(lambda: ref.cudeep_ref_conv2d_forward_f32(
            P(xc), P(wc), P(bc), P(yc), nb, ch, oc, size, size, 3, 3, 1, 1, 1, 1, stream), 5, cmp=True)
    emit("C4 conv 3x3 64x256x56x56 -> 256, bias + ReLU", workloads.conv_flops(nb, ch, oc, size, size, 3, 3),
         trim(rows))


def run_b1(lib, ref, timed, emit, ok, P, stream, trim):
    """The two products of matmul's backward pass at 4096^3, operands consumed as stored:
    dA = dC B^T (NT) and dB = A^T dC (TN)."""
    import torch
    torch.backends.cuda.matmul.allow_tf32 = True
    n = 4096
    a = torch.randn((n, n), device="cuda")
    b = torch.randn((n, n), device="cuda")
    dc = torch.randn((n, n), device="cuda")
    out = torch.empty((n, n), device="cuda")
    rows = {"ours": timed(lambda: ok(lib.cudeep_b200_matmul_nt_f32(P(dc), P(b), P(out), n, n, n, stream)), 20),
            "cublas_tf32": timed(lambda: torch.matmul(dc, b.t(), out=out), 20, cmp=True)}
    emit(f"B1 matmul backward dA = dC B^T {n}^3", 2.0 * n ** 3, trim(rows))
    rows = {"ours": timed(lambda: ok(lib.cudeep_b200_matmul_tn_f32(P(a), P(dc), P(out), n, n, n, stream)), 20),
            "cublas_tf32": timed(lambda: torch.matmul(a.t(), dc, out=out), 20, cmp=True)}
    emit(f"B1 matmul backward dB = A^T dC {n}^3", 2.0 * n ** 3, trim(rows))


def run_b2(lib, ref, timed, emit, ok, P, stream, trim):
    """Backward of the C4 layer: grad_input and grad_weight."""
    import torch
    from cudeep_b200 import workloads
    nb, ch, size, oc = 64, 256, 56, 256
    x = torch.randn((nb, ch, size, size), device="cuda")
    w = torch.randn((oc, ch, 3, 3), device="cuda") * (2.0 / (ch * 9)) ** 0.5
    dy = torch.randn((nb, oc, size, size), device="cuda")
    dx = torch.empty_like(x)
    dw = torch.empty_like(w)
    torch.backends.cudnn.allow_tf32 = True
    torch.backends.cudnn.benchmark = True
    flops = workloads.conv_flops(nb, ch, oc, size, size, 3, 3)
    geom = (nb, ch, oc, size, size, 3, 3, 1, 1, 1, 1)
    rows = {"ours": timed(lambda: ok(lib.cudeep_b200_conv2d_backward_data_f32(P(dy), P(w), P(dx), *geom, stream)), 15),
            "cudnn_tf32_torch": timed(lambda: torch.nn.grad.conv2d_input(x.shape, w, dy, padding=1), 15, cmp=True)}
    emit("B2 conv backward grad_input, C4 layer", flops, trim(rows))
    rows = {"ours": timed(lambda: ok(lib.cudeep_b200_conv2d_backward_weight_f32(P(dy), P(x), P(dw), *geom, stream)), 15),
            "cudnn_tf32_torch": timed(lambda: torch.nn.grad.conv2d_weight(x, w.shape, dy, padding=1), 15, cmp=True)}
    emit("B2 conv backward grad_weight, C4 layer", flops, trim(rows))


def run_v1(lib, timed, emit, ok, P, stream, trim):
    """Convolution layers of a ResNet-style network other than C4, batch 64: a 7 x 7 stride-2 stem over
    three channels, the 3 x 3 layers of the 56 x 56, 28 x 28, 14 x 14 and 7 x 7 feature maps and a stride-2
    down-sampling layer; forward
    (bias, no activation), grad_input and grad_weight against cuDNN (TF32) through torch."""
    import torch
    import torch.nn.functional as F
    from cudeep_b200 import workloads
    torch.backends.cudnn.allow_tf32 = True
    torch.backends.cudnn.benchmark = True
    nb = 64
    for ch, size, oc, k, s, p in [(3, 224, 64, 7, 2, 3), (64, 56, 64, 3, 1, 1), (64, 56, 128, 3, 2, 1),
                                  (128, 28, 128, 3, 1, 1), (256, 14, 256, 3, 1, 1), (512, 7, 512, 3, 1, 1)]:
        out = (size + 2 * p - k) // s + 1
        x = torch.randn((nb, ch, size, size), device="cuda")
        w = torch.randn((oc, ch, k, k), device="cuda") * (2.0 / (ch * k * k)) ** 0.5
        b = (torch.rand(oc, device="cuda") * 2 - 1) * 0.01
        y = torch.empty((nb, oc, out, out), device="cuda")
        dy = torch.randn((nb, oc, out, out), device="cuda")
        dx, dw = torch.empty_like(x), torch.empty_like(w)
        geom = (nb, ch, oc, size, size, k, k, s, s, p, p)
        flops = workloads.conv_flops(nb, ch, oc, out, out, k, k)
        tag = f"{nb}x{ch}x{size}x{size} -> {oc}, {k}x{k} stride {s}"
        rows = {"ours": timed(lambda: ok(lib.cudeep_b200_conv2d_forward_f32(P(x), P(w), P(b), P(y), *geom, stream)), 15),
                "cudnn_tf32_torch": timed(lambda: F.conv2d(x, w, b, stride=s, padding=p), 15, cmp=True)}
        emit(f"V1 conv forward {tag}", flops, trim(rows))
        if ch >= 32:        # a stem's input is the images: no network asks for their gradient
            rows = {"ours": timed(lambda: ok(lib.cudeep_b200_conv2d_backward_data_f32(P(dy), P(w), P(dx), *geom, stream)), 15),
                    "cudnn_tf32_torch": timed(lambda: torch.nn.grad.conv2d_input(x.shape, w, dy, stride=s, padding=p), 15, cmp=True)}
            emit(f"V1 conv grad_input {tag}", flops, trim(rows))
        rows = {"ours": timed(lambda: ok(lib.cudeep_b200_conv2d_backward_weight_f32(P(dy), P(x), P(dw), *geom, stream)), 15),
                "cudnn_tf32_torch": timed(lambda: torch.nn.grad.conv2d_weight(x, w.shape, dy, stride=s, padding=p), 15, cmp=True)}
        emit(f"V1 conv grad_weight {tag}", flops, trim(rows))


def run_s1(lib, ref, timed, emit, ok, P, stream, trim):
    """Linear layers with a small batch (few output tiles, long K): bias + GELU fused, W as stored."""
    import torch
    import torch.nn.functional as F
    torch.backends.cuda.matmul.allow_tf32 = True
    for m, n, k in [(128, 4096, 4096), (256, 1024, 8192), (512, 512, 4096), (1024, 1024, 4096)]:
        x = torch.randn((m, k), device="cuda")
        w = torch.randn((n, k), device="cuda") * (1.0 / k) ** 0.5
        bias = torch.randn(n, device="cuda") * 0.01
        y = torch.empty((m, n), device="cuda")
        rows = {"ours": timed(lambda: ok(lib.cudeep_b200_linear_forward_f32(P(x), P(w), P(bias), P(y), m, n, k, 2, stream)), 30),
                "cublas_tf32_torch": timed(lambda: F.gelu(F.linear(x, w, bias), approximate="tanh"), 30, cmp=True)}
        if hasattr(torch, "_addmm_activation"):
            rows["cublaslt_fused_epilogue_torch"] = timed(
                lambda: torch._addmm_activation(bias, x, w.t(), use_gelu=True), 30, cmp=True)
        emit(f"S1 Linear + GELU, batch {m}: {k} -> {n}", 2.0 * m * n * k, trim(rows))


def run_h1(lib, timed, emit, ok, P, stream, trim):
    """FP16 operands, FP32 accumulate and FP32 result (launch_matmul_kernel_fp16).  cuBLAS through torch
    writes an FP16 result (half the output bytes); it is the nearest library comparator at hand."""
    import torch
    for n in (4096, 8192):
        a = torch.randn((n, n), device="cuda").half()
        b = torch.randn((n, n), device="cuda").half()
        c = torch.empty((n, n), device="cuda")
        ch = torch.empty((n, n), device="cuda", dtype=torch.half)
        rows = {"ours": timed(lambda: ok(lib.cudeep_b200_matmul_f16(P(a), P(b), P(c), n, n, n, stream)), 15),
                "cublas_f16_result_torch": timed(lambda: torch.matmul(a, b, out=ch), 15, cmp=True)}
        try:        # cuBLAS with the same FP32 result this library writes (torch versions that offer out_dtype)
            torch.mm(a, b, out_dtype=torch.float32)
            rows["cublas_f32_result_torch"] = timed(lambda: torch.mm(a, b, out_dtype=torch.float32), 15, cmp=True)
        except Exception:
            pass
        ab, bb = a.to(torch.bfloat16), b.to(torch.bfloat16)
        cb = torch.empty((n, n), device="cuda", dtype=torch.bfloat16)
        rows["ours_bf16"] = timed(lambda: ok(lib.cudeep_b200_matmul_bf16(P(ab), P(bb), P(c), n, n, n, stream)), 15)
        rows["cublas_bf16_result_torch"] = timed(lambda: torch.matmul(ab, bb, out=cb), 15, cmp=True)
        emit(f"H1 FP16 GEMM {n}^3, FP32 result", 2.0 * n ** 3, trim(rows))


def run_g1(lib, emit, ok, P):
    """Small and skinny GEMMs, timed as launches back to back inside a CUDA graph over rotating
    operand sets that together exceed L2: cold operands, no host gaps between launches and none
    of the ~2 us granularity of per-launch events."""
    import torch
    torch.backends.cuda.matmul.allow_tf32 = True
    shapes = [(256, 256, 256), (512, 512, 512), (1024, 1024, 1024), (1536, 1536, 1536), (2048, 2048, 2048),
              (3072, 3072, 3072), (4096, 4096, 4096), (1024, 1024, 4096), (128, 4096, 4096), (512, 512, 4096),
              (256, 1024, 8192), (128, 128, 8192), (8192, 1024, 1024), (4096, 1024, 4096), (5000, 3000, 520)]
    side = torch.cuda.Stream()
    sp = ctypes.c_void_p(side.cuda_stream)

    def graph_ms(launch, sets):
        with torch.cuda.stream(side):
            for i in range(sets):
                launch(i)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(sets):
                    launch(i)
            graph.replay()
            torch.cuda.synchronize()
            ts = []
            for _ in range(5):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(side)
                graph.replay()
                e1.record(side)
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1) / sets)
        return float(np.median(ts)), float(np.min(ts))

    for m, n, k in shapes:
        per_set = (m * k + k * n + m * n) * 4
        sets = max(3, min(40, (400 << 20) // per_set + 1))
        a = [torch.randn((m, k), device="cuda") for _ in range(sets)]
        b = [torch.randn((k, n), device="cuda") for _ in range(sets)]
        c = [torch.empty((m, n), device="cuda") for _ in range(sets)]
        rows = {"ours": graph_ms(lambda i: ok(lib.cudeep_b200_matmul_f32(P(a[i]), P(b[i]), P(c[i]), m, n, k, sp)), sets),
                "cublas_tf32": graph_ms(lambda i: torch.matmul(a[i], b[i], out=c[i]), sets)}
        emit(f"G1 TF32 GEMM {m} x {n} x {k}, graph-timed over {sets} operand sets", 2.0 * m * n * k, rows)
        del a, b, c


def main():
    args = parse_args()
    # Libraries (NCCL's version banner, for one) may print to stdout; the contract is ONE JSON
    # line there.  Everything else this process prints goes to stderr, the result line to the
    # real stdout.
    real_stdout = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    sys.stdout = real_stdout
    if args.suite:
        run_suite(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
