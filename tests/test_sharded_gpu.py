"""cudeep::dist::ShardedGemm on real GPUs, through the C ABI, against the float64 oracle.

On one GPU: a world of one runs every gather mode (NCCL with a single rank, the band pipeline, the
peer-store kernel with no peers).  On two or more GPUs (skipped otherwise): one process driving all
of them, and one process per GPU with the communicator id and the memory handles carried by a TCP
store; every rank's full copy of C is checked.  NVLS is off in NCCL for these tests and the
library's own kernel uses plain peer stores, never multimem.
"""
import os
import socket

import numpy as np
import pytest

from cudeep_b200.sharded import (GATHER_AFTER_GEMM, GATHER_BANDED, GATHER_COLLECTIVE_ONLY, GATHER_COPY_ENGINE,
                                 GATHER_MULTIMEM, GATHER_NONE, GATHER_PEER_STORE, ShardedGemm,
                                 unix_socket_fd_sharing)

pytestmark = pytest.mark.gpu

TF32_MODEL_TOL = 2e-5
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")


def _inputs(m, n, k, seed=7):
    rng = np.random.default_rng(seed)
    return rng.standard_normal((m, k), dtype=np.float32), rng.standard_normal((k, n), dtype=np.float32)


def _load(g, a, b):
    g.set_b(b)
    for local, rank in enumerate(g.local_ranks):
        s = g.rows_of(rank)
        g.set_a(local, a[s.row0:s.row0 + s.rows])


def _poison(g, lib, devices):
    """NaN into every local copy of C, each filled by a kernel on the device that holds it."""
    import ctypes
    import torch
    from cudeep_b200 import _lib
    before = torch.cuda.current_device()
    for local, dev in enumerate(devices):
        torch.cuda.set_device(dev)
        _lib.check(lib.cudeep_b200_fill_f32(ctypes.c_void_p(g.buffers(local)[2]), float("nan"), g.m * g.n, None))
        _lib.check(lib.cudeep_b200_device_synchronize())
    torch.cuda.set_device(before)


@pytest.mark.parametrize("m,n,k", [(1024, 512, 384), (1000, 520, 100)])
def test_world_of_one_every_gather_mode(lib, cuda, oracle, m, n, k):
    from cudeep_b200 import _lib
    a, b = _inputs(m, n, k)
    want = oracle.gemm(a, b, input_mode=oracle.INPUT_TF32_TRUNC)
    with ShardedGemm.local([0], m, n, k, bands=3) as g:
        assert g.rows_of(0).rows == m
        _load(g, a, b)
        for mode in (GATHER_NONE, GATHER_AFTER_GEMM, GATHER_BANDED, GATHER_PEER_STORE, GATHER_COPY_ENGINE):
            _poison(g, lib, [0])
            g.run(mode)
            g.synchronize()
            assert _lib.device_status(True) == 0
            got = g.read_c()
            assert not np.isnan(got).any(), mode
            assert oracle.rel_frobenius(got, want) <= TF32_MODEL_TOL, mode
        g.run(GATHER_COLLECTIVE_ONLY)
        g.synchronize()
        assert oracle.rel_frobenius(g.read_c(), want) <= TF32_MODEL_TOL
        ms = g.time_steps(GATHER_BANDED, 3, 1)
        assert 0.0 < ms < 1000.0
        assert g.steps_enqueued(0) == 6 + 4


def _check_every_rank_has_all_of_c(g, want, oracle, only_own_rows=False):
    for local, rank in enumerate(g.local_ranks):
        got = g.read_c(local)
        if only_own_rows:
            s = g.rows_of(rank)
            got, ref = got[s.row0:s.row0 + s.rows], want[s.row0:s.row0 + s.rows]
        else:
            ref = want
        assert not np.isnan(got).any(), (rank, "rows left unwritten")
        assert oracle.rel_frobenius(got, ref) <= TF32_MODEL_TOL, rank


@pytest.mark.parametrize("m,n,k", [(2048, 768, 512), (1900, 520, 260)])
def test_one_process_all_gpus(lib, cuda, oracle, m, n, k):
    """One process, one host thread per device.  The second shape is ragged in every extent: shares
    of 1024 and 876 rows, tiles that hang over the shard's last row and over N."""
    from cudeep_b200 import _lib
    world = min(cuda.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two GPUs")
    a, b = _inputs(m, n, k, seed=11)
    want = oracle.gemm(a, b, input_mode=oracle.INPUT_TF32_TRUNC)
    with ShardedGemm.local(list(range(world)), m, n, k, bands=2) as g:
        _load(g, a, b)
        g.run(GATHER_NONE)
        g.synchronize()
        _check_every_rank_has_all_of_c(g, want, oracle, only_own_rows=True)
        for mode in (GATHER_AFTER_GEMM, GATHER_BANDED, GATHER_PEER_STORE, GATHER_COPY_ENGINE):
            _poison(g, lib, list(range(world)))
            g.run(mode)
            g.synchronize()
            _check_every_rank_has_all_of_c(g, want, oracle)
        for dev in range(world):
            cuda.cuda.set_device(dev)
            assert _lib.device_status(True) == 0
        cuda.cuda.set_device(0)


@pytest.mark.parametrize("m,n,k", [(2048, 768, 512), (1900, 520, 260)])
def test_one_process_all_gpus_through_the_switch(lib, cuda, oracle, m, n, k):
    """C bound to an NVLink multicast object: the GEMM's epilogue writes each tile once with multimem.st
    and the NVSwitch replicates it into every GPU's C.  NCCL's forms work on the same buffers."""
    from cudeep_b200 import _lib
    world = min(cuda.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two GPUs")
    a, b = _inputs(m, n, k, seed=17)
    want = oracle.gemm(a, b, input_mode=oracle.INPUT_TF32_TRUNC)
    with ShardedGemm.local(list(range(world)), m, n, k, bands=2, multicast=True) as g:
        _load(g, a, b)
        for mode in (GATHER_MULTIMEM, GATHER_AFTER_GEMM, GATHER_MULTIMEM):
            _poison(g, lib, list(range(world)))
            g.run(mode)
            g.synchronize()
            _check_every_rank_has_all_of_c(g, want, oracle)
        with pytest.raises(_lib.CudeepError, match="multicast option"):
            g.run(GATHER_PEER_STORE)
        for dev in range(world):
            cuda.cuda.set_device(dev)
            assert _lib.device_status(True) == 0
        cuda.cuda.set_device(0)
    with ShardedGemm.local(list(range(world)), m, n, k) as g:
        with pytest.raises(_lib.CudeepError, match="multicast option"):
            g.run(GATHER_MULTIMEM)


def _multicast_rank_worker(rank, world, port, out_dir):
    """One process per GPU, C behind a multicast object; the descriptor travels over a unix socket."""
    import datetime
    import torch
    import torch.distributed as dist
    from cudeep_b200 import _lib
    from oracle import oracle as o
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=60))
    counter = [0]

    def barrier():
        counter[0] += 1
        store.set(f"b{counter[0]}/{rank}", "1")
        store.wait([f"b{counter[0]}/{r}" for r in range(world)])

    def broadcast_from_0(x):
        if rank == 0:
            store.set("id", x)
        return store.get("id")

    m, n, k = 2048, 1024, 512
    a, b = _inputs(m, n, k, seed=19)
    want = o.gemm(a, b, input_mode=o.INPUT_TF32_TRUNC)
    lib = _lib.load()
    errs = []
    g = ShardedGemm.rank(rank, world, rank, m, n, k, bands=2, multicast=True)
    try:
        g.connect(broadcast_from_0, lambda x: [], peers=False)
        g.connect_multicast(unix_socket_fd_sharing(rank, world, os.path.join(out_dir, "mc.sock")), barrier)
        _load(g, a, b)
        stream = torch.cuda.current_stream().cuda_stream
        for mode in (GATHER_MULTIMEM, GATHER_AFTER_GEMM, GATHER_MULTIMEM):
            _poison(g, lib, [rank])
            barrier()
            g.run(mode, stream)
            torch.cuda.synchronize()
            g.synchronize()
            barrier()
            got = g.read_c()
            errs.append(float("inf") if np.isnan(got).any() else o.rel_frobenius(got, want))
        status = _lib.device_status(True)
    finally:
        barrier()                      # nobody unbinds while another rank may still write through the switch
        g.close()
    np.save(os.path.join(out_dir, f"m_{rank}.npy"), np.array([status, *errs]))


def test_one_process_per_gpu_through_the_switch(cuda, lib, tmp_path):
    if cuda.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_multicast_rank_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        status, *errs = np.load(tmp_path / f"m_{rank}.npy")
        assert status == 0
        assert all(e <= TF32_MODEL_TOL for e in errs), errs


def _rank_worker(rank, world, port, out_dir):
    """One process per GPU; the id and the handles travel through a TCP store."""
    import datetime
    import torch
    import torch.distributed as dist
    from cudeep_b200 import _lib
    from oracle import oracle as o
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=60))

    def broadcast_from_0(x):
        if rank == 0:
            store.set("id", x)
        return store.get("id")

    def all_gather(x):
        store.set(f"h{rank}", x)
        return [store.get(f"h{r}") for r in range(world)]

    def barrier(tag):
        store.set(f"{tag}/{rank}", "1")
        store.wait([f"{tag}/{r}" for r in range(world)])

    m, n, k = 2048, 1024, 512
    a, b = _inputs(m, n, k, seed=13)
    want = o.gemm(a, b, input_mode=o.INPUT_TF32_TRUNC)
    lib = _lib.load()
    errs = []
    with ShardedGemm.rank(rank, world, rank, m, n, k, bands=2) as g:
        g.connect(broadcast_from_0, all_gather)
        _load(g, a, b)
        stream = torch.cuda.current_stream().cuda_stream
        for mode in (GATHER_AFTER_GEMM, GATHER_BANDED, GATHER_PEER_STORE, GATHER_COPY_ENGINE):
            _poison(g, lib, [rank])
            barrier(f"poisoned{mode}")
            g.run(mode, stream)
            torch.cuda.synchronize()
            g.synchronize()
            barrier(f"ran{mode}")            # peers' stores into this rank's C have completed with their kernels
            got = g.read_c()
            errs.append(float("inf") if np.isnan(got).any() else o.rel_frobenius(got, want))
        status = _lib.device_status(True)
        barrier("done")
    np.save(os.path.join(out_dir, f"r_{rank}.npy"), np.array([status, *errs]))


def test_one_process_per_gpu(cuda, lib, tmp_path):
    if cuda.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_rank_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        status, *errs = np.load(tmp_path / f"r_{rank}.npy")
        assert status == 0
        assert all(e <= TF32_MODEL_TOL for e in errs), errs
