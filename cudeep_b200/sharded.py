"""Row-sharded GEMM over the GPUs of one node: C[M,N] = A[M,K] @ B[K,N], A and C split by rows.

The work is done by `cudeep::dist::ShardedGemm` inside libcudeep_b200.so
(include/cudeep/dist/sharded_gemm.cuh); this module is its ctypes face and needs neither torch nor
any other framework.  The reference is single-device (device 0 is hard-coded in its capability
queries, src/kernels/matmul_kernel.cu:1745); this is the multi-GPU form of its
launch_matmul_kernel<float>.

Each rank owns rows [row0, row0 + rows) of A and C and a replica of B, so computing needs no
exchange.  The optional all-gather of C comes in the forms `GATHER_*` below; GATHER_PEER_STORE is
the fused one (the GEMM's epilogue stores every tile into all GPUs' C).

One process may drive all GPUs (`ShardedGemm.local`), or one process per GPU (`ShardedGemm.rank`);
in the second form the caller moves two small byte strings between the processes (`connect`), with
whatever transport it has: a torch.distributed store, MPI, files.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Callable, Optional, Sequence

import numpy as np

from . import _lib

(GATHER_NONE, GATHER_AFTER_GEMM, GATHER_BANDED, GATHER_PEER_STORE, GATHER_COLLECTIVE_ONLY, GATHER_COPY_ENGINE,
 GATHER_COPY_ONLY, GATHER_MULTIMEM) = range(8)
COMM_ID_BYTES = 128
MEM_HANDLE_BYTES = 64


@dataclass(frozen=True)
class RowShard:
    rank: int
    world: int
    row0: int
    rows: int


def row_partition(m: int, world: int, align: int = 1) -> list[RowShard]:
    """Split m rows over `world` ranks as evenly as possible in units of `align` rows; the last
    ranks get the shorter shares, a rank may get zero rows when m < world * align.  With
    align = 128 this is the partition the library uses (ShardedGemm.rows_of)."""
    if m < 0 or world < 1 or align < 1:
        raise ValueError("row_partition: m >= 0, world >= 1 and align >= 1 required")
    units = -(-m // align)
    base, extra = divmod(units, world)
    shards, row0 = [], 0
    for r in range(world):
        rows = min((base + (1 if r < extra else 0)) * align, m - row0)
        shards.append(RowShard(r, world, row0, max(rows, 0)))
        row0 += max(rows, 0)
    return shards


class PeerFailure(RuntimeError):
    """Another rank of the sharded product reported an error, or did not report in time."""


class StepGuard:
    """Host-side liveness check between processes, so that a rank that failed is noticed before the
    others enqueue anything that would wait for it.

    Every rank calls report(step) when its host-side preparation for that step is done (or
    report(step, ok=False, message=...) from its exception handler), then wait_all(step) before it
    enqueues the step.  Reports go through a key-value store with set / wait / get (a
    torch.distributed store, for one); nothing here touches a GPU.  A rank that leaves does so
    between steps, with none of its kernels or collectives in flight."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 30.0, prefix: str = "cudeep_b200/step"):
        self.store, self.rank, self.world = store, rank, world
        self.timeout_s = timeout_s
        self.prefix = prefix

    def _key(self, step: int, rank: int) -> str:
        return f"{self.prefix}/{step}/{rank}"

    def report(self, step: int, ok: bool = True, message: str = "") -> None:
        self.store.set(self._key(step, self.rank), "ok" if ok else "error: " + message)

    def wait_all(self, step: int) -> None:
        """Returns when every rank has reported success for `step`; raises PeerFailure naming the
        ranks that reported an error or did not report within the timeout."""
        import datetime
        import time
        deadline = time.monotonic() + self.timeout_s
        failed, missing = {}, []
        for r in range(self.world):
            key = self._key(step, r)
            left = max(deadline - time.monotonic(), 0.001)
            try:
                self.store.wait([key], datetime.timedelta(seconds=left))
            except Exception:
                missing.append(r)
                continue
            value = self.store.get(key)
            value = value.decode("utf-8", "replace") if isinstance(value, bytes) else str(value)
            if value != "ok":
                failed[r] = value
        if failed or missing:
            parts = [f"rank {r} {v}" for r, v in sorted(failed.items())]
            parts += [f"rank {r} did not report within {self.timeout_s:g} s" for r in missing]
            raise PeerFailure(f"step {step}: " + "; ".join(parts))


class ShardedGemm:
    """A row-sharded product held by libcudeep_b200.so; see the module docstring."""

    def __init__(self, handle: ctypes.c_void_p, m: int, n: int, k: int, world: int, local_ranks: Sequence[int]):
        self._h, self.m, self.n, self.k, self.world = handle, m, n, k, world
        self.local_ranks = list(local_ranks)

    # ---- construction -----------------------------------------------------------------------

    @classmethod
    def local(cls, devices: Sequence[int], m: int, n: int, k: int, *, bands: int = 4, comm_sms: int = 20,
              dry_run: bool = False, multicast: bool = False) -> "ShardedGemm":
        """One process drives all of `devices` (rank i on devices[i]).  multicast: C is bound to an NVLink
        multicast object, which GATHER_MULTIMEM writes through (the peer-mapped forms are then unavailable)."""
        lib = _lib.load()
        arr = (ctypes.c_int * len(devices))(*devices)
        h = ctypes.c_void_p()
        _lib.check(lib.cudeep_b200_sharded_gemm_create_local(arr, len(devices), m, n, k, bands, comm_sms,
                                                             int(dry_run) | (2 if multicast else 0), ctypes.byref(h)))
        return cls(h, m, n, k, len(devices), range(len(devices)))

    @classmethod
    def rank(cls, rank: int, world: int, device: int, m: int, n: int, k: int, *, bands: int = 4,
             comm_sms: int = 20, dry_run: bool = False, multicast: bool = False) -> "ShardedGemm":
        """This process is rank `rank` of `world` and drives `device`."""
        lib = _lib.load()
        h = ctypes.c_void_p()
        _lib.check(lib.cudeep_b200_sharded_gemm_create_rank(rank, world, device, m, n, k, bands, comm_sms,
                                                            int(dry_run) | (2 if multicast else 0), ctypes.byref(h)))
        return cls(h, m, n, k, world, [rank])

    def close(self) -> None:
        if self._h:
            _lib.check(_lib.load().cudeep_b200_sharded_gemm_destroy(self._h))
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ---- plan and buffers -------------------------------------------------------------------

    def rows_of(self, rank: int, band: int = -1) -> RowShard:
        row0, rows = ctypes.c_longlong(), ctypes.c_longlong()
        _lib.check(_lib.load().cudeep_b200_sharded_gemm_rows(self._h, rank, band, ctypes.byref(row0),
                                                             ctypes.byref(rows)))
        return RowShard(rank, self.world, row0.value, rows.value)

    def buffers(self, local: int = 0) -> tuple[int, int, int]:
        """Device addresses of local rank `local`: its rows of A, its replica of B, the whole C."""
        a, b, c = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
        _lib.check(_lib.load().cudeep_b200_sharded_gemm_buffers(self._h, local, ctypes.byref(a), ctypes.byref(b),
                                                                ctypes.byref(c)))
        return a.value or 0, b.value or 0, c.value or 0

    def _h2d(self, dst: int, array: np.ndarray) -> None:
        src = np.ascontiguousarray(array, dtype=np.float32)
        _lib.check(_lib.load().cudeep_b200_memcpy_h2d(ctypes.c_void_p(dst), src.ctypes.data_as(ctypes.c_void_p),
                                                      src.nbytes, None))

    def set_a(self, local: int, rows: np.ndarray) -> None:
        shard = self.rows_of(self.local_ranks[local])
        if rows.shape != (shard.rows, self.k):
            raise ValueError(f"set_a: expected {(shard.rows, self.k)}, got {rows.shape}")
        if shard.rows:
            self._h2d(self.buffers(local)[0], rows)

    def set_b(self, b: np.ndarray) -> None:
        if b.shape != (self.k, self.n):
            raise ValueError(f"set_b: expected {(self.k, self.n)}, got {b.shape}")
        for local in range(len(self.local_ranks)):
            self._h2d(self.buffers(local)[1], b)

    def read_c(self, local: int = 0, row0: int = 0, rows: Optional[int] = None) -> np.ndarray:
        """Rows [row0, row0 + rows) of local rank `local`'s copy of C (blocking)."""
        rows = self.m - row0 if rows is None else rows
        out = np.empty((rows, self.n), dtype=np.float32)
        if rows:
            _lib.check(_lib.load().cudeep_b200_sharded_gemm_read_c(self._h, local, row0, rows,
                                                                   out.ctypes.data_as(ctypes.c_void_p)))
        return out

    # ---- one process per GPU: the two exchanges ----------------------------------------------

    @staticmethod
    def new_comm_id() -> bytes:
        buf = ctypes.create_string_buffer(COMM_ID_BYTES)
        _lib.check(_lib.load().cudeep_b200_sharded_gemm_comm_id(buf))
        return buf.raw

    def init_comm(self, comm_id: bytes) -> None:
        if len(comm_id) != COMM_ID_BYTES:
            raise ValueError("init_comm: a communicator id has 128 bytes")
        _lib.check(_lib.load().cudeep_b200_sharded_gemm_init_comm(self._h, comm_id))

    def export_c(self) -> bytes:
        buf = ctypes.create_string_buffer(MEM_HANDLE_BYTES)
        _lib.check(_lib.load().cudeep_b200_sharded_gemm_export_c(self._h, buf))
        return buf.raw

    def open_peers(self, handles: Sequence[bytes]) -> None:
        if len(handles) != self.world or any(len(h) != MEM_HANDLE_BYTES for h in handles):
            raise ValueError("open_peers: one 64-byte handle per rank, in rank order")
        _lib.check(_lib.load().cudeep_b200_sharded_gemm_open_peers(self._h, b"".join(handles)))

    def connect(self, broadcast_from_0: Callable[[Optional[bytes]], bytes],
                all_gather: Callable[[bytes], Sequence[bytes]], *, peers: bool = True) -> None:
        """The whole hand-shake of the one-process-per-GPU form.  `broadcast_from_0(x)` returns
        rank 0's `x` on every rank (other ranks pass None); `all_gather(x)` returns every rank's `x`
        in rank order."""
        me = self.local_ranks[0]
        self.init_comm(broadcast_from_0(self.new_comm_id() if me == 0 else None))
        if peers and self.world > 1:
            self.open_peers(list(all_gather(self.export_c())))

    def connect_multicast(self, share_fd: Callable[[Optional[int]], int], barrier: Callable[[], None]) -> None:
        """The extra hand-shake of an object made with multicast=True (one process per GPU).
        `share_fd(fd)`: rank 0 passes the descriptor of the multicast object and every other rank
        (passing None) gets a descriptor of its own for the same object - descriptors cross processes
        over a unix socket (socket.send_fds / recv_fds).  `barrier()` returns once every rank reached it."""
        import os
        lib = _lib.load()
        me = self.local_ranks[0]
        if me == 0:
            fd = ctypes.c_int(-1)
            _lib.check(lib.cudeep_b200_sharded_gemm_multicast_fd(self._h, ctypes.byref(fd)))
            try:
                share_fd(fd.value)
            finally:
                os.close(fd.value)
            _lib.check(lib.cudeep_b200_sharded_gemm_multicast_join(self._h, -1))
        else:
            fd = share_fd(None)
            try:
                _lib.check(lib.cudeep_b200_sharded_gemm_multicast_join(self._h, fd))
            finally:
                os.close(fd)
        barrier()                      # every device has been added
        _lib.check(lib.cudeep_b200_sharded_gemm_multicast_bind(self._h))
        barrier()

    # ---- steps --------------------------------------------------------------------------------

    def run(self, gather: int = GATHER_NONE, stream: Optional[int] = None) -> None:
        """Enqueue one step; asynchronous.  `stream` (a cudaStream_t as an integer) only in the
        one-process-per-GPU form."""
        _lib.check(_lib.load().cudeep_b200_sharded_gemm_run(self._h, gather, ctypes.c_void_p(stream or 0)))

    def run_guarded(self, gather: int, guard: StepGuard, step: int, stream: Optional[int] = None) -> None:
        """The two-phase step between processes: report, wait for every rank's report, and only then
        enqueue.  Raises PeerFailure (and enqueues nothing) when a rank failed or is absent."""
        guard.report(step)
        guard.wait_all(step)
        self.run(gather, stream)

    def synchronize(self) -> None:
        _lib.check(_lib.load().cudeep_b200_sharded_gemm_synchronize(self._h))

    def time_steps(self, gather: int, steps: int, warmup: int) -> float:
        """Mean device milliseconds per step (slowest local rank)."""
        ms = ctypes.c_float()
        _lib.check(_lib.load().cudeep_b200_sharded_gemm_time(self._h, gather, steps, warmup, ctypes.byref(ms)))
        return ms.value

    def steps_enqueued(self, local: int = 0) -> int:
        out = ctypes.c_longlong()
        _lib.check(_lib.load().cudeep_b200_sharded_gemm_steps(self._h, local, ctypes.byref(out)))
        return out.value

    def inject_failure(self, rank: int) -> None:
        _lib.check(_lib.load().cudeep_b200_sharded_gemm_inject_failure(self._h, rank))


def unix_socket_fd_sharing(rank: int, world: int, path: str):
    """A `share_fd` for ShardedGemm.connect_multicast over a unix-domain socket at `path` (all ranks on
    one host): rank 0 listens and sends the descriptor to each rank that connects."""
    import socket
    import time

    def share_fd(fd):
        if rank == 0:
            with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as server:
                server.bind(path)
                server.listen(world)
                try:
                    for _ in range(world - 1):
                        conn, _addr = server.accept()
                        with conn:
                            socket.send_fds(conn, [b"fd"], [fd])
                finally:
                    import os
                    os.unlink(path)
            return fd
        deadline = time.monotonic() + 60.0
        while True:
            try:
                with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as client:
                    client.connect(path)
                    _msg, fds, _flags, _addr = socket.recv_fds(client, 16, 1)
                    return fds[0]
            except (FileNotFoundError, ConnectionRefusedError):
                if time.monotonic() > deadline:
                    raise
                time.sleep(0.05)

    return share_fd
