"""Row-sharded GEMM over the GPUs of one node: C[M,N] = A[M,K] @ B[K,N], A and C split by rows.

One process per GPU (torchrun); each rank owns rows [row0, row0 + rows) of A and C and a full
replica of B, so no exchange is needed to compute.  The only collective is the optional
all-gather of C (NCCL over NVLink) for callers that need the whole product on every rank.
The reference is single-device (device 0 is hard-coded in its capability queries,
src/kernels/matmul_kernel.cu:1745); this module is the multi-GPU form of its
launch_matmul_kernel<float>.

torch is used here for what it is good at: device buffers, streams and torch.distributed.
The product itself is computed by libcudeep_b200.so.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Callable, Optional


@dataclass(frozen=True)
class RowShard:
    rank: int
    world: int
    row0: int
    rows: int


def row_partition(m: int, world: int, align: int = 1) -> list[RowShard]:
    """Split m rows over `world` ranks as evenly as possible in units of `align` rows; the last
    ranks get the shorter shares, a rank may get zero rows when m < world * align."""
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


def _device_matmul(a, b, c, stream) -> None:
    from . import _lib
    m, k = a.shape
    n = b.shape[1]
    _lib.check(_lib.load().cudeep_b200_matmul_f32(ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(b.data_ptr()),
                                                  ctypes.c_void_p(c.data_ptr()), m, n, k, stream))


class PeerFailure(RuntimeError):
    """Another rank of the sharded product reported an error, or did not report in time."""


class StepGuard:
    """Host-side liveness check, so that a rank that failed is noticed before the others enter a
    collective they would hang in.

    Every rank calls report(step) when its kernels for that step are queued (or report(step,
    ok=False, message=...) from its exception handler), then wait_all(step) before the collective.
    Reports go through a torch.distributed store (the TCP store of the process group, or any other
    `Store`); nothing here touches a GPU.  A rank that leaves does so between steps, with none of
    its kernels or collectives in flight."""

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
            value = self.store.get(key).decode("utf-8", "replace")
            if value != "ok":
                failed[r] = value
        if failed or missing:
            parts = [f"rank {r} {v}" for r, v in sorted(failed.items())]
            parts += [f"rank {r} did not report within {self.timeout_s:g} s" for r in missing]
            raise PeerFailure(f"step {step}: " + "; ".join(parts))


class ShardedGemm:
    """This rank's share of a row-sharded product.

    a_shard: [rows, K] and b: [K, N] are torch tensors on this rank's device (CPU tensors are
    accepted when a `compute` callback is given, which is how the host logic is tested without GPUs).
    """

    def __init__(self, shard: RowShard, a_shard, b, *, compute: Optional[Callable] = None):
        import torch
        if a_shard.shape[0] != shard.rows or a_shard.shape[1] != b.shape[0]:
            raise ValueError("ShardedGemm: a_shard must be [shard.rows, K] and b [K, N]")
        self.shard = shard
        self.a, self.b = a_shard, b
        self.c = torch.empty((shard.rows, b.shape[1]), dtype=a_shard.dtype, device=a_shard.device)
        self._compute = compute

    def run(self):
        """Compute this rank's rows of C (asynchronous on the current CUDA stream)."""
        if self.shard.rows == 0:
            return self.c
        if self._compute is not None:
            self._compute(self.a, self.b, self.c)
        else:
            import torch
            _device_matmul(self.a, self.b, self.c, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        return self.c

    def gather(self, shards: list[RowShard], group=None, guard: Optional[StepGuard] = None, step: int = 0):
        """All-gather the row shards into the full C on every rank (shards may differ in size).
        With a guard, every rank first confirms that all ranks reached this step: a failed or
        absent peer raises PeerFailure here instead of leaving the collective to hang."""
        import torch
        import torch.distributed as dist
        if guard is not None:
            guard.report(step)
            guard.wait_all(step)
        n = self.b.shape[1]
        if all(s.rows == shards[0].rows for s in shards):
            full = torch.empty((sum(s.rows for s in shards), n), dtype=self.c.dtype, device=self.c.device)
            dist.all_gather_into_tensor(full, self.c.contiguous(), group=group)
            return full
        # Collectives want equal contributions: pad every shard to the longest one, gather,
        # then drop the padding rows.
        longest = max(s.rows for s in shards)
        padded = torch.zeros((longest, n), dtype=self.c.dtype, device=self.c.device)
        padded[:self.shard.rows] = self.c
        stacked = torch.empty((len(shards) * longest, n), dtype=self.c.dtype, device=self.c.device)
        dist.all_gather_into_tensor(stacked, padded, group=group)
        return torch.cat([stacked[i * longest:i * longest + s.rows] for i, s in enumerate(shards)], dim=0)
