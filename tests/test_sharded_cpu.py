"""Row-sharded GEMM host logic without a GPU: the partition and band plan of cudeep::dist::ShardedGemm
(through the C ABI, in its dry-run form that makes no CUDA or NCCL call), the two-phase step that keeps a
failed rank from leaving anything in flight on the others, and the same between two processes
(world size 2 over a gloo / TCP store)."""
import os
import socket

import pytest

from cudeep_b200 import _lib
from cudeep_b200.sharded import (GATHER_BANDED, GATHER_NONE, GATHER_PEER_STORE, RowShard, ShardedGemm,
                                 row_partition)


def test_row_partition_even_and_ragged():
    shards = row_partition(65536, 8)
    assert [s.rows for s in shards] == [8192] * 8 and shards[3].row0 == 3 * 8192
    shards = row_partition(1000, 3, align=128)
    assert [s.rows for s in shards] == [384, 384, 232] and sum(s.rows for s in shards) == 1000
    assert [s.row0 for s in shards] == [0, 384, 768]
    shards = row_partition(100, 4, align=128)
    assert [s.rows for s in shards] == [100, 0, 0, 0]
    assert row_partition(0, 2)[1] == RowShard(1, 2, 0, 0)
    with pytest.raises(ValueError):
        row_partition(10, 0)


@pytest.mark.parametrize("m,world", [(65536, 8), (16384, 4), (16384, 2), (1000, 3), (100, 4), (8192 * 3 + 7, 5)])
def test_library_partition_matches_the_python_one_and_bands_tile_each_share(lib, m, world):
    with ShardedGemm.local(list(range(world)), m, 256, 64, bands=4, dry_run=True) as g:
        want = row_partition(m, world, 128)
        got = [g.rows_of(r) for r in range(world)]
        assert got == want
        assert sum(s.rows for s in got) == m
        for r in range(world):
            bands = [g.rows_of(r, b) for b in range(4)]
            assert bands[0].row0 == got[r].row0
            for a, b in zip(bands, bands[1:]):
                assert a.row0 + a.rows == b.row0                 # contiguous, in order
            assert bands[-1].row0 + bands[-1].rows == got[r].row0 + got[r].rows
            assert all(b.rows >= 0 for b in bands)
            end = got[r].row0 + got[r].rows
            assert all(b.rows % 256 == 0 for b in bands if b.row0 + b.rows != end)   # whole 256-row tiles


def test_c5_shards(lib):
    """The sharded benchmark configurations: 65536 x 8192 x 8192 and 16384^3 on 1 / 2 / 4 / 8 GPUs."""
    for m, n, k in ((65536, 8192, 8192), (16384, 16384, 16384)):
        for world in (1, 2, 4, 8):
            with ShardedGemm.local(list(range(world)), m, n, k, dry_run=True) as g:
                assert [g.rows_of(r).rows for r in range(world)] == [m // world] * world
                assert [g.rows_of(r, 1).rows for r in range(world)] == [m // world // 4] * world


def test_bad_arguments_are_errors(lib):
    with pytest.raises(_lib.CudeepError, match="positive"):
        ShardedGemm.local([0, 1], 0, 8, 8, dry_run=True)
    with pytest.raises(_lib.CudeepError, match="rank out of range"):
        ShardedGemm.rank(2, 2, 0, 128, 8, 8, dry_run=True)
    with ShardedGemm.local([0, 1], 512, 8, 8, dry_run=True) as g:
        with pytest.raises(_lib.CudeepError, match="rank out of range"):
            g.rows_of(2)
        with pytest.raises(_lib.CudeepError, match="band out of range"):
            g.rows_of(0, 4)
        with pytest.raises(_lib.CudeepError, match="unknown gather mode"):
            g.run(9)


def test_a_failed_rank_stops_the_step_before_anything_is_enqueued(lib):
    """One process, four ranks: rank 2's host-side preparation fails.  No rank enqueues the step (so
    nothing on any GPU waits for the absent one), the error names the rank, and the object is spent."""
    with ShardedGemm.local([0, 1, 2, 3], 4096, 256, 64, dry_run=True) as g:
        g.run(GATHER_BANDED)
        g.run(GATHER_PEER_STORE)
        assert [g.steps_enqueued(i) for i in range(4)] == [2, 2, 2, 2]
        g.inject_failure(2)
        with pytest.raises(_lib.CudeepError, match=r"before anything was enqueued: rank 2: failure injected"):
            g.run(GATHER_BANDED)
        assert [g.steps_enqueued(i) for i in range(4)] == [2, 2, 2, 2]
        with pytest.raises(_lib.CudeepError, match="had a failed step"):
            g.run(GATHER_NONE)
        assert [g.steps_enqueued(i) for i in range(4)] == [2, 2, 2, 2]


# ---- two processes: a rank that fails is noticed on the host, before the step is enqueued -----------

def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _guard_worker(rank, world, port, mode, out_dir):
    """mode 'error': rank 1 reports a failure and leaves; 'silent': rank 1 leaves without a word;
    'fine': both ranks enqueue the step."""
    import datetime
    import torch.distributed as dist
    from cudeep_b200.sharded import PeerFailure, StepGuard
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=20))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world)
    guard = StepGuard(store, rank, world, timeout_s=2.0)
    outcome = "none"
    try:
        g = ShardedGemm.rank(rank, world, 0, 1024, 64, 32, dry_run=True)
        assert g.rows_of(rank) == row_partition(1024, world, 128)[rank]
        if rank == 1 and mode == "error":
            guard.report(0, ok=False, message="kernel launch failed on this rank")
            outcome = "left"
        elif rank == 1 and mode == "silent":
            outcome = "left"
        else:
            try:
                g.run_guarded(GATHER_BANDED, guard, step=0)
                outcome = f"enqueued {g.steps_enqueued()}"
            except PeerFailure as e:
                outcome = f"enqueued {g.steps_enqueued()}; PeerFailure: {e}"
        g.close()
    finally:
        with open(os.path.join(out_dir, f"outcome_{rank}.txt"), "w") as f:
            f.write(outcome)
        # no destroy_process_group barrier: a rank that found its peer gone just leaves
        store = None


@pytest.mark.parametrize("mode", ["fine", "error", "silent"])
def test_failed_rank_is_detected_before_the_step_is_enqueued(tmp_path, lib, mode):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_guard_worker, args=(2, port, mode, str(tmp_path)), nprocs=2, join=True)
    out0 = (tmp_path / "outcome_0.txt").read_text()
    out1 = (tmp_path / "outcome_1.txt").read_text()
    if mode == "fine":
        assert out0 == "enqueued 1" and out1 == "enqueued 1"
    elif mode == "error":
        assert out0.startswith("enqueued 0; PeerFailure: step 0: rank 1 error: kernel launch failed") and out1 == "left"
    else:
        assert out0.startswith("enqueued 0;") and "rank 1 did not report within 2 s" in out0 and out1 == "left"
