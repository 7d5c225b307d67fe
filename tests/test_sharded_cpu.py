"""Row-sharded GEMM host logic on CPU: partitioning, and a world-size-2 gloo run in which each rank
computes its shard with the CPU oracle and the shards are all-gathered (no GPU involved)."""
import os
import socket

import numpy as np
import pytest

from cudeep_b200.sharded import RowShard, ShardedGemm, row_partition


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


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, m, n, k, align, out_dir):
    import torch
    import torch.distributed as dist
    from oracle import oracle as o
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        shards = row_partition(m, world, align)
        me = shards[rank]
        rng = np.random.default_rng(42)
        a = rng.standard_normal((m, k), dtype=np.float32)
        b = rng.standard_normal((k, n), dtype=np.float32)

        def compute(ta, tb, tc):
            tc.copy_(torch.from_numpy(o.gemm(ta.numpy(), tb.numpy()).astype(np.float32)))

        g = ShardedGemm(me, torch.from_numpy(a[me.row0:me.row0 + me.rows].copy()), torch.from_numpy(b), compute=compute)
        g.run()
        full = g.gather(shards).numpy()
        want = o.gemm(a, b).astype(np.float32)
        np.save(os.path.join(out_dir, f"ok_{rank}.npy"), np.array([np.array_equal(full, want), full.shape[0]]))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("m,align", [(256, 1), (300, 64)])
def test_two_rank_gloo_gather(tmp_path, m, align):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_worker, args=(2, port, m, 48, 40, align, str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        ok, rows = np.load(tmp_path / f"ok_{rank}.npy")
        assert ok == 1 and rows == m


# ---- a rank that fails is noticed on the host, before the collective -------------------------------

def _guard_worker(rank, world, port, mode, out_dir):
    """mode 'error': rank 1 reports a failure and leaves; 'silent': rank 1 leaves without a word;
    'fine': everybody gathers."""
    import datetime
    import torch
    import torch.distributed as dist
    from cudeep_b200.sharded import PeerFailure, StepGuard
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=20))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world)
    guard = StepGuard(store, rank, world, timeout_s=2.0)
    outcome = "none"
    try:
        shards = row_partition(64, world)
        me = shards[rank]
        a = torch.ones((me.rows, 8))
        b = torch.ones((8, 4))
        g = ShardedGemm(me, a, b, compute=lambda ta, tb, tc: tc.copy_(ta @ tb))
        g.run()
        if rank == 1 and mode == "error":
            guard.report(0, ok=False, message="kernel launch failed on this rank")
            outcome = "left"
        elif rank == 1 and mode == "silent":
            outcome = "left"
        else:
            try:
                full = g.gather(shards, guard=guard, step=0)
                outcome = f"gathered {tuple(full.shape)}"
            except PeerFailure as e:
                outcome = "PeerFailure: " + str(e)
    finally:
        with open(os.path.join(out_dir, f"outcome_{rank}.txt"), "w") as f:
            f.write(outcome)
        # no destroy_process_group barrier: a rank that found its peer gone just leaves
        store = None


@pytest.mark.parametrize("mode", ["fine", "error", "silent"])
def test_failed_rank_is_detected_before_the_collective(tmp_path, mode):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_guard_worker, args=(2, port, mode, str(tmp_path)), nprocs=2, join=True)
    out0 = (tmp_path / "outcome_0.txt").read_text()
    out1 = (tmp_path / "outcome_1.txt").read_text()
    if mode == "fine":
        assert out0 == "gathered (64, 4)" and out1 == "gathered (64, 4)"
    elif mode == "error":
        assert out0.startswith("PeerFailure: step 0: rank 1 error: kernel launch failed") and out1 == "left"
    else:
        assert "rank 1 did not report within 2 s" in out0 and out1 == "left"
