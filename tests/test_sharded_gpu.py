"""Row-sharded GEMM on two GPUs with NCCL (skipped on a single-GPU box)."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    from cudeep_b200 import _lib
    from cudeep_b200.sharded import ShardedGemm, row_partition
    from oracle import oracle as o
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        m, n, k = 1024, 512, 384
        shards = row_partition(m, world, 128)
        me = shards[rank]
        rng = np.random.default_rng(7)
        a = rng.standard_normal((m, k), dtype=np.float32)
        b = rng.standard_normal((k, n), dtype=np.float32)
        g = ShardedGemm(me, torch.from_numpy(a[me.row0:me.row0 + me.rows].copy()).cuda(), torch.from_numpy(b).cuda())
        g.run()
        full = g.gather(shards)
        torch.cuda.synchronize()
        status = _lib.device_status(True)
        err = o.rel_frobenius(full.cpu().numpy(), o.gemm(a, b, input_mode=o.INPUT_TF32_TRUNC))
        np.save(os.path.join(out_dir, f"r_{rank}.npy"), np.array([status, err]))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gpu_sharded_gemm_with_gather(cuda, lib, tmp_path):
    if cuda.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        status, err = np.load(tmp_path / f"r_{rank}.npy")
        assert status == 0 and err <= 2e-5
