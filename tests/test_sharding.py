"""Host logic of the row-sharded multi-GPU GEMM, on CPU: the partition itself,
and a world-size-2 gloo run of the step's plumbing (B broadcast from rank 0,
each rank producing its own row block, blocks tiling C exactly).  The per-rank
product is done by the CPU oracle here: this test covers the bookkeeping and
the collective, not the kernel."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "go-nngpu_b200"))
from sharding import all_shards, shard_rows  # noqa: E402


@pytest.mark.parametrize("m,world", [(131072, 1), (131072, 2), (131072, 4), (131072, 8), (1000, 3),
                                     (128, 8), (1, 4), (129, 2), (4096, 5)])
def test_shards_tile_the_rows(m, world):
    shards = all_shards(m, world)
    assert shards[0][0] == 0 and shards[-1][1] == m
    for (lo, hi), (lo2, _) in zip(shards, shards[1:]):
        assert hi == lo2 and lo <= hi
    for lo, hi in shards[:-1]:
        assert (hi - lo) % 256 == 0 or hi == m     # full tiles except where the rows run out
    assert sum(hi - lo for lo, hi in shards) == m
    with pytest.raises(ValueError):
        shard_rows(m, world, world)


def _worker(rank, world, port, m, k, n, out_dir):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from oracle import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lo, hi = shard_rows(m, world, rank)
    rng = np.random.default_rng(4)
    A = rng.standard_normal((m, k)).astype(np.float32)   # every rank can regenerate A; it keeps its rows only
    B_full = rng.standard_normal((k, n)).astype(np.float32)
    A_shard = A[lo:hi]
    B = torch.from_numpy(B_full.copy() if rank == 0 else np.zeros((k, n), np.float32))
    dist.broadcast(B, src=0)                              # the step's only collective
    C_shard = oracle.gemm_f64(A_shard, B.numpy()).astype(np.float32) if hi > lo else np.zeros((0, n), np.float32)
    np.save(os.path.join(out_dir, f"c_{rank}.npy"), C_shard)
    t = torch.tensor([float(hi - lo)])
    dist.all_reduce(t)                                    # rows processed by the whole job
    assert int(t.item()) == m
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_step_assembles_the_full_product(tmp_path):
    import torch.multiprocessing as mp
    from oracle import oracle
    m, k, n, world = 300, 64, 48, 2
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, m, k, n, str(tmp_path)), nprocs=world, join=True)
    rng = np.random.default_rng(4)
    A = rng.standard_normal((m, k)).astype(np.float32)
    B = rng.standard_normal((k, n)).astype(np.float32)
    C = np.concatenate([np.load(tmp_path / f"c_{r}.npy") for r in range(world)], axis=0)
    assert C.shape == (m, n)
    assert np.array_equal(C, oracle.gemm_f64(A, B).astype(np.float32))
