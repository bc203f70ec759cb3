"""Row partition of the tall GEMM across GPUs (ranks of a job, or devices of one process).

A[M,K] is split into contiguous row blocks, B[K,N] is replicated, and shard r
owns rows [lo, hi) of C.  The plan itself is the library's (`gonngpu_shard_plan`,
also what `gonngpu_matmul_sharded` uses): blocks of ceil(M / n) rows rounded up
to the 256-row tile of the pair kernel so that no tile straddles two shards; the
last blocks may be short or empty.  It is host arithmetic: no GPU is needed.
"""
import gonngpu

TILE_M = 256


def shard_rows(m_total, world, rank):
    """Returns (lo, hi) of rank `rank`'s row block."""
    if world < 1 or not (0 <= rank < world) or m_total < 0:
        raise ValueError("bad world/rank")
    return gonngpu.shard_plan(m_total, world, rank)


def all_shards(m_total, world):
    return [shard_rows(m_total, world, r) for r in range(world)]
