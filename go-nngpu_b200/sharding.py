"""Row partition of the tall GEMM across ranks (one process per GPU).

A[M,K] is split into contiguous row blocks, B[K,N] is replicated, and rank r
owns rows [lo, hi) of C.  Blocks are multiples of the GEMM's 128-row tile so
that no tile straddles two ranks; the last block may be short or empty.
"""

TILE_M = 128


def shard_rows(m_total, world, rank, align=TILE_M):
    """Returns (lo, hi) of rank `rank`'s row block."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("bad world/rank")
    per = -(-m_total // world)
    per = -(-per // align) * align
    lo = min(rank * per, m_total)
    hi = min(lo + per, m_total)
    return lo, hi


def all_shards(m_total, world, align=TILE_M):
    return [shard_rows(m_total, world, r, align) for r in range(world)]
