"""Row sharding of an M-sharded GEMM (or batch-sharded block) over the ranks of one box.

Rank r of g owns rows [r*M/g, (r+1)*M/g) of A and of C; B, bias and weights are replicated; the
shards of C are completed on every rank by ONE in-place all-gather (rank order = shard order:
NVSwitch gives every pair of GPUs the same bandwidth, so there is no placement to tune).
The reference has no multi-device execution; its only partitioning logic is the contiguous
chunking of include/cg/backend/parallel_executor.hpp:55-79, which this follows (even split, the
first `extra` shards one unit longer) - except that the in-place all-gather needs equal shards, so
an uneven M is padded up to a multiple of g by `padded_rows`.
"""


def shard_bounds(total, world, rank):
    """Half-open [lo, hi) of `rank`'s contiguous share of `total` units (ParallelExecutor's rule)."""
    if world < 1 or not (0 <= rank < world) or total < 0:
        raise ValueError("bad shard request")
    per, extra = divmod(total, world)
    lo = rank * per + min(rank, extra)
    return lo, lo + per + (1 if rank < extra else 0)


def padded_rows(total, world):
    """Rows per rank when every shard must have the same size (all-gather), and the padded total."""
    per = -(-total // world)
    return per, per * world


def equal_shard(total, world, rank):
    """[lo, hi) clipped to `total` for equal-size shards of the padded range."""
    per, _ = padded_rows(total, world)
    lo = min(rank * per, total)
    return lo, min(lo + per, total)
