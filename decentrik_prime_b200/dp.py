"""Data parallelism over token rows: the only way this path shards.

Every projection is row-independent (y[m, :] depends on x[m, :] only) and the NF4 weights are
read-only, so rank g of G takes a contiguous block of packed token rows, all weights and LoRA factors
are replicated, forward and dX need no communication, and the single exchange is the sum of the fp32
LoRA gradients (blocks.GradBucket.all_reduce). The reference itself is single-GPU
(solution/integration.py:466-467); this layer is an addition.
"""


def shard_rows(n_rows, world, rank, multiple=128):
    """[start, end) of the packed token rows rank `rank` of `world` owns. Boundaries fall on multiples
    of `multiple` (the kernels' 128-row M tile) so that no tile straddles two ranks; sequence
    boundaries need not be respected because attention is outside the path."""
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    units = -(-n_rows // multiple)
    lo = (units * rank) // world * multiple
    hi = (units * (rank + 1)) // world * multiple
    return min(lo, n_rows), min(hi, n_rows)
