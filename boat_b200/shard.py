"""Host-side bookkeeping of the data-parallel attention step.

The path shards over (batch, head) units: rank r of `world` owns a contiguous range of the
global batch, computes forward and backward on it with no exchange, and the only collective
is the sum of the parameter-gradient bucket.  Contiguous equal ranges are cost-balanced even
with a causal mask, because every unit is a full S x S problem of its own.
"""


def batch_range(global_batch, world, rank):
    """[begin, end) of the batch entries rank `rank` owns; earlier ranks take the remainder."""
    if not 0 <= rank < world:
        raise ValueError("rank %d outside world %d" % (rank, world))
    base, extra = divmod(global_batch, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def unit_range(global_batch, heads, world, rank):
    """The same ownership expressed in (batch, head) units."""
    b0, b1 = batch_range(global_batch, world, rank)
    return b0 * heads, b1 * heads


def element_offset(global_batch, seq, hidden, world, rank):
    """Offset, in elements of the [global_batch, seq, hidden] input, of this rank's slice."""
    return batch_range(global_batch, world, rank)[0] * seq * hidden
