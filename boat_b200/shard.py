"""Host-side bookkeeping of the data-parallel attention step.

The path shards over (batch, head) units.  Two ways to own them:

* whole batch entries (weak scaling: every rank brings its own slice of a growing global batch) -
  `batch_range`, `unit_range`, `element_offset`;
* a contiguous range of units of ONE fixed [B, S, H] problem, at head granularity (strong scaling:
  B=4 with 16 heads is 64 units, 8 per GPU on 8 GPUs, i.e. half a sequence of one batch entry) -
  `head_unit_range`, `unit_rows`.  Boat's head split is a reshape, so with the head count dividing
  S, unit u owns exactly rows [u*S/heads, (u+1)*S/heads) of the flattened [B*S, H] input.

Either way forward and the input gradients need no exchange and the only collective is the sum
of the parameter-gradient bucket.  Contiguous equal ranges are cost-balanced even with a causal
mask, because every unit is a full S x S problem of its own.
"""


def split_range(n, world, rank):
    """[begin, end) of `n` items for rank `rank` of `world`; earlier ranks take the remainder."""
    if not 0 <= rank < world:
        raise ValueError("rank %d outside world %d" % (rank, world))
    base, extra = divmod(n, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def batch_range(global_batch, world, rank):
    """[begin, end) of the batch entries rank `rank` owns."""
    return split_range(global_batch, world, rank)


def unit_range(global_batch, heads, world, rank):
    """Whole-batch-entry ownership expressed in (batch, head) units."""
    b0, b1 = batch_range(global_batch, world, rank)
    return b0 * heads, b1 * heads


def element_offset(global_batch, seq, hidden, world, rank):
    """Offset, in elements of the [global_batch, seq, hidden] input, of this rank's slice."""
    return batch_range(global_batch, world, rank)[0] * seq * hidden


def head_unit_range(global_batch, heads, world, rank):
    """[begin, end) of the global_batch*heads units of one fixed problem, split at head granularity."""
    return split_range(global_batch * heads, world, rank)


def unit_rows(units, seq, heads):
    """Token rows [begin, end) of the flattened [B*seq, H] input that the unit range `units` owns.
    Needs heads to divide seq (otherwise a unit's pseudo-rows straddle token rows and only whole
    batch entries can be split off)."""
    if seq % heads != 0:
        raise ValueError("sequence length %d is not a multiple of the head count %d: split whole batch entries "
                         "instead" % (seq, heads))
    per_unit = seq // heads
    return units[0] * per_unit, units[1] * per_unit
