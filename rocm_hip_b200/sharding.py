"""Row sharding of the layer-op path over the GPUs of one box: every token row is independent, so a rank owns a
contiguous row range, the gammas and the quantised table are replicated, and nothing is exchanged. The only
collective a multi-GPU run needs is the benchmark's barrier and its max over ranks of the device-timed duration."""


def shard(T, rank, world):
    """Rows [lo, hi) of `rank` out of `world` for T rows: contiguous, disjoint, covering, sizes differing by <= 1."""
    return T * rank // world, T * (rank + 1) // world


def shard_positions(pos0, lo):
    """A shard starting at row lo of a batch whose row t sits at position pos0 + t starts at pos0 + lo."""
    return pos0 + lo
