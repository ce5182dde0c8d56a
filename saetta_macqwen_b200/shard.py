"""Host-side plan for split-KV sharding across the GPUs of one box.

No counterpart in the reference (it runs on one GPU).  Attention over disjoint
key sets composes through (m, l, O) exactly as the reference's chunk merge does
(kernels/attention.metal:381-408): each rank holds a contiguous range of a
sequence's KV rows, computes partials over it, the partials are all-gathered and
merged.  This module only decides who holds what and which rows a shard's
kernel may see; the kernels are in the shared library.
"""


def shard_ranges(tokens, world, align=128):
    """Contiguous [lo, hi) token ranges, one per rank, cut at multiples of `align`
    (the cache chunk, KV_ALIGN) so every shard keeps the reference's row layout."""
    if world < 1:
        raise ValueError("world must be >= 1")
    chunks = (tokens + align - 1) // align
    out = []
    for r in range(world):
        lo = min(tokens, chunks * r // world * align)
        hi = min(tokens, chunks * (r + 1) // world * align)
        out.append((lo, hi))
    return out


def owner_of(position, ranges):
    """Rank whose shard holds token `position` (new rows are appended there)."""
    for r, (lo, hi) in enumerate(ranges):
        if lo <= position < hi:
            return r
    return len(ranges) - 1


def local_decode_params(position, m, ranges, rank):
    """What rank `rank` passes to saetta_decode_partial_cache for m verify rows at
    `position`..`position+m-1` of the global sequence: (local_kv_len, row_step).

    Row r sees global keys 0..position+r.  A shard entirely below `position`
    shows all its rows to every query row (row_step 0).  The shard holding the
    new rows shows row r one more key per row (row_step 1).  A shard with no
    visible key returns kv_len 0 and must be skipped by the caller (its partial
    is m = -inf, l = 0)."""
    lo, hi = ranges[rank]
    first_new = position  # global index of row 0's own key
    if hi <= first_new:
        return hi - lo, 0
    if lo > first_new + m - 1:
        return 0, 0
    if lo > first_new:
        raise ValueError("the new rows must lie inside one shard")
    return first_new + 1 - lo, 1
