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


def local_rows(first, rows, ranges, rank):
    """The part of the global rows [first, first + rows) that rank `rank` holds, as rows of its own
    buffers (row 0 of a shard's buffers is the token at its range's start): (local_first, count);
    count 0 when the shard holds none of them."""
    lo, hi = ranges[rank]
    a, b = max(first, lo), min(first + rows, hi)
    return (a - lo, b - a) if b > a else (0, 0)


def local_capacity(tokens, ranges, rank, align=128):
    """Rows rank `rank`'s cache needs so that the sequence's first `tokens` tokens have a place: the
    length of its range below `tokens`, rounded up to the cache chunk (KV_ALIGN).  The cuts of `ranges`
    never move, so growing a sharded cache (GpuKvCache::resize, src/gpu_layers.rs:249-292) is every rank
    growing its own cache to this many rows; rows already stored keep their places."""
    lo, hi = ranges[rank]
    n = min(max(tokens - lo, 0), hi - lo)
    return (n + align - 1) // align * align


def backup_save(backup, caches, first, rows, ranges, rank, stream=None):
    """RowBackup::save (src/gpu_cache.rs:234-256) over a sharded cache: the rank saves the rows of the
    global range [first, first + rows) that its shard holds (nothing, when it holds none: the backup is
    then empty and its restore a no-op).  `caches` are the rank's own caches (one per layer).  Every rank
    makes the same call; RowBackup::restore is the rank's own backup.restore(caches)."""
    a, n = local_rows(first, rows, ranges, rank)
    if n:
        backup.save(caches, a, n, stream)
    else:
        backup.clear()
    return n
