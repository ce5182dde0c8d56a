"""Split-KV across shards on one GPU: two caches stand for two ranks' shards,
each produces (m, l, O) partials through saetta_decode_partial_cache, and
saetta_merge_partials must reproduce the oracle on the whole sequence."""
import numpy as np
import pytest

import saetta_macqwen_b200 as sa
from saetta_macqwen_b200 import shard
from util import DIM, HEADS, KV, ROW, dev, max_abs, params_dev, rel_rms

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits,m,world", [(8, 1, 2), (8, 4, 3), (4, 2, 2), (16, 1, 2)])
def test_sharded_partials_merge_to_the_whole(oracle, bits, m, world):
    import torch

    tokens = 3000
    pos = tokens - m
    keys, values = oracle.normal(tokens * ROW, 1), oracle.normal(tokens * ROW, 2)
    q, qg = oracle.normal(m * HEADS * DIM, 3), oracle.normal(m * HEADS * 2 * DIM, 4)
    ranges = shard.shard_ranges(tokens, world)
    parts = torch.zeros((world, m * HEADS * sa.PART_STRIDE), device="cuda")
    op = sa.AttentionRows(0, HEADS, KV, 4096, m)
    caches = []
    for r, (lo, hi) in enumerate(ranges):
        c = sa.GpuKvCache(0, bits, hi - lo)
        c.store_at(dev(keys[lo * ROW:hi * ROW]), dev(values[lo * ROW:hi * ROW]), 0, hi - lo)
        caches.append(c)
        kv_len, step = shard.local_decode_params(pos, m, ranges, r)
        assert kv_len > 0
        p = torch.tensor([0, kv_len - 1, kv_len, 0], dtype=torch.int32, device="cuda")
        op.partial_cache(m, dev(q), c, parts[r], p, row_step=step)
    out = torch.zeros(m * HEADS * DIM, device="cuda")
    sa.merge_partials(0, parts, world, m, HEADS, dev(qg), out)
    torch.cuda.synchronize()
    got = out.cpu().numpy().reshape(m, HEADS, DIM)
    kr, vr = oracle.round_trip(keys, bits), oracle.round_trip(values, bits)
    want = oracle.attention_rows(q, qg, kr, vr, [pos + r + 1 for r in range(m)], threads=8)
    assert max_abs(got, want) < 2e-3 and rel_rms(got, want) < 1e-3, (max_abs(got, want), rel_rms(got, want))


@pytest.mark.parametrize("bits", [8, 16])
def test_row_backup_and_resize_over_shards(oracle, bits):
    """RowBackup::save / restore and GpuKvCache::resize (src/gpu_cache.rs:234-274, src/gpu_layers.rs:249-292)
    over a cache whose rows are split over three shards: every shard saves the part of a global row range it
    holds (the range spans a cut), the rows are overwritten as a rejected speculation would, and restored;
    a shard grows to take more of its range without moving a stored row.  Checked by decoding the whole
    sequence through the shards' partials before and after."""
    import torch

    tokens, world, m = 1500, 3, 1
    keys, values = oracle.normal(tokens * ROW, 11), oracle.normal(tokens * ROW, 12)
    q, qg = oracle.normal(HEADS * DIM, 13), oracle.normal(HEADS * 2 * DIM, 14)
    ranges = shard.shard_ranges(2048, world)  # cuts fixed by the sequence's maximum length
    op = sa.AttentionRows(0, HEADS, KV, 4096, m)
    caches = []
    for r, (lo, hi) in enumerate(ranges):
        n = max(min(tokens, hi) - lo, 0)
        c = sa.GpuKvCache(0, bits, max(shard.local_capacity(tokens, ranges, r), 128))
        if n:
            c.store_at(dev(keys[lo * ROW:(lo + n) * ROW]), dev(values[lo * ROW:(lo + n) * ROW]), 0, n)
        caches.append(c)

    def attend(total):
        parts = torch.zeros((world, HEADS * sa.PART_STRIDE), device="cuda")
        live = 0
        for r in range(world):
            kv_len, step = shard.local_decode_params(total - 1, 1, ranges, r)
            if kv_len:
                p = torch.tensor([0, kv_len - 1, kv_len, 0], dtype=torch.int32, device="cuda")
                op.partial_cache(1, dev(q), caches[r], parts[live], p, row_step=step)
                live += 1
        out = torch.zeros(HEADS * DIM, device="cuda")
        sa.merge_partials(0, parts[:live].contiguous(), live, 1, HEADS, dev(qg), out)
        torch.cuda.synchronize()
        return out.cpu().numpy()

    before = attend(tokens)
    first, rows = ranges[0][1] - 3, 9  # spans the cut between shards 0 and 1
    backups = [sa.RowBackup() for _ in range(world)]
    held = [shard.backup_save(backups[r], [caches[r]], first, rows, ranges, r) for r in range(world)]
    assert held == [3, 6, 0] and backups[2].bytes() == 0
    junk = oracle.normal(rows * ROW, 15) * 3.0
    for r in range(world):
        a, n = shard.local_rows(first, rows, ranges, r)
        if n:
            off = (ranges[r][0] + a - first) * ROW
            caches[r].store_at(dev(junk[off:off + n * ROW]), dev(junk[off:off + n * ROW]), a, n)
    assert not np.array_equal(attend(tokens), before)
    for r in range(world):
        backups[r].restore([caches[r]])
    assert np.array_equal(attend(tokens), before)  # byte-exact rows back: bit-identical output

    # the sequence grows into the last shard: it alone resizes; the others keep their rows
    more = 1900
    k2, v2 = oracle.normal((more - tokens) * ROW, 16), oracle.normal((more - tokens) * ROW, 17)
    for r in range(world):
        need = shard.local_capacity(more, ranges, r)
        if need > caches[r].capacity:
            caches[r].resize(need)
    for r, (lo, hi) in enumerate(ranges):
        a, n = shard.local_rows(tokens, more - tokens, ranges, r)
        if n:
            off = (lo + a - tokens) * ROW
            caches[r].store_at(dev(k2[off:off + n * ROW]), dev(v2[off:off + n * ROW]), a, n)
    got = attend(more).reshape(1, HEADS, DIM)
    kk, vv = np.concatenate([keys, k2]), np.concatenate([values, v2])
    rt = (lambda x: oracle.round_trip(x, bits)) if bits != 16 else oracle.round_f16
    want = oracle.attention_rows(q, qg, rt(kk), rt(vv), [more], threads=8)
    assert max_abs(got, want) < 2e-3 and rel_rms(got, want) < 1e-3, (max_abs(got, want), rel_rms(got, want))
