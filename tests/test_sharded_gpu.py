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
