"""Split-KV sharding with two CPU ranks (gloo): the host plan and the (m, l, O)
merge algebra the GPU path uses across ranks, with no GPU involved.

Each rank computes the partial of its shard in numpy, the partials are
all-gathered and merged exactly as saetta_merge_partials does, and the result
must equal the oracle on the whole sequence.
"""
import os

import numpy as np
import pytest

from saetta_macqwen_b200 import shard

HEADS, KV, DIM, STRIDE = 16, 2, 256, 264


def test_shard_ranges_cover_and_align():
    for tokens, world in [(262144, 8), (32768, 2), (1000, 4), (100, 8), (1, 2)]:
        r = shard.shard_ranges(tokens, world)
        assert r[0][0] == 0 and r[-1][1] == tokens and len(r) == world
        for (a, b), (c, d) in zip(r, r[1:]):
            assert b == c and a <= b
        assert all(lo % 128 == 0 for lo, _ in r)
    ranges = shard.shard_ranges(1000, 4)
    assert shard.owner_of(999, ranges) == 3 and shard.owner_of(0, ranges) == 0
    assert shard.local_decode_params(996, 4, ranges, 0) == (ranges[0][1], 0)
    kv_len, step = shard.local_decode_params(996, 4, ranges, 3)
    assert step == 1 and kv_len == 996 + 1 - ranges[3][0]


def partial(q, keys, values, lens):
    """(O, m, l) of rows over keys[:len] in the layout of the exchanged partial."""
    rows = len(lens)
    out = np.zeros((rows, HEADS, STRIDE), np.float32)
    for r in range(rows):
        for h in range(HEADS):
            kv = h // (HEADS // KV)
            n = lens[r]
            if n == 0:
                out[r, h, 256] = -np.inf
                continue
            s = (keys[:n, kv] @ q[r, h]).astype(np.float64) / 16.0 * np.log2(np.e)
            m = s.max()
            p = np.exp2(s - m)
            out[r, h, :256] = p @ values[:n, kv]
            out[r, h, 256], out[r, h, 257] = m, p.sum()
    return out


def merge(parts, qg):
    m = parts[..., 256].max(0)
    w = np.where(np.isinf(parts[..., 256]), 0.0, np.exp2(parts[..., 256] - m))
    l = (parts[..., 257] * w).sum(0)
    o = (parts[..., :256] * w[..., None]).sum(0)
    g = qg.reshape(o.shape[0], HEADS, 2 * DIM)[..., DIM:]
    return o / l[..., None] / (1.0 + np.exp(-g))


def _rank(rank, world, port, tokens, m, out_q):
    import torch.distributed as dist
    import torch

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as o

    pos = tokens - m
    keys = o.normal(tokens * KV * DIM, 1).reshape(tokens, KV, DIM)
    values = o.normal(tokens * KV * DIM, 2).reshape(tokens, KV, DIM)
    q = o.normal(m * HEADS * DIM, 3).reshape(m, HEADS, DIM)
    qg = o.normal(m * HEADS * 2 * DIM, 4)
    ranges = shard.shard_ranges(tokens, world)
    lo, hi = ranges[rank]
    kv_len, step = shard.local_decode_params(pos, m, ranges, rank)
    lens = [kv_len + r * step if kv_len else 0 for r in range(m)]
    mine = partial(q, keys[lo:hi], values[lo:hi], lens)
    gathered = [torch.zeros(mine.shape) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(mine))
    got = merge(np.stack([g.numpy() for g in gathered]), qg)
    if rank == 0:
        want = o.attention_rows(q, qg, keys, values, [pos + r + 1 for r in range(m)], threads=2)
        out_q.put(float(np.abs(got - want).max()))
    dist.destroy_process_group()


def test_local_rows_and_capacity_of_a_sharded_cache():
    """RowBackup and resize over a sharded page layout (src/gpu_cache.rs:196-280, src/gpu_layers.rs:249-292): a
    global row range falls apart into one local range per shard, disjoint and complete; capacities grow shard by
    shard without moving a stored row."""
    for tokens, world in ((3000, 2), (3000, 3), (262144, 8), (100, 4)):
        ranges = shard.shard_ranges(tokens, world)
        cuts = [hi for lo, hi in ranges if 0 < hi < tokens]
        spans = [(0, tokens), (0, 1), (tokens - 1, 1), (1000 % tokens, min(700, tokens - 1000 % tokens))]
        spans += [(cuts[0] - 1, 2)] if cuts else []  # one row either side of a cut
        for first, rows in spans:
            covered = []
            for r, (lo, hi) in enumerate(ranges):
                a, n = shard.local_rows(first, rows, ranges, r)
                assert 0 <= a and a + n <= hi - lo
                covered += [lo + a + i for i in range(n)]
            assert covered == list(range(first, first + rows)), (tokens, world, first, rows)
        # nothing beyond a shard's range, nothing for a range elsewhere
        assert shard.local_rows(tokens, 5, ranges, 0) == (0, 0)
        # growing: the capacity a rank needs is monotone in the tokens, reaches its range, and is chunk-aligned
        for r, (lo, hi) in enumerate(ranges):
            last = 0
            for t in (0, 1, lo, lo + 1, (lo + hi) // 2, hi, tokens):
                c = shard.local_capacity(t, ranges, r)
                assert c % 128 == 0 and c >= min(max(t - lo, 0), hi - lo) and c < hi - lo + 128
            caps = [shard.local_capacity(t, ranges, r) for t in range(0, tokens + 1, max(1, tokens // 50))]
            assert caps == sorted(caps)
            assert shard.local_capacity(tokens, ranges, r) >= hi - lo
            last = caps[-1]


@pytest.mark.parametrize("tokens,m", [(1000, 1), (777, 4)])
def test_two_gloo_ranks_merge_to_the_whole(tokens, m):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = 29500 + (os.getpid() + tokens) % 2000
    procs = [ctx.Process(target=_rank, args=(r, 2, port, tokens, m, out_q)) for r in range(2)]
    for p in procs:
        p.start()
    err = out_q.get(timeout=120)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert err < 2e-5, err
