"""Split-KV decode over two GPUs with the fused peer-memory merge: each rank
holds half of the sequence, computes its (m, l, O) partial, and one kernel per
rank reads the other rank's partial over NVLink and merges.  Needs two GPUs
(skipped otherwise); the ranks are separate processes, as in production."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
HEADS, KV, DIM, ROW = 16, 2, 256, 512


def _rank(rank, world, port, tokens, m, bits, out_q):
    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.cuda.set_device(rank)
    import saetta_macqwen_b200 as sa
    from saetta_macqwen_b200 import shard
    from oracle import oracle as o

    def gather(b):
        lst = [None] * world
        dist.all_gather_object(lst, b)
        return lst

    pos = tokens - m
    keys, values = o.normal(tokens * ROW, 1), o.normal(tokens * ROW, 2)
    q, qg = o.normal(m * HEADS * DIM, 3), o.normal(m * HEADS * 2 * DIM, 4)
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    ranges = shard.shard_ranges(tokens, world)
    lo, hi = ranges[rank]
    cache = sa.GpuKvCache(rank, bits, hi - lo)
    cache.store_at(dev(keys[lo * ROW:hi * ROW]), dev(values[lo * ROW:hi * ROW]), 0, hi - lo)
    op = sa.AttentionRows(rank, HEADS, KV, 4096, m)
    group = sa.PeerGroup(rank, rank, world, m, HEADS, gather)
    kv_len, step = shard.local_decode_params(pos, m, ranges, rank)
    p = torch.tensor([0, kv_len - 1, kv_len, 0], dtype=torch.int32, device="cuda")
    out = torch.zeros(m * HEADS * DIM, device="cuda")
    qd, gd = dev(q), dev(qg)
    worst = 0.0
    kr, vr = o.round_trip(keys, bits), o.round_trip(values, bits)
    want = o.attention_rows(q, qg, kr, vr, [pos + r + 1 for r in range(m)], threads=4)
    for _ in range(3):  # several exchanges in a row: both mailbox slots get used
        out.zero_()
        op.partial_cache(m, qd, cache, group.staging, p, row_step=step)
        group.merge(m, gd, out)
        torch.cuda.synchronize()
        assert group.status() == 0
        worst = max(worst, float(np.abs(out.cpu().numpy().reshape(m, HEADS, DIM) - want).max()))
    dist.barrier()
    out_q.put((rank, worst))
    dist.destroy_process_group()


@pytest.mark.parametrize("bits,m", [(8, 1), (8, 4)])
def test_two_ranks_merge_over_peer_memory(bits, m):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = 29700 + (os.getpid() + m) % 1000
    procs = [ctx.Process(target=_rank, args=(r, 2, port, 3000, m, bits, out_q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out_q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, err in results:
        assert err < 2e-3, (rank, err)
