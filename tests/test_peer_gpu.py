"""Split-KV decode over several GPUs with the exchange fused into the kernels:
each rank holds a slice of the sequence, stores its (m, l, O) partial into every
rank's mailbox over NVLink, and merges what arrived from local memory.  Needs
two GPUs or more (skipped otherwise); the ranks are separate processes, as in
production."""
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
    rt = (lambda x: o.round_trip(x, bits)) if bits in (4, 8) else o.round_f16
    kr, vr = rt(keys), rt(values)
    want = o.attention_rows(q, qg, kr, vr, [pos + r + 1 for r in range(m)], threads=4)
    for it in range(4):  # several exchanges in a row: both mailbox slots get used
        out.zero_()
        if it % 2 == 0:  # the decode's merge kernel stores the partial into the mailboxes itself
            op.publish_cache(m, qd, cache, group, p, row_step=step)
            group.collect(m, gd, out)
        else:            # any partial in the staging buffer: publish, then collect
            op.partial_cache(m, qd, cache, group.staging, p, row_step=step)
            group.merge(m, gd, out)
        torch.cuda.synchronize()
        assert group.status() == 0
        worst = max(worst, float(np.abs(out.cpu().numpy().reshape(m, HEADS, DIM) - want).max()))
    dist.barrier()
    out_q.put((rank, worst))
    dist.destroy_process_group()


@pytest.mark.parametrize("bits,m,world", [(8, 1, 2), (8, 4, 2), (4, 2, 2), (16, 1, 2), (8, 2, 4), (8, 1, 8)])
def test_ranks_merge_through_peer_mailboxes(bits, m, world):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = 29700 + (os.getpid() + 7 * m + world) % 1000
    procs = [ctx.Process(target=_rank, args=(r, world, port, 3000, m, bits, out_q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [out_q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, err in results:
        assert err < 2e-3, (rank, err)
