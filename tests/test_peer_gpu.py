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



def _rank_with_absent_peer(rank, world, port, out_q):
    import time

    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.cuda.set_device(rank)
    import saetta_macqwen_b200 as sa

    def gather(b):
        lst = [None] * world
        dist.all_gather_object(lst, b)
        return lst

    group = sa.PeerGroup(rank, rank, world, 1, HEADS, gather)
    qg = torch.zeros(HEADS * 2 * DIM, device="cuda")
    out = torch.full((HEADS * DIM,), 7.0, device="cuda")
    part = torch.zeros(HEADS, sa.PART_STRIDE, device="cuda")
    part[:, :DIM], part[:, 256], part[:, 257] = 2.0, 0.0, 4.0  # O, m, l
    import ctypes
    rt = ctypes.CDLL("libcudart.so.12")
    rt.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
    assert rt.cudaMemcpy(ctypes.c_void_p(group.staging), ctypes.c_void_p(part.data_ptr()), part.numel() * 4, 3) == 0
    group.merge(1, qg, out)  # one ordinary exchange: both ranks publish
    torch.cuda.synchronize()
    ok = group.status() == 0 and bool(torch.allclose(out, torch.full_like(out, 0.25)))
    dist.barrier()
    result = ("ok", ok)
    if rank == 0:  # the next exchange: rank 1 stays away, between steps, with nothing in flight
        out.fill_(7.0)
        t0 = time.perf_counter()
        group.merge(1, qg, out)
        torch.cuda.synchronize()
        waited = time.perf_counter() - t0
        try:
            group.status()
            code = 0
        except sa.SaettaError as e:
            code = e.code
        result = ("timeout", ok and code == sa.TIMEOUT and waited < 20.0 and bool((out == 7.0).all()))
        # the GPU still answers
        x = torch.ones(8, device="cuda")
        result = (result[0], result[1] and float(x.sum()) == 8.0)
    dist.barrier()
    out_q.put((rank, result))
    dist.destroy_process_group()


def test_collect_gives_up_when_a_peer_stays_away():
    """Failure detection without a fault: rank 1 sits out an exchange (on the host, between steps); rank
    0's collect polls words nobody writes, runs out of its bounded wait (about a second), sets the status
    word and leaves `out` alone; its context stays usable."""
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = 29700 + (os.getpid() + 555) % 1000
    procs = [ctx.Process(target=_rank_with_absent_peer, args=(r, 2, port, out_q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(out_q.get(timeout=240) for _ in procs)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert results[0] == ("timeout", True), results
    assert results[1] == ("ok", True), results
