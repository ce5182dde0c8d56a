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


def _finish(procs):
    """Joins the ranks; one that is still waiting for a rank that died is ended, not waited for."""
    for p in procs:
        p.join(60)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.terminate()
        p.join(10)
    assert not alive and all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]


def _guarded(fn, rank, *args):
    """Spawn target: runs fn(rank, *args); a rank that raises still reports, so the parent fails at once."""
    out_q = args[-1]
    try:
        fn(rank, *args)
    except BaseException as e:  # noqa: BLE001 - reported to the parent, which fails the test
        out_q.put((rank, f"rank {rank} raised {type(e).__name__}: {e}"))
        raise


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
    for it in range(6):  # several exchanges in a row: both mailbox slots get used, the routes interleave
        out.zero_()
        if it % 3 == 0:    # one launch: the decode's merge CTAs publish and collect
            op.exchange_cache(m, qd, cache, group, gd, out, p, row_step=step)
        elif it % 3 == 1:  # the decode's merge CTAs store the partial into the mailboxes, a second launch collects
            op.publish_cache(m, qd, cache, group, p, row_step=step)
            group.collect(m, gd, out)
        else:              # any partial in the staging buffer: publish, then collect
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
    procs = [ctx.Process(daemon=True, target=_guarded, args=(_rank, r, world, port, 3000, m, bits, out_q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [out_q.get(timeout=120) for _ in procs]
    _finish(procs)
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
    # recovery, on the host: the ranks' exchange counters now differ (rank 0 counted the exchange, rank 1
    # never sent it); every rank resets its group to the same number between two barriers, and the next
    # exchange goes through
    torch.cuda.synchronize()
    group.reset(10)
    dist.barrier()
    out.fill_(7.0)
    assert rt.cudaMemcpy(ctypes.c_void_p(group.staging), ctypes.c_void_p(part.data_ptr()), part.numel() * 4, 3) == 0
    group.merge(1, qg, out)
    torch.cuda.synchronize()
    recovered = group.status() == 0 and bool(torch.allclose(out, torch.full_like(out, 0.25)))
    result = (result[0], result[1] and recovered)
    dist.barrier()
    out_q.put((rank, result))
    dist.destroy_process_group()


def test_collect_gives_up_when_a_peer_stays_away():
    """Failure detection without a fault: rank 1 sits out an exchange (on the host, between steps); rank
    0's collect polls words nobody writes, runs out of its bounded wait (about a second), sets the status
    word and leaves `out` alone; its context stays usable.  Then both ranks reset their groups (host side,
    between barriers) and one more exchange succeeds."""
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = 29700 + (os.getpid() + 555) % 1000
    procs = [ctx.Process(daemon=True, target=_guarded, args=(_rank_with_absent_peer, r, 2, port, out_q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(out_q.get(timeout=120) for _ in procs)
    _finish(procs)
    assert results[0] == ("timeout", True), results
    assert results[1] == ("ok", True), results


def _rank_prefill(rank, world, port, out_q):
    """A prefill chunk with the keys split over the ranks: partial over this rank's key range, row-sliced
    exchange, every rank finalises its slice of the chunk's rows."""
    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.cuda.set_device(rank)
    import saetta_macqwen_b200 as sa
    from oracle import oracle as o

    def gather(b):
        lst = [None] * world
        dist.all_gather_object(lst, b)
        return lst

    pos, tokens = 900, 72
    total = pos + tokens
    rb = lambda x: o.round_bf16(x)
    q = rb(o.normal(tokens * HEADS * DIM, 1))
    k, v = rb(o.normal(total * ROW, 2)), rb(o.normal(total * ROW, 3))
    qg = o.normal(tokens * HEADS * 2 * DIM, 4)
    to_bf16 = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda().to(torch.bfloat16)
    group = sa.PeerGroup(rank, rank, world, tokens, HEADS, gather)
    op = sa.AttGemm(rank, 4096, KV)
    p = sa.FlashParams(HEADS, KV, pos, tokens, 1.0 / 16.0)
    # this rank's keys: [cuts[rank], cuts[rank + 1]), cut at multiples of 64; it STORES only those rows
    # (row 0 of its buffers is the key at global position cuts[rank])
    cuts = [min(total, (total * r // world + 63) // 64 * 64) for r in range(world)] + [total]
    lo_k, hi_k = cuts[rank], cuts[rank + 1]
    mine_k, mine_v = to_bf16(k[lo_k * ROW:hi_k * ROW]), to_bf16(v[lo_k * ROW:hi_k * ROW])
    out = torch.zeros(tokens * HEADS * DIM, device="cuda")
    gd = torch.from_numpy(qg).cuda()
    for _ in range(3):
        out.zero_()
        op.partial(to_bf16(q), mine_k, mine_v, None, group.staging, p, lo_k, hi_k, dtype=sa.BF16, key_base=lo_k)
        group.merge_sliced(tokens, gd, out)
        torch.cuda.synchronize()
        assert group.status() == 0
    lo, hi = group.slice(tokens)
    want = o.attention_rows(q, qg, k, v, [pos + i + 1 for i in range(tokens)], threads=4)
    got = out.cpu().numpy().reshape(tokens, HEADS, DIM)
    worst = float(np.abs(got[lo:hi] - want[lo:hi]).max())
    untouched = bool((got[:lo] == 0).all() and (got[hi:] == 0).all())
    dist.barrier()
    out_q.put((rank, (worst, untouched, hi - lo)))
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_prefill_partials_exchanged_by_row_slices(world):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = 29700 + (os.getpid() + 333 + world) % 1000
    procs = [ctx.Process(daemon=True, target=_guarded, args=(_rank_prefill, r, world, port, out_q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(out_q.get(timeout=120) for _ in procs)
    _finish(procs)
    assert sum(r[2] for r in results.values()) == 72
    for rank, (worst, untouched, _) in results.items():
        assert worst < 2e-3 and untouched, (rank, worst, untouched)


def _rank_batch(rank, world, port, out_q):
    """Ragged batch decode with every sequence's keys split over the ranks."""
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

    lens, bits = [700, 64, 2500, 333, 1024], 8
    n = len(lens)
    q, qg = o.normal(n * HEADS * DIM, 50), o.normal(n * HEADS * 2 * DIM, 51)
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    caches, mine, refs = [], [], []
    for i, L in enumerate(lens):
        k, v = o.normal(L * ROW, 60 + i), o.normal(L * ROW, 80 + i)
        lo, hi = shard.shard_ranges(L, world)[rank]
        c = sa.GpuKvCache(rank, bits, max(hi - lo, 128))
        if hi > lo:  # the 64-token sequence fits in rank 0's shard: rank 1 publishes an empty partial for it
            c.store_at(dev(k[lo * ROW:hi * ROW]), dev(v[lo * ROW:hi * ROW]), 0, hi - lo)
        caches.append(c), mine.append(hi - lo), refs.append((o.round_trip(k, bits), o.round_trip(v, bits)))
    op = sa.DecodeBatch(rank, 8)
    group = sa.PeerGroup(rank, rank, world, 8, HEADS, gather)
    out = torch.zeros(n * HEADS * DIM, device="cuda")
    qd, gd = dev(q), dev(qg)
    worst = 0.0
    for _ in range(3):
        out.zero_()
        op.publish(caches, mine, qd, group)
        group.collect(n, gd, out)
        torch.cuda.synchronize()
        assert group.status() == 0
        got = out.cpu().numpy().reshape(n, HEADS, DIM)
        for i, L in enumerate(lens):
            want = o.attention_rows(q.reshape(n, -1)[i], qg.reshape(n, -1)[i], refs[i][0], refs[i][1], [L])
            worst = max(worst, float(np.abs(got[i] - want[0]).max()))
    dist.barrier()
    out_q.put((rank, worst))
    dist.destroy_process_group()


def test_ragged_batch_split_over_two_ranks():
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = 29700 + (os.getpid() + 444) % 1000
    procs = [ctx.Process(daemon=True, target=_guarded, args=(_rank_batch, r, 2, port, out_q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out_q.get(timeout=120) for _ in procs]
    _finish(procs)
    for rank, err in results:
        assert err < 2e-3, (rank, err)
