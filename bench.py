#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A step is one decode token's attention (split-KV kernel + merge/gate kernel per
layer) over LAYERS separate 8-bit KV caches of CTX tokens, so every cache byte
comes from HBM (the caches of one step are far larger than L2).  Rank r of N
holds its own CTX-token shard of an N*CTX-token context (split-KV by sequence);
the per-shard (m, l, O) partials are all-gathered over NCCL and merged, which is
the path's only exchange.  The printed value is the whole job's algorithmic KV
bytes per second.  Further measured points (32k decode, MTP verify, 4-bit,
ragged batch, prefill TFLOP/s) ride along under "points".

--impl reference times the reference's CPU attention (the oracle restatement,
all host threads) on a bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HEADS, KV, DIM = 16, 2, 256
ROW = KV * DIM
BYTES_PER_TOKEN = {8: 1088, 4: 576, 16: 2048}  # K + V, both kv heads, codes + scales + biases
CTX = 262144
LAYERS = 4
TRAFFIC_PER_TOKEN = 1125.4  # measured dram bytes per token per layer (ncu), see profiles/
METRIC = "Decode-attn achieved HBM GB/s @32k/256k KV; prefill-attn TFLOP/s per 4k chunk"


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return p["hbm_gbs"], p["bf16_tflops"], "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx = max(mx, float(s[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def fill_cache(sa, torch, cache, tokens, seed):
    """N(0,1) K and V rows quantised on the device by the store kernel (bit-exact
    with the oracle's quantiser, which the parity tests pin)."""
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    chunk = 8192
    for p in range(0, tokens, chunk):
        n = min(chunk, tokens - p)
        k = torch.randn(n * ROW, device="cuda", generator=g)
        v = torch.randn(n * ROW, device="cuda", generator=g)
        cache.store_at(k, v, p, n)


def time_graph(torch, fn, steps, warmup, stream):
    """CUDA-event time of `steps` replays of fn() captured once in a CUDA graph
    (record once, replay per token, as the reference replays its plan)."""
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        fn()
        stream.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            fn()
        for _ in range(warmup):
            graph.replay()
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
    return e0.elapsed_time(e1) / steps


def decode_point(sa, torch, ctx, bits, m, layers, steps, warmup, stream):
    """GB/s of one m-row decode/verify step over `layers` caches of `ctx` tokens."""
    cap = ctx + 128
    caches = [sa.GpuKvCache(torch.cuda.current_device(), bits, cap) for _ in range(layers)]
    for i, c in enumerate(caches):
        fill_cache(sa, torch, c, ctx + m - 1, 1000 + i)
    dev = torch.cuda.current_device()
    op = sa.AttentionRows(dev, HEADS, KV, cap, m)
    q = torch.randn(m * HEADS * DIM, device="cuda")
    qg = torch.randn(m * HEADS * 2 * DIM, device="cuda")
    out = torch.zeros(m * HEADS * DIM, device="cuda")
    params = torch.tensor([0, ctx - 1, ctx, 0], dtype=torch.int32, device="cuda")

    def step():
        for c in caches:
            op.record_cache(m, q, c, qg, out, params, stream=stream)

    ms = time_graph(torch, step, steps, warmup, stream)
    nbytes = layers * (ctx + m - 1) * BYTES_PER_TOKEN[bits]
    assert op.device_status(stream=stream) == 0
    return {"gbs": nbytes / ms / 1e6, "us_per_layer": ms * 1e3 / layers, "layers": layers, "launches": 2 * layers}


def batch_point(sa, torch, bits, steps, warmup, stream, seqs=64, lo=8192, hi=262144, seed=5):
    """Config 5: 64 sequences, ragged lengths U[8192, 262144], one row each."""
    rng = np.random.default_rng(seed)
    lens = rng.integers(lo, hi + 1, seqs)
    dev = torch.cuda.current_device()
    caches = []
    for i, n in enumerate(lens):
        c = sa.GpuKvCache(dev, bits, int(n))
        fill_cache(sa, torch, c, int(n), 2000 + i)
        caches.append(c)
    op = sa.DecodeBatch(dev, seqs)
    q = torch.randn(seqs * HEADS * DIM, device="cuda")
    qg = torch.randn(seqs * HEADS * 2 * DIM, device="cuda")
    out = torch.zeros(seqs * HEADS * DIM, device="cuda")
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            op.record(caches, lens, q, qg, out, stream=stream)
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            op.record(caches, lens, q, qg, out, stream=stream)
        e1.record(stream)
        stream.synchronize()
    ms = e0.elapsed_time(e1) / steps
    nbytes = int(lens.sum()) * BYTES_PER_TOKEN[bits]
    return {"gbs": nbytes / ms / 1e6, "ms": ms, "tokens": int(lens.sum()), "seqs": seqs}


def prefill_point(sa, torch, pos, tokens, steps, warmup, stream, quant_bits=None):
    """TFLOP/s of one causal chunk (flops = 4*H*D*(t*pos + t(t+1)/2), src/attention_prefill.rs:139-142)."""
    dev = torch.cuda.current_device()
    total = pos + tokens
    q = torch.randn(tokens * HEADS * DIM, device="cuda").to(torch.bfloat16)
    qg = torch.randn(tokens * HEADS * 2 * DIM, device="cuda")
    out = torch.zeros(tokens * HEADS * DIM, device="cuda")
    op = sa.AttGemm(dev, tokens, KV)
    p = sa.FlashParams(HEADS, KV, pos, tokens, 1.0 / 16.0)
    if quant_bits:
        cache = sa.GpuKvCache(dev, quant_bits, total)
        fill_cache(sa, torch, cache, total, 77)
        quant = cache.quant()
        op.reserve(total)
        fn = lambda: op.encode(q, None, None, quant, qg, out, p, dtype=sa.BF16, stream=stream)
    else:
        k = torch.randn(total * ROW, device="cuda").to(torch.bfloat16)
        v = torch.randn(total * ROW, device="cuda").to(torch.bfloat16)
        fn = lambda: op.encode(q, k, v, None, qg, out, p, dtype=sa.BF16, stream=stream)
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            fn()
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        stream.synchronize()
    ms = e0.elapsed_time(e1) / steps
    flops = 4.0 * HEADS * DIM * (tokens * pos + tokens * (tokens + 1) / 2)
    return {"tflops": flops / ms / 1e9, "ms": ms, "flops": flops}


def half_point(sa, torch, ctx, layers, steps, warmup, stream):
    """Decode over a binary16 cache (the reference's default cache format): 2048 bytes per token."""
    dev = torch.cuda.current_device()
    caches = [sa.GpuKvCache(dev, 16, ctx, dtype=sa.F16) for _ in range(layers)]
    x = torch.randn(4096 * ROW, device="cuda")
    for c in caches:
        for p0 in range(0, ctx, 4096):
            c.store_at(x, x.flip(0).contiguous(), p0, min(4096, ctx - p0))
    op = sa.AttentionRows(dev, HEADS, KV, ctx, 1)
    q = torch.randn(HEADS * DIM, device="cuda")
    qg = torch.randn(HEADS * 2 * DIM, device="cuda")
    out = torch.zeros(HEADS * DIM, device="cuda")
    params = torch.tensor([0, ctx - 1, ctx, 0], dtype=torch.int32, device="cuda")

    def step():
        for c in caches:
            op.record_cache(1, q, c, qg, out, params, stream=stream)

    with torch.cuda.stream(stream):
        step()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step()
        for _ in range(warmup):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
    ms = e0.elapsed_time(e1) / steps / layers
    assert op.device_status(stream=stream) == 0
    return {"gbs": ctx * 2048 / ms / 1e6, "us_per_layer": ms * 1e3, "layers": layers}


def qmv_point(sa, torch, rows, cols, bits, m, steps, warmup, stream):
    """GB/s of weights for y[m][rows] = x[m][cols] W^T over MLX affine matrices; sixteen matrices rotate so
    that no launch finds its weights in L2."""
    dev = torch.cuda.current_device()
    copies = 16
    words = [torch.randint(-2**31, 2**31 - 1, (rows * cols * bits // 32,), dtype=torch.int32, device="cuda") for _ in range(copies)]
    scales = torch.full((rows * cols // 64,), 0x3C00, dtype=torch.int16, device="cuda")  # bfloat16 0.0078
    biases = torch.full((rows * cols // 64,), -0x4200, dtype=torch.int16, device="cuda")
    x = torch.randn(m * cols, device="cuda")
    y = torch.zeros(m * rows, device="cuda")
    # recorded once and replayed as one graph, the way the per-token plan issues them: launched one by one
    # from the host a kernel this short is bounded by the launch rate
    per_plan = 4 * copies
    plan = sa.Plan(dev)
    with plan.recording():
        for i in range(per_plan):
            sa.qmv_rows(dev, words[i % copies], scales, biases, bits, rows, cols, m, x, y, stream=plan.stream)
    for _ in range(max(warmup, 3)):
        plan.run()
    reps = max(1, steps // per_plan)
    ms = sum(plan.run_timed() for _ in range(reps)) / (reps * per_plan)
    nbytes = rows * cols * bits // 8 + 2 * (rows * cols // 64) * 2
    return {"gbs": nbytes / ms / 1e6, "us": ms * 1e3, "bytes": nbytes}


def prep_point(sa, torch, tokens, bits, steps, warmup, stream):
    """GB/s of attention prep fused with the quantised store for one prefill chunk: reads the q halves of
    q_and_gate, k, v (f32), writes q as bf16 and the cache rows.  The inputs of consecutive steps are
    distinct buffers, larger than L2 together."""
    dev = torch.cuda.current_device()
    copies = 6
    qg = [torch.randn(tokens * HEADS * 2 * DIM, device="cuda") for _ in range(copies)]
    k = [torch.randn(tokens * ROW, device="cuda") for _ in range(copies)]
    v = [torch.randn(tokens * ROW, device="cuda") for _ in range(copies)]
    qn, kn = torch.ones(DIM, device="cuda"), torch.ones(DIM, device="cuda")
    q_out = torch.zeros(tokens * HEADS * DIM, dtype=torch.bfloat16, device="cuda")
    cache = sa.GpuKvCache(dev, bits, tokens)
    pp = sa.PrepParams(HEADS, KV, DIM, 64, 1.0e7, 1.0e-6)
    fn = lambda i: sa.attention_prep(pp, tokens, qg[i % copies], k[i % copies], v[i % copies], qn, kn, q_out, sa.BF16,
                                     cache, pos=0, stream=stream)
    with torch.cuda.stream(stream):
        for i in range(warmup):
            fn(i)
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(steps):
            fn(i)
        e1.record(stream)
        stream.synchronize()
    ms = e0.elapsed_time(e1) / steps
    nbytes = tokens * (HEADS * DIM * 4 + 2 * ROW * 4 + HEADS * DIM * 2 + BYTES_PER_TOKEN[bits])
    return {"gbs": nbytes / ms / 1e6, "ms": ms, "bytes": nbytes}


_CPU_DATA = {}


def point_table(sa, torch, stream, s, w):
    return {
        "decode_32k_8bit": lambda: decode_point(sa, torch, 32768, 8, 1, 10, s, w, stream),
        "decode_128k_8bit": lambda: decode_point(sa, torch, 131072, 8, 1, 4, s, w, stream),
        "decode_256k_8bit": lambda: decode_point(sa, torch, 262144, 8, 1, 4, s, w, stream),
        "decode_256k_4bit": lambda: decode_point(sa, torch, 262144, 4, 1, 4, s, w, stream),
        "decode_128k_f16": lambda: half_point(sa, torch, 131072, 4, s, w, stream),
        "verify_m4_32k_8bit": lambda: decode_point(sa, torch, 32768, 8, 4, 10, s, w, stream),
        "batch64_ragged_8bit": lambda: batch_point(sa, torch, 8, min(s, 3), 2, stream),
        "batch64_ragged_4bit": lambda: batch_point(sa, torch, 4, min(s, 3), 2, stream),
        "qmv_8192x2048_5bit_m1": lambda: qmv_point(sa, torch, 8192, 2048, 5, 1, max(s, 32), w, stream),
        "qmv_8192x2048_5bit_m4": lambda: qmv_point(sa, torch, 8192, 2048, 5, 4, max(s, 32), w, stream),
        "qmv_2048x4096_5bit_m1": lambda: qmv_point(sa, torch, 2048, 4096, 5, 1, max(s, 32), w, stream),
        "prep_store_4k_8bit": lambda: prep_point(sa, torch, 4096, 8, max(s, 12), w, stream),
        "prefill_4k_pos0_bf16": lambda: prefill_point(sa, torch, 0, 4096, s, w, stream),
        "prefill_4k_pos32k_8bit": lambda: prefill_point(sa, torch, 32768, 4096, min(s, 5), 2, stream, quant_bits=8),
        "prefill_4k_pos128k_8bit": lambda: prefill_point(sa, torch, 131072, 4096, min(s, 3), 2, stream, quant_bits=8),
    }


def run_only(args):
    """One point alone, few launches: the command the ncu captures under profiles/ run."""
    import torch
    import saetta_macqwen_b200 as sa

    torch.cuda.set_device(0)
    stream = torch.cuda.Stream()
    table = point_table(sa, torch, stream, args.steps, args.warmup)
    r = table[args.only]()
    r["point"] = args.only
    print(json.dumps(r), flush=True)


def cpu_sample(ctx, layers_sample, threads):
    """The oracle (the reference's CPU attention restated) on `layers_sample`
    layers of one decode row at `ctx` tokens; returns seconds per layer.  The
    inputs are made once (N(0,1) through the 8-bit round trip, held as f32 the
    way the reference's CPU cache holds them) and are not part of the time."""
    from oracle import oracle as o
    o.build()
    if ctx not in _CPU_DATA:
        keys = o.round_trip(o.normal(ctx * ROW, 1), 8)
        values = o.round_trip(o.normal(ctx * ROW, 2), 8)
        _CPU_DATA[ctx] = (keys, values, o.normal(HEADS * DIM, 3), o.normal(HEADS * 2 * DIM, 4))
        k, v, q, qg = _CPU_DATA[ctx]
        o.attention_rows(q, qg, k[: 1024 * ROW], v[: 1024 * ROW], [1024], threads=threads)  # warm
    keys, values, q, qg = _CPU_DATA[ctx]
    t0 = time.perf_counter()
    for _ in range(layers_sample):
        o.attention_rows(q, qg, keys, values, [ctx], threads=threads)
    return (time.perf_counter() - t0) / layers_sample


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    threads = min(cores, HEADS)
    per_layer = []
    for _ in range(args.warmup):
        cpu_sample(CTX, 1, threads)
    for _ in range(args.steps):
        per_layer.append(cpu_sample(CTX, 1, threads))
    sec = float(np.mean(per_layer))
    gbs = CTX * BYTES_PER_TOKEN[8] / sec / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3 * LAYERS, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"decode attention, 1 row, 16q/2kv heads of 256, {CTX}-token 8-bit KV per layer",
                   "layers": LAYERS, "ctx": CTX, "kv_bits": 8},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"1 of {LAYERS} layers per step (each layer is the same work), "
                                   f"{CTX} tokens, all 16 heads, {threads} threads over heads"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--points", default="all", help="'none' skips the extra measured points")
    ap.add_argument("--only", default=None, help="run one named point alone (for profiling) and print its result")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: partials stored into the peers' mailboxes over NVLink by the kernel that makes them (peer), "
                         "or NCCL all-gather + merge")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.only:
        return run_only(args)
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist
    import saetta_macqwen_b200 as sa

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = local
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    sa.lib()  # fails loudly when the CUDA library is missing
    stream = torch.cuda.Stream()
    hbm_peak, tc_peak, peak_kind = peaks()

    # ---- the step: LAYERS caches of CTX tokens on every rank
    cap = CTX + 128
    caches = [sa.GpuKvCache(dev, 8, cap) for _ in range(LAYERS)]
    for i, c in enumerate(caches):
        fill_cache(sa, torch, c, CTX, 100 * rank + i)
    op = sa.AttentionRows(dev, HEADS, KV, cap, 1)
    q = torch.randn(HEADS * DIM, device="cuda")
    qg = torch.randn(HEADS * 2 * DIM, device="cuda")
    out = torch.zeros(HEADS * DIM, device="cuda")
    params = torch.tensor([0, CTX - 1, CTX, 0], dtype=torch.int32, device="cuda")
    part = torch.zeros(HEADS * sa.PART_STRIDE, device="cuda")
    gathered = torch.zeros(world * HEADS * sa.PART_STRIDE, device="cuda")
    launches_per_step = 2 * LAYERS

    group = None
    if world > 1 and args.exchange == "peer":
        def gather_bytes(b):
            lst = [None] * world
            dist.all_gather_object(lst, b)
            return lst
        group = sa.PeerGroup(dev, rank, world, 1, HEADS, gather_bytes)

    def attend(c):
        """One layer: every rank's shard is full, so every row sees all kv_len keys of the shard."""
        if world == 1:
            op.record_cache(1, q, c, qg, out, params, stream=stream)
        elif group is not None:
            op.publish_cache(1, q, c, group, params, row_step=0, stream=stream)  # partial -> every peer's mailbox
            group.collect(1, qg, out, stream=stream)  # waits on local flags, merges what the peers stored
        else:
            op.partial_cache(1, q, c, part, params, row_step=0, stream=stream)
            dist.all_gather_into_tensor(gathered, part)
            sa.merge_partials(dev, gathered, world, 1, HEADS, qg, out, stream=stream)

    if world > 1:
        launches_per_step = (4 if group is not None else 3) * LAYERS

    def step():
        for c in caches:
            attend(c)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    with torch.cuda.stream(stream):
        if world == 1 or group is not None:  # no library collective inside: the step is one CUDA graph
            graph = torch.cuda.CUDAGraph()
            step()
            stream.synchronize()
            barrier()
            with torch.cuda.graph(graph, stream=stream):
                step()
            run = graph.replay
        else:
            run = step
        for _ in range(args.warmup):
            run()
        barrier()
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            run()
        e1.record(stream)
        stream.synchronize()
        barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    assert op.device_status(stream=stream) == 0, "a bounded device wait gave up"
    if group is not None:
        assert group.status(stream=stream) == 0, "a peer never published its partial"
    step_bytes = world * LAYERS * CTX * BYTES_PER_TOKEN[8]
    value = step_bytes / ms / 1e6  # GB/s

    # ---- end to end through the C ABI with host buffers.  Per step the token's raw q_and_gate, k and v
    # of every layer sit in one pinned host buffer; the step uploads them, and per layer runs
    # attention prep (q/k norm + RoPE, the new K/V row quantised into the cache) and the attention,
    # then reads every layer's output back and synchronises.  With no library collective inside,
    # the whole step -- both copies included -- is recorded once in a Plan (the reference's
    # record-once / replay-per-token runtime) and replayed with one graph launch.
    per_layer = HEADS * 2 * DIM + 2 * ROW
    h_in = torch.randn(LAYERS * per_layer).pin_memory()
    d_in = torch.zeros(LAYERS * per_layer, device="cuda")
    d_q = torch.zeros(LAYERS * HEADS * DIM, device="cuda")
    d_out = torch.zeros(LAYERS * HEADS * DIM, device="cuda")
    h_out = torch.zeros(LAYERS * HEADS * DIM).pin_memory()
    q_norm, k_norm = torch.ones(DIM, device="cuda"), torch.ones(DIM, device="cuda")
    prep = sa.PrepParams(HEADS, KV, DIM, 64, 1.0e7, 1.0e-6)
    h2d, d2h = 4 * h_in.numel(), 4 * h_out.numel()

    def layer_views(l):
        base = l * per_layer
        return (d_in[base:base + HEADS * 2 * DIM], d_in[base + HEADS * 2 * DIM:base + HEADS * 2 * DIM + ROW],
                d_in[base + HEADS * 2 * DIM + ROW:base + per_layer], d_q[l * HEADS * DIM:(l + 1) * HEADS * DIM],
                d_out[l * HEADS * DIM:(l + 1) * HEADS * DIM])

    def e2e_body(pp, st):
        d_in.copy_(h_in, non_blocking=True)
        for l, c in enumerate(caches):
            lqg, lk, lv, lq, lout = layer_views(l)
            sa.attention_prep(prep, 1, lqg, lk, lv, q_norm, k_norm, lq, sa.F32, c, params=pp, stream=st)
            if world == 1:
                op.record_cache(1, lq, c, lqg, lout, pp, stream=st)
            elif group is not None:
                op.publish_cache(1, lq, c, group, pp, row_step=0, stream=st)
                group.collect(1, lqg, lout, stream=st)
            else:
                op.partial_cache(1, lq, c, part, pp, row_step=0, stream=st)
                dist.all_gather_into_tensor(gathered, part)
                sa.merge_partials(dev, gathered, world, 1, HEADS, lqg, lout, stream=st)
        h_out.copy_(d_out, non_blocking=True)

    if world == 1 or group is not None:
        plan = sa.Plan(dev)
        with torch.cuda.stream(torch.cuda.ExternalStream(plan.stream)):
            with plan.recording():
                e2e_body(plan.params, plan.stream)

        def e2e_step():
            plan.set_params(0, CTX - 1)
            plan.run()  # one graph launch, then the wait: the caller reads the result
    else:
        def e2e_step():
            e2e_body(params, stream)
            stream.synchronize()

    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        e0.record(stream)
        for _ in range(args.steps):
            e2e_step()
        e1.record(stream)
        stream.synchronize()
        barrier()
        wall_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    e2e_ms = max(e0.elapsed_time(e1) / args.steps, 0.0)
    if world > 1:
        t = torch.tensor([e2e_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = step_bytes / e2e_ms / 1e6

    # ---- the other measured points (rank 0 of a 1-GPU run only)
    points = {}
    cpu = None
    if world == 1 and args.points != "none":
        del caches, op
        torch.cuda.empty_cache()
        s, w = max(5, args.steps // 2), 3
        table = point_table(sa, torch, stream, s, w)
        for name in ["decode_32k_8bit", "decode_128k_8bit", "decode_256k_4bit", "decode_128k_f16", "verify_m4_32k_8bit",
                     "batch64_ragged_8bit", "batch64_ragged_4bit", "qmv_8192x2048_5bit_m1", "qmv_8192x2048_5bit_m4",
                     "prep_store_4k_8bit", "prefill_4k_pos0_bf16",
                     "prefill_4k_pos32k_8bit", "prefill_4k_pos128k_8bit"]:
            fn = table[name]
            try:
                r = fn()
                if "gbs" in r:
                    r["frac_of_hbm_peak"] = r["gbs"] / hbm_peak
                if "tflops" in r:
                    r["frac_of_bf16_peak"] = r["tflops"] / tc_peak
                points[name] = r
            except Exception as e:  # a point that cannot run is reported, not hidden
                points[name] = {"error": str(e)[:200]}
            torch.cuda.empty_cache()
        # CPU baseline: the oracle on one layer of the step's workload, all host threads over heads
        cores = os.cpu_count() or 1
        threads = min(cores, HEADS)
        sec = cpu_sample(CTX, 1, threads)
        cpu = {"value": CTX * BYTES_PER_TOKEN[8] / sec / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
               "sample": f"1 of {LAYERS} layers of the step ({CTX} tokens, all 16 heads), f32 KV as the "
                         f"reference's CPU cache holds it, {threads} threads; {sec:.2f} s"}

    if rank == 0:
        per_layer_ms = ms / LAYERS
        achieved = CTX * BYTES_PER_TOKEN[8] / per_layer_ms / 1e6
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32 accumulate over u8 codes (f16 tensor-core operands)",
            "data": "synthetic",
            "config": {"workload": f"decode attention, 1 row, 16q/2kv heads of 256, {CTX}-token 8-bit KV shard per GPU, "
                                   f"{LAYERS} layers with separate caches per step",
                       "layers": LAYERS, "ctx_per_gpu": CTX, "kv_bits": 8, "l2": "inputs larger than L2 "
                       f"({LAYERS * CTX * BYTES_PER_TOKEN[8] / 1e6:.0f} MB per step per GPU)",
                       "replay": "CUDA graph" if (world == 1 or group is not None) else "eager launches",
                       "exchange": None if world == 1 else ("(m,l,O) stored into the peers' mailboxes over NVLink by the merge kernel"
                                                            if group is not None else "NCCL all-gather of (m,l,O) + merge")},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                         "frac": achieved / hbm_peak, "peak_kind": peak_kind + " copy bandwidth",
                         "frac_of_nominal_8TBs": achieved / 8000.0,
                         "kernel": "decode_quant_kernel<8,1> + merge_frag_kernel, per layer",
                         # dram bytes read + written by one launch pair, from the ncu capture at
                         # 131072 tokens (1122.5 B per token; profiles/decode_quant_8bit_128k.md), scaled by tokens
                         "traffic": int(CTX * TRAFFIC_PER_TOKEN)},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms, "wall_ms_per_step": wall_ms},
            "gpu_launches": args.steps * launches_per_step,
            "clocks": clocks,
            "points": points,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
