#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A step is TOKENS_PER_STEP decode tokens; a token's attention is one launch per
layer (split-KV CTAs and merge CTAs in the same kernel) over LAYERS separate
8-bit KV caches of CTX tokens, so every cache byte comes from HBM (the caches of
one token are far larger than L2).  Rank r of N holds its own CTX-token shard of
an N*CTX-token context (split-KV by sequence, weak scaling); the per-shard
(m, l, O) partials are exchanged over NVLink inside the same launch.  The
printed value is the whole job's algorithmic KV bytes per second.  Further
measured points ride along under "points": 32k / 64k / 128k decode, MTP verify,
4-bit, ragged batch, prefill TFLOP/s; at N > 1 the strong-scaling split of ONE
262144-token context, the long-context prefill chunk and the ragged batch over N
GPUs, and a parity check of the exchange against the CPU oracle.

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
TOKENS_PER_STEP = 256  # so that the timed region of the default 20 steps is over a second long
TRAFFIC_PER_TOKEN = 1118.7  # measured dram bytes read + written per cached token per layer (one ncu capture)
METRIC = "Decode-attn achieved HBM GB/s @32k/256k KV; prefill-attn TFLOP/s per 4k chunk"


def bench_config():
    """What both arms measure, word for word the same in both JSON lines."""
    return {"workload": f"decode attention, 1 row, 16q/2kv heads of 256, {CTX}-token 8-bit KV shard per GPU, "
                        f"{LAYERS} layers with separate caches per token, {TOKENS_PER_STEP} tokens per step",
            "layers": LAYERS, "ctx_per_gpu": CTX, "kv_bits": 8, "tokens_per_step": TOKENS_PER_STEP,
            "l2": f"inputs larger than L2 ({LAYERS * CTX * BYTES_PER_TOKEN[8] / 1e6:.0f} MB per token per GPU)"}


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return p["hbm_gbs"], p["bf16_tflops"], "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def sustained_tc_peak():
    """cuBLAS bf16 in a seconds-long loop under the power cap: the denominator for a point replayed for a
    quarter of a second and more (the burst figure is for a kernel timed alone)."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops_sustained"])
    except Exception:
        return 1400.0


class ClockSampler:
    """nvidia-smi clocks and throttle reasons (a read-only query) while the timed region runs: the query
    loop starts early, each sample is stamped when it is read, and only the samples inside the window
    between mark_start() and mark_stop() count."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.proc, self.t0, self.t1 = index, [], None, None, None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), [x.strip() for x in line.split(",")]))

    def mark_start(self):
        self.t0 = time.time()

    def mark_stop(self):
        self.t1 = time.time()

    def result(self):
        if self.proc:
            time.sleep(0.1)
            self.proc.terminate()
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, s in self.samples:
            if self.t0 is None or self.t1 is None or not (self.t0 <= t <= self.t1 + 0.06):
                continue
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


def fill_cache(sa, torch, cache, tokens, seed, pos0=0):
    """N(0,1) K and V rows quantised on the device by the store kernel (bit-exact
    with the oracle's quantiser, which the parity tests pin)."""
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    chunk = 8192
    for p in range(0, tokens, chunk):
        n = min(chunk, tokens - p)
        k = torch.randn(n * ROW, device="cuda", generator=g)
        v = torch.randn(n * ROW, device="cuda", generator=g)
        cache.store_at(k, v, pos0 + p, n)


def time_replays(torch, run, replays, warmup, stream):
    """CUDA-event milliseconds per call of run() over `replays` calls on `stream`."""
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            run()
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(replays):
            run()
        e1.record(stream)
        stream.synchronize()
    return e0.elapsed_time(e1) / replays


def graph_of(torch, fn, stream):
    """fn() captured once in a CUDA graph (record once, replay per token, as the reference replays its plan)."""
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        fn()
        stream.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            fn()
    return graph


def replays_for(ms_estimate, budget_ms=250.0, lo=5, hi=4000):
    return int(min(hi, max(lo, budget_ms / max(ms_estimate, 1e-3))))


def time_graph(torch, fn, warmup, stream, budget_ms=250.0):
    """ms per replay of fn() captured in a graph, over enough replays to fill about `budget_ms` of device time."""
    graph = graph_of(torch, fn, stream)
    est = time_replays(torch, graph.replay, 3, max(warmup, 3), stream)
    return time_replays(torch, graph.replay, replays_for(est, budget_ms), 1, stream)


def decode_point(sa, torch, ctx, bits, m, layers, warmup, stream):
    """GB/s of one m-row decode/verify token over `layers` caches of `ctx` tokens."""
    cap = ctx + 128
    dev = torch.cuda.current_device()
    caches = [sa.GpuKvCache(dev, bits, cap) for _ in range(layers)]
    for i, c in enumerate(caches):
        fill_cache(sa, torch, c, ctx + m - 1, 1000 + i)
    op = sa.AttentionRows(dev, HEADS, KV, cap, m)
    q = torch.randn(m * HEADS * DIM, device="cuda")
    qg = torch.randn(m * HEADS * 2 * DIM, device="cuda")
    out = torch.zeros(m * HEADS * DIM, device="cuda")
    params = torch.tensor([0, ctx - 1, ctx, 0], dtype=torch.int32, device="cuda")

    def token():
        for c in caches:
            op.record_cache(m, q, c, qg, out, params, stream=stream)

    ms = time_graph(torch, token, warmup, stream)
    nbytes = layers * (ctx + m - 1) * BYTES_PER_TOKEN[bits]
    assert op.device_status(stream=stream) == 0
    return {"gbs": nbytes / ms / 1e6, "us_per_layer": ms * 1e3 / layers, "layers": layers, "launches": layers}


def batch_point(sa, torch, bits, warmup, stream, seqs=64, lo=8192, hi=262144, seed=5):
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
    run = lambda: op.record(caches, lens, q, qg, out, stream=stream)
    est = time_replays(torch, run, 2, max(warmup, 2), stream)
    ms = time_replays(torch, run, replays_for(est), 1, stream)
    nbytes = int(lens.sum()) * BYTES_PER_TOKEN[bits]
    return {"gbs": nbytes / ms / 1e6, "ms": ms, "tokens": int(lens.sum()), "seqs": seqs}


def prefill_point(sa, torch, pos, tokens, warmup, stream, quant_bits=None, staged=False, blocks=128):
    """TFLOP/s of one causal chunk (flops = 4*H*D*(t*pos + t(t+1)/2), src/attention_prefill.rs:139-142).  A
    quantised prefix is read in place; with `staged`, through the op's 16-bit staging copy, which already holds
    the prefix, as after the chunk before (every call converts the chunk's own rows again)."""
    dev = torch.cuda.current_device()
    total = pos + tokens
    q = torch.randn(tokens * HEADS * DIM, device="cuda").to(torch.bfloat16)
    qg = torch.randn(tokens * HEADS * 2 * DIM, device="cuda")
    out = torch.zeros(tokens * HEADS * DIM, device="cuda")
    op = sa.AttGemm(dev, tokens, KV)
    op.score_blocks(blocks)  # 16-bit caches: the kernel with 128-key score blocks (default) or the one with 64
    p = sa.FlashParams(HEADS, KV, pos, tokens, 1.0 / 16.0)
    if quant_bits:
        cache = sa.GpuKvCache(dev, quant_bits, total)
        fill_cache(sa, torch, cache, total, 77)
        quant = cache.quant()
        op.stage_quantised(staged)
        op.reserve(total)
        fn = lambda: op.encode(q, None, None, quant, qg, out, p, dtype=sa.BF16, stream=stream)
    else:
        k = torch.randn(total * ROW, device="cuda").to(torch.bfloat16)
        v = torch.randn(total * ROW, device="cuda").to(torch.bfloat16)
        fn = lambda: op.encode(q, k, v, None, qg, out, p, dtype=sa.BF16, stream=stream)
    est = time_replays(torch, fn, 2, max(warmup, 2), stream)
    ms = time_replays(torch, fn, replays_for(est, hi=1500), 1, stream)
    flops = 4.0 * HEADS * DIM * (tokens * pos + tokens * (tokens + 1) / 2)
    return {"tflops": flops / ms / 1e9, "ms": ms, "flops": flops}


def half_point(sa, torch, ctx, layers, warmup, stream):
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

    def token():
        for c in caches:
            op.record_cache(1, q, c, qg, out, params, stream=stream)

    ms = time_graph(torch, token, warmup, stream) / layers
    assert op.device_status(stream=stream) == 0
    return {"gbs": ctx * 2048 / ms / 1e6, "us_per_layer": ms * 1e3, "layers": layers}


def qmv_point(sa, torch, rows, cols, bits, m, warmup, stream):
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
    reps = 200
    ms = sum(plan.run_timed() for _ in range(reps)) / (reps * per_plan)
    nbytes = rows * cols * bits // 8 + 2 * (rows * cols // 64) * 2
    return {"gbs": nbytes / ms / 1e6, "us": ms * 1e3, "bytes": nbytes}


def prep_point(sa, torch, tokens, bits, warmup, stream):
    """GB/s of attention prep fused with the quantised store for one prefill chunk: reads the q halves of
    q_and_gate, k, v (f32), writes q as bf16 and the cache rows.  The inputs of consecutive calls are
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
    state = {"i": 0}

    def fn():
        i = state["i"] = state["i"] + 1
        sa.attention_prep(pp, tokens, qg[i % copies], k[i % copies], v[i % copies], qn, kn, q_out, sa.BF16, cache, pos=0,
                          stream=stream)

    ms = time_replays(torch, fn, 3000, max(warmup, 6), stream)
    nbytes = tokens * (HEADS * DIM * 4 + 2 * ROW * 4 + HEADS * DIM * 2 + BYTES_PER_TOKEN[bits])
    return {"gbs": nbytes / ms / 1e6, "ms": ms, "bytes": nbytes}


def e2e_prefill_point(sa, torch, tokens, bits, warmup, stream):
    """One 4096-token prefill chunk at position 0 end to end through the C ABI with HOST buffers: the raw
    q_and_gate, k and v rows from pinned host memory, attention prep (norm, RoPE, quantised store), the
    tensor-core attention over the quantised cache, and the result back to pinned host memory -- one
    recorded Plan, one graph launch per chunk.  The copies dominate: the chunk's f32 inputs and outputs are
    a thousand times its KV bytes."""
    dev = torch.cuda.current_device()
    h_qg = torch.randn(tokens * HEADS * 2 * DIM).pin_memory()
    h_k, h_v = torch.randn(tokens * ROW).pin_memory(), torch.randn(tokens * ROW).pin_memory()
    h_out = torch.zeros(tokens * HEADS * DIM).pin_memory()
    d_qg, d_k, d_v = (torch.zeros_like(x, device="cuda") for x in (h_qg, h_k, h_v))
    d_q = torch.zeros(tokens * HEADS * DIM, dtype=torch.bfloat16, device="cuda")
    d_out = torch.zeros(tokens * HEADS * DIM, device="cuda")
    ones = torch.ones(DIM, device="cuda")
    cache = sa.GpuKvCache(dev, bits, tokens)
    op = sa.AttGemm(dev, tokens, KV)
    op.reserve(tokens)
    pp = sa.PrepParams(HEADS, KV, DIM, 64, 1.0e7, 1.0e-6)
    p = sa.FlashParams(HEADS, KV, 0, tokens, 1.0 / 16.0)
    plan = sa.Plan(dev)
    with torch.cuda.stream(torch.cuda.ExternalStream(plan.stream)):
        with plan.recording():
            d_qg.copy_(h_qg, non_blocking=True), d_k.copy_(h_k, non_blocking=True), d_v.copy_(h_v, non_blocking=True)
            sa.attention_prep(pp, tokens, d_qg, d_k, d_v, ones, ones, d_q, sa.BF16, cache, pos=0, stream=plan.stream)
            op.encode(d_q, None, None, cache.quant(), d_qg, d_out, p, dtype=sa.BF16, stream=plan.stream)
            h_out.copy_(d_out, non_blocking=True)
    for _ in range(max(warmup, 2)):
        plan.run()
    reps = 20
    ms = sum(plan.run_timed() for _ in range(reps)) / reps
    flops = 4.0 * HEADS * DIM * (tokens * (tokens + 1) / 2)
    h2d = 4 * (h_qg.numel() + h_k.numel() + h_v.numel())
    return {"tflops": flops / ms / 1e9, "ms": ms, "h2d_bytes": h2d, "d2h_bytes": 4 * h_out.numel()}


_CPU_DATA = {}


def point_table(sa, torch, stream, s, w):
    return {
        "decode_32k_8bit": lambda: decode_point(sa, torch, 32768, 8, 1, 10, w, stream),
        "decode_64k_8bit": lambda: decode_point(sa, torch, 65536, 8, 1, 6, w, stream),
        "decode_128k_8bit": lambda: decode_point(sa, torch, 131072, 8, 1, 4, w, stream),
        "decode_256k_8bit": lambda: decode_point(sa, torch, 262144, 8, 1, 4, w, stream),
        "decode_256k_4bit": lambda: decode_point(sa, torch, 262144, 4, 1, 4, w, stream),
        "decode_128k_f16": lambda: half_point(sa, torch, 131072, 4, w, stream),
        "verify_m4_32k_8bit": lambda: decode_point(sa, torch, 32768, 8, 4, 10, w, stream),
        "batch64_ragged_8bit": lambda: batch_point(sa, torch, 8, 2, stream),
        "batch64_ragged_4bit": lambda: batch_point(sa, torch, 4, 2, stream),
        "qmv_8192x2048_5bit_m1": lambda: qmv_point(sa, torch, 8192, 2048, 5, 1, w, stream),
        "qmv_8192x2048_5bit_m4": lambda: qmv_point(sa, torch, 8192, 2048, 5, 4, w, stream),
        "qmv_2048x4096_5bit_m1": lambda: qmv_point(sa, torch, 2048, 4096, 5, 1, w, stream),
        "prep_store_4k_8bit": lambda: prep_point(sa, torch, 4096, 8, w, stream),
        "prefill_4k_pos0_bf16": lambda: prefill_point(sa, torch, 0, 4096, w, stream),
        "prefill_4k_pos32k_8bit": lambda: prefill_point(sa, torch, 32768, 4096, 2, stream, quant_bits=8),
        "prefill_4k_pos128k_8bit": lambda: prefill_point(sa, torch, 131072, 4096, 2, stream, quant_bits=8),
        "prefill_4k_pos32k_4bit": lambda: prefill_point(sa, torch, 32768, 4096, 2, stream, quant_bits=4),
        "prefill_4k_pos32k_8bit_staged": lambda: prefill_point(sa, torch, 32768, 4096, 2, stream, quant_bits=8, staged=True),
        "prefill_4k_pos128k_8bit_staged": lambda: prefill_point(sa, torch, 131072, 4096, 2, stream, quant_bits=8, staged=True),
        "prefill_4k_pos128k_8bit_staged_64key": lambda: prefill_point(sa, torch, 131072, 4096, 2, stream, quant_bits=8, staged=True, blocks=64),
        "e2e_prefill_4k_8bit": lambda: e2e_prefill_point(sa, torch, 4096, 8, w, stream),
    }


def run_only(args):
    """One point alone, few launches: the command an ncu capture of that point runs."""
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


def cpu_baseline(sec, threads):
    """The CPU arm's figure in the metric's unit: the bytes of the 8-bit cache the GPU arm reads for the same
    tokens, over the CPU's time (the CPU itself holds the dequantised values as f32, 4096 bytes per token)."""
    return {"value": CTX * BYTES_PER_TOKEN[8] / sec / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"1 of the {LAYERS} layers of 1 of the {TOKENS_PER_STEP} tokens of a step ({CTX} cached tokens, all 16 "
                      f"heads; every layer of every token is the same work), {threads} threads over heads, {sec:.2f} s; GB/s "
                      f"counts the 8-bit cache's bytes ({BYTES_PER_TOKEN[8]} per token), what the GPU arm reads for the same tokens"}


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
    cpu = cpu_baseline(sec, threads)
    line = {
        "impl": "reference", "metric": METRIC, "value": cpu["value"], "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(),
        "method": "the CPU oracle (the reference's CPU attention restated); each step times a bounded sample, one layer of "
                  "one token, and ms_per_step is that sample's time (the whole step is layers x tokens_per_step times as long)",
        "cpu_baseline": cpu,
        "e2e": {"value": cpu["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------- N > 1

def exchange_parity(sa, torch, dist, group_of, rank, world, dev, stream):
    """One exchange outside every timed region, checked against the CPU oracle: rank r holds tokens
    [4096 r, 4096 (r + 1)) of a seeded sequence as an 8-bit shard, every rank has the same seeded query, the
    partials are exchanged and merged by the decode launch itself, and rank 0 compares its result with the
    oracle's attention over the whole sequence (2e-3 max-abs, the tolerance of the parity tests)."""
    from oracle import oracle as o
    o.build()
    per, total = 4096, 4096 * world
    keys, values = o.normal(total * ROW, 11), o.normal(total * ROW, 12)
    q, qg = o.normal(HEADS * DIM, 13), o.normal(HEADS * 2 * DIM, 14)
    to_dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    cache = sa.GpuKvCache(dev, 8, per)
    cache.store_at(to_dev(keys[rank * per * ROW:(rank + 1) * per * ROW]), to_dev(values[rank * per * ROW:(rank + 1) * per * ROW]), 0, per)
    op = sa.AttentionRows(dev, HEADS, KV, per, 1)
    group = group_of(1)
    out = torch.zeros(HEADS * DIM, device="cuda")
    params = torch.tensor([0, per - 1, per, 0], dtype=torch.int32, device="cuda")
    with torch.cuda.stream(stream):
        for _ in range(2):  # both mailbox slots
            op.exchange_cache(1, to_dev(q), cache, group, to_dev(qg), out, params, row_step=0, stream=stream)
        stream.synchronize()
    assert group.status(stream=stream) == 0 and op.device_status(stream=stream) == 0
    dist.barrier()
    want = o.attention_rows(q, qg, o.round_trip(keys, 8), o.round_trip(values, 8), [total], threads=8)
    err = float(np.abs(out.cpu().numpy().reshape(1, HEADS, DIM) - want).max())
    return {"max_abs": err, "tolerance": 2e-3, "tokens_per_rank": per, "ranks": world}


def strong_decode(sa, torch, dist, group_of, rank, world, dev, stream, warmup):
    """ONE 262144-token context split over the ranks by sequence: 4 layers per token, each rank reads its
    262144 / N rows, the decode launch exchanges and merges."""
    from saetta_macqwen_b200 import shard
    lo, hi = shard.shard_ranges(CTX, world)[rank]
    n = hi - lo
    caches = [sa.GpuKvCache(dev, 8, n) for _ in range(LAYERS)]
    for i, c in enumerate(caches):
        fill_cache(sa, torch, c, n, 300 + 10 * rank + i)
    op = sa.AttentionRows(dev, HEADS, KV, caches[0].capacity, 1)
    group = group_of(1)
    g = torch.Generator(device="cuda")
    g.manual_seed(77)  # the same query on every rank
    q = torch.randn(HEADS * DIM, device="cuda", generator=g)
    qg = torch.randn(HEADS * 2 * DIM, device="cuda", generator=g)
    out = torch.zeros(HEADS * DIM, device="cuda")
    params = torch.tensor([0, n - 1, n, 0], dtype=torch.int32, device="cuda")

    def token():
        for c in caches:
            op.exchange_cache(1, q, c, group, qg, out, params, row_step=0, stream=stream)

    graph = graph_of(torch, token, stream)
    dist.barrier()
    reps = 2000
    ms = time_replays(torch, graph.replay, reps, max(warmup, 3), stream)
    t = torch.tensor([ms], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    assert group.status(stream=stream) == 0 and op.device_status(stream=stream) == 0
    return {"ms_per_token": ms, "us_per_layer": ms * 1e3 / LAYERS, "gbs": LAYERS * CTX * BYTES_PER_TOKEN[8] / ms / 1e6,
            "ctx_total": CTX, "ctx_per_gpu": n, "layers": LAYERS}


def sharded_prefill(sa, torch, dist, group_of, rank, world, dev, stream, warmup, pos=131072, tokens=4096, bits=8, staged=False):
    """Config 4 over N GPUs: a 4096-token chunk at 131072 over an 8-bit cache whose rows are split over the
    ranks by sequence (every rank STORES only its slice); partial over the rank's keys, row-sliced exchange,
    every rank finalises its slice of the chunk's rows.  The slice is read in place, or (`staged`) through the op's
    binary16 copy of it, which holds the slice from the chunk before."""
    from saetta_macqwen_b200 import shard
    total = pos + tokens
    lo, hi = shard.shard_ranges(total, world)[rank]
    cache = sa.GpuKvCache(dev, bits, hi - lo)
    fill_cache(sa, torch, cache, hi - lo, 500 + rank)
    g = torch.Generator(device="cuda")
    g.manual_seed(78)
    q = torch.randn(tokens * HEADS * DIM, device="cuda", generator=g).to(torch.bfloat16)
    qg = torch.randn(tokens * HEADS * 2 * DIM, device="cuda", generator=g)
    out = torch.zeros(tokens * HEADS * DIM, device="cuda")
    op = sa.AttGemm(dev, tokens, KV)
    op.stage_quantised(staged)
    op.reserve(hi - lo)
    group = group_of(tokens)
    p = sa.FlashParams(HEADS, KV, pos, tokens, 1.0 / 16.0)
    quant = cache.quant()

    def chunk():
        op.partial(q, None, None, quant, group.staging, p, lo, hi, dtype=sa.BF16, stream=stream, key_base=lo)
        group.merge_sliced(tokens, qg, out, stream=stream)

    dist.barrier()
    ms = time_replays(torch, chunk, 30, 2, stream)
    t = torch.tensor([ms], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    assert group.status(stream=stream) == 0
    flops = 4.0 * HEADS * DIM * (tokens * pos + tokens * (tokens + 1) / 2)
    return {"tflops": flops / ms / 1e9, "ms": ms, "flops": flops, "keys_per_gpu": hi - lo}


def sharded_batch(sa, torch, dist, group_of, rank, world, dev, stream, warmup, bits, seqs=64, lo=8192, hi=262144, seed=5):
    """Config 5 over N GPUs: every sequence's rows split over the ranks by sequence; one ragged launch per
    rank publishes the shard partials, one launch collects."""
    from saetta_macqwen_b200 import shard
    rng = np.random.default_rng(seed)
    lens = rng.integers(lo, hi + 1, seqs)
    caches, mine = [], []
    for i, n in enumerate(lens):
        a, b = shard.shard_ranges(int(n), world)[rank]
        c = sa.GpuKvCache(dev, bits, max(b - a, 1))
        if b > a:
            fill_cache(sa, torch, c, b - a, 2000 + 64 * rank + i)
        caches.append(c)
        mine.append(b - a)
    op = sa.DecodeBatch(dev, seqs)
    group = group_of(seqs)
    g = torch.Generator(device="cuda")
    g.manual_seed(79)
    q = torch.randn(seqs * HEADS * DIM, device="cuda", generator=g)
    qg = torch.randn(seqs * HEADS * 2 * DIM, device="cuda", generator=g)
    out = torch.zeros(seqs * HEADS * DIM, device="cuda")

    def run():
        op.publish(caches, mine, q, group, stream=stream)
        group.collect(seqs, qg, out, stream=stream)

    dist.barrier()
    ms = time_replays(torch, run, 100, 3, stream)
    t = torch.tensor([ms], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    assert group.status(stream=stream) == 0
    nbytes = int(lens.sum()) * BYTES_PER_TOKEN[bits]
    return {"gbs": nbytes / ms / 1e6, "ms": ms, "tokens": int(lens.sum()), "seqs": seqs}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--points", default="all", help="'none' skips the extra measured points")
    ap.add_argument("--only", default=None, help="run one named point alone (for profiling) and print its result")
    ap.add_argument("--exchange", default="fused", choices=["fused", "peer", "nccl"],
                    help="N > 1: partials stored into the peers' mailboxes over NVLink and collected by the decode launch's own "
                         "merge CTAs (fused), collected by a second launch (peer), or NCCL all-gather + merge")
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
    sampler = ClockSampler(local)
    stream = torch.cuda.Stream()
    hbm_peak, tc_peak, peak_kind = peaks()

    def group_of(rows):
        def gather_bytes(b):
            lst = [None] * world
            dist.all_gather_object(lst, b)
            return lst
        return sa.PeerGroup(dev, rank, world, rows, HEADS, gather_bytes)

    # ---- the step: TOKENS_PER_STEP tokens over LAYERS caches of CTX tokens on every rank
    cap = CTX + 128
    caches = [sa.GpuKvCache(dev, 8, cap) for _ in range(LAYERS)]
    for i, c in enumerate(caches):
        fill_cache(sa, torch, c, CTX, 100 * rank + i)
    op = sa.AttentionRows(dev, HEADS, KV, cap, 1)
    g = torch.Generator(device="cuda")
    g.manual_seed(1234)  # every rank draws the same query: the merged result means something
    q = torch.randn(HEADS * DIM, device="cuda", generator=g)
    qg = torch.randn(HEADS * 2 * DIM, device="cuda", generator=g)
    out = torch.zeros(HEADS * DIM, device="cuda")
    params = torch.tensor([0, CTX - 1, CTX, 0], dtype=torch.int32, device="cuda")
    part = torch.zeros(HEADS * sa.PART_STRIDE, device="cuda")
    gathered = torch.zeros(world * HEADS * sa.PART_STRIDE, device="cuda")
    group = group_of(1) if world > 1 and args.exchange != "nccl" else None
    launches_per_token = LAYERS * (1 if world == 1 or args.exchange == "fused" else 2 if args.exchange == "peer" else 2)

    def attend(c, lq, lqg, lout, pp, st):
        """One layer: every rank's shard is full, so every row sees all kv_len keys of the shard."""
        if world == 1:
            op.record_cache(1, lq, c, lqg, lout, pp, stream=st)
        elif args.exchange == "fused":
            op.exchange_cache(1, lq, c, group, lqg, lout, pp, row_step=0, stream=st)  # one launch: partial, exchange, merge
        elif args.exchange == "peer":
            op.publish_cache(1, lq, c, group, pp, row_step=0, stream=st)  # partial -> every peer's mailbox
            group.collect(1, lqg, lout, stream=st)  # waits on local words, merges what the peers stored
        else:
            op.partial_cache(1, lq, c, part, pp, row_step=0, stream=st)
            dist.all_gather_into_tensor(gathered, part)
            sa.merge_partials(dev, gathered, world, 1, HEADS, lqg, lout, stream=st)

    def token():
        for c in caches:
            attend(c, q, qg, out, params, stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    graphed = world == 1 or group is not None  # no library collective inside: a token is one CUDA graph
    run = graph_of(torch, token, stream).replay if graphed else token
    barrier()
    with torch.cuda.stream(stream):
        for _ in range(args.warmup * TOKENS_PER_STEP // 8 + 8):
            run()
        barrier()
        sampler.mark_start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps * TOKENS_PER_STEP):
            run()
        e1.record(stream)
        stream.synchronize()
        sampler.mark_stop()
        barrier()
    clocks = sampler.result()
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    assert op.device_status(stream=stream) == 0, "a bounded device wait gave up"
    if group is not None:
        assert group.status(stream=stream) == 0, "a peer never published its partial"
    step_bytes = world * TOKENS_PER_STEP * LAYERS * CTX * BYTES_PER_TOKEN[8]
    value = step_bytes / ms / 1e6  # GB/s

    # ---- end to end through the C ABI with host buffers.  Per token the raw q_and_gate, k and v of every
    # layer sit in one pinned host buffer; the token's graph uploads them, per layer runs attention prep
    # (q/k norm + RoPE, the new K/V row quantised into the cache) and the attention, reads every layer's
    # output back, and the caller waits for it.  The prep of layer l + 1 is recorded on the Plan's side
    # branch (op_parallel): it depends on the upload only and runs on the SMs that layer l's split-KV CTAs
    # leave while its merge CTAs still work.  With no library collective inside, the whole token -- both
    # copies included -- is recorded once in a Plan (the reference's record-once / replay-per-token
    # runtime) and replayed with one graph launch.
    per_layer = HEADS * 2 * DIM + 2 * ROW
    h_in = torch.randn(LAYERS * per_layer).pin_memory()
    d_in = torch.zeros(LAYERS * per_layer, device="cuda")
    d_q = torch.zeros(LAYERS * HEADS * DIM, device="cuda")
    d_out = torch.zeros(LAYERS * HEADS * DIM, device="cuda")
    h_out = torch.zeros(LAYERS * HEADS * DIM).pin_memory()
    q_norm, k_norm = torch.ones(DIM, device="cuda"), torch.ones(DIM, device="cuda")
    prep = sa.PrepParams(HEADS, KV, DIM, 64, 1.0e7, 1.0e-6)
    h2d, d2h = 4 * h_in.numel() * TOKENS_PER_STEP, 4 * h_out.numel() * TOKENS_PER_STEP

    def layer_views(l):
        base = l * per_layer
        return (d_in[base:base + HEADS * 2 * DIM], d_in[base + HEADS * 2 * DIM:base + HEADS * 2 * DIM + ROW],
                d_in[base + HEADS * 2 * DIM + ROW:base + per_layer], d_q[l * HEADS * DIM:(l + 1) * HEADS * DIM],
                d_out[l * HEADS * DIM:(l + 1) * HEADS * DIM])

    def prep_layer(l, pp, st):
        lqg, lk, lv, lq, _ = layer_views(l)
        sa.attention_prep(prep, 1, lqg, lk, lv, q_norm, k_norm, lq, sa.F32, caches[l], params=pp, stream=st)

    if graphed:
        plan = sa.Plan(dev)
        with torch.cuda.stream(torch.cuda.ExternalStream(plan.stream)):
            with plan.recording():
                d_in.copy_(h_in, non_blocking=True)
                prep_layer(0, plan.params, plan.stream)
                for l, c in enumerate(caches):
                    lqg, _, _, lq, lout = layer_views(l)
                    if l + 1 < LAYERS:
                        prep_layer(l + 1, plan.params, plan.parallel_begin())
                    attend(c, lq, lqg, lout, plan.params, plan.stream)
                    if l + 1 < LAYERS:
                        plan.parallel_end()
                h_out.copy_(d_out, non_blocking=True)

        def e2e_token():
            plan.set_params(0, CTX - 1)
            plan.run()  # one graph launch, then the wait: the caller reads the result
    else:
        def e2e_token():
            d_in.copy_(h_in, non_blocking=True)
            for l, c in enumerate(caches):
                lqg, _, _, lq, lout = layer_views(l)
                prep_layer(l, params, stream)
                attend(c, lq, lqg, lout, params, stream)
            h_out.copy_(d_out, non_blocking=True)
            stream.synchronize()

    with torch.cuda.stream(stream):
        for _ in range(args.warmup * 8):
            e2e_token()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps * TOKENS_PER_STEP):
            e2e_token()
        stream.synchronize()
        wall_ms = (time.perf_counter() - t0) * 1e3 / args.steps
        barrier()
    # every token ends with a wait for its result, so the host clock around the loop is the device time
    # of the step plus the launch and wake-up of each token: the end-to-end time a caller sees
    e2e_ms = wall_ms
    if world > 1:
        t = torch.tensor([e2e_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = step_bytes / e2e_ms / 1e6

    # ---- the other measured points
    points, cpu, parity_n = {}, None, None
    del caches, op
    torch.cuda.empty_cache()
    if world == 1 and args.points != "none":
        table = point_table(sa, torch, stream, args.steps, 3)
        for name in ["decode_32k_8bit", "decode_64k_8bit", "decode_128k_8bit", "decode_256k_4bit", "decode_128k_f16",
                     "verify_m4_32k_8bit", "batch64_ragged_8bit", "batch64_ragged_4bit", "qmv_8192x2048_5bit_m1",
                     "qmv_8192x2048_5bit_m4", "prep_store_4k_8bit", "prefill_4k_pos0_bf16", "prefill_4k_pos32k_8bit",
                     "prefill_4k_pos128k_8bit", "prefill_4k_pos32k_4bit", "prefill_4k_pos32k_8bit_staged", "prefill_4k_pos128k_8bit_staged",
                     "e2e_prefill_4k_8bit"]:
            try:
                r = table[name]()
                if "gbs" in r:
                    r["frac_of_hbm_peak"] = r["gbs"] / hbm_peak
                if "tflops" in r and not name.startswith("e2e"):
                    r["frac_of_bf16_peak"] = r["tflops"] / tc_peak
                    r["frac_of_bf16_sustained"] = r["tflops"] / sustained_tc_peak()
                    r["frac_of_nominal_2250"] = r["tflops"] / 2250.0
                points[name] = r
            except Exception as e:  # a point that cannot run is reported, not hidden
                points[name] = {"error": str(e)[:200]}
            torch.cuda.empty_cache()
        # CPU baseline: the oracle on one layer of one token of the step, all host threads over heads
        threads = min(os.cpu_count() or 1, HEADS)
        cpu = cpu_baseline(cpu_sample(CTX, 1, threads), threads)
    if world > 1 and args.exchange == "fused":
        # driver-visible proof that the exchange merges right, outside every timed region
        parity_n = exchange_parity(sa, torch, dist, group_of, rank, world, dev, stream)
        if args.points != "none":
            for name, fn in [("strong_256k_8bit", lambda: strong_decode(sa, torch, dist, group_of, rank, world, dev, stream, 3)),
                             ("prefill_4k_pos128k_8bit", lambda: sharded_prefill(sa, torch, dist, group_of, rank, world, dev, stream, 2)),
                             ("prefill_4k_pos128k_8bit_staged", lambda: sharded_prefill(sa, torch, dist, group_of, rank, world, dev, stream, 2, staged=True)),
                             ("batch64_ragged_8bit", lambda: sharded_batch(sa, torch, dist, group_of, rank, world, dev, stream, 3, 8)),
                             ("batch64_ragged_4bit", lambda: sharded_batch(sa, torch, dist, group_of, rank, world, dev, stream, 3, 4))]:
                try:
                    r = fn()
                    if "gbs" in r:
                        r["frac_of_n_hbm_peaks"] = r["gbs"] / (world * hbm_peak)
                    if "tflops" in r:
                        r["frac_of_n_bf16_peaks"] = r["tflops"] / (world * tc_peak)
                    points[name] = r
                except Exception as e:
                    points[name] = {"error": str(e)[:200]}
                torch.cuda.empty_cache()
                dist.barrier()

    if rank == 0:
        per_layer_ms = ms / TOKENS_PER_STEP / LAYERS
        achieved = CTX * BYTES_PER_TOKEN[8] / per_layer_ms / 1e6
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32 accumulate over u8 codes (f16 tensor-core operands)",
            "data": "synthetic",
            "config": bench_config(),
            "method": {"replay": "one CUDA graph per token" if graphed else "eager launches",
                       "exchange": None if world == 1 else
                       {"fused": "(m,l,O) stored into the peers' mailboxes over NVLink and collected by the merge CTAs of the same launch",
                        "peer": "(m,l,O) stored into the peers' mailboxes over NVLink by the merge CTAs, collected by a second launch",
                        "nccl": "NCCL all-gather of (m,l,O) + merge"}[args.exchange],
                       "timed_region_s": ms * args.steps / 1e3},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                         "frac": achieved / hbm_peak, "peak_kind": peak_kind + " copy bandwidth",
                         "frac_of_nominal_8TBs": achieved / 8000.0,
                         "kernel": "decode_quant_kernel<8,1> (split-KV CTAs + merge CTAs), one launch per layer",
                         # dram bytes read + written by one launch, from an ncu capture at 131072 tokens,
                         # scaled by tokens (the traffic is proportional to the cached tokens)
                         "traffic": int(CTX * TRAFFIC_PER_TOKEN)},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms, "timing": "host clock around the step: every token's graph launch is waited for"},
            "gpu_launches": args.steps * TOKENS_PER_STEP * launches_per_token,
            "clocks": clocks,
            "points": points,
        }
        if parity_n is not None:
            line["parity_n"] = parity_n
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if parity_n is not None and parity_n["max_abs"] > parity_n["tolerance"]:
        sys.exit(3)


if __name__ == "__main__":
    main()
