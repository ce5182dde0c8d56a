"""Chunked causal prefill attention (tcgen05 kernel) against the CPU oracle.

Mirrors tests/attention_prefill.rs of the reference: its chunk shapes (partial
tiles and key blocks), its `spread` inputs and (i % 7) - 3 gate pattern, and its
2e-3 max-abs bound -- here against the CPU oracle instead of another GPU kernel
-- plus the benchmark configurations on bfloat16 N(0,1) inputs with partial RoPE,
a quantised prefix read in place, and the split-key partials.
Tolerance: 2e-3 max-abs and 1e-3 relative RMS.
"""
import numpy as np
import pytest

import saetta_macqwen_b200 as sa
from util import DIM, HEADS, KV, ROW, dev, max_abs, rel_rms

pytestmark = pytest.mark.gpu


def to16(torch, x, dtype):
    return dev(x).to(torch.float16 if dtype == sa.F16 else torch.bfloat16)


def run(torch, q, k, v, qg, pos, tokens, dtype, quant=None, op=None):
    out = torch.full((tokens * HEADS * DIM,), float("nan"), dtype=torch.float32, device="cuda")
    op = op or sa.AttGemm(0, 4096, KV)
    p = sa.FlashParams(HEADS, KV, pos, tokens, 1.0 / 16.0)
    op.encode(to16(torch, q, dtype), None if quant else to16(torch, k, dtype), None if quant else to16(torch, v, dtype),
              quant, dev(qg), out, p, dtype=dtype)
    torch.cuda.synchronize()
    return out.cpu().numpy().reshape(tokens, HEADS, DIM)


@pytest.mark.parametrize("blocks", [128, 64])
@pytest.mark.parametrize("pos,tokens", [(0, 1), (0, 7), (5, 8), (70, 100), (1000, 64), (0, 300), (4093, 37)])
def test_matches_cpu_on_reference_shapes(oracle, pos, tokens, blocks):
    """The reference's own shapes (tests/attention_prefill.rs) through both kernels for 16-bit caches: score
    blocks of 128 keys (the default) and of 64."""
    import torch

    capacity = (pos + tokens + 63) // 64 * 64 + 64
    q = oracle.round_f16(oracle.spread(tokens * HEADS * DIM, 1))
    k = oracle.round_f16(oracle.spread(capacity * ROW, 2))
    v = oracle.round_f16(oracle.spread(capacity * ROW, 3))
    qg = ((np.arange(tokens * HEADS * 2 * DIM) % 7) - 3).astype(np.float32)
    op = sa.AttGemm(0, 4096, KV)
    op.score_blocks(blocks)
    got = run(torch, q, k, v, qg, pos, tokens, sa.F16, op=op)
    want = oracle.attention_rows(q, qg, k, v, [pos + i + 1 for i in range(tokens)], threads=8)
    assert np.isfinite(got).all()
    assert max_abs(got, want) < 2e-3 and rel_rms(got, want) < 1e-3, (pos, tokens, max_abs(got, want), rel_rms(got, want))
    if blocks == 64:
        with pytest.raises(sa.SaettaError):
            op.score_blocks(96)


@pytest.mark.parametrize("pos,tokens", [(0, 1), (0, 7), (5, 8), (70, 100), (1000, 64), (0, 300), (4093, 37)])
def test_prefill_encode_matches_cpu_on_reference_shapes(oracle, pos, tokens):
    """attention_prefill::encode (src/attention_prefill.rs:39-72), the entry point without an op object,
    on the shapes of tests/attention_prefill.rs:10-62: binary16 q and cache, `spread` inputs, the
    (i % 7) - 3 gate pattern.  2e-3 max-abs / 1e-3 relative RMS against the CPU oracle."""
    import torch

    capacity = (pos + tokens + 63) // 64 * 64 + 64
    q = oracle.round_f16(oracle.spread(tokens * HEADS * DIM, 1))
    k = oracle.round_f16(oracle.spread(capacity * ROW, 2))
    v = oracle.round_f16(oracle.spread(capacity * ROW, 3))
    qg = ((np.arange(tokens * HEADS * 2 * DIM) % 7) - 3).astype(np.float32)
    out = torch.full((tokens * HEADS * DIM,), float("nan"), dtype=torch.float32, device="cuda")
    p = sa.FlashParams(HEADS, KV, pos, tokens, 1.0 / 16.0)
    sa.prefill_encode(0, to16(torch, q, sa.F16), to16(torch, k, sa.F16), to16(torch, v, sa.F16), dev(qg), out, p)
    torch.cuda.synchronize()
    got = out.cpu().numpy().reshape(tokens, HEADS, DIM)
    want = oracle.attention_rows(q, qg, k, v, [pos + i + 1 for i in range(tokens)], threads=8)
    assert np.isfinite(got).all()
    assert max_abs(got, want) < 2e-3 and rel_rms(got, want) < 1e-3, (pos, tokens, max_abs(got, want), rel_rms(got, want))


def test_prefill_encode_matches_att_gemm_and_refuses_bfloat16(oracle):
    """N(0,1) binary16 inputs with partial RoPE at a position past the first tile: the object-less entry
    point gives what AttGemm::encode gives, bit for bit (one kernel, no staging on either route), and
    bfloat16 -- which it could only run with P rounded to 8 bits -- comes back as UNSUPPORTED."""
    import torch

    pos, tokens = 700, 150
    q, k, v, qg = bf16_inputs(oracle, pos, tokens, 600)
    q, k, v = oracle.round_f16(q), oracle.round_f16(k), oracle.round_f16(v)
    a = run(torch, q, k, v, qg, pos, tokens, sa.F16)
    out = torch.full((tokens * HEADS * DIM,), float("nan"), dtype=torch.float32, device="cuda")
    p = sa.FlashParams(HEADS, KV, pos, tokens, 1.0 / 16.0)
    qd, kd, vd, gd = to16(torch, q, sa.F16), to16(torch, k, sa.F16), to16(torch, v, sa.F16), dev(qg)
    sa.prefill_encode(0, qd, kd, vd, gd, out, p)
    torch.cuda.synchronize()
    got = out.cpu().numpy().reshape(tokens, HEADS, DIM)
    assert np.array_equal(got, a)
    check_rows(oracle, got, q, qg, k, v, pos, np.arange(tokens))
    with pytest.raises(sa.SaettaError) as e:
        sa.prefill_encode(0, qd, kd, vd, gd, out, p, dtype=sa.BF16)
    assert e.value.code == sa.UNSUPPORTED


def bf16_inputs(oracle, pos, tokens, seed):
    total = pos + tokens
    k = oracle.rope_rows(oracle.normal(total * ROW, seed).reshape(total, ROW), DIM, 64, range(total), 1e7)
    v = oracle.normal(total * ROW, seed + 1)
    q = oracle.rope_rows(oracle.normal(tokens * HEADS * DIM, seed + 2).reshape(tokens, -1), DIM, 64,
                         range(pos, total), 1e7)
    qg = np.zeros((tokens * HEADS, 2 * DIM), np.float32)
    qg[:, DIM:] = oracle.normal(tokens * HEADS * DIM, seed + 3).reshape(-1, DIM)
    return oracle.round_bf16(q.ravel()), oracle.round_bf16(k.ravel()), oracle.round_bf16(v), qg.ravel()


def check_rows(oracle, got, q, qg, k, v, pos, rows):
    qs = q.reshape(-1, HEADS * DIM)[rows]
    gs = qg.reshape(-1, HEADS * 2 * DIM)[rows]
    want = oracle.attention_rows(qs, gs, k, v, [pos + int(r) + 1 for r in rows], threads=8)
    g = got[rows]
    assert np.isfinite(got).all()
    assert max_abs(g, want) < 2e-3 and rel_rms(g, want) < 1e-3, (max_abs(g, want), rel_rms(g, want))
    return max_abs(g, want), rel_rms(g, want)


def test_config2_chunk_4096_bf16(oracle):
    """4096-token chunk, no prior context, bf16 Q/K/V ~N(0,1) with partial RoPE, causal, gate."""
    import torch

    pos, tokens = 0, 4096
    q, k, v, qg = bf16_inputs(oracle, pos, tokens, 200)
    got = run(torch, q, k, v, qg, pos, tokens, sa.BF16)
    rng = np.random.default_rng(0)
    rows = np.unique(np.concatenate([[0, 1, 15, 16, 17, 63, 64, 65, 2047, 2048, 4079, 4080, 4095],
                                     rng.integers(0, tokens, 51)]))
    print("config 2:", check_rows(oracle, got, q, qg, k, v, pos, rows))


@pytest.mark.parametrize("bits", [8, 4])
def test_quantised_prefix_is_read_in_place(oracle, bits):
    """AttGemm::encode with quant: the chunk's rows are quantised into the cache
    first (src/prefill.rs:1656-1666), then the kernel reads the codes per key block and
    uses keys and values as the binary16 rounding of s*q+z (src/kv_quant.rs:121-126,
    kernels/attention_rows_q.metal:16-31); bfloat16 queries go in as binary16."""
    import torch

    pos, tokens = 1000, 72
    total = pos + tokens
    q, k, v, qg = bf16_inputs(oracle, pos, tokens, 300)
    cache = sa.GpuKvCache(0, bits, total)
    cache.store_at(dev(k), dev(v), 0, total)
    got = run(torch, q, None, None, qg, pos, tokens, sa.BF16, quant=cache.quant())
    kr = oracle.round_trip_as_half(k, bits)  # keys and values as binary16, the reference's own reading (src/kv_quant.rs:121-126)
    vr = oracle.round_trip_as_half(v, bits)             # values as binary16, the reference's own reading
    check_rows(oracle, got, q, qg, kr, vr, pos, np.arange(tokens))


def test_split_key_partials_merge_to_the_whole(oracle):
    import torch

    pos, tokens = 500, 40
    total = pos + tokens
    q, k, v, qg = bf16_inputs(oracle, pos, tokens, 400)
    whole = run(torch, q, k, v, qg, pos, tokens, sa.BF16)
    op = sa.AttGemm(0, 4096, KV)
    p = sa.FlashParams(HEADS, KV, pos, tokens, 1.0 / 16.0)
    cuts = [0, 200, 517, total]
    parts = torch.zeros((len(cuts) - 1, tokens * HEADS * sa.PART_STRIDE), dtype=torch.float32, device="cuda")
    qd, kd, vd = to16(torch, q, sa.BF16), to16(torch, k, sa.BF16), to16(torch, v, sa.BF16)
    for i in range(len(cuts) - 1):
        op.partial(qd, kd, vd, None, parts[i], p, cuts[i], cuts[i + 1], dtype=sa.BF16)
    out = torch.zeros(tokens * HEADS * DIM, dtype=torch.float32, device="cuda")
    sa.merge_partials(0, parts, len(cuts) - 1, tokens, HEADS, dev(qg), out)
    torch.cuda.synchronize()
    got = out.cpu().numpy().reshape(tokens, HEADS, DIM)
    assert max_abs(got, whole) < 2e-3 and rel_rms(got, whole) < 1e-3  # two roundings of P apart
    want = oracle.attention_rows(q, qg, k, v, [pos + i + 1 for i in range(tokens)], threads=8)
    assert max_abs(got, want) < 2e-3 and rel_rms(got, want) < 1e-3


def test_long_context_chunk_uses_key_splits(oracle):
    """Past 16384 keys each tile's key range is cut into two work items whose
    partials are merged; the result must still be the oracle's."""
    import torch

    pos, tokens = 17000, 40
    q, k, v, qg = bf16_inputs(oracle, pos, tokens, 500)
    got = run(torch, q, k, v, qg, pos, tokens, sa.BF16)
    check_rows(oracle, got, q, qg, k, v, pos, np.array([0, 1, 7, 15, 16, 17, 31, 32, 39]))


@pytest.mark.parametrize("bits", [32, 8])
def test_row_route_of_the_exact_mode(oracle, bits):
    """src/prefill.rs:1674-1686: in exact mode the chunk goes through the AttentionRows kernels.  Over an f32 cache
    that is f32 arithmetic throughout (5e-6 rel-RMS, the tolerance of the f32 configuration); over an 8-bit cache the
    quantised row kernel (2e-3 / 1e-3)."""
    import torch

    pos, tokens = 37, 21  # three groups of 8, the last one ragged
    total = pos + tokens
    q = oracle.normal(tokens * HEADS * DIM, 31)
    k, v = oracle.normal(total * ROW, 32), oracle.normal(total * ROW, 33)
    qg = oracle.normal(tokens * HEADS * 2 * DIM, 34)
    cache = sa.GpuKvCache(0, bits, 128)
    cache.store_at(dev(k), dev(v), 0, total)
    op = sa.AttentionRows(0, HEADS, KV, 128, 8)
    out = torch.full((tokens * HEADS * DIM,), float("nan"), device="cuda")
    scratch = torch.zeros(4 * 4, dtype=torch.int32, device="cuda")
    op.prefill_rows(dev(q), cache, dev(qg), out, sa.FlashParams(HEADS, KV, pos, tokens, 1.0 / 16.0), scratch)
    torch.cuda.synchronize()
    assert op.device_status() == 0
    got = out.cpu().numpy().reshape(tokens, HEADS, DIM)
    kr, vr = (k, v) if bits == 32 else (oracle.round_trip(k, bits), oracle.round_trip(v, bits))
    want = oracle.attention_rows(q, qg, kr, vr, [pos + i + 1 for i in range(tokens)], threads=8)
    assert np.isfinite(got).all()
    if bits == 32:
        assert rel_rms(got, want) < 5e-6, rel_rms(got, want)
    else:
        assert max_abs(got, want) < 2e-3 and rel_rms(got, want) < 1e-3, (max_abs(got, want), rel_rms(got, want))
    with pytest.raises(sa.SaettaError):  # the chunk must fit the cache
        op.prefill_rows(dev(q), cache, dev(qg), out, sa.FlashParams(HEADS, KV, 120, tokens, 1.0 / 16.0), scratch)


def test_shape_errors(oracle):
    import torch

    op = sa.AttGemm(0, 64, KV)
    z = torch.zeros(16, device="cuda")
    with pytest.raises(sa.SaettaError):  # more tokens than the op's chunk
        op.encode(z, z, z, None, z, z, sa.FlashParams(HEADS, KV, 0, 65, 0.0625))
    with pytest.raises(sa.SaettaError):  # 8 q heads per kv head
        op.encode(z, z, z, None, z, z, sa.FlashParams(12, KV, 0, 8, 0.0625))


def test_config4_long_context_chunk_over_8bit_prefix(oracle):
    """A 4096-token chunk at position 131072 on top of a 131072-token 8-bit cache
    (the chunk's own rows quantised into the cache first), bf16 queries.  The
    oracle is evaluated on a sample of 64 or more rows.  Keys and values are read as the binary16 rounding of s*q+z."""
    import torch

    pos, tokens, bits = 131072, 4096, 8
    total = pos + tokens
    cache = sa.GpuKvCache(0, bits, total)
    g = torch.Generator(device="cuda")
    g.manual_seed(4)
    kr = np.empty((total, ROW), np.float32)
    vr = np.empty((total, ROW), np.float32)
    for p0 in range(0, total, 16384):  # N(0,1) rows made on the device, kept for the oracle
        n = min(16384, total - p0)
        k = torch.randn(n * ROW, device="cuda", generator=g)
        v = torch.randn(n * ROW, device="cuda", generator=g)
        cache.store_at(k, v, p0, n)
        kr[p0:p0 + n] = oracle.round_trip_as_half(k.cpu().numpy(), bits).reshape(n, ROW)
        vr[p0:p0 + n] = oracle.round_trip_as_half(v.cpu().numpy(), bits).reshape(n, ROW)
    q = oracle.round_bf16(oracle.normal(tokens * HEADS * DIM, 41))
    qg = oracle.normal(tokens * HEADS * 2 * DIM, 42)
    got = run(torch, q, None, None, qg, pos, tokens, sa.BF16, quant=cache.quant())
    # 64+ rows: first and last, the 16-token tile edges, the middle of the chunk (where the halves of a
    # two-GPU row slicing meet), the quarter points, and random rows; all 16 heads of each
    rng = np.random.default_rng(4)
    rows = np.unique(np.concatenate([[0, 1, 15, 16, 17, 31, 32, 1023, 1024, 2047, 2048, 2049, 3071, 3072, 4079, 4080, 4094, 4095],
                                     rng.integers(0, tokens, 50)]))
    assert len(rows) >= 64
    print("config 4:", len(rows), "rows", check_rows(oracle, got, q, qg, kr.ravel(), vr.ravel(), pos, rows))


@pytest.mark.parametrize("bits", [8, 4])
def test_chunks_of_a_prompt_over_a_quantised_cache(oracle, bits):
    """A prompt prefilled in chunks over a quantised cache, read in place: no encode allocates device memory
    (there is no 16-bit copy of the cache), every chunk matches the oracle, the same call records into a Plan
    with or without `reserve`, and rows rewritten below the next chunk are simply seen."""
    import torch

    chunks = [(0, 200), (200, 120), (320, 64)]
    total = 384
    q, k, v, qg = bf16_inputs(oracle, 0, total, 700)
    cache = sa.GpuKvCache(0, bits, total)
    op = sa.AttGemm(0, 4096, KV)
    op.reserve(total)
    kr = oracle.round_trip_as_half(k, bits)
    vr = oracle.round_trip_as_half(v, bits)
    kd, vd = dev(k), dev(v)
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    for pos, n in chunks:
        cache.store_at(kd[pos * ROW:(pos + n) * ROW], vd[pos * ROW:(pos + n) * ROW], pos, n)  # src/prefill.rs:1656-1666
        sl = slice(pos * HEADS * DIM, (pos + n) * HEADS * DIM)
        gl = slice(pos * HEADS * 2 * DIM, (pos + n) * HEADS * 2 * DIM)
        got = run(torch, q[sl], None, None, qg[gl], pos, n, sa.BF16, quant=cache.quant(), op=op)
        check_rows(oracle, got, q[sl], qg[gl], kr, vr, pos, np.arange(n))
    # nothing was allocated by the library on the way (the test's own tensors come from torch's pool)
    assert torch.cuda.mem_get_info()[0] >= free0 - (8 << 20)

    # the last chunk again, recorded: an encode that has its scratch is capturable
    pos, n = chunks[-1]
    sl = slice(pos * HEADS * DIM, (pos + n) * HEADS * DIM)
    gl = slice(pos * HEADS * 2 * DIM, (pos + n) * HEADS * 2 * DIM)
    out = torch.zeros(n * HEADS * DIM, device="cuda")
    qd, gd = to16(torch, q[sl], sa.BF16), dev(qg[gl])
    plan = sa.Plan(0)
    with plan.recording():
        op.encode(qd, None, None, cache.quant(), gd, out, sa.FlashParams(HEADS, KV, pos, n, 1.0 / 16.0), dtype=sa.BF16,
                  stream=plan.stream)
    plan.run()
    check_rows(oracle, out.cpu().numpy().reshape(n, HEADS, DIM), q[sl], qg[gl], kr, vr, pos, np.arange(n))
    # an op that never reserved anything records the same call: nothing has to be allocated
    bare = sa.AttGemm(0, 4096, KV)
    plan2 = sa.Plan(0)
    out.zero_()
    with plan2.recording():
        bare.encode(qd, None, None, cache.quant(), gd, out, sa.FlashParams(HEADS, KV, pos, n, 1.0 / 16.0), dtype=sa.BF16,
                    stream=plan2.stream)
    plan2.run()
    check_rows(oracle, out.cpu().numpy().reshape(n, HEADS, DIM), q[sl], qg[gl], kr, vr, pos, np.arange(n))

    # rows below the chunk rewritten: the next encode reads the cache as it is
    k2 = k.copy()
    k2[:100 * ROW] = oracle.round_bf16(oracle.normal(100 * ROW, 701))
    cache.store_at(dev(k2[:100 * ROW]), vd[:100 * ROW], 0, 100)
    got = run(torch, q[sl], None, None, qg[gl], pos, n, sa.BF16, quant=cache.quant(), op=op)
    check_rows(oracle, got, q[sl], qg[gl], oracle.round_trip_as_half(k2, bits), vr, pos, np.arange(n))


@pytest.mark.parametrize("bits", [8, 4])
def test_quantised_cache_through_the_staging_copy(oracle, bits):
    """The other route to a quantised cache (kv_stage): with `stage_quantised` the op reads its 16-bit copy, of
    which every call converts only the rows it does not hold yet.  Same results as in place; the copy is
    allocated by `reserve`, and an encode that would have to grow it cannot be recorded."""
    import torch

    chunks = [(0, 200), (200, 120), (320, 64)]
    total = 384
    q, k, v, qg = bf16_inputs(oracle, 0, total, 710)
    cache = sa.GpuKvCache(0, bits, total)
    op = sa.AttGemm(0, 4096, KV)
    op.stage_quantised()
    op.reserve(total)
    kr = oracle.round_trip_as_half(k, bits)
    vr = oracle.round_trip_as_half(v, bits)
    kd, vd = dev(k), dev(v)
    in_place = sa.AttGemm(0, 4096, KV)
    for pos, n in chunks:
        cache.store_at(kd[pos * ROW:(pos + n) * ROW], vd[pos * ROW:(pos + n) * ROW], pos, n)
        sl = slice(pos * HEADS * DIM, (pos + n) * HEADS * DIM)
        gl = slice(pos * HEADS * 2 * DIM, (pos + n) * HEADS * 2 * DIM)
        got = run(torch, q[sl], None, None, qg[gl], pos, n, sa.BF16, quant=cache.quant(), op=op)
        check_rows(oracle, got, q[sl], qg[gl], kr, vr, pos, np.arange(n))
        same = run(torch, q[sl], None, None, qg[gl], pos, n, sa.BF16, quant=cache.quant(), op=in_place)
        # both routes feed the tensor cores the same binary16 operands (in blocks of 128 and of 64 keys: the
        # rounding of P sees different running maxima)
        assert np.abs(got - same).max() <= 2e-4 * max(1.0, np.abs(same).max())
    bare = sa.AttGemm(0, 4096, KV)
    bare.stage_quantised()
    pos, n = chunks[-1]
    sl = slice(pos * HEADS * DIM, (pos + n) * HEADS * DIM)
    out = torch.zeros(n * HEADS * DIM, device="cuda")
    plan = sa.Plan(0)
    qd, gd = to16(torch, q[sl], sa.BF16), dev(qg[:n * HEADS * 2 * DIM])
    with pytest.raises(sa.SaettaError):
        with plan.recording():
            bare.encode(qd, None, None, cache.quant(), gd, out, sa.FlashParams(HEADS, KV, pos, n, 1.0 / 16.0), dtype=sa.BF16,
                        stream=plan.stream)
    bare.stage_quantised(False)
    with pytest.raises(sa.SaettaError):
        sa._check(sa.lib().saetta_att_gemm_stage_quantised(None, 1))


@pytest.mark.parametrize("quant_bits,staged", [(None, False), (8, False), (8, True)])
def test_shards_that_store_only_their_slice(oracle, quant_bits, staged):
    """Split-KV prefill where every shard STORES only its own keys: row 0 of shard r's cache is the key at
    global position cuts[r].  The shards' partials merge to the oracle's result over the whole sequence."""
    import torch

    pos, tokens = 500, 150
    total = pos + tokens
    q, k, v, qg = bf16_inputs(oracle, pos, tokens, 800)
    cuts = [0, 192, 512, total]  # multiples of 64; the last shard holds part of the chunk itself
    p = sa.FlashParams(HEADS, KV, pos, tokens, 1.0 / 16.0)
    parts = torch.zeros((len(cuts) - 1, tokens * HEADS * sa.PART_STRIDE), dtype=torch.float32, device="cuda")
    qd = to16(torch, q, sa.BF16)
    keep = []
    for r in range(len(cuts) - 1):
        lo, hi = cuts[r], cuts[r + 1]
        op = sa.AttGemm(0, 4096, KV)
        op.stage_quantised(staged)  # the slice through the op's binary16 copy of it, or in place
        if quant_bits:
            c = sa.GpuKvCache(0, quant_bits, hi - lo)
            c.store_at(dev(k[lo * ROW:hi * ROW]), dev(v[lo * ROW:hi * ROW]), 0, hi - lo)
            op.partial(qd, None, None, c.quant(), parts[r], p, lo, hi, dtype=sa.BF16, key_base=lo)
            keep.append(c)
        else:
            kd, vd = to16(torch, k[lo * ROW:hi * ROW], sa.BF16), to16(torch, v[lo * ROW:hi * ROW], sa.BF16)
            op.partial(qd, kd, vd, None, parts[r], p, lo, hi, dtype=sa.BF16, key_base=lo)
            keep.append((kd, vd))
        keep.append(op)
    out = torch.zeros(tokens * HEADS * DIM, dtype=torch.float32, device="cuda")
    sa.merge_partials(0, parts, len(cuts) - 1, tokens, HEADS, dev(qg), out)
    torch.cuda.synchronize()
    got = out.cpu().numpy().reshape(tokens, HEADS, DIM)
    if quant_bits:
        kr, vr = oracle.round_trip_as_half(k, quant_bits), oracle.round_trip_as_half(v, quant_bits)
    else:
        kr, vr = k, v
    check_rows(oracle, got, q, qg, kr, vr, pos, np.arange(tokens))
    # a cache whose first row is not at a multiple of 64 is refused
    with pytest.raises(sa.SaettaError) as e:
        op.partial(qd, kd if not quant_bits else None, vd if not quant_bits else None, c.quant() if quant_bits else None,
                   parts[0], p, 100, 200, dtype=sa.BF16, key_base=100)
    assert e.value.code == sa.BAD_SHAPE


def test_bfloat16_values_keep_their_binary16_copy_between_chunks(oracle):
    """A bfloat16 cache: the values go through a binary16 copy (P takes the values' type), kept between the
    chunks of a prompt -- only rows from the chunk's first row on are converted again.  Rows rewritten below
    the next chunk behind the op's back are picked up after `invalidate`."""
    import torch

    total = 256
    q, k, v, qg = bf16_inputs(oracle, 0, total, 900)
    op = sa.AttGemm(0, 4096, KV)
    op.reserve(total)
    kd, vd = to16(torch, k, sa.BF16), to16(torch, v, sa.BF16)

    def chunk(pos, n, vref):
        sl = slice(pos * HEADS * DIM, (pos + n) * HEADS * DIM)
        gl = slice(pos * HEADS * 2 * DIM, (pos + n) * HEADS * 2 * DIM)
        out = torch.full((n * HEADS * DIM,), float("nan"), dtype=torch.float32, device="cuda")
        op.encode(to16(torch, q[sl], sa.BF16), kd, vd, None, dev(qg[gl]), out, sa.FlashParams(HEADS, KV, pos, n, 1.0 / 16.0), dtype=sa.BF16)
        torch.cuda.synchronize()
        return check_rows(oracle, out.cpu().numpy().reshape(n, HEADS, DIM), q[sl], qg[gl], k, vref, pos, np.arange(n))

    chunk(0, 160, v)
    chunk(160, 96, v)
    v2 = v.copy()
    v2[:64 * ROW] = oracle.round_bf16(oracle.normal(64 * ROW, 901))
    vd[:64 * ROW] = to16(torch, v2[:64 * ROW], sa.BF16)
    op.invalidate()
    chunk(160, 96, v2)
