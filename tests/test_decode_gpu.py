"""Decode and MTP-verify attention against the CPU oracle.

Mirrors tests/attention.rs of the reference (lengths around the 128-token chunk,
keys x4 so the softmax is peaky, quantised cache against the values the codes
stand for) and src/rows.rs:666-743 (m rows against the oracle's row-by-row
causal lengths), plus the benchmark configurations.  Tolerances: the f32 path
5e-6 relative RMS; the 16-bit and quantised paths 2e-3 max-abs and 1e-3
relative RMS (the reference's own GPU-vs-CPU bound is 2e-5 max-abs, which the
f32-arithmetic kernel is also held to).
"""
import numpy as np
import pytest

import saetta_macqwen_b200 as sa
from util import DIM, HEADS, KV, ROW, dev, max_abs, params_dev, quant_rows_from_oracle, rel_rms

pytestmark = pytest.mark.gpu


def inputs(oracle, capacity, m=1, key_gain=4.0):
    keys = oracle.noise(capacity * ROW, 1) * np.float32(key_gain)
    values = oracle.noise(capacity * ROW, 2)
    q = oracle.noise(m * HEADS * DIM, 3)
    qg = oracle.noise(m * HEADS * 2 * DIM, 4)
    return keys, values, q, qg


def run(op, m, q, qg, position, **kw):
    import torch

    out = torch.zeros(m * HEADS * DIM, dtype=torch.float32, device="cuda")
    p = params_dev(position)
    if "quant" in kw:
        op.record_quant(m, dev(q), kw["quant"][0], kw["quant"][1], dev(qg), out, p)
    elif "cache" in kw:
        op.record_cache(m, dev(q), kw["cache"], dev(qg), out, p)
    else:
        op.record(m, dev(q), kw["keys"], kw["values"], dev(qg), out, p, dtype=kw["dtype"])
    torch.cuda.synchronize()
    assert op.device_status() == 0
    return out.cpu().numpy().reshape(m, HEADS, DIM)


@pytest.mark.parametrize("dtype", [sa.F16, sa.BF16, sa.F32])
def test_plain_cache_matches_cpu_at_several_lengths(oracle, dtype):
    import torch

    capacity = 4096
    keys, values, q, qg = inputs(oracle, capacity)
    if dtype == sa.F16:
        keys, values = oracle.round_f16(keys), oracle.round_f16(values)
        kd, vd = dev(keys, torch.float16), dev(values, torch.float16)
    elif dtype == sa.BF16:
        keys, values = oracle.round_bf16(keys), oracle.round_bf16(values)
        kd, vd = dev(keys, torch.bfloat16), dev(values, torch.bfloat16)
    else:
        kd, vd = dev(keys), dev(values)
    op = sa.AttentionRows(0, HEADS, KV, capacity, 1)
    for n in [1, 2, 127, 128, 129, 1000, 4096]:
        got = run(op, 1, q, qg, n - 1, keys=kd, values=vd, dtype=dtype)
        want = oracle.attention_rows(q, qg, keys, values, [n])
        assert np.isfinite(got).all()
        # f32 rows: f32 arithmetic; binary16 rows: two 11-bit halves of q and of P, as good as f32;
        # bfloat16 rows: two 8-bit halves (16 bits), still 20x inside the 16-bit contract (2e-3 / 1e-3)
        tol_abs, tol_rms = (2e-4, 5e-5) if dtype == sa.BF16 else (2e-5, 5e-6)
        assert max_abs(got, want) < tol_abs, (dtype, n, max_abs(got, want))
        assert rel_rms(got, want) < tol_rms, (dtype, n, rel_rms(got, want))


@pytest.mark.parametrize("m", [1, 3])
def test_half_cache_long_context(oracle, m):
    """A binary16 cache long enough that every CTA walks several tiles and its copy ring wraps:
    one row (f32-exact: 5e-6) and three rows (two passes, rows rounded to binary16)."""
    tokens = 40000 + m - 1
    capacity = (tokens + 127) // 128 * 128
    keys, values = oracle.round_f16(oracle.normal(tokens * ROW, 21)), oracle.round_f16(oracle.normal(tokens * ROW, 22))
    q, qg = oracle.normal(m * HEADS * DIM, 23), oracle.normal(m * HEADS * 2 * DIM, 24)
    cache = sa.GpuKvCache(0, 16, capacity, dtype=sa.F16)
    cache.store_at(dev(keys), dev(values), 0, tokens)
    op = sa.AttentionRows(0, HEADS, KV, capacity, 4)
    pos = tokens - m
    got = run(op, m, q, qg, pos, cache=cache)
    want = oracle.attention_rows(q, qg, keys, values, [pos + r + 1 for r in range(m)], threads=8)
    if m == 1:
        assert rel_rms(got, want) < 5e-6, rel_rms(got, want)
    else:
        assert max_abs(got, want) < 2e-3 and rel_rms(got, want) < 1e-3, (max_abs(got, want), rel_rms(got, want))
    again = run(op, m, q, qg, pos, cache=cache)
    assert np.array_equal(got, again)  # fixed summation order: replays are bit-identical


@pytest.mark.parametrize("bits", [8, 4])
def test_quantized_matches_cpu(oracle, bits):
    capacity = 1024
    keys, values, q, qg = inputs(oracle, capacity)
    kq = quant_rows_from_oracle(sa, oracle, keys.reshape(-1, ROW), bits, capacity)
    vq = quant_rows_from_oracle(sa, oracle, values.reshape(-1, ROW), bits, capacity)
    keys, values = oracle.round_trip(keys, bits), oracle.round_trip(values, bits)
    op = sa.DecodeAttention(0, HEADS, KV, DIM, capacity)
    worst = 0.0
    for n in [1, 2, 15, 16, 17, 31, 32, 33, 127, 129, 1000, 1024]:
        import torch

        out = torch.zeros(HEADS * DIM, dtype=torch.float32, device="cuda")
        op.record_quant(dev(q), kq, vq, dev(qg), out, params_dev(n - 1))
        torch.cuda.synchronize()
        assert op.device_status() == 0
        got = out.cpu().numpy().reshape(1, HEADS, DIM)
        want = oracle.attention_rows(q, qg, keys, values, [n])
        assert np.isfinite(got).all(), n
        worst = max(worst, max_abs(got, want))
        assert max_abs(got, want) < 2e-3 and rel_rms(got, want) < 1e-3, (bits, n, max_abs(got, want), rel_rms(got, want))
    print(f"quantised {bits}-bit decode: worst abs error {worst:.3e}")


def test_config1_f32_decode(oracle):
    """1 row, 16 q / 2 kv heads of 256, context 4096, f32 Q/K/V ~N(0,1), partial
    RoPE on the first 64 dims (theta 1e7), scale 1/16, sigmoid gate."""
    n = 4096
    keys = oracle.rope_rows(oracle.normal(n * ROW, 101).reshape(n, ROW), DIM, 64, range(n), 1e7)
    values = oracle.normal(n * ROW, 102)
    q = oracle.rope_rows(oracle.normal(HEADS * DIM, 103).reshape(1, -1), DIM, 64, [n - 1], 1e7).ravel()
    qg = np.zeros((HEADS, 2 * DIM), np.float32)
    qg[:, DIM:] = oracle.normal(HEADS * DIM, 104).reshape(HEADS, DIM)
    cache = sa.GpuKvCache(0, 32, n)
    cache.store_at(dev(keys.ravel()), dev(values), 0, n)
    op = sa.DecodeAttention(0, HEADS, KV, DIM, n)
    got = run(op, 1, q, qg.ravel(), n - 1, cache=cache)
    want = oracle.attention_rows(q, qg, keys, values, [n])
    assert rel_rms(got, want) < 5e-6, rel_rms(got, want)


@pytest.mark.parametrize("bits", [8, 4, 16])
@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 8])
def test_verify_rows_match_cpu(oracle, bits, m):
    """Row r at position pos + r sees pos + r + 1 keys (src/rows.rs:379-381)."""
    capacity = 2048
    keys = oracle.normal(capacity * ROW, 7)
    values = oracle.normal(capacity * ROW, 8)
    q = oracle.normal(m * HEADS * DIM, 9)
    qg = oracle.normal(m * HEADS * 2 * DIM, 10)
    cache = sa.GpuKvCache(0, bits, capacity)
    cache.store_at(dev(keys), dev(values), 0, capacity)
    keys, values = oracle.round_trip(keys, bits), oracle.round_trip(values, bits)
    op = sa.AttentionRows(0, HEADS, KV, capacity, 8)
    for pos in [0, 37, 40, 1000, capacity - m]:
        got = run(op, m, q, qg, pos, cache=cache)
        want = oracle.attention_rows(q, qg, keys, values, [pos + r + 1 for r in range(m)], threads=8)
        assert np.isfinite(got).all()
        assert max_abs(got, want) < 2e-3 and rel_rms(got, want) < 1e-3, (bits, m, pos, max_abs(got, want), rel_rms(got, want))
    bad = sa.AttentionRows(0, HEADS, KV, capacity, 2)
    if m > 2:
        with pytest.raises(sa.SaettaError):
            run(bad, m, q, qg, 0, cache=cache)


@pytest.mark.parametrize("bits", [8])
def test_config3_mtp_verify_32k(oracle, bits):
    """4 query rows over a 32768-token 8-bit cache, the 4 new rows quantised on
    the device first (the store site), then attention; K, V ~ N(0,1)."""
    pos, m = 32768, 4
    capacity = pos + 128
    keys = oracle.normal((pos + m) * ROW, 31)
    values = oracle.normal((pos + m) * ROW, 32)
    q = oracle.normal(m * HEADS * DIM, 33)
    qg = oracle.normal(m * HEADS * 2 * DIM, 34)
    cache = sa.GpuKvCache(0, bits, capacity)
    cache.store_at(dev(keys[:pos * ROW]), dev(values[:pos * ROW]), 0, pos)
    cache.store(dev(keys[pos * ROW:]), dev(values[pos * ROW:]), params_dev(pos), rows=m)
    op = sa.AttentionRows(0, HEADS, KV, capacity, m)
    got = run(op, m, q, qg, pos, cache=cache)
    kr, vr = oracle.round_trip(keys, bits), oracle.round_trip(values, bits)
    want = oracle.attention_rows(q, qg, kr, vr, [pos + r + 1 for r in range(m)], threads=8)
    print(f"config 3: max abs {max_abs(got, want):.3e} rel rms {rel_rms(got, want):.3e}")
    assert max_abs(got, want) < 2e-3 and rel_rms(got, want) < 1e-3
    # replaying the same op is bit-identical (fixed merge order)
    again = run(op, m, q, qg, pos, cache=cache)
    assert np.array_equal(got, again)


def test_stale_rows_past_the_length_are_ignored(oracle):
    """Rows past kv_len may hold anything, NaN scales included."""
    import torch

    capacity, n = 256, 70
    keys, values, q, qg = inputs(oracle, capacity, key_gain=1.0)
    kq = quant_rows_from_oracle(sa, oracle, keys.reshape(-1, ROW), 8, capacity)
    vq = quant_rows_from_oracle(sa, oracle, values.reshape(-1, ROW), 8, capacity)
    for r in (kq, vq):
        d, s, z = r._keep
        s[n * 8:] = 0x7e00  # NaN
        z[n * 8:] = 0x7c00  # +inf
        d[n * 128:] = -1
    op = sa.DecodeAttention(0, HEADS, KV, DIM, capacity)
    out = torch.zeros(HEADS * DIM, dtype=torch.float32, device="cuda")
    op.record_quant(dev(q), kq, vq, dev(qg), out, params_dev(n - 1))
    got = out.cpu().numpy().reshape(1, HEADS, DIM)
    want = oracle.attention_rows(q, qg, oracle.round_trip(keys, 8), oracle.round_trip(values, 8), [n])
    assert np.isfinite(got).all() and max_abs(got, want) < 2e-3


@pytest.mark.parametrize("bits", [8, 4])
def test_batched_ragged_decode(oracle, bits):
    """Several sequences of ragged length in one launch against per-sequence oracles."""
    import torch

    lens = [1, 31, 32, 33, 500, 2047, 4096, 777, 64, 3000]
    n = len(lens)
    q = oracle.normal(n * HEADS * DIM, 50)
    qg = oracle.normal(n * HEADS * 2 * DIM, 51)
    caches, refs = [], []
    for i, L in enumerate(lens):
        k, v = oracle.normal(L * ROW, 60 + i), oracle.normal(L * ROW, 80 + i)
        c = sa.GpuKvCache(0, bits, L)
        c.store_at(dev(k), dev(v), 0, L)
        caches.append(c)
        refs.append((oracle.round_trip(k, bits), oracle.round_trip(v, bits)))
    op = sa.DecodeBatch(0, 16)
    out = torch.zeros(n * HEADS * DIM, dtype=torch.float32, device="cuda")
    op.record(caches, lens, dev(q), dev(qg), out)
    torch.cuda.synchronize()
    got = out.cpu().numpy().reshape(n, HEADS, DIM)
    for i, L in enumerate(lens):
        want = oracle.attention_rows(q.reshape(n, -1)[i], qg.reshape(n, -1)[i], refs[i][0], refs[i][1], [L])
        assert max_abs(got[i], want[0]) < 2e-3 and rel_rms(got[i], want[0]) < 1e-3, (bits, i, L)


@pytest.mark.parametrize("bits", [8, 4])
def test_config5_ragged_batch_of_64_long_sequences(oracle, bits):
    """64 sequences with lengths U[8192, 262144], 8- or 4-bit cache, one launch; the
    oracle checks the shortest, the longest and two others (the rest are checked
    for being finite)."""
    import torch

    rng = np.random.default_rng(5)
    lens = rng.integers(8192, 262145, 64)
    picked = sorted({int(np.argmin(lens)), int(np.argmax(lens)), 7, 40})
    g = torch.Generator(device="cuda")
    g.manual_seed(9)
    caches, refs = [], {}
    for i, L in enumerate(lens):
        L = int(L)
        c = sa.GpuKvCache(0, bits, L)
        for p0 in range(0, L, 32768):
            n = min(32768, L - p0)
            k = torch.randn(n * ROW, device="cuda", generator=g)
            v = torch.randn(n * ROW, device="cuda", generator=g)
            c.store_at(k, v, p0, n)
            if i in picked:
                kk, vv = refs.setdefault(i, ([], []))
                kk.append(oracle.round_trip(k.cpu().numpy(), bits))
                vv.append(oracle.round_trip(v.cpu().numpy(), bits))
        caches.append(c)
    n = len(lens)
    q = oracle.normal(n * HEADS * DIM, 50)
    qg = oracle.normal(n * HEADS * 2 * DIM, 51)
    op = sa.DecodeBatch(0, 64)
    out = torch.zeros(n * HEADS * DIM, dtype=torch.float32, device="cuda")
    op.record(caches, lens, dev(q), dev(qg), out)
    torch.cuda.synchronize()
    got = out.cpu().numpy().reshape(n, HEADS, DIM)
    assert np.isfinite(got).all()
    for i in picked:
        kk, vv = np.concatenate(refs[i][0]), np.concatenate(refs[i][1])
        want = oracle.attention_rows(q.reshape(n, -1)[i], qg.reshape(n, -1)[i], kk, vv, [int(lens[i])], threads=16)
        print(f"config 5, {bits}-bit, sequence {i} of {int(lens[i])} tokens: max abs {max_abs(got[i], want[0]):.3e} "
              f"rel rms {rel_rms(got[i], want[0]):.3e}")
        assert max_abs(got[i], want[0]) < 2e-3 and rel_rms(got[i], want[0]) < 1e-3, (bits, i, int(lens[i]))


def test_row_backup_and_resize_keep_rows(oracle):
    """src/gpu_cache.rs:234-274 and src/gpu_layers.rs:261-292: rows copied aside
    and put back, and a resize, leave attention results unchanged."""
    capacity, n = 512, 300
    keys, values, q, qg = inputs(oracle, capacity, key_gain=1.0)
    cache = sa.GpuKvCache(0, 8, capacity)
    cache.store_at(dev(keys), dev(values), 0, capacity)
    op = sa.DecodeAttention(0, HEADS, KV, DIM, 1024)
    base = run(op, 1, q, qg, n - 1, cache=cache)
    backup = sa.RowBackup()
    backup.save([cache], 100, 64)
    assert backup.bytes() == 64 * (512 + 512 + 4 * 16)
    junk = oracle.normal(64 * ROW, 99)
    cache.store_at(dev(junk), dev(junk), 100, 64)
    assert not np.array_equal(run(op, 1, q, qg, n - 1, cache=cache), base)
    backup.restore([cache])
    assert backup.bytes() == 0
    assert np.array_equal(run(op, 1, q, qg, n - 1, cache=cache), base)
    cache.resize(1024)
    assert cache.capacity == 1024
    assert np.array_equal(run(op, 1, q, qg, n - 1, cache=cache), base)
    cache.resize(384)
    assert np.array_equal(run(op, 1, q, qg, n - 1, cache=cache), base)
