"""Attention prep fused with the cache store: q and k RMS-norm + partial RoPE, k and v
into the cache in its own format (kernels/layers.metal:637-697 followed by
QuantRows::record, src/gpu_layers.rs:373-411, 483-507; src/prefill.rs:1607-1666).

q and the f32 copy of k are compared with the oracle's rms_norm and rope
(src/cpu/ops.rs:19-36, 64-74): only the order of the sum of squares differs, so
a few ulp.  What lands in a quantised cache must be, bit for bit, the oracle's
quantisation of that f32 copy, and of v as given."""
import numpy as np
import pytest

import saetta_macqwen_b200 as sa
from util import DIM, HEADS, KV, ROW, dev, params_dev, read_dev

pytestmark = pytest.mark.gpu
ROPE_DIMS, THETA, EPS = 64, 1.0e7, 1.0e-6
P = sa.PrepParams(HEADS, KV, DIM, ROPE_DIMS, THETA, EPS)


def inputs(oracle, rows, seed):
    qg = oracle.normal(rows * HEADS * 2 * DIM, seed) * 1.7
    k = oracle.normal(rows * ROW, seed + 1) * 0.6
    v = oracle.normal(rows * ROW, seed + 2)
    qn = 1.0 + 0.1 * oracle.normal(DIM, seed + 3)
    kn = 1.0 + 0.1 * oracle.normal(DIM, seed + 4)
    return [np.ascontiguousarray(a, np.float32) for a in (qg, k, v, qn, kn)]


def want_heads(oracle, x, w, positions):
    """rope(rms_norm(head) * w) for x [rows][heads][DIM] at positions[row]."""
    out = np.empty_like(x)
    for r in range(x.shape[0]):
        for h in range(x.shape[1]):
            out[r, h] = oracle.rope(oracle.rms_norm(x[r, h], w, EPS), ROPE_DIMS, int(positions[r]), THETA)
    return out


def check_f32(got, want, what):
    err = np.abs(got.astype(np.float64) - want.astype(np.float64)).max()
    assert err <= 4e-6 * max(1.0, float(np.abs(want).max())), f"{what}: max abs error {err}"


def cache_rows(cache, first, rows, bits):
    """(key data, k scales, k biases, value data, v scales, v biases) of `rows` tokens, as stored."""
    bufs = cache.buffers()
    out = []
    for i in (0, 2, 3, 1, 4, 5):
        p, rb = bufs[i]
        raw = read_dev(p + first * rb, rows * rb)
        out.append(raw.view(np.uint32) if i < 2 else raw.view(np.uint16))
    return out


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("rows,position", [(1, 41), (4, 32768), (3, 200000)])
def test_decode_rows_into_a_quantised_cache(oracle, bits, rows, position):
    import torch

    capacity = (position + rows + 127) // 128 * 128
    qg, k, v, qn, kn = inputs(oracle, rows, 100 + rows)
    cache = sa.GpuKvCache(0, bits, capacity)
    q_out = torch.zeros(rows * HEADS * DIM, device="cuda")
    k_out = torch.zeros(rows * ROW, device="cuda")
    sa.attention_prep(P, rows, dev(qg), dev(k), dev(v), dev(qn), dev(kn), q_out, sa.F32, cache,
                      params=params_dev(position), k_out=k_out)
    positions = position + np.arange(rows)
    q = qg.reshape(rows, HEADS, 2 * DIM)[:, :, :DIM]
    check_f32(q_out.cpu().numpy().reshape(rows, HEADS, DIM), want_heads(oracle, q, qn, positions), "q")
    k_gpu = k_out.cpu().numpy()
    check_f32(k_gpu.reshape(rows, KV, DIM), want_heads(oracle, k.reshape(rows, KV, DIM), kn, positions), "k")
    kd, ks, kz, vd, vs, vz = cache_rows(cache, position, rows, bits)
    for got, want, what in ((( kd, ks, kz), oracle.quantize(k_gpu, bits), "keys"), ((vd, vs, vz), oracle.quantize(v, bits), "values")):
        assert np.array_equal(got[1], want[1]), f"{what}: scales"
        assert np.array_equal(got[2], want[2]), f"{what}: biases"
        assert np.array_equal(got[0], want[0]), f"{what}: {(got[0] != want[0]).sum()} code words differ"


@pytest.mark.parametrize("dtype", [sa.F16, sa.BF16])
def test_prefill_rows_into_a_16_bit_cache(oracle, dtype):
    import torch

    rows, pos, capacity = 70, 1000, 1152
    qg, k, v, qn, kn = inputs(oracle, rows, 7)
    cache = sa.GpuKvCache(0, 16, capacity, dtype=dtype)
    q_out = torch.zeros(rows * HEADS * DIM, dtype=torch.int16, device="cuda")
    sa.attention_prep(P, rows, dev(qg), dev(k), dev(v), dev(qn), dev(kn), q_out, dtype, cache, pos=pos)
    positions = pos + np.arange(rows)
    narrow = oracle.to_f16_bits if dtype == sa.F16 else oracle.to_bf16_bits
    widen = (lambda b: b.view(np.float16).astype(np.float32)) if dtype == sa.F16 else \
        (lambda b: (b.astype(np.uint32) << 16).view(np.float32))
    ulp = 2.0 ** -10 if dtype == sa.F16 else 2.0 ** -7
    q_want = want_heads(oracle, qg.reshape(rows, HEADS, 2 * DIM)[:, :, :DIM], qn, positions)
    k_want = want_heads(oracle, k.reshape(rows, KV, DIM), kn, positions)
    q_got = widen(q_out.cpu().numpy().view(np.uint16)).reshape(q_want.shape)
    assert (np.abs(q_got - q_want) <= ulp * np.abs(q_want) + 1e-6).all()
    (kp, rb), (vp, _) = cache.buffers()
    k_got = widen(read_dev(kp + pos * rb, rows * rb).view(np.uint16)).reshape(k_want.shape)
    assert (np.abs(k_got - k_want) <= ulp * np.abs(k_want) + 1e-6).all()
    # values are narrowed and nothing else
    v_got = read_dev(vp + pos * rb, rows * rb).view(np.uint16)
    assert np.array_equal(v_got, narrow(v))


def test_f32_cache_and_in_place_keys(oracle):
    import torch

    rows, pos = 5, 17
    qg, k, v, qn, kn = inputs(oracle, rows, 31)
    cache = sa.GpuKvCache(0, 32, 128)
    q_out = torch.zeros(rows * HEADS * DIM, device="cuda")
    kd = dev(k)
    sa.attention_prep(P, rows, dev(qg), kd, dev(v), dev(qn), dev(kn), q_out, sa.F32, cache, pos=pos, k_out=kd)
    k_want = want_heads(oracle, k.reshape(rows, KV, DIM), kn, pos + np.arange(rows))
    check_f32(kd.cpu().numpy().reshape(k_want.shape), k_want, "k written back in place")
    (kp, rb), (vp, _) = cache.buffers()
    assert np.array_equal(read_dev(kp + pos * rb, rows * rb).view(np.float32), kd.cpu().numpy())
    assert np.array_equal(read_dev(vp + pos * rb, rows * rb).view(np.float32), v)


def test_prep_then_decode_matches_the_oracle_layer(oracle):
    """Prep + quantised store + decode attention for one new token, against the CPU path run the
    same way: norm, rope, round trip through the 8-bit format, attend, gate."""
    import torch

    ctx, bits = 2048, 8
    keys, values = oracle.normal(ctx * ROW, 1), oracle.normal(ctx * ROW, 2)
    qg, k, v, qn, kn = inputs(oracle, 1, 55)
    cache = sa.GpuKvCache(0, bits, ctx + 128)
    cache.store_at(dev(keys), dev(values), 0, ctx)
    q_out = torch.zeros(HEADS * DIM, device="cuda")
    out = torch.zeros(HEADS * DIM, device="cuda")
    p = params_dev(ctx)
    sa.attention_prep(P, 1, dev(qg), dev(k), dev(v), dev(qn), dev(kn), q_out, sa.F32, cache, params=p)
    op = sa.AttentionRows(0, HEADS, KV, ctx + 128, 1)
    op.record_cache(1, q_out, cache, dev(qg), out, p)
    q_want = want_heads(oracle, qg.reshape(1, HEADS, 2 * DIM)[:, :, :DIM], qn, [ctx])
    k_want = want_heads(oracle, k.reshape(1, KV, DIM), kn, [ctx])
    all_k = np.concatenate([oracle.round_trip(keys, bits), oracle.round_trip(k_want.ravel(), bits)])
    all_v = np.concatenate([oracle.round_trip(values, bits), oracle.round_trip(v, bits)])
    want = oracle.attention_rows(q_want, qg, all_k, all_v, [ctx + 1], threads=4)
    err = np.abs(out.cpu().numpy().reshape(want.shape) - want).max()
    assert err < 2e-3, err


def test_shape_errors(oracle):
    import torch

    cache = sa.GpuKvCache(0, 8, 128)
    x = torch.zeros(HEADS * 2 * DIM, device="cuda")
    bad = sa.PrepParams(HEADS, KV, 128, ROPE_DIMS, THETA, EPS)
    with pytest.raises(sa.SaettaError) as e:
        sa.attention_prep(bad, 1, x, x, x, x, x, x, sa.F32, cache, pos=0)
    assert e.value.code == sa.BAD_SHAPE
    with pytest.raises(sa.SaettaError) as e:
        sa.attention_prep(P, 2, x, x, x, x, x, x, sa.F32, cache, pos=127)
    assert e.value.code == sa.BAD_SHAPE
