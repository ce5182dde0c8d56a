"""kv_quantize / kv_dequantize kernels against the oracle, bit for bit.

Mirrors tests/kv_quant.rs of the reference (prefill_rows_match_cpu,
decode_row_matches_cpu, dequantize_matches_cpu) with its inputs -- groups
scaled by 20, a constant group, 37 tokens at position 5, a decode row at 41 --
but with no slack: codes, scales and biases must all be equal.
"""
import numpy as np
import pytest

import saetta_macqwen_b200 as sa
from util import ROW, dev, params_dev, read_dev

pytestmark = pytest.mark.gpu
GROUP = 64


def rows(oracle, tokens):
    x = oracle.noise(tokens * ROW, 7)
    scale = np.where((np.arange(x.size) // GROUP) % 3 == 0, 20.0, 1.0).astype(np.float32)
    x = x * scale
    x[GROUP:2 * GROUP] = -1.5
    return x


def read_rows(q, tokens_from, tokens, bits):
    import torch

    d, s, z = q._keep
    torch.cuda.synchronize()
    words = 8 * 2 * bits
    data = d[tokens_from * words:(tokens_from + tokens) * words].cpu().numpy().view(np.uint32)
    sc = s[tokens_from * 8:(tokens_from + tokens) * 8].cpu().numpy().view(np.uint16)
    bi = z[tokens_from * 8:(tokens_from + tokens) * 8].cpu().numpy().view(np.uint16)
    return data, sc, bi


def make(bits, capacity):
    import torch

    words = 8 * 2 * bits
    d = torch.full((capacity * words,), 0x5a5a5a5a, dtype=torch.int32, device="cuda")
    s = torch.full((capacity * 8,), 0x3c00, dtype=torch.int16, device="cuda")
    z = torch.full((capacity * 8,), 0x3c00, dtype=torch.int16, device="cuda")
    return sa.QuantRows.wrap(0, bits, ROW, capacity, d, s, z)


def compare(q, oracle, x, from_token, bits):
    tokens = x.size // ROW
    got = read_rows(q, from_token, tokens, bits)
    want = oracle.quantize(x, bits)
    assert np.array_equal(got[1], want[1]), f"{bits} scales"
    assert np.array_equal(got[2], want[2]), f"{bits} biases"
    assert np.array_equal(got[0], want[0]), f"{bits} codes: {(got[0] != want[0]).sum()} words differ"


@pytest.mark.parametrize("bits", [8, 4])
def test_prefill_rows_match_cpu(oracle, bits):
    tokens = 37
    q = make(bits, 64)
    x = rows(oracle, tokens)
    q.encode(dev(x), 5, tokens)
    compare(q, oracle, x, 5, bits)
    # rows outside 5..42 are untouched
    before = read_rows(q, 0, 5, bits)
    assert (before[0] == 0x5a5a5a5a).all() and (before[1] == 0x3c00).all()
    after = read_rows(q, 42, 22, bits)
    assert (after[0] == 0x5a5a5a5a).all() and (after[2] == 0x3c00).all()


@pytest.mark.parametrize("bits", [8, 4])
def test_decode_row_matches_cpu(oracle, bits):
    q = make(bits, 64)
    x = rows(oracle, 1)
    q.record(dev(x), params_dev(41))
    compare(q, oracle, x, 41, bits)


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("dtype", [sa.F16, sa.BF16])
def test_dequantize_matches_cpu(oracle, bits, dtype):
    import torch

    tokens = 9
    q = make(bits, 64)
    x = rows(oracle, tokens)
    q.encode(dev(x), 0, tokens)
    out = torch.zeros(tokens * ROW, dtype=torch.int16, device="cuda")
    q.encode_dequantize(out, tokens, dtype=dtype)
    got = out.cpu().numpy().view(np.uint16)
    want = oracle.dequantize(*oracle.quantize(x, bits), bits)
    want = oracle.to_f16_bits(want) if dtype == sa.F16 else oracle.to_bf16_bits(want)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("bits", [8, 4])
def test_verify_rows_append_bit_exact(oracle, bits):
    """The MTP-verify store: 4 new K and V rows ~N(0,1) at positions 32768.. of a cache."""
    import torch

    cache = sa.GpuKvCache(0, bits, 32768 + 128)
    k = oracle.normal(4 * ROW, 11)
    v = oracle.normal(4 * ROW, 12)
    cache.store(dev(k), dev(v), params_dev(32768), rows=4)
    torch.cuda.synchronize()
    bufs = cache.buffers()
    assert [rb for _, rb in bufs] == [64 * bits, 64 * bits, 16, 16, 16, 16]
    # the raw words, scales and biases of the four rows, both sides, straight from the cache's buffers
    pos = 32768
    (kd, cb), (vd, _), (ks, pb), (kz, _), (vs, _), (vz, _) = bufs
    for data, scales, biases, x in ((kd, ks, kz, k), (vd, vs, vz, v)):
        want_d, want_s, want_z = oracle.quantize(x, bits)
        assert np.array_equal(read_dev(data + pos * cb, 4 * cb).view(np.uint32), want_d)
        assert np.array_equal(read_dev(scales + pos * pb, 4 * pb).view(np.uint16), want_s)
        assert np.array_equal(read_dev(biases + pos * pb, 4 * pb).view(np.uint16), want_z)
    # and through a dequantise of the whole prefix
    kq, vq = cache.quant()
    for side, x in ((kq, k), (vq, v)):
        out = torch.zeros((32768 + 4) * ROW, dtype=torch.int16, device="cuda")
        side.encode_dequantize(out, 32768 + 4)
        got = out[32768 * ROW:].cpu().numpy().view(np.uint16)
        want = oracle.to_f16_bits(oracle.round_trip(x, bits))
        assert np.array_equal(got, want)
    assert sa.lib().saetta_kv_cache_store(cache.h, dev(k).data_ptr(), dev(v).data_ptr(),
                                          params_dev(0).data_ptr(), 9, None) == sa.BAD_SHAPE


@pytest.mark.parametrize("bits", [8, 4])
def test_large_chunk_and_edge_values(oracle, bits):
    """A 4096-token prefill chunk with hostile values: zeros, a constant group,
    huge and tiny ranges, ties at half codes, a NaN-free but denormal group."""
    tokens = 4096
    x = oracle.normal(tokens * ROW, 5).reshape(-1, GROUP)
    x[0] = 0.0
    x[1] = 0.37
    x[2] *= 1e4
    x[3] *= 1e-6
    x[4] = np.arange(64, dtype=np.float32) / 2.0  # exact ties for round-half-even
    x[5] = 1e-41
    x[6] = np.linspace(-65504, 65504, 64, dtype=np.float32)
    x[7] = np.float32(3.0e38) * np.sign(x[7])
    q = make(bits, tokens)
    q.encode(dev(x.ravel()), 0, tokens)
    compare(q, oracle, x.ravel(), 0, bits)


def test_store_into_half_and_f32_caches(oracle):
    import torch

    k, v = oracle.normal(3 * ROW, 21), oracle.normal(3 * ROW, 22)
    for bits, dtype in ((16, sa.F16), (16, sa.BF16), (32, sa.F16)):
        cache = sa.GpuKvCache(0, bits, 128, dtype=dtype)
        cache.store_at(dev(k), dev(v), 7, 3)
        torch.cuda.synchronize()
        (kp, rb), (vp, _) = cache.buffers()
        assert rb == ROW * (4 if bits == 32 else 2)
        # the stored rows, read back raw: the reference's to_half narrowing (binary16), this build's
        # bfloat16 twin, or the f32 values themselves; and again after a resize up and down
        for _ in range(2):
            (kp, rb), (vp, _) = cache.buffers()
            for ptr, x in ((kp, k), (vp, v)):
                raw = read_dev(ptr + 7 * rb, 3 * rb)
                if bits == 32:
                    assert np.array_equal(raw.view(np.float32), x)
                elif dtype == sa.F16:
                    assert np.array_equal(raw.view(np.uint16), oracle.to_f16_bits(x))
                else:
                    assert np.array_equal(raw.view(np.uint16), oracle.to_bf16_bits(x))
            cache.resize(256)
            assert cache.capacity == 256
            cache.resize(128)
            assert cache.capacity == 128
