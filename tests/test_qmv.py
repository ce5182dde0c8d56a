"""Quantised projections (src/qmv.rs, src/rows.rs:47-110): the oracle's restatement of the CPU's
quantised matvec (src/cpu/matrix.rs:73-135) on the reference's own test matrices, then the kernel
against the oracle."""
import numpy as np
import pytest

import saetta_macqwen_b200 as sa


def bf16_bits(x):
    """Round-to-nearest-even bfloat16 bit patterns of f32 values (crate half's bf16::from_f32)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def bf16_to_f32(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


def pack(q, bits):
    """[rows][cols] integers -> the little-endian bit stream of src/quant.rs:1-30, as u32 words."""
    rows, cols = q.shape
    bitsarr = ((q[:, :, None].astype(np.uint64) >> np.arange(bits, dtype=np.uint64)) & 1).astype(np.uint8)
    stream = bitsarr.reshape(rows, cols * bits)
    return np.packbits(stream, axis=1, bitorder="little").view(np.uint32).reshape(rows, cols * bits // 32)


def reference_sample(bits, rows, cols):
    """The matrices of the reference's own test (src/cpu/matrix.rs:147-181) and its x (:204-206)."""
    r, i = np.arange(rows)[:, None], np.arange(cols)[None, :]
    q = ((r * 7 + i * 13) % (1 << bits)).astype(np.uint32)
    n = rows * cols // 64
    scales = bf16_bits(np.float32(0.01) + np.arange(n, dtype=np.float32) * np.float32(1e-3))
    biases = bf16_bits(np.float32(-0.1) + np.arange(n, dtype=np.float32) * np.float32(2e-3))
    x = ((np.arange(cols) * 31 % 17).astype(np.float32) - np.float32(8.0)) * np.float32(0.1)
    return q, pack(q, bits), scales, biases, x


def dense(q, scales, biases):
    rows, cols = q.shape
    s = bf16_to_f32(scales).reshape(rows, cols // 64).repeat(64, axis=1)
    b = bf16_to_f32(biases).reshape(rows, cols // 64).repeat(64, axis=1)
    return s * q.astype(np.float32) + b  # src/quant.rs:33-39, f32 like the reference


@pytest.mark.parametrize("bits", [5, 8])
def test_oracle_matvec_matches_dequantize_on_the_reference_sample(oracle, bits):
    """src/cpu/matrix.rs:183-237 `quantized_matvec_matches_dequantize`: 300 x 1024, tolerance 1e-3 * max(1, |want|)."""
    rows, cols = 300, 1024
    q, words, scales, biases, x = reference_sample(bits, rows, cols)
    got = oracle.quant_matvec(words, scales, biases, bits, rows, cols, x)
    w = dense(q, scales, biases)
    want = np.array([np.float32(0)] * rows)
    for r in range(rows):  # ops::matvec: left-to-right f32 sum of products
        t = np.float32(0)
        for v in (w[r] * x):
            t = np.float32(t + v)
        want[r] = t
    assert (np.abs(got - want) <= 1e-3 * np.maximum(1.0, np.abs(want))).all()
    exact = (w.astype(np.float64) * x.astype(np.float64)).sum(axis=1)
    assert np.abs(got - exact).max() < 2e-3 * max(1.0, np.abs(exact).max())


@pytest.mark.gpu
@pytest.mark.parametrize("bits", [5, 6, 8])
@pytest.mark.parametrize("m", [1, 2, 3, 4, 8])
def test_kernel_matches_oracle(oracle, bits, m):
    """The reference's GPU test metric (tests/qmv.rs:66-82): worst |y - exact| / sum|w x| < 1e-5, here against
    f64 sums of the dequantised matrix, on the reference's sample and on a projection-sized random matrix."""
    import torch

    from util import dev

    rng = np.random.default_rng(bits * 10 + m)
    cases = [reference_sample(bits, 300, 1024)]
    # teams of 16, 32 and 8 lanes (the last with three units per lane), and a row length only the general kernel takes
    for rows, cols in ((1100, 2048), (70, 4096), (37, 3072), (33, 320)):
        q = rng.integers(0, 1 << bits, (rows, cols), dtype=np.uint32)
        cases.append((q, pack(q, bits), bf16_bits(rng.uniform(0.001, 0.02, rows * cols // 64).astype(np.float32)),
                      bf16_bits(rng.uniform(-0.2, 0.0, rows * cols // 64).astype(np.float32)), None))
    for q, words, scales, biases, x0 in cases:
        rows, cols = q.shape
        x = rng.standard_normal((m, cols)).astype(np.float32)
        if x0 is not None:
            x[0] = x0
        y = torch.full((m, rows + 5), 9.0, device="cuda")
        sa.qmv_rows(0, dev(words.view(np.int32)), dev(scales.view(np.int16)), dev(biases.view(np.int16)), bits, rows, cols, m,
                    dev(x), y, y_stride=rows + 5)
        torch.cuda.synchronize()
        got = y.cpu().numpy()
        assert (got[:, rows:] == 9.0).all()
        w = dense(q, scales, biases).astype(np.float64)
        for r in range(m):
            exact = w @ x[r].astype(np.float64)
            scale = np.abs(w) @ np.abs(x[r].astype(np.float64))
            assert (np.abs(got[r, :rows] - exact) / (scale + 1e-12)).max() < 1e-5
            want = oracle.quant_matvec(words, scales, biases, bits, rows, cols, x[r])
            assert (np.abs(got[r, :rows] - want) / (scale + 1e-12)).max() < 1e-5


@pytest.mark.gpu
def test_shape_errors():
    import torch

    z = torch.zeros(4096, device="cuda")
    for bits, rows, cols, m in [(4, 8, 64, 1), (5, 8, 100, 1), (5, 8, 64, 9), (5, 8, 64, 0)]:
        with pytest.raises(sa.SaettaError):
            sa.qmv_rows(0, z, z, z, bits, rows, cols, m, z, z)
