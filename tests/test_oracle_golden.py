"""The CPU oracle against the reference's own golden vectors and known answers.

Mirrors src/cpu/attention.rs:188-221, src/cpu/ops.rs:81-110 and
src/kv_quant.rs:302-332 of the reference, on the fixtures under tests/golden/.
"""
import json
import os

import numpy as np


def _load(golden_dir, name):
    with open(os.path.join(golden_dir, name)) as f:
        return json.load(f)


def _assert_close(what, got, want, tol):
    # cpu::testdata::assert_close: |g - w| <= tol * max(1, |w|)
    got, want = np.asarray(got, np.float32), np.asarray(want, np.float32)
    assert got.shape == want.shape, what
    limit = tol * np.maximum(np.abs(want), 1.0)
    bad = np.abs(got - want) > limit
    assert not bad.any(), f"{what}: {np.argwhere(bad)[:4].ravel()} worst {np.abs(got - want).max()}"


def test_ops_match_mlx(oracle, golden_dir):
    f = _load(golden_dir, "ops_mlx.json")
    _assert_close("rms_norm", oracle.rms_norm(f["x"], f["w"], 1e-6), f["rms_norm"], 1e-5)
    _assert_close("softmax", oracle.softmax(f["x"]), f["softmax"], 1e-6)


def test_rope_matches_mlx(oracle, golden_dir):
    f = _load(golden_dir, "ops_mlx.json")
    for pos, want in zip(f["rope_positions"], f["rope_out"]):
        x = np.asarray(f["rope_in"], np.float32).reshape(-1, 16)
        got = np.concatenate([oracle.rope(h, 4, pos, 1e7) for h in x])
        _assert_close(f"rope at {pos}", got, want, 1e-4)


def test_attention_matches_mlx_over_four_tokens(oracle, golden_dir):
    f = _load(golden_dir, "attention_mlx.json")
    cfg = {k: f[k] for k in ("hidden", "heads", "kv_heads", "head_dim", "rope_dims", "rope_theta", "eps")}
    w = {k: f[k] for k in ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm")}
    layer = oracle.Layer(cfg, w)
    for t, (x, want) in enumerate(zip(f["inputs"], f["outputs"])):
        _assert_close(f"token {t}", layer.step(x), want, 1e-4)
    assert layer.len.value == 4


def test_attention_rows_equals_layer_inner_part(oracle, golden_dir):
    """attention_rows (the function the CUDA path is checked against) is the same
    arithmetic as the layer replay: feed it the layer's own cache."""
    f = _load(golden_dir, "attention_mlx.json")
    h, kv, d = f["heads"], f["kv_heads"], f["head_dim"]
    cfg = {k: f[k] for k in ("hidden", "heads", "kv_heads", "head_dim", "rope_dims", "rope_theta", "eps")}
    w = {k: np.asarray(f[k], np.float32) for k in ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm")}
    layer = oracle.Layer(cfg, w)
    for t, (x, want) in enumerate(zip(f["inputs"], f["outputs"])):
        layer.step(x)
        x = np.asarray(x, np.float32)
        qg = (w["q_proj"].reshape(2 * h * d, -1) @ x).astype(np.float32)
        qg = np.array([oracle.dot(r, x) for r in w["q_proj"].reshape(2 * h * d, -1)], np.float32)
        q = qg.reshape(h, 2 * d)[:, :d].copy()
        q = np.stack([oracle.rope(oracle.rms_norm(r, w["q_norm"], f["eps"]), f["rope_dims"], t, f["rope_theta"]) for r in q])
        out = oracle.attention_rows(q, qg, layer.keys, layer.values, [t + 1], heads=h, kv_heads=kv, d=d)
        y = np.array([oracle.dot(r, out.ravel()) for r in w["o_proj"].reshape(-1, h * d)], np.float32)
        _assert_close(f"token {t}", y, want, 1e-4)


def test_codes_pack_lowest_bits_first(oracle, golden_dir):
    k = _load(golden_dir, "kv_quant_known.json")
    x = np.zeros(64, np.float32)
    x[k["ones_at"]] = 1.0
    data, _, _ = oracle.quantize(x, 8)
    assert len(data) == k["bits8"]["words"]
    assert data[0] == k["bits8"]["word0"] and data[15] == k["bits8"]["word15"]
    data, _, _ = oracle.quantize(x, 4)
    assert len(data) == k["bits4"]["words"]
    assert data[0] == k["bits4"]["word0"] and data[7] == k["bits4"]["word7"]


def test_round_trip_is_within_half_a_step(oracle):
    x = oracle.noise(4 * 64, 1)
    x[64:128] = 0.37  # a constant group: scale 0, every value exact
    for bits in (8, 4):
        _, scales, _ = oracle.quantize(x, bits)
        y = oracle.round_trip(x, bits)
        step = np.repeat(oracle.from_f16_bits(scales), 64)
        slack = step / 2 + np.abs(x) * 1e-3 + 1e-6
        assert (np.abs(x - y) <= slack).all(), bits
        assert np.array_equal(y[64:128], oracle.round_f16(x[64:128]))


def test_f16_conversion_matches_numpy(oracle):
    rng = np.random.default_rng(0)
    x = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * 10.0 ** rng.integers(-9, 6, 20000),
        np.array([0.0, -0.0, 65504.0, 65520.0, 65519.9, 1e-8, 5.96e-8, 2.98e-8, 2.981e-8, 6.1e-5, np.inf, -np.inf], np.float32),
        np.arange(0, 70000, 7).astype(np.float32),
    ]).astype(np.float32)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16)
    assert np.array_equal(oracle.to_f16_bits(x), want.view(np.uint16))
    assert np.array_equal(oracle.from_f16_bits(want.view(np.uint16)).view(np.uint32), want.astype(np.float32).view(np.uint32))
    allbits = np.arange(65536, dtype=np.uint16)
    back = oracle.from_f16_bits(allbits)
    ref = allbits.view(np.float16).astype(np.float32)
    ok = np.isnan(ref) | (back.view(np.uint32) == ref.view(np.uint32))
    assert ok.all()


def test_bf16_conversion_matches_torch(oracle):
    import torch

    x = torch.randn(20000) * 10.0 ** torch.randint(-9, 6, (20000,))
    want = x.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(oracle.to_bf16_bits(x.numpy()), want)


def test_quantize_matches_numpy_restatement(oracle):
    """A second, independent restatement in numpy f32 arithmetic agrees bit for bit."""
    x = (oracle.noise(37 * 512, 7).reshape(-1, 64) * np.where(np.arange(37 * 8) % 3 == 0, 20.0, 1.0)[:, None]).astype(np.float32)
    x[1] = -1.5
    for bits in (8, 4):
        levels = np.float32((1 << bits) - 1)
        lo, hi = x.min(1), x.max(1)
        s = ((hi - lo) / levels).astype(np.float32).astype(np.float16)
        z = lo.astype(np.float16)
        sf, zf = s.astype(np.float32), z.astype(np.float32)
        with np.errstate(divide="ignore"):
            inv = np.where(sf > 0, np.float32(1) / sf, np.float32(0)).astype(np.float32)
        q = np.clip(np.rint(((x - zf[:, None]).astype(np.float32) * inv[:, None]).astype(np.float32)), 0, levels).astype(np.uint32)
        per = 32 // bits
        words = (q.reshape(-1, per) << (np.arange(per, dtype=np.uint32) * bits)).sum(1).astype(np.uint32)
        data, gs, gz = oracle.quantize(x.ravel(), bits)
        assert np.array_equal(gs, s.view(np.uint16)) and np.array_equal(gz, z.view(np.uint16))
        assert np.array_equal(data, words)
        want = (sf[:, None] * q.astype(np.float32)).astype(np.float32) + zf[:, None]
        assert np.array_equal(oracle.dequantize(data, gs, gz, bits), want.ravel().astype(np.float32))
