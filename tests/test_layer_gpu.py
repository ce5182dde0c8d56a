"""The attention layer as the reference runs it for one token (src/cpu/attention.rs:103-156,
GpuAttention::record in src/gpu_layers.rs:300-368), chained from this library's pieces and recorded once in
a Plan: quantised q/k/v projections, attention prep with the quantise-on-append, decode attention over the 8-bit
cache, quantised o projection.  Replayed for a run of tokens from an empty cache and compared with the
oracle's layer on the dequantised weights."""
import numpy as np
import pytest

import saetta_macqwen_b200 as sa
from test_qmv import bf16_bits, dense, pack
from util import DIM, HEADS, KV, dev

pytestmark = pytest.mark.gpu
HIDDEN, BITS = 1024, 5


def mlx_matrix(rng, rows, cols, gain):
    q = rng.integers(0, 1 << BITS, (rows, cols), dtype=np.uint32)
    n = rows * cols // 64
    scales = bf16_bits((rng.uniform(0.5, 1.5, n) * gain / 16.0).astype(np.float32))
    biases = bf16_bits((-rng.uniform(0.9, 1.1, n) * gain).astype(np.float32))  # about -15.5 * scale: zero-mean weights
    return q, pack(q, BITS), scales, biases


def test_layer_replayed_over_six_tokens(oracle):
    import torch

    rng = np.random.default_rng(11)
    hd, kd = HEADS * DIM, KV * DIM
    mats = {"q_proj": mlx_matrix(rng, 2 * hd, HIDDEN, 0.06), "k_proj": mlx_matrix(rng, kd, HIDDEN, 0.06),
            "v_proj": mlx_matrix(rng, kd, HIDDEN, 0.06), "o_proj": mlx_matrix(rng, HIDDEN, hd, 0.03)}
    q_norm = (1.0 + 0.1 * rng.standard_normal(DIM)).astype(np.float32)
    k_norm = (1.0 + 0.1 * rng.standard_normal(DIM)).astype(np.float32)
    weights = {name: dense(m[0], m[2], m[3]).ravel() for name, m in mats.items()}
    weights.update(q_norm=q_norm, k_norm=k_norm)
    cfg = dict(hidden=HIDDEN, heads=HEADS, kv_heads=KV, head_dim=DIM, rope_dims=64, rope_theta=1.0e7, eps=1.0e-6)
    layer = oracle.Layer(cfg, weights, capacity=64, rounding=8)

    gpu = {name: tuple(dev(a.view(np.int32) if a.dtype == np.uint32 else a.view(np.int16)) for a in m[1:]) for name, m in mats.items()}
    cache = sa.GpuKvCache(0, 8, 128)
    op = sa.AttentionRows(0, HEADS, KV, 128, 1)
    x = torch.zeros(HIDDEN, device="cuda")
    qg, k, v = torch.zeros(2 * hd, device="cuda"), torch.zeros(kd, device="cuda"), torch.zeros(kd, device="cuda")
    q, attn, y = torch.zeros(hd, device="cuda"), torch.zeros(hd, device="cuda"), torch.zeros(HIDDEN, device="cuda")
    prep = sa.PrepParams(HEADS, KV, DIM, 64, 1.0e7, 1.0e-6)
    qn, kn = dev(q_norm), dev(k_norm)  # nothing may allocate while the plan records
    plan = sa.Plan(0)
    with plan.recording():
        st = plan.stream
        sa.qmv_rows(0, *gpu["q_proj"], BITS, 2 * hd, HIDDEN, 1, x, qg, stream=st)
        side = plan.parallel_begin()  # k and v projections do not depend on the q projection
        sa.qmv_rows(0, *gpu["k_proj"], BITS, kd, HIDDEN, 1, x, k, stream=side)
        sa.qmv_rows(0, *gpu["v_proj"], BITS, kd, HIDDEN, 1, x, v, stream=side)
        plan.parallel_end()
        sa.attention_prep(prep, 1, qg, k, v, qn, kn, q, sa.F32, cache, params=plan.params, stream=st)
        op.record_cache(1, q, cache, qg, attn, plan.params, stream=st)
        sa.qmv_rows(0, *gpu["o_proj"], BITS, HIDDEN, hd, 1, attn, y, stream=st)
    assert len(plan) == 6  # three projections, prep, attention (one launch), o projection

    worst = 0.0
    for pos in range(6):
        xt = rng.standard_normal(HIDDEN).astype(np.float32)
        x.copy_(dev(xt))
        torch.cuda.synchronize()
        plan.set_params(pos, pos)
        plan.run()
        got = y.cpu().numpy()
        want = layer.step(xt, pos)
        assert np.isfinite(got).all()
        scale = float(np.abs(want).max())
        worst = max(worst, float(np.abs(got - want).max()) / scale)
    assert op.device_status() == 0
    # the keys are quantised on both sides from values that differ in the last bits: a code may flip
    assert worst < 5e-3, worst
