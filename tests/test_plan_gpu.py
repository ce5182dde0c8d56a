"""Plan / Built (src/plan.rs:52-260) on CUDA graphs: a decode step -- attention prep with the
quantised store, then attention over the cache -- is recorded once and replayed for a run of
positions with nothing but TokenParams changing; every replay must equal the same calls issued
directly, bit for bit, and the cache must end up with the same rows."""
import numpy as np
import pytest

import saetta_macqwen_b200 as sa
from util import DIM, HEADS, KV, ROW, dev, params_dev, read_dev

pytestmark = pytest.mark.gpu
P = sa.PrepParams(HEADS, KV, DIM, 64, 1.0e7, 1.0e-6)


def test_recorded_decode_step_replays_for_every_position(oracle):
    import torch

    ctx, steps, bits = 1500, 4, 8
    cap = 2048
    keys, values = dev(oracle.normal(ctx * ROW, 1)), dev(oracle.normal(ctx * ROW, 2))
    qn, kn = dev(1.0 + 0.1 * oracle.normal(DIM, 3)), dev(1.0 + 0.1 * oracle.normal(DIM, 4))
    caches = [sa.GpuKvCache(0, bits, cap) for _ in range(2)]
    for c in caches:
        c.store_at(keys, values, 0, ctx)
    op = sa.AttentionRows(0, HEADS, KV, cap, 1)
    # per-step inputs live in fixed buffers the host refills, as the reference's layers do
    qg, k, v = (torch.zeros(n, device="cuda") for n in (HEADS * 2 * DIM, ROW, ROW))
    q, out = torch.zeros(HEADS * DIM, device="cuda"), torch.zeros(HEADS * DIM, device="cuda")

    plan = sa.Plan(0)
    with plan.recording():
        sa.attention_prep(P, 1, qg, k, v, qn, kn, q, sa.F32, caches[0], params=plan.params, stream=plan.stream)
        op.record_cache(1, q, caches[0], qg, out, plan.params, stream=plan.stream)
    assert len(plan) == 2  # prep, attention (split-KV CTAs and merge CTAs in one launch)

    for s in range(steps):
        pos = ctx + s
        qg.copy_(dev(oracle.normal(qg.numel(), 10 + s)))
        k.copy_(dev(oracle.normal(ROW, 20 + s)))
        v.copy_(dev(oracle.normal(ROW, 30 + s)))
        torch.cuda.synchronize()
        plan.set_params(7, pos)
        ms = plan.run_timed()
        assert 0.0 < ms < 50.0
        replayed = out.cpu().numpy().copy()
        # the same step issued directly, on the second cache
        p = params_dev(pos)
        sa.attention_prep(P, 1, qg, k, v, qn, kn, q, sa.F32, caches[1], params=p)
        op.record_cache(1, q, caches[1], qg, out, p)
        torch.cuda.synchronize()
        assert np.array_equal(replayed, out.cpu().numpy()), f"step {s}"
    for (pa, rb), (pb, _) in zip(caches[0].buffers(), caches[1].buffers()):
        assert np.array_equal(read_dev(pa + ctx * rb, steps * rb), read_dev(pb + ctx * rb, steps * rb))


def test_parallel_branch_and_misuse():
    import torch

    plan = sa.Plan(0)
    a, b = torch.zeros(1 << 16, device="cuda"), torch.zeros(1 << 16, device="cuda")
    with pytest.raises(sa.SaettaError):
        plan.run()  # not built
    with pytest.raises(sa.SaettaError):
        plan.parallel_begin()  # not recording
    plan.begin()
    main = torch.cuda.ExternalStream(plan.stream)
    side = torch.cuda.ExternalStream(plan.parallel_begin())
    with torch.cuda.stream(side):  # `op_parallel`: independent of what the main stream does meanwhile
        b.add_(2.0)
    with torch.cuda.stream(main):
        a.add_(1.0)
    plan.parallel_end()
    with torch.cuda.stream(main):
        a.add_(b)  # after the join: sees both
    plan.build()
    assert len(plan) == 3
    for _ in range(3):
        plan.run()
    torch.cuda.synchronize()
    # replay r: b = 2r, a_r = a_{r-1} + 1 + 2r  ->  after 3 replays a = 3 + 2*(1+2+3) = 15
    assert float(b[0]) == 6.0 and float(a[0]) == 15.0 and float(a[-1]) == 15.0


def test_build_where_replays_the_ops_of_chosen_kernels(oracle):
    """Plan::build_where (src/plan.rs:190-226) as src/profile.rs:39-121 uses it: the whole recording again,
    the ops of one kernel alone, and the recording without its barriers."""
    import torch

    ctx, bits, cap, layers = 900, 8, 1024, 3
    keys, values = dev(oracle.normal(ctx * ROW, 1)), dev(oracle.normal(ctx * ROW, 2))
    ones = torch.ones(DIM, device="cuda")
    caches = [sa.GpuKvCache(0, bits, cap) for _ in range(layers)]
    for c in caches:
        c.store_at(keys, values, 0, ctx)
    op = sa.AttentionRows(0, HEADS, KV, cap, 1)
    qg = dev(oracle.normal(HEADS * 2 * DIM, 5))
    k, v = dev(oracle.normal(ROW, 6)), dev(oracle.normal(ROW, 7))
    q = torch.zeros(layers, HEADS * DIM, device="cuda")
    out = torch.zeros(layers, HEADS * DIM, device="cuda")
    plan = sa.Plan(0)
    with plan.recording():
        for l, c in enumerate(caches):
            sa.attention_prep(P, 1, qg, k, v, ones, ones, q[l], sa.F32, c, params=plan.params, stream=plan.stream)
            op.record_cache(1, q[l], c, qg, out[l], plan.params, stream=plan.stream)
    kernels = plan.kernels()
    assert [n for _, n in kernels] == [layers, layers] and sum(n for _, n in kernels) == len(plan)
    assert "attention_prep" in kernels[0][0] and "decode_quant_kernel" in kernels[1][0]

    plan.set_params(3, ctx)
    plan.run()
    want = out.cpu().numpy().copy()

    whole = plan.build_where()  # keep = |_| true, with barriers: the plan itself again
    assert len(whole) == len(plan)
    out.zero_()
    assert whole.run_timed() > 0.0
    assert np.array_equal(out.cpu().numpy(), want)

    only = plan.build_where(["decode_quant_kernel"])  # the attention ops alone: q and the cache rows are still there
    assert len(only) == layers
    out.zero_()
    assert only.run_timed() > 0.0
    assert np.array_equal(out.cpu().numpy(), want)

    prep_only = plan.build_where(["attention_prep"])
    assert len(prep_only) == layers
    out.zero_()
    prep_only.run()
    assert not out.any()  # no attention op ran

    free = plan.build_where(barriers=False)  # a lower bound on the time; its results are not the plan's
    assert len(free) == len(plan) and free.run_timed() > 0.0
    assert len(plan.build_where(["no such kernel"])) == 0
