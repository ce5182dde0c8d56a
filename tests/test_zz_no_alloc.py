"""The allocation-free decode entry point against the ordinary one.

saetta_decode_record_quant_static serves callers that must not allocate device
memory (a host with a fixed, pre-sized memory pool; a decode loop where
cudaMalloc's device-wide serialisation is unacceptable): its split-KV scratch is
a fixed array inside the library.  It must give exactly what
saetta_decode_record_quant gives, call after call, because both run the same
kernels with the same split count.  This file sorts last on purpose: a run that
stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest

import saetta_macqwen_b200 as sa
from util import DIM, HEADS, KV, ROW, dev, max_abs, params_dev, quant_rows_from_oracle, rel_rms

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits", [8, 4])
def test_static_scratch_matches_allocating_entry_point(oracle, bits):
    import torch

    capacity = 8192
    keys = oracle.normal(capacity * ROW, 41)
    values = oracle.normal(capacity * ROW, 42)
    kq = quant_rows_from_oracle(sa, oracle, keys.reshape(-1, ROW), bits, capacity)
    vq = quant_rows_from_oracle(sa, oracle, values.reshape(-1, ROW), bits, capacity)
    op = sa.AttentionRows(0, HEADS, KV, capacity, 2)
    for call, (m, pos) in enumerate([(1, 8000), (2, 5000), (1, 0), (2, 33)]):
        q = dev(oracle.normal(m * HEADS * DIM, 50 + call))
        qg = dev(oracle.normal(m * HEADS * 2 * DIM, 60 + call))
        want = torch.zeros(m * HEADS * DIM, device="cuda")
        got = torch.full((m * HEADS * DIM,), float("nan"), device="cuda")
        p = params_dev(pos)
        op.record_quant(m, q, kq, vq, qg, want, p)
        sa.decode_record_quant_static(0, m, q, kq, vq, qg, got, p)
        torch.cuda.synchronize()
        # same kernels, same split count, fixed merge order: equal to the last bit
        assert np.array_equal(got.cpu().numpy(), want.cpu().numpy()), (bits, call)
        # no bounded wait of the fixed-scratch path gave up (the word is shared by all calls on the device)
        assert sa.decode_static_status(0) == 0
        if call < 2:  # and pinned on the CPU oracle too, not only on the other GPU path
            kr, vr = oracle.round_trip(keys, bits), oracle.round_trip(values, bits)
            ref = oracle.attention_rows(q.cpu().numpy(), qg.cpu().numpy(), kr, vr, [pos + r + 1 for r in range(m)], threads=8)
            assert max_abs(got.cpu().numpy().reshape(m, HEADS, DIM), ref) < 2e-3
            assert rel_rms(got.cpu().numpy().reshape(m, HEADS, DIM), ref) < 1e-3
    # a size beyond the fixed scratch is refused, nothing is launched
    q3 = torch.zeros(3 * HEADS * DIM, device="cuda")
    with pytest.raises(sa.SaettaError) as e:
        sa.decode_record_quant_static(0, 3, q3, kq, vq, torch.zeros(3 * HEADS * 2 * DIM, device="cuda"), q3, params_dev(10))
    assert e.value.code == sa.BAD_SHAPE and "at most 2 query rows" in str(e.value)
    # rows that live on another device than the one named are refused before any launch
    with pytest.raises(sa.SaettaError) as e:
        sa.decode_record_quant_static(1, 1, q3, kq, vq, torch.zeros(HEADS * 2 * DIM, device="cuda"), q3, params_dev(10))
    assert e.value.code == sa.BAD_ARG
