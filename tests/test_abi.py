"""Host-side checks that need no GPU: the library loads, exports every symbol
the header declares, rejects what the reference asserts on, and its host
quantiser is the oracle's bit for bit."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import saetta_macqwen_b200 as sa

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(sa.LIB_PATH):
        sa.build()
    return sa.lib()


def test_every_declared_symbol_is_exported(lib):
    header = open(os.path.join(ROOT, "include", "saetta_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(saetta_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 40
    raw = C.CDLL(sa.LIB_PATH)
    missing = [n for n in sorted(declared) if not hasattr(raw, n)]
    assert not missing, missing
    assert declared == set(sa.SYMBOLS), declared ^ set(sa.SYMBOLS)
    assert b"sm_100a" in lib.saetta_version()


def test_struct_layouts_match_the_reference():
    assert C.sizeof(sa.TokenParams) == 16  # src/plan.rs:17-35
    p = sa.TokenParams.new(7, 41)
    assert (p.token, p.position, p.kv_len, p.pad) == (7, 41, 42, 0)
    assert C.sizeof(sa.FlashParams) == 20  # src/attention_prefill.rs:5-14


def test_shape_errors_come_back_as_status_codes(lib):
    h = C.c_void_p()
    # what the reference asserts (src/kv_quant.rs:168, src/attention.rs:49-57, src/rows.rs:390)
    assert lib.saetta_quant_rows_create(0, 16, 512, 64, C.byref(h)) == sa.BAD_SHAPE
    assert b"8 or 4" in lib.saetta_last_error()
    assert lib.saetta_quant_rows_create(0, 8, 100, 64, C.byref(h)) == sa.BAD_SHAPE
    assert lib.saetta_decode_create(0, 16, 2, 128, 4096, 1, C.byref(h)) == sa.BAD_SHAPE
    assert b"head dim 256" in lib.saetta_last_error()
    assert lib.saetta_decode_create(0, 12, 2, 256, 4096, 1, C.byref(h)) == sa.BAD_SHAPE
    assert b"8 q heads per kv head" in lib.saetta_last_error()
    assert lib.saetta_decode_create(0, 16, 2, 256, 4096, 9, C.byref(h)) == sa.BAD_SHAPE
    assert lib.saetta_kv_cache_create(0, 5, 16, 2, 256, 128, C.byref(h)) == sa.BAD_SHAPE
    assert lib.saetta_quant_rows_create(0, 8, 512, 64, None) == sa.BAD_ARG
    with pytest.raises(sa.SaettaError):
        sa.QuantRows(0, 16, 512, 64)


def test_null_arguments_are_refused_before_any_device_work(lib):
    """Misuse of the entry points added around the attention kernels -- prep, plan, peer exchange --
    comes back as BAD_ARG with a message and never reaches the GPU (so this runs without one)."""
    z = C.c_size_t()
    f = C.c_float()
    p = sa.PrepParams(16, 2, 256, 64, 1.0e7, 1.0e-6)
    assert lib.saetta_attention_prep(p, 1, None, None, None, None, None, None, sa.F32, None, None, 0, None, None) == sa.BAD_ARG
    assert b"attention prep" in lib.saetta_last_error()
    for fn in (lib.saetta_plan_begin, lib.saetta_plan_build, lib.saetta_plan_commit, lib.saetta_plan_wait, lib.saetta_plan_run,
               lib.saetta_plan_parallel_end):
        assert fn(None) == sa.BAD_ARG
    assert lib.saetta_plan_create(0, None) == sa.BAD_ARG
    assert lib.saetta_plan_len(None, C.byref(z)) == sa.BAD_ARG
    assert lib.saetta_plan_set_params(None, 0, 0) == sa.BAD_ARG
    assert lib.saetta_plan_run_timed(None, C.byref(f)) == sa.BAD_ARG
    assert lib.saetta_plan_kernels(None, None, None, 0, C.byref(z)) == sa.BAD_ARG
    assert lib.saetta_plan_build_where(None, None, 0, 1, C.byref(C.c_void_p())) == sa.BAD_ARG
    assert lib.saetta_built_len(None, C.byref(z)) == sa.BAD_ARG and lib.saetta_built_run_timed(None, C.byref(f)) == sa.BAD_ARG
    lib.saetta_built_destroy(None)
    assert lib.saetta_plan_params(None) is None and lib.saetta_plan_stream(None) is None
    lib.saetta_plan_destroy(None)  # a no-op, as free(NULL)
    handle = (C.c_uint8 * 64)()
    assert lib.saetta_peer_group_create(0, 0, 9, 1, 16, handle, C.byref(C.c_void_p())) == sa.BAD_SHAPE  # 1..8 ranks
    assert lib.saetta_peer_group_create(0, 2, 2, 1, 16, handle, C.byref(C.c_void_p())) == sa.BAD_SHAPE  # rank < world
    for fn in (lib.saetta_peer_merge, lib.saetta_peer_collect, lib.saetta_peer_merge_sliced):
        assert fn(None, 1, None, None, None) == sa.BAD_ARG
    assert lib.saetta_peer_slice(None, 8, C.byref(z), C.byref(z)) == sa.BAD_ARG
    assert lib.saetta_peer_group_reset(None, 0, None) == sa.BAD_ARG
    assert lib.saetta_att_gemm_stage_quantised(None, 1) == sa.BAD_ARG
    assert lib.saetta_att_gemm_score_blocks(None, 64) == sa.BAD_ARG
    assert lib.saetta_decode_publish_cache(None, 1, None, None, None, 0, None, None) == sa.BAD_ARG
    assert lib.saetta_decode_exchange_cache(None, 1, None, None, None, 0, None, None, None, None) == sa.BAD_ARG
    assert lib.saetta_decode_batch_publish(None, 1, None, None, None, None, None) == sa.BAD_ARG
    # attention_prefill::encode without an object: nulls, then bfloat16 (binary16 only), both before any device work
    fp = sa.FlashParams(16, 2, 0, 8, 0.0625)
    assert lib.saetta_prefill_encode(0, None, sa.F16, None, None, None, None, fp, None) == sa.BAD_ARG
    fake = 4096  # a non-null, 16-byte aligned address that is never dereferenced
    assert lib.saetta_prefill_encode(0, fake, sa.BF16, fake, fake, fake, fake, fp, None) == sa.UNSUPPORTED
    assert b"binary16 only" in lib.saetta_last_error()
    assert lib.saetta_decode_static_status(0, None, None, 0) == sa.BAD_ARG
    assert lib.saetta_prefill_rows_cache(None, None, None, None, None, fp, None, None) == sa.BAD_ARG


def test_host_quantiser_is_the_oracle_bit_for_bit(lib, oracle):
    x = oracle.noise(37 * 512, 7).reshape(-1, 64)
    x *= np.where(np.arange(x.shape[0]) % 3 == 0, 20.0, 1.0)[:, None].astype(np.float32)
    x[1] = -1.5
    for bits in (8, 4):
        want = oracle.quantize(x.ravel(), bits)
        got = sa.quantize_host(x.ravel(), bits)
        for g, w in zip(got, want):
            assert np.array_equal(g, w)
        assert np.array_equal(sa.dequantize_host(*got, bits).view(np.uint32),
                              oracle.dequantize(*want, bits).view(np.uint32))
    known = np.zeros(64, np.float32)
    known[[1, 63]] = 1.0  # src/kv_quant.rs:319-332
    d8 = sa.quantize_host(known, 8)[0]
    d4 = sa.quantize_host(known, 4)[0]
    assert d8[0] == 255 << 8 and d8[15] == 255 << 24 and d4[0] == 15 << 4 and d4[7] == 15 << 28
