"""saetta attention path for B200: ctypes binding of libsaetta_b200.so.

The product is the shared library (CUDA C++ behind the C ABI of
include/saetta_b200.h).  This module only loads it and mirrors, name for name,
the reference's Rust operator structs so tests and benchmarks read like the
reference's own (paths inside the reference project):

    QuantRows         src/kv_quant.rs:158-283
    GpuKvCache        src/gpu_layers.rs:179-293
    RowBackup         src/gpu_cache.rs:192-286
    DecodeAttention   src/attention.rs:19-171
    AttentionRows     src/rows.rs:307-494
    AttGemm           src/attention_gemm.rs:93-363
    TokenParams       src/plan.rs:17-35
    FlashParams       src/attention_prefill.rs:5-14

There is no CPU or PyTorch fallback: without the built library every call
raises.  Device memory is whatever the caller hands in as raw device pointers
(ints) or objects with ``data_ptr()`` (torch tensors).
"""
import ctypes as C
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libsaetta_b200.so")

F16, BF16, F32 = 0, 1, -1
KV_ALIGN = 128
MAX_ROWS = 8
PART_STRIDE = 264
OK, BAD_ARG, BAD_SHAPE, NO_MEM, CUDA, TIMEOUT, UNSUPPORTED = range(7)


class SaettaError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"saetta status {code}: {message}")
        self.code = code


class TokenParams(C.Structure):
    """src/plan.rs:17-35."""
    _fields_ = [("token", C.c_uint32), ("position", C.c_uint32), ("kv_len", C.c_uint32), ("pad", C.c_uint32)]

    @classmethod
    def new(cls, token, position):
        return cls(token, position, position + 1, 0)


class FlashParams(C.Structure):
    """src/attention_prefill.rs:5-14."""
    _fields_ = [("heads", C.c_uint32), ("kv_heads", C.c_uint32), ("pos", C.c_uint32), ("tokens", C.c_uint32),
                ("scale", C.c_float)]


class PrepParams(C.Structure):
    """kernels/layers.metal:637-644 `PrepParams` (theta instead of its log2, rope_dims instead of half)."""
    _fields_ = [("heads", C.c_uint32), ("kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("rope_dims", C.c_uint32),
                ("rope_theta", C.c_float), ("eps", C.c_float)]


def build(verbose=False):
    """Compiles the library in-tree with nvcc for sm_100a (make in csrc/)."""
    cmd = ["make", "-C", os.path.join(_HERE, "csrc"), "-j8"]
    subprocess.check_call(cmd, stdout=None if verbose else subprocess.DEVNULL)
    return LIB_PATH


_lib = None

# name -> (restype, argtypes); every symbol include/saetta_b200.h declares.
_P, _Z, _I, _U32, _U64 = C.c_void_p, C.c_size_t, C.c_int, C.c_uint32, C.c_uint64
_PP = C.POINTER(C.c_void_p)
SYMBOLS = {
    "saetta_last_error": (C.c_char_p, []),
    "saetta_version": (C.c_char_p, []),
    "saetta_quant_rows_create": (_I, [_I, _I, _Z, _Z, _PP]),
    "saetta_quant_rows_wrap": (_I, [_I, _I, _Z, _Z, _P, _P, _P, _PP]),
    "saetta_quant_rows_destroy": (None, [_P]),
    "saetta_quant_rows_buffers": (_I, [_P, _PP, _PP, _PP]),
    "saetta_quant_rows_record_at": (_I, [_P, _P, _P, _P]),
    "saetta_quant_rows_encode": (_I, [_P, _P, _Z, _Z, _P]),
    "saetta_quant_rows_encode_dequantize": (_I, [_P, _P, _I, _Z, _P]),
    "saetta_quantize_host": (_I, [_P, _Z, _I, _P, _P, _P]),
    "saetta_dequantize_host": (_I, [_P, _P, _P, _Z, _I, _P]),
    "saetta_kv_cache_create": (_I, [_I, _I, _Z, _Z, _Z, _Z, _PP]),
    "saetta_kv_cache_destroy": (None, [_P]),
    "saetta_kv_cache_capacity": (_Z, [_P]),
    "saetta_kv_cache_bits": (_I, [_P]),
    "saetta_kv_cache_buffers": (_I, [_P, _PP, C.POINTER(_Z), C.POINTER(_I)]),
    "saetta_kv_cache_quant": (_I, [_P, _PP, _PP]),
    "saetta_kv_cache_resize": (_I, [_P, _Z, _P]),
    "saetta_kv_cache_store": (_I, [_P, _P, _P, _P, _Z, _P]),
    "saetta_kv_cache_store_at": (_I, [_P, _P, _P, _Z, _Z, _P]),
    "saetta_kv_cache_set_dtype": (_I, [_P, _I]),
    "saetta_qmv_rows": (_I, [_I, _P, _P, _P, _I, _Z, _Z, _Z, _P, _P, _Z, _P]),
    "saetta_plan_create": (_I, [_I, _PP]),
    "saetta_plan_destroy": (None, [_P]),
    "saetta_plan_params": (_P, [_P]),
    "saetta_plan_stream": (_P, [_P]),
    "saetta_plan_begin": (_I, [_P]),
    "saetta_plan_parallel_begin": (_I, [_P, _PP]),
    "saetta_plan_parallel_end": (_I, [_P]),
    "saetta_plan_build": (_I, [_P]),
    "saetta_plan_len": (_I, [_P, C.POINTER(_Z)]),
    "saetta_plan_set_params": (_I, [_P, _U32, _U32]),
    "saetta_plan_commit": (_I, [_P]),
    "saetta_plan_wait": (_I, [_P]),
    "saetta_plan_run": (_I, [_P]),
    "saetta_plan_run_timed": (_I, [_P, C.POINTER(C.c_float)]),
    "saetta_plan_kernels": (_I, [_P, C.POINTER(C.c_char_p), C.POINTER(_Z), _Z, C.POINTER(_Z)]),
    "saetta_plan_build_where": (_I, [_P, C.POINTER(C.c_char_p), _Z, _I, _PP]),
    "saetta_built_destroy": (None, [_P]),
    "saetta_built_len": (_I, [_P, C.POINTER(_Z)]),
    "saetta_built_run_timed": (_I, [_P, C.POINTER(C.c_float)]),
    "saetta_attention_prep": (_I, [PrepParams, _Z, _P, _P, _P, _P, _P, _P, _I, _P, _P, _Z, _P, _P]),
    "saetta_row_backup_create": (_I, [_PP]),
    "saetta_row_backup_destroy": (None, [_P]),
    "saetta_row_backup_save": (_I, [_P, _PP, _Z, _Z, _Z, _P]),
    "saetta_row_backup_restore": (_I, [_P, _PP, _Z, _P]),
    "saetta_row_backup_clear": (None, [_P]),
    "saetta_row_backup_bytes": (_U64, [_P]),
    "saetta_decode_create": (_I, [_I, _Z, _Z, _Z, _Z, _Z, _PP]),
    "saetta_decode_destroy": (None, [_P]),
    "saetta_decode_record": (_I, [_P, _Z, _P, _P, _P, _I, _P, _P, _P, _P]),
    "saetta_decode_record_quant": (_I, [_P, _Z, _P, _P, _P, _P, _P, _P, _P]),
    "saetta_decode_record_cache": (_I, [_P, _Z, _P, _P, _P, _P, _P, _P]),
    "saetta_decode_record_quant_static": (_I, [_I, _Z, _P, _P, _P, _P, _P, _P, _P]),
    "saetta_decode_static_status": (_I, [_I, _P, C.POINTER(_U32), _I]),
    "saetta_decode_splits": (_I, [_P]),
    "saetta_decode_device_status": (_I, [_P, _P, C.POINTER(_U32)]),
    "saetta_decode_batch_create": (_I, [_I, _Z, _Z, _Z, _Z, _Z, _PP]),
    "saetta_decode_batch_destroy": (None, [_P]),
    "saetta_decode_batch_record": (_I, [_P, _Z, _PP, C.POINTER(_U32), _P, _P, _P, _P]),
    "saetta_decode_partial_cache": (_I, [_P, _Z, _P, _P, _P, _U32, _P, _P]),
    "saetta_merge_partials": (_I, [_I, _P, _Z, _Z, _Z, _P, _P, _P]),
    "saetta_peer_group_create": (_I, [_I, _I, _I, _Z, _Z, _P, _PP]),
    "saetta_peer_group_connect": (_I, [_P, _P]),
    "saetta_peer_group_destroy": (None, [_P]),
    "saetta_peer_group_staging": (_P, [_P]),
    "saetta_peer_merge": (_I, [_P, _Z, _P, _P, _P]),
    "saetta_peer_collect": (_I, [_P, _Z, _P, _P, _P]),
    "saetta_peer_merge_sliced": (_I, [_P, _Z, _P, _P, _P]),
    "saetta_peer_slice": (_I, [_P, _Z, C.POINTER(_Z), C.POINTER(_Z)]),
    "saetta_decode_batch_publish": (_I, [_P, _Z, _P, _P, _P, _P, _P]),
    "saetta_decode_publish_cache": (_I, [_P, _Z, _P, _P, _P, _U32, _P, _P]),
    "saetta_decode_exchange_cache": (_I, [_P, _Z, _P, _P, _P, _U32, _P, _P, _P, _P]),
    "saetta_peer_group_status": (_I, [_P, _P, C.POINTER(_U32)]),
    "saetta_peer_group_reset": (_I, [_P, C.c_uint32, _P]),
    "saetta_att_gemm_create": (_I, [_I, _Z, _Z, _PP]),
    "saetta_att_gemm_destroy": (None, [_P]),
    "saetta_att_gemm_reserve": (_I, [_P, _Z]),
    "saetta_att_gemm_invalidate": (_I, [_P]),
    "saetta_att_gemm_stage_quantised": (_I, [_P, _I]),
    "saetta_att_gemm_score_blocks": (_I, [_P, _I]),
    "saetta_att_gemm_partial_shard": (_I, [_P, _P, _I, _P, _P, _P, _P, _P, FlashParams, _Z, _Z, _Z, _P]),
    "saetta_att_gemm_encode": (_I, [_P, _P, _I, _P, _P, _P, _P, _P, _P, FlashParams, _P]),
    "saetta_att_gemm_partial": (_I, [_P, _P, _I, _P, _P, _P, _P, _P, FlashParams, _Z, _Z, _P]),
    "saetta_prefill_encode": (_I, [_I, _P, _I, _P, _P, _P, _P, FlashParams, _P]),
    "saetta_prefill_rows_cache": (_I, [_P, _P, _P, _P, _P, FlashParams, _P, _P]),
}


def lib():
    """The loaded library; raises if it has not been built (no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise SaettaError(CUDA, f"{LIB_PATH} is missing: build it with saetta_macqwen_b200.build() "
                                    "(nvcc, sm_100a); there is no CPU fallback")
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            f = getattr(l, name)
            f.restype, f.argtypes = res, args
        _lib = l
    return _lib


def _check(rc):
    if rc:
        raise SaettaError(rc, lib().saetta_last_error().decode())


def ptr(x):
    """Device (or host) address of a torch tensor, numpy array, ctypes object or int."""
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    if hasattr(x, "ctypes"):
        return x.ctypes.data
    return C.addressof(x)


def _stream(stream):
    if stream is None:
        import torch
        return torch.cuda.current_stream().cuda_stream
    return getattr(stream, "cuda_stream", stream)


class QuantRows:
    """src/kv_quant.rs:158-283."""

    def __init__(self, device, bits, values, capacity, _handle=None, _borrowed=False):
        self.bits, self.per_token, self.capacity = bits, values // 64, capacity
        self._borrowed = _borrowed
        if _handle is None:
            h = C.c_void_p()
            _check(lib().saetta_quant_rows_create(device, bits, values, capacity, C.byref(h)))
            _handle = h
        self.h = _handle

    @classmethod
    def wrap(cls, device, bits, values, capacity, data, scales, biases):
        h = C.c_void_p()
        _check(lib().saetta_quant_rows_wrap(device, bits, values, capacity, ptr(data), ptr(scales), ptr(biases),
                                            C.byref(h)))
        r = cls(device, bits, values, capacity, _handle=h)
        r._keep = (data, scales, biases)
        return r

    def buffers(self):
        d, s, z = C.c_void_p(), C.c_void_p(), C.c_void_p()
        _check(lib().saetta_quant_rows_buffers(self.h, C.byref(d), C.byref(s), C.byref(z)))
        return d.value, s.value, z.value

    def record_at(self, x, params, stream=None):
        """record / record_at: one row at params.position (params on the device)."""
        _check(lib().saetta_quant_rows_record_at(self.h, ptr(x), ptr(params), _stream(stream)))

    record = record_at

    def encode(self, x, pos, tokens, stream=None):
        _check(lib().saetta_quant_rows_encode(self.h, ptr(x), pos, tokens, _stream(stream)))

    def encode_dequantize(self, out, tokens, dtype=F16, stream=None):
        _check(lib().saetta_quant_rows_encode_dequantize(self.h, ptr(out), dtype, tokens, _stream(stream)))

    def __del__(self):
        if getattr(self, "h", None) and not self._borrowed and _lib is not None:
            _lib.saetta_quant_rows_destroy(self.h)
            self.h = None


class GpuKvCache:
    """src/gpu_layers.rs:179-293; bits 16/8/4 (and 32 for the f32 configuration)."""

    def __init__(self, device, bits, capacity, heads=16, kv_heads=2, head_dim=256, dtype=F16):
        h = C.c_void_p()
        _check(lib().saetta_kv_cache_create(device, bits, heads, kv_heads, head_dim, capacity, C.byref(h)))
        self.h, self.bits, self.device = h, bits, device
        self.heads, self.kv_heads, self.head_dim = heads, kv_heads, head_dim
        if bits == 16:
            _check(lib().saetta_kv_cache_set_dtype(h, dtype))

    @classmethod
    def with_bits(cls, device, capacity, bits, **kw):
        return cls(device, bits, capacity, **kw)

    @property
    def capacity(self):
        return lib().saetta_kv_cache_capacity(self.h)

    def buffers(self):
        """[(device pointer, row bytes)] in the order of GpuKvCache::buffers."""
        b, rb, n = (C.c_void_p * 6)(), (C.c_size_t * 6)(), C.c_int()
        _check(lib().saetta_kv_cache_buffers(self.h, b, rb, C.byref(n)))
        return [(b[i], rb[i]) for i in range(n.value)]

    def quant(self):
        k, v = C.c_void_p(), C.c_void_p()
        _check(lib().saetta_kv_cache_quant(self.h, C.byref(k), C.byref(v)))
        if not k.value:
            return None
        values = self.kv_heads * self.head_dim
        return (QuantRows(self.device, self.bits, values, self.capacity, _handle=k, _borrowed=True),
                QuantRows(self.device, self.bits, values, self.capacity, _handle=v, _borrowed=True))

    def resize(self, capacity, stream=None):
        _check(lib().saetta_kv_cache_resize(self.h, capacity, _stream(stream)))

    def store(self, k, v, params, rows=1, stream=None):
        """The decode/verify store site: rows at params.position + r."""
        _check(lib().saetta_kv_cache_store(self.h, ptr(k), ptr(v), ptr(params), rows, _stream(stream)))

    def store_at(self, k, v, pos, tokens, stream=None):
        """The prefill store site: tokens rows at pos."""
        _check(lib().saetta_kv_cache_store_at(self.h, ptr(k), ptr(v), pos, tokens, _stream(stream)))

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.saetta_kv_cache_destroy(self.h)
            self.h = None


class RowBackup:
    """src/gpu_cache.rs:192-286."""

    def __init__(self):
        h = C.c_void_p()
        _check(lib().saetta_row_backup_create(C.byref(h)))
        self.h = h

    @staticmethod
    def _arr(caches):
        return (C.c_void_p * len(caches))(*[c.h for c in caches])

    def save(self, caches, start, n, stream=None):
        _check(lib().saetta_row_backup_save(self.h, self._arr(caches), len(caches), start, n, _stream(stream)))

    def restore(self, caches, stream=None):
        _check(lib().saetta_row_backup_restore(self.h, self._arr(caches), len(caches), _stream(stream)))

    def clear(self):
        lib().saetta_row_backup_clear(self.h)

    def bytes(self):
        return lib().saetta_row_backup_bytes(self.h)

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.saetta_row_backup_destroy(self.h)
            self.h = None


class AttentionRows:
    """src/rows.rs:307-494; with rows == 1 it is src/attention.rs:19-171 DecodeAttention."""

    def __init__(self, device, heads, kv_heads, capacity, rows, head_dim=256):
        h = C.c_void_p()
        _check(lib().saetta_decode_create(device, heads, kv_heads, head_dim, capacity, rows, C.byref(h)))
        self.h, self.rows = h, rows

    @property
    def splits(self):
        return lib().saetta_decode_splits(self.h)

    def record(self, m, q, keys, values, q_and_gate, out, params, dtype=F16, stream=None):
        _check(lib().saetta_decode_record(self.h, m, ptr(q), ptr(keys), ptr(values), dtype, ptr(q_and_gate),
                                          ptr(out), ptr(params), _stream(stream)))

    def record_quant(self, m, q, keys, values, q_and_gate, out, params, stream=None):
        _check(lib().saetta_decode_record_quant(self.h, m, ptr(q), keys.h, values.h, ptr(q_and_gate), ptr(out),
                                                ptr(params), _stream(stream)))

    def record_cache(self, m, q, cache, q_and_gate, out, params, stream=None):
        _check(lib().saetta_decode_record_cache(self.h, m, ptr(q), cache.h, ptr(q_and_gate), ptr(out), ptr(params),
                                                _stream(stream)))

    def prefill_rows(self, q, cache, q_and_gate, out, p, params_scratch, stream=None):
        """The prefill's row route (exact mode): the chunk in groups of up to `rows` rows through this op."""
        _check(lib().saetta_prefill_rows_cache(self.h, ptr(q), cache.h, ptr(q_and_gate), ptr(out), p, ptr(params_scratch),
                                               _stream(stream)))

    def partial_cache(self, m, q, cache, part, params, row_step=1, stream=None):
        _check(lib().saetta_decode_partial_cache(self.h, m, ptr(q), cache.h, ptr(part), row_step, ptr(params),
                                                 _stream(stream)))

    def publish_cache(self, m, q, cache, group, params, row_step=1, stream=None):
        """partial_cache with the partial stored straight into every peer's mailbox."""
        _check(lib().saetta_decode_publish_cache(self.h, m, ptr(q), cache.h, group.h, row_step, ptr(params),
                                                 _stream(stream)))

    def exchange_cache(self, m, q, cache, group, q_and_gate, out, params, row_step=1, stream=None):
        """publish_cache and the group's collect in one launch: the gated result over every rank's shard."""
        _check(lib().saetta_decode_exchange_cache(self.h, m, ptr(q), cache.h, group.h, row_step, ptr(q_and_gate), ptr(out),
                                                  ptr(params), _stream(stream)))

    def device_status(self, stream=None):
        s = C.c_uint32()
        _check(lib().saetta_decode_device_status(self.h, _stream(stream), C.byref(s)))
        return s.value

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.saetta_decode_destroy(self.h)
            self.h = None


class DecodeAttention(AttentionRows):
    """src/attention.rs:19-171."""

    def __init__(self, device, heads, kv_heads, head_dim, capacity):
        super().__init__(device, heads, kv_heads, capacity, 1, head_dim=head_dim)

    def record(self, q, keys, values, q_and_gate, out, params, dtype=F16, stream=None):
        super().record(1, q, keys, values, q_and_gate, out, params, dtype=dtype, stream=stream)

    def record_quant(self, q, keys, values, q_and_gate, out, params, stream=None):
        super().record_quant(1, q, keys, values, q_and_gate, out, params, stream=stream)


def decode_record_quant_static(device, m, q, keys, values, q_and_gate, out, params, stream=None):
    """Decode / 2-row verify over a quantised cache without any allocation: the
    split-KV scratch is a fixed array inside the library (see the header).  For
    callers that may not call cudaMalloc; m <= 2."""
    _check(lib().saetta_decode_record_quant_static(device, m, ptr(q), keys.h, values.h, ptr(q_and_gate), ptr(out),
                                                   ptr(params), _stream(stream)))


def decode_static_status(device, stream=None, clear=False):
    """The status word of the allocation-free entry point on `device` (0: no bounded wait ever gave up)."""
    s = C.c_uint32()
    _check(lib().saetta_decode_static_status(device, _stream(stream), C.byref(s), 1 if clear else 0))
    return s.value


class DecodeBatch:
    """One decode row for each of many sequences with ragged lengths (no reference counterpart)."""

    def __init__(self, device, max_seqs, heads=16, kv_heads=2, head_dim=256):
        h = C.c_void_p()
        _check(lib().saetta_decode_batch_create(device, heads, kv_heads, head_dim, max_seqs, 0, C.byref(h)))
        self.h = h

    def record(self, caches, kv_lens, q, q_and_gate, out, stream=None):
        n = len(caches)
        arr = (C.c_void_p * n)(*[c.h for c in caches])
        lens = (C.c_uint32 * n)(*[int(x) for x in kv_lens])
        _check(lib().saetta_decode_batch_record(self.h, n, arr, lens, ptr(q), ptr(q_and_gate), ptr(out),
                                                _stream(stream)))

    def publish(self, caches, kv_lens, q, group, stream=None):
        """record() on this rank's shard of every sequence, the partials stored into the peers' mailboxes."""
        n = len(caches)
        arr = (C.c_void_p * n)(*[c.h for c in caches])
        lens = (C.c_uint32 * n)(*[int(x) for x in kv_lens])
        _check(lib().saetta_decode_batch_publish(self.h, n, arr, lens, ptr(q), group.h, _stream(stream)))

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.saetta_decode_batch_destroy(self.h)
            self.h = None


def attention_prep(p, rows, q_and_gate, k, v, q_norm, k_norm, q_out, q_dtype, cache, params=None, pos=0, k_out=None,
                   stream=None):
    """GpuAttention::record_store / the prep loop of record_rows / the prefill's norm + rope + store
    (src/gpu_layers.rs:373-411, 483-507, src/prefill.rs:1607-1666): q normed and roped into q_out,
    k normed and roped and v as it is into the cache slots of `rows` tokens, at params.position + r
    (device-side) or at pos + r."""
    _check(lib().saetta_attention_prep(p, rows, ptr(q_and_gate), ptr(k), ptr(v), ptr(q_norm), ptr(k_norm), ptr(q_out),
                                       q_dtype, cache.h, ptr(params) if params is not None else None, pos,
                                       ptr(k_out) if k_out is not None else None, _stream(stream)))


def qmv_rows(device, words, scales, biases, bits, rows, cols, m, x, y, y_stride=None, stream=None):
    """GpuQuant::record / rows::record_proj (src/qmv.rs:27-170, src/rows.rs:47-110): y[m][rows] = x[m][cols] W^T
    for an MLX affine matrix W (u32 words, bfloat16 scales and biases per 64 values)."""
    _check(lib().saetta_qmv_rows(device, ptr(words), ptr(scales), ptr(biases), bits, rows, cols, m, ptr(x), ptr(y),
                                 rows if y_stride is None else y_stride, _stream(stream)))


def merge_partials(device, parts, ranks, rows, heads, q_and_gate, out, stream=None):
    """LSE merge of [ranks][rows][heads][PART_STRIDE] partials, then the gate."""
    _check(lib().saetta_merge_partials(device, ptr(parts), ranks, rows, heads, ptr(q_and_gate), ptr(out),
                                       _stream(stream)))


class PeerGroup:
    """Split-KV merge across the GPUs of one box: partials are stored into the peers'
    mailboxes over NVLink and merged from local memory (no counterpart in the
    reference).  `all_gather_bytes(bytes) -> [bytes]` is any host-side all-gather
    in rank order (torch.distributed works)."""

    def __init__(self, device, rank, world, rows_max, heads, all_gather_bytes):
        h = C.c_void_p()
        handle = (C.c_uint8 * 64)()
        _check(lib().saetta_peer_group_create(device, rank, world, rows_max, heads, handle, C.byref(h)))
        self.h = h
        handles = b"".join(all_gather_bytes(bytes(handle)))
        assert len(handles) == 64 * world
        _check(lib().saetta_peer_group_connect(h, handles))

    @property
    def staging(self):
        """Device address the partial entry points write this rank's (m, l, O) to."""
        return lib().saetta_peer_group_staging(self.h)

    def merge(self, rows, q_and_gate, out, stream=None):
        """Publishes the partial in `staging`, then collects."""
        _check(lib().saetta_peer_merge(self.h, rows, ptr(q_and_gate), ptr(out), _stream(stream)))

    def merge_sliced(self, rows, q_and_gate, out, stream=None):
        """Publishes to every rank its slice of the rows of the partial in `staging`, then finalises this rank's slice."""
        _check(lib().saetta_peer_merge_sliced(self.h, rows, ptr(q_and_gate), ptr(out), _stream(stream)))

    def slice(self, rows):
        """The rows this rank finalises in merge_sliced: (lo, hi)."""
        lo, hi = C.c_size_t(), C.c_size_t()
        _check(lib().saetta_peer_slice(self.h, rows, C.byref(lo), C.byref(hi)))
        return lo.value, hi.value

    def collect(self, rows, q_and_gate, out, stream=None):
        """Waits for every rank's published partial, merges and gates."""
        _check(lib().saetta_peer_collect(self.h, rows, ptr(q_and_gate), ptr(out), _stream(stream)))

    def status(self, stream=None):
        s = C.c_uint32()
        _check(lib().saetta_peer_group_status(self.h, _stream(stream), C.byref(s)))
        return s.value

    def reset(self, seq=0, stream=None):
        """After a collect that gave up: on every rank, the same `seq`, between two host barriers."""
        _check(lib().saetta_peer_group_reset(self.h, seq, _stream(stream)))

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.saetta_peer_group_destroy(self.h)
            self.h = None


class Plan:
    """src/plan.rs:52-260 `Plan` + `Built`: record once (stream capture), replay per token (graph launch).

        plan = Plan(0)
        with plan.recording():
            sa.attention_prep(..., params=plan.params, stream=plan.stream)
            op.record_cache(1, q, cache, qg, out, plan.params, stream=plan.stream)
        plan.set_params(token, position); plan.run()
    """

    def __init__(self, device):
        h = C.c_void_p()
        _check(lib().saetta_plan_create(device, C.byref(h)))
        self.h = h

    @property
    def params(self):
        """Device address of the plan's TokenParams (an int: every entry point accepts it as params)."""
        return lib().saetta_plan_params(self.h)

    @property
    def stream(self):
        """The raw stream the ops are recorded on (an int: every entry point accepts it as stream)."""
        return lib().saetta_plan_stream(self.h)

    def begin(self):
        _check(lib().saetta_plan_begin(self.h))

    def build(self):
        _check(lib().saetta_plan_build(self.h))

    def recording(self):
        plan = self

        class _Rec:
            def __enter__(self):
                plan.begin()
                return plan

            def __exit__(self, et, ev, tb):
                if et is None:
                    plan.build()
                else:  # the recording failed: close the capture, keep the caller's exception
                    lib().saetta_plan_build(plan.h)
                return False

        return _Rec()

    def parallel_begin(self):
        s = C.c_void_p()
        _check(lib().saetta_plan_parallel_begin(self.h, C.byref(s)))
        return s.value

    def parallel_end(self):
        _check(lib().saetta_plan_parallel_end(self.h))

    def __len__(self):
        n = C.c_size_t()
        _check(lib().saetta_plan_len(self.h, C.byref(n)))
        return n.value

    def set_params(self, token, position):
        _check(lib().saetta_plan_set_params(self.h, token, position))

    def commit(self):
        _check(lib().saetta_plan_commit(self.h))

    def wait(self):
        _check(lib().saetta_plan_wait(self.h))

    def run(self):
        _check(lib().saetta_plan_run(self.h))

    def run_timed(self):
        ms = C.c_float()
        _check(lib().saetta_plan_run_timed(self.h, C.byref(ms)))
        return ms.value

    def kernels(self):
        """Plan::kernels: [(kernel name, ops)] in the order of each kernel's first op."""
        n = C.c_size_t()
        _check(lib().saetta_plan_kernels(self.h, None, None, 0, C.byref(n)))
        names, ops = (C.c_char_p * n.value)(), (C.c_size_t * n.value)()
        _check(lib().saetta_plan_kernels(self.h, names, ops, n.value, C.byref(n)))
        return [(names[i].decode(), ops[i]) for i in range(n.value)]

    def build_where(self, keep=None, barriers=True):
        """Plan::build_where: a Built of only the ops whose kernel name contains one of `keep` (None: all)."""
        keep = list(keep or [])
        arr = (C.c_char_p * max(len(keep), 1))(*[k.encode() for k in keep])
        h = C.c_void_p()
        _check(lib().saetta_plan_build_where(self.h, arr if keep else None, len(keep), 1 if barriers else 0, C.byref(h)))
        return Built(h, self)

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.saetta_plan_destroy(self.h)
            self.h = None


class Built:
    """src/plan.rs:229-260 `Built` as Plan::build_where returns it (a profiling replay)."""

    def __init__(self, h, plan):
        self.h, self._plan = h, plan  # it replays on the plan's stream and reads the plan's buffers

    def __len__(self):
        n = C.c_size_t()
        _check(lib().saetta_built_len(self.h, C.byref(n)))
        return n.value

    def run_timed(self):
        ms = C.c_float()
        _check(lib().saetta_built_run_timed(self.h, C.byref(ms)))
        return ms.value

    run = run_timed

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.saetta_built_destroy(self.h)
            self.h = None


class AttGemm:
    """src/attention_gemm.rs:93-363."""

    def __init__(self, device, chunk, kv_heads):
        h = C.c_void_p()
        _check(lib().saetta_att_gemm_create(device, chunk, kv_heads, C.byref(h)))
        self.h = h

    def reserve(self, tokens):
        _check(lib().saetta_att_gemm_reserve(self.h, tokens))

    def encode(self, q, keys, values, quant, q_and_gate, out, p, dtype=BF16, stream=None):
        kq, vq = (quant[0].h, quant[1].h) if quant else (None, None)
        _check(lib().saetta_att_gemm_encode(self.h, ptr(q), dtype, ptr(keys), ptr(values), kq, vq, ptr(q_and_gate),
                                            ptr(out), p, _stream(stream)))

    def partial(self, q, keys, values, quant, part, p, key_lo, key_hi, dtype=BF16, stream=None, key_base=None):
        """Keys [key_lo, key_hi) only, the result left as (O, m, l) partials.  With key_base the cache handed
        in holds only this shard's slice of the sequence: its row 0 is the key at global position key_base."""
        kq, vq = (quant[0].h, quant[1].h) if quant else (None, None)
        if key_base is None:
            _check(lib().saetta_att_gemm_partial(self.h, ptr(q), dtype, ptr(keys), ptr(values), kq, vq, ptr(part), p,
                                                 key_lo, key_hi, _stream(stream)))
        else:
            _check(lib().saetta_att_gemm_partial_shard(self.h, ptr(q), dtype, ptr(keys), ptr(values), kq, vq, ptr(part), p,
                                                       key_base, key_lo, key_hi, _stream(stream)))

    def invalidate(self):
        _check(lib().saetta_att_gemm_invalidate(self.h))

    def score_blocks(self, keys):
        """16-bit caches: score blocks of 128 keys (default) or 64 (the older kernel)."""
        _check(lib().saetta_att_gemm_score_blocks(self.h, keys))

    def stage_quantised(self, on=True):
        """Read 8/4-bit caches through the op's 16-bit staging copy (kv_stage) instead of in place."""
        _check(lib().saetta_att_gemm_stage_quantised(self.h, int(bool(on))))

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.saetta_att_gemm_destroy(self.h)
            self.h = None


def prefill_encode(device, q, keys, values, q_and_gate, out, p, dtype=F16, stream=None):
    """src/attention_prefill.rs:39-72 `encode` (binary16 q and cache, as the reference's)."""
    _check(lib().saetta_prefill_encode(device, ptr(q), dtype, ptr(keys), ptr(values), ptr(q_and_gate), ptr(out), p,
                                       _stream(stream)))


def quantize_host(x, bits):
    """saetta_quantize_host on a numpy f32 array: (data, scales, biases)."""
    import numpy as np
    x = np.ascontiguousarray(x, np.float32).ravel()
    g = x.size // 64
    data, s, z = np.empty(g * 2 * bits, np.uint32), np.empty(g, np.uint16), np.empty(g, np.uint16)
    _check(lib().saetta_quantize_host(ptr(x), x.size, bits, ptr(data), ptr(s), ptr(z)))
    return data, s, z


def dequantize_host(data, scales, biases, bits):
    import numpy as np
    data = np.ascontiguousarray(data, np.uint32)
    s, z = np.ascontiguousarray(scales, np.uint16), np.ascontiguousarray(biases, np.uint16)
    out = np.empty(s.size * 64, np.float32)
    _check(lib().saetta_dequantize_host(ptr(data), ptr(s), ptr(z), s.size, bits, ptr(out)))
    return out
