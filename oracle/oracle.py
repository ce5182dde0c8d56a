"""ctypes front end of the CPU oracle in saetta_oracle.c.

TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and the CPU
baseline leg of the benchmark; the shipped library never touches it.  Each
function names the reference code it restates (paths inside the reference
project).
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libsaetta_oracle.so")
GROUP = 64  # src/kv_quant.rs:9


def build(force=False):
    """Compiles saetta_oracle.c next to this file (gcc, a second or two)."""
    src = os.path.join(_HERE, "saetta_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "libsaetta_oracle.so"])
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.so_dot.restype = C.c_float
        _lib.so_sigmoid.restype = C.c_float
        _lib.so_sigmoid.argtypes = [C.c_float]
    return _lib


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def quantize(x, bits):
    """src/kv_quant.rs:54-87: (data u32, scales f16 bits, biases f16 bits)."""
    x = _f32(x).ravel()
    groups = x.size // GROUP
    data = np.empty(groups * 2 * bits, np.uint32)
    s = np.empty(groups, np.uint16)
    z = np.empty(groups, np.uint16)
    rc = lib().so_quantize(_p(x), C.c_size_t(x.size), bits, _p(data), _p(s), _p(z))
    if rc:
        raise ValueError("quantize: bits must be 8 or 4 and the length a multiple of 64")
    return data, s, z


def dequantize(data, scales, biases, bits):
    """src/kv_quant.rs:90-105."""
    data = np.ascontiguousarray(data, np.uint32)
    s = np.ascontiguousarray(scales, np.uint16)
    z = np.ascontiguousarray(biases, np.uint16)
    out = np.empty(s.size * GROUP, np.float32)
    rc = lib().so_dequantize(_p(data), _p(s), _p(z), C.c_size_t(s.size), bits, _p(out))
    if rc:
        raise ValueError("dequantize: bits must be 8 or 4")
    return out


def round_trip(x, bits):
    """src/kv_quant.rs:129-135."""
    x = _f32(x)
    y = np.empty_like(x)
    if lib().so_round_trip(_p(x), C.c_size_t(x.size), bits, _p(y)):
        raise ValueError("round_trip: bad bits or length")
    return y


def round_trip_as_half(x, bits, bf16=False):
    """src/kv_quant.rs:121-126; bf16=True narrows to bfloat16 instead of binary16."""
    x = _f32(x)
    y = np.empty_like(x)
    if lib().so_round_trip_as_half(_p(x), C.c_size_t(x.size), bits, int(bf16), _p(y)):
        raise ValueError("round_trip_as_half: bad bits or length")
    return y


def round_f16(x):
    x = _f32(x)
    y = np.empty_like(x)
    lib().so_round_f16(_p(x), _p(y), C.c_size_t(x.size))
    return y


def round_bf16(x):
    x = _f32(x)
    y = np.empty_like(x)
    lib().so_round_bf16(_p(x), _p(y), C.c_size_t(x.size))
    return y


def to_f16_bits(x):
    x = _f32(x)
    y = np.empty(x.shape, np.uint16)
    lib().so_to_f16(_p(x), _p(y), C.c_size_t(x.size))
    return y


def to_bf16_bits(x):
    x = _f32(x)
    y = np.empty(x.shape, np.uint16)
    lib().so_to_bf16(_p(x), _p(y), C.c_size_t(x.size))
    return y


def from_f16_bits(h):
    h = np.ascontiguousarray(h, np.uint16)
    y = np.empty(h.shape, np.float32)
    lib().so_from_f16(_p(h), _p(y), C.c_size_t(h.size))
    return y


def from_bf16_bits(h):
    h = np.ascontiguousarray(h, np.uint16)
    y = np.empty(h.shape, np.float32)
    lib().so_from_bf16(_p(h), _p(y), C.c_size_t(h.size))
    return y


def dot(a, b):
    """src/cpu/ops.rs:13-15."""
    a, b = _f32(a), _f32(b)
    return float(lib().so_dot(_p(a), _p(b), C.c_size_t(a.size)))


def softmax(x):
    """src/cpu/ops.rs:51-59."""
    y = _f32(x).copy()
    lib().so_softmax(_p(y), C.c_size_t(y.size))
    return y


def sigmoid(x):
    """src/cpu/ops.rs:38-40."""
    return float(lib().so_sigmoid(float(x)))


def quant_matvec(words, scales, biases, bits, rows, cols, x):
    """src/cpu/matrix.rs:73-135: y = W x for an MLX affine matrix (u32 words, bfloat16 scale / bias bits per 64)."""
    words = np.ascontiguousarray(words, np.uint32)
    s, z = np.ascontiguousarray(scales, np.uint16), np.ascontiguousarray(biases, np.uint16)
    x = _f32(x)
    assert words.size == rows * cols * bits // 32 and s.size == rows * cols // 64 == z.size and x.size == cols
    y = np.empty(rows, np.float32)
    if lib().so_quant_matvec(_p(words), _p(s), _p(z), bits, C.c_size_t(rows), C.c_size_t(cols), _p(x), _p(y)):
        raise ValueError("quant_matvec: bits must be 4, 5, 6 or 8 and cols a multiple of 64")
    return y


def rms_norm(x, w, eps):
    """src/cpu/ops.rs:19-36."""
    y, w = _f32(x).copy(), _f32(w)
    lib().so_rms_norm(_p(y), _p(w), C.c_size_t(y.size), C.c_float(eps))
    return y


def rope(head, dims, pos, theta):
    """src/cpu/ops.rs:64-74 on one head."""
    y = _f32(head).copy()
    lib().so_rope(_p(y), C.c_size_t(dims), C.c_size_t(pos), C.c_float(theta))
    return y


def rope_rows(x, head_dim, dims, positions, theta):
    """rope on every head of x [tokens][heads*head_dim], token t at positions[t]."""
    y = _f32(x).copy().reshape(len(positions), -1, head_dim)
    for t, pos in enumerate(positions):
        for h in range(y.shape[1]):
            lib().so_rope(_p(y[t, h]), C.c_size_t(dims), C.c_size_t(int(pos)), C.c_float(theta))
    return y.reshape(np.shape(x))


def attention_rows(q, q_and_gate, keys, values, lens, heads=16, kv_heads=2, d=256, threads=1):
    """Inner attention for len(lens) rows: src/cpu/attention.rs:144-181.

    q [rows][heads][d], q_and_gate [rows][heads][2d] (gate in the second half of
    each head), keys/values [>=max(lens)][kv_heads][d] f32, row r sees lens[r] keys.
    """
    q, qg, k, v = _f32(q), _f32(q_and_gate), _f32(keys), _f32(values)
    lens = np.ascontiguousarray(lens, np.uint32)
    rows = lens.size
    assert q.size == rows * heads * d and qg.size == 2 * q.size
    assert k.size >= int(lens.max()) * kv_heads * d and v.size >= int(lens.max()) * kv_heads * d
    out = np.empty((rows, heads, d), np.float32)
    rc = lib().so_attention_rows(
        _p(q), _p(qg), _p(k), _p(v), _p(lens), C.c_size_t(rows), C.c_size_t(heads),
        C.c_size_t(kv_heads), C.c_size_t(d), int(threads), _p(out))
    if rc:
        raise ValueError("attention_rows: bad shape")
    return out


class Layer:
    """src/cpu/attention.rs:103-156 with its KvCache, for replaying attention.json."""

    def __init__(self, cfg, weights, capacity=64, rounding=0):
        self.cfg, self.w, self.rounding = cfg, {k: _f32(v) for k, v in weights.items()}, rounding
        kd = cfg["kv_heads"] * cfg["head_dim"]
        self.keys = np.zeros(capacity * kd, np.float32)
        self.values = np.zeros(capacity * kd, np.float32)
        self.len = C.c_size_t(0)

    def step(self, x, pos=None):
        c, w = self.cfg, self.w
        x = _f32(x)
        y = np.empty(c["hidden"], np.float32)
        pos = self.len.value if pos is None else pos
        rc = lib().so_attention_layer(
            C.c_size_t(c["hidden"]), C.c_size_t(c["heads"]), C.c_size_t(c["kv_heads"]),
            C.c_size_t(c["head_dim"]), C.c_size_t(c["rope_dims"]), C.c_float(c["rope_theta"]),
            C.c_float(c["eps"]), _p(w["q_proj"]), _p(w["k_proj"]), _p(w["v_proj"]),
            _p(w["o_proj"]), _p(w["q_norm"]), _p(w["k_norm"]), _p(x), C.c_size_t(pos),
            _p(self.keys), _p(self.values), C.byref(self.len), int(self.rounding), _p(y))
        if rc:
            raise ValueError("attention_layer: bad rounding")
        return y


def noise(n, seed):
    """tests/attention.rs:16-26 / src/kv_quant.rs:290-300."""
    x = np.empty(n, np.float32)
    lib().so_noise(_p(x), C.c_size_t(n), C.c_uint64(seed))
    return x


def spread(n, seed):
    """src/attention_prefill.rs:103-108, before the narrowing to half."""
    x = np.empty(n, np.float32)
    lib().so_spread(_p(x), C.c_size_t(n), C.c_size_t(seed))
    return x


def normal(n, seed):
    """Seeded N(0,1) (splitmix64 + Box-Muller); the benchmark configs' inputs."""
    x = np.empty(n, np.float32)
    lib().so_normal(_p(x), C.c_size_t(n), C.c_uint64(seed))
    return x
