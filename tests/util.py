"""Helpers shared by the GPU parity tests: seeded inputs and error measures."""
import numpy as np

HEADS, KV, DIM = 16, 2, 256
ROW = KV * DIM  # values per token of one cache side


def rel_rms(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.sqrt(((got - want) ** 2).mean() / max((want ** 2).mean(), 1e-300)))


def max_abs(got, want):
    return float(np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64)).max())


def dev(x, dtype=None):
    import torch

    t = torch.from_numpy(np.ascontiguousarray(x))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def params_dev(position):
    """A saetta_token_params on the device: token 0 at `position`."""
    import torch

    return torch.tensor([0, position, position + 1, 0], dtype=torch.int32).cuda()


def quant_rows_from_oracle(sa, oracle, x, bits, capacity):
    """QuantRows over torch buffers holding the oracle's codes for x [tokens][512]."""
    import torch

    tokens = x.shape[0]
    data, s, z = oracle.quantize(x.ravel(), bits)
    words = 8 * 2 * bits
    d = torch.zeros(capacity * words, dtype=torch.int32, device="cuda")
    sc = torch.zeros(capacity * 8, dtype=torch.int16, device="cuda")
    bi = torch.zeros(capacity * 8, dtype=torch.int16, device="cuda")
    d[: tokens * words] = torch.from_numpy(data.view(np.int32)).cuda()
    sc[: tokens * 8] = torch.from_numpy(s.view(np.int16)).cuda()
    bi[: tokens * 8] = torch.from_numpy(z.view(np.int16)).cuda()
    return sa.QuantRows.wrap(0, bits, ROW, capacity, d, sc, bi)


def read_dev(ptr, nbytes):
    """`nbytes` of device memory at the raw address `ptr`, as a numpy byte array."""
    import ctypes

    import torch

    torch.cuda.synchronize()
    out = np.empty(nbytes, np.uint8)
    rt = ctypes.CDLL("libcudart.so.12")
    rt.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
    rc = rt.cudaMemcpy(out.ctypes.data, ctypes.c_void_p(ptr), nbytes, 2)  # cudaMemcpyDeviceToHost
    assert rc == 0, f"cudaMemcpy failed with {rc}"
    return out
