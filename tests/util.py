"""Helpers of the GPU parity tests: seeded host data in the oracle's containers, device copies, and ``nvfp4a_tensor``
structs over torch device memory.  The data generators restate the reference's test fixtures (tests/test_util.h:82-120 and
tests/test_nvfp4effma.cu:278-287 there): random nibbles, finite non-negative scale codes with one zero block in 16, and
quantizer inputs with zero, underflowing and saturating blocks."""
import ctypes

import numpy as np
import torch

import oracle as O
from nvfp4effma_b200 import _lib as L

NP_OF = {O.BF16: np.uint16, O.FP16: np.uint16, O.FP32: np.float32}


def dev(a):
    """numpy array -> torch CUDA tensor holding the same bytes."""
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    elif a.dtype == np.uint32:
        a = a.view(np.int32)
    return torch.from_numpy(a.copy()).cuda()


def host(t, dtype=None):
    a = t.detach().cpu().numpy()
    return a.view(dtype) if dtype is not None else a


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def tensor(data, dtype, scales=None, ld_scale=0, glob=None, amax=None, flags=0, scale_max=0):
    return L.Tensor(ptr(data), dtype, ptr(scales), ld_scale, ptr(glob), ptr(amax), flags, scale_max)


def stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class DevFp4:
    """Device copy of an ``oracle.Fp4``."""

    def __init__(self, h):
        self.h = h
        self.data, self.scales = dev(h.data), dev(h.scales)
        self.glob = None if h.glob is None else dev(h.glob)

    def tensor(self, amax=None):
        return tensor(self.data, L.NVFP4, self.scales, self.h.ld_scale, self.glob, amax, self.h.flags, self.h.scale_max)


def rand_fp4(rng, rows, cols, ld=None, ld_scale=None, flags=0, scale_max=0, glob=None):
    """Random NVFP4 matrix: every nibble pattern, scale codes 1..0x7E (E4M3) / 1..0xFD (UE5M3) with 1/16 zero blocks;
    per-row globals spread around ``glob``."""
    h = O.Fp4(rows, cols, ld=ld, ld_scale=ld_scale, flags=flags, scale_max=scale_max, glob=glob)
    h.data[:] = rng.integers(0, 256, h.data.size, dtype=np.uint8)
    top = 0xFD if flags & O.UE5M3 else 0x7E
    codes = rng.integers(1, top + 1, h.scales.size).astype(np.uint8)
    codes[rng.integers(0, 16, h.scales.size) == 0] = 0
    h.scales[:] = codes
    if glob is not None and flags & O.PER_ROW:
        h.glob[:] = (glob * (0.5 + rng.integers(0, 256, h.glob.size) / 256.0)).astype(np.float32)
    return h


def rand_q8(rng, rows, cols, ld=None, ld_scale=None, glob=None):
    h = O.Q8(rows, cols, ld=ld, ld_scale=ld_scale, glob=glob)
    h.data[:] = rng.integers(-127, 128, h.data.size).astype(np.int8)
    s = np.ldexp(1.0 + rng.integers(0, 1024, h.scales.size) / 1024.0, rng.integers(-10, 2, h.scales.size)).astype(np.float32)
    s[rng.integers(0, 16, h.scales.size) == 0] = 0.0
    h.scales[:] = s
    return h


def rand_dense(rng, dtype, n, scale):
    """``n`` values uniform in (-scale, scale) rounded to ``dtype``; returns the raw buffer."""
    x = ((rng.integers(0, 1 << 24, n) / float(1 << 24)) * 2.0 - 1.0).astype(np.float32) * np.float32(scale)
    return O.from_f32(x, dtype)


def quant_input(rng, rows, cols, lds, dtype):
    """Quantizer stress data: per block zero / tiny (scale underflows) / huge (saturates) / 2^(-12..11); row 1 all zero."""
    x = np.zeros((rows, lds), np.float32)
    nb = cols // 16
    kind = rng.integers(0, 8, (rows, nb))
    if rows > 1:
        kind[1, :] = 0
    mag = np.ldexp(1.0, rng.integers(-12, 12, (rows, nb))).astype(np.float32)
    mag[kind == 1] = 1e-9
    mag[kind == 2] = 3e4
    mag[kind == 0] = 0.0
    u = ((rng.integers(0, 1 << 24, (rows, nb, 16)) / float(1 << 24)) * 2.0 - 1.0).astype(np.float32)
    x[:, :cols] = (u * mag[:, :, None]).reshape(rows, cols)
    raw = O.from_f32(x, dtype)
    return O.to_f32(raw, dtype), raw  # the exactly representable values, and their raw buffer


def ulp_bf16(x):
    """Spacing of BF16 at |x| (float64 array)."""
    a = np.maximum(np.abs(x), 2.0 ** -126)
    return np.ldexp(1.0, np.floor(np.log2(a)).astype(np.int64) - 7)
