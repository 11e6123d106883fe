"""Glue between torch tensors and the C ABI: pointers, the current stream, dtype codes, ``nvfp4a_tensor`` structs and the
layout fix-ups (a copy when a tensor's pitch or base does not satisfy the library's alignment rules).

torch is used for device memory and streams only; nothing here computes.
"""
import ctypes

import torch

from . import _lib as L

DENSE_CODES = {torch.bfloat16: L.BF16, torch.float16: L.FP16, torch.float32: L.FP32}


def stream():
    """The current CUDA stream as the ``cudaStream_t`` argument of an entry point."""
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def addr(t):
    """Device address of ``t`` (``None`` stays NULL)."""
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def ref(struct):
    """``byref`` that lets an absent struct through as NULL."""
    return None if struct is None else ctypes.byref(struct)


def dense_code(dtype):
    try:
        return DENSE_CODES[dtype]
    except KeyError:
        raise TypeError(f"{dtype} is not one of the dense element types (bfloat16, float16, float32)") from None


def on_gpu(t, name):
    if not t.is_cuda:
        raise ValueError(f"{name} lives on {t.device}; the library works on CUDA memory only")


def matrix(t, pitch_multiple, name):
    """``t`` as a 2-D matrix the library can address: unit stride along rows, a row pitch that is a multiple of
    ``pitch_multiple`` elements and not below the row length, a 16-byte aligned base.  Anything else is copied once."""
    if t.dim() != 2:
        raise ValueError(f"{name}: expected a matrix, got {t.dim()} dimensions {tuple(t.shape)}")
    pitch = t.stride(0)
    if t.stride(1) != 1 or pitch < t.shape[1] or pitch % pitch_multiple or t.data_ptr() & 15:
        t = t.contiguous()
    return t


def padded_scale_shape(rows, cols):
    """Shape of the swizzled block-scale buffer of a [rows, cols] matrix: rows up to 128, scale columns up to 4."""
    return (-(-rows // 128) * 128, -(-(cols // 16) // 4) * 4)


def dense_tensor(t, amax=None):
    return L.Tensor(addr(t), dense_code(t.dtype), None, 0, None, addr(amax), 0, 0)


def fp4_tensor(data, scales, glob, flags, scale_max, amax=None):
    """(struct, values between rows, tensors to keep alive) of an NVFP4 matrix given as uint8 nibbles and uint8 scale codes."""
    data = matrix(data, 32, "NVFP4 data")
    if flags & L.SCALES_SWIZZLED:
        pitch = 0
    else:
        if scales.stride(-1) != 1 or scales.stride(0) % 4 or scales.data_ptr() & 3:
            scales = scales.contiguous()
            if scales.stride(0) % 4:   # a scale row is cols / 16 bytes: pad the pitch to a multiple of 4
                wide = torch.zeros((scales.shape[0], -(-scales.shape[1] // 4) * 4), dtype=torch.uint8, device=scales.device)
                wide[:, :scales.shape[1]] = scales
                scales = wide
        pitch = scales.stride(0)
    return L.Tensor(addr(data), L.NVFP4, addr(scales), pitch, addr(glob), addr(amax), flags, scale_max), 2 * data.stride(0), (data, scales, glob)


def int8_tensor(q, scales):
    """(struct, pitch, keep-alive) of INT8 activations with an FP32 scale per 16 values."""
    q = matrix(q, 64, "int8 activations")
    scales = scales.contiguous()
    if scales.data_ptr() & 15 or scales.stride(0) % 4:
        wide = torch.zeros((scales.shape[0], -(-scales.shape[1] // 4) * 4), dtype=torch.float32, device=scales.device)
        wide[:, :scales.shape[1]] = scales
        scales = wide
    return L.Tensor(addr(q), L.INT8, addr(scales), scales.stride(0), None, None, 0, 0), q.stride(0), (q, scales)


def activation_tensor(x, scales, glob, flags, scale_max):
    """The B operand of a GEMM call from whatever the caller holds: uint8 = NVFP4, int8 = INT8 + FP32 scales, else dense."""
    if x.dtype == torch.uint8:
        return fp4_tensor(x, scales, glob, flags, scale_max)
    if x.dtype == torch.int8:
        return int8_tensor(x, scales)
    x = matrix(x, 64, "activations")
    return dense_tensor(x), x.stride(0), (x,)


_workspace_of = {}


def workspace(device):
    """The zeroed scratch buffer the ``_tc`` entry points want, one per (device, stream): calls on one stream are ordered,
    and every call leaves the buffer zeroed."""
    key = (device.index, torch.cuda.current_stream().cuda_stream)
    buf = _workspace_of.get(key)
    if buf is None:
        buf = _workspace_of[key] = torch.zeros(L.lib.nvfp4a_tc_workspace_bytes(), dtype=torch.uint8, device=device)
    return buf
