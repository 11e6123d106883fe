"""Host-side operations over the C ABI on torch tensors: the counterpart of the reference's operator layer
(binds/python/csrc/nvfp4effma_torch.cpp:70-469 and binds/python/nvfp4effma/_ops.py there), written as ctypes calls.

torch provides device memory, dtypes and the current stream; every computation is an ``nvfp4a_*`` call.  Argument checks
that the reference makes in C++ before calling the library are made here; the library validates the rest.  A result is
row-major ``[T, N]``, which is the column-major D of the C ABI with ``ldd = N`` (m = N output features, n = T tokens).
"""
import ctypes

import torch

from . import _lib as L

_DENSE = {torch.bfloat16: L.BF16, torch.float16: L.FP16, torch.float32: L.FP32}


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _dense_code(dtype):
    if dtype not in _DENSE:
        raise TypeError(f"expected bfloat16, float16 or float32, got {dtype}")
    return _DENSE[dtype]


def _cuda(t, what):
    if not t.is_cuda:
        raise ValueError(f"{what} must be a CUDA tensor")


def _rows_2d(t, align_elems, what):
    """A 2-D tensor whose rows are contiguous and whose row pitch and base satisfy the library's alignment; else a copy."""
    if t.dim() != 2:
        raise ValueError(f"{what} must be 2-D, got shape {tuple(t.shape)}")
    ok = t.stride(1) == 1 and t.stride(0) % align_elems == 0 and t.stride(0) >= t.shape[1] and t.data_ptr() % 16 == 0
    return t if ok else t.contiguous()


def swizzled_scale_shape(rows, cols):
    return ((rows + 127) // 128 * 128, (cols // 16 + 3) // 4 * 4)


def quantize_ex(x, rowwise, columnwise, g_row, g_col, flags, scale_max, tile_rows, four_over_six, compute_amax, want_amax):
    """``nvfp4a_quantize_ex`` on x [rows, cols]: returns (data_row, scales_row, data_col, scales_col, g_row, g_col, amax)."""
    _cuda(x, "x")
    code = _dense_code(x.dtype)
    if x.dim() != 2:
        raise ValueError("x must be 2-D here")
    rows, cols = x.shape
    if cols % 16:
        raise ValueError(f"the last dimension ({cols}) must be a multiple of 16")
    x = _rows_2d(x, 16, "x")
    swz = bool(flags & L.SCALES_SWIZZLED)
    dev = x.device
    amax = torch.zeros(1, dtype=torch.float32, device=dev)
    rows16 = (rows + 15) // 16 * 16

    def dest(orows, ocols, g, per_row_ok):
        data = torch.empty((orows, ocols // 2), dtype=torch.uint8, device=dev)
        shape = swizzled_scale_shape(orows, ocols) if swz else (orows, ocols // 16)
        sc = torch.zeros(shape, dtype=torch.uint8, device=dev)
        f = flags if per_row_ok else flags & ~L.GLOBAL_PER_ROW
        return data, sc, L.Tensor(_ptr(data), L.NVFP4, _ptr(sc), 0, _ptr(g), _ptr(amax) if want_amax else None, f, scale_max)

    src = L.Tensor(_ptr(x), code, None, 0, None, None, 0, 0)
    dr = sr = dc = sc_ = None
    tr = tc = None
    if rowwise:
        dr, sr, tr = dest(rows, cols, g_row, True)
    if columnwise:
        dc, sc_, tc = dest(cols, rows16, g_col, False)
    cfg = L.QuantConfig(tile_rows, four_over_six, int(bool(compute_amax)))
    L.check(L.lib.nvfp4a_quantize_ex(ctypes.byref(src), x.stride(0), rows, cols, ctypes.byref(tr) if tr is not None else None, cols,
                                     ctypes.byref(tc) if tc is not None else None, rows16, ctypes.byref(cfg), _stream()))
    return dr, sr, dc, sc_, g_row, g_col, amax


def quantize_int8(x):
    """``nvfp4a_quantize`` to INT8 with one FP32 scale per 16 values: returns (int8 [rows, cols], float32 [rows, cols / 16])."""
    _cuda(x, "x")
    code = _dense_code(x.dtype)
    rows, cols = x.shape
    if cols % 16:
        raise ValueError(f"the last dimension ({cols}) must be a multiple of 16")
    x = _rows_2d(x, 16, "x")
    q = torch.empty((rows, cols), dtype=torch.int8, device=x.device)
    s = torch.empty((rows, cols // 16), dtype=torch.float32, device=x.device)
    src = L.Tensor(_ptr(x), code, None, 0, None, None, 0, 0)
    dst = L.Tensor(_ptr(q), L.INT8, _ptr(s), 0, None, None, 0, 0)
    L.check(L.lib.nvfp4a_quantize(ctypes.byref(src), x.stride(0), ctypes.byref(dst), cols, rows, cols, _stream()))
    return q, s


def dequantize(data, scales, glob, flags, scale_max, cols, dtype):
    _cuda(data, "data")
    code = _dense_code(dtype)
    rows = data.shape[0]
    data = _rows_2d(data, 8, "data")
    out = torch.empty((rows, cols), dtype=dtype, device=data.device)
    ld_scale = 0 if flags & L.SCALES_SWIZZLED else scales.stride(0)
    src = L.Tensor(_ptr(data), L.NVFP4, _ptr(scales), ld_scale, _ptr(glob), None, flags, scale_max)
    dst = L.Tensor(_ptr(out), code, None, 0, None, None, 0, 0)
    L.check(L.lib.nvfp4a_dequantize(ctypes.byref(src), data.stride(0) * 2, ctypes.byref(dst), cols, rows, cols, _stream()))
    return out


def swizzle_scales(scales, rows, cols, to_swizzled):
    _cuda(scales, "scales")
    scales = scales.contiguous()
    if to_swizzled:
        out = torch.empty(swizzled_scale_shape(rows, cols), dtype=torch.uint8, device=scales.device)
        L.check(L.lib.nvfp4a_swizzle_scales(_ptr(scales), _ptr(out), scales.stride(0), rows, cols, 1, _stream()))
    else:
        out = torch.empty((rows, cols // 16), dtype=torch.uint8, device=scales.device)
        L.check(L.lib.nvfp4a_swizzle_scales(_ptr(scales), _ptr(out), cols // 16, rows, cols, 0, _stream()))
    return out


def transpose(data, scales, flags, scale_max, cols):
    rows = data.shape[0]
    data = _rows_2d(data, 8, "data")
    swz = bool(flags & L.SCALES_SWIZZLED)
    out = torch.empty((cols, rows // 2), dtype=torch.uint8, device=data.device)
    osc = torch.zeros(swizzled_scale_shape(cols, rows) if swz else (cols, rows // 16), dtype=torch.uint8, device=data.device)
    src = L.Tensor(_ptr(data), L.NVFP4, _ptr(scales), 0 if swz else scales.stride(0), None, None, flags & ~L.GLOBAL_PER_ROW, scale_max)
    dst = L.Tensor(_ptr(out), L.NVFP4, _ptr(osc), 0, None, None, flags & ~L.GLOBAL_PER_ROW, scale_max)
    L.check(L.lib.nvfp4a_transpose(ctypes.byref(src), data.stride(0) * 2, ctypes.byref(dst), rows, rows, cols, _stream()))
    return out, osc


def _fp4_operand(data, scales, glob, flags, scale_max, k):
    """NVFP4 operand -> (struct, ld, keep-alive): rows 16-byte aligned with a pitch that is a multiple of 64 values."""
    data = _rows_2d(data, 32, "NVFP4 data")
    swz = bool(flags & L.SCALES_SWIZZLED)
    if not swz:
        scales = scales if (scales.stride(1) == 1 and scales.stride(0) % 4 == 0 and scales.data_ptr() % 4 == 0) else None
    if scales is None:
        raise ValueError("linear block scales need a row pitch that is a multiple of 4 bytes and a 4-byte aligned base")
    ld_scale = 0 if swz else scales.stride(0)
    return L.Tensor(_ptr(data), L.NVFP4, _ptr(scales), ld_scale, _ptr(glob), None, flags, scale_max), data.stride(0) * 2, (data, scales, glob)


def _b_operand(x, x_scales, x_global, x_flags, x_smax, k):
    if x.dtype == torch.uint8:
        return _fp4_operand(x, x_scales, x_global, x_flags, x_smax, k)
    if x.dtype == torch.int8:
        x = _rows_2d(x, 64, "int8 x")
        s = x_scales.contiguous()
        if s.data_ptr() % 16 or s.stride(0) % 4:
            s = s.clone()
        return L.Tensor(_ptr(x), L.INT8, _ptr(s), s.stride(0), _ptr(x_global), None, 0, 0), x.stride(0), (x, s)
    x = _rows_2d(x, 64, "x")
    return L.Tensor(_ptr(x), _dense_code(x.dtype), None, 0, None, None, 0, 0), x.stride(0), (x,)


def linear(x, x_scales, x_global, x_flags, x_smax, w, w_scales, w_global, w_flags, w_smax, k, bias=None, out_dtype=None, out=None, alpha=1.0,
           beta=0.0, amax_out=None, w_img=None, w_rows=None, swiglu=False):
    """``alpha * x @ W^T + bias + beta * out``: ``nvfp4a_gemm``, or ``nvfp4a_gemv_tc`` when the weight's image is given and T <= 8.
    ``swiglu``: W holds gate and up rows interleaved per 16-row slice (8 gate rows, then their 8 up rows); the result is
    ``silu(gate) * up``, [T, N / 2], through the ``_ex`` entry points."""
    if beta != 0.0 and out is None:
        raise ValueError("beta != 0 accumulates into out, so out must be given")
    if out is not None and out_dtype is not None and out_dtype != out.dtype:
        raise ValueError(f"out_dtype {out_dtype} does not match out.dtype {out.dtype}")
    _cuda(w if w is not None else w_img, "weight")
    if k % 64:
        raise ValueError(f"in_features (K = {k}) must be a multiple of 64")
    N, T = (w.shape[0] if w is not None else w_rows), x.shape[0]
    dev = w.device if w is not None else w_img.device
    tB, ldb, keepB = _b_operand(x, x_scales, x_global, x_flags, x_smax, k)
    od = out.dtype if out is not None else (out_dtype or (x.dtype if x.dtype in _DENSE else torch.bfloat16))
    NO = N // 2 if swiglu else N
    if out is None:
        out = torch.empty((T, NO), dtype=od, device=dev)
    elif out.dim() != 2 or tuple(out.shape) != (T, NO) or out.stride(1) != 1:
        raise ValueError(f"out must be a [T, N] = [{T}, {NO}] tensor with contiguous rows")
    amax = torch.zeros(1, dtype=torch.float32, device=dev) if amax_out is not None else None
    ex = L.Epilogue()
    ex.swiglu = 1
    pe = ctypes.byref(ex)
    tD = L.Tensor(_ptr(out), _dense_code(od), None, 0, None, _ptr(amax), 0, 0)
    tbias = None
    if bias is not None:
        if bias.numel() != N:
            raise ValueError(f"bias must have {N} elements")
        bias = bias.contiguous()
        tbias = L.Tensor(_ptr(bias), _dense_code(bias.dtype), None, 0, None, None, 0, 0)
    pb = ctypes.byref(tbias) if tbias is not None else None
    pc, ldc = (ctypes.byref(tD), out.stride(0)) if beta != 0.0 else (None, 0)  # beta accumulates into out: C is D
    if w_img is not None and T <= 8:
        tA = L.Tensor(_ptr(w_img), L.NVFP4, None, 0, _ptr(w_global), None, w_flags, w_smax)
        args = (N, T, k, alpha, ctypes.byref(tA), ctypes.byref(tB), ldb, beta, pc, ldc, ctypes.byref(tD), out.stride(0), pb)
        st = L.lib.nvfp4a_gemv_tc_ex(*args, pe, _stream()) if swiglu else L.lib.nvfp4a_gemv_tc(*args, _stream())
    else:
        tA, lda, keepA = _fp4_operand(w, w_scales, w_global, w_flags, w_smax, k)
        args = (N, T, k, alpha, ctypes.byref(tA), lda, ctypes.byref(tB), ldb, beta, pc, ldc, ctypes.byref(tD), out.stride(0), pb)
        st = L.lib.nvfp4a_gemm_ex(*args, pe, _stream()) if swiglu else L.lib.nvfp4a_gemm(*args, _stream())
    L.check(st)
    if amax_out is not None:
        torch.maximum(amax_out, amax, out=amax_out)
    return out


def tc_image(operand, data, scales, flags, k):
    """``nvfp4a_tc_image``: operand 0 / 2 = weight image (A16 / A8) of an NVFP4 matrix, 1 = activation image (NVFP4, int8, bfloat16)."""
    _cuda(data, "data")
    rows = data.shape[0]
    if data.dtype == torch.uint8:
        t, ld, keep = _fp4_operand(data, scales, None, flags & (L.SCALES_SWIZZLED | L.SCALES_UE5M3), 0, k)
        dt = L.NVFP4
    else:
        t, ld, keep = _b_operand(data, scales, None, 0, 0, k)
        dt = t.dtype
    nbytes = L.lib.nvfp4a_tc_image_bytes(operand, dt, rows, k)
    if nbytes == 0:
        raise NotImplementedError(f"no image of kind {operand} for this operand type")
    img = torch.empty(nbytes, dtype=torch.uint8, device=data.device)
    L.check(L.lib.nvfp4a_tc_image(operand, ctypes.byref(t), ld, rows, k, _ptr(img), _stream()))
    return img


_workspaces = {}


def _workspace(device):
    key = (device.index, torch.cuda.current_stream().cuda_stream)
    if key not in _workspaces:
        _workspaces[key] = torch.zeros(L.lib.nvfp4a_tc_workspace_bytes(), dtype=torch.uint8, device=device)
    return _workspaces[key]


def linear_tc(x_img, x_dtype, x_global, x_flags, x_smax, T, w_img, w_global, w_flags, w_smax, N, K, bias=None, out_dtype=torch.bfloat16, out=None,
              alpha=1.0, beta=0.0, amax_out=None, swiglu=False):
    """``nvfp4a_gemm_tc`` on images; x_dtype 0 NVFP4, 1 int8, 2 bfloat16.  ``swiglu`` as in ``linear`` (``nvfp4a_gemm_tc_ex``)."""
    if beta != 0.0 and out is None:
        raise ValueError("beta != 0 accumulates into out, so out must be given")
    od = out.dtype if out is not None else out_dtype
    if out is None:
        out = torch.empty((T, N // 2 if swiglu else N), dtype=od, device=w_img.device)
    amax = torch.zeros(1, dtype=torch.float32, device=w_img.device) if amax_out is not None else None
    tA = L.Tensor(_ptr(w_img), L.NVFP4, None, 0, _ptr(w_global), None, w_flags, w_smax)
    bt = (L.NVFP4, L.INT8, L.BF16)[x_dtype]
    tB = L.Tensor(_ptr(x_img), bt, None, 0, _ptr(x_global), None, x_flags if bt == L.NVFP4 else 0, x_smax if bt == L.NVFP4 else 0)
    tD = L.Tensor(_ptr(out), _dense_code(od), None, 0, None, _ptr(amax), 0, 0)
    tbias = None
    if bias is not None:
        bias = bias.contiguous()
        tbias = L.Tensor(_ptr(bias), _dense_code(bias.dtype), None, 0, None, None, 0, 0)
    pc, ldc = (ctypes.byref(tD), out.stride(0)) if beta != 0.0 else (None, 0)
    args = (N, T, K, alpha, ctypes.byref(tA), ctypes.byref(tB), beta, pc, ldc, ctypes.byref(tD), out.stride(0),
            ctypes.byref(tbias) if tbias is not None else None)
    if swiglu:
        ex = L.Epilogue()
        ex.swiglu = 1
        L.check(L.lib.nvfp4a_gemm_tc_ex(*args, ctypes.byref(ex), _ptr(_workspace(w_img.device)), _stream()))
    else:
        L.check(L.lib.nvfp4a_gemm_tc(*args, _ptr(_workspace(w_img.device)), _stream()))
    if amax_out is not None:
        torch.maximum(amax_out, amax, out=amax_out)
    return out


def tp_gather(buffer_ptrs, flag_ptrs, rank, rows, row_pitch_bytes, col_offset_bytes, shard_bytes):
    """``nvfp4a_b200_tp_gather``: push this rank's columns of a peer-mapped activation buffer to every peer, then barrier."""
    world = len(buffer_ptrs)
    bufs = (ctypes.c_void_p * world)(*buffer_ptrs)
    flags = (ctypes.c_void_p * world)(*flag_ptrs)
    L.check(L.lib.nvfp4a_b200_tp_gather(bufs, flags, world, rank, rows, row_pitch_bytes, col_offset_bytes, shard_bytes, _stream()))


def gemv_tp(x, w_img, w_rows, w_global, w_flags, w_smax, k, bias, out, swiglu, buffer_ptrs, flag_ptrs, rank):
    """``nvfp4a_b200_gemv_tc_tp``: up to 8 rows of bfloat16 ``x`` against a weight image; ``out`` (a view into this rank's
    peer-mapped buffer) is also written into every peer's buffer and the ranks meet in a barrier."""
    T = x.shape[0]
    x = _rows_2d(x, 64, "x")
    world = len(buffer_ptrs)
    bufs = (ctypes.c_void_p * world)(*buffer_ptrs)
    flags = (ctypes.c_void_p * world)(*flag_ptrs)
    tA = L.Tensor(_ptr(w_img), L.NVFP4, None, 0, _ptr(w_global), None, w_flags, w_smax)
    tB = L.Tensor(_ptr(x), L.BF16, None, 0, None, None, 0, 0)
    tD = L.Tensor(_ptr(out), _dense_code(out.dtype), None, 0, None, None, 0, 0)
    tbias = L.Tensor(_ptr(bias), _dense_code(bias.dtype), None, 0, None, None, 0, 0) if bias is not None else None
    ex = L.Epilogue()
    ex.swiglu = int(bool(swiglu))
    L.check(L.lib.nvfp4a_b200_gemv_tc_tp(w_rows, T, k, 1.0, ctypes.byref(tA), ctypes.byref(tB), x.stride(0), ctypes.byref(tD), out.stride(0),
                                         ctypes.byref(tbias) if tbias is not None else None, ctypes.byref(ex), bufs, flags, world, rank, _stream()))
    return out


def gemm_tp(x, w_img, w_rows, w_global, w_flags, w_smax, k, bias, out, swiglu, buffer_ptrs, flag_ptrs, rank):
    """``nvfp4a_b200_gemm_tc_tp``: more than 8 rows of contiguous bfloat16 ``x`` [T, k] (used as its own activation image)
    against a weight image; the GEMM's epilogue also stores ``out`` into every peer's buffer, then the ranks' barrier."""
    T = x.shape[0]
    if not (x.is_contiguous() and x.data_ptr() % 16 == 0):
        x = x.contiguous()
    world = len(buffer_ptrs)
    bufs = (ctypes.c_void_p * world)(*buffer_ptrs)
    flags = (ctypes.c_void_p * world)(*flag_ptrs)
    tA = L.Tensor(_ptr(w_img), L.NVFP4, None, 0, _ptr(w_global), None, w_flags, w_smax)
    tB = L.Tensor(_ptr(x), L.BF16, None, 0, None, None, 0, 0)
    tD = L.Tensor(_ptr(out), _dense_code(out.dtype), None, 0, None, None, 0, 0)
    tbias = L.Tensor(_ptr(bias), _dense_code(bias.dtype), None, 0, None, None, 0, 0) if bias is not None else None
    ex = L.Epilogue()
    ex.swiglu = int(bool(swiglu))
    L.check(L.lib.nvfp4a_b200_gemm_tc_tp(w_rows, T, k, 1.0, ctypes.byref(tA), ctypes.byref(tB), ctypes.byref(tD), out.stride(0),
                                         ctypes.byref(tbias) if tbias is not None else None, ctypes.byref(ex), _ptr(_workspace(w_img.device)), bufs, flags,
                                         world, rank, _stream()))
    return out
