"""The torch operator layer: ``torch.ops.nvfp4effma.*`` with the schemas of the reference's extension
(binds/python/csrc/nvfp4effma_torch.cpp:721-743 there), a CUDA implementation that calls the C ABI of
``libnvfp4effma.so`` and a Meta implementation (shapes and dtypes only), so that code written against the reference's
operators -- or traced through them by ``torch.compile`` / ``torch.library.opcheck`` -- runs unchanged.

Conventions shared with the reference's operators: NVFP4 data is ``uint8`` [rows, cols / 2], block scales ``uint8``
(linear [rows, >= cols / 16] or the padded swizzled buffer), globals ``float32``; a result is row-major ``[T, N]``, which
is the column-major ``D`` of the C ABI with ``ldd = N`` (m = N output features, n = T tokens).  ``want_amax`` returns
max |result| as a fresh one-element tensor.  There is no fallback: every CUDA implementation is one or two ``nvfp4a_*`` calls.
"""
import ctypes

import torch

from . import _abi as A
from . import _lib as L

_NS = "nvfp4effma"
_lib = torch.library.Library(_NS, "FRAGMENT")
_OPT7 = "(Tensor?, Tensor?, Tensor?, Tensor?, Tensor?, Tensor?, Tensor?)"
_X = "Tensor x, Tensor? x_scales, Tensor? x_global, int x_flags, int x_smax"
_W = "Tensor w, Tensor w_scales, Tensor? w_global, int w_flags, int w_smax"
_XI = "Tensor x_img, int x_dtype, Tensor? x_global, int x_flags, int x_smax, int T, Tensor w_img, Tensor? w_global, int w_flags, int w_smax, int N, int K"
SCHEMAS = {
    "quantize_ex": "(Tensor x, bool rowwise, bool columnwise, Tensor? g_row, Tensor? g_col, int flags, int scale_max, int tile_rows, "
                   f"int four_over_six, bool compute_amax, bool want_amax) -> {_OPT7}",
    "quantize_int8": "(Tensor x) -> (Tensor, Tensor)",
    "dequantize": "(Tensor data, Tensor scales, Tensor? global_, int flags, int scale_max, int cols, ScalarType dtype) -> Tensor",
    "transpose": "(Tensor data, Tensor scales, int flags, int scale_max, int cols) -> (Tensor, Tensor)",
    "swizzle_scales": "(Tensor scales, int rows, int cols, bool to_swizzled) -> Tensor",
    "linear": f"({_X}, {_W}, int k, Tensor? bias, ScalarType? out_dtype, float alpha, bool want_amax, Tensor? w_img) -> (Tensor, Tensor?)",
    "linear_out": f"({_X}, {_W}, int k, Tensor? bias, Tensor(a!) out, float alpha, float beta, bool want_amax, Tensor? w_img) -> Tensor?",
    "grouped_linear": f"({_X}, Tensor seg, {_W}, int k, int groups, Tensor? bias, ScalarType? out_dtype, float alpha, bool want_amax) -> (Tensor, Tensor?)",
    "grouped_linear_out": f"({_X}, Tensor seg, {_W}, int k, int groups, Tensor? bias, Tensor(a!) out, float alpha, float beta, bool want_amax) -> Tensor?",
    "tc_image": "(int operand, Tensor x, Tensor? scales, int flags, int k) -> Tensor",
    "linear_tc": f"({_XI}, Tensor? bias, ScalarType out_dtype, float alpha, bool want_amax) -> (Tensor, Tensor?)",
    "linear_tc_out": f"({_XI}, Tensor? bias, Tensor(a!) out, float alpha, float beta, bool want_amax) -> Tensor?",
}
for _name, _schema in SCHEMAS.items():
    _lib.define(_name + _schema)


def _op(name):
    """Registers the decorated pair member: ``@_op(name).cuda`` / ``@_op(name).meta``."""
    class _Reg:
        @staticmethod
        def cuda(fn):
            _lib.impl(name, fn, "CUDA")
            return fn

        @staticmethod
        def meta(fn):
            torch.library.register_fake(f"{_NS}::{name}", fn, lib=_lib)
            return fn
    return _Reg


def _u8(shape, like, zero=False):
    return (torch.zeros if zero else torch.empty)(shape, dtype=torch.uint8, device=like.device)


def _one_float(like):
    return torch.zeros(1, dtype=torch.float32, device=like.device)


def _scale_shape(rows, cols, flags):
    return A.padded_scale_shape(rows, cols) if flags & L.SCALES_SWIZZLED else (rows, cols // 16)


def _need_cols16(cols):
    if cols % 16:
        raise ValueError(f"{cols} values per row: NVFP4 / INT8 blocks hold 16, so the last dimension must be a multiple of 16")


# ---- quantize_ex -----------------------------------------------------------------------------------------------------------------
def _quantize_ex_outputs(x, rowwise, columnwise, flags, compute_amax, want_amax, fill):
    """Allocates what quantize_ex returns.  A column-wise half describes the transpose [cols, rows padded to 16]."""
    if x.dim() != 2:
        raise ValueError(f"quantize_ex takes a matrix, got shape {tuple(x.shape)}")
    A.dense_code(x.dtype)
    rows, cols = x.shape
    _need_cols16(cols)
    rows16 = -(-rows // 16) * 16
    per_row = bool(flags & L.GLOBAL_PER_ROW)
    out = [None] * 7
    if rowwise:
        out[0], out[1] = _u8((rows, cols // 2), x), _u8(_scale_shape(rows, cols, flags), x, zero=fill)
        if compute_amax:
            out[4] = torch.zeros(rows if per_row else 1, dtype=torch.float32, device=x.device)
    if columnwise:
        out[2], out[3] = _u8((cols, rows16 // 2), x, zero=fill and rows16 != rows), _u8(_scale_shape(cols, rows16, flags), x, zero=fill)
        if compute_amax:
            out[5] = _one_float(x)
    if want_amax:
        out[6] = _one_float(x)
    return out, rows16


@_op("quantize_ex").meta
def _quantize_ex_meta(x, rowwise, columnwise, g_row, g_col, flags, scale_max, tile_rows, four_over_six, compute_amax, want_amax):
    return tuple(_quantize_ex_outputs(x, rowwise, columnwise, flags, compute_amax, want_amax, False)[0])


@_op("quantize_ex").cuda
def _quantize_ex(x, rowwise, columnwise, g_row, g_col, flags, scale_max, tile_rows, four_over_six, compute_amax, want_amax):
    """``nvfp4a_quantize_ex``.  With ``compute_amax`` the globals are computed here and returned in positions 4 / 5 (the
    ``g_row`` / ``g_col`` arguments are not used); otherwise the given decode factors are applied and those positions are None."""
    out, rows16 = _quantize_ex_outputs(x, rowwise, columnwise, flags, compute_amax, want_amax, True)
    rows, cols = x.shape
    x = A.matrix(x, 16, "x")
    src = A.dense_tensor(x)
    halves = []
    for data, scales, glob, half_flags in ((out[0], out[1], out[4] if compute_amax else g_row, flags),
                                           (out[2], out[3], out[5] if compute_amax else g_col, flags & ~L.GLOBAL_PER_ROW)):
        halves.append(None if data is None else L.Tensor(A.addr(data), L.NVFP4, A.addr(scales), 0, A.addr(glob), A.addr(out[6]), half_flags, scale_max))
    cfg = L.QuantConfig(tile_rows, four_over_six, int(compute_amax))
    L.check(L.lib.nvfp4a_quantize_ex(ctypes.byref(src), x.stride(0), rows, cols, A.ref(halves[0]), cols, A.ref(halves[1]), rows16,
                                     ctypes.byref(cfg), A.stream()))
    return tuple(out)


# ---- quantize_int8 / dequantize / transpose / swizzle_scales ------------------------------------------------------------------------
@_op("quantize_int8").meta
def _quantize_int8_meta(x):
    if x.dim() != 2:
        raise ValueError(f"quantize_int8 takes a matrix, got shape {tuple(x.shape)}")
    A.dense_code(x.dtype)
    _need_cols16(x.shape[1])
    return (torch.empty(x.shape, dtype=torch.int8, device=x.device),
            torch.empty((x.shape[0], x.shape[1] // 16), dtype=torch.float32, device=x.device))


@_op("quantize_int8").cuda
def _quantize_int8(x):
    q, s = _quantize_int8_meta(x)
    x = A.matrix(x, 16, "x")
    src, dst = A.dense_tensor(x), L.Tensor(A.addr(q), L.INT8, A.addr(s), 0, None, None, 0, 0)
    L.check(L.lib.nvfp4a_quantize(ctypes.byref(src), x.stride(0), ctypes.byref(dst), x.shape[1], x.shape[0], x.shape[1], A.stream()))
    return q, s


@_op("dequantize").meta
def _dequantize_meta(data, scales, global_, flags, scale_max, cols, dtype):
    A.dense_code(dtype)
    return torch.empty((data.shape[0], cols), dtype=dtype, device=data.device)


@_op("dequantize").cuda
def _dequantize(data, scales, global_, flags, scale_max, cols, dtype):
    out = _dequantize_meta(data, scales, global_, flags, scale_max, cols, dtype)
    src, ld, _keep = A.fp4_tensor(data, scales, global_, flags, scale_max)
    dst = A.dense_tensor(out)
    L.check(L.lib.nvfp4a_dequantize(ctypes.byref(src), ld, ctypes.byref(dst), cols, data.shape[0], cols, A.stream()))
    return out


@_op("transpose").meta
def _transpose_meta(data, scales, flags, scale_max, cols):
    rows = data.shape[0]
    return _u8((cols, rows // 2), data), _u8(_scale_shape(cols, rows, flags), data)


@_op("transpose").cuda
def _transpose(data, scales, flags, scale_max, cols):
    rows = data.shape[0]
    out, out_scales = _u8((cols, rows // 2), data), _u8(_scale_shape(cols, rows, flags), data, zero=True)
    f = flags & ~L.GLOBAL_PER_ROW
    src, ld, _keep = A.fp4_tensor(data, scales, None, f, scale_max)
    dst = L.Tensor(A.addr(out), L.NVFP4, A.addr(out_scales), 0, None, None, f, scale_max)
    L.check(L.lib.nvfp4a_transpose(ctypes.byref(src), ld, ctypes.byref(dst), rows, rows, cols, A.stream()))
    return out, out_scales


@_op("swizzle_scales").meta
def _swizzle_scales_meta(scales, rows, cols, to_swizzled):
    return _u8(A.padded_scale_shape(rows, cols) if to_swizzled else (rows, cols // 16), scales)


@_op("swizzle_scales").cuda
def _swizzle_scales(scales, rows, cols, to_swizzled):
    out = _swizzle_scales_meta(scales, rows, cols, to_swizzled)
    scales = scales.contiguous()
    pitch = scales.stride(0) if to_swizzled else cols // 16   # the pitch of the LINEAR side, whichever it is
    L.check(L.lib.nvfp4a_swizzle_scales(A.addr(scales), A.addr(out), pitch, rows, cols, int(to_swizzled), A.stream()))
    return out


# ---- linear ----------------------------------------------------------------------------------------------------------------------
def _result_dtype(x, out_dtype):
    return out_dtype if out_dtype is not None else (x.dtype if x.dtype in A.DENSE_CODES else torch.bfloat16)


def _check_out(out, T, N):
    if out.dim() != 2 or out.shape[0] != T or out.shape[1] != N or out.stride(1) != 1:
        raise ValueError(f"out must be a [{T}, {N}] matrix with unit stride along its rows, got {tuple(out.shape)} / strides {out.stride()}")
    A.dense_code(out.dtype)


def _bias_tensor(bias, N):
    if bias is None:
        return None, None
    if bias.numel() != N:
        raise ValueError(f"bias has {bias.numel()} elements for {N} output features")
    bias = bias.contiguous()
    return A.dense_tensor(bias), bias


def _gemm_into(out, x, x_scales, x_global, x_flags, x_smax, w, w_scales, w_global, w_flags, w_smax, k, bias, alpha, beta, want_amax, w_img):
    """One ``nvfp4a_gemm`` (or ``nvfp4a_gemv_tc`` on the weight's image up to 8 tokens) writing ``out``; returns the amax tensor or None."""
    if k % 64:
        raise ValueError(f"k = {k}: the reduction length must be a multiple of 64")
    T, N = x.shape[0], w.shape[0]
    _check_out(out, T, N)
    amax = _one_float(out) if want_amax else None
    b, ldb, _kb = A.activation_tensor(x, x_scales, x_global, x_flags, x_smax)
    d = A.dense_tensor(out, amax)
    tb, _bias = _bias_tensor(bias, N)
    c, ldc = (ctypes.byref(d), out.stride(0)) if beta != 0.0 else (None, 0)   # beta accumulates into out itself
    if w_img is not None and T <= 8:
        a = L.Tensor(A.addr(w_img), L.NVFP4, None, 0, A.addr(w_global), None, w_flags, w_smax)
        st = L.lib.nvfp4a_gemv_tc(N, T, k, alpha, ctypes.byref(a), ctypes.byref(b), ldb, beta, c, ldc, ctypes.byref(d), out.stride(0), A.ref(tb), A.stream())
    else:
        a, lda, _ka = A.fp4_tensor(w, w_scales, w_global, w_flags, w_smax)
        st = L.lib.nvfp4a_gemm(N, T, k, alpha, ctypes.byref(a), lda, ctypes.byref(b), ldb, beta, c, ldc, ctypes.byref(d), out.stride(0), A.ref(tb), A.stream())
    L.check(st)
    return amax


@_op("linear").meta
def _linear_meta(x, x_scales, x_global, x_flags, x_smax, w, w_scales, w_global, w_flags, w_smax, k, bias, out_dtype, alpha, want_amax, w_img):
    out = torch.empty((x.shape[0], w.shape[0]), dtype=_result_dtype(x, out_dtype), device=w.device)
    return out, (_one_float(out) if want_amax else None)


@_op("linear").cuda
def _linear(x, x_scales, x_global, x_flags, x_smax, w, w_scales, w_global, w_flags, w_smax, k, bias, out_dtype, alpha, want_amax, w_img):
    out = torch.empty((x.shape[0], w.shape[0]), dtype=_result_dtype(x, out_dtype), device=w.device)
    return out, _gemm_into(out, x, x_scales, x_global, x_flags, x_smax, w, w_scales, w_global, w_flags, w_smax, k, bias, alpha, 0.0, want_amax, w_img)


@_op("linear_out").meta
def _linear_out_meta(x, x_scales, x_global, x_flags, x_smax, w, w_scales, w_global, w_flags, w_smax, k, bias, out, alpha, beta, want_amax, w_img):
    _check_out(out, x.shape[0], w.shape[0])
    return _one_float(out) if want_amax else None


@_op("linear_out").cuda
def _linear_out(x, x_scales, x_global, x_flags, x_smax, w, w_scales, w_global, w_flags, w_smax, k, bias, out, alpha, beta, want_amax, w_img):
    return _gemm_into(out, x, x_scales, x_global, x_flags, x_smax, w, w_scales, w_global, w_flags, w_smax, k, bias, alpha, beta, want_amax, w_img)


# ---- grouped linear (mixture of experts): rows seg[g] .. seg[g + 1] of x meet the g-th block of N / groups weight rows ---------------
def _grouped_into(out, x, x_scales, x_global, x_flags, x_smax, seg, w, w_scales, w_global, w_flags, w_smax, k, groups, bias, alpha, beta, want_amax):
    if k % 64:
        raise ValueError(f"k = {k}: the reduction length must be a multiple of 64")
    if groups < 1 or w.shape[0] % groups:
        raise ValueError(f"{w.shape[0]} weight rows do not split into {groups} groups")
    if seg.dtype != torch.int32 or seg.numel() != groups + 1:
        raise ValueError(f"seg must hold {groups + 1} int32 row offsets")
    T, N = x.shape[0], w.shape[0] // groups
    _check_out(out, T, N)
    amax = _one_float(out) if want_amax else None
    b, ldb, _kb = A.activation_tensor(x, x_scales, x_global, x_flags, x_smax)
    a, lda, _ka = A.fp4_tensor(w, w_scales, w_global, w_flags, w_smax)
    d = A.dense_tensor(out, amax)
    tb, _bias = _bias_tensor(bias, w.shape[0])
    c, ldc = (ctypes.byref(d), out.stride(0)) if beta != 0.0 else (None, 0)
    seg = seg.contiguous()
    L.check(L.lib.nvfp4a_gemm_grouped(groups, N, k, T, alpha, ctypes.byref(a), lda, ctypes.byref(b), ldb, beta, c, ldc, ctypes.byref(d), out.stride(0),
                                      A.ref(tb), A.addr(seg), A.stream()))
    return amax


@_op("grouped_linear").meta
def _grouped_linear_meta(x, x_scales, x_global, x_flags, x_smax, seg, w, w_scales, w_global, w_flags, w_smax, k, groups, bias, out_dtype, alpha, want_amax):
    out = torch.empty((x.shape[0], w.shape[0] // groups), dtype=_result_dtype(x, out_dtype), device=w.device)
    return out, (_one_float(out) if want_amax else None)


@_op("grouped_linear").cuda
def _grouped_linear(x, x_scales, x_global, x_flags, x_smax, seg, w, w_scales, w_global, w_flags, w_smax, k, groups, bias, out_dtype, alpha, want_amax):
    # rows of x past seg[groups] belong to no group: the library leaves their outputs alone, so they read zero
    out = torch.zeros((x.shape[0], w.shape[0] // max(groups, 1)), dtype=_result_dtype(x, out_dtype), device=w.device)
    return out, _grouped_into(out, x, x_scales, x_global, x_flags, x_smax, seg, w, w_scales, w_global, w_flags, w_smax, k, groups, bias, alpha, 0.0, want_amax)


@_op("grouped_linear_out").meta
def _grouped_linear_out_meta(x, x_scales, x_global, x_flags, x_smax, seg, w, w_scales, w_global, w_flags, w_smax, k, groups, bias, out, alpha, beta, want_amax):
    return _one_float(out) if want_amax else None


@_op("grouped_linear_out").cuda
def _grouped_linear_out(x, x_scales, x_global, x_flags, x_smax, seg, w, w_scales, w_global, w_flags, w_smax, k, groups, bias, out, alpha, beta, want_amax):
    return _grouped_into(out, x, x_scales, x_global, x_flags, x_smax, seg, w, w_scales, w_global, w_flags, w_smax, k, groups, bias, alpha, beta, want_amax)


# ---- images and the image GEMM ----------------------------------------------------------------------------------------------------
def _image_dtype_code(x):
    return L.NVFP4 if x.dtype == torch.uint8 else L.INT8 if x.dtype == torch.int8 else A.dense_code(x.dtype)


def image_bytes(operand, x, k):
    """Size of the image of kind ``operand`` of ``x`` (the reference's size formula; computed without the library for Meta tensors)."""
    rows, code = x.shape[0], _image_dtype_code(x)
    if code == L.NVFP4:
        return -(-rows // 128) * -(-k // 256) * 18432
    if operand != L.TC_B or code not in (L.INT8, L.BF16):
        raise NotImplementedError(f"no image of kind {operand} for a {x.dtype} operand")
    return -(-(rows * k) // 16) * 16 + rows * (k // 16) * 4 if code == L.INT8 else rows * k * 2


@_op("tc_image").meta
def _tc_image_meta(operand, x, scales, flags, k):
    return _u8((image_bytes(operand, x, k),), x)


@_op("tc_image").cuda
def _tc_image(operand, x, scales, flags, k):
    """``nvfp4a_tc_image``: operand 0 / 2 = the image of an NVFP4 weight (A16 / A8), 1 = of activations (NVFP4, int8, bfloat16)."""
    rows = x.shape[0]
    src, ld, _keep = A.activation_tensor(x, scales, None, flags & (L.SCALES_SWIZZLED | L.SCALES_UE5M3), 0)
    size = L.lib.nvfp4a_tc_image_bytes(operand, src.dtype, rows, k)
    if size == 0:
        raise NotImplementedError(f"no image of kind {operand} for a {x.dtype} operand with k = {k}")
    image = _u8((size,), x)
    L.check(L.lib.nvfp4a_tc_image(operand, ctypes.byref(src), ld, rows, k, A.addr(image), A.stream()))
    return image


_IMAGE_B_CODES = (L.NVFP4, L.INT8, L.BF16)   # x_dtype 0, 1, 2 of linear_tc


def _image_gemm_into(out, x_img, x_dtype, x_global, x_flags, x_smax, T, w_img, w_global, w_flags, w_smax, N, K, bias, alpha, beta, want_amax):
    if not 0 <= x_dtype < 3:
        raise ValueError(f"x_dtype = {x_dtype}: 0 NVFP4, 1 int8, 2 bfloat16")
    _check_out(out, T, N)
    code = _IMAGE_B_CODES[x_dtype]
    fp4 = code == L.NVFP4
    amax = _one_float(out) if want_amax else None
    a = L.Tensor(A.addr(w_img), L.NVFP4, None, 0, A.addr(w_global), None, w_flags, w_smax)
    b = L.Tensor(A.addr(x_img), code, None, 0, A.addr(x_global) if fp4 else None, None, x_flags if fp4 else 0, x_smax if fp4 else 0)
    d = A.dense_tensor(out, amax)
    tb, _bias = _bias_tensor(bias, N)
    c, ldc = (ctypes.byref(d), out.stride(0)) if beta != 0.0 else (None, 0)
    L.check(L.lib.nvfp4a_gemm_tc(N, T, K, alpha, ctypes.byref(a), ctypes.byref(b), beta, c, ldc, ctypes.byref(d), out.stride(0), A.ref(tb),
                                 A.addr(A.workspace(w_img.device)), A.stream()))
    return amax


@_op("linear_tc").meta
def _linear_tc_meta(x_img, x_dtype, x_global, x_flags, x_smax, T, w_img, w_global, w_flags, w_smax, N, K, bias, out_dtype, alpha, want_amax):
    out = torch.empty((T, N), dtype=out_dtype, device=w_img.device)
    return out, (_one_float(out) if want_amax else None)


@_op("linear_tc").cuda
def _linear_tc(x_img, x_dtype, x_global, x_flags, x_smax, T, w_img, w_global, w_flags, w_smax, N, K, bias, out_dtype, alpha, want_amax):
    out = torch.empty((T, N), dtype=out_dtype, device=w_img.device)
    return out, _image_gemm_into(out, x_img, x_dtype, x_global, x_flags, x_smax, T, w_img, w_global, w_flags, w_smax, N, K, bias, alpha, 0.0, want_amax)


@_op("linear_tc_out").meta
def _linear_tc_out_meta(x_img, x_dtype, x_global, x_flags, x_smax, T, w_img, w_global, w_flags, w_smax, N, K, bias, out, alpha, beta, want_amax):
    _check_out(out, T, N)
    return _one_float(out) if want_amax else None


@_op("linear_tc_out").cuda
def _linear_tc_out(x_img, x_dtype, x_global, x_flags, x_smax, T, w_img, w_global, w_flags, w_smax, N, K, bias, out, alpha, beta, want_amax):
    return _image_gemm_into(out, x_img, x_dtype, x_global, x_flags, x_smax, T, w_img, w_global, w_flags, w_smax, N, K, bias, alpha, beta, want_amax)


ops = getattr(torch.ops, _NS)
