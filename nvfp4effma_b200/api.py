"""The functional API: ``quantize``, ``quantize_int8``, ``dequantize``, ``linear``, ``grouped_linear`` -- the function names,
arguments and error types of the reference's Python package (binds/python/nvfp4effma/__init__.py there) over this
library's operators (``torch.ops.nvfp4effma.*``, which call the C ABI).

Every ``linear`` call goes through the same three steps: the activations are normalised into an ``_Activations`` record
(quantizing them first if ``act`` asks for it), the result buffer is resolved (``out`` / ``out_dtype`` / the activations'
own type), and one operator runs: ``linear`` on the plain weight or on the weight's image (up to 8 rows), or ``linear_tc``
on the images of both operands.  The module is imported on first use so that the build step can run before the shared
library exists.
"""
import math
import os
from typing import List, NamedTuple, Optional, Tuple, Union

import torch

from . import __version__  # noqa: F401  (re-exported)
from . import _abi as A
from . import _lib as L
from ._ops import ops
from .tensor import Fp4Operand, Int8Tensor, NVFP4Linear, NVFP4Tensor, TCWeight, quantize_linear_

__all__ = ["quantize", "quantize_int8", "dequantize", "linear", "grouped_linear", "NVFP4Tensor", "Int8Tensor", "NVFP4Linear", "TCWeight",
           "quantize_linear_", "get_include", "__version__"]

# act="auto" on a plain NVFP4Tensor weight: dense activations of up to this many rows are used as they are (W4A16, the
# decode case, where the weights dominate the traffic anyway); more rows are quantized to INT8 first (W4A8).
AUTO_EXACT_MAX_ROWS = 2

_BLOCKS = {"1x16": (1, 16), "16x16": (16, 16)}
_FOUR_OVER_SIX = {None: L.FOS_OFF, "mae": L.FOS_MAE, "mse": L.FOS_MSE}
_SCALE_TYPES = ("e4m3", "ue5m3")
_ACT_MODES = ("exact", "int8", "nvfp4")


def _as_matrix(x: torch.Tensor) -> torch.Tensor:
    return x if x.dim() == 2 else x.reshape(-1, x.shape[-1])


def _dense_input(x, name="x"):
    if not isinstance(x, torch.Tensor):
        raise TypeError(f"{name} is a {type(x).__name__}, not a torch.Tensor")
    if x.dim() == 0:
        raise ValueError(f"{name} is a scalar; it needs at least the dimension that is quantized")
    A.on_gpu(x, name)
    A.dense_code(x.dtype)


# ---- quantization ----------------------------------------------------------------------------------------------------------------
def quantize(x: torch.Tensor, global_scale: Optional[torch.Tensor] = None, *, amax: Optional[torch.Tensor] = None, block: str = "1x16",
             four_over_six: Optional[str] = None, scale_max: Optional[int] = None, row_scaled: bool = False, columnwise: bool = False,
             swizzled: bool = False, scale_dtype: str = "e4m3") -> NVFP4Tensor:
    """``x`` (bfloat16 / float16 / float32 on the GPU, ``[..., K]``, K a multiple of 16, finite values) as an ``NVFP4Tensor``
    in Transformer Engine's arithmetic.

    ``global_scale`` given: it is the decode factor (one value, or one per row).  Not given: max |x| is measured (per row
    with ``row_scaled``) and kept as the tensor's amax.  ``amax``: a one-element float32 tensor that is raised to max |x|.
    ``block``: "1x16" or "16x16" tiles; ``four_over_six``: None / "mae" / "mse" (scale bound 256 unless ``scale_max`` says
    otherwise); ``columnwise``: also quantize the transpose (rows a multiple of 16) into ``.columnwise``; ``swizzled``: block
    scales in the GEMM-swizzled layout; ``scale_dtype``: "e4m3" or "ue5m3"."""
    _dense_input(x)
    if block not in _BLOCKS:
        raise ValueError(f"block = {block!r}; the tile shapes are {tuple(_BLOCKS)}")
    mode = four_over_six.lower() if isinstance(four_over_six, str) else four_over_six
    if mode not in _FOUR_OVER_SIX:
        raise ValueError(f"four_over_six = {four_over_six!r}; use None, 'mae' or 'mse'")
    if scale_dtype not in _SCALE_TYPES:
        raise ValueError(f"scale_dtype = {scale_dtype!r}; the block scale types are {_SCALE_TYPES}")
    fos, ue5m3 = _FOUR_OVER_SIX[mode], scale_dtype == "ue5m3"
    bound = (256 if fos else 0) if scale_max is None else scale_max
    matrix = _as_matrix(x)
    rows, cols = matrix.shape
    if columnwise and row_scaled:
        raise ValueError("columnwise and row_scaled exclude each other: per-row globals do not survive the transpose")
    if columnwise and rows % 16:
        raise ValueError(f"columnwise needs whole 16-row blocks; x has {rows} rows")
    measured = global_scale is None
    flags = (L.SCALES_SWIZZLED if swizzled else 0) | (L.SCALES_UE5M3 if ue5m3 else 0) | (L.GLOBAL_AMAX if measured else 0)
    given = None
    if measured:
        if row_scaled and rows > 1:
            flags |= L.GLOBAL_PER_ROW
    else:
        given = global_scale.reshape(-1).to(torch.float32).contiguous()
        if given.numel() != 1:
            if given.numel() != rows:
                raise ValueError(f"global_scale holds {given.numel()} values; x has {rows} rows (give one value, or one per row)")
            if columnwise:
                raise ValueError("one global per row and columnwise exclude each other")
            flags |= L.GLOBAL_PER_ROW
    d_row, s_row, d_col, s_col, g_row, g_col, seen = ops.quantize_ex(matrix, True, columnwise, given, given if columnwise else None, flags, bound,
                                                                     _BLOCKS[block][0], fos, measured, amax is not None)
    if amax is not None:
        torch.maximum(amax, seen, out=amax)

    def build(data, codes, glob, ncols):
        extra = {"amax": glob} if measured else {"global_scale": glob}
        return NVFP4Tensor(data, codes, scale_max=bound, swizzled=swizzled, ue5m3=ue5m3, cols=ncols, block=_BLOCKS[block], **extra)

    lead = tuple(x.shape[:-1])
    result = build(d_row.reshape(*lead, cols // 2), s_row if swizzled else s_row.reshape(*lead, cols // 16), g_row if measured else given, cols)
    if columnwise:
        result.columnwise = build(d_col, s_col, g_col if measured else given, rows)
    return result


def quantize_int8(x: torch.Tensor) -> Int8Tensor:
    """``x`` as INT8 with a float32 scale per 16 values of the last dimension: scale = max |x| of the block / 127,
    value = round-to-nearest-even(x / scale), 0 where the scale is 0."""
    _dense_input(x)
    q, s = ops.quantize_int8(_as_matrix(x))
    return Int8Tensor(q.reshape(x.shape), s.reshape(*x.shape[:-1], x.shape[-1] // 16), x.dtype)


def dequantize(x: NVFP4Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Every element of ``x`` as ``dtype``: the exact product nibble x block scale x global, rounded once."""
    if not isinstance(x, NVFP4Tensor):
        raise TypeError(f"dequantize takes an NVFP4Tensor; got a {type(x).__name__}")
    op = x._operand()
    return ops.dequantize(op.data, op.scales, op.glob, op.flags, op.scale_max, op.cols, dtype).reshape(x.shape)


def get_include() -> List[str]:
    """The directory that holds ``nvfp4effma.h`` (the C ABI) and ``nvfp4effma_b200.h``, for building against the library."""
    package_dir = os.path.dirname(os.path.abspath(__file__))
    return [os.path.join(os.path.dirname(package_dir), "include")]


# ---- linear ----------------------------------------------------------------------------------------------------------------------
class _Activations(NamedTuple):
    """Activations as the operators take them: a matrix [rows, K] (dense, int8 or NVFP4 nibbles), its block scales and
    global where it has them, the leading shape of the caller's ``x`` and the result type when the caller names none."""
    kind: str                      # "dense" | "int8" | "nvfp4"
    data: torch.Tensor
    scales: Optional[torch.Tensor]
    glob: Optional[torch.Tensor]
    flags: int
    scale_max: int
    lead: Tuple[int, ...]
    result_dtype: torch.dtype

    @property
    def rows(self) -> int:
        return self.data.shape[0]

    @property
    def image_code(self) -> int:
        return {"nvfp4": 0, "int8": 1, "dense": 2}[self.kind]


def _from_fp4(t: NVFP4Tensor, K: int, lead=None, result_dtype=torch.bfloat16) -> _Activations:
    if t.dim() != 2 or t.shape[1] != K:
        raise ValueError(f"NVFP4 activations are a matrix [T, {K}] for this weight; got shape {t.shape}")
    op = t._operand()
    return _Activations("nvfp4", op.data, op.scales, op.glob, op.flags, op.scale_max, (op.rows,) if lead is None else lead, result_dtype)


def _from_int8(t: Int8Tensor, K: int) -> _Activations:
    if t.shape[-1] != K:
        raise ValueError(f"the weight takes {K} input features; the INT8 activations have shape {t.shape}")
    return _Activations("int8", t.data.reshape(-1, K), t.scales.reshape(-1, K // 16), None, 0, 0, t.shape[:-1], t.dtype)


def _activations(x, K: int, mode: str) -> _Activations:
    """``mode`` ("exact" / "int8" / "nvfp4") says what to make of dense activations; quantized ones are taken as they are."""
    if isinstance(x, NVFP4Tensor):
        return _from_fp4(x, K)
    if isinstance(x, Int8Tensor):
        return _from_int8(x, K)
    lead = tuple(x.shape[:-1])
    matrix = x.reshape(-1, K)
    if mode == "int8":
        return _from_int8(quantize_int8(matrix), K)._replace(lead=lead, result_dtype=x.dtype)
    if mode == "nvfp4":
        return _from_fp4(quantize(matrix), K, lead, x.dtype)
    return _Activations("dense", matrix, None, None, 0, 0, lead, x.dtype)


def _check_dense_x(x, K):
    if not isinstance(x, torch.Tensor):
        raise TypeError(f"x is a {type(x).__name__}; linear takes a torch.Tensor, an NVFP4Tensor or an Int8Tensor")
    if x.dim() == 0 or x.shape[-1] != K:
        raise ValueError(f"the weight takes {K} input features; x has shape {tuple(x.shape)}")


def _check_mode(act, allowed):
    if act not in allowed:
        raise ValueError(f"act = {act!r}; choose from {allowed}")


def _resolve_out(a: _Activations, N: int, out_dtype, out, beta):
    """(out as a [rows, N] matrix or None, result dtype).  ``beta`` accumulates into ``out``, so it needs one."""
    if out is None:
        if beta != 0.0:
            raise ValueError("beta != 0 adds beta * out to the product, so an out tensor has to be passed")
        return None, (out_dtype if out_dtype is not None else a.result_dtype)
    if out_dtype is not None and out_dtype != out.dtype:
        raise ValueError(f"out is {out.dtype} but out_dtype asks for {out_dtype}")
    return out.reshape(-1, N), out.dtype


def _raise_amax(amax_out, seen):
    if amax_out is not None:
        torch.maximum(amax_out, seen, out=amax_out)


def _run(a: _Activations, w: Fp4Operand, image, N, K, bias, out_dtype, out, alpha, beta, amax_out):
    out2d, dtype = _resolve_out(a, N, out_dtype, out, beta)
    want = amax_out is not None
    if image is not None and a.rows > 8:      # both operands as images: the tensor-core GEMM entry
        x_image = ops.tc_image(L.TC_B, a.data, a.scales, a.flags, K)
        head = (x_image, a.image_code, a.glob, a.flags, a.scale_max, a.rows, image, w.glob, w.flags, w.scale_max, N, K, bias)
        if out2d is None:
            y, seen = ops.linear_tc(*head, dtype, alpha, want)
        else:
            y, seen = out2d, ops.linear_tc_out(*head, out2d, alpha, beta, want)
    else:                                     # the plain entry; with an image and up to 8 rows, the GEMV on the image
        head = (a.data, a.scales, a.glob, a.flags, a.scale_max, w.data, w.scales, w.glob, w.flags, w.scale_max, K, bias)
        if out2d is None:
            y, seen = ops.linear(*head, dtype, alpha, want, image)
        else:
            y, seen = out2d, ops.linear_out(*head, out2d, alpha, beta, want, image)
    _raise_amax(amax_out, seen)
    return out if out is not None else y.reshape(*a.lead, N)


def linear(x: Union[torch.Tensor, NVFP4Tensor, Int8Tensor], weight, bias: Optional[torch.Tensor] = None, *, act: str = "auto",
           out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None, alpha: float = 1.0, beta: float = 0.0,
           amax_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``alpha * x @ weight.T + bias + beta * out``.

    ``weight``: an ``NVFP4Tensor`` ``[N, K]`` (K a multiple of 64) or a ``TCWeight``.  ``x``: dense ``[..., K]``, a 2-D
    ``NVFP4Tensor`` or an ``Int8Tensor``.  ``act`` decides what happens to a dense ``x``: "exact" uses it as it is (W4A16),
    "int8" / "nvfp4" quantize it first (W4A8 / W4A4), "auto" picks "exact" up to ``AUTO_EXACT_MAX_ROWS`` rows and "int8"
    beyond -- or, for a ``TCWeight``, what its image was built for.  ``amax_out`` is raised to max |result|."""
    if isinstance(weight, TCWeight):
        return _linear_on_image(x, weight, bias, act, out_dtype, out, alpha, beta, amax_out)
    if not isinstance(weight, NVFP4Tensor):
        raise TypeError(f"weight is a {type(weight).__name__}; linear takes an NVFP4Tensor or a TCWeight")
    if weight.dim() != 2:
        raise ValueError(f"a weight is a matrix [out_features, in_features]; got shape {weight.shape}")
    N, K = weight.shape
    mode = act
    if not isinstance(x, (NVFP4Tensor, Int8Tensor)):
        _check_dense_x(x, K)
        _check_mode(act, ("auto",) + _ACT_MODES)
        if mode == "auto":
            mode = "exact" if math.prod(x.shape[:-1]) <= AUTO_EXACT_MAX_ROWS else "int8"
    return _run(_activations(x, K, mode), weight._operand(), None, N, K, bias, out_dtype, out, alpha, beta, amax_out)


def _linear_on_image(x, weight: TCWeight, bias, act, out_dtype, out, alpha, beta, amax_out):
    N, K = weight.shape
    mode = weight.act if act == "auto" else act
    _check_mode(mode, _ACT_MODES)
    if isinstance(x, (NVFP4Tensor, Int8Tensor)):
        if weight.act == "exact":
            raise ValueError("quantized activations need a TCWeight built with act='int8' or act='nvfp4'; this one is 'exact'")
    else:
        _check_dense_x(x, K)
        if (mode == "exact") != (weight.act == "exact"):
            raise ValueError(f"act = {mode!r} cannot use an image built for act = {weight.act!r}")
        if mode == "exact" and x.dtype != torch.bfloat16:
            raise TypeError(f"the W4A16 image path multiplies bfloat16 activations; x is {x.dtype}")
    return _run(_activations(x, K, mode), weight.weight._operand(), weight.image, N, K, bias, out_dtype, out, alpha, beta, amax_out)


def grouped_linear(x: Union[torch.Tensor, NVFP4Tensor, Int8Tensor], weight: NVFP4Tensor, seg: torch.Tensor, groups: int,
                   bias: Optional[torch.Tensor] = None, *, act: str = "auto", out_dtype: Optional[torch.dtype] = None,
                   out: Optional[torch.Tensor] = None, alpha: float = 1.0, beta: float = 0.0,
                   amax_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Mixture-of-experts linear layer: ``weight`` stacks ``groups`` matrices ``[N, K]`` (``[groups * N, K]``), ``seg`` is a
    device tensor of ``groups + 1`` non-decreasing int32 row offsets (``seg[0] == 0``), and rows ``seg[g] .. seg[g + 1]`` of
    ``x`` ``[T, K]`` meet expert ``g``: result ``[T, N]``.  The row counts stay on the device (no host synchronisation).
    ``act`` as in ``linear`` ("auto" = "int8")."""
    if not isinstance(weight, NVFP4Tensor) or weight.dim() != 2:
        raise TypeError("grouped_linear takes the stacked experts as one 2-D NVFP4Tensor")
    if groups < 1 or weight.shape[0] % groups:
        raise ValueError(f"{weight.shape[0]} weight rows do not split into {groups} experts")
    N, K = weight.shape[0] // groups, weight.shape[1]
    mode = act
    if not isinstance(x, (NVFP4Tensor, Int8Tensor)):
        _check_dense_x(x, K)
        _check_mode(act, ("auto",) + _ACT_MODES)
        mode = "int8" if act == "auto" else act
    a = _activations(x, K, mode)
    w = weight._operand()
    out2d, dtype = _resolve_out(a, N, out_dtype, out, beta)
    head = (a.data, a.scales, a.glob, a.flags, a.scale_max, seg, w.data, w.scales, w.glob, w.flags, w.scale_max, K, groups, bias)
    want = amax_out is not None
    if out2d is None:
        y, seen = ops.grouped_linear(*head, dtype, alpha, want)
    else:
        y, seen = out2d, ops.grouped_linear_out(*head, out2d, alpha, beta, want)
    _raise_amax(amax_out, seen)
    return out if out is not None else y.reshape(*a.lead, N)
