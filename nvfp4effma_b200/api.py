"""The functional API of the package (see the package docstring); imported on first use so that the build module can run
before the shared library exists."""
import math
import os
from typing import List, Optional, Union

import torch

from . import _lib, _ops
from ._lib import GLOBAL_AMAX, GLOBAL_PER_ROW, SCALES_SWIZZLED, SCALES_UE5M3
from .tensor import Int8Tensor, NVFP4Linear, NVFP4Tensor, TCWeight, quantize_linear_

from . import __version__

__all__ = ["quantize", "quantize_int8", "dequantize", "linear", "grouped_linear", "NVFP4Tensor", "Int8Tensor", "NVFP4Linear", "TCWeight",
           "quantize_linear_", "get_include", "__version__"]

# act="auto": up to this many rows of x the exact W4A16 path runs; beyond it x is quantized to int8 first (W4A8)
AUTO_EXACT_MAX_ROWS = 2


def quantize(x: torch.Tensor, global_scale: Optional[torch.Tensor] = None, *, amax: Optional[torch.Tensor] = None, block: str = "1x16",
             four_over_six: Optional[str] = None, scale_max: Optional[int] = None, row_scaled: bool = False, columnwise: bool = False,
             swizzled: bool = False, scale_dtype: str = "e4m3") -> NVFP4Tensor:
    """Quantize ``x`` (bfloat16 / float16 / float32 CUDA tensor ``[..., K]``, K a multiple of 16, finite) to NVFP4 in
    Transformer Engine's arithmetic.  Without ``global_scale`` the amax of ``x`` (of each row with ``row_scaled``) is
    computed and stored (decode factor amax / (6 * scale_max)); a given ``global_scale`` is the decode factor itself."""
    if not isinstance(x, torch.Tensor):
        raise TypeError("x must be a tensor")
    if x.dim() < 1:
        raise ValueError("x must have at least one dimension")
    if block not in ("1x16", "16x16"):
        raise ValueError(f"block must be '1x16' or '16x16', got {block!r}")
    fos = {None: 0, "mae": 1, "mse": 2}.get(four_over_six.lower() if isinstance(four_over_six, str) else four_over_six)
    if fos is None:
        raise ValueError(f"four_over_six must be None, 'mae' or 'mse', got {four_over_six!r}")
    if scale_dtype not in ("e4m3", "ue5m3"):
        raise ValueError(f"scale_dtype must be 'e4m3' or 'ue5m3', got {scale_dtype!r}")
    smax = scale_max if scale_max is not None else (256 if fos else 0)
    x2 = x.reshape(-1, x.shape[-1]) if x.dim() != 2 else x
    rows = x2.shape[0]
    if columnwise and row_scaled:
        raise ValueError("row-scaled tensors have no columnwise representation")
    if columnwise and rows % 16:
        raise ValueError(f"a columnwise representation needs rows % 16 == 0 (got {rows})")
    te = global_scale is None
    flags = (SCALES_SWIZZLED if swizzled else 0) | (SCALES_UE5M3 if scale_dtype == "ue5m3" else 0) | (GLOBAL_AMAX if te else 0)
    if te:
        g_row = torch.zeros(rows if row_scaled else 1, dtype=torch.float32, device=x.device)
        g_col = torch.zeros(1, dtype=torch.float32, device=x.device) if columnwise else None
        if row_scaled and rows > 1:
            flags |= GLOBAL_PER_ROW
    else:
        g_row = global_scale.reshape(-1).float().contiguous()
        if g_row.numel() > 1:
            if g_row.numel() != rows:
                raise ValueError(f"global_scale has {g_row.numel()} elements: 1 or one per row ({rows})")
            if columnwise:
                raise ValueError("per-row globals have no columnwise representation")
            flags |= GLOBAL_PER_ROW
        g_col = g_row if columnwise else None
    dr, sr, dc, sc, g_row, g_col, amax_x = _ops.quantize_ex(x2, True, columnwise, g_row, g_col, flags, smax, 16 if block == "16x16" else 1, fos,
                                                            te, amax is not None)
    if amax is not None:
        torch.maximum(amax, amax_x, out=amax)
    shape = tuple(x.shape)
    ue = scale_dtype == "ue5m3"
    blk = (16, 16) if block == "16x16" else (1, 16)

    def wrap(d, s, g, cols):
        kw = dict(scale_max=smax, swizzled=swizzled, ue5m3=ue, cols=cols, block=blk)
        s = s if ue else s.view(torch.float8_e4m3fn)
        return NVFP4Tensor(d, s, amax=g, **kw) if te else NVFP4Tensor(d, s, g, **kw)

    data = dr.reshape(*shape[:-1], shape[-1] // 2)
    out = wrap(data, sr if swizzled else sr.reshape(*shape[:-1], shape[-1] // 16), g_row, shape[-1])
    if columnwise:
        out.columnwise = wrap(dc, sc, g_col, rows)
    return out


def quantize_int8(x: torch.Tensor) -> Int8Tensor:
    """Quantize ``x`` to int8 with an FP32 scale per 16 values: scale = max |x| / 127 over the block, data = round(x / scale)."""
    if not isinstance(x, torch.Tensor):
        raise TypeError("x must be a tensor")
    if x.dim() < 1:
        raise ValueError("x must have at least one dimension")
    q, s = _ops.quantize_int8(x.reshape(-1, x.shape[-1]) if x.dim() != 2 else x)
    return Int8Tensor(q.reshape(x.shape), s.reshape(*x.shape[:-1], x.shape[-1] // 16), x.dtype)


def get_include() -> List[str]:
    """Directory with ``nvfp4effma.h`` (the C ABI) and ``nvfp4effma_b200.h``."""
    return [os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include")]


def dequantize(x: NVFP4Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """The values of ``x`` rounded once to ``dtype``."""
    if not isinstance(x, NVFP4Tensor):
        raise TypeError(f"expected an NVFP4Tensor, got {type(x).__name__}")
    d, s, g, flags, smax, cols = x._flat()
    return _ops.dequantize(d, s.view(torch.uint8), g, flags, smax, cols, dtype).reshape(x.shape)


def linear(x: Union[torch.Tensor, NVFP4Tensor, Int8Tensor], weight, bias: Optional[torch.Tensor] = None, *, act: str = "auto",
           out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None, alpha: float = 1.0, beta: float = 0.0,
           amax_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``alpha * x @ weight.T + bias + beta * out``; ``weight``: ``NVFP4Tensor`` ``[N, K]`` (K a multiple of 64) or ``TCWeight``;
    ``x``: dense ``[..., K]``, a 2-D ``NVFP4Tensor`` or an ``Int8Tensor``; ``act``: "auto", "exact" (W4A16), "int8" (W4A8), "nvfp4" (W4A4)."""
    if isinstance(weight, TCWeight):
        return _linear_tc(x, weight, bias, act, out_dtype, out, alpha, beta, amax_out)
    if not isinstance(weight, NVFP4Tensor):
        raise TypeError(f"weight must be an NVFP4Tensor, got {type(weight).__name__}")
    if weight.dim() != 2:
        raise ValueError(f"weight must be 2-D [out_features, in_features], got shape {weight.shape}")
    N, K = weight.shape
    wd, ws, wg, wf, wm, _ = weight._flat()
    ws = ws.view(torch.uint8)
    common = dict(alpha=alpha, beta=beta, amax_out=amax_out)
    if isinstance(x, NVFP4Tensor):
        if x.dim() != 2 or x.shape[1] != K:
            raise ValueError(f"an NVFP4 x must have shape [T, {K}], got {x.shape}")
        xd, xs, xg, xf, xm, _ = x._flat()
        return _ops.linear(xd, xs.view(torch.uint8), xg, xf, xm, wd, ws, wg, wf, wm, K, bias, out_dtype, out, **common)
    if isinstance(x, Int8Tensor):
        if x.shape[-1] != K:
            raise ValueError(f"x must have shape [..., {K}], got {x.shape}")
        o2 = out.reshape(-1, N) if out is not None else None
        od = out_dtype if out_dtype is not None or out is not None else x.dtype
        y = _ops.linear(x.data.reshape(-1, K), x.scales.reshape(-1, K // 16), None, 0, 0, wd, ws, wg, wf, wm, K, bias, od, o2, **common)
        return out if out is not None else y.reshape(*x.shape[:-1], N)
    if not isinstance(x, torch.Tensor):
        raise TypeError("x must be a tensor, an NVFP4Tensor or an Int8Tensor")
    if x.dim() < 1 or x.shape[-1] != K:
        raise ValueError(f"x must have shape [..., {K}], got {tuple(x.shape)}")
    if act not in ("auto", "exact", "int8", "nvfp4"):
        raise ValueError(f"act must be 'auto', 'exact', 'int8' or 'nvfp4', got {act!r}")
    x2 = x.reshape(-1, K)
    if act == "auto":
        act = "exact" if x2.shape[0] <= AUTO_EXACT_MAX_ROWS else "int8"
    if act == "int8":
        y = linear(quantize_int8(x2), weight, bias, out_dtype=out_dtype, out=out, **common)
        return out if out is not None else y.reshape(*x.shape[:-1], N)
    o2 = out.reshape(-1, N) if out is not None else None
    od = out_dtype if out_dtype is not None or out is not None else x.dtype
    if act == "nvfp4":
        qd, qs, qg, qf, qm, _ = quantize(x2)._flat()
        y = _ops.linear(qd, qs.view(torch.uint8), qg, qf, qm, wd, ws, wg, wf, wm, K, bias, od, o2, **common)
    else:
        y = _ops.linear(x2, None, None, 0, 0, wd, ws, wg, wf, wm, K, bias, out_dtype, o2, **common)
    return out if out is not None else y.reshape(*x.shape[:-1], N)


def grouped_linear(*args, **kwargs):
    """Mixture-of-experts grouped linear layer: not part of this build (``nvfp4a_gemm_grouped`` returns NOT_SUPPORTED)."""
    raise NotImplementedError("grouped_linear is not part of this build")


def _linear_tc(x, weight, bias, act, out_dtype, out, alpha, beta, amax_out):
    """``linear`` with a ``TCWeight``: the GEMV on the weight's image up to 8 rows of ``x``, the image GEMM beyond."""
    N, K = weight.shape
    if act == "auto":
        act = weight.act
    if act not in ("exact", "int8", "nvfp4"):
        raise ValueError(f"act must be 'auto', 'exact', 'int8' or 'nvfp4', got {act!r}")
    if isinstance(x, torch.Tensor):
        if (act == "exact") != (weight.act == "exact"):
            raise ValueError(f"act {act!r} does not match the weight's image ({weight.act!r})")
        if act == "exact" and x.dtype != torch.bfloat16:
            raise TypeError(f"the exact tensor-core path (W4A16) takes a bfloat16 x, got {x.dtype}")
        od = out_dtype or (out.dtype if out is not None else x.dtype)
        lead = tuple(x.shape[:-1])
        x2 = x.reshape(-1, K)
        x = quantize_int8(x2) if act == "int8" else quantize(x2) if act == "nvfp4" else x2
    else:
        if weight.act == "exact":
            raise ValueError("an Int8Tensor / NVFP4Tensor x needs a weight image for int8 / nvfp4")
        od = out_dtype or (out.dtype if out is not None else x.dtype if isinstance(x, Int8Tensor) else torch.bfloat16)
        lead = tuple(x.shape[:-1])
    rows = x.rows if isinstance(x, NVFP4Tensor) else math.prod(x.shape[:-1])
    _, _, wg, wf, wm, _ = weight.weight._flat()
    wd, ws = weight.weight._flat()[:2]
    o2 = out.reshape(-1, N) if out is not None else None
    common = dict(alpha=alpha, beta=beta, amax_out=amax_out)
    if rows <= 8:
        if isinstance(x, NVFP4Tensor):
            xd, xs, xg, xf, xm, _ = x._flat()
            y = _ops.linear(xd, xs.view(torch.uint8), xg, xf, xm, wd, ws.view(torch.uint8), wg, wf, wm, K, bias, od, o2, w_img=weight.image, **common)
        elif isinstance(x, Int8Tensor):
            y = _ops.linear(x.data.reshape(-1, K), x.scales.reshape(-1, K // 16), None, 0, 0, wd, ws.view(torch.uint8), wg, wf, wm, K, bias, od, o2,
                            w_img=weight.image, **common)
        else:
            y = _ops.linear(x, None, None, 0, 0, wd, ws.view(torch.uint8), wg, wf, wm, K, bias, od, o2, w_img=weight.image, **common)
    elif isinstance(x, NVFP4Tensor):
        xd, xs, xg, xf, xm, _ = x._flat()
        img = _ops.tc_image(1, xd, xs.view(torch.uint8), xf, K)
        y = _ops.linear_tc(img, 0, xg, xf, xm, rows, weight.image, wg, wf, wm, N, K, bias, od, o2, **common)
    elif isinstance(x, Int8Tensor):
        img = _ops.tc_image(1, x.data.reshape(-1, K), x.scales.reshape(-1, K // 16), 0, K)
        y = _ops.linear_tc(img, 1, None, 0, 0, rows, weight.image, wg, wf, wm, N, K, bias, od, o2, **common)
    else:
        img = _ops.tc_image(1, x, None, 0, K)
        y = _ops.linear_tc(img, 2, None, 0, 0, rows, weight.image, wg, wf, wm, N, K, bias, od, o2, **common)
    return out if out is not None else y.reshape(*lead, N)
