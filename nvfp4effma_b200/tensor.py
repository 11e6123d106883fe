"""Tensor containers of the Python surface: ``NVFP4Tensor``, ``Int8Tensor``, ``TCWeight`` and the ``NVFP4Linear`` module.

They mirror the classes of the reference's Python package (binds/python/nvfp4effma/tensor.py:14-323 there): same
constructor arguments, attribute names, checkpoint buffer names (``weight`` / ``weight_scale`` / ``weight_scale_2``) and
errors, so code written against the reference keeps working.  Inference only; no autograd.
"""
import math
from typing import Optional, Tuple

import torch

from . import _lib as L
from . import _ops


class NVFP4Tensor:
    """An NVFP4 tensor of logical shape ``[..., cols]``: ``value = e2m1 * block_scale * global``."""

    def __init__(self, data: torch.Tensor, scales: torch.Tensor, global_scale: Optional[torch.Tensor] = None, *,
                 amax: Optional[torch.Tensor] = None, scale_max: int = 0, swizzled: bool = False, ue5m3: bool = False,
                 cols: Optional[int] = None, columnwise: Optional["NVFP4Tensor"] = None, block: Optional[Tuple[int, int]] = None):
        if data.dtype != torch.uint8:
            raise TypeError(f"data must be torch.uint8 (two E2M1 values per byte), got {data.dtype}")
        if ue5m3:
            if scales.dtype != torch.uint8:
                raise TypeError(f"UE5M3 scales are stored as torch.uint8, got {scales.dtype}")
        elif scales.dtype == torch.uint8:
            scales = scales.view(torch.float8_e4m3fn)
        elif scales.dtype != torch.float8_e4m3fn:
            raise TypeError(f"scales must be torch.float8_e4m3fn (or uint8), got {scales.dtype}")
        if global_scale is not None and amax is not None:
            raise ValueError("give either global_scale (a decode factor) or amax, not both")
        g = global_scale if global_scale is not None else amax
        if g is not None and (g.dtype != torch.float32 or g.numel() < 1):
            raise TypeError("global_scale / amax must be a float32 tensor")
        if data.dim() < 1:
            raise ValueError("data must have at least one dimension")
        self.cols = int(cols) if cols is not None else 2 * data.shape[-1]
        if self.cols > 2 * data.shape[-1] or self.cols % 16:
            raise ValueError(f"cols = {self.cols}: a multiple of 16 with at most 2 * data.shape[-1] = {2 * data.shape[-1]} values")
        rows = math.prod(data.shape[:-1])
        if swizzled:
            want = _ops.swizzled_scale_shape(rows, self.cols)
            if tuple(scales.shape) != want:
                raise ValueError(f"swizzled scales of a [{rows}, {self.cols}] matrix are {list(want)}, got {tuple(scales.shape)}")
        elif scales.dim() == data.dim() and scales.shape[:-1] == data.shape[:-1]:
            if scales.shape[-1] < self.cols // 16:
                raise ValueError(f"scales {tuple(scales.shape)} have fewer than cols / 16 = {self.cols // 16} columns")
        elif scales.dim() != 2 or scales.shape[0] < rows or scales.shape[1] < self.cols // 16:
            raise ValueError(f"data {tuple(data.shape)} and scales {tuple(scales.shape)} do not describe the same matrix")
        if g is not None and g.numel() not in (1, rows):
            raise ValueError(f"the global has {g.numel()} elements: 1 (per tensor) or {rows} (one per row)")
        if not (data.device == scales.device and (g is None or g.device == data.device)):
            raise ValueError("data, scales and the global must be on one device")
        if scale_max not in (0, 256, 448, 114688):
            raise ValueError(f"scale_max must be 0, 256, 448 or 114688, got {scale_max}")
        self.data, self.scales = data, scales
        self.global_scale = g.reshape(-1) if g is not None else None
        self.global_is_amax = amax is not None
        self.scale_max, self.swizzled, self.ue5m3 = scale_max, swizzled, ue5m3
        self.columnwise, self.block = columnwise, block

    @property
    def shape(self) -> Tuple[int, ...]:
        return (*self.data.shape[:-1], self.cols)

    def dim(self) -> int:
        return self.data.dim()

    @property
    def device(self) -> torch.device:
        return self.data.device

    @property
    def rows(self) -> int:
        return math.prod(self.data.shape[:-1])

    @property
    def per_row(self) -> bool:
        return self.global_scale is not None and self.global_scale.numel() > 1

    @property
    def amax(self) -> Optional[torch.Tensor]:
        return self.global_scale if self.global_is_amax else None

    @property
    def flags(self) -> int:
        return ((L.SCALES_SWIZZLED if self.swizzled else 0) | (L.SCALES_UE5M3 if self.ue5m3 else 0) |
                (L.GLOBAL_AMAX if self.global_is_amax else 0) | (L.GLOBAL_PER_ROW if self.per_row else 0))

    def _flat(self):
        """(data 2-D, scales 2-D, global, flags, scale_max, cols) as ``_ops`` takes them."""
        d = self.data.reshape(-1, self.data.shape[-1]) if self.data.dim() != 2 else self.data
        s = self.scales if self.scales.dim() == 2 else self.scales.reshape(-1, self.scales.shape[-1])
        return d, s, self.global_scale, self.flags, self.scale_max, self.cols

    @classmethod
    def from_float(cls, x: torch.Tensor, global_scale: Optional[torch.Tensor] = None, **recipe) -> "NVFP4Tensor":
        from .api import quantize
        return quantize(x, global_scale, **recipe)

    @classmethod
    def from_te(cls, t) -> "NVFP4Tensor":
        """Adopt, without a copy, a Transformer Engine NVFP4 tensor through TE's attribute names (``_rowwise_data``,
        ``_rowwise_scale_inv``, ``_amax_rowwise`` and the ``_columnwise_*`` ones, ``_with_gemm_swizzled_scales``,
        ``_nvfp4_e4m3_max``, ``_scale_dtype``).  A tensor holding only the columnwise half becomes the tensor of the transpose."""
        swizzled = bool(getattr(t, "_with_gemm_swizzled_scales", False))
        ue5m3 = "ue5m3" in str(getattr(t, "_scale_dtype", "")).lower()
        bound = int(getattr(t, "_nvfp4_e4m3_max", 0) or 0)
        halves = []
        for prefix, amax_name in (("_rowwise", "_amax_rowwise"), ("_columnwise", "_amax_columnwise")):
            data = getattr(t, prefix + "_data", None)
            if data is None:
                halves.append(None)
                continue
            sc = getattr(t, prefix + "_scale_inv")
            sc = sc.reshape(sc.shape[0], -1) if swizzled else sc
            a = getattr(t, amax_name, None)
            halves.append(cls(data, sc.view(torch.uint8) if ue5m3 else sc, amax=a.float() if a is not None else None, scale_max=bound,
                              swizzled=swizzled, ue5m3=ue5m3))
        row, col = halves
        if row is None and col is None:
            raise ValueError("the tensor holds neither rowwise nor columnwise NVFP4 data")
        if row is None:
            return col
        row.columnwise = col
        return row

    def dequantize(self, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        from .api import dequantize
        return dequantize(self, dtype)

    def _like(self, data, scales, swizzled, cols, block):
        g = self.global_scale
        return NVFP4Tensor(data, scales, None if self.global_is_amax else g, amax=g if self.global_is_amax else None,
                           scale_max=self.scale_max, swizzled=swizzled, ue5m3=self.ue5m3, cols=cols, block=block)

    def with_scale_layout(self, swizzled: bool) -> "NVFP4Tensor":
        """The same tensor with its block scales in the linear or the swizzled GEMM layout (both halves, if present)."""
        out = self
        if swizzled != self.swizzled:
            d, s, _, _, _, cols = self._flat()
            sc = _ops.swizzle_scales(s.view(torch.uint8), d.shape[0], cols, swizzled)
            out = self._like(self.data, sc if self.ue5m3 else sc.view(torch.float8_e4m3fn), swizzled, cols, self.block)
        if self.columnwise is not None and self.columnwise.swizzled != swizzled:
            if out is self:
                out = self._like(self.data, self.scales, self.swizzled, self.cols, self.block)
            out.columnwise = self.columnwise.with_scale_layout(swizzled)
        return out

    def transpose_2d(self) -> "NVFP4Tensor":
        """Transpose of a 16 x 16-tile tensor: exactly the columnwise quantization of the original."""
        if self.block is not None and tuple(self.block) != (16, 16):
            raise ValueError("transpose_2d needs a tensor quantized with 16 x 16 tiles")
        if self.per_row:
            raise ValueError("per-row globals do not transpose")
        d, s, _, flags, smax, cols = self._flat()
        dt, st = _ops.transpose(d, s.view(torch.uint8), flags, smax, cols)
        return self._like(dt, st if self.ue5m3 else st.view(torch.float8_e4m3fn), self.swizzled, d.shape[0], (16, 16))

    def __repr__(self):
        parts = [f"shape={self.shape}", f"device={self.device}"]
        if self.global_scale is not None:
            kind = "amax" if self.global_is_amax else "global_scale"
            parts.append(f"{kind}={'per row' if self.per_row else f'{float(self.global_scale):.6g}'}")
        for flag, text in ((self.swizzled, "swizzled scales"), (self.ue5m3, "UE5M3 scales")):
            if flag:
                parts.append(text)
        if self.scale_max:
            parts.append(f"scale_max={self.scale_max}")
        if self.block is not None:
            parts.append(f"block={self.block[0]}x{self.block[1]}")
        if self.columnwise is not None:
            parts.append("+ columnwise")
        return f"NVFP4Tensor({', '.join(parts)})"


class Int8Tensor:
    """int8 activations with one FP32 scale per 16 values of the last dimension (W4A8): ``value = data * scale``."""

    def __init__(self, data: torch.Tensor, scales: torch.Tensor, dtype: torch.dtype = torch.bfloat16):
        if data.dtype != torch.int8:
            raise TypeError(f"data must be torch.int8, got {data.dtype}")
        if scales.dtype != torch.float32:
            raise TypeError(f"scales must be torch.float32, got {scales.dtype}")
        if dtype not in (torch.bfloat16, torch.float16, torch.float32):
            raise TypeError(f"dtype must be bfloat16, float16 or float32, got {dtype}")
        if data.dim() < 1 or data.shape[-1] % 16:
            raise ValueError(f"data must be [..., cols] with cols a multiple of 16, got {tuple(data.shape)}")
        want = (*data.shape[:-1], data.shape[-1] // 16)
        if tuple(scales.shape) != want:
            raise ValueError(f"scales of a {tuple(data.shape)} tensor are {want}, got {tuple(scales.shape)}")
        if data.device != scales.device:
            raise ValueError("data and scales must be on one device")
        self.data, self.scales, self.dtype = data, scales, dtype

    @property
    def shape(self) -> Tuple[int, ...]:
        return tuple(self.data.shape)

    def dim(self) -> int:
        return self.data.dim()

    @property
    def device(self) -> torch.device:
        return self.data.device

    @classmethod
    def from_float(cls, x: torch.Tensor) -> "Int8Tensor":
        from .api import quantize_int8
        return quantize_int8(x)

    def dequantize(self, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        k = self.data.shape[-1]
        v = self.data.float().reshape(-1, k // 16, 16) * self.scales.reshape(-1, k // 16, 1)
        return v.reshape(self.data.shape).to(dtype or self.dtype)

    def __repr__(self):
        return f"Int8Tensor(shape={self.shape}, device={self.device}, dtype={self.dtype})"


class TCWeight:
    """An NVFP4 weight ``[N, K]`` with its image, built once here; serves the tensor-core GEMM and, up to 8 rows of ``x``, the
    GEMV.  ``act``: ``"exact"`` (bfloat16 activations, W4A16), ``"int8"`` or ``"nvfp4"`` (W4A8 / W4A4)."""

    def __init__(self, weight: NVFP4Tensor, act: str = "exact"):
        if not isinstance(weight, NVFP4Tensor) or weight.dim() != 2:
            raise TypeError("weight must be a 2-D NVFP4Tensor")
        if act not in ("exact", "int8", "nvfp4"):
            raise ValueError(f"act must be 'exact', 'int8' or 'nvfp4', got {act!r}")
        d, s, _, f, _, k = weight._flat()
        self.weight, self.act = weight, act
        self.image = _ops.tc_image(0 if act == "exact" else 2, d, s.view(torch.uint8), f, k)

    @property
    def shape(self) -> Tuple[int, ...]:
        return self.weight.shape

    def dim(self) -> int:
        return 2


class NVFP4Linear(torch.nn.Module):
    """``y = x @ W.T + bias`` with an NVFP4 weight ``[out_features, in_features]`` (in_features a multiple of 64)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype: torch.dtype = torch.bfloat16,
                 act: str = "auto"):
        super().__init__()
        if in_features % 64:
            raise ValueError(f"in_features ({in_features}) must be a multiple of 64")
        self.act = act
        self.in_features, self.out_features = in_features, out_features
        self.register_buffer("weight", torch.zeros(out_features, in_features // 2, dtype=torch.uint8, device=device))
        self.register_buffer("weight_scale", torch.zeros(out_features, in_features // 16, dtype=torch.float8_e4m3fn, device=device))
        self.register_buffer("weight_scale_2", torch.ones(1, dtype=torch.float32, device=device))
        self.bias = torch.nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device), requires_grad=False) if bias else None

    @classmethod
    def from_linear(cls, linear: torch.nn.Linear, global_scale: Optional[torch.Tensor] = None, act: str = "auto") -> "NVFP4Linear":
        """Quantize ``linear`` (a CUDA module) into the ModelOpt checkpoint layout: 1 x 16 blocks, linear scales, a global
        decode factor (amax / (6 * 448) unless given)."""
        w = linear.weight.detach()
        m = cls(linear.in_features, linear.out_features, linear.bias is not None, device=w.device,
                dtype=linear.bias.dtype if linear.bias is not None else w.dtype, act=act)
        if global_scale is None:
            a = w.abs().amax().float().reshape(1)
            global_scale = torch.where(a > 0, a / (6.0 * 448.0), torch.ones_like(a))
        q = NVFP4Tensor.from_float(w, global_scale)
        m.weight.copy_(q.data)
        m.weight_scale.copy_(q.scales)
        m.weight_scale_2.copy_(q.global_scale)
        if linear.bias is not None:
            m.bias.data.copy_(linear.bias.detach())
        return m

    def nvfp4_weight(self) -> NVFP4Tensor:
        return NVFP4Tensor(self.weight, self.weight_scale, self.weight_scale_2)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from .api import linear
        bias = self.bias if self.bias is None or self.bias.dtype == x.dtype else self.bias.to(x.dtype)
        return linear(x, self.nvfp4_weight(), bias, act=self.act)

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, NVFP4, act={self.act}"


def quantize_linear_(module: torch.nn.Module, *, act: str = "auto") -> torch.nn.Module:
    """Replace, in place, every ``nn.Linear`` inside ``module`` whose in_features is a multiple of 64 by an ``NVFP4Linear``."""
    for name, child in list(module.named_children()):
        if isinstance(child, torch.nn.Linear) and child.in_features % 64 == 0:
            setattr(module, name, NVFP4Linear.from_linear(child, act=act))
        else:
            quantize_linear_(child, act=act)
    return module
