"""Containers of the Python surface: ``NVFP4Tensor``, ``Int8Tensor``, ``TCWeight`` and the ``NVFP4Linear`` module.

The names, constructor arguments, attributes and checkpoint buffer names (``weight`` / ``weight_scale`` /
``weight_scale_2``) are those of the reference's Python package (binds/python/nvfp4effma/tensor.py there), so code written
against it keeps working; the implementation is this library's own.  All three containers are validated by one set of
helpers (``_expect_dtype``, ``_same_device``, ``_block_count``) and hand their buffers to the operator layer as an
``Fp4Operand`` tuple.  Inference only; no autograd.
"""
import math
from typing import NamedTuple, Optional, Tuple

import torch

from . import _abi as A
from . import _lib as L
from ._ops import ops

_SCALE_BOUNDS = (0, 256, 448, 114688)
_ACTS = ("exact", "int8", "nvfp4")
_FLOATS = (torch.bfloat16, torch.float16, torch.float32)


class Fp4Operand(NamedTuple):
    """What the operators take for one NVFP4 matrix: 2-D nibbles, 2-D scale codes (uint8), the global, flag bits, bound, columns."""
    data: torch.Tensor
    scales: torch.Tensor
    glob: Optional[torch.Tensor]
    flags: int
    scale_max: int
    cols: int

    @property
    def rows(self) -> int:
        return self.data.shape[0]


# ---- validation shared by the containers ------------------------------------------------------------------------------------------
def _expect_dtype(what: str, t: torch.Tensor, *allowed: torch.dtype):
    if t.dtype not in allowed:
        names = " or ".join(str(a).replace("torch.", "") for a in allowed)
        raise TypeError(f"{what} holds {t.dtype}; it has to be {names}")


def _same_device(*named: Tuple[str, Optional[torch.Tensor]]):
    present = [(n, t) for n, t in named if t is not None]
    first_name, first = present[0]
    for name, t in present[1:]:
        if t.device != first.device:
            raise ValueError(f"{name} is on {t.device} but {first_name} is on {first.device}")


def _block_count(what: str, values: int) -> int:
    if values % 16:
        raise ValueError(f"{what}: {values} values do not divide into blocks of 16")
    return values // 16


def _leading_rows(t: torch.Tensor) -> int:
    return math.prod(t.shape[:-1])


class NVFP4Tensor:
    """An NVFP4 tensor of logical shape ``[..., cols]``: element = e2m1 nibble x block scale x global.

    ``data``: uint8, two values per byte (the even column in the low nibble).  ``scales``: one code per 16 values of a row --
    ``float8_e4m3fn`` (uint8 is accepted and re-viewed) or, with ``ue5m3``, uint8 -- either laid out like ``data``
    (``[..., >= cols / 16]``, or any 2-D buffer with at least as many rows and columns) or, with ``swizzled``, the padded
    128 x 4-tile buffer of the whole matrix.  The global is a float32 decode factor (``global_scale``) or an amax (``amax``,
    decode factor amax / (6 x scale_max)), one value or one per row.
    """

    def __init__(self, data: torch.Tensor, scales: torch.Tensor, global_scale: Optional[torch.Tensor] = None, *,
                 amax: Optional[torch.Tensor] = None, scale_max: int = 0, swizzled: bool = False, ue5m3: bool = False,
                 cols: Optional[int] = None, columnwise: Optional["NVFP4Tensor"] = None, block: Optional[Tuple[int, int]] = None):
        _expect_dtype("NVFP4 data", data, torch.uint8)
        if ue5m3:
            _expect_dtype("UE5M3 block scales", scales, torch.uint8)
        else:
            _expect_dtype("E4M3 block scales", scales, torch.float8_e4m3fn, torch.uint8)
            if scales.dtype == torch.uint8:
                scales = scales.view(torch.float8_e4m3fn)
        if amax is not None and global_scale is not None:
            raise ValueError("a tensor has ONE global: pass the decode factor as global_scale or the amax as amax")
        glob = amax if amax is not None else global_scale
        if glob is not None:
            _expect_dtype("the global", glob, torch.float32)
        if data.dim() == 0:
            raise ValueError("NVFP4 data needs a last dimension to hold the packed values")
        held = 2 * data.shape[-1]
        self.cols = held if cols is None else int(cols)
        nblocks = _block_count("cols", self.cols)
        if self.cols > held:
            raise ValueError(f"cols = {self.cols} exceeds the {held} values the last dimension of data holds")
        rows = _leading_rows(data)
        self._check_scale_shape(data, scales, rows, nblocks, swizzled)
        if glob is not None and glob.numel() != 1 and glob.numel() != rows:
            raise ValueError(f"{glob.numel()} global values for {rows} rows: there is one per tensor or one per row")
        _same_device(("data", data), ("scales", scales), ("the global", glob))
        if scale_max not in _SCALE_BOUNDS:
            raise ValueError(f"scale_max = {scale_max} is not one of {_SCALE_BOUNDS}")
        self.data, self.scales = data, scales
        self.global_scale = None if glob is None else glob.reshape(-1)
        self.global_is_amax = amax is not None
        self.scale_max, self.swizzled, self.ue5m3 = scale_max, bool(swizzled), bool(ue5m3)
        self.columnwise, self.block = columnwise, block

    def _check_scale_shape(self, data, scales, rows, nblocks, swizzled):
        got = tuple(scales.shape)
        if swizzled:
            if got != A.padded_scale_shape(rows, self.cols):
                raise ValueError(f"swizzled scales of {rows} x {self.cols} values fill a {A.padded_scale_shape(rows, self.cols)} buffer, got {got}")
            return
        alongside = scales.dim() == data.dim() and got[:-1] == tuple(data.shape[:-1])
        plain_2d = scales.dim() == 2 and got[0] >= rows
        if not (alongside or plain_2d) or got[-1] < nblocks:
            raise ValueError(f"scales of shape {got} cannot hold {rows} x {nblocks} block scales for data of shape {tuple(data.shape)}")

    # ---- what the tensor is ------------------------------------------------------------------------------------------------------
    @property
    def shape(self) -> Tuple[int, ...]:
        return tuple(self.data.shape[:-1]) + (self.cols,)

    def dim(self) -> int:
        return self.data.dim()

    @property
    def device(self) -> torch.device:
        return self.data.device

    @property
    def rows(self) -> int:
        return _leading_rows(self.data)

    @property
    def per_row(self) -> bool:
        return self.global_scale is not None and self.global_scale.numel() > 1

    @property
    def amax(self) -> Optional[torch.Tensor]:
        return self.global_scale if self.global_is_amax else None

    @property
    def flags(self) -> int:
        bits = ((self.swizzled, L.SCALES_SWIZZLED), (self.ue5m3, L.SCALES_UE5M3), (self.global_is_amax, L.GLOBAL_AMAX), (self.per_row, L.GLOBAL_PER_ROW))
        return sum(bit for on, bit in bits if on)

    def _operand(self) -> Fp4Operand:
        data = self.data if self.data.dim() == 2 else self.data.reshape(self.rows, self.data.shape[-1])
        scales = self.scales if self.scales.dim() == 2 else self.scales.reshape(-1, self.scales.shape[-1])
        return Fp4Operand(data, scales.view(torch.uint8), self.global_scale, self.flags, self.scale_max, self.cols)

    def _rebuilt(self, data, scale_codes, *, swizzled, cols, block) -> "NVFP4Tensor":
        """A tensor with this one's global, bound and scale type over other buffers."""
        kind = {"amax": self.global_scale} if self.global_is_amax else {"global_scale": self.global_scale}
        return NVFP4Tensor(data, scale_codes, scale_max=self.scale_max, swizzled=swizzled, ue5m3=self.ue5m3, cols=cols, block=block, **kind)

    # ---- construction ------------------------------------------------------------------------------------------------------------
    @classmethod
    def from_float(cls, x: torch.Tensor, global_scale: Optional[torch.Tensor] = None, **recipe) -> "NVFP4Tensor":
        from .api import quantize
        return quantize(x, global_scale, **recipe)

    @classmethod
    def from_te(cls, t) -> "NVFP4Tensor":
        """Wraps a Transformer Engine NVFP4 tensor without copying, reading TE's private attributes: ``_rowwise_data`` /
        ``_rowwise_scale_inv`` / ``_amax_rowwise``, their ``_columnwise_*`` twins, ``_with_gemm_swizzled_scales``,
        ``_nvfp4_e4m3_max`` and ``_scale_dtype``.  With only the column-wise half present the result is the tensor of the transpose."""
        swizzled = bool(getattr(t, "_with_gemm_swizzled_scales", False))
        ue5m3 = "ue5m3" in str(getattr(t, "_scale_dtype", "")).lower()
        bound = int(getattr(t, "_nvfp4_e4m3_max", 0) or 0)

        def half(which):
            data = getattr(t, f"_{which}_data", None)
            if data is None:
                return None
            codes = getattr(t, f"_{which}_scale_inv")
            if swizzled:
                codes = codes.reshape(codes.shape[0], -1)
            stat = getattr(t, f"_amax_{which}", None)
            return cls(data, codes.view(torch.uint8) if ue5m3 else codes, amax=None if stat is None else stat.float(), scale_max=bound,
                       swizzled=swizzled, ue5m3=ue5m3)

        rowwise, colwise = half("rowwise"), half("columnwise")
        if rowwise is None:
            if colwise is None:
                raise ValueError("this Transformer Engine tensor carries no NVFP4 data in either direction")
            return colwise
        rowwise.columnwise = colwise
        return rowwise

    # ---- operations --------------------------------------------------------------------------------------------------------------
    def dequantize(self, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        from .api import dequantize
        return dequantize(self, dtype)

    def with_scale_layout(self, swizzled: bool) -> "NVFP4Tensor":
        """This tensor with its block scales in the linear (False) or the GEMM-swizzled (True) layout; a column-wise half
        follows.  Returns ``self`` when nothing has to change."""
        swizzled = bool(swizzled)
        mine_ok = self.swizzled == swizzled
        col_ok = self.columnwise is None or self.columnwise.swizzled == swizzled
        if mine_ok and col_ok:
            return self
        if mine_ok:
            result = self._rebuilt(self.data, self.scales, swizzled=swizzled, cols=self.cols, block=self.block)
        else:
            op = self._operand()
            codes = ops.swizzle_scales(op.scales, op.rows, op.cols, swizzled)
            result = self._rebuilt(self.data, codes, swizzled=swizzled, cols=self.cols, block=self.block)
        if self.columnwise is not None:
            result.columnwise = self.columnwise.with_scale_layout(swizzled)
        return result

    def transpose_2d(self) -> "NVFP4Tensor":
        """The transpose of a tensor quantized in 16 x 16 tiles (a tile's scale serves both directions), bit-identical to
        the column-wise quantization of the original."""
        if self.block is not None and tuple(self.block) != (16, 16):
            raise ValueError(f"only 16 x 16-tile tensors transpose exactly; this one has {self.block[0]} x {self.block[1]} blocks")
        if self.per_row:
            raise ValueError("a tensor with one global per row has no transpose in this format")
        op = self._operand()
        data_t, codes_t = ops.transpose(op.data, op.scales, op.flags, op.scale_max, op.cols)
        return self._rebuilt(data_t, codes_t, swizzled=self.swizzled, cols=op.rows, block=(16, 16))

    def __repr__(self):
        bits = [f"shape={self.shape}", f"device={self.device}"]
        if self.global_scale is not None:
            name = "amax" if self.global_is_amax else "global_scale"
            bits.append(f"{name}=<{self.global_scale.numel()} per-row values>" if self.per_row else f"{name}={self.global_scale.item():.6g}")
        bits += [label for on, label in ((self.swizzled, "scales=swizzled"), (self.ue5m3, "scales=ue5m3")) if on]
        if self.scale_max:
            bits.append(f"scale_max={self.scale_max}")
        if self.block is not None:
            bits.append("block=%dx%d" % tuple(self.block))
        if self.columnwise is not None:
            bits.append("columnwise=yes")
        return "NVFP4Tensor(" + ", ".join(bits) + ")"


class Int8Tensor:
    """INT8 activations for W4A8: ``data`` int8 ``[..., cols]`` and one float32 ``scales`` value per 16 values
    (``[..., cols / 16]``); ``dtype`` is the dense type the activations came from (the default result type of ``linear``)."""

    def __init__(self, data: torch.Tensor, scales: torch.Tensor, dtype: torch.dtype = torch.bfloat16):
        _expect_dtype("INT8 data", data, torch.int8)
        _expect_dtype("INT8 block scales", scales, torch.float32)
        if dtype not in _FLOATS:
            raise TypeError(f"dtype = {dtype}: the source type is bfloat16, float16 or float32")
        if data.dim() == 0:
            raise ValueError("INT8 data needs a last dimension")
        nblocks = _block_count("INT8 data", data.shape[-1])
        if tuple(scales.shape) != tuple(data.shape[:-1]) + (nblocks,):
            raise ValueError(f"data of shape {tuple(data.shape)} takes scales of shape {tuple(data.shape[:-1]) + (nblocks,)}, not {tuple(scales.shape)}")
        _same_device(("data", data), ("scales", scales))
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
        """data x scale, one float32 product per element, rounded to ``dtype`` (default: the source type)."""
        per_value = self.scales.unsqueeze(-1).expand(*self.scales.shape, 16).reshape(self.data.shape)
        return (self.data.to(torch.float32) * per_value).to(self.dtype if dtype is None else dtype)

    def __repr__(self):
        return f"Int8Tensor(shape={self.shape}, from={str(self.dtype).replace('torch.', '')}, device={self.device})"


class TCWeight:
    """A 2-D NVFP4 weight ``[N, K]`` together with its image (``nvfp4a_tc_image``), which is built here, once.  ``linear``
    runs the GEMV on the image up to 8 rows of ``x`` and the image GEMM beyond.  ``act`` names the activations the image
    is meant for: "exact" = bfloat16 as they are (W4A16), "int8" (W4A8), "nvfp4" (W4A4)."""

    def __init__(self, weight: NVFP4Tensor, act: str = "exact"):
        if not isinstance(weight, NVFP4Tensor) or weight.dim() != 2:
            raise TypeError("TCWeight wraps a 2-D NVFP4Tensor [out_features, in_features]")
        if act not in _ACTS:
            raise ValueError(f"act = {act!r}; choose from {_ACTS}")
        op = weight._operand()
        self.weight, self.act = weight, act
        self.image = ops.tc_image(L.TC_A16 if act == "exact" else L.TC_A8, op.data, op.scales, op.flags, op.cols)

    @property
    def shape(self) -> Tuple[int, ...]:
        return self.weight.shape

    def dim(self) -> int:
        return 2


class NVFP4Linear(torch.nn.Module):
    """``x @ W.T + bias`` with ``W`` [out_features, in_features] held in NVFP4 (in_features a multiple of 64).  The buffers
    carry the names of ModelOpt NVFP4 checkpoints: ``weight`` (nibbles), ``weight_scale`` (E4M3 block scales),
    ``weight_scale_2`` (the global decode factor)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype: torch.dtype = torch.bfloat16,
                 act: str = "auto"):
        super().__init__()
        if in_features % 64:
            raise ValueError(f"in_features = {in_features}: the GEMM kernels need a multiple of 64")
        self.in_features, self.out_features, self.act = in_features, out_features, act
        new = dict(device=device)
        self.register_buffer("weight", torch.zeros((out_features, in_features // 2), dtype=torch.uint8, **new))
        self.register_buffer("weight_scale", torch.zeros((out_features, in_features // 16), dtype=torch.float8_e4m3fn, **new))
        self.register_buffer("weight_scale_2", torch.ones(1, dtype=torch.float32, **new))
        self.bias = torch.nn.Parameter(torch.zeros(out_features, dtype=dtype, **new), requires_grad=False) if bias else None

    @classmethod
    def from_linear(cls, linear: torch.nn.Linear, global_scale: Optional[torch.Tensor] = None, act: str = "auto") -> "NVFP4Linear":
        """The NVFP4 version of a CUDA ``nn.Linear``: 1 x 16 blocks, linear E4M3 scales, and as global the decode factor
        ``max |W| / (6 x 448)`` (1 for an all-zero weight) unless one is given."""
        source = linear.weight.detach()
        has_bias = linear.bias is not None
        layer = cls(linear.in_features, linear.out_features, has_bias, device=source.device, dtype=linear.bias.dtype if has_bias else source.dtype,
                    act=act)
        if global_scale is None:
            peak = source.abs().max().to(torch.float32).reshape(1)
            global_scale = torch.where(peak > 0, peak / (6.0 * 448.0), torch.ones_like(peak))
        packed = NVFP4Tensor.from_float(source, global_scale)
        with torch.no_grad():
            layer.weight.copy_(packed.data)
            layer.weight_scale.copy_(packed.scales)
            layer.weight_scale_2.copy_(packed.global_scale)
            if has_bias:
                layer.bias.copy_(linear.bias.detach())
        return layer

    def nvfp4_weight(self) -> NVFP4Tensor:
        return NVFP4Tensor(self.weight, self.weight_scale, self.weight_scale_2)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from .api import linear
        bias = self.bias
        if bias is not None and bias.dtype != x.dtype:
            bias = bias.to(x.dtype)
        return linear(x, self.nvfp4_weight(), bias, act=self.act)

    def extra_repr(self):
        return f"{self.in_features} -> {self.out_features}, bias={self.bias is not None}, weight=NVFP4, act={self.act}"


def quantize_linear_(module: torch.nn.Module, *, act: str = "auto") -> torch.nn.Module:
    """Walks ``module`` and swaps, in place, each ``nn.Linear`` whose in_features is a multiple of 64 for an ``NVFP4Linear``
    built from it; other layers (and linears of other widths) stay as they are.  Returns ``module``."""
    for name, child in module.named_children():
        convertible = isinstance(child, torch.nn.Linear) and child.in_features % 64 == 0
        if convertible:
            module.add_module(name, NVFP4Linear.from_linear(child, act=act))
        else:
            quantize_linear_(child, act=act)
    return module
