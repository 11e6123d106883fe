"""CPU oracle of the NVFP4 hot path -- TEST INFRASTRUCTURE ONLY.

numpy front end of ``oracle/liboracle.so`` (built from ``oracle/oracle.cpp`` by ``make -f oracle/Makefile``).  Only the
tests, ``__graft_entry__.smoke()`` and the CPU-baseline / reference arm of ``bench.py`` may import this package; the
product package ``nvfp4effma_b200`` never does.  Every function restates arithmetic that the reference
(srose69/nvfp4effma) documents in ``include/nvfp4effma.h`` and emulates on the host in ``tests/``; the C functions cite
the lines they follow.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_HERE)

NVFP4, BF16, FP16, FP32, INT8 = 0, 1, 2, 3, 4
SWIZZLED, UE5M3, GLOBAL_AMAX, PER_ROW = 1, 2, 4, 8
NCPU = os.cpu_count() or 1


def build():
    """Compile the oracle (g++) and, where the reference sources are mounted, the reference-side checkers."""
    subprocess.run(["make", "-s", "-f", "oracle/Makefile"], cwd=_ROOT, check=True)


def _load():
    path = os.path.join(_HERE, "liboracle.so")
    if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(os.path.join(_HERE, "oracle.cpp")):
        build()
    return ctypes.CDLL(path)


_lib = _load()


class Tensor(ctypes.Structure):
    """Host mirror of ``nvfp4a_tensor`` (``orc_tensor`` in oracle.h)."""
    _fields_ = [("data", ctypes.c_void_p), ("dtype", ctypes.c_int), ("block_scale", ctypes.c_void_p),
                ("ld_scale", ctypes.c_int), ("global_scale", ctypes.c_void_p), ("flags", ctypes.c_uint),
                ("scale_max", ctypes.c_int)]


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


_c = ctypes
_lib.orc_encoder_fold.restype = _c.c_uint64
_lib.orc_encoder_fold.argtypes = [_c.c_int, _c.c_uint64, _c.c_uint64, _c.c_int]
_lib.orc_encode_array.argtypes = [_c.c_int, _c.c_void_p, _c.c_void_p, _c.c_size_t]
_lib.orc_scale_pos.restype = _c.c_size_t
_lib.orc_scale_pos.argtypes = [_c.c_int] * 5
_lib.orc_scale_bytes.restype = _c.c_size_t
_lib.orc_scale_bytes.argtypes = [_c.c_int] * 4
for _n in ("orc_e4m3_value", "orc_ue5m3_value", "orc_e2m1_value"):
    getattr(_lib, _n).restype = _c.c_float
    getattr(_lib, _n).argtypes = [_c.c_uint32]
_lib.orc_quantize.argtypes = [_c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.POINTER(Tensor), _c.c_int, _c.c_int, _c.c_int,
                              _c.c_int, _c.c_int, _c.c_void_p, _c.c_int]
_lib.orc_quantize_int8.argtypes = [_c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_void_p, _c.c_int, _c.c_void_p, _c.c_int,
                                   _c.c_void_p, _c.c_int]
_lib.orc_dequantize.argtypes = [_c.POINTER(Tensor), _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_void_p, _c.c_int, _c.c_void_p]
_lib.orc_swizzle_scales.argtypes = [_c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_int]
_lib.orc_gemm.argtypes = [_c.c_int, _c.c_int, _c.c_int, _c.c_float, _c.POINTER(Tensor), _c.c_int, _c.POINTER(Tensor), _c.c_int,
                          _c.c_float, _c.c_void_p, _c.c_int, _c.c_int, _c.c_void_p, _c.c_int, _c.c_int, _c.c_void_p, _c.c_int,
                          _c.c_int, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int]
_lib.orc_norm_scale.restype = _c.c_float
_lib.orc_norm_scale.argtypes = [_c.c_void_p, _c.c_int, _c.c_float, _c.c_float]
_lib.orc_epilogue_ex.argtypes = [_c.c_int, _c.c_int, _c.c_void_p, _c.c_float, _c.c_void_p, _c.c_int, _c.c_float, _c.c_float,
                                 _c.c_float, _c.c_void_p, _c.c_int, _c.c_int, _c.c_void_p, _c.c_int, _c.c_int,
                                 _c.c_void_p, _c.c_int, _c.c_int, _c.c_float, _c.c_float,
                                 _c.c_void_p, _c.c_int, _c.c_int, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_void_p,
                                 _c.c_int, _c.c_void_p, _c.c_int, _c.c_void_p]

ENC_E4M3, ENC_E2M1, ENC_UE5M3, ENC_BF16 = 0, 1, 2, 3


# ---- dense element types as numpy -------------------------------------------------------------------------------------
def to_f32(a, dtype):
    """Raw dense buffer (uint16 for BF16 / FP16 bit patterns, float32) -> float32 values."""
    if dtype == BF16:
        return (a.astype(np.uint32) << 16).view(np.float32)
    if dtype == FP16:
        return a.view(np.float16).astype(np.float32)
    return a.astype(np.float32, copy=False)


def from_f32(x, dtype):
    """float32 values -> raw dense buffer of ``dtype`` with one RNE rounding (the oracle's own BF16 encoder)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if dtype == BF16:
        return encode(ENC_BF16, x).astype(np.uint16)
    if dtype == FP16:
        return x.astype(np.float16).view(np.uint16)
    return x


def np_dtype(dtype):
    return np.float32 if dtype == FP32 else np.uint16


def encode(which, x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint32)
    _lib.orc_encode_array(which, _p(x), _p(out), x.size)
    return out


def encoder_fold(which, first=0, count=1 << 32, nthreads=NCPU):
    return int(_lib.orc_encoder_fold(which, first, count, nthreads))


def scale_pos(swizzled, ld, cols, r, c):
    return int(_lib.orc_scale_pos(int(bool(swizzled)), ld, cols, r, c))


def scale_bytes(swizzled, ld, rows, cols):
    return int(_lib.orc_scale_bytes(int(bool(swizzled)), ld, rows, cols))


def e4m3_value(code):
    return float(_lib.orc_e4m3_value(code))


def ue5m3_value(code):
    return float(_lib.orc_ue5m3_value(code))


def e2m1_value(nib):
    return float(_lib.orc_e2m1_value(nib))


# ---- NVFP4 host tensors ------------------------------------------------------------------------------------------------
class Fp4:
    """A host NVFP4 matrix [rows][cols]: packed nibbles (ld values per row), block scales (linear with ``ld_scale`` bytes per
    row, or swizzled), global (one float or one per row; decode factor or amax)."""

    def __init__(self, rows, cols, ld=None, ld_scale=None, flags=0, scale_max=0, glob=None, fill=0):
        self.rows, self.cols = rows, cols
        self.ld = ld if ld is not None else cols
        self.flags, self.scale_max = flags, scale_max
        self.swz = bool(flags & SWIZZLED)
        self.ld_scale = 0 if self.swz else (ld_scale if ld_scale is not None else cols // 16)
        self.data = np.full(max(rows, 1) * self.ld // 2, fill, dtype=np.uint8)
        self.scales = np.full(max(scale_bytes(self.swz, self.ld_scale, rows, cols), 1), fill, dtype=np.uint8)
        n = rows if flags & PER_ROW else 1
        self.glob = None if glob is None else np.array(np.broadcast_to(np.asarray(glob, np.float32), (max(n, 1),)), dtype=np.float32, copy=True)

    def tensor(self):
        return Tensor(_p(self.data), NVFP4, _p(self.scales), self.ld_scale, _p(self.glob), self.flags, self.scale_max)

    def M(self):
        return float(self.scale_max) if self.scale_max else (114688.0 if self.flags & UE5M3 else 448.0)


class Q8:
    """A host INT8 activation matrix: int8 [rows][ld] and one float32 scale per 16 values ([rows][ld_scale])."""

    def __init__(self, rows, cols, ld=None, ld_scale=None, glob=None):
        self.rows, self.cols = rows, cols
        self.ld = ld if ld is not None else cols
        self.ld_scale = ld_scale if ld_scale is not None else cols // 16
        self.data = np.zeros(max(rows, 1) * self.ld, dtype=np.int8)
        self.scales = np.zeros(max(rows, 1) * self.ld_scale, dtype=np.float32)
        self.glob = None if glob is None else np.asarray([glob], np.float32)

    def tensor(self):
        return Tensor(_p(self.data), INT8, _p(self.scales), self.ld_scale, _p(self.glob), 0, 0)


class Dense:
    """A host dense matrix [rows][ld] of BF16 / FP16 (uint16 bit patterns) or FP32."""

    def __init__(self, dtype, raw, ld):
        self.dtype, self.raw, self.ld = dtype, np.ascontiguousarray(raw), ld

    def tensor(self):
        return Tensor(_p(self.raw), self.dtype, None, 0, None, 0, 0)


# ---- operations ----------------------------------------------------------------------------------------------------------
def quantize(x, dst, cols=None, transposed=False, tile=1, fos=0, compute_amax=False, nthreads=NCPU):
    """Quantize float32 ``x`` (2-D [rows][ldx], the first ``cols`` columns of each row) into the ``Fp4`` ``dst``: rowwise
    [rows][cols], or with ``transposed`` the quantization of x^T, [cols][roundup(rows, 16)].  Returns max |x|."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, ldx = x.shape
    cols = ldx if cols is None else cols
    amax = np.zeros(1, np.float32)
    t = dst.tensor()
    rc = _lib.orc_quantize(_p(x), ldx, rows, cols, ctypes.byref(t), dst.ld, int(transposed), tile, fos, int(compute_amax),
                           _p(amax), nthreads)
    assert rc == 0, "orc_quantize rejected its arguments"
    return float(amax[0])


def quantize_int8(x, dst, ldx=None, nthreads=NCPU):
    x = np.ascontiguousarray(x, dtype=np.float32)
    if ldx is None:
        ldx = x.shape[1]
    amax = np.zeros(1, np.float32)
    rc = _lib.orc_quantize_int8(_p(x), ldx, dst.rows, dst.cols, _p(dst.data), dst.ld, _p(dst.scales), dst.ld_scale, _p(amax),
                                nthreads)
    assert rc == 0
    return float(amax[0])


def dequantize(src, out_dtype=FP32):
    y = np.zeros((src.rows, src.cols), np.float32)
    amax = np.zeros(1, np.float32)
    t = src.tensor()
    rc = _lib.orc_dequantize(ctypes.byref(t), src.ld, src.rows, src.cols, out_dtype, _p(y), src.cols, _p(amax))
    assert rc == 0
    return y, float(amax[0])


def swizzle_scales(src, ld_linear, rows, cols, to_swizzled, dst=None):
    src = np.ascontiguousarray(src, dtype=np.uint8)
    if dst is None:
        dst = np.zeros(scale_bytes(True, 0, rows, cols) if to_swizzled else rows * ld_linear, np.uint8)
    rc = _lib.orc_swizzle_scales(_p(src), _p(dst), ld_linear, rows, cols, int(to_swizzled))
    assert rc == 0
    return dst


def gemm(m, n, k, A, B, D_dtype=BF16, alpha=1.0, beta=0.0, C=None, C_dtype=None, ldc=None, ldd=None, bias=None,
         bias_dtype=FP32, lda=None, ldb=None, order=0, D_init=None, want_ref=False, want_acc=False, nthreads=NCPU):
    """The exact GEMM / GEMV definition on the host.  A: ``Fp4``; B: ``Fp4`` | ``Q8`` | ``Dense``.  Returns a dict with the raw
    D buffer [n][ldd] (``D``), ``amax`` and optionally ``acc``, ``ref64``, ``bound`` ([n][m])."""
    ldd = ldd if ldd is not None else m
    ldc = ldc if ldc is not None else ldd
    lda = lda if lda is not None else A.ld
    ldb = ldb if ldb is not None else B.ld
    D = np.zeros(max(n * ldd, 1), np_dtype(D_dtype)) if D_init is None else np.array(D_init, copy=True)
    amax = np.zeros(1, np.float32)
    acc = np.zeros((n, m), np.float32) if want_acc else None
    ref = np.zeros((n, m), np.float64) if want_ref else None
    bnd = np.zeros((n, m), np.float64) if want_ref else None
    ta, tb = A.tensor(), B.tensor()
    rc = _lib.orc_gemm(m, n, k, alpha, ctypes.byref(ta), lda, ctypes.byref(tb), ldb, beta, _p(C),
                       C_dtype if C_dtype is not None else D_dtype, ldc, _p(D), D_dtype, ldd, _p(bias), bias_dtype, order,
                       _p(amax), _p(acc), _p(ref), _p(bnd), nthreads)
    assert rc == 0, "orc_gemm rejected its arguments"
    return {"D": D, "amax": float(amax[0]), "acc": acc, "ref64": ref, "bound": bnd}


def norm_scale(parts, inv_n, eps):
    parts = np.ascontiguousarray(parts, np.float32)
    return float(_lib.orc_norm_scale(_p(parts), parts.size, inv_n, eps))


def epilogue_ex(m, n, acc, alpha=1.0, ga=None, per_row_a=False, gb=1.0, gf=1.0, beta=0.0, C=None, C_dtype=FP32, ldc=0,
                bias=None, bias_dtype=FP32, mask=0, norm_parts=None, norm_nparts=0, norm_ld=0, norm_inv_n=1.0, norm_eps=0.0,
                D_dtype=BF16, ldd=None, w2=None, w2_dtype=FP32, d2_dtype=BF16, ldd2=None, ld_sq=None):
    """The extended epilogue on the host, applied to accumulators ``acc`` [n][m]."""
    glu, out2 = bool(mask & 2), bool(mask & 4)
    mo = m // 2 if glu else m
    ldd = ldd if ldd is not None else mo
    acc = np.ascontiguousarray(acc, np.float32)
    D = np.zeros(n * ldd, np_dtype(D_dtype))
    sw = np.zeros((n, m // 2), np.float64) if glu else None
    ldd2 = ldd2 if ldd2 is not None else m
    ld_sq = ld_sq if ld_sq is not None else m // 16
    d2 = np.zeros(n * ldd2, np_dtype(d2_dtype)) if out2 else None
    sq = np.zeros(n * ld_sq, np.float32) if out2 else None
    v = np.zeros((n, m), np.float32)
    rc = _lib.orc_epilogue_ex(m, n, _p(acc), alpha, _p(ga), int(per_row_a), gb, gf, beta, _p(C), C_dtype, ldc, _p(bias),
                              bias_dtype, mask, _p(norm_parts), norm_nparts, norm_ld, norm_inv_n, norm_eps, _p(D), D_dtype, ldd,
                              _p(sw), _p(d2), d2_dtype, ldd2, _p(w2), w2_dtype, _p(sq), ld_sq, _p(v))
    assert rc == 0
    return {"D": D, "swiglu64": sw, "d2": d2, "sq": sq, "v": v}
