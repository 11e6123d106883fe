"""ctypes binding of ``libnvfp4effma.so``: the structs and prototypes of ``include/nvfp4effma.h`` (which mirrors the
reference's ``include/nvfp4effma.h``) and of ``include/nvfp4effma_b200.h``.

There is no fallback: if the shared library is missing or does not load, importing this module raises.  Status codes
map to exceptions the way the reference's torch extension maps them (binds/python/csrc/nvfp4effma_torch.cpp:54-60):
``NOT_SUPPORTED`` -> ``NotImplementedError``, ``INVALID_VALUE`` -> ``ValueError``, anything else -> ``RuntimeError``.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnvfp4effma.so")

NVFP4, BF16, FP16, FP32, INT8 = 0, 1, 2, 3, 4
OK, INVALID_VALUE, NOT_SUPPORTED, CUDA_ERROR = 0, 1, 2, 3
SCALES_SWIZZLED, SCALES_UE5M3, GLOBAL_AMAX, GLOBAL_PER_ROW = 1, 2, 4, 8
TC_A16, TC_B, TC_A8 = 0, 1, 2
FOS_OFF, FOS_MAE, FOS_MSE = 0, 1, 2


class Tensor(C.Structure):
    """``nvfp4a_tensor``"""
    _fields_ = [("data", C.c_void_p), ("dtype", C.c_int), ("block_scale", C.c_void_p), ("ld_scale", C.c_int),
                ("global_scale", C.c_void_p), ("amax", C.c_void_p), ("flags", C.c_uint), ("scale_max", C.c_int)]


class DualTensor(C.Structure):
    """``nvfp4a_dual_tensor``"""
    _fields_ = [("row", Tensor), ("col", Tensor), ("ld_row", C.c_int), ("ld_col", C.c_int)]


class QuantConfig(C.Structure):
    """``nvfp4a_quant_config``"""
    _fields_ = [("tile_rows", C.c_int), ("four_over_six", C.c_int), ("compute_amax", C.c_int)]


class Epilogue(C.Structure):
    """``nvfp4a_epilogue``"""
    _fields_ = [("norm_parts", C.c_void_p), ("norm_nparts", C.c_int), ("norm_ld", C.c_int), ("norm_inv_n", C.c_float),
                ("norm_eps", C.c_float), ("swiglu", C.c_int), ("d2", C.c_void_p), ("d2_dtype", C.c_int), ("ldd2", C.c_int),
                ("w2", C.c_void_p), ("w2_dtype", C.c_int), ("sq", C.c_void_p), ("ld_sq", C.c_int)]


if not os.path.exists(LIB_PATH):
    raise ImportError(f"{LIB_PATH} is missing: build it with `python -m nvfp4effma_b200.build` (nvcc, sm_100a). "
                      "There is no CPU or PyTorch fallback.")
lib = C.CDLL(LIB_PATH)

_T, _E, _i, _f, _v, _s = C.POINTER(Tensor), C.POINTER(Epilogue), C.c_int, C.c_float, C.c_void_p, C.c_void_p
_GEMM = [_i, _i, _i, _f, _T, _i, _T, _i, _f, _T, _i, _T, _i, _T]
_PROTOS = {
    "nvfp4a_gemm": (_i, _GEMM + [_s]),
    "nvfp4a_gemm_ex": (_i, _GEMM + [_E, _s]),
    "nvfp4a_gemm_dual": (_i, [_i, _i, _i, _f, C.POINTER(DualTensor), _i, C.POINTER(DualTensor), _i, _f, _T, _i, _T, _i, _T, _s]),
    "nvfp4a_gemm_grouped": (_i, [_i, _i, _i, _i, _f, _T, _i, _T, _i, _f, _T, _i, _T, _i, _T, _v, _s]),
    "nvfp4a_quantize": (_i, [_T, _i, _T, _i, _i, _i, _s]),
    "nvfp4a_quantize_ex": (_i, [_T, _i, _i, _i, _T, _i, _T, _i, C.POINTER(QuantConfig), _s]),
    "nvfp4a_dequantize": (_i, [_T, _i, _T, _i, _i, _i, _s]),
    "nvfp4a_swizzle_scales": (_i, [_v, _v, _i, _i, _i, _i, _s]),
    "nvfp4a_transpose": (_i, [_T, _i, _T, _i, _i, _i, _s]),
    "nvfp4a_tc_image_bytes": (C.c_size_t, [_i, _i, _i, _i]),
    "nvfp4a_tc_image": (_i, [_i, _T, _i, _i, _i, _v, _s]),
    "nvfp4a_tc_image_convert": (_i, [_i, _i, _v, _i, _i, _v, _s]),
    "nvfp4a_tc_image_to_raw": (_i, [_i, _v, _i, _i, _T, _i, _s]),
    "nvfp4a_tc_workspace_bytes": (C.c_size_t, []),
    "nvfp4a_gemm_tc": (_i, [_i, _i, _i, _f, _T, _T, _f, _T, _i, _T, _i, _T, _v, _s]),
    "nvfp4a_gemv_tc": (_i, [_i, _i, _i, _f, _T, _T, _i, _f, _T, _i, _T, _i, _T, _s]),
    "nvfp4a_gemv_tc_ex": (_i, [_i, _i, _i, _f, _T, _T, _i, _f, _T, _i, _T, _i, _T, _E, _s]),
    "nvfp4a_gemm_tc_ex": (_i, [_i, _i, _i, _f, _T, _T, _f, _T, _i, _T, _i, _T, _E, _v, _s]),
    "nvfp4a_status_string": (C.c_char_p, [_i]),
    "nvfp4a_last_error": (C.c_char_p, []),
    "nvfp4a_b200_codec_selftest": (_i, [C.c_ulonglong, C.c_ulonglong, _v, _s]),
    "nvfp4a_b200_set_route": (_i, [_i]),
    "nvfp4a_b200_kernel_status": (_i, [C.POINTER(C.c_uint), _i]),
    "nvfp4a_b200_set_tile_n": (_i, [_i]),
    "nvfp4a_b200_set_pair": (_i, [_i]),
    "nvfp4a_b200_set_swap": (_i, [_i]),
    "nvfp4a_b200_set_gemv_splits": (_i, [_i]),
    "nvfp4a_b200_last_route": (_i, []),
    "nvfp4a_b200_gemv_tc_tp": (_i, [_i, _i, _i, _f, _T, _T, _i, _T, _i, _T, _E, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), _i, _i, _s]),
    "nvfp4a_b200_gemv_tc_tp_deferred": (_i, [_i, _i, _i, _f, _T, _T, _i, _T, _i, _T, _E, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), _i, _i, _i, _s]),
    "nvfp4a_b200_tp_gather_post": (_i, [C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), _i, _i, _i, C.c_longlong, C.c_longlong, C.c_longlong, _s]),
    "nvfp4a_b200_tp_wait": (_i, [C.POINTER(C.c_void_p), _i, _i, _s]),
    "nvfp4a_b200_gemm_tc_tp": (_i, [_i, _i, _i, _f, _T, _T, _T, _i, _T, _E, _v, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), _i, _i, _s]),
    "nvfp4a_b200_tp_gather": (_i, [C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), _i, _i, _i, C.c_longlong, C.c_longlong, C.c_longlong, _s]),
    "nvfp4a_b200_gemm_ex_static": (_i, _GEMM + [_E, _s]),
    "nvfp4a_b200_static_scratch_tokens": (_i, []),
    "nvfp4a_b200_mma_ceiling": (_i, [_i, _i, _i, _i, _v, _s]),
    "nvfp4a_b200_last_launch": (C.c_uint, []),
    "nvfp4a_b200_set_quant_fused": (_i, [_i]),
    "nvfp4a_b200_set_wait_limit": (_i, [C.c_longlong]),
    "nvfp4a_b200_set_pdl": (_i, [_i]),
    "nvfp4a_b200_trim_scratch": (_i, []),
}
EXPORTS = tuple(_PROTOS)

for _name, (_res, _args) in _PROTOS.items():
    _fn = getattr(lib, _name)  # AttributeError here = the library does not export a declared symbol
    _fn.restype, _fn.argtypes = _res, _args


def last_error():
    return lib.nvfp4a_last_error().decode()


def check(status, what=""):
    """Raise the exception the reference binding raises for a failed status."""
    if status == OK:
        return
    msg = last_error() or lib.nvfp4a_status_string(status).decode()
    if status == NOT_SUPPORTED:
        raise NotImplementedError(msg)
    if status == INVALID_VALUE:
        raise ValueError(msg)
    raise RuntimeError(msg)
