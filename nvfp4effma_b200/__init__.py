"""nvfp4effma_b200 -- NVFP4 linear layers, GEMM / GEMV and quantization for NVIDIA B200 (sm_100a) behind the NVFP4EffMA API.

The functions and classes here keep the surface of the reference's Python package (binds/python/nvfp4effma/__init__.py
there): ``quantize``, ``quantize_int8``, ``dequantize``, ``linear``, ``NVFP4Tensor``, ``Int8Tensor``, ``TCWeight``,
``NVFP4Linear``, ``quantize_linear_``.  They call the C-ABI shared library ``libnvfp4effma.so`` through ctypes; there is no
fallback -- importing the package without the built library raises.  Errors: ``TypeError`` (dtype), ``ValueError``
(device, shape, K % 64), ``NotImplementedError`` (a GPU that is not sm_100, an unsupported combination), ``RuntimeError``.
"""
__version__ = "0.7.0"

_API = ("quantize", "quantize_int8", "dequantize", "linear", "grouped_linear", "NVFP4Tensor", "Int8Tensor", "NVFP4Linear", "TCWeight",
        "quantize_linear_", "get_include", "AUTO_EXACT_MAX_ROWS")
__all__ = [*_API, "__version__"]


def __getattr__(name):
    # The API loads the shared library; ``python -m nvfp4effma_b200.build`` must be importable without it.
    if name in _API:
        from . import api
        return getattr(api, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
