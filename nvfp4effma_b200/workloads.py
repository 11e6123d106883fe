"""Seeded synthetic operands for the benchmark configurations, built on the GPU through the library's own C ABI
(quantization included), plus thin call helpers.  Shapes and distributions are those of the benchmark definition:

* GEMV  W4A16: weight 8192 x 8192 BF16 ~ N(0, 0.02^2) quantized to NVFP4 (1 x 16 E4M3 linear scales, FP32 decode factor
  amax / (6 * 448)), x BF16 ~ N(0, 1), y BF16, alpha = 1, beta = 0;
* quantize: 8192 x 8192 BF16 ~ N(0, 1) with 1 % of the entries x 50, swizzled E4M3 scales, amax computed;
* GEMM  W4A4: M = N = K = 4096, both operands BF16 ~ N(0, 1) quantized like the GEMV weight, D BF16 column major.

torch supplies device memory, streams and the random generator only; every computation goes through ``_lib``.
"""
import ctypes

import torch

from . import _lib as L


def stream_ptr(stream=None):
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def tensor(data, dtype, scales=None, ld_scale=0, glob=None, amax=None, flags=0, scale_max=0):
    return L.Tensor(ptr(data), dtype, ptr(scales), ld_scale, ptr(glob), ptr(amax), flags, scale_max)


def randn_bf16(rows, cols, std, seed, device):
    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(rows, cols, generator=g, device=device, dtype=torch.float32) * std).to(torch.bfloat16)


def outlier_input(rows, cols, seed, device):
    """N(0, 1) with an independent Bernoulli(0.01) mask multiplying entries by 50."""
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn(rows, cols, generator=g, device=device, dtype=torch.float32)
    mask = torch.rand(rows, cols, generator=g, device=device) < 0.01
    return torch.where(mask, x * 50.0, x).to(torch.bfloat16)


class QuantizedMatrix:
    """NVFP4 matrix on the device: packed nibbles, block scales (linear or swizzled), one FP32 global."""

    def __init__(self, rows, cols, swizzled, device):
        self.rows, self.cols, self.swizzled = rows, cols, swizzled
        self.data = torch.empty(rows * cols // 2, dtype=torch.uint8, device=device)
        nsc = ((rows + 127) // 128 * 128) * ((cols // 16 + 3) // 4 * 4) if swizzled else rows * (cols // 16)
        self.scales = torch.empty(nsc, dtype=torch.uint8, device=device)
        self.glob = torch.zeros(1, dtype=torch.float32, device=device)
        self.flags = L.SCALES_SWIZZLED if swizzled else 0

    def tensor(self, amax=None, extra_flags=0):
        return tensor(self.data, L.NVFP4, self.scales, 0, self.glob, amax, self.flags | extra_flags, 0)

    def nbytes(self):
        return self.data.numel() + self.scales.numel() + 4


def quantize_decode_factor(x, swizzled=False, stream=None):
    """x (BF16 [rows][cols]) -> NVFP4 with the global stored as the decode factor g = amax / (6 * 448) (ModelOpt form)."""
    rows, cols = x.shape
    q = QuantizedMatrix(rows, cols, swizzled, x.device)
    amax = x.abs().max().float()
    q.glob.copy_(torch.where(amax > 0, amax / (6.0 * 448.0), torch.ones_like(amax)).reshape(1))
    src, dst = tensor(x, L.BF16), q.tensor()
    L.check(L.lib.nvfp4a_quantize(ctypes.byref(src), cols, ctypes.byref(dst), cols, rows, cols, stream_ptr(stream)))
    return q


def quantize_amax_swizzled(x, out, stream=None):
    """The quantization benchmark's call: swizzled E4M3 scales, amax computed by the library (Transformer Engine form)."""
    rows, cols = x.shape
    src = tensor(x, L.BF16)
    dst = tensor(out.data, L.NVFP4, out.scales, 0, out.glob, None, L.SCALES_SWIZZLED | L.GLOBAL_AMAX, 0)
    cfg = L.QuantConfig(1, L.FOS_OFF, 1)
    L.check(L.lib.nvfp4a_quantize_ex(ctypes.byref(src), cols, rows, cols, ctypes.byref(dst), cols, None, 0, ctypes.byref(cfg),
                                     stream_ptr(stream)))


def gemm(m, n, k, A, B, D, alpha=1.0, stream=None):
    """D[i + j m] = alpha * sum_k A(i, k) B(j, k); A, B ``nvfp4a_tensor`` structs, D a BF16 device tensor of n * m values."""
    tD = tensor(D, L.BF16)
    L.check(L.lib.nvfp4a_gemm(m, n, k, alpha, ctypes.byref(A), k, ctypes.byref(B), k, 0.0, None, 0, ctypes.byref(tD), m, None,
                              stream_ptr(stream)))


def weight_image(q):
    """The tensor-core image of a quantized weight (what ``TCWeight`` holds): returns (image tensor, nvfp4a_tensor on it)."""
    nb = L.lib.nvfp4a_tc_image_bytes(L.TC_A16, L.NVFP4, q.rows, q.cols)
    img = torch.empty(nb, dtype=torch.uint8, device=q.data.device)
    t = q.tensor()
    L.check(L.lib.nvfp4a_tc_image(L.TC_A16, ctypes.byref(t), q.cols, q.rows, q.cols, ptr(img), stream_ptr()))
    return img, tensor(img, L.NVFP4, glob=q.glob)


def quantize_given_amax(x, out, stream=None):
    """Quantization with the amax global already in ``out.glob`` (a delayed-scaling step): one read, one write."""
    rows, cols = x.shape
    src = tensor(x, L.BF16)
    dst = tensor(out.data, L.NVFP4, out.scales, 0, out.glob, None, L.SCALES_SWIZZLED | L.GLOBAL_AMAX, 0)
    cfg = L.QuantConfig(1, L.FOS_OFF, 0)
    L.check(L.lib.nvfp4a_quantize_ex(ctypes.byref(src), cols, rows, cols, ctypes.byref(dst), cols, None, 0, ctypes.byref(cfg),
                                     stream_ptr(stream)))


def kernel_status(reset=True):
    st = ctypes.c_uint(0)
    L.check(L.lib.nvfp4a_b200_kernel_status(ctypes.byref(st), int(reset)))
    return st.value
