"""nvfp4a_b200_gemm_ex_static: nvfp4a_gemm_ex with its scratch (the RMSNorm column scales of all tokens) in a device array
that belongs to the library image.  The results must equal nvfp4a_gemm_ex's bit for bit, call after call, and a call must
leave the amount of free device memory unchanged.  The file name keeps this test last in collection order: it must pass
alone as well as after every other test has used the device."""
import ctypes

import numpy as np
import pytest
import torch

import oracle as O
from nvfp4effma_b200 import _lib as L
from util import DevFp4, dev, host, rand_dense, rand_fp4, stream, tensor

pytestmark = pytest.mark.gpu


def operands(m, n, k, mask, seed):
    rng = np.random.default_rng(seed)
    norm, glu, out2 = bool(mask & 1), bool(mask & 2), bool(mask & 4)
    mo = m // 2 if glu else m
    A = DevFp4(rand_fp4(rng, m, k, glob=None))
    x = dev(rand_dense(rng, L.BF16, n * k, 2.0))
    bias = dev(rand_dense(rng, L.BF16, m, 4.0))
    parts = dev((rng.integers(0, 4096, 40 * n) / 64.0).astype(np.float32))
    w2 = dev(rand_dense(rng, L.BF16, m, 2.0))
    ex = L.Epilogue()
    if norm:
        ex.norm_parts, ex.norm_nparts, ex.norm_ld, ex.norm_inv_n, ex.norm_eps = parts.data_ptr(), 37, 40, 1.0 / 1024.0, 1e-6
    ex.swiglu = int(glu)
    keep = [A, x, bias, parts, w2]
    return A, x, bias, w2, ex, mo, out2, keep


def run(entry, m, n, k, mask, seed):
    A, x, bias, w2, ex, mo, out2, keep = operands(m, n, k, mask, seed)
    D = torch.full((n * (mo + 3),), 0x5A5A, dtype=torch.int16, device="cuda")
    d2 = torch.zeros(m * n, dtype=torch.int16, device="cuda")
    sq = torch.full((n * (m // 16),), -1.0, dtype=torch.float32, device="cuda")
    if out2:
        ex.d2, ex.d2_dtype, ex.ldd2, ex.w2, ex.w2_dtype, ex.sq, ex.ld_sq = d2.data_ptr(), L.BF16, m, w2.data_ptr(), L.BF16, sq.data_ptr(), m // 16
    tA, tB, tD, tb = A.tensor(), tensor(x, L.BF16), tensor(D, L.BF16), tensor(bias, L.BF16)
    st = entry(m, n, k, 0.75, ctypes.byref(tA), k, ctypes.byref(tB), k, 0.0, None, 0, ctypes.byref(tD), mo + 3, ctypes.byref(tb), ctypes.byref(ex),
               stream())
    assert st == 0, L.lib.nvfp4a_last_error()
    torch.cuda.synchronize()
    return host(D), host(d2), host(sq)


@pytest.mark.parametrize("mask", [1, 3, 5])
@pytest.mark.parametrize("shape", [(512, 200, 1024), (256, 300, 512), (128, 5, 256)])
def test_equals_gemm_ex_on_two_calls_in_a_row(shape, mask):
    m, n, k = shape
    ref = run(L.lib.nvfp4a_gemm_ex, m, n, k, mask, 7)
    for call in range(2):
        got = run(L.lib.nvfp4a_b200_gemm_ex_static, m, n, k, mask, 7)
        for a, b in zip(got, ref):
            assert np.array_equal(a.view(np.uint8), b.view(np.uint8)), f"call {call}, mask {mask}, shape {shape}"
    # a different problem in between must not leave anything behind that the next call depends on
    run(L.lib.nvfp4a_b200_gemm_ex_static, 128, 64, 256, 1, 8)
    got = run(L.lib.nvfp4a_b200_gemm_ex_static, m, n, k, mask, 7)
    assert all(np.array_equal(a.view(np.uint8), b.view(np.uint8)) for a, b in zip(got, ref))


def test_a_call_allocates_no_device_memory():
    m, n, k = 512, 200, 1024
    A, x, bias, w2, ex, mo, out2, keep = operands(m, n, k, 1, 9)
    D = torch.zeros(n * mo, dtype=torch.int16, device="cuda")
    tA, tB, tD = A.tensor(), tensor(x, L.BF16), tensor(D, L.BF16)
    args = (m, n, k, 1.0, ctypes.byref(tA), k, ctypes.byref(tB), k, 0.0, None, 0, ctypes.byref(tD), mo, None, ctypes.byref(ex), stream())
    assert L.lib.nvfp4a_b200_gemm_ex_static(*args) == 0      # first call on the device: looks the scratch up
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    for _ in range(3):
        assert L.lib.nvfp4a_b200_gemm_ex_static(*args) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0


def test_more_tokens_than_the_scratch_holds_are_refused():
    limit = L.lib.nvfp4a_b200_static_scratch_tokens()
    assert limit == 16384
    t = L.Tensor()
    ex = L.Epilogue()
    st = L.lib.nvfp4a_b200_gemm_ex_static(128, limit + 1, 256, 1.0, ctypes.byref(t), 256, ctypes.byref(t), 256, 0.0, None, 0, ctypes.byref(t), 128, None,
                                          ctypes.byref(ex), stream())
    assert st == L.INVALID_VALUE and "exceeds" in L.last_error()
