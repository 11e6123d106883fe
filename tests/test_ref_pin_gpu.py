"""Pins the CPU oracle against the REFERENCE ITSELF on the GPU: the unmodified reference library, built for sm_100 from its
own sources by oracle/ref.mk into oracle/_ref/libnvfp4effma_ref.so, runs its CUDA-core kernels (DP4A / FFMA tiled GEMM,
its GEMV kernel, its quantizer) on the same seeded inputs, and the oracle must reproduce its bytes exactly -- the
tiled order where the reference runs its tiled kernels, the GEMV lane order where it runs its GEMV kernel
(n <= kGemvMaxN = 48 / 56 / 56 / 32 / 56 for NVFP4 / BF16 / FP16 / FP32 / INT8, src/nvfp4effma.cuh:403 there).
Only the reference's CUDA-core paths run here (NVFP4A_DP4A=1 keeps its mma.sync paths off).  Skipped when the built
reference library did not travel with the repository."""
import ctypes
import os

import numpy as np
import pytest
import torch

import oracle as O
from nvfp4effma_b200 import _lib as L
from test_gemm_gpu import Case, build_case, cases_formats, cases_tiled, oracle_case, run_gemm
from test_quant_gpu import SPECS
from util import dev, host, quant_input, stream, tensor

pytestmark = pytest.mark.gpu

REF_SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libnvfp4effma_ref.so")
GEMV_MAX_N = {L.NVFP4: 48, L.BF16: 56, L.FP16: 56, L.FP32: 32, L.INT8: 56}


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF_SO):
        pytest.skip("oracle/_ref/libnvfp4effma_ref.so was not built (needs the reference sources: make -f oracle/ref.mk)")
    os.environ["NVFP4A_DP4A"] = "1"
    lib = ctypes.CDLL(REF_SO)
    for name in ("nvfp4a_gemm", "nvfp4a_quantize_ex", "nvfp4a_quantize", "nvfp4a_last_error"):
        fn, mine = getattr(lib, name), getattr(L.lib, name)
        fn.restype, fn.argtypes = mine.restype, mine.argtypes
    return lib


def test_oracle_gemm_equals_reference_kernels_bit_for_bit(ref):
    fmt_sizes = [(257, 129, 256), (200, 64, 128), (300, 300, 320), (150, 192, 256)]
    gemv_sizes = [(300, 3, 1024), (1000, 8, 576), (130, 20, 4160), (77, 1, 128), (64, 5, 64)]
    cases = cases_tiled() + cases_formats(fmt_sizes)[::3] + cases_formats(gemv_sizes)[::3]
    bad = []
    for i, c in enumerate(cases):
        h = build_case(c, 20000 + i)
        order = 1 if c.n <= GEMV_MAX_N[c.bt] else 0
        exp = oracle_case(c, h, order=order)
        got, amax = run_gemm(c, h, lib=ref)
        if not np.array_equal(got, exp["D"]) or amax != exp["amax"]:
            bad.append(repr(c))
    assert not bad, f"{len(bad)} of {len(cases)} cases differ from the reference: {bad[:6]}"


@pytest.mark.parametrize("dtype", [L.BF16, L.FP32])
def test_oracle_quantizer_equals_reference_kernels_bit_for_bit(ref, dtype):
    for si, spec in enumerate(SPECS):
        name, tile, fos, flags, smax, compute, col = spec
        rows, cols = 517, 1056
        rng = np.random.default_rng(30000 + si)
        lds = cols + 16
        x, raw = quant_input(rng, rows, cols, lds, dtype)
        per_row, amax_mode = bool(flags & L.GLOBAL_PER_ROW), bool(flags & L.GLOBAL_AMAX)
        n_g = rows if per_row else 1
        g0 = np.zeros(n_g, np.float32) if compute else ((2000.0 + 37.0 * np.arange(n_g)).astype(np.float32) if amax_mode else np.full(n_g, 0.0625, np.float32))
        hr = O.Fp4(rows, cols, ld=cols + 32, ld_scale=cols // 16 + 3, flags=flags, scale_max=smax, glob=g0.copy(), fill=0xEE)
        d_d, d_s, d_g, d_a = dev(hr.data), dev(hr.scales), dev(g0), dev(np.zeros(1, np.float32))
        S = tensor(dev(raw), dtype)
        R = tensor(d_d, L.NVFP4, d_s, hr.ld_scale, d_g, d_a, flags, smax)
        cfg = L.QuantConfig(tile, fos, int(compute))
        st = ref.nvfp4a_quantize_ex(ctypes.byref(S), lds, rows, cols, ctypes.byref(R), hr.ld, None, 0, ctypes.byref(cfg), stream())
        assert st == 0, ref.nvfp4a_last_error()
        torch.cuda.synchronize()
        O.quantize(x, hr, cols=cols, tile=tile, fos=fos, compute_amax=compute)
        assert np.array_equal(host(d_g), hr.glob), name
        assert np.array_equal(host(d_d), hr.data), name
        assert np.array_equal(host(d_s), hr.scales), name
