"""The FP4 tensor-core GEMV (n <= 2 BF16 activation vectors, weights fed to tcgen05 as stored, activations as FP4 digit
planes) against the CPU oracle: plain epilogue within the FP32-accumulation bound, extended epilogue bit for bit given the
kernel's own accumulators -- the checks of test_gemm_gpu / test_epilogue_gpu, with the kernel pinned by
nvfp4a_b200_set_gemv_splits and its use confirmed by nvfp4a_b200_last_route."""
import ctypes

import numpy as np
import pytest
import torch

import oracle as O
from nvfp4effma_b200 import _lib as L
from test_epilogue_gpu import run_case
from test_gemm_gpu import AM, OUTS, PR, SW, Case, build_case, check_bound, kernel_status, oracle_case, run_gemm, run_tc
from util import DevFp4, dev, host, stream, tensor

pytestmark = pytest.mark.gpu
FP4_GEMV = 3


@pytest.fixture
def pin():
    def set_splits(s):
        assert L.lib.nvfp4a_b200_set_gemv_splits(s) == 0
    yield set_splits
    L.lib.nvfp4a_b200_set_gemv_splits(0)


@pytest.mark.parametrize("splits", [1, 2, 4, 8])
def test_image_operand_all_splits(pin, splits):
    pin(splits)
    sizes = [(77, 1, 2048), (300, 2, 2048), (256, 1, 4096), (515, 2, 2048), (1100, 1, 2304), (4096, 2, 2048)]
    for i, (m, n, k) in enumerate(sizes):
        for fa in (0, AM | PR):
            c = Case(m, n, k, L.BF16, OUTS[i % 3], -1 if i % 4 == 1 else OUTS[i % 3], L.BF16 if i % 2 else -1, 1.25 if i % 2 else 1.0,
                     1.0 if i % 4 == 1 else 0.0, fa=fa)
            h = build_case(c, 900 + i)
            exp = oracle_case(c, h, want_ref=True)
            got, amax = run_tc(c, h, gemv=True)
            assert L.lib.nvfp4a_b200_last_route() == FP4_GEMV, c
            check_bound(c, h, got, amax, exp)
    assert kernel_status() == 0


def test_plain_operand_with_swizzled_scales(pin):
    pin(2)
    for i, (m, n, k) in enumerate([(200, 1, 512), (513, 2, 1024), (2048, 1, 4096)]):
        c = Case(m, n, k, L.BF16, OUTS[i % 3], OUTS[i % 3], L.FP32, 0.5, 0.0, fa=SW | (AM if i else 0))
        h = build_case(c, 950 + i)
        exp = oracle_case(c, h, want_ref=True)
        got, amax = run_gemm(c, h)
        assert L.lib.nvfp4a_b200_last_route() == FP4_GEMV, c
        check_bound(c, h, got, amax, exp)
    # linear scales are left to the mma.sync GEMV
    c = Case(200, 1, 512, L.BF16, L.BF16, L.BF16, -1, 1.0, 0.0)
    run_gemm(c, build_case(c, 960))
    assert L.lib.nvfp4a_b200_last_route() == 2
    assert kernel_status() == 0


def test_automatic_route_by_size():
    c = Case(300, 1, 2048, L.BF16, L.BF16, L.BF16, -1, 1.0, 0.0, fa=SW)
    run_gemm(c, build_case(c, 961))
    assert L.lib.nvfp4a_b200_last_route() == 2          # small: the mma.sync GEMV
    c = Case(8192, 1, 8192, L.BF16, L.BF16, L.BF16, -1, 1.0, 0.0, fa=SW)
    h = build_case(c, 962)
    exp = oracle_case(c, h, want_ref=True)
    got, amax = run_gemm(c, h)
    assert L.lib.nvfp4a_b200_last_route() == FP4_GEMV   # 38 MB of weights
    check_bound(c, h, got, amax, exp)


@pytest.mark.parametrize("spread", [0, 12, 23, 31, 60, 120])
def test_activations_with_a_wide_dynamic_range(pin, spread):
    """|x| spread over 2^-spread .. 1 (and exact zeros): up to 2^-24 of the largest element the digit planes hold every bit;
    a CTA that meets anything smaller computes its share on the CUDA cores instead."""
    pin(2)
    m, n, k = 384, 2, 2048
    c = Case(m, n, k, L.BF16, L.FP32, L.FP32, -1, 1.0, 0.0, fa=SW)
    h = build_case(c, 970 + spread)
    rng = np.random.default_rng(spread)
    x = rng.standard_normal(h["ldb"] * n).astype(np.float32) * np.exp2(-rng.integers(0, spread + 1, h["ldb"] * n)).astype(np.float32)
    x[rng.random(x.size) < 0.1] = 0.0
    h["B"] = O.Dense(L.BF16, O.from_f32(x, L.BF16), h["ldb"])
    exp = oracle_case(c, h, want_ref=True)
    got, amax = run_gemm(c, h)
    assert L.lib.nvfp4a_b200_last_route() == FP4_GEMV
    check_bound(c, h, got, amax, exp)


@pytest.mark.parametrize("splits", [1, 2])
@pytest.mark.parametrize("linear", [False, True])
def test_large_activations_that_meet_zero_weights(pin, linear, splits):
    """A few activations of magnitude 1 at positions where every weight is zero, all others near 2^-40: the result consists of
    the small terms alone, so bits dropped relative to the LARGEST activation would show (the FP32 accumulation bound is
    relative to sum |a_i x_i|).  Both tokens; swizzled and linear block scales; one token left narrow."""
    from util import rand_fp4
    pin(splits)   # one CTA per row tile: sixteen chunks through a ring of four stages, the eight consumer warps far apart
    m, n, k = 640, 2, 4096
    c = Case(m, n, k, L.BF16, L.FP32, L.FP32, -1, 1.0, 0.0, fa=0 if linear else SW)
    h = build_case(c, 990)
    rng = np.random.default_rng(991)
    if linear:
        h["A"] = rand_fp4(rng, m, k, ld=h["lda"], ld_scale=k // 16, glob=0.375)
    big = rng.choice(k, 9, replace=False)
    a = h["A"].data.reshape(m, h["lda"] // 2)
    for kk in big:                                    # zero nibble kk of every weight row
        a[:, kk // 2] &= 0xF0 if kk % 2 == 0 else 0x0F
    x = (rng.standard_normal(h["ldb"] * n) * 2.0 ** -40).astype(np.float32)
    x[big] = rng.choice([-1.0, 1.0, 1.5], big.size)   # token 0 only; token 1 stays within a few binades
    x[h["ldb"]:] *= 2.0 ** 40
    h["B"] = O.Dense(L.BF16, O.from_f32(x, L.BF16), h["ldb"])
    exp = oracle_case(c, h, want_ref=True)
    got, amax = run_gemm(c, h)
    assert L.lib.nvfp4a_b200_last_route() == FP4_GEMV
    check_bound(c, h, got, amax, exp)
    assert np.abs(exp["ref64"][0]).max() < 1e-6       # token 0's outputs really are made of the small terms
    assert kernel_status() == 0


def test_linear_scales_back_to_back_at_the_benchmark_size():
    """8192 x 8192 weights with linear block scales, automatic split, 300 launches back to back in one CUDA graph (as a decode
    step issues them): every launch gives the bytes of the first, and those are within the bound of the oracle.  The stages of
    the weight ring land in any order here; a warp that re-tiles scales must not take a stage's second fill for its first."""
    from util import rand_fp4
    m, n, k = 8192, 1, 8192
    c = Case(m, n, k, L.BF16, L.BF16, -1, -1, 1.0, 0.0)
    h = build_case(c, 995)
    rng = np.random.default_rng(996)
    h["A"] = rand_fp4(rng, m, k, ld=h["lda"], ld_scale=k // 16, glob=0.375)
    exp = oracle_case(c, h, want_ref=True)
    got, amax = run_gemm(c, h)
    assert L.lib.nvfp4a_b200_last_route() == FP4_GEMV
    check_bound(c, h, got, amax, exp)
    dA = DevFp4(h["A"])
    tA, x = dA.tensor(), dev(h["B"].raw)
    tx = tensor(x, L.BF16)
    outs = [torch.zeros(h["ldd"], dtype=torch.int16, device="cuda") for _ in range(50)]
    touts = [tensor(o, L.BF16) for o in outs]

    def launch(i):
        st = L.lib.nvfp4a_gemm(m, n, k, 1.0, ctypes.byref(tA), h["lda"], ctypes.byref(tx), h["ldb"], 0.0, None, 0, ctypes.byref(touts[i]), h["ldd"],
                               None, stream())
        assert st == 0, L.lib.nvfp4a_last_error()

    launch(0)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(50):
            launch(i)
    for _ in range(6):
        g.replay()
    torch.cuda.synchronize()
    assert kernel_status() == 0
    first = outs[0][:m].cpu()
    assert np.array_equal(first.numpy().view(np.uint16), got.reshape(-1)[:m])
    assert all(torch.equal(o[:m].cpu(), first) for o in outs[1:])


def test_extended_epilogue(pin):
    pin(2)
    v = 0
    for (m, n, k) in [(64, 1, 512), (1024, 1, 1024), (528, 2, 2304), (4096, 2, 1024)]:
        for mask in range(1, 6):
            glu = bool(mask & 2)
            run_case(m, n, k, L.BF16, L.FP32 if v % 2 else L.BF16, mask, (not glu) and v % 3 == 1, (not glu) and v % 4 == 2, True)
            assert L.lib.nvfp4a_b200_last_route() == FP4_GEMV
            v += 1
    assert kernel_status() == 0


def test_plain_operand_with_linear_scales(pin):
    """Linear block scales with a 16-byte aligned pitch: a TMA box brings [256 rows][16 bytes] per chunk, four warps re-tile it."""
    from util import rand_dense, rand_fp4
    pin(2)
    for i, (m, n, k) in enumerate([(300, 1, 512), (1000, 2, 2048), (4096, 1, 4096)]):
        c = Case(m, n, k, L.BF16, OUTS[i % 3], OUTS[i % 3], L.BF16 if i % 2 else -1, 1.0, 0.0)
        h = build_case(c, 980 + i)
        rng = np.random.default_rng(981 + i)
        h["A"] = rand_fp4(rng, m, k, ld=h["lda"], ld_scale=k // 16, glob=0.375)   # compact scale rows: pitch k / 16, a multiple of 16
        exp = oracle_case(c, h, want_ref=True)
        got, amax = run_gemm(c, h)
        assert L.lib.nvfp4a_b200_last_route() == FP4_GEMV, c
        check_bound(c, h, got, amax, exp)
    assert kernel_status() == 0
