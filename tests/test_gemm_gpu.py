"""GPU parity of nvfp4a_gemm / nvfp4a_gemm_ex / the image entries against the CPU oracle, through the C ABI.

Two kinds of check, as the reference's own tests make them (tests/test_util.h:153-155, :292-321 there):
  * the CUDA-core route computes the documented tiled order, so D and amax are compared bit for bit;
  * the tcgen05 and GEMV routes sum in their own order, so they are compared with the float64 value within the
    FP32-accumulation bound (k + 2) 2^-24 sum|a b| |s| + 4 2^-24 (|r s| + |bias| + |beta C|) + out_rel |v| + out_abs,
    amax within 2^-7 relative; the share of outputs within 1 BF16 ulp of the exact block-sum oracle is reported too.
Shapes, leading-dimension padding and format combinations follow tests/test_gemm.cu:13-41 and tests/test_gemv.cu:13-42 there."""
import ctypes
import os

import numpy as np
import pytest
import torch

import oracle as O
from nvfp4effma_b200 import _lib as L
from util import DevFp4, dev, host, ptr, rand_dense, rand_fp4, rand_q8, stream, tensor

pytestmark = pytest.mark.gpu

OUTS = [L.BF16, L.FP32, L.FP16]
OPS = [L.NVFP4, L.INT8, L.BF16, L.FP16, L.FP32]
SW, UE, AM, PR = L.SCALES_SWIZZLED, L.SCALES_UE5M3, L.GLOBAL_AMAX, L.GLOBAL_PER_ROW


def esize(t):
    return 4 if t == L.FP32 else 2


class Case:
    def __init__(self, m, n, k, bt, dt, ct, bias, alpha, beta, fa=0, fb=0, ma=0, mb=0):
        self.m, self.n, self.k, self.bt, self.dt, self.ct, self.bias, self.alpha, self.beta = m, n, k, bt, dt, ct, bias, alpha, beta
        self.fa, self.fb, self.ma, self.mb = fa, fb, ma, mb

    def __repr__(self):
        return f"m{self.m}n{self.n}k{self.k}-B{self.bt}-D{self.dt}-C{self.ct}-b{self.bias}-fa{self.fa:x}/{self.ma}-fb{self.fb:x}/{self.mb}"


def build_case(c, seed):
    """Host operands of a case, padded as the reference's run_case pads them."""
    rng = np.random.default_rng(seed)
    fp4b, q8b = c.bt == L.NVFP4, c.bt == L.INT8
    lda, ldb = c.k + 64, c.k + (128 if fp4b else 64)
    ldd = c.m + 3
    ldc = c.m + 1 if c.ct >= 0 else ldd
    ct = c.ct if c.ct >= 0 else c.dt
    A = rand_fp4(rng, c.m, c.k, ld=lda, ld_scale=c.k // 16 + 4, flags=c.fa, scale_max=c.ma, glob=37.5 if c.fa & AM else 0.375)
    if fp4b:
        B = rand_fp4(rng, c.n, c.k, ld=ldb, ld_scale=c.k // 16 + 8, flags=c.fb, scale_max=c.mb, glob=175.0 if c.fb & AM else 1.75)
    elif q8b:
        B = rand_q8(rng, c.n, c.k, ld=ldb, ld_scale=c.k // 16 + 8, glob=1.75)
    else:
        B = O.Dense(c.bt, rand_dense(rng, c.bt, ldb * c.n, 2.0), ldb)
    Cbuf = rand_dense(rng, ct, ldc * c.n, 4.0)
    if c.ct < 0:
        Dinit = rand_dense(rng, c.dt, ldd * c.n, 4.0)
        Cbuf = None
    else:
        Dinit = np.frombuffer(b"\xA5" * (ldd * c.n * esize(c.dt)), dtype=np.float32 if c.dt == L.FP32 else np.uint16).copy()
    bias = rand_dense(rng, c.bias, c.m, 8.0) if c.bias >= 0 else None
    return dict(A=A, B=B, C=Cbuf, ct=ct, ldc=ldc, Dinit=Dinit, ldd=ldd, bias=bias, lda=lda, ldb=ldb)


def oracle_case(c, h, want_ref=False, order=0):
    return O.gemm(c.m, c.n, c.k, h["A"], h["B"], D_dtype=c.dt, alpha=c.alpha, beta=c.beta, C=h["C"], C_dtype=h["ct"], ldc=h["ldc"],
                  ldd=h["ldd"], bias=h["bias"], bias_dtype=c.bias if c.bias >= 0 else L.FP32, lda=h["lda"], ldb=h["ldb"],
                  D_init=h["Dinit"], want_ref=want_ref, order=order)


def device_b(c, h):
    B = h["B"]
    if c.bt == L.NVFP4:
        d = DevFp4(B)
        return d, d.tensor()
    if c.bt == L.INT8:
        keep = (dev(B.data), dev(B.scales), dev(B.glob))
        return keep, tensor(keep[0], L.INT8, keep[1], B.ld_scale, keep[2])
    keep = dev(B.raw)
    return keep, tensor(keep, c.bt)


def run_gemm(c, h, lib=None):
    """nvfp4a_gemm on the device (of this library, or of ``lib``); returns (raw D buffer, amax)."""
    lib = lib or L.lib
    dA = DevFp4(h["A"])
    keepB, tB = device_b(c, h)
    dD, damax = dev(h["Dinit"]), dev(np.zeros(1, np.float32))
    dC = dev(h["C"]) if h["C"] is not None else None
    dbias = dev(h["bias"]) if h["bias"] is not None else None
    tA = dA.tensor()
    tC = tensor(dC, h["ct"]) if dC is not None else None
    tD = tensor(dD, c.dt, amax=damax)
    tbias = tensor(dbias, c.bias) if dbias is not None else None
    st = lib.nvfp4a_gemm(c.m, c.n, c.k, c.alpha, ctypes.byref(tA), h["lda"], ctypes.byref(tB), h["ldb"], c.beta,
                           ctypes.byref(tC) if tC is not None else None, h["ldc"], ctypes.byref(tD), h["ldd"],
                           ctypes.byref(tbias) if tbias is not None else None, stream())
    assert st == 0, lib.nvfp4a_last_error()
    torch.cuda.synchronize()
    return host(dD).view(h["Dinit"].dtype), float(host(damax)[0])


def values(raw, c, h):
    return O.to_f32(raw.reshape(c.n, h["ldd"])[:, : c.m], c.dt).astype(np.float64)


def check_bound(c, h, got_raw, got_amax, exp):
    """Tolerance check of a kernel that sums in its own order (reference tests/test_util.h:292-320)."""
    got = values(got_raw, c, h)
    with np.errstate(invalid="ignore", over="ignore"):
        err = np.abs(got - exp["ref64"])
        # an output that overflowed its dtype (FP16 Inf) counts as equal when the float64 value rounds to the same bits
        same = got == values(O.from_f32(exp["ref64"].astype(np.float32).reshape(-1), c.dt).reshape(c.n, c.m), c, dict(h, ldd=c.m))
        ratio = np.where(same, 0.0, err / exp["bound"])
    worst = float(np.nanmax(ratio)) if ratio.size else 0.0
    assert not np.isnan(ratio).any() and worst <= 1.0, f"{c}: max |error| / bound = {worst:.3f}"
    # padding between columns untouched
    g2 = got_raw.reshape(c.n, h["ldd"])[:, c.m:]
    i2 = h["Dinit"].reshape(c.n, h["ldd"])[:, c.m:]
    assert np.array_equal(g2, i2), f"{c}: padding of D was written"
    assert abs(got_amax - exp["amax"]) <= 2.0 ** -7 * exp["amax"] + 1e-30, f"{c}: amax {got_amax} vs {exp['amax']}"
    return worst


def cases_tiled():
    out, idx = [], 0
    sizes = [(1, 9, 64), (37, 45, 128), (200, 300, 192), (257, 129, 256), (128, 128, 64), (200, 64, 128), (150, 192, 256)]
    for bt in OPS:
        for m, n, k in sizes:
            out.append(Case(m, n, k, bt, OUTS[idx % 3], -1 if idx % 4 == 1 else (OUTS[(idx + 1) % 3] if idx % 4 == 2 else OUTS[idx % 3]),
                            -1 if idx % 3 == 0 else (L.BF16 if idx % 3 == 1 else L.FP32), 1.25 if idx % 2 else 1.0,
                            1.0 if idx % 4 == 1 else (0.5 if idx % 4 == 3 else 0.0)))
            idx += 1
    for bt in OPS:
        out.append(Case(1100, 1300, 512, bt, L.BF16, -1, -1, 1.0, 0.0))
        out.append(Case(1029, 700, 1024, bt, L.FP32, -1, L.FP32, 0.5, 1.0))
    return out


def set_formats(c, f, v):
    """The reference's format matrix (tests/test_util.h:135-151): bits 0..3 scale layout / type of A and B, 16 amax, 32 / 64 per-row."""
    fp4b = c.bt == L.NVFP4
    c.fa = (SW if f & 1 else 0) | (UE if f & 2 else 0) | (PR if f & 32 else 0)
    c.fb = ((SW if f & 4 else 0) | (UE if f & 8 else 0) | (PR if f & 64 else 0)) if fp4b else 0
    if f & 16:
        on = v % 3 if fp4b else 0
        if on != 1:
            c.fa |= AM
        if on != 0:
            c.fb |= AM
    c.ma = 256 if (c.fa & AM) and not (f & 2) and v % 2 else 0
    c.mb = 256 if (c.fb & AM) and not (f & 8) and v % 4 >= 2 else 0
    return c


def cases_formats(sizes):
    out, v = [], 0
    for bt in OPS:
        nf = 128 if bt == L.NVFP4 else 16
        for i in range(nf):
            m, n, k = sizes[v % len(sizes)]
            c = Case(m, n, k, bt, OUTS[v % 3], -1 if v % 4 == 1 else OUTS[v % 3], L.BF16 if v % 3 else -1, 1.25 if v % 2 else 1.0,
                     1.0 if v % 4 == 1 else 0.0)
            f = i if bt == L.NVFP4 else ((i & 3) | (16 if i & 4 else 0) | (32 if i & 8 else 0))
            out.append(set_formats(c, f, v))
            v += 1
    return out


@pytest.fixture
def exact_route():
    """Pins the GEMM entries to the CUDA-core kernel (the documented tiled order) for one test."""
    old = L.lib.nvfp4a_b200_set_route(1)
    yield
    L.lib.nvfp4a_b200_set_route(old)


def test_cuda_core_route_is_bit_exact_in_the_tiled_order(exact_route):
    """Every B dtype, tails, padded leading dimensions, C / accumulate / alpha / beta / bias / amax, all 128 + 4 x 16 formats."""
    fmt_sizes = [(257, 129, 256), (200, 64, 128), (300, 300, 320), (150, 192, 256)]
    bad = []
    for i, c in enumerate(cases_tiled()[:35] + cases_formats(fmt_sizes)):
        h = build_case(c, 1000 + i)
        exp = oracle_case(c, h)
        got, amax = run_gemm(c, h)
        if not np.array_equal(got, exp["D"]) or amax != exp["amax"]:
            bad.append(repr(c))
    assert not bad, f"{len(bad)} cases differ: {bad[:5]}"


def test_cuda_core_route_decodes_signed_block_scales_like_the_reference(exact_route):
    """Block-scale codes with the sign bit set are legal E4M3 for the reference (src/nvfp4effma.cuh:56-60 there); the tensor cores
    read scales as unsigned, so such tensors belong on the CUDA-core route, which must decode them exactly: D and amax equal the
    oracle's bit for bit with negative scales on both operands, linear and swizzled."""
    for i, (fa, fb) in enumerate([(0, 0), (SW, SW), (SW | AM, PR)]):
        c = Case(200, 150, 256, L.NVFP4, OUTS[i % 3], -1, L.FP32, 1.25, 0.0, fa=fa, fb=fb)
        h = build_case(c, 1500 + i)
        rng = np.random.default_rng(1500 + i)
        for t in (h["A"], h["B"]):
            flip = rng.integers(0, 3, t.scales.size) == 0
            t.scales[flip & (t.scales != 0)] |= 0x80
        assert (h["A"].scales & 0x80).any() and (h["B"].scales & 0x80).any()
        exp = oracle_case(c, h)
        got, amax = run_gemm(c, h)
        assert L.lib.nvfp4a_b200_last_route() == 1
        assert np.array_equal(got, exp["D"]) and amax == exp["amax"], c


def test_default_routes_within_the_accumulation_bound():
    """nvfp4a_gemm as routed by default (tcgen05 / GEMV / CUDA cores) against the float64 reference within the bound."""
    fmt_sizes = [(257, 129, 256), (200, 64, 128), (300, 300, 320), (150, 192, 256)]
    gemv_sizes = [(300, 3, 1024), (1000, 8, 576), (130, 20, 4160), (77, 1, 128), (64, 5, 64)]
    worst_all = 0.0
    for i, c in enumerate(cases_tiled() + cases_formats(fmt_sizes) + cases_formats(gemv_sizes)):
        h = build_case(c, 5000 + i)
        exp = oracle_case(c, h, want_ref=True)
        got, amax = run_gemm(c, h)
        worst_all = max(worst_all, check_bound(c, h, got, amax, exp))
    print(f"max |error| / bound over all cases = {worst_all:.3f}")


def test_gemv_shapes_n_1_to_8_and_groups():
    idx = 0
    gs = [(1, 64), (33, 576), (300, 1024), (1000, 4160)]
    cases = []
    for bt in OPS:
        for n in range(1, 9):
            m, k = gs[(n + bt) % 4]
            cases.append(Case(m, n, k, bt, OUTS[idx % 3], -1 if n == 3 else OUTS[idx % 3], -1 if idx % 3 == 0 else L.BF16,
                              0.75 if idx % 2 else 1.0, 1.0 if n == 3 else (-1.5 if idx % 4 == 1 else 0.0)))
            idx += 1
        for n in (12, 17, 32, 33, 48, 49):
            cases.append(Case(300, n, 1024, bt, OUTS[idx % 3], -1 if n == 17 else OUTS[idx % 3], L.BF16 if idx % 2 else -1, 1.0,
                              1.0 if n == 17 else 0.0))
            idx += 1
    for i, c in enumerate(cases):
        h = build_case(c, 9000 + i)
        exp = oracle_case(c, h, want_ref=True)
        got, amax = run_gemm(c, h)
        check_bound(c, h, got, amax, exp)


def test_k_zero_and_empty():
    c = Case(50, 3, 0, L.BF16, L.FP32, L.FP32, L.FP32, 1.0, 0.5)
    h = build_case(Case(50, 3, 64, L.BF16, L.FP32, L.FP32, L.FP32, 1.0, 0.5), 77)
    exp = O.gemm(50, 3, 0, h["A"], h["B"], D_dtype=L.FP32, alpha=1.0, beta=0.5, C=h["C"], C_dtype=L.FP32, ldc=h["ldc"], ldd=h["ldd"],
                 bias=h["bias"], bias_dtype=L.FP32, lda=h["lda"], ldb=h["ldb"], D_init=h["Dinit"])
    got, amax = run_gemm(c, h)
    assert np.array_equal(got, exp["D"]) and amax == exp["amax"]


def kernel_status(reset=True):
    st = ctypes.c_uint(0)
    L.check(L.lib.nvfp4a_b200_kernel_status(ctypes.byref(st), int(reset)))
    return st.value


def frac_within_1ulp_bf16(got, exact):
    """Share of outputs within one BF16 ulp of the exact block-sum oracle (both as float64 arrays of BF16 values)."""
    from util import ulp_bf16
    return float(np.mean(np.abs(got - exact) <= ulp_bf16(exact)))


@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("fa,fb", [(0, 0), (SW, SW), (SW, 0), (0, SW), (AM, AM | PR), (SW | PR, SW | AM)])
def test_w4a4_tcgen05_kernel(bn, fa, fb):
    """NVFP4 x NVFP4 on the tcgen05 route: every scale layout pair, m / n / k tails, both tile widths."""
    assert L.lib.nvfp4a_b200_set_tile_n(bn) == 0
    try:
        for i, (m, n, k) in enumerate([(128, 128, 256), (257, 129, 320), (200, 300, 192), (1100, 1300, 512), (64, 40, 64), (384, 512, 1024)]):
            c = Case(m, n, k, L.NVFP4, OUTS[i % 3], -1 if i % 4 == 1 else OUTS[i % 3], L.BF16 if i % 2 else -1, 1.25 if i % 2 else 1.0,
                     1.0 if i % 4 == 1 else 0.0, fa=fa, fb=fb, ma=256 if fa & AM else 0)
            h = build_case(c, 700 + i)
            exp = oracle_case(c, h, want_ref=True)
            got, amax = run_gemm(c, h)
            assert kernel_status() == 0
            check_bound(c, h, got, amax, exp)
    finally:
        L.lib.nvfp4a_b200_set_tile_n(0)


def test_w4a4_cta_pair_kernel_matches_the_single_cta_kernel():
    """The CTA-pair form (tcgen05.mma.cta_group::2, 256 x 256 tiles) against the bound and, bit for bit, against the single-CTA
    kernel, which feeds the same block products to the tensor cores in the same k order: odd numbers of 128-row tiles, tails
    in m / n / k, several tiles per pair (the barrier phases wrap), every epilogue input."""
    sizes = [(256, 256, 256), (129, 130, 64), (384, 512, 1024), (1100, 1300, 512), (257, 129, 320), (2304, 2100, 1344), (4096, 4096, 2048)]
    try:
        for i, (m, n, k) in enumerate(sizes):
            c = Case(m, n, k, L.NVFP4, OUTS[i % 3], -1 if i % 4 == 1 else OUTS[i % 3], L.BF16 if i % 2 else -1, 1.25 if i % 2 else 1.0,
                     1.0 if i % 4 == 1 else 0.0, fa=SW, fb=SW | (PR if i % 3 == 2 else 0))
            h = build_case(c, 900 + i)
            if i in (2, 6):   # dense D (ldd = m): the epilogue stores by TMA
                h["ldd"] = m
                h["Dinit"] = np.frombuffer(b"\xA5" * (m * n * esize(c.dt)), dtype=np.float32 if c.dt == L.FP32 else np.uint16).copy()
            exp = oracle_case(c, h, want_ref=True) if m * n <= 1500 * 1500 else None
            res = []
            for mode in (1, 0):
                assert L.lib.nvfp4a_b200_set_pair(mode) == 0
                got, amax = run_gemm(c, h)
                assert L.lib.nvfp4a_b200_last_route() == 4 and kernel_status() == 0
                if exp is not None:
                    check_bound(c, h, got, amax, exp)
                res.append((got, amax))
            assert np.array_equal(res[0][0], res[1][0]) and res[0][1] == res[1][1], (m, n, k)
    finally:
        L.lib.nvfp4a_b200_set_pair(-1)


def test_w4a4_swapped_orientation_matches_the_bound_and_the_other_orientation():
    """D that TMA can store (16-bit, 16-byte aligned pitch) runs with the tokens on the MMA's M side; the same cases with the
    orientation pinned the other way must agree within the bound too: bias, beta * C, per-row globals on either operand, FP16
    and BF16, tails in m / n / k, padded pitch."""
    sizes = [(128, 128, 256), (136, 40, 64), (200, 300, 192), (1104, 1300, 512), (264, 129, 320), (2304, 520, 1344)]
    try:
        for i, (m, n, k) in enumerate(sizes):
            dt = L.BF16 if i % 2 == 0 else L.FP16
            c = Case(m, n, k, L.NVFP4, dt, -1 if i % 3 == 0 else dt, L.BF16 if i % 2 else -1, 1.25 if i % 2 else 1.0,
                     0.0 if i % 3 == 0 else 0.5, fa=(SW if i % 2 else 0) | (PR if i in (2, 5) else 0), fb=(SW if i < 4 else 0) | (PR if i in (3, 5) else 0))
            h = build_case(c, 950 + i)
            h["ldd"] = m + (8 if i % 2 else 0)
            fill = np.frombuffer(b"\xA5" * (h["ldd"] * n * 2), dtype=np.uint16).copy()
            h["Dinit"] = fill
            exp = oracle_case(c, h, want_ref=True)
            res = []
            for mode in (1, 0):
                assert L.lib.nvfp4a_b200_set_swap(mode) == 0
                got, amax = run_gemm(c, h)
                assert L.lib.nvfp4a_b200_last_route() == 4 and kernel_status() == 0
                check_bound(c, h, got, amax, exp)
                res.append(got)
            print(f"{c}: equal bits between orientations: {np.mean(res[0] == res[1]):.6f}")
    finally:
        L.lib.nvfp4a_b200_set_swap(-1)


def make_image(kind, dfp4, rows, k, ld):
    nbytes = L.lib.nvfp4a_tc_image_bytes(kind, L.NVFP4, rows, k)
    img = torch.full((nbytes + 16,), 0xEE, dtype=torch.uint8, device="cuda")
    t = dfp4.tensor()
    L.check(L.lib.nvfp4a_tc_image(kind, ctypes.byref(t), ld, rows, k, ptr(img), stream()))
    return img, nbytes


@pytest.mark.parametrize("flags", [0, SW, UE])
def test_image_round_trip_and_convert(flags):
    rng = np.random.default_rng(61)
    for rows, k in [(128, 256), (200, 320), (517, 1088), (1, 64)]:
        ld = k + 64
        h = rand_fp4(rng, rows, k, ld=ld, ld_scale=k // 16 + 4, flags=flags, glob=0.375)
        d = DevFp4(h)
        img, nbytes = make_image(L.TC_A16, d, rows, k, ld)
        assert nbytes == ((rows + 127) // 128) * ((k + 255) // 256) * 18432
        img8 = torch.zeros_like(img)
        L.check(L.lib.nvfp4a_tc_image_convert(L.TC_A16, L.TC_A8, ptr(img), rows, k, ptr(img8), stream()))
        built8, _ = make_image(L.TC_A8, d, rows, k, ld)
        torch.cuda.synchronize()
        assert torch.equal(img8[:nbytes], built8[:nbytes])
        assert int(img[nbytes]) == 0xEE  # nothing written past the image
        # back to the plain tensor with linear scales
        out = O.Fp4(rows, k, ld=ld, ld_scale=k // 16 + 4, fill=0xEE)
        dout = DevFp4(out)
        t = dout.tensor()
        L.check(L.lib.nvfp4a_tc_image_to_raw(L.TC_A8, ptr(img8), rows, k, ctypes.byref(t), ld, stream()))
        torch.cuda.synchronize()
        gd, gs = host(dout.data).reshape(rows, ld // 2), host(dout.scales).reshape(rows, k // 16 + 4)
        assert np.array_equal(gd[:, : k // 2], h.data.reshape(rows, ld // 2)[:, : k // 2]) and np.all(gd[:, k // 2:] == 0xEE)
        lin = np.array([[h.scales[O.scale_pos(h.swz, h.ld_scale, k, r, c)] for c in range(k // 16)] for r in range(rows)], np.uint8)
        assert np.array_equal(gs[:, : k // 16], lin) and np.all(gs[:, k // 16:] == 0xEE)


def run_tc(c, h, gemv):
    """nvfp4a_gemm_tc (images of A and B) or nvfp4a_gemv_tc (image of A, B as it is)."""
    dA = DevFp4(h["A"])
    kindA = L.TC_A16 if c.bt == L.BF16 else L.TC_A8
    imgA, _ = make_image(kindA, dA, c.m, c.k, h["lda"])
    keepB, tB = device_b(c, h)
    dD, damax = dev(h["Dinit"]), dev(np.zeros(1, np.float32))
    dC = dev(h["C"]) if h["C"] is not None else None
    dbias = dev(h["bias"]) if h["bias"] is not None else None
    tA = dA.tensor()
    tA.data = imgA.data_ptr()
    tC = tensor(dC, h["ct"]) if dC is not None else None
    tD = tensor(dD, c.dt, amax=damax)
    tbias = tensor(dbias, c.bias) if dbias is not None else None
    cC, cb = (ctypes.byref(tC) if tC is not None else None), (ctypes.byref(tbias) if tbias is not None else None)
    if gemv:
        st = L.lib.nvfp4a_gemv_tc(c.m, c.n, c.k, c.alpha, ctypes.byref(tA), ctypes.byref(tB), h["ldb"], c.beta, cC, h["ldc"], ctypes.byref(tD),
                                  h["ldd"], cb, stream())
    else:
        nb = L.lib.nvfp4a_tc_image_bytes(L.TC_B, c.bt, c.n, c.k)
        imgB = torch.zeros(nb + 16, dtype=torch.uint8, device="cuda")
        L.check(L.lib.nvfp4a_tc_image(L.TC_B, ctypes.byref(tB), h["ldb"], c.n, c.k, ptr(imgB), stream()))
        tBi = L.Tensor.from_buffer_copy(tB)
        tBi.data = imgB.data_ptr()
        ws = torch.zeros(L.lib.nvfp4a_tc_workspace_bytes(), dtype=torch.uint8, device="cuda")
        st = L.lib.nvfp4a_gemm_tc(c.m, c.n, c.k, c.alpha, ctypes.byref(tA), ctypes.byref(tBi), c.beta, cC, h["ldc"], ctypes.byref(tD), h["ldd"], cb,
                                  ptr(ws), stream())
    L.check(st)
    torch.cuda.synchronize()
    return host(dD).view(h["Dinit"].dtype), float(host(damax)[0])


@pytest.mark.parametrize("bt", [L.NVFP4, L.INT8, L.BF16])
def test_image_entries_gemm_tc_and_gemv_tc(bt):
    sizes = [(37, 45, 128), (200, 300, 192), (257, 129, 256), (1100, 1300, 512), (300, 3, 1024), (1000, 8, 576), (77, 1, 128)]
    for i, (m, n, k) in enumerate(sizes):
        for fa in (0, SW, AM | PR):
            c = Case(m, n, k, bt, OUTS[i % 3], -1 if i % 4 == 1 else OUTS[i % 3], L.BF16 if i % 2 else -1, 1.25 if i % 2 else 1.0,
                     1.0 if i % 4 == 1 else 0.0, fa=fa, fb=SW if (bt == L.NVFP4 and i % 2) else 0)
            h = build_case(c, 800 + i)
            exp = oracle_case(c, h, want_ref=True)
            got, amax = run_tc(c, h, gemv=False)
            check_bound(c, h, got, amax, exp)
            if n <= 8:
                got, amax = run_tc(c, h, gemv=True)
                check_bound(c, h, got, amax, exp)
    assert kernel_status() == 0


def test_w4a4_4096_cubed_against_block_sum_oracle_sample():
    """The W4A4 GEMM 4096^3 at full size: BF16 N(0,1) operands quantized to NVFP4 (linear E4M3 scales, FP32 decode-factor
    globals), D BF16 column major.  The oracle checks a slab of 64 columns x all rows within the bound and reports the share
    within 1 BF16 ulp; linearity (alpha = 2 doubles every output exactly) is checked on the whole matrix."""
    m = n = k = 4096
    rng = np.random.default_rng(2)
    hs = []
    for seed in (2, 3):
        x = np.random.default_rng(seed).standard_normal((m, k), dtype=np.float32)
        x = O.to_f32(O.from_f32(x, L.BF16), L.BF16).reshape(m, k)
        g = np.array([np.abs(x).max() / (6.0 * 448.0)], np.float32)
        h = O.Fp4(m, k, glob=g)
        O.quantize(x, h)
        hs.append(h)
    A, B = hs
    dA, dB = DevFp4(A), DevFp4(B)
    outs = []
    for alpha in (1.0, 2.0):
        dD, damax = torch.zeros(m * n, dtype=torch.int16, device="cuda"), dev(np.zeros(1, np.float32))
        tA, tB, tD = dA.tensor(), dB.tensor(), tensor(dD, L.BF16, amax=damax)
        L.check(L.lib.nvfp4a_gemm(m, n, k, alpha, ctypes.byref(tA), k, ctypes.byref(tB), k, 0.0, None, 0, ctypes.byref(tD), m, None, stream()))
        torch.cuda.synchronize()
        outs.append((O.to_f32(host(dD).view(np.uint16), L.BF16).reshape(n, m), float(host(damax)[0])))
    assert kernel_status() == 0
    (d1, a1), (d2, a2) = outs
    assert np.array_equal(d2, 2.0 * d1) and a2 == 2.0 * a1
    # slab: columns 1000..1063
    j0, nj = 1000, 64
    Bs = O.Fp4(nj, k, glob=B.glob)
    Bs.data[:] = B.data.reshape(n, k // 2)[j0:j0 + nj].reshape(-1)
    Bs.scales[:] = B.scales.reshape(n, k // 16)[j0:j0 + nj].reshape(-1)
    exp = O.gemm(m, nj, k, A, Bs, D_dtype=L.BF16, want_ref=True)
    got = d1[j0:j0 + nj].astype(np.float64)
    assert np.all(np.abs(got - exp["ref64"]) <= exp["bound"])
    exact = O.to_f32(exp["D"], L.BF16).reshape(nj, m).astype(np.float64)
    share = frac_within_1ulp_bf16(got, exact)
    print(f"4096^3 W4A4: share of outputs within 1 BF16 ulp of the block-sum oracle = {share:.6f}; equal bits = {np.mean(got == exact):.6f}")
    assert share >= 0.999
    assert abs(a1 - np.abs(d1).max()) <= 2.0 ** -7 * a1


@pytest.mark.parametrize("bt", [L.INT8, L.NVFP4])
def test_gemv_with_block_scaled_activations_uses_the_dp4a_kernel(bt):
    """n <= 8 with INT8 / NVFP4 activations: exact integer block sums by DP4A (route 6), FP32 accumulation in the kernel's order."""
    for i, (m, n, k) in enumerate([(70, 1, 64), (515, 3, 1024), (4096, 8, 4096), (33, 5, 2304)]):
        for fa in (0, SW, AM | PR):
            c = Case(m, n, k, bt, OUTS[i % 3], OUTS[i % 3] if i % 2 else -1, L.FP32 if i % 2 else -1, 0.75, 1.0 if not i % 2 else 0.0, fa=fa,
                     fb=(SW | AM) if (bt == L.NVFP4 and i % 2) else 0)
            h = build_case(c, 1200 + i)
            exp = oracle_case(c, h, want_ref=True)
            got, amax = run_gemm(c, h)
            assert L.lib.nvfp4a_b200_last_route() == 6, c
            check_bound(c, h, got, amax, exp)


def test_w4a8_dp4a_gemm_is_bit_exact_in_the_tiled_order():
    """INT8 activations, n > 8, with the tensor-core W4A8 GEMM switched off (nvfp4a_b200_set_route(3)): the DP4A GEMM (route 7)
    sums blocks in the reference's tiled order, so D and amax equal the oracle's bit for bit; tails in m and n, padded leading
    dimensions, every output type, bias, beta, alpha.  The default route on the same inputs stays within the bound."""
    old = L.lib.nvfp4a_b200_set_route(3)
    try:
        for i, (m, n, k) in enumerate([(128, 128, 64), (130, 9, 128), (517, 300, 1024), (1000, 129, 576), (64, 2048, 256)]):
            for fa in (0, SW, AM | PR):
                c = Case(m, n, k, L.INT8, OUTS[i % 3], OUTS[(i + 1) % 3] if i % 2 else -1, L.BF16 if i % 2 else -1, 1.25, 0.5 if i % 2 else 1.0, fa=fa)
                h = build_case(c, 1300 + i)
                exp = oracle_case(c, h, want_ref=True)
                got, amax = run_gemm(c, h)
                assert L.lib.nvfp4a_b200_last_route() == 7, c
                assert np.array_equal(got.view(np.uint8), exp["D"].view(np.uint8)), c
                assert amax == exp["amax"], c
                L.lib.nvfp4a_b200_set_route(0)
                got, amax = run_gemm(c, h)
                assert L.lib.nvfp4a_b200_last_route() == (8 if m >= 128 and n >= 64 else 7), c
                check_bound(c, h, got, amax, exp)
                L.lib.nvfp4a_b200_set_route(3)
    finally:
        L.lib.nvfp4a_b200_set_route(old)


def test_gemm_dual_forward_dgrad_and_wgrad():
    """nvfp4a_gemm_dual picks, per operand, the half whose blocks run along k (reference include/nvfp4effma.h:97-103):
    forward Y = X W^T (trans 0, 0), dgrad dX = dY W (A = W with trans_a = 1: the column half of the [k][m] weight),
    wgrad dW = dY^T X (both column halves).  Each must equal nvfp4a_gemm on the chosen halves bit for bit (the call only
    forwards) and lie within the bound of the exact definition; a missing half is INVALID_VALUE."""
    T, I, Ou = 256, 384, 192
    rng = np.random.default_rng(77)

    def dual(x):
        rows, cols = x.shape
        row = O.Fp4(rows, cols, flags=O.GLOBAL_AMAX, glob=0.0)
        col = O.Fp4(cols, rows, flags=O.GLOBAL_AMAX, glob=0.0)
        O.quantize(x, row, tile=16, compute_amax=True)
        O.quantize(x, col, transposed=True, tile=16, compute_amax=True)
        dr, dc = DevFp4(row), DevFp4(col)
        return row, col, dr, dc, L.DualTensor(dr.tensor(), dc.tensor(), cols, rows)

    W = dual(rng.standard_normal((Ou, I)).astype(np.float32))
    X = dual(rng.standard_normal((T, I)).astype(np.float32))
    dY = dual(rng.standard_normal((T, Ou)).astype(np.float32))
    cases = [("forward", Ou, T, I, W, 0, X, 0), ("dgrad", I, T, Ou, W, 1, dY, 0), ("wgrad", I, Ou, T, X, 1, dY, 1)]
    for name, m, n, k, A, ta, B, tb in cases:
        hA, hB = A[1 if ta else 0], B[1 if tb else 0]
        dA, dB = A[3 if ta else 2], B[3 if tb else 2]
        outs = []
        for use_dual in (True, False):
            dD, damax = torch.zeros(m * n, dtype=torch.float32, device="cuda"), dev(np.zeros(1, np.float32))
            tD = tensor(dD, L.FP32, amax=damax)
            if use_dual:
                st = L.lib.nvfp4a_gemm_dual(m, n, k, 1.0, ctypes.byref(A[4]), ta, ctypes.byref(B[4]), tb, 0.0, None, 0, ctypes.byref(tD), m, None, stream())
            else:
                tA, tB = dA.tensor(), dB.tensor()
                st = L.lib.nvfp4a_gemm(m, n, k, 1.0, ctypes.byref(tA), hA.ld, ctypes.byref(tB), hB.ld, 0.0, None, 0, ctypes.byref(tD), m, None, stream())
            assert st == 0, (name, L.last_error())
            torch.cuda.synchronize()
            outs.append((host(dD).copy(), float(host(damax)[0])))
        assert np.array_equal(outs[0][0], outs[1][0]) and outs[0][1] == outs[1][1], name
        exp = O.gemm(m, n, k, hA, hB, D_dtype=L.FP32, want_ref=True)
        assert np.all(np.abs(outs[0][0].reshape(n, m).astype(np.float64) - exp["ref64"]) <= exp["bound"]), name
    # 16 x 16 tiles: the column half of W decodes to the transpose of its row half, so dgrad really multiplies by W
    assert np.array_equal(O.dequantize(W[1])[0], O.dequantize(W[0])[0].T)
    lone = L.DualTensor(W[2].tensor(), L.Tensor(), I, 0)
    dD = torch.zeros(I * T, dtype=torch.float32, device="cuda")
    tD = tensor(dD, L.FP32)
    st = L.lib.nvfp4a_gemm_dual(I, T, Ou, 1.0, ctypes.byref(lone), 1, ctypes.byref(dY[4]), 0, 0.0, None, 0, ctypes.byref(tD), I, None, stream())
    assert st == L.INVALID_VALUE and "column" in L.last_error()
    assert kernel_status() == 0


@pytest.mark.parametrize("bt", [L.INT8, L.NVFP4, L.BF16, L.FP32])
def test_grouped_gemm_gives_every_group_the_bytes_of_its_own_gemm(bt):
    """nvfp4a_gemm_grouped (reference include/nvfp4effma.h:104-116): three experts of 40 weight rows stacked in A, the row counts
    of B per expert in a device array (one expert empty, rows past seg[groups] left alone); every group's rows of D are the
    bytes the oracle's tiled order gives for that group's own GEMM -- bias, beta * C and per-row globals of the stacked A included."""
    for groups, m, k, rows, seg in ((3, 40, 192, 45, [0, 19, 19, 41]), (3, 200, 256, 300, [0, 130, 130, 290])):
        _grouped_case(bt, groups, m, k, rows, np.array(seg, np.int32))


def _grouped_case(bt, groups, m, k, rows, seg):
    from util import rand_fp4, rand_q8
    rng = np.random.default_rng(4100 + bt + m)
    lda, ldb, ldd = k + 64, k + 64, m + 8
    A = rand_fp4(rng, groups * m, k, ld=lda, ld_scale=k // 16 + 4, flags=O.PER_ROW, glob=0.375)
    if bt == L.NVFP4:
        B = rand_fp4(rng, rows, k, ld=ldb, ld_scale=k // 16 + 8, flags=O.PER_ROW, glob=1.75)
    elif bt == L.INT8:
        B = rand_q8(rng, rows, k, ld=ldb, ld_scale=k // 16 + 8)
    else:
        B = O.Dense(bt, rand_dense(rng, bt, ldb * rows, 2.0), ldb)
    bias = rand_dense(rng, L.BF16, groups * m, 3.0)
    Dinit = rand_dense(rng, L.BF16, ldd * rows, 4.0)     # D is also C (beta != 0)
    alpha, beta = 1.25, 0.5

    def rows_of(t, lo, hi):
        """The sub-matrix of rows [lo, hi) of a host operand (linear scales: whole rows of every array)."""
        if isinstance(t, O.Dense):
            return O.Dense(t.dtype, t.raw[lo * t.ld: hi * t.ld], t.ld)
        if isinstance(t, O.Q8):
            q = O.Q8(hi - lo, t.cols, ld=t.ld, ld_scale=t.ld_scale)
            q.data[:], q.scales[:] = t.data[lo * t.ld: hi * t.ld], t.scales[lo * t.ld_scale: hi * t.ld_scale]
            return q
        q = O.Fp4(hi - lo, t.cols, ld=t.ld, ld_scale=t.ld_scale, flags=t.flags, scale_max=t.scale_max, glob=0.0)
        q.data[:], q.scales[:], q.glob[:] = t.data[lo * t.ld // 2: hi * t.ld // 2], t.scales[lo * t.ld_scale: hi * t.ld_scale], t.glob[lo:hi]
        return q

    want = Dinit.copy()
    amax = 0.0
    for q in range(groups):
        lo, hi = int(seg[q]), int(seg[q + 1])
        if hi == lo:
            continue
        exp = O.gemm(m, hi - lo, k, rows_of(A, q * m, (q + 1) * m), rows_of(B, lo, hi), D_dtype=L.BF16, alpha=alpha, beta=beta,
                     C=Dinit[lo * ldd: hi * ldd], C_dtype=L.BF16, ldc=ldd, ldd=ldd, bias=bias[q * m: (q + 1) * m], bias_dtype=L.BF16,
                     lda=lda, ldb=ldb, D_init=Dinit[lo * ldd: hi * ldd])
        want[lo * ldd: hi * ldd] = exp["D"]
        amax = max(amax, exp["amax"])

    dA = DevFp4(A)
    if bt == L.NVFP4:
        keep = DevFp4(B); tB = keep.tensor()
    elif bt == L.INT8:
        keep = (dev(B.data), dev(B.scales)); tB = tensor(keep[0], L.INT8, keep[1], B.ld_scale)
    else:
        keep = dev(B.raw); tB = tensor(keep, bt)
    dD, damax, dbias, dseg = dev(Dinit), dev(np.zeros(1, np.float32)), dev(bias), dev(seg)
    tA, tD, tbias = dA.tensor(), tensor(dD, L.BF16, amax=damax), tensor(dbias, L.BF16)
    st = L.lib.nvfp4a_gemm_grouped(groups, m, k, rows, alpha, ctypes.byref(tA), lda, ctypes.byref(tB), ldb, beta, ctypes.byref(tD), ldd,
                                   ctypes.byref(tD), ldd, ctypes.byref(tbias), ctypes.c_void_p(dseg.data_ptr()), stream())
    assert st == 0, L.lib.nvfp4a_last_error()
    assert L.lib.nvfp4a_b200_last_route() == (7 if bt == L.INT8 else 1)   # INT8: the 128 x 128 DP4A kernel, else the generic one
    torch.cuda.synchronize()
    got = host(dD).view(np.uint16)
    assert np.array_equal(got, want)          # groups bit for bit; padding, the empty group and the rows past seg[groups] untouched
    assert float(host(damax)[0]) == amax


def test_w4a8_on_the_tensor_cores_and_the_exact_route_beside_it():
    """INT8 activations, more than 8 tokens: by default the W4A16 tcgen05 kernel on the activations split into three BF16 planes
    (route 8; within the FP32 accumulation bound of the exact definition: one rounding of q * s_b per activation); with
    nvfp4a_b200_set_route(3) the DP4A kernel (route 7), bit-identical to the reference's tiled order.  Tails in m, n and k, padded
    leading dimensions, bias, beta * C, every output type."""
    sizes = [(128, 64, 64), (300, 200, 320), (1000, 77, 192), (2048, 512, 1024), (515, 130, 4160)]
    for i, (m, n, k) in enumerate(sizes):
        c = Case(m, n, k, L.INT8, OUTS[i % 3], OUTS[i % 3] if i % 2 else -1, L.BF16 if i % 3 == 1 else -1, 1.25 if i % 2 else 1.0, 0.5 if i % 2 else 0.0)
        h = build_case(c, 4300 + i)
        exp = oracle_case(c, h, want_ref=True)
        got, amax = run_gemm(c, h)
        assert L.lib.nvfp4a_b200_last_route() == 8, c
        check_bound(c, h, got, amax, exp)
        old = L.lib.nvfp4a_b200_set_route(3)
        try:
            got, amax = run_gemm(c, h)
            assert L.lib.nvfp4a_b200_last_route() == 7, c
        finally:
            L.lib.nvfp4a_b200_set_route(old)
        assert np.array_equal(got, exp["D"]) and amax == exp["amax"], c
    assert kernel_status() == 0
    # the planes' pool: trimmed, refilled by the next call; and the whole call (allocation, conversion, GEMM, free) inside a CUDA graph
    assert L.lib.nvfp4a_b200_trim_scratch() == 0
    c = Case(300, 200, 320, L.INT8, L.BF16, -1, -1, 1.0, 0.0)
    h = build_case(c, 4390)
    want, _ = run_gemm(c, h)
    assert L.lib.nvfp4a_b200_last_route() == 8
    dA = DevFp4(h["A"])
    keepB, tB = device_b(c, h)
    dD = dev(h["Dinit"])
    tA, tD = dA.tensor(), tensor(dD, c.dt)

    def call():
        st = L.lib.nvfp4a_gemm(c.m, c.n, c.k, c.alpha, ctypes.byref(tA), h["lda"], ctypes.byref(tB), h["ldb"], 0.0, None, 0, ctypes.byref(tD), h["ldd"],
                               None, stream())
        assert st == 0, L.lib.nvfp4a_last_error()

    call()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        call()
    fresh = dev(h["Dinit"])
    for _ in range(3):
        dD.copy_(fresh)
        graph.replay()
        torch.cuda.synchronize()
        assert np.array_equal(host(dD).view(np.uint16), want.view(np.uint16))
    assert kernel_status() == 0


def test_gemv_long_reductions_in_sections():
    """The mma.sync GEMV cuts k >= 8192 into 2 and k >= 12288 into 4 sections; a matrix of few rows gives each section to a
    CTA of a cluster (partial sums through distributed shared memory), a taller one walks them in one CTA.  Both against the
    float64 reference within the bound, images and plain operands, 1 to 8 activation vectors, tails in m; and the two forms
    agree bit for bit on the rows they share (a row's sum depends on k alone)."""
    old = L.lib.nvfp4a_b200_set_route(2)   # keep the FP4 tensor-core GEMV out of it
    try:
        for i, (m, n, k) in enumerate([(300, 1, 8192), (130, 5, 14336), (1300, 3, 14336), (77, 8, 12288), (2500, 2, 8192)]):
            c = Case(m, n, k, L.BF16, OUTS[i % 3], -1, L.BF16 if i % 2 else -1, 1.25 if i % 2 else 1.0, 0.0, fa=SW if i % 2 else 0)
            h = build_case(c, 4700 + i)
            exp = oracle_case(c, h, want_ref=True)
            got, amax = run_gemm(c, h)
            assert L.lib.nvfp4a_b200_last_route() == 2, c
            check_bound(c, h, got, amax, exp)
            got_tc, amax_tc = run_tc(c, h, gemv=True)
            assert L.lib.nvfp4a_b200_last_route() == 2, c
            check_bound(c, h, got_tc, amax_tc, exp)
        # the same rows as part of a short matrix (cluster per slice) and of a tall one (one CTA per slice): identical bytes
        k = 14336
        tall = Case(1600, 2, k, L.BF16, L.FP32, -1, -1, 1.0, 0.0)
        h = build_case(tall, 4750)
        got_tall, _ = run_gemm(tall, h)
        short = Case(160, 2, k, L.BF16, L.FP32, -1, -1, 1.0, 0.0)
        hs = dict(h)
        A = h["A"]
        As = O.Fp4(160, k, ld=A.ld, ld_scale=A.ld_scale, flags=A.flags, scale_max=A.scale_max, glob=0.0)
        As.data[:], As.scales[:], As.glob[:] = A.data[:160 * A.ld // 2], A.scales[:160 * A.ld_scale], A.glob
        hs["A"] = As
        got_short, _ = run_gemm(short, hs)
        a = values(got_tall, tall, h)[:, :160]
        b = values(got_short, short, hs)
        assert np.array_equal(a, b)
    finally:
        L.lib.nvfp4a_b200_set_route(old)
    assert kernel_status() == 0


def test_blocked_gemv_with_sixteen_and_thirty_two_rows_per_cta():
    """The DP4A GEMV for INT8 / NVFP4 activations gives a CTA 16 rows while the matrix would leave SMs without a CTA and 32 rows
    from about 4700 rows up: both against the float64 reference within the bound, and bit for bit against each other on shared rows."""
    for bt in (L.INT8, L.NVFP4):
        outs = {}
        for m in (4800, 160):
            c = Case(m, 3, 320, bt, L.FP32, -1, -1, 1.0, 0.0)
            h = build_case(c, 4800 + bt)          # the same seed: the short matrix is not a prefix of the tall one, so each is checked alone
            exp = oracle_case(c, h, want_ref=True)
            got, amax = run_gemm(c, h)
            assert L.lib.nvfp4a_b200_last_route() == 6, c
            check_bound(c, h, got, amax, exp)
            outs[m] = (c, h, got)
        # shared rows: the first 160 rows of the tall matrix as a matrix of their own (16 rows per CTA)
        c, h, got_tall = outs[4800]
        A = h["A"]
        As = O.Fp4(160, c.k, ld=A.ld, ld_scale=A.ld_scale, flags=A.flags, scale_max=A.scale_max, glob=0.0)
        As.data[:], As.scales[:], As.glob[:] = A.data[:160 * A.ld // 2], A.scales[:160 * A.ld_scale], A.glob
        cs = Case(160, 3, 320, bt, L.FP32, -1, -1, 1.0, 0.0)
        hs = dict(h, A=As)
        got_short, _ = run_gemm(cs, hs)
        assert np.array_equal(values(got_tall, c, h)[:, :160], values(got_short, cs, hs))
