"""The extended epilogue (nvfp4a_gemm_ex, nvfp4a_gemv_tc_ex, nvfp4a_gemm_tc_ex) against the CPU oracle, the way the
reference tests it (tests/test_epilogue.cu:94-168 there): the accumulators come from the same entry without the
descriptor (unit scales, FP32 D, same kernel and order), the epilogue is emulated on the host; D, the second output and
the sums of squares must match bit for bit, SwiGLU within |h| (4e-7 (2 + |g|) + out_rel) + 1e-30 (fast exp / division)."""
import ctypes

import numpy as np
import pytest
import torch

import oracle as O
from nvfp4effma_b200 import _lib as L
from util import DevFp4, dev, host, ptr, rand_dense, rand_fp4, rand_q8, stream, tensor

pytestmark = pytest.mark.gpu

SHAPES = [(64, 1, 64), (1024, 1, 1024), (4096, 1, 1024), (528, 3, 576), (6144, 8, 1024), (2048, 5, 3072), (1024, 12, 2048), (512, 17, 1024),
          (512, 64, 1024), (1024, 200, 512)]


def out_rel(t):
    return {L.BF16: 2.0 ** -8, L.FP16: 2.0 ** -11, L.FP32: 2.0 ** -24}[t]


def run_case(m, n, k, bt, dt, mask, use_bias, use_c, tc):
    rng = np.random.default_rng(1000 * m + 10 * n + mask + bt)
    q8 = bt == L.INT8
    norm, glu, out2 = bool(mask & 1), bool(mask & 2), bool(mask & 4)
    mo = m // 2 if glu else m
    ldd, npart, ldp, lsq = mo + 3, 37, 40, m // 16 + 1
    A = rand_fp4(rng, m, k, glob=None)
    dA = DevFp4(A)
    if q8:
        B = rand_q8(rng, n, k, glob=1.75)
        keepB = (dev(B.data), dev(B.scales), dev(B.glob))
        tB = tensor(keepB[0], L.INT8, keepB[1], B.ld_scale, keepB[2])
        tBu = tensor(keepB[0], L.INT8, keepB[1], B.ld_scale, None)
    else:
        B = O.Dense(L.BF16, rand_dense(rng, L.BF16, n * k, 2.0), k)
        keepB = dev(B.raw)
        tB = tBu = tensor(keepB, L.BF16)
    bias = rand_dense(rng, L.BF16, m, 4.0)
    w2 = rand_dense(rng, L.BF16, m, 2.0)
    parts = (rng.integers(0, 4096, ldp * n) / 64.0).astype(np.float32)
    Dinit = rand_dense(rng, dt, ldd * n, 4.0)
    alpha, beta = 0.75, (1.0 if use_c else 0.0)
    d_bias, d_w2, d_parts = dev(bias), dev(w2), dev(parts)
    dD = dev(Dinit)
    d2 = torch.zeros(m * n, dtype=torch.int16, device="cuda")
    sq = torch.full((lsq * n,), -1.0, dtype=torch.float32, device="cuda")
    ex = L.Epilogue()
    if norm:
        ex.norm_parts, ex.norm_nparts, ex.norm_ld, ex.norm_inv_n, ex.norm_eps = d_parts.data_ptr(), npart, ldp, 1.0 / 1024.0, 1e-6
    ex.swiglu = int(glu)
    if out2:
        ex.d2, ex.d2_dtype, ex.ldd2, ex.w2, ex.w2_dtype, ex.sq, ex.ld_sq = d2.data_ptr(), L.BF16, m, d_w2.data_ptr(), L.BF16, sq.data_ptr(), lsq
    tA = dA.tensor()
    img = None
    if tc:
        kind = L.TC_A8 if q8 else L.TC_A16
        img = torch.zeros(L.lib.nvfp4a_tc_image_bytes(kind, L.NVFP4, m, k), dtype=torch.uint8, device="cuda")
        L.check(L.lib.nvfp4a_tc_image(kind, ctypes.byref(tA), k, m, k, ptr(img), stream()))
        tA = dA.tensor()
        tA.data = img.data_ptr()
    tbias = tensor(d_bias, L.BF16)
    ws = torch.zeros(L.lib.nvfp4a_tc_workspace_bytes(), dtype=torch.uint8, device="cuda")

    def call(tBx, al, be, tD, ld, bias_p, exp):
        if not tc:
            return L.lib.nvfp4a_gemm_ex(m, n, k, al, ctypes.byref(tA), k, ctypes.byref(tBx), k, be, None, ld, ctypes.byref(tD), ld, bias_p, exp, stream())
        if n <= 8:
            return L.lib.nvfp4a_gemv_tc_ex(m, n, k, al, ctypes.byref(tA), ctypes.byref(tBx), k, be, None, ld, ctypes.byref(tD), ld, bias_p, exp, stream())
        nb = L.lib.nvfp4a_tc_image_bytes(L.TC_B, bt, n, k)
        ib = torch.zeros(nb, dtype=torch.uint8, device="cuda")
        L.check(L.lib.nvfp4a_tc_image(L.TC_B, ctypes.byref(tBx), k, n, k, ptr(ib), stream()))
        tBi = L.Tensor.from_buffer_copy(tBx)
        tBi.data = ib.data_ptr()
        st = L.lib.nvfp4a_gemm_tc_ex(m, n, k, al, ctypes.byref(tA), ctypes.byref(tBi), be, None, ld, ctypes.byref(tD), ld, bias_p, exp, ptr(ws), stream())
        torch.cuda.synchronize()
        return st

    L.check(call(tB, alpha, beta, tensor(dD, dt), ldd, ctypes.byref(tbias) if use_bias else None, ctypes.byref(ex)))
    torch.cuda.synchronize()
    # accumulators: the same entry, no descriptor, unit scales, FP32 D
    dR = torch.zeros(m * n, dtype=torch.float32, device="cuda")
    L.check(call(tBu, 1.0, 0.0, tensor(dR, L.FP32), m, None, None))
    torch.cuda.synchronize()
    acc = host(dR).reshape(n, m)
    r = O.epilogue_ex(m, n, acc, alpha=alpha, gb=1.75 if q8 else 1.0, beta=beta, C=Dinit if use_c else None, C_dtype=dt, ldc=ldd,
                      bias=bias if use_bias else None, bias_dtype=L.BF16, mask=mask, norm_parts=parts if norm else None, norm_nparts=npart,
                      norm_ld=ldp, norm_inv_n=1.0 / 1024.0, norm_eps=1e-6, D_dtype=dt, ldd=ldd, w2=w2 if out2 else None, w2_dtype=L.BF16,
                      d2_dtype=L.BF16, ldd2=m, ld_sq=lsq)
    got = host(dD).view(Dinit.dtype).reshape(n, ldd)
    tag = f"m{m} n{n} k{k} B{bt} D{dt} ex{mask} bias{use_bias} c{use_c} tc{tc}"
    if glu:
        y = O.to_f32(got[:, :mo], dt).astype(np.float64)
        h = r["swiglu64"]
        g = r["v"].reshape(n, m // 16, 16)[:, :, :8].reshape(n, mo).astype(np.float64)
        tol = np.abs(h) * (4e-7 * (2.0 + np.abs(g)) + out_rel(dt)) + 1e-30
        assert np.all(np.abs(y - h) <= tol), tag
    else:
        assert np.array_equal(got[:, :mo], r["D"].reshape(n, ldd)[:, :mo]), tag
    assert np.array_equal(got[:, mo:], Dinit.reshape(n, ldd)[:, mo:]), tag + " (padding)"
    if out2:
        assert np.array_equal(host(d2).view(np.uint16), r["d2"]), tag + " (d2)"
        gsq = host(sq).reshape(n, lsq)
        assert np.array_equal(gsq[:, : m // 16].view(np.uint32), r["sq"].reshape(n, lsq)[:, : m // 16].view(np.uint32)), tag + " (sq)"
        assert np.all(gsq[:, m // 16:] == -1.0)
    assert not bool(ws.any()), tag + " (the workspace is left zeroed)"


@pytest.mark.parametrize("tc", [False, True])
@pytest.mark.parametrize("bt", [L.BF16, L.INT8])
def test_extended_epilogue(tc, bt):
    v = 0
    for (m, n, k) in SHAPES:
        for mask in range(1, 6):
            glu = bool(mask & 2)
            run_case(m, n, k, bt, L.FP32 if v % 2 else L.BF16, mask, (not glu) and v % 3 == 1, (not glu) and v % 4 == 2, tc)
            v += 1


@pytest.mark.parametrize("which", ["gate_up", "down"])
def test_llama_mlp_gemms_at_full_size_on_a_token_slab(which):
    """The fused transformer-MLP calls at their full size, 2048 tokens, through nvfp4a_gemm_tc_ex on images: gate / up
    28672 x 4096 with the deferred RMSNorm column scale, bias, SwiGLU and amax, and down 4096 x 14336 with bias, the second
    output times w2 and the sums of squares.  The whole problem runs (224 x 8 tiles of weight rows and tokens, the column
    scales of all 2048 tokens staged in the workspace); a slab of 64 tokens is checked the way the small cases are: the
    accumulators of the same entry without the descriptor, the epilogue emulated on the host."""
    glu = which == "gate_up"
    m, n, k = (28672, 2048, 4096) if glu else (4096, 2048, 14336)
    mask = 3 if glu else 4
    rng = np.random.default_rng(31 + glu)
    mo = m // 2 if glu else m
    npart, lsq = 256, m // 16
    A = rand_fp4(rng, m, k, glob=None)
    dA = DevFp4(A)
    dB = dev(rand_dense(rng, L.BF16, n * k, 2.0))
    bias = rand_dense(rng, L.BF16, m, 4.0)
    w2 = rand_dense(rng, L.FP32, m, 1.5)
    parts = (rng.integers(1, 4096, npart * n) / 64.0).astype(np.float32)
    d_bias, d_w2, d_parts = dev(bias), dev(w2), dev(parts)
    dD, damax = torch.zeros(mo * n, dtype=torch.int16, device="cuda"), dev(np.zeros(1, np.float32))
    d2 = torch.zeros(m * n if not glu else 1, dtype=torch.int16, device="cuda")
    sq = torch.full((lsq * n,), -1.0, dtype=torch.float32, device="cuda")
    ex = L.Epilogue()
    if glu:
        ex.norm_parts, ex.norm_nparts, ex.norm_ld, ex.norm_inv_n, ex.norm_eps, ex.swiglu = d_parts.data_ptr(), npart, npart, 1.0 / 4096.0, 1e-6, 1
    else:
        ex.d2, ex.d2_dtype, ex.ldd2, ex.w2, ex.w2_dtype, ex.sq, ex.ld_sq = d2.data_ptr(), L.BF16, m, d_w2.data_ptr(), L.FP32, sq.data_ptr(), lsq
    tA = dA.tensor()
    img = torch.zeros(L.lib.nvfp4a_tc_image_bytes(L.TC_A16, L.NVFP4, m, k), dtype=torch.uint8, device="cuda")
    L.check(L.lib.nvfp4a_tc_image(L.TC_A16, ctypes.byref(tA), k, m, k, ptr(img), stream()))
    tA.data = img.data_ptr()
    tB, tbias = tensor(dB, L.BF16), tensor(d_bias, L.BF16)   # contiguous BF16 [n][k] is its own activation image
    ws = torch.zeros(L.lib.nvfp4a_tc_workspace_bytes(), dtype=torch.uint8, device="cuda")
    alpha = 0.75
    tD = tensor(dD, L.BF16, amax=damax)
    L.check(L.lib.nvfp4a_gemm_tc_ex(m, n, k, alpha, ctypes.byref(tA), ctypes.byref(tB), 0.0, None, 0, ctypes.byref(tD), mo, ctypes.byref(tbias),
                                    ctypes.byref(ex), ptr(ws), stream()))
    assert L.lib.nvfp4a_b200_last_route() == 5
    dR = torch.zeros(m * n, dtype=torch.float32, device="cuda")
    tR = tensor(dR, L.FP32)
    L.check(L.lib.nvfp4a_gemm_tc(m, n, k, 1.0, ctypes.byref(tA), ctypes.byref(tB), 0.0, None, 0, ctypes.byref(tR), m, None, ptr(ws), stream()))
    torch.cuda.synchronize()
    st = ctypes.c_uint(0)
    L.check(L.lib.nvfp4a_b200_kernel_status(ctypes.byref(st), 1))
    assert st.value == 0 and not bool(ws.any())
    for j0 in (0, 1977):   # the first tokens, and a slab that ends in the last, partly filled token tile
        nj = min(64, n - j0)
        acc = host(dR.view(n, m)[j0:j0 + nj])
        r = O.epilogue_ex(m, nj, acc, alpha=alpha, bias=bias, bias_dtype=L.BF16, mask=mask, norm_parts=parts[j0 * npart:(j0 + nj) * npart] if glu else None,
                          norm_nparts=npart, norm_ld=npart, norm_inv_n=1.0 / 4096.0, norm_eps=1e-6, D_dtype=L.BF16, ldd=mo, w2=None if glu else w2,
                          w2_dtype=L.FP32, d2_dtype=L.BF16, ldd2=m, ld_sq=lsq)
        got = host(dD.view(n, mo)[j0:j0 + nj]).view(np.uint16)
        if glu:
            y, h = O.to_f32(got, L.BF16).astype(np.float64), r["swiglu64"]
            g = r["v"].reshape(nj, m // 16, 16)[:, :, :8].reshape(nj, mo).astype(np.float64)
            assert np.all(np.abs(y - h) <= np.abs(h) * (4e-7 * (2.0 + np.abs(g)) + out_rel(L.BF16)) + 1e-30), (which, j0)
        else:
            assert np.array_equal(got, r["D"].reshape(nj, mo)), (which, j0)
            assert np.array_equal(host(d2.view(n, m)[j0:j0 + nj]).view(np.uint16), r["d2"].reshape(nj, m)), (which, j0, "d2")
            assert np.array_equal(host(sq.view(n, lsq)[j0:j0 + nj]).view(np.uint32), r["sq"].reshape(nj, lsq).view(np.uint32)), (which, j0, "sq")
        # amax covers every output: at least the slab's largest value before rounding, and a value some output attains
        vmax = float(np.abs(r["swiglu64"] if glu else r["v"].astype(np.float64)).max())
        assert float(host(damax)[0]) >= vmax * (1 - 2.0 ** -7)
    out = O.to_f32(host(dD).view(np.uint16), L.BF16)
    assert abs(float(host(damax)[0]) - float(np.abs(out).max())) <= 2.0 ** -7 * float(host(damax)[0])
