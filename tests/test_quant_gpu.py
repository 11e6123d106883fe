"""GPU parity of the quantization entry points against the CPU oracle, through the C ABI: bit-exact nibbles, scale bytes
(linear and swizzled, padding untouched), globals and the amax statistic.  Recipes and shapes follow the reference's
own quantizer test (tests/test_nvfp4effma.cu:498-524 there)."""
import ctypes

import numpy as np
import pytest
import torch

import oracle as O
from nvfp4effma_b200 import _lib as L
from util import dev, host, ptr, quant_input, stream, tensor

pytestmark = pytest.mark.gpu

SW, UE, AM, PR = L.SCALES_SWIZZLED, L.SCALES_UE5M3, L.GLOBAL_AMAX, L.GLOBAL_PER_ROW
SPECS = [  # name, tile, fos, flags, smax, compute, col
    ("1x16 given g", 1, 0, 0, 0, False, False),
    ("1x16 amax given, swizzled", 1, 0, AM | SW, 0, False, True),
    ("1x16 amax computed, swizzled", 1, 0, AM | SW, 0, True, False),
    ("16x16 amax computed", 16, 0, AM, 0, True, True),
    ("16x16 amax given, swizzled", 16, 0, AM | SW, 0, False, True),
    ("1x16 per-row amax computed", 1, 0, AM | PR, 0, True, True),
    ("1x16 4over6 MAE, 256", 1, 1, AM, 256, True, True),
    ("1x16 4over6 MSE, 448", 1, 2, AM | SW, 448, True, True),
    ("16x16 4over6 MAE, 256", 16, 1, AM | SW, 256, True, True),
    ("16x16 4over6 MSE, 256", 16, 2, AM, 256, False, True),
    ("1x16 per-row 4over6 MAE", 1, 1, AM | PR, 256, True, False),
    ("1x16 UE5M3 amax, swizzled", 1, 0, UE | AM | SW, 0, True, True),
    ("16x16 UE5M3 given g", 16, 0, UE, 0, False, True),
]


def test_hardware_conversions_equal_software_encoders_on_every_fp32():
    bad = torch.zeros(4, dtype=torch.int64, device="cuda")
    L.check(L.lib.nvfp4a_b200_codec_selftest(0, 1 << 32, ptr(bad), stream()))
    torch.cuda.synchronize()
    assert bad.tolist() == [0, 0, 0, 0]   # E2M1 low / high nibble, E4M3, packed BF16 rounding of the GEMM epilogues


def run_quant(dtype, rows, cols, spec, seed):
    name, tile, fos, flags, smax, compute, col = spec
    rng = np.random.default_rng(seed)
    lds = cols + 16
    x, raw = quant_input(rng, rows, cols, lds, dtype)
    amax_mode, per_row = bool(flags & AM), bool(flags & PR)
    rows16 = (rows + 15) // 16 * 16
    tam = float(np.abs(x[:, :cols]).max())
    ram = np.abs(x[:, :cols]).max(1).astype(np.float32)
    n_g = rows if per_row else 1
    g_given = (2000.0 + 37.0 * np.arange(n_g)).astype(np.float32) if amax_mode else np.full(n_g, 0.0625, np.float32)
    g_row0 = np.zeros(n_g, np.float32) if compute else g_given
    g_col0 = np.zeros(1, np.float32) if compute else g_given[:1].copy()
    # destinations with padded leading dimensions and 0xEE everywhere (padding must stay untouched)
    hr = O.Fp4(rows, cols, ld=cols + 32, ld_scale=cols // 16 + 3, flags=flags, scale_max=smax, glob=g_row0.copy(), fill=0xEE)
    hc = O.Fp4(cols, rows16, ld=rows16 + 32, ld_scale=rows16 // 16 + 1, flags=flags & ~PR, scale_max=smax, glob=g_col0.copy(), fill=0xEE)
    d_x = dev(raw)
    dr_d, dr_s, dr_g, dr_a = dev(hr.data), dev(hr.scales), dev(g_row0), dev(np.zeros(1, np.float32))
    dc_d, dc_s, dc_g, dc_a = dev(hc.data), dev(hc.scales), dev(g_col0), dev(np.zeros(1, np.float32))
    S = tensor(d_x, dtype)
    R = tensor(dr_d, L.NVFP4, dr_s, hr.ld_scale, dr_g, dr_a, flags, smax)
    Cc = tensor(dc_d, L.NVFP4, dc_s, hc.ld_scale, dc_g, dc_a, flags & ~PR, smax)
    cfg = L.QuantConfig(tile, fos, int(compute))
    st = L.lib.nvfp4a_quantize_ex(ctypes.byref(S), lds, rows, cols, ctypes.byref(R), hr.ld, ctypes.byref(Cc) if col else None, hc.ld,
                                  ctypes.byref(cfg), stream())
    L.check(st)
    torch.cuda.synchronize()
    # oracle
    O.quantize(x, hr, cols=cols, tile=tile, fos=fos, compute_amax=compute)
    assert np.array_equal(host(dr_g), hr.glob), f"{name}: rowwise global"
    assert np.array_equal(host(dr_d), hr.data), f"{name}: rowwise nibbles"
    assert np.array_equal(host(dr_s), hr.scales), f"{name}: rowwise scales"
    assert float(host(dr_a)[0]) == tam, f"{name}: amax statistic"
    if compute:
        assert np.array_equal(hr.glob, ram if per_row else np.array([tam], np.float32))
    if col:
        O.quantize(x, hc, cols=cols, transposed=True, tile=tile, fos=fos, compute_amax=compute)
        assert np.array_equal(host(dc_g), hc.glob), f"{name}: columnwise global"
        assert np.array_equal(host(dc_d), hc.data), f"{name}: columnwise nibbles"
        assert np.array_equal(host(dc_s), hc.scales), f"{name}: columnwise scales"
        assert float(host(dc_a)[0]) == tam
    return hr, dr_d, dr_s, dr_g


@pytest.mark.parametrize("spec", SPECS, ids=[s[0] for s in SPECS])
@pytest.mark.parametrize("dtype", [L.BF16, L.FP32])
def test_quantize_ex_recipes(spec, dtype):
    run_quant(dtype, 517, 1056, spec, 11)
    run_quant(dtype, 256, 320, spec, 12)


def test_quantize_ex_small_and_fp16():
    run_quant(L.FP16, 40, 48, SPECS[8], 13)
    for dtype in (L.BF16, L.FP16, L.FP32):
        run_quant(dtype, 3, 16, SPECS[0], 14)
        run_quant(dtype, 517, 1056, SPECS[0], 15)
        run_quant(dtype, 130, 80, SPECS[2], 16)  # cols/16 = 5: swizzled rows with a ragged last group of 4


@pytest.mark.parametrize("dtype", [L.BF16, L.FP16, L.FP32])
def test_quantize_int8(dtype):
    rng = np.random.default_rng(21)
    rows, cols = 517, 1056
    lds, ld8, lsc = cols + 16, cols + 16, cols // 16 + 4
    u = ((rng.integers(0, 1 << 24, (rows, lds)) / float(1 << 24)) * 2 - 1) * np.ldexp(1.0, rng.integers(-10, 10, (rows, lds)))
    raw = O.from_f32(u.astype(np.float32), dtype)
    x = O.to_f32(raw, dtype).reshape(rows, lds)
    x[5, :32] = 0  # zero blocks: scale 0, codes 0
    raw = O.from_f32(x, dtype)
    h = O.Q8(rows, cols, ld=ld8, ld_scale=lsc)
    h.data[:] = 0x55
    h.scales[:] = np.frombuffer(b"\x55" * 4, np.float32)[0]
    d_q, d_s, d_a = dev(h.data), dev(h.scales), dev(np.zeros(1, np.float32))
    S = tensor(dev(raw), dtype)
    Q = tensor(d_q, L.INT8, d_s, lsc, None, d_a)
    L.check(L.lib.nvfp4a_quantize(ctypes.byref(S), lds, ctypes.byref(Q), ld8, rows, cols, stream()))
    torch.cuda.synchronize()
    amax = O.quantize_int8(x, h)
    assert np.array_equal(host(d_q), h.data)
    assert np.array_equal(host(d_s).view(np.uint32), h.scales.view(np.uint32))
    assert float(host(d_a)[0]) == amax


@pytest.mark.parametrize("flags,smax", [(0, 0), (AM | SW, 0), (AM, 256), (UE | AM | SW, 0), (AM | PR, 0)])
@pytest.mark.parametrize("dtype", [L.BF16, L.FP16, L.FP32])
def test_dequantize(flags, smax, dtype):
    from util import rand_fp4, DevFp4
    rng = np.random.default_rng(31)
    rows, cols = 517, 1056
    h = rand_fp4(rng, rows, cols, ld=cols + 32, ld_scale=cols // 16 + 3, flags=flags, scale_max=smax, glob=37.5 if flags & AM else 0.375)
    d = DevFp4(h)
    ldy = cols + 48
    esz = 4 if dtype == L.FP32 else 2
    y = torch.full((rows * ldy * esz,), 0xEE, dtype=torch.uint8, device="cuda")
    am = dev(np.zeros(1, np.float32))
    src, dst = d.tensor(), tensor(y, dtype, amax=am)
    L.check(L.lib.nvfp4a_dequantize(ctypes.byref(src), h.ld, ctypes.byref(dst), ldy, rows, cols, stream()))
    torch.cuda.synchronize()
    want, wamax = O.dequantize(h, dtype)
    got_raw = host(y).view(np.float32 if dtype == L.FP32 else np.uint16).reshape(rows, ldy)
    got = O.to_f32(got_raw[:, :cols], dtype)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    pad = host(y).reshape(rows, ldy * esz)[:, cols * esz:]
    assert np.all(pad == 0xEE)
    assert float(host(am)[0]) == wamax


@pytest.mark.parametrize("rows,cols", [(517, 1056), (3, 16), (128, 64)])
def test_swizzle_scales_both_ways(rows, cols):
    rng = np.random.default_rng(41)
    ld = cols // 16 + 5
    lin = rng.integers(0, 256, rows * ld, dtype=np.uint8)
    d_lin = dev(lin)
    d_swz = torch.full((O.scale_bytes(True, 0, rows, cols),), 0xEE, dtype=torch.uint8, device="cuda")
    d_back = torch.full((rows * ld,), 0xEE, dtype=torch.uint8, device="cuda")
    L.check(L.lib.nvfp4a_swizzle_scales(ptr(d_lin), ptr(d_swz), ld, rows, cols, 1, stream()))
    L.check(L.lib.nvfp4a_swizzle_scales(ptr(d_swz), ptr(d_back), ld, rows, cols, 0, stream()))
    torch.cuda.synchronize()
    assert np.array_equal(host(d_swz), O.swizzle_scales(lin, ld, rows, cols, True))
    b = host(d_back).reshape(rows, ld)
    assert np.array_equal(b[:, : cols // 16], lin.reshape(rows, ld)[:, : cols // 16]) and np.all(b[:, cols // 16:] == 0xEE)


def test_transpose_of_16x16_tiles_is_the_columnwise_quantization():
    spec = ("16x16 amax given", 16, 0, AM, 0, False, True)
    rows, cols = 256, 320
    rng = np.random.default_rng(51)
    x, raw = quant_input(rng, rows, cols, cols, L.BF16)
    g = np.array([2000.0], np.float32)
    hr = O.Fp4(rows, cols, flags=AM, glob=g)
    hc = O.Fp4(cols, rows, flags=AM, glob=g)
    O.quantize(x, hr, tile=16)
    O.quantize(x, hc, transposed=True, tile=16)
    from util import DevFp4
    dr = DevFp4(hr)
    ht = O.Fp4(cols, rows, flags=AM, glob=g, fill=0xEE)
    dt = DevFp4(ht)
    s, d = dr.tensor(), dt.tensor()
    L.check(L.lib.nvfp4a_transpose(ctypes.byref(s), cols, ctypes.byref(d), rows, rows, cols, stream()))
    torch.cuda.synchronize()
    assert np.array_equal(host(dt.data), hc.data) and np.array_equal(host(dt.scales), hc.scales)


def test_full_size_8192_square_bf16_swizzled_amax_computed():
    """Quantization of 8192 x 8192 at full size: N(0,1) with 1 % of entries x 50, swizzled scales, amax computed; bit-exact."""
    rng = np.random.default_rng(1)
    rows = cols = 8192
    x = rng.standard_normal((rows, cols), dtype=np.float32)
    x[rng.random((rows, cols)) < 0.01] *= 50.0
    raw = O.from_f32(x, L.BF16)
    x = O.to_f32(raw, L.BF16).reshape(rows, cols)
    flags = AM | SW
    h = O.Fp4(rows, cols, flags=flags, glob=np.zeros(1, np.float32))
    d_d = torch.zeros(h.data.size, dtype=torch.uint8, device="cuda")
    d_s = torch.zeros(h.scales.size, dtype=torch.uint8, device="cuda")
    d_g, d_a = dev(np.zeros(1, np.float32)), dev(np.zeros(1, np.float32))
    S = tensor(dev(raw), L.BF16)
    R = tensor(d_d, L.NVFP4, d_s, 0, d_g, d_a, flags, 0)
    cfg = L.QuantConfig(1, 0, 1)
    L.check(L.lib.nvfp4a_quantize_ex(ctypes.byref(S), cols, rows, cols, ctypes.byref(R), cols, None, 0, ctypes.byref(cfg), stream()))
    torch.cuda.synchronize()
    amax = O.quantize(x, h, compute_amax=True)
    assert float(host(d_g)[0]) == amax == float(host(d_a)[0])
    assert np.array_equal(host(d_d), h.data)
    assert np.array_equal(host(d_s), h.scales)


@pytest.mark.parametrize("dtype,flags,lds_pad,rows,cols", [(L.BF16, AM | SW, 0, 3001, 4160), (L.FP16, AM, 64, 2100, 4096), (L.BF16, AM | UE, 0, 8190, 1088)])
def test_one_read_kernel_equals_the_two_launch_path(dtype, flags, lds_pad, rows, cols):
    """Large matrices with the common recipe run as one cooperative kernel that keeps part of the matrix on the chip between the
    amax visit and the encode visit; nvfp4a_b200_set_quant_fused(0) pins the amax kernel + encode kernel pair instead.  Both must
    write the same bytes (rows that do not divide over the SMs, a ragged last 64-block unit per row, padded source pitch, FP16,
    UE5M3 scales) -- and repeated calls must agree (the grid barrier's counter carries over from launch to launch)."""
    rng = np.random.default_rng(rows + cols)
    lds = cols + lds_pad
    x = rng.standard_normal((rows, lds), dtype=np.float32) * 3.0
    x[rng.random((rows, lds)) < 0.002] *= 100.0
    d_x = dev(O.from_f32(x, dtype))
    sbytes = O.scale_bytes(bool(flags & SW), 0 if flags & SW else cols // 16, rows, cols)
    outs = []
    try:
        for fused in (1, 0, 1):
            assert L.lib.nvfp4a_b200_set_quant_fused(fused) == 0
            d_d = torch.full((rows * cols // 2,), 0xEE, dtype=torch.uint8, device="cuda")
            d_s = torch.full((sbytes,), 0xEE, dtype=torch.uint8, device="cuda")
            d_g, d_a = dev(np.zeros(1, np.float32)), dev(np.zeros(1, np.float32))
            S, R = tensor(d_x, dtype), tensor(d_d, L.NVFP4, d_s, 0, d_g, d_a, flags, 0)
            cfg = L.QuantConfig(1, 0, 1)
            L.check(L.lib.nvfp4a_quantize_ex(ctypes.byref(S), lds, rows, cols, ctypes.byref(R), cols, None, 0, ctypes.byref(cfg), stream()))
            torch.cuda.synchronize()
            outs.append((host(d_d), host(d_s), float(host(d_g)[0]), float(host(d_a)[0])))
    finally:
        L.lib.nvfp4a_b200_set_quant_fused(1)
    st = ctypes.c_uint(0)
    L.check(L.lib.nvfp4a_b200_kernel_status(ctypes.byref(st), 1))
    assert st.value == 0
    for other in outs[1:]:
        assert np.array_equal(outs[0][0], other[0]) and np.array_equal(outs[0][1], other[1]) and outs[0][2:] == other[2:]
    xr = O.to_f32(O.from_f32(x, dtype), dtype).reshape(rows, lds)[:, :cols]
    assert outs[0][2] == float(np.abs(xr).max()) == outs[0][3]
