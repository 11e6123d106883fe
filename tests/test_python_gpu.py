"""The Python surface on the GPU -- quantize / dequantize / linear / TCWeight / NVFP4Linear / torch.ops.nvfp4effma -- checked
against the CPU oracle: a device tensor is copied into the oracle's host containers, and

  * quantization results (nibbles, block-scale codes, globals) are compared bit for bit with ``oracle.quantize``;
  * ``linear`` results are compared with the float64 value of the exact definition (``oracle.gemm(..., want_ref=True)``)
    within the FP32-accumulation bound that call returns -- the bound the reference applies to its own tensor-core path
    (tests/test_util.h:292-313 there), output rounding included.

The behaviours covered are those the reference pins in binds/python/tests/test_nvfp4effma.py.
"""
import itertools
import os
import re
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu
nf = pytest.importorskip("nvfp4effma_b200") if torch.cuda.is_available() else None

GPU = "cuda"
ORACLE_DTYPE = {torch.bfloat16: O.BF16, torch.float16: O.FP16, torch.float32: O.FP32}


# ---- helpers: seeded inputs, host copies, the two kinds of comparison ---------------------------------------------------------------
def normal(shape, dtype=torch.float32, std=1.0, seed=0):
    gen = torch.Generator().manual_seed(1000 + seed)
    return torch.randn(shape, generator=gen).mul_(std).to(dtype).to(GPU)


def host_fp4(t):
    """An ``oracle.Fp4`` holding the bytes of the 2-D view of an ``NVFP4Tensor``."""
    op = t._operand()
    pitch = 0 if t.swizzled else op.scales.shape[1]
    h = O.Fp4(op.rows, op.cols, ld=2 * op.data.shape[1], ld_scale=pitch, flags=op.flags, scale_max=op.scale_max,
              glob=None if op.glob is None else op.glob.cpu().numpy())
    h.data[:] = op.data.contiguous().cpu().numpy().reshape(-1)
    h.scales[:] = op.scales.contiguous().cpu().numpy().reshape(-1)[:h.scales.size]
    return h


def host_dense(x):
    """An ``oracle.Dense`` of a 2-D dense tensor."""
    code = ORACLE_DTYPE[x.dtype]
    raw = x.contiguous().cpu()
    raw = raw.view(torch.int16).numpy().view(np.uint16) if code != O.FP32 else raw.numpy()
    return O.Dense(code, raw.reshape(-1), x.shape[1])


def host_int8(t):
    K = t.shape[-1]
    h = O.Q8(t.data.numel() // K, K)
    h.data[:] = t.data.reshape(-1).cpu().numpy()
    h.scales[:] = t.scales.reshape(-1).cpu().numpy()
    return h


def host_operand(x):
    if isinstance(x, nf.NVFP4Tensor):
        return host_fp4(x)
    if isinstance(x, nf.Int8Tensor):
        return host_int8(x)
    return host_dense(x)


def decoded(t):
    """float64 values of an NVFP4Tensor, by the oracle's dequantizer (exact in float32 for these magnitudes)."""
    return torch.from_numpy(O.dequantize(host_fp4(t))[0].astype(np.float64)).to(GPU)


def scale_codes(t):
    """Block-scale codes of ``t`` in linear order [rows, cols / 16], whatever layout they are stored in."""
    op = t._operand()
    nb = op.cols // 16
    raw = op.scales.contiguous().cpu().numpy()
    if not t.swizzled:
        return raw[:op.rows, :nb].copy()
    return O.swizzle_scales(raw.reshape(-1), nb, op.rows, op.cols, False).reshape(op.rows, nb)


def assert_linear(y, x, w, bias=None, alpha=1.0, beta=0.0, before=None):
    """``y`` [T, N] against the exact definition for activations ``x`` and weight ``w`` (device objects)."""
    T, N = y.shape
    K = w.shape[1]
    kw = {}
    if bias is not None:
        kw.update(bias=host_dense(bias.reshape(1, -1)).raw, bias_dtype=ORACLE_DTYPE[bias.dtype])
    if beta != 0.0:
        kw.update(C=host_dense(before).raw, C_dtype=ORACLE_DTYPE[before.dtype])
    exp = O.gemm(N, T, K, host_fp4(w), host_operand(x), D_dtype=ORACLE_DTYPE[y.dtype], alpha=alpha, beta=beta, want_ref=True, **kw)
    err = np.abs(y.double().cpu().numpy() - exp["ref64"])
    worst = float((err / exp["bound"]).max())
    assert worst <= 1.0, f"|error| reaches {worst:.3f} of the accumulation bound"


def recipe_name(r):
    return "+".join(f"{k}:{v}" for k, v in sorted(r.items())) or "plain"


RECIPES = [
    {},
    {"swizzled": True},
    {"block": "16x16"},
    {"row_scaled": True},
    {"four_over_six": "mae"},
    {"four_over_six": "mse", "row_scaled": True},
    {"four_over_six": "mse", "block": "16x16"},
    {"four_over_six": "mae", "scale_max": 448},
    {"four_over_six": "mae", "block": "16x16", "swizzled": True},
]


# ---- quantization ----------------------------------------------------------------------------------------------------------------
def awkward_matrix(rows, cols, dtype, seed):
    """Normal data with the blocks that stress the scale arithmetic: an all-zero block, an all-zero row, a block far below
    the rest (its scale underflows) and one far above (it sets the amax)."""
    x = normal((rows, cols), torch.float32, 2.5, seed)
    x[2, 16:32] = 0
    x[rows // 2] = 0
    x[4, :16] *= 1e-28
    x[6, 32:48] *= 300.0
    return x.to(dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32], ids=["bf16", "f32"])
@pytest.mark.parametrize("recipe", RECIPES, ids=recipe_name)
def test_quantize_is_bit_identical_to_the_oracle(recipe, dtype):
    rows, cols = 75, 288
    x = awkward_matrix(rows, cols, dtype, seed=1)
    q = nf.quantize(x, **recipe)
    fos = {None: 0, "mae": 1, "mse": 2}[recipe.get("four_over_six")]
    bound = recipe.get("scale_max", 256 if fos else 0)
    want = O.Fp4(rows, cols, flags=O.GLOBAL_AMAX | (O.PER_ROW if recipe.get("row_scaled") else 0), scale_max=bound, glob=0.0)
    O.quantize(x.float().cpu().numpy(), want, tile=16 if recipe.get("block") == "16x16" else 1, fos=fos, compute_amax=True)
    assert q.shape == (rows, cols) and q.global_is_amax and q.scale_max == bound and q.swizzled == bool(recipe.get("swizzled"))
    assert np.array_equal(q.data.cpu().numpy().reshape(-1), want.data), "nibbles"
    assert np.array_equal(scale_codes(q), want.scales.reshape(rows, cols // 16)), "block-scale codes"
    assert np.array_equal(q.global_scale.cpu().numpy(), want.glob), "amax"


def test_quantize_with_a_given_decode_factor_an_amax_output_and_ue5m3_scales():
    x = normal((48, 224), torch.bfloat16, 1.7, seed=2)
    factor = torch.tensor([0.0035], device=GPU)
    seen = torch.zeros(1, device=GPU)
    q = nf.quantize(x, factor, amax=seen)
    want = O.Fp4(48, 224, glob=0.0035)
    O.quantize(x.float().cpu().numpy(), want)
    assert not q.global_is_amax and q.amax is None and torch.equal(q.global_scale, factor)
    assert np.array_equal(q.data.cpu().numpy().reshape(-1), want.data) and np.array_equal(scale_codes(q).reshape(-1), want.scales)
    assert seen.item() == x.float().abs().max().item()
    u = nf.quantize(x, scale_dtype="ue5m3")
    want_u = O.Fp4(48, 224, flags=O.GLOBAL_AMAX | O.UE5M3, glob=0.0)
    O.quantize(x.float().cpu().numpy(), want_u, compute_amax=True)
    assert u.ue5m3 and u.scales.dtype == torch.uint8 and np.array_equal(scale_codes(u).reshape(-1), want_u.scales)
    assert np.array_equal(u.data.cpu().numpy().reshape(-1), want_u.data)
    per_row = nf.quantize(x, torch.linspace(0.002, 0.004, 48, device=GPU))
    assert per_row.per_row and per_row.global_scale.numel() == 48


@pytest.mark.parametrize("block", ["1x16", "16x16"])
def test_the_columnwise_half_is_the_quantization_of_the_transpose(block):
    x = normal((112, 144), torch.bfloat16, 1.2, seed=3)
    q = nf.quantize(x, block=block, columnwise=True)
    col = q.columnwise
    assert col.shape == (144, 112) and col.global_is_amax and torch.equal(col.global_scale, q.global_scale)
    direct = nf.quantize(x.t().contiguous(), block=block)          # the transpose sees the same amax
    assert torch.equal(col._operand().data[:, :56], direct.data) and np.array_equal(scale_codes(col), scale_codes(direct))
    if block == "16x16":
        flipped = q.transpose_2d()
        assert flipped.shape == (144, 112) and flipped.block == (16, 16)
        assert torch.equal(flipped.data, col._operand().data[:, :56]) and np.array_equal(scale_codes(flipped), scale_codes(col))
    else:
        with pytest.raises(ValueError):
            q.transpose_2d()


@pytest.mark.parametrize("recipe", RECIPES + [{"scale_dtype": "ue5m3", "swizzled": True}], ids=recipe_name)
def test_switching_the_scale_layout_keeps_every_value_and_dequantize_matches_the_oracle(recipe):
    x = normal((210, 176), torch.float32, 3.0, seed=4)
    q = nf.quantize(x, **recipe)
    other = q.with_scale_layout(not q.swizzled)
    assert other.swizzled != q.swizzled and q.with_scale_layout(q.swizzled) is q
    assert np.array_equal(scale_codes(q), scale_codes(other))
    for t in (q, other):
        for dtype, code in ((torch.float32, O.FP32), (torch.bfloat16, O.BF16)):
            want = O.dequantize(host_fp4(t), code)[0]
            got = nf.dequantize(t, dtype)
            assert got.dtype == dtype and np.array_equal(got.float().cpu().numpy(), want)
    assert torch.equal(q.dequantize(torch.float32), nf.dequantize(q, torch.float32))


# ---- linear ----------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("tokens", [1, 6, 37, 270])
@pytest.mark.parametrize("recipe", RECIPES[:6] + [{"scale_dtype": "ue5m3"}], ids=recipe_name)
def test_linear_takes_every_weight_format(recipe, tokens):
    N, K = 136, 320
    w = nf.quantize(normal((N, K), seed=10), **recipe)
    x = normal((tokens, K), torch.bfloat16, seed=11)
    assert_linear(nf.linear(x, w, act="exact", out_dtype=torch.float32), x, w)
    xq = nf.quantize(x, row_scaled=tokens > 1, swizzled=True)
    assert_linear(nf.linear(xq, w, out_dtype=torch.float32), xq, w)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32], ids=["bf16", "f16", "f32"])
@pytest.mark.parametrize("tokens", [1, 2, 8, 9, 190])
def test_linear_on_dense_activations_with_bias(tokens, dtype):
    N, K = 200, 384
    w = nf.quantize(normal((N, K), seed=12))
    x, bias = normal((tokens, K), dtype, seed=13), normal((N,), dtype, seed=14)
    y = nf.linear(x, w, bias, act="exact")
    assert y.dtype == dtype and tuple(y.shape) == (tokens, N)
    assert_linear(y, x, w, bias)


@pytest.mark.parametrize("tokens", [1, 7, 8, 40, 300])
def test_linear_on_nvfp4_activations(tokens):
    w = nf.quantize(normal((144, 256), seed=15))
    x = nf.quantize(normal((tokens, 256), seed=16))
    y = nf.linear(x, w, out_dtype=torch.float32)
    assert y.dtype == torch.float32
    assert_linear(y, x, w)
    assert nf.linear(x, w).dtype == torch.bfloat16
    assert torch.equal(nf.linear(normal((tokens, 256), seed=16), w, act="nvfp4", out_dtype=torch.float32), y)


@pytest.mark.parametrize("tokens", [1, 8, 24, 210])
def test_int8_quantization_and_w4a8_linear(tokens):
    N, K = 136, 256
    w = nf.quantize(normal((N, K), seed=17))
    x = normal((tokens, K), torch.bfloat16, seed=18)
    xq = nf.quantize_int8(x)
    want = O.Q8(tokens, K)
    O.quantize_int8(x.float().cpu().numpy(), want)
    assert np.array_equal(xq.data.cpu().numpy().reshape(-1), want.data) and np.array_equal(xq.scales.cpu().numpy().reshape(-1), want.scales)
    y = nf.linear(x, w, act="int8", out_dtype=torch.float32)
    assert_linear(y, xq, w)
    assert torch.equal(nf.linear(xq, w, out_dtype=torch.float32), y) and nf.linear(x, w, act="int8").dtype == torch.bfloat16


def test_int8_tensor_container():
    w = nf.quantize(normal((128, 192), seed=19))
    x = normal((3, 5, 192), torch.float16, seed=20)
    t = nf.quantize_int8(x)
    assert isinstance(t, nf.Int8Tensor) and t.shape == (3, 5, 192) and t.dim() == 3 and tuple(t.scales.shape) == (3, 5, 12) and t.dtype == torch.float16
    assert torch.equal(nf.Int8Tensor.from_float(x).data, t.data)
    y = nf.linear(t, w)
    assert y.dtype == torch.float16 and tuple(y.shape) == (3, 5, 128) and torch.equal(y, nf.linear(x, w, act="int8"))
    products = t.data.float() * t.scales.repeat_interleave(16, dim=-1)
    assert torch.equal(t.dequantize(torch.float32), products) and t.dequantize().dtype == torch.float16
    with pytest.raises(ValueError):
        nf.linear(nf.quantize_int8(normal((4, 128), seed=21)), w)   # 128 features against a 192-feature weight
    with pytest.raises(TypeError):
        nf.Int8Tensor(t.data.to(torch.int16), t.scales)
    with pytest.raises(TypeError):
        nf.Int8Tensor(t.data, t.scales.double())
    with pytest.raises(ValueError):
        nf.Int8Tensor(t.data, t.scales[..., :11])


@pytest.mark.parametrize("act", ["exact", "int8", "nvfp4"])
@pytest.mark.parametrize("tokens", [1, 4, 8, 9, 180])
def test_tc_weight_serves_gemv_and_gemm(tokens, act):
    N, K = 208, 384
    w = nf.quantize(normal((N, K), seed=22))
    image_weight = nf.TCWeight(w, act)
    assert image_weight.shape == (N, K) and image_weight.dim() == 2 and image_weight.image.dtype == torch.uint8
    x, bias = normal((tokens, K), torch.bfloat16, seed=23), normal((N,), torch.float32, seed=24)
    seen_by_kernel = x if act == "exact" else nf.quantize_int8(x) if act == "int8" else nf.quantize(x)
    y = nf.linear(x, image_weight, bias, out_dtype=torch.float32)
    assert_linear(y, seen_by_kernel, w, bias)
    assert nf.linear(x, image_weight).dtype == torch.bfloat16
    start = normal((tokens, N), torch.float32, seed=25)
    acc = start.clone()
    assert nf.linear(x, image_weight, out=acc, alpha=0.5, beta=2.0) is acc
    assert_linear(acc, seen_by_kernel, w, alpha=0.5, beta=2.0, before=start)
    if act != "exact":
        assert torch.equal(nf.linear(seen_by_kernel, image_weight, out_dtype=torch.float32), nf.linear(x, image_weight, out_dtype=torch.float32))
    with pytest.raises(ValueError):
        nf.linear(x, image_weight, act="exact" if act != "exact" else "nvfp4")
    if act == "exact":
        with pytest.raises(TypeError):
            nf.linear(x.float(), image_weight)
        with pytest.raises(ValueError):
            nf.linear(nf.quantize(x), image_weight)


def test_backward_products_from_columnwise_halves():
    tokens, fan_in, fan_out = 128, 256, 64
    w = nf.quantize(normal((fan_out, fan_in), seed=26), block="16x16", columnwise=True)
    x = nf.quantize(normal((tokens, fan_in), seed=27), columnwise=True)
    dy = nf.quantize(normal((tokens, fan_out), seed=28), columnwise=True)
    assert torch.equal(decoded(w.columnwise), decoded(w).t())       # 16 x 16 tiles: one scale serves both directions
    assert_linear(nf.linear(dy, w.columnwise, out_dtype=torch.float32), dy, w.columnwise)                       # dX = dY W
    assert_linear(nf.linear(dy.columnwise, x.columnwise, out_dtype=torch.float32), dy.columnwise, x.columnwise)  # dW = dY^T X


def test_adopting_a_transformer_engine_tensor():
    q = nf.quantize(normal((160, 128), torch.bfloat16, seed=29), swizzled=True, columnwise=True, four_over_six="mse")
    fake = SimpleNamespace(_rowwise_data=q.data, _rowwise_scale_inv=q.scales.view(torch.uint8), _amax_rowwise=q.global_scale,
                           _columnwise_data=q.columnwise.data, _columnwise_scale_inv=q.columnwise.scales.view(torch.uint8),
                           _amax_columnwise=q.columnwise.global_scale, _with_gemm_swizzled_scales=True, _nvfp4_e4m3_max=256,
                           _scale_dtype="DType.kFloat8E4M3")
    t = nf.NVFP4Tensor.from_te(fake)
    assert (t.swizzled, t.global_is_amax, t.scale_max, t.ue5m3) == (True, True, 256, False) and t.columnwise.shape == (128, 160)
    assert t.data.data_ptr() == q.data.data_ptr()
    assert torch.equal(nf.dequantize(t, torch.float32), nf.dequantize(q, torch.float32))
    w = nf.quantize(normal((96, 128), seed=30))
    assert torch.equal(nf.linear(t, w, out_dtype=torch.float32), nf.linear(q, w, out_dtype=torch.float32))
    only_columns = SimpleNamespace(_rowwise_data=None, _columnwise_data=q.columnwise.data, _columnwise_scale_inv=q.columnwise.scales.view(torch.uint8),
                                   _amax_columnwise=q.columnwise.global_scale, _with_gemm_swizzled_scales=True, _nvfp4_e4m3_max=256)
    assert nf.NVFP4Tensor.from_te(only_columns).shape == (128, 160)
    with pytest.raises(ValueError):
        nf.NVFP4Tensor.from_te(SimpleNamespace(_rowwise_data=None, _columnwise_data=None))


def test_auto_picks_exact_for_decode_and_int8_beyond():
    w = nf.quantize(normal((112, 256), seed=31))
    for tokens in (1, nf.AUTO_EXACT_MAX_ROWS, nf.AUTO_EXACT_MAX_ROWS + 1, 50):
        x = normal((tokens, 256), torch.bfloat16, seed=32 + tokens)
        chosen = "exact" if tokens <= nf.AUTO_EXACT_MAX_ROWS else "int8"
        assert torch.equal(nf.linear(x, w), nf.linear(x, w, act=chosen))
    with pytest.raises(ValueError):
        nf.linear(x, w, act="fp8")


def test_leading_dimensions_accumulation_amax_and_strided_views():
    w = nf.quantize(normal((80, 128), seed=33))
    x = normal((2, 4, 128), torch.bfloat16, seed=34)
    assert tuple(nf.linear(x, w).shape) == (2, 4, 80)
    flat = x.reshape(8, 128)
    start = normal((8, 80), torch.float32, seed=35)
    acc = start.clone()
    peak = torch.zeros(1, device=GPU)
    nf.linear(flat, w, out=acc, beta=1.0, act="exact", amax_out=peak)
    assert_linear(acc, flat, w, beta=1.0, before=start)
    assert abs(peak.item() - acc.abs().max().item()) <= 2.0 ** -7 * peak.item()
    wide = normal((12, 384), torch.bfloat16, seed=36)
    window = wide[:, 64:320]                                     # rows 768 bytes apart, 256 values each
    w2 = nf.quantize(normal((72, 256), seed=37))
    for act in ("exact", "int8"):
        assert torch.equal(nf.linear(window, w2, act=act), nf.linear(window.contiguous(), w2, act=act))


def test_module_checkpoint_names_and_in_place_conversion():
    torch.manual_seed(3)
    dense = torch.nn.Linear(320, 112).to(GPU).bfloat16()
    layer = nf.NVFP4Linear.from_linear(dense, act="exact")
    assert set(layer.state_dict()) == {"weight", "weight_scale", "weight_scale_2", "bias"}
    assert layer.weight.dtype == torch.uint8 and layer.weight_scale.dtype == torch.float8_e4m3fn and layer.weight_scale_2.dtype == torch.float32
    x = normal((6, 320), torch.bfloat16, seed=38)
    assert_linear(layer(x), x, layer.nvfp4_weight(), dense.bias.detach())
    twin = nf.NVFP4Linear(320, 112, device=GPU, act="exact")
    twin.load_state_dict(layer.state_dict())
    assert torch.equal(twin(x), layer(x))
    assert nf.NVFP4Linear.from_linear(dense, act="int8")(normal((20, 320), torch.bfloat16, seed=39)).shape == (20, 112)
    net = torch.nn.Sequential(torch.nn.Linear(192, 64), torch.nn.GELU(), torch.nn.Linear(64, 40), torch.nn.Linear(40, 8)).to(GPU).bfloat16()
    assert nf.quantize_linear_(net) is net
    assert [type(m).__name__ for m in net] == ["NVFP4Linear", "GELU", "NVFP4Linear", "Linear"]   # 40 inputs: not a multiple of 64
    assert net(normal((5, 192), torch.bfloat16, seed=40)).shape == (5, 8)


def test_header_version_matches_the_package():
    header = open(os.path.join(nf.get_include()[0], "nvfp4effma.h")).read()
    assert re.search(r'#define\s+NVFP4EFFMA_VERSION\s+"([^"]+)"', header).group(1) == nf.__version__.split("+")[0]


def test_bad_arguments_raise_the_documented_exception_types():
    w = nf.quantize(normal((64, 128), seed=41))
    x = normal((3, 128), torch.bfloat16, seed=42)
    bad = [
        (ValueError, lambda: nf.quantize(normal((4, 40)))),                                     # 40 is not a multiple of 16
        (ValueError, lambda: nf.quantize(torch.zeros(4, 32))),                                  # host memory
        (TypeError, lambda: nf.quantize(torch.zeros(4, 32, dtype=torch.int64, device=GPU))),
        (ValueError, lambda: nf.quantize(x, block="8x8")),
        (ValueError, lambda: nf.quantize(x, four_over_six="max")),
        (ValueError, lambda: nf.quantize(x, row_scaled=True, columnwise=True)),
        (ValueError, lambda: nf.quantize(x, columnwise=True)),                                  # 3 rows: not whole 16-row blocks
        (ValueError, lambda: nf.linear(normal((3, 64), torch.bfloat16), w)),                    # 64 features against 128
        (TypeError, lambda: nf.linear(x, w.data)),
        (ValueError, lambda: nf.linear(x, w, beta=1.0)),                                        # beta without out
        (ValueError, lambda: nf.linear(x, w, out=torch.zeros(3, 64, device=GPU), out_dtype=torch.bfloat16)),
        (TypeError, lambda: nf.dequantize(x)),
        (ValueError, lambda: nf.NVFP4Linear(96, 16)),
        (TypeError, lambda: nf.TCWeight(w.data)),
        (ValueError, lambda: nf.TCWeight(w, "fp8")),
    ]
    for exc, call in bad:
        with pytest.raises(exc):
            call()


# ---- the operator layer ------------------------------------------------------------------------------------------------------------
def test_operators_pass_opcheck_and_trace_without_graph_breaks():
    """``torch.ops.nvfp4effma.*`` carry schemas (mutation annotations included) and Meta kernels that agree with the CUDA
    ones, and ``torch.compile`` traces functions built on them as opaque nodes (reference test_nvfp4effma.py:514-538)."""
    ops = torch.ops.nvfp4effma
    w = nf.quantize(normal((128, 128), seed=43))
    x = normal((36, 128), torch.bfloat16, seed=44)
    xq = nf.quantize_int8(x)
    wo = w._operand()
    tests = ("test_schema", "test_faketensor")
    torch.library.opcheck(ops.quantize_int8, (x,), test_utils=tests)
    torch.library.opcheck(ops.dequantize, (wo.data, wo.scales, wo.glob, wo.flags, wo.scale_max, 128, torch.float32), test_utils=tests)
    torch.library.opcheck(ops.swizzle_scales, (wo.scales, 128, 128, True), test_utils=tests)
    torch.library.opcheck(ops.quantize_ex, (x, True, False, None, None, 4, 0, 1, 0, True, True), test_utils=tests)
    torch.library.opcheck(ops.linear, (xq.data, xq.scales, None, 0, 0, wo.data, wo.scales, wo.glob, wo.flags, wo.scale_max, 128, None, torch.bfloat16,
                                       1.0, True, None), test_utils=tests)
    torch.library.opcheck(ops.linear_out, (x, None, None, 0, 0, wo.data, wo.scales, wo.glob, wo.flags, wo.scale_max, 128, None,
                                           torch.zeros(36, 128, device=GPU), 1.0, 1.0, False, None), test_utils=tests)
    image = ops.tc_image(0, wo.data, wo.scales, wo.flags, 128)
    torch.library.opcheck(ops.tc_image, (1, x, None, 0, 128), test_utils=tests)
    torch.library.opcheck(ops.linear_tc, (ops.tc_image(1, x, None, 0, 128), 2, None, 0, 0, 36, image, wo.glob, wo.flags, wo.scale_max, 128, 128, None,
                                          torch.bfloat16, 1.0, False), test_utils=tests)

    def fn(a):
        return nf.dequantize(w, torch.float32).sum() + nf.linear(nf.quantize_int8(a), w).float().sum()

    compiled = torch.compile(fn, backend="aot_eager", fullgraph=True)
    assert torch.allclose(compiled(x), fn(x))
