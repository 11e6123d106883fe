"""The Python surface (quantize / linear / TCWeight / NVFP4Linear) on the GPU, in the shape of the reference's own pytest
(binds/python/tests/test_nvfp4effma.py there): quantization bit for bit against the CPU oracle, linear layers against a
float64 product of the decoded operands within half an ulp of the output type plus the FP32 accumulation bound."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

import oracle  # noqa: E402

nf = pytest.importorskip("nvfp4effma_b200") if torch.cuda.is_available() else None
DEV = "cuda"
E2M1 = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], dtype=torch.float64)


def rand(shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(DEV).to(dtype)


def linear_scales(t):
    """Scale bytes of t as a linear [rows, cols / 16] uint8 tensor."""
    d, s, *_ = t._flat()
    s = s.view(torch.uint8)
    rows, nb = d.shape[0], t.cols // 16
    if not t.swizzled:
        return s[:rows, :nb]
    pr, pc = s.shape
    return s.reshape(pr // 128, pc // 4, 32, 4, 4).permute(0, 3, 2, 1, 4).reshape(pr, pc)[:rows, :nb]


def scale_values(t):
    s = linear_scales(t)
    if not t.ue5m3:
        return s.contiguous().view(torch.float8_e4m3fn).double()
    e, m = (s.long() >> 3) & 31, (s.long() & 7).double()
    return torch.where(e > 0, torch.ldexp(1 + m / 8, e - 15), m * 2.0 ** -17)


def values(t):
    """float64 values of an NVFP4Tensor: e2m1 * block scale * decode factor."""
    d = t._flat()[0]
    codes = torch.stack([d & 15, d >> 4], -1).reshape(d.shape[0], -1)[:, :t.cols].long()
    v = E2M1.to(d.device)[codes]
    g = t.global_scale.double() if t.global_scale is not None else torch.ones(1, dtype=torch.float64, device=d.device)
    if t.global_is_amax:
        g = g / (6.0 * (t.scale_max or (114688 if t.ue5m3 else 448)))
    g = g.reshape(-1, 1) if g.numel() > 1 else g
    return (v * scale_values(t).repeat_interleave(16, -1) * g).reshape(*t.shape)


def check_close(y, ref, mag, k, out_dtype):
    eps = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 2.0 ** -24}[out_dtype]
    err = (y.double() - ref).abs()
    bound = eps * ref.abs() + k * 2.0 ** -23 * mag + 1e-30
    assert bool((err <= bound * 1.0001).all()), f"max excess {float((err - bound).max())}"


RECIPES = [dict(), dict(block="16x16"), dict(four_over_six="mae"), dict(four_over_six="mse", block="16x16"),
           dict(four_over_six="mae", scale_max=448), dict(row_scaled=True), dict(row_scaled=True, four_over_six="mse"),
           dict(swizzled=True), dict(block="16x16", swizzled=True, four_over_six="mae")]


def rid(r):
    return ",".join(f"{k}={v}" for k, v in r.items()) or "default"


@pytest.mark.parametrize("recipe", RECIPES, ids=rid)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_quantize_equals_the_oracle(recipe, dtype):
    x = rand((67, 320), dtype, 3.0)
    x[3, :16] = 0
    x[5, 16:32] *= 1e-30
    x[7] = 0
    q = nf.quantize(x, **recipe)
    fos = {"mae": 1, "mse": 2}.get(recipe.get("four_over_six"), 0)
    smax = recipe.get("scale_max", 256 if fos else 0)
    rows = x.shape[0]
    flags = oracle.GLOBAL_AMAX | (oracle.PER_ROW if recipe.get("row_scaled") else 0)
    dst = oracle.Fp4(rows, 320, flags=flags, scale_max=smax, glob=0.0)
    oracle.quantize(x.float().cpu().numpy(), dst, tile=16 if recipe.get("block") == "16x16" else 1, fos=fos, compute_amax=True)
    assert np.array_equal(q._flat()[0].cpu().numpy().reshape(-1), dst.data)
    assert np.array_equal(linear_scales(q).cpu().numpy(), dst.scales.reshape(rows, 20)), "block scales differ"
    assert q.global_is_amax and np.array_equal(q.global_scale.cpu().numpy(), dst.glob.reshape(-1))


def test_quantize_given_global_and_ue5m3():
    x = rand((40, 256), torch.bfloat16, 2.0)
    g = torch.tensor([0.004], device=DEV)
    amax = torch.zeros(1, device=DEV)
    q = nf.quantize(x, g, amax=amax)
    assert not q.global_is_amax and float(amax) == float(x.float().abs().max())
    assert float((values(q) - x.double()).abs().max()) <= 0.5 * float(x.abs().max())
    u = nf.quantize(x, scale_dtype="ue5m3")
    assert u.ue5m3 and u.scales.dtype == torch.uint8
    assert float((values(u) - x.double()).abs().max()) <= 0.5 * float(x.abs().max())


@pytest.mark.parametrize("block", ["1x16", "16x16"])
def test_columnwise_is_the_quantized_transpose(block):
    x = rand((96, 160), torch.bfloat16, 1.5, seed=3)
    q = nf.quantize(x, block=block, columnwise=True)
    c = q.columnwise
    assert c.shape == (160, 96) and c.global_is_amax and torch.equal(c.global_scale, q.global_scale)
    ref = nf.quantize(x.t().contiguous(), block=block)
    assert torch.equal(c._flat()[0][:, :48], ref.data) and torch.equal(scale_values(c), scale_values(ref))
    if block == "16x16":
        t = q.transpose_2d()
        assert torch.equal(t.data, c._flat()[0][:, :48]) and torch.equal(scale_values(t), scale_values(c))


def test_scale_layouts_and_dequantize():
    x = rand((200, 192), torch.float32, 4.0, seed=4)
    for recipe in RECIPES + [dict(scale_dtype="ue5m3", swizzled=True)]:
        q = nf.quantize(x, **recipe)
        o = q.with_scale_layout(not q.swizzled)
        assert o.swizzled != q.swizzled and torch.equal(scale_values(q), scale_values(o))
        for t in (q, o):
            y = nf.dequantize(t, torch.float32)
            assert torch.allclose(y.double(), values(t), rtol=2 ** -22, atol=0), rid(recipe)


@pytest.mark.parametrize("recipe", RECIPES[:6] + [dict(scale_dtype="ue5m3")], ids=rid)
@pytest.mark.parametrize("T", [1, 5, 40, 260])
def test_linear_every_weight_format(recipe, T):
    N, K = 130, 256
    w = nf.quantize(rand((N, K), seed=14), **recipe)
    x = rand((T, K), torch.bfloat16, seed=15)
    wv = values(w)
    y = nf.linear(x, w, act="exact", out_dtype=torch.float32)
    check_close(y, x.double() @ wv.t(), x.double().abs() @ wv.abs().t(), K, torch.float32)
    xq = nf.quantize(x, row_scaled=T > 1, swizzled=True)
    xv = values(xq)
    y = nf.linear(xq, w, out_dtype=torch.float32)
    check_close(y, xv @ wv.t(), xv.abs() @ wv.abs().t(), K, torch.float32)


def test_backward_gemms_with_columnwise_halves():
    Tk, I, O = 128, 192, 64
    w = nf.quantize(rand((O, I), seed=16), block="16x16", columnwise=True)
    x = nf.quantize(rand((Tk, I), seed=17), columnwise=True)
    dy = nf.quantize(rand((Tk, O), seed=18), columnwise=True)
    wv, dyv = values(w), values(dy)
    wcv = values(w.columnwise)
    assert torch.equal(wcv, wv.t())
    dx = nf.linear(dy, w.columnwise, out_dtype=torch.float32)
    check_close(dx, dyv @ wcv.t(), dyv.abs() @ wcv.abs().t(), O, torch.float32)
    dw = nf.linear(dy.columnwise, x.columnwise, out_dtype=torch.float32)
    a, b = values(dy.columnwise), values(x.columnwise)
    check_close(dw, a @ b.t(), a.abs() @ b.abs().t(), Tk, torch.float32)


def test_from_transformer_engine_tensor():
    from types import SimpleNamespace
    x = rand((144, 128), torch.bfloat16, seed=19)
    q = nf.quantize(x, swizzled=True, columnwise=True, four_over_six="mae")
    te = SimpleNamespace(_rowwise_data=q.data, _rowwise_scale_inv=q.scales.view(torch.uint8), _amax_rowwise=q.global_scale,
                         _columnwise_data=q.columnwise.data, _columnwise_scale_inv=q.columnwise.scales.view(torch.uint8),
                         _amax_columnwise=q.columnwise.global_scale, _with_gemm_swizzled_scales=True, _row_scaled_nvfp4=False,
                         _nvfp4_e4m3_max=256, _scale_dtype="DType.kFloat8E4M3")
    t = nf.NVFP4Tensor.from_te(te)
    assert t.swizzled and t.global_is_amax and t.scale_max == 256 and t.columnwise is not None
    assert torch.equal(nf.dequantize(t, torch.float32), nf.dequantize(q, torch.float32))
    w = nf.quantize(rand((64, 128), seed=20))
    assert torch.equal(nf.linear(t, w, out_dtype=torch.float32), nf.linear(q, w, out_dtype=torch.float32))


@pytest.mark.parametrize("T", [1, 3, 8, 9, 200])
@pytest.mark.parametrize("xdtype", [torch.bfloat16, torch.float16, torch.float32])
def test_linear_dense_x(T, xdtype):
    N, K = 192, 320
    w = nf.quantize(rand((N, K), seed=1))
    x = rand((T, K), xdtype, seed=2)
    bias = rand((N,), xdtype, seed=3)
    y = nf.linear(x, w, bias, act="exact")
    assert y.shape == (T, N) and y.dtype == xdtype
    wv = values(w)
    check_close(y, x.double() @ wv.t() + bias.double(), x.double().abs() @ wv.abs().t(), K, xdtype)


@pytest.mark.parametrize("T", [1, 5, 8, 33, 260])
def test_linear_nvfp4_x(T):
    N, K = 130, 256
    w = nf.quantize(rand((N, K), seed=4))
    x = nf.quantize(rand((T, K), seed=5))
    y = nf.linear(x, w, out_dtype=torch.float32)
    assert y.shape == (T, N) and y.dtype == torch.float32
    xv, wv = values(x), values(w)
    check_close(y, xv @ wv.t(), xv.abs() @ wv.abs().t(), K, torch.float32)


@pytest.mark.parametrize("T", [1, 8, 20, 200])
def test_linear_int8_activations(T):
    N, K = 130, 256
    w = nf.quantize(rand((N, K), seed=10))
    x = rand((T, K), torch.bfloat16, seed=11)
    xq = nf.quantize_int8(x)
    q, s = xq.data, xq.scales
    xb = x.float().reshape(T, -1, 16)
    bmax = xb.abs().amax(-1)
    assert torch.equal(s, bmax / torch.full_like(bmax, 127.0))
    assert torch.equal(q.float(), torch.where(s[..., None] > 0, torch.round(xb / s[..., None]), torch.zeros_like(xb)).reshape(T, K))
    xv, wv = q.double() * s.double().repeat_interleave(16, -1), values(w)
    y = nf.linear(x, w, act="int8", out_dtype=torch.float32)
    check_close(y, xv @ wv.t(), xv.abs() @ wv.abs().t(), K // 16, torch.float32)
    assert nf.linear(x, w, act="int8").dtype == torch.bfloat16
    m = nf.NVFP4Linear.from_linear(torch.nn.Linear(K, N).cuda().bfloat16(), act="int8")
    assert m(x).shape == (T, N)


@pytest.mark.parametrize("T", [1, 8, 200])
def test_int8_tensor(T):
    N, K = 130, 256
    w = nf.quantize(rand((N, K), seed=10))
    x = rand((2, T, K), torch.float16, seed=11)
    xq = nf.quantize_int8(x)
    assert isinstance(xq, nf.Int8Tensor) and xq.shape == (2, T, K) and xq.scales.shape == (2, T, K // 16)
    assert xq.dtype == torch.float16 and nf.Int8Tensor.from_float(x).data.equal(xq.data)
    y = nf.linear(xq, w)
    assert y.dtype == torch.float16 and y.shape == (2, T, N)
    assert torch.equal(y, nf.linear(x, w, act="int8"))
    assert torch.equal(nf.linear(xq, w, out_dtype=torch.float32), nf.linear(x, w, act="int8", out_dtype=torch.float32))
    xd = (xq.data.float().reshape(-1, K // 16, 16) * xq.scales.reshape(-1, K // 16, 1)).reshape(2, T, K)
    assert torch.equal(xq.dequantize(torch.float32), xd) and xq.dequantize().dtype == torch.float16
    with pytest.raises(ValueError):
        nf.linear(nf.quantize_int8(rand((T, 128), seed=1)), w)
    with pytest.raises(TypeError):
        nf.Int8Tensor(xq.data.float(), xq.scales)
    with pytest.raises(ValueError):
        nf.Int8Tensor(xq.data, xq.scales[..., :4])


@pytest.mark.parametrize("T", [1, 3, 8, 9, 200])
@pytest.mark.parametrize("act", ["exact", "int8", "nvfp4"])
def test_tc_weight(T, act):
    N, K = 192, 320
    w = nf.quantize(rand((N, K), seed=30))
    tw = nf.TCWeight(w, act)
    assert tw.shape == (N, K)
    x = rand((T, K), torch.bfloat16, seed=31)
    bias = rand((N,), torch.float32, seed=32)
    if act == "exact":
        xv = x.double()
    elif act == "int8":
        xq = nf.quantize_int8(x)
        xv = xq.data.double() * xq.scales.double().repeat_interleave(16, -1)
    else:
        xv = values(nf.quantize(x))
    wv = values(w)
    y = nf.linear(x, tw, bias, out_dtype=torch.float32)
    assert y.shape == (T, N) and y.dtype == torch.float32
    check_close(y, xv @ wv.t() + bias.double(), xv.abs() @ wv.abs().t(), K, torch.float32)
    assert nf.linear(x, tw).dtype == torch.bfloat16
    acc = torch.ones(T, N, device=DEV)
    nf.linear(x, tw, out=acc, beta=1.0)
    check_close(acc, xv @ wv.t() + 1.0, xv.abs() @ wv.abs().t() + 1.0, K, torch.float32)
    if act != "exact":
        xq = nf.quantize_int8(x) if act == "int8" else nf.quantize(x)
        assert torch.equal(nf.linear(xq, tw, out_dtype=torch.float32), nf.linear(x, tw, out_dtype=torch.float32))
    with pytest.raises(ValueError):
        nf.linear(x, tw, act="int8" if act == "exact" else "exact")


def test_get_include():
    import re
    inc = nf.get_include()[0]
    hdr = open(os.path.join(inc, "nvfp4effma.h")).read()
    assert re.search(r'#define NVFP4EFFMA_VERSION "([^"]+)"', hdr).group(1) == nf.__version__.split("+")[0]


def test_linear_auto_activations():
    w = nf.quantize(rand((96, 256), seed=12))
    for T in (1, 2, 3, 40):
        x = rand((T, 256), torch.bfloat16, seed=13 + T)
        want = "exact" if T <= nf.AUTO_EXACT_MAX_ROWS else "int8"
        assert torch.equal(nf.linear(x, w), nf.linear(x, w, act=want))
    with pytest.raises(ValueError):
        nf.linear(x, w, act="fp8")


def test_linear_batched_input_and_accumulate():
    w = nf.quantize(rand((64, 128), seed=6))
    x = rand((2, 3, 128), torch.bfloat16, seed=7)
    assert nf.linear(x, w).shape == (2, 3, 64)
    acc = torch.ones(6, 64, device=DEV)
    nf.linear(x.reshape(6, 128), w, out=acc, beta=1.0, act="exact")
    wv = values(w)
    ref = x.reshape(6, 128).double() @ wv.t() + 1
    check_close(acc, ref, x.reshape(6, 128).double().abs() @ wv.abs().t() + 1, 128, torch.float32)


def test_strided_inputs_are_copied():
    w = nf.quantize(rand((64, 256), seed=8))
    big = rand((10, 320), torch.bfloat16, seed=9)
    x = big[:, 32:288]
    assert torch.equal(nf.linear(x, w, act="exact"), nf.linear(x.contiguous(), w, act="exact"))
    assert torch.equal(nf.linear(x, w), nf.linear(x.contiguous(), w))


def test_grouped_linear_is_not_part_of_this_build():
    with pytest.raises(NotImplementedError):
        nf.grouped_linear()


def test_nvfp4_linear_module():
    torch.manual_seed(0)
    lin = torch.nn.Linear(256, 96).cuda().bfloat16()
    m = nf.NVFP4Linear.from_linear(lin, act="exact")
    x = rand((5, 256), torch.bfloat16, seed=40)
    wv = values(m.nvfp4_weight())
    check_close(m(x), x.double() @ wv.t() + lin.bias.double(), x.double().abs() @ wv.abs().t(), 256, torch.bfloat16)
    m2 = nf.NVFP4Linear(256, 96, device=DEV, act="exact")
    m2.load_state_dict(m.state_dict())
    assert torch.equal(m2(x), m(x))
    seq = nf.quantize_linear_(torch.nn.Sequential(torch.nn.Linear(128, 64), torch.nn.ReLU(), torch.nn.Linear(64, 50)).cuda().bfloat16())
    assert isinstance(seq[0], nf.NVFP4Linear) and isinstance(seq[2], nf.NVFP4Linear)
    assert seq(rand((4, 128), torch.bfloat16)).shape == (4, 50)


def test_rejects_bad_input():
    w = nf.quantize(rand((64, 128), seed=1))
    with pytest.raises(ValueError):
        nf.quantize(rand((4, 24)))
    with pytest.raises(ValueError):
        nf.quantize(torch.zeros(4, 32))  # CPU tensor
    with pytest.raises(TypeError):
        nf.quantize(torch.zeros(4, 32, dtype=torch.int32, device=DEV))
    with pytest.raises(ValueError):
        nf.linear(rand((3, 64), torch.bfloat16), w)
    with pytest.raises(TypeError):
        nf.linear(rand((3, 128), torch.bfloat16), w.data)
    with pytest.raises(ValueError):
        nf.linear(rand((3, 128), torch.bfloat16), w, beta=1.0)
    with pytest.raises(ValueError):
        nf.NVFP4Linear(100, 10)
