"""CPU tests of the oracle: pins against the reference (golden folds of its codecs, its torch quantizer statement) and
self-consistency of the layout helpers.  No GPU."""
import json
import os

import numpy as np
import pytest

import oracle as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("which,name", [(O.ENC_E4M3, "e4m3"), (O.ENC_E2M1, "e2m1"), (O.ENC_UE5M3, "ue5m3"), (O.ENC_BF16, "bf16")])
def test_encoders_equal_reference_on_every_fp32(which, name):
    want = int(json.load(open(os.path.join(GOLD, "codec_folds.json")))[name], 16)
    assert O.encoder_fold(which) == want


def test_encoder_known_answers():
    # the reference's probe values and the rounding edges of each format
    x = np.array([0.25, 0.26, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 5.01, 6.0, 7.0, -0.0, -0.2, -6.5], np.float32)
    assert list(O.encode(O.ENC_E2M1, x)) == [0, 1, 2, 2, 4, 4, 6, 6, 7, 7, 7, 8, 8, 15]
    assert int(O.encode(O.ENC_E4M3, np.array([448.0], np.float32))[0]) == 0x7E
    assert int(O.encode(O.ENC_E4M3, np.array([1e9], np.float32))[0]) == 0x7E
    assert int(O.encode(O.ENC_E4M3, np.array([2.0 ** -9], np.float32))[0]) == 0x01
    assert int(O.encode(O.ENC_E4M3, np.array([2.0 ** -10], np.float32))[0]) == 0x00  # tie to even (0)
    assert int(O.encode(O.ENC_E4M3, np.array([3 * 2.0 ** -10], np.float32))[0]) == 0x02  # tie to even (2)
    assert int(O.encode(O.ENC_UE5M3, np.array([114688.0], np.float32))[0]) == 0xFE
    assert int(O.encode(O.ENC_UE5M3, np.array([-1.0], np.float32))[0]) == 0


def test_decoders():
    assert [O.e2m1_value(n) for n in range(8)] == [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    assert O.e2m1_value(15) == -6.0
    assert O.e4m3_value(0x7E) == 448.0 and O.e4m3_value(0x01) == 2.0 ** -9 and O.e4m3_value(0x38) == 1.0
    assert O.ue5m3_value(0xFE) == 114688.0 and O.ue5m3_value(0x01) == 2.0 ** -17
    # encode(decode(code)) is the identity on every finite code
    codes = np.arange(0x7F, dtype=np.uint32)
    vals = np.array([O.e4m3_value(int(c)) for c in codes], np.float32)
    assert np.array_equal(O.encode(O.ENC_E4M3, vals), codes)
    codes = np.arange(0xFF, dtype=np.uint32)
    vals = np.array([O.ue5m3_value(int(c)) for c in codes], np.float32)
    assert np.array_equal(O.encode(O.ENC_UE5M3, vals), codes)


def test_swizzled_addressing_matches_its_definition():
    # ScaleIdx{-512}.at(129, 5) = 66065: the value the reference's own codec returns for this probe
    assert O.scale_pos(True, 0, 512 * 16, 129, 5) == 66065
    rows, cols = 300, 1056
    sc = (cols // 16 + 3) // 4 * 4
    seen = set()
    for r in range(rows):
        for c in range(cols // 16):
            p = O.scale_pos(True, 0, cols, r, c)
            assert p == ((r // 128) * (sc // 4) + c // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + c % 4
            seen.add(p)
    assert len(seen) == rows * (cols // 16) and max(seen) < O.scale_bytes(True, 0, rows, cols)


def test_swizzle_round_trip():
    rng = np.random.default_rng(3)
    for rows, cols in ((517, 1056), (3, 16), (128, 64)):
        ld = cols // 16 + 5
        lin = rng.integers(0, 256, rows * ld, dtype=np.uint8)
        swz = O.swizzle_scales(lin, ld, rows, cols, True)
        back = O.swizzle_scales(swz, ld, rows, cols, False, dst=np.full(rows * ld, 0xEE, np.uint8))
        l2, b2 = lin.reshape(rows, ld), back.reshape(rows, ld)
        assert np.array_equal(b2[:, : cols // 16], l2[:, : cols // 16]) and np.all(b2[:, cols // 16:] == 0xEE)


def _golden_cases():
    g = np.load(os.path.join(GOLD, "quant_torch_ref.npz"))
    recipes = [r.split(":") for r in g["recipes"]] + [["given_g", "1", "0", "448", "0"]]
    return g, recipes


@pytest.mark.parametrize("dn", ["bf16", "f32"])
def test_quantizer_equals_reference_torch_statement(dn):
    g, recipes = _golden_cases()
    x = g[f"x_{dn}"]
    for name, tile, fos, smax, rs in recipes:
        tile, fos, smax, rs = int(tile), int(fos), int(smax), int(rs)
        given = name == "given_g"
        flags = 0 if given else O.GLOBAL_AMAX | (O.PER_ROW if rs else 0)
        glob = g[f"{dn}/{name}/global"] if given else np.zeros(67 if rs else 1, np.float32)
        d = O.Fp4(67, 320, flags=flags, scale_max=0 if given else smax, glob=glob)
        O.quantize(x, d, tile=tile, fos=fos, compute_amax=not given)
        assert np.array_equal(d.data.reshape(67, 160), g[f"{dn}/{name}/data"]), name
        assert np.array_equal(d.scales.reshape(67, 20), g[f"{dn}/{name}/scales"]), name
        if not given:
            assert np.array_equal(d.glob, g[f"{dn}/{name}/global"]), name


def test_quantize_dequantize_properties():
    rng = np.random.default_rng(5)
    x = rng.standard_normal((64, 256)).astype(np.float32)
    for flags in (O.GLOBAL_AMAX, O.GLOBAL_AMAX | O.SWIZZLED, O.GLOBAL_AMAX | O.UE5M3):
        d = O.Fp4(64, 256, flags=flags, glob=np.zeros(1, np.float32))
        amax = O.quantize(x, d, compute_amax=True)
        assert amax == np.abs(x).max() == d.glob[0]
        y, _ = O.dequantize(d)
        # every value is within half a grid step (block max / 6 * 1.0 at most ... coarse bound: 1/4 of the block max)
        bmax = np.abs(x).reshape(64, 16, 16).max(-1).repeat(16, -1)
        assert np.all(np.abs(y - x) <= 0.26 * bmax + 1e-6)
        # idempotence: quantizing the dequantized values with the same global reproduces the codes
        d2 = O.Fp4(64, 256, flags=flags, glob=d.glob.copy())
        O.quantize(y, d2, compute_amax=False)
        assert np.array_equal(d2.data, d.data)


def test_gemm_orders_agree_within_bound_and_linearity():
    rng = np.random.default_rng(7)
    from util import rand_fp4, rand_q8, rand_dense
    m, n, k = 37, 5, 192
    A = rand_fp4(rng, m, k, glob=0.375)
    for B in (rand_fp4(rng, n, k, glob=1.75), rand_q8(rng, n, k, glob=1.75), O.Dense(O.BF16, rand_dense(rng, O.BF16, n * k, 2.0), k)):
        r0 = O.gemm(m, n, k, A, B, D_dtype=O.FP32, want_ref=True)
        r1 = O.gemm(m, n, k, A, B, D_dtype=O.FP32, order=1)
        d0, d1 = r0["D"].reshape(n, m), r1["D"].reshape(n, m)
        assert np.all(np.abs(d0 - r0["ref64"]) <= r0["bound"]) and np.all(np.abs(d1 - r0["ref64"]) <= r0["bound"])
        # alpha scales the result exactly by a power of two
        r2 = O.gemm(m, n, k, A, B, D_dtype=O.FP32, alpha=4.0)
        assert np.array_equal(r2["D"], 4.0 * r0["D"])


def test_norm_scale_and_epilogue_ex():
    rng = np.random.default_rng(9)
    parts = (rng.integers(0, 4096, 37) / 64.0).astype(np.float32)
    s = O.norm_scale(parts, 1.0 / 1024.0, 1e-6)
    assert abs(s - 1.0 / np.sqrt(parts.astype(np.float64).sum() / 1024.0 + 1e-6)) < 1e-6 * s
    m, n = 32, 3
    acc = rng.standard_normal((n, m)).astype(np.float32)
    w2 = np.ones(m, np.float32)
    r = O.epilogue_ex(m, n, acc, mask=4, w2=w2, D_dtype=O.FP32, d2_dtype=O.FP32)
    assert np.array_equal(r["d2"].reshape(n, m), acc)
    want = (acc.reshape(n, 2, 16).astype(np.float32) ** 2)
    assert np.allclose(r["sq"].reshape(n, 2), want.sum(-1), rtol=1e-6)
    r = O.epilogue_ex(m, n, acc, mask=2, D_dtype=O.FP32)
    g, u = acc.reshape(n, 2, 2, 8)[:, :, 0, :], acc.reshape(n, 2, 2, 8)[:, :, 1, :]
    assert np.allclose(r["D"].reshape(n, 2, 8), g / (1 + np.exp(-g)) * u, rtol=1e-6)
