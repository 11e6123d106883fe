"""The C-ABI library loads and exports every symbol the headers declare; the host-side validation rejects bad arguments
before touching a device (none of these calls reaches a kernel launch).  No GPU."""
import ctypes
import os
import re

import pytest

from nvfp4effma_b200 import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(nvfp4a_[a-z0-9_]+)\s*\(", text))


def test_every_declared_symbol_is_exported():
    names = _declared("nvfp4effma.h") | _declared("nvfp4effma_b200.h")
    assert len(names) >= 21
    for n in sorted(names):
        assert hasattr(L.lib, n), f"{n} is declared but not exported"
        assert n in L.EXPORTS, f"{n} has no ctypes prototype"


def test_struct_layouts_match_the_reference_abi():
    # field order / offsets of nvfp4a_tensor on LP64 (reference include/nvfp4effma.h:46-57)
    T = L.Tensor
    assert [f[0] for f in T._fields_] == ["data", "dtype", "block_scale", "ld_scale", "global_scale", "amax", "flags", "scale_max"]
    assert (T.data.offset, T.dtype.offset, T.block_scale.offset, T.ld_scale.offset, T.global_scale.offset, T.amax.offset,
            T.flags.offset, T.scale_max.offset) == (0, 8, 16, 24, 32, 40, 48, 52)
    assert ctypes.sizeof(T) == 56
    assert ctypes.sizeof(L.QuantConfig) == 12
    E = L.Epilogue
    assert (E.norm_parts.offset, E.swiglu.offset, E.d2.offset, E.w2.offset, E.sq.offset, E.ld_sq.offset) == (0, 24, 32, 48, 64, 72)


def test_status_strings_and_error_text():
    assert L.lib.nvfp4a_status_string(0) == b"NVFP4A_OK"
    assert L.lib.nvfp4a_status_string(2) == b"NVFP4A_NOT_SUPPORTED"
    st = L.lib.nvfp4a_swizzle_scales(None, None, 4, 16, 64, 1, None)
    assert st == L.INVALID_VALUE and b"NULL" in L.lib.nvfp4a_last_error()
    # a successful call clears the text: rows == 0 is a no-op that needs no device
    buf = (ctypes.c_uint8 * 16)()
    assert L.lib.nvfp4a_swizzle_scales(buf, buf, 4, 0, 64, 1, None) == L.OK
    assert L.lib.nvfp4a_last_error() == b""


def _fake(dtype, flags=0, scale_max=0, ld_scale=0, with_scales=True, addr=0x1000):
    return L.Tensor(addr, dtype, addr + 0x100000 if with_scales else None, ld_scale, None, None, flags, scale_max)


def test_gemm_argument_checks():
    A, B, D = _fake(L.NVFP4), _fake(L.BF16, with_scales=False), _fake(L.BF16, with_scales=False)
    call = lambda *a: L.lib.nvfp4a_gemm(*a)
    assert call(16, 4, 100, 1.0, A, 128, B, 128, 0.0, None, 0, D, 16, None, None) == L.INVALID_VALUE  # k % 64
    assert call(16, 4, 128, 1.0, A, 96, B, 128, 0.0, None, 0, D, 16, None, None) == L.INVALID_VALUE   # lda % 64
    assert call(16, 4, 128, 1.0, A, 128, B, 128, 0.0, None, 0, D, 8, None, None) == L.INVALID_VALUE   # ldd < m
    assert call(-1, 4, 128, 1.0, A, 128, B, 128, 0.0, None, 0, D, 16, None, None) == L.INVALID_VALUE
    assert call(0, 4, 128, 1.0, A, 128, B, 128, 0.0, None, 0, D, 16, None, None) == L.OK              # empty: no-op
    notfp4 = _fake(L.BF16, with_scales=False)
    assert call(16, 4, 128, 1.0, notfp4, 128, B, 128, 0.0, None, 0, D, 16, None, None) == L.NOT_SUPPORTED
    bad = _fake(L.NVFP4, scale_max=100)
    assert call(16, 4, 128, 1.0, bad, 128, B, 128, 0.0, None, 0, D, 16, None, None) == L.INVALID_VALUE
    assert b"scale_max" in L.lib.nvfp4a_last_error()
    mis = _fake(L.NVFP4, addr=0x1008)
    assert call(16, 4, 128, 1.0, mis, 128, B, 128, 0.0, None, 0, D, 16, None, None) == L.INVALID_VALUE
    swz = _fake(L.NVFP4, flags=L.SCALES_SWIZZLED, ld_scale=12)
    assert call(16, 4, 128, 1.0, swz, 128, B, 128, 0.0, None, 0, D, 16, None, None) == L.INVALID_VALUE
    grouped = L.lib.nvfp4a_gemm_grouped
    assert grouped(1, 16, 64, 4, 1.0, A, 64, B, 64, 0.0, None, 0, D, 16, None, None, None) == L.INVALID_VALUE   # seg is NULL
    assert b"seg" in L.lib.nvfp4a_last_error()
    seg = ctypes.c_void_p(0x1000)
    assert grouped(-1, 16, 64, 4, 1.0, A, 64, B, 64, 0.0, None, 0, D, 16, None, seg, None) == L.INVALID_VALUE
    assert grouped(2, 16, 64, 4, 1.0, A, 64, B, 64, 0.0, None, 0, D, 8, None, seg, None) == L.INVALID_VALUE     # ldd < m
    assert grouped(0, 16, 64, 4, 1.0, A, 64, B, 64, 0.0, None, 0, D, 16, None, seg, None) == L.OK               # no groups: no-op
    assert grouped(2, 16, 64, 0, 1.0, A, 64, B, 64, 0.0, None, 0, D, 16, None, seg, None) == L.OK               # no rows: no-op


def test_quantize_and_epilogue_argument_checks():
    src, dst = _fake(L.BF16, with_scales=False), _fake(L.NVFP4)
    q = lambda *a: L.lib.nvfp4a_quantize_ex(*a)
    assert q(src, 64, 4, 60, dst, 64, None, 0, None, None) == L.INVALID_VALUE       # cols % 16
    cfg = L.QuantConfig(8, 0, 0)
    assert q(src, 64, 4, 64, dst, 64, None, 0, ctypes.byref(cfg), None) == L.INVALID_VALUE  # tile_rows
    cfg = L.QuantConfig(1, 1, 0)
    assert q(src, 64, 4, 64, dst, 64, None, 0, ctypes.byref(cfg), None) == L.INVALID_VALUE  # 4over6 without amax global
    cfg = L.QuantConfig(1, 0, 1)
    assert q(src, 64, 4, 64, dst, 64, None, 0, ctypes.byref(cfg), None) == L.INVALID_VALUE  # compute_amax without storage
    assert q(src, 64, 4, 64, None, 64, None, 0, None, None) == L.INVALID_VALUE
    assert q(src, 64, 0, 64, dst, 64, None, 0, None, None) == L.OK
    A, B, D = _fake(L.NVFP4), _fake(L.BF16, with_scales=False), _fake(L.BF16, with_scales=False)
    ex = L.Epilogue()
    ex.swiglu = 1
    st = L.lib.nvfp4a_gemm_ex(24, 4, 128, 1.0, A, 128, B, 128, 0.0, None, 0, D, 24, None, ctypes.byref(ex), None)
    assert st == L.INVALID_VALUE and b"swiglu" in L.lib.nvfp4a_last_error()
    assert L.lib.nvfp4a_tc_image_bytes(L.TC_A16, L.NVFP4, 4096, 4096) == 32 * 16 * 18432
    assert L.lib.nvfp4a_tc_image_bytes(L.TC_A8, L.NVFP4, 129, 320) == 2 * 2 * 18432
    assert L.lib.nvfp4a_tc_image_bytes(L.TC_A16, L.BF16, 128, 256) == 0
    assert L.check(L.OK) is None
    with pytest.raises(ValueError):
        L.check(L.lib.nvfp4a_swizzle_scales(None, None, 4, 16, 64, 1, None))


def test_tensor_parallel_entries_reject_layouts_the_push_cannot_move():
    """The fused all-gather moves 16-byte vectors / TMA boxes: with world > 1, D's base, its column pitch and a shard row must be
    multiples of 16 bytes, and D must lie inside the rank's buffer -- INVALID_VALUE before any device is touched."""
    A, B = _fake(L.NVFP4, with_scales=False), _fake(L.BF16, with_scales=False, addr=0x2000)
    bufs = (ctypes.c_void_p * 2)(0x100000, 0x200000)
    flags = (ctypes.c_void_p * 2)(0x300000, 0x300100)
    ws = ctypes.c_void_p(0x400000)

    def gemv(d_addr, m, ldd, world=2):
        D = L.Tensor(d_addr, L.BF16, None, 0, None, None, 0, 0)
        return L.lib.nvfp4a_b200_gemv_tc_tp(m, 1, 256, 1.0, A, B, 256, D, ldd, None, None, bufs, flags, world, 0, None)

    def gemm(d_addr, m, ldd, world=2):
        D = L.Tensor(d_addr, L.BF16, None, 0, None, None, 0, 0)
        return L.lib.nvfp4a_b200_gemm_tc_tp(m, 64, 256, 1.0, A, B, D, ldd, None, None, ws, bufs, flags, world, 0, None)

    def gemv_deferred(d_addr, m, ldd, world=2):
        D = L.Tensor(d_addr, L.BF16, None, 0, None, None, 0, 0)
        return L.lib.nvfp4a_b200_gemv_tc_tp_deferred(m, 1, 256, 1.0, A, B, 256, D, ldd, None, None, bufs, flags, world, 0, 1, None)

    for call in (gemv, gemm, gemv_deferred):
        assert call(0x100002, 128, 256) == L.INVALID_VALUE and b"16 bytes" in L.lib.nvfp4a_last_error()     # base
        assert call(0x100000, 128, 260) == L.INVALID_VALUE and b"16 bytes" in L.lib.nvfp4a_last_error()     # pitch: 520 bytes
        assert call(0x100000, 132, 256) == L.INVALID_VALUE and b"16 bytes" in L.lib.nvfp4a_last_error()     # shard row: 264 bytes
        assert call(0x0FFFF0, 128, 256) == L.INVALID_VALUE and b"inside" in L.lib.nvfp4a_last_error()       # below the buffer
    bad_flags = (ctypes.c_void_p * 2)(0x300000, 0x300104)
    D = L.Tensor(0x100000, L.BF16, None, 0, None, None, 0, 0)
    assert L.lib.nvfp4a_b200_gemv_tc_tp(128, 1, 256, 1.0, A, B, 256, D, 256, None, None, bufs, bad_flags, 2, 0, None) == L.INVALID_VALUE
    assert L.lib.nvfp4a_b200_set_wait_limit(10) == -1 and L.lib.nvfp4a_b200_set_wait_limit(2000000000) == 0
    # the deferred form's other two entries: argument checks before any device is touched
    assert L.lib.nvfp4a_b200_tp_wait(None, 2, 0, None) == L.INVALID_VALUE
    assert L.lib.nvfp4a_b200_tp_wait(flags, 9, 0, None) == L.INVALID_VALUE and L.lib.nvfp4a_b200_tp_wait(flags, 2, 2, None) == L.INVALID_VALUE
    post = L.lib.nvfp4a_b200_tp_gather_post
    assert post(bufs, flags, 2, 0, 1, 512, 8, 256, None) == L.INVALID_VALUE        # column offset not a multiple of 16
    assert post(bufs, flags, 2, 0, 1, 512, 384, 256, None) == L.INVALID_VALUE      # the shard leaves the row
    assert post(None, flags, 2, 0, 1, 512, 0, 256, None) == L.INVALID_VALUE


def test_route_and_launch_knobs_take_their_documented_values():
    """The process-wide knobs of include/nvfp4effma_b200.h (no device needed): routes 0 .. 3, programmatic launch on / off, the
    one-read quantizer on / off; each setter returns what its header says."""
    old = L.lib.nvfp4a_b200_set_route(3)
    assert L.lib.nvfp4a_b200_set_route(2) == 3 and L.lib.nvfp4a_b200_set_route(1) == 2 and L.lib.nvfp4a_b200_set_route(0) == 1
    L.lib.nvfp4a_b200_set_route(old)
    assert L.lib.nvfp4a_b200_set_pdl(0) == 0 and L.lib.nvfp4a_b200_set_pdl(1) == 0
    assert L.lib.nvfp4a_b200_set_pair(2) == -1 and L.lib.nvfp4a_b200_set_pair(-1) == 0
    assert L.lib.nvfp4a_b200_set_gemv_splits(3) == -1 and L.lib.nvfp4a_b200_set_gemv_splits(0) == 0
    assert L.lib.nvfp4a_b200_last_launch() >= 0
