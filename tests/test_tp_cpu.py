"""Host logic of the tensor-parallel layers on CPU ranks (gloo, world size 2): row shards of a quantized weight, the
feature all-gather and its token-major reassembly.  The per-shard products come from the CPU oracle here; the CUDA layers
are covered by the GPU tests."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from nvfp4effma_b200.tensor import NVFP4Tensor
from nvfp4effma_b200.tp import gather_features, shard_bounds, shard_rows


def quantized(rows, cols, swizzled, seed):
    """A weight quantized on the host with a given per-tensor decode factor, as CPU torch tensors."""
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    g = np.float32(np.abs(w).max() / (6 * 448))
    q = oracle.Fp4(rows, cols, flags=oracle.SWIZZLED if swizzled else 0, glob=g)
    oracle.quantize(w, q)
    sc = torch.from_numpy(q.scales.copy())
    sc = sc.reshape((rows + 127) // 128 * 128, (cols // 16 + 3) // 4 * 4) if swizzled else sc.reshape(rows, cols // 16)
    t = NVFP4Tensor(torch.from_numpy(q.data.copy()).reshape(rows, cols // 2), sc, torch.tensor([g]), swizzled=swizzled)
    return w, q, t


def to_oracle(t):
    """NVFP4Tensor (CPU) -> oracle.Fp4"""
    rows, cols = t.shape
    q = oracle.Fp4(rows, cols, flags=oracle.SWIZZLED if t.swizzled else 0, glob=float(t.global_scale[0]))
    q.data[:] = t.data.contiguous().numpy().reshape(-1)
    q.scales[:] = t.scales.contiguous().view(torch.uint8).numpy().reshape(-1)
    return q


def test_shard_bounds():
    assert shard_bounds(6144, 8, 3) == (2304, 3072)
    assert [shard_bounds(28672, 8, r)[1] - shard_bounds(28672, 8, r)[0] for r in range(8)] == [3584] * 8
    with pytest.raises(ValueError):
        shard_bounds(4096 + 128, 8, 0)
    with pytest.raises(ValueError):
        shard_bounds(4096, 8, 8)


@pytest.mark.parametrize("swizzled", [False, True])
def test_a_shard_is_the_quantization_of_its_rows(swizzled):
    rows, cols, world = 512, 192, 2
    w, _, t = quantized(rows, cols, swizzled, 5)
    for r in range(world):
        a, b = shard_bounds(rows, world, r)
        sh = shard_rows(t, world, r)
        ref = oracle.Fp4(b - a, cols, flags=oracle.SWIZZLED if swizzled else 0, glob=float(t.global_scale[0]))
        oracle.quantize(w[a:b], ref)
        assert np.array_equal(sh.data.contiguous().numpy().reshape(-1), ref.data)
        assert np.array_equal(sh.scales.contiguous().view(torch.uint8).numpy().reshape(-1), ref.scales)
        assert sh.shape == (b - a, cols) and sh.swizzled == swizzled


def _rank_main(rank, world, port, T, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rows, cols = 256 * world, 128
        w, full, t = quantized(rows, cols, True, 9)
        rng = np.random.default_rng(10)
        x32 = rng.standard_normal((T, cols)).astype(np.float32)
        xb = (x32.view(np.uint32) >> 16).astype(np.uint16)  # truncated to BF16 bit patterns
        X = oracle.Dense(oracle.BF16, xb, cols)
        want = oracle.gemm(rows, T, cols, full, X, D_dtype=oracle.FP32)["D"].reshape(T, rows)
        sh = shard_rows(t, world, rank)
        mine = oracle.gemm(sh.shape[0], T, cols, to_oracle(sh), X, D_dtype=oracle.FP32)["D"].reshape(T, sh.shape[0])
        a, b = shard_bounds(rows, world, rank)
        ok_local = np.array_equal(mine, want[:, a:b])
        y = gather_features(torch.from_numpy(mine.copy()))
        ok_full = tuple(y.shape) == (T, rows) and np.array_equal(y.numpy(), want)
        q.put((rank, ok_local, ok_full))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("T", [1, 5])
def test_two_ranks_reassemble_the_one_rank_result(T):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, T, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res == [(0, True, True), (1, True, True)]
