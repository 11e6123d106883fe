"""Tensor-parallel layers on the GPU: one rank against the plain linear call, and (with two or more GPUs) two NCCL ranks
against the unsharded layers, bit for bit."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def rand(shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to("cuda").to(dtype)


@pytest.mark.parametrize("T", [1, 4, 8, 40])
def test_one_rank_layer_equals_linear(T):
    import nvfp4effma_b200 as nf
    from nvfp4effma_b200.tp import TPLinear
    w = nf.quantize(rand((256, 320), seed=1), torch.tensor([0.002], device="cuda"))
    bias = rand((256,), torch.bfloat16, seed=2)
    x = rand((T, 320), torch.bfloat16, seed=3)
    y = TPLinear(w, bias)(x)
    ref = nf.linear(x, nf.TCWeight(w, "exact"), bias)
    assert y.shape == (T, 256) and torch.equal(y, ref)


@pytest.mark.parametrize("T", [1, 8, 33])
def test_swiglu_layer(T):
    import nvfp4effma_b200 as nf
    from nvfp4effma_b200.tp import TPLinear
    w = nf.quantize(rand((512, 256), seed=4, scale=0.05), torch.tensor([0.0002], device="cuda"))
    x = rand((T, 256), torch.bfloat16, seed=5)
    y = TPLinear(w, swiglu=True)(x)
    z = nf.linear(x, w, act="exact", out_dtype=torch.float32).reshape(T, 32, 2, 8)  # slices of 8 gate rows, 8 up rows
    want = (torch.nn.functional.silu(z[:, :, 0]) * z[:, :, 1]).reshape(T, 256)
    assert y.shape == (T, 256)
    assert torch.allclose(y.float(), want, rtol=2 ** -7, atol=1e-6)


def test_decoder_stack_runs_decode_and_prefill():
    from nvfp4effma_b200.tp import TPDecoderLinears
    stack = TPDecoderLinears(layers=2, hidden=256, intermediate=512, qkv=384, std=0.06)
    for T in (1, 8, 64):
        h = stack(rand((T, 256), torch.bfloat16, seed=6))
        assert h.shape == (T, 256) and bool(torch.isfinite(h.float()).all()) and float(h.float().abs().max()) > 0


def test_a_barrier_whose_peer_never_arrives_gives_up_and_reports_it():
    """The bounded wait of the ranks' barrier, made to run out on ONE GPU without hanging anything: a group of two whose second
    rank does not exist -- both "ranks'" buffers and flag arrays are ordinary local allocations and nobody ever posts the peer's
    flag.  With the wait limit set to 2e5 cycles the kernel copies its shard, waits a tenth of a millisecond, records 0x401 with the
    launch's sequence number in the status word and returns; the word reads back, resets, and a normal call then works."""
    import ctypes
    from nvfp4effma_b200 import _lib as L
    rows, pitch, shard = 4, 512, 256
    bufs = [torch.zeros(rows * pitch, dtype=torch.uint8, device="cuda") for _ in range(2)]
    flags = [torch.zeros(16, dtype=torch.int64, device="cuda") for _ in range(2)]
    bufs[0].view(rows, pitch)[:, :shard] = 7
    st = ctypes.c_uint(0)
    L.check(L.lib.nvfp4a_b200_kernel_status(ctypes.byref(st), 1))
    assert L.lib.nvfp4a_b200_set_wait_limit(200000) == 0
    try:
        pb = (ctypes.c_void_p * 2)(*[b.data_ptr() for b in bufs])
        pf = (ctypes.c_void_p * 2)(*[f.data_ptr() for f in flags])
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        L.check(L.lib.nvfp4a_b200_tp_gather(pb, pf, 2, 0, rows, pitch, 0, shard, stream))
        seq = L.lib.nvfp4a_b200_last_launch()
        L.check(L.lib.nvfp4a_b200_kernel_status(ctypes.byref(st), 1))        # synchronises: the kernel has returned
        assert st.value & 0xFFF == 0x401 and st.value >> 12 == seq and seq > 0
        assert bool((bufs[1].view(rows, pitch)[:, :shard] == 7).all())           # the shard did reach the "peer"
        assert int(flags[1][0]) == 1 and int(flags[0][1]) == 0                   # our epoch was posted; the peer's never came
        L.check(L.lib.nvfp4a_b200_kernel_status(ctypes.byref(st), 0))
        assert st.value == 0                                                     # the read above cleared the word
        # the layer stack's own health check turns the same word into an exception (and clears it)
        from nvfp4effma_b200.tp import TPDecoderLinears
        stack = TPDecoderLinears(layers=1, hidden=256, intermediate=512, qkv=384, std=0.06)
        stack.check()
        L.check(L.lib.nvfp4a_b200_tp_gather(pb, pf, 2, 0, rows, pitch, 0, shard, stream))
        with pytest.raises(RuntimeError, match="barrier ran out of time"):
            stack.check()
        stack.check()
    finally:
        L.lib.nvfp4a_b200_set_wait_limit(2000000000)
    import nvfp4effma_b200 as nf
    w = nf.quantize(rand((128, 256), seed=7))
    y = nf.linear(rand((16, 256), torch.bfloat16, seed=8), w, act="exact")
    torch.cuda.synchronize()
    L.check(L.lib.nvfp4a_b200_kernel_status(ctypes.byref(st), 1))
    assert st.value == 0 and bool(torch.isfinite(y.float()).all())


RANK_SCRIPT = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["NVB_ROOT"])
rank = int(os.environ["RANK"]); torch.cuda.set_device(rank)
dist.init_process_group("nccl", rank=rank, world_size=int(os.environ["WORLD_SIZE"]), device_id=torch.device("cuda", rank))
from nvfp4effma_b200.tp import TPDecoderLinears
kw = dict(layers=2, hidden=256, intermediate=512, qkv=512, std=0.06)
peer, nccl, solo = TPDecoderLinears(collective="peer", max_tokens=64, **kw), TPDecoderLinears(collective="nccl", **kw), TPDecoderLinears(replicate=True, **kw)
fused = TPDecoderLinears(collective="peer", max_tokens=64, fused_decode=True, **kw)
unfused = TPDecoderLinears(collective="peer", max_tokens=64, fused_prefill=False, **kw)
deferred = TPDecoderLinears(collective="peer", max_tokens=64, fused_decode="deferred", **kw)
deferred_push = TPDecoderLinears(collective="peer", max_tokens=64, fused_decode="deferred_push", **kw)
ok = peer.collective == "peer" and nccl.collective == "nccl"
for rep in range(2):
    for T in (1, 5, 48):
        g = torch.Generator(device="cpu").manual_seed(T)
        x = torch.randn((T, 256), generator=g).cuda().bfloat16()
        want = solo(x, collect=True)
        same = lambda got: all(torch.equal(g, w) for g, w in zip(got, want))
        ok = ok and all(same(stack(x, collect=True)) for stack in (peer, nccl, fused, unfused, deferred, deferred_push))
        ok = ok and torch.equal(deferred(x).clone(), want[-1])   # the whole step with one closing wait
# the deferred decode step replayed as a CUDA graph: the epochs live on the device, so every replay synchronises anew
x = torch.randn((3, 256), generator=torch.Generator(device="cpu").manual_seed(9)).cuda().bfloat16()
want = solo(x)
out = deferred(x); torch.cuda.synchronize()
graph = torch.cuda.CUDAGraph()
with torch.cuda.graph(graph):
    out = deferred(x)
for _ in range(5):
    graph.replay()
    ok = ok and torch.equal(out.clone(), want)
from nvfp4effma_b200 import workloads
ok = ok and workloads.kernel_status() == 0
torch.cuda.synchronize(); dist.barrier(); dist.destroy_process_group()
print("RANK_OK" if ok else "RANK_MISMATCH", flush=True)
"""


@pytest.mark.skipif(torch.cuda.is_available() and torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_equal_one_rank_bit_for_bit(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = tmp_path / "rank.py"
    script.write_text(RANK_SCRIPT)
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NVB_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert all("RANK_OK" in o for o in outs), outs
