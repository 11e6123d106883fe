"""Tensor-parallel NVFP4 linear layers: a weight's output rows are split over the GPUs of one node, every rank computes
its rows of ``y = x @ W.T`` from the full (replicated) ``x``, and an NCCL all-gather over NVLink reassembles ``y``.

The reference has no multi-GPU code; this module shards the units its API already treats as independent -- output rows
(include/nvfp4effma.h:78-92 there: every D[i, j] depends on row i of A only).  Rows are cut on multiples of 128, so that a
shard's swizzled block scales are a contiguous range of the tensor's (128-row tiles) and the 16-row gate / up slices of a
SwiGLU weight stay whole.  A tensor is quantized BEFORE it is sharded: the per-tensor global is shared by all shards and a
rank's outputs equal the corresponding outputs of the one-GPU call bit for bit.

One process per GPU (``torch.distributed``).  The layout functions (``shard_bounds``, ``shard_rows``, ``gather_features``)
work on tensors of any device and with any backend, which is how the host logic is tested on CPU ranks over gloo; the
layers themselves run the CUDA library only.
"""
import math
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

import ctypes

from . import _abi as A
from . import _lib as L
from ._ops import ops
from .tensor import NVFP4Tensor

ROW_ALIGN = 128


def shard_bounds(rows: int, world: int, rank: int, align: int = ROW_ALIGN) -> Tuple[int, int]:
    """Rows ``[start, stop)`` of rank ``rank``: equal shares that are multiples of ``align``."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} is outside a group of {world}")
    if rows % (world * align):
        raise ValueError(f"{rows} rows do not split into {world} equal shards of a multiple of {align} rows")
    per = rows // world
    return rank * per, (rank + 1) * per


def shard_rows(w: NVFP4Tensor, world: int, rank: int) -> NVFP4Tensor:
    """The rows of rank ``rank`` of a 2-D ``NVFP4Tensor`` as views of its buffers (no copy): nibbles, block scales (linear or
    swizzled), per-row globals.  The per-tensor global is shared."""
    if w.dim() != 2:
        raise ValueError("only 2-D weights are sharded")
    a, b = shard_bounds(w.shape[0], world, rank)
    g = w.global_scale
    if g is not None and g.numel() > 1:
        g = g[a:b]
    kw = dict(scale_max=w.scale_max, swizzled=w.swizzled, ue5m3=w.ue5m3, cols=w.cols, block=w.block)
    scales = w.scales[a:b]  # swizzled: 128-row tiles are contiguous row ranges of the [rows, cols / 16] buffer
    return NVFP4Tensor(w.data[a:b], scales, amax=g, **kw) if w.global_is_amax else NVFP4Tensor(w.data[a:b], scales, g, **kw)


def gather_features(y_shard: torch.Tensor, group=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-gather of ``y_shard`` [T, n_local] along the feature dimension -> [T, world * n_local].

    One ``all_gather_into_tensor`` yields the rank-major [world, T, n_local]; for T == 1 that already is the result, for
    T > 1 one strided copy turns it into the token-major layout the next layer reads."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return y_shard
    T, nl = y_shard.shape
    y_shard = y_shard.contiguous()
    stage = torch.empty((world * T, nl), dtype=y_shard.dtype, device=y_shard.device)  # rank-major: rank r holds rows [r * T, (r + 1) * T)
    dist.all_gather_into_tensor(stage, y_shard, group=group)
    if T == 1:
        return stage.view(1, world * nl)
    stage = stage.view(world, T, nl)
    if out is None:
        out = torch.empty((T, world * nl), dtype=y_shard.dtype, device=y_shard.device)
    out.view(T, world, nl).copy_(stage.permute(1, 0, 2))
    return out


# ---- calls into the C ABI that the operator layer does not cover (SwiGLU on images, the fused all-gather entries) -------------
def _ptr_array(ptrs):
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


def _image_tensor(image, glob, flags, scale_max):
    return L.Tensor(A.addr(image), L.NVFP4, None, 0, A.addr(glob), None, flags, scale_max)


def _swiglu_descriptor(on):
    ex = L.Epilogue()
    ex.swiglu = int(bool(on))
    return ex


def _tp_gather(buffer_ptrs, flag_ptrs, rank, rows, row_pitch_bytes, col_offset_bytes, shard_bytes):
    """``nvfp4a_b200_tp_gather``: push this rank's columns of a peer-mapped activation buffer to every peer, then barrier."""
    L.check(L.lib.nvfp4a_b200_tp_gather(_ptr_array(buffer_ptrs), _ptr_array(flag_ptrs), len(buffer_ptrs), rank, rows, row_pitch_bytes,
                                        col_offset_bytes, shard_bytes, A.stream()))


def _local_gemv(x, layer, out):
    """Up to 8 tokens against this rank's image: ``nvfp4a_gemv_tc(_ex)`` writing ``out`` [T, rows (/ 2 with SwiGLU)]."""
    x = A.matrix(x, 64, "x")
    a, b, d = _image_tensor(layer.image, layer.global_scale, layer.flags, layer.scale_max), A.dense_tensor(x), A.dense_tensor(out)
    bias = A.dense_tensor(layer.bias) if layer.bias is not None else None
    ex = _swiglu_descriptor(layer.swiglu)
    L.check(L.lib.nvfp4a_gemv_tc_ex(layer.rows, x.shape[0], layer.in_features, 1.0, ctypes.byref(a), ctypes.byref(b), x.stride(0), 0.0, None, 0,
                                    ctypes.byref(d), out.stride(0), A.ref(bias), ctypes.byref(ex), A.stream()))
    return out


def _local_gemm(x, layer, out):
    """More than 8 tokens: ``nvfp4a_gemm_tc(_ex)`` with contiguous bfloat16 ``x`` serving as its own activation image."""
    if not (x.is_contiguous() and x.data_ptr() % 16 == 0):
        x = x.contiguous()
    a, b, d = _image_tensor(layer.image, layer.global_scale, layer.flags, layer.scale_max), A.dense_tensor(x), A.dense_tensor(out)
    bias = A.dense_tensor(layer.bias) if layer.bias is not None else None
    ex = _swiglu_descriptor(layer.swiglu)
    L.check(L.lib.nvfp4a_gemm_tc_ex(layer.rows, x.shape[0], layer.in_features, 1.0, ctypes.byref(a), ctypes.byref(b), 0.0, None, 0, ctypes.byref(d),
                                    out.stride(0), A.ref(bias), ctypes.byref(ex), A.addr(A.workspace(x.device)), A.stream()))
    return out


def _fused_call(entry, x, layer, out, buffer_ptrs, flag_ptrs, rank, push=1):
    """``nvfp4a_b200_gemv_tc_tp`` / ``nvfp4a_b200_gemm_tc_tp``: ``out`` (a view into this rank's peer-mapped buffer) is also
    written into every peer's buffer and the ranks meet in a barrier."""
    gemv = entry in ("gemv", "gemv_deferred")
    deferred = entry == "gemv_deferred"
    x = A.matrix(x, 64, "x") if gemv else (x if x.is_contiguous() and x.data_ptr() % 16 == 0 else x.contiguous())
    a, b, d = _image_tensor(layer.image, layer.global_scale, layer.flags, layer.scale_max), A.dense_tensor(x), A.dense_tensor(out)
    bias = A.dense_tensor(layer.bias) if layer.bias is not None else None
    ex = _swiglu_descriptor(layer.swiglu)
    tail = (_ptr_array(buffer_ptrs), _ptr_array(flag_ptrs), len(buffer_ptrs), rank) + ((int(push),) if deferred else ()) + (A.stream(),)
    if gemv:
        fn = L.lib.nvfp4a_b200_gemv_tc_tp_deferred if deferred else L.lib.nvfp4a_b200_gemv_tc_tp
        st = fn(layer.rows, x.shape[0], layer.in_features, 1.0, ctypes.byref(a), ctypes.byref(b), x.stride(0), ctypes.byref(d),
                                          out.stride(0), A.ref(bias), ctypes.byref(ex), *tail)
    else:
        st = L.lib.nvfp4a_b200_gemm_tc_tp(layer.rows, x.shape[0], layer.in_features, 1.0, ctypes.byref(a), ctypes.byref(b), ctypes.byref(d), out.stride(0),
                                          A.ref(bias), ctypes.byref(ex), A.addr(A.workspace(x.device)), *tail)
    L.check(st)
    return out


class PeerGather:
    """Activation buffers that exist at the same place on every GPU of the node (torch symmetric memory: peer-mapped device
    memory) and the library's own all-gather over them: a rank writes its columns of ``y`` into its local buffer, one launch
    stores them into every peer's buffer over NVLink and joins a barrier (``nvfp4a_b200_tp_gather``).  Two buffers alternate
    between consecutive layers: a rank that runs ahead writes the buffer its peers have finished reading (they passed the
    previous barrier)."""

    def __init__(self, group, max_elems: int, device):
        import torch.distributed._symmetric_memory as symm
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.bufs = [symm.empty(max_elems, dtype=torch.bfloat16, device=device) for _ in range(2)]
        self.flags = symm.empty(16, dtype=torch.int64, device=device)
        self.flags.zero_()
        torch.cuda.synchronize()
        self.buf_ptrs = [list(symm.rendezvous(b, group).buffer_ptrs) for b in self.bufs]
        self.flag_ptrs = list(symm.rendezvous(self.flags, group).buffer_ptrs)
        dist.barrier(group)   # every rank's flags are zero before anyone signals

    def view(self, slot: int, T: int, M: int) -> torch.Tensor:
        return self.bufs[slot][:T * M].view(T, M)

    def push(self, slot: int, T: int, M: int, col0: int, cols: int):
        _tp_gather(self.buf_ptrs[slot], self.flag_ptrs, self.rank, T, M * 2, col0 * 2, cols * 2)

    def post(self, slot: int, T: int, M: int, col0: int, cols: int):
        """The deferred form of ``push``: copy and post, no wait."""
        L.check(L.lib.nvfp4a_b200_tp_gather_post(_ptr_array(self.buf_ptrs[slot]), _ptr_array(self.flag_ptrs), self.world, self.rank, T, M * 2, col0 * 2,
                                                 cols * 2, A.stream()))

    def wait(self):
        """Closes a sequence of deferred calls (``nvfp4a_b200_gemv_tc_tp_deferred``): after it the last gathered buffer is complete."""
        L.check(L.lib.nvfp4a_b200_tp_wait(_ptr_array(self.flag_ptrs), self.world, self.rank, A.stream()))


class TPLinear:
    """One rank's part of ``y = x @ W.T + bias`` (optionally ``silu(gate) * up`` of interleaved gate / up rows).

    Holds the image of its rows of ``W`` (built once), the shared global and its part of the bias.  ``forward`` takes the
    replicated ``x`` [T, K] (bfloat16) and returns the full ``y``; ``forward_local`` returns this rank's columns only."""

    def __init__(self, weight: NVFP4Tensor, bias: Optional[torch.Tensor] = None, *, group=None, swiglu: bool = False, replicate: bool = False,
                 gather: Optional["PeerGather"] = None, fused_decode=False, fused_prefill: bool = True):
        """``fused_decode`` (up to 8 tokens): ``"deferred"`` -- GEMV, then a launch that copies the rank's outputs to the peers and
        posts the rank's epoch without waiting; the wait for the peers moves to the start of the NEXT GEMV
        (``nvfp4a_b200_gemv_tc_tp_deferred`` + ``nvfp4a_b200_tp_gather_post``; a sequence is closed by ``PeerGather.wait``);
        ``"deferred_push"`` -- the same with the copy and the post done by the GEMV's last CTA; ``True`` -- the GEMV's last CTA
        copies the rank's outputs and joins the barrier itself (``nvfp4a_b200_gemv_tc_tp``); ``False`` -- GEMV, then the gather
        launch with its barrier.  The two forms with a fused copy measured slower than their two-launch counterparts."""
        self.group = group
        self.gather = gather
        self.fused_decode = fused_decode
        self.fused_prefill = fused_prefill   # more than 8 tokens: the GEMM stores its tiles to the peers itself
        solo = replicate or not dist.is_initialized()  # replicate: the whole weight on this rank, no collective
        self.world = 1 if solo else dist.get_world_size(group)
        self.rank = 0 if solo else dist.get_rank(group)
        if swiglu and weight.shape[0] % 16:
            raise ValueError("a SwiGLU weight has a multiple of 16 rows")
        self.out_features, self.in_features = weight.shape[0] // (2 if swiglu else 1), weight.shape[1]
        self.swiglu = swiglu
        shard = shard_rows(weight, self.world, self.rank)
        op = shard._operand()
        self.rows = op.rows
        self.global_scale, self.flags, self.scale_max = op.glob, op.flags, op.scale_max
        self.image = ops.tc_image(L.TC_A16, op.data, op.scales, op.flags, op.cols)
        a, b = shard_bounds(weight.shape[0], self.world, self.rank)
        self.bias = bias[a:b].contiguous() if bias is not None else None

    def forward_local(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if x.dtype != torch.bfloat16 or x.dim() != 2 or x.shape[1] != self.in_features:
            raise ValueError(f"x must be bfloat16 [T, {self.in_features}]")
        T = x.shape[0]
        if out is None:
            out = torch.empty((T, self.rows // (2 if self.swiglu else 1)), dtype=torch.bfloat16, device=x.device)
        return _local_gemv(x, self, out) if T <= 8 else _local_gemm(x, self, out)

    def forward(self, x: torch.Tensor, slot: int = 0, close: bool = True) -> torch.Tensor:
        """``close = False`` (deferred form only): the caller goes on with another deferred call or ``PeerGather.wait``."""
        if self.world == 1:
            return self.forward_local(x)
        if self.gather is None:
            return gather_features(self.forward_local(x), self.group)
        T, nl, M = x.shape[0], self.rows // (2 if self.swiglu else 1), self.out_features
        y = self.gather.view(slot, T, M)
        mine = y[:, self.rank * nl:(self.rank + 1) * nl]
        if T <= 8 and self.fused_decode in ("deferred", "deferred_push"):
            if x.dtype != torch.bfloat16 or x.dim() != 2 or x.shape[1] != self.in_features:
                raise ValueError(f"x must be bfloat16 [T, {self.in_features}]")
            push = self.fused_decode == "deferred_push"
            _fused_call("gemv_deferred", x, self, mine, self.gather.buf_ptrs[slot], self.gather.flag_ptrs, self.rank, push=push)
            if not push:
                self.gather.post(slot, T, M, self.rank * nl, nl)
            if close:
                self.gather.wait()
        elif T <= 8 and self.fused_decode:   # the GEMV's last CTA stores to every rank and joins the barrier itself
            if x.dtype != torch.bfloat16 or x.dim() != 2 or x.shape[1] != self.in_features:
                raise ValueError(f"x must be bfloat16 [T, {self.in_features}]")
            _fused_call("gemv", x, self, mine, self.gather.buf_ptrs[slot], self.gather.flag_ptrs, self.rank)
        elif T > 8 and self.fused_prefill and x.dtype == torch.bfloat16:
            # the GEMM's epilogue stores every tile into all ranks' buffers (TMA stores to peer memory), then the barrier
            _fused_call("gemm", x, self, mine, self.gather.buf_ptrs[slot], self.gather.flag_ptrs, self.rank)
        else:
            self.forward_local(x, out=mine)
            self.gather.push(slot, T, M, self.rank * nl, nl)
        return y

    __call__ = forward


class TPDecoderLinears:
    """The linear layers of a Llama-style decoder stack under tensor parallelism: per layer QKV (hidden -> qkv), O (hidden ->
    hidden), gate / up with SwiGLU (hidden -> 2 x intermediate, interleaved per 16 rows) and down (intermediate -> hidden).
    Attention, norms and residuals are not part of this path: O reads the first ``hidden`` features of the QKV output, and every
    layer starts from the stack's input (see ``forward``)."""

    def __init__(self, layers: int = 32, hidden: int = 4096, intermediate: int = 14336, qkv: int = 6144, *, group=None, seed: int = 4,
                 device="cuda", std: float = 0.02, replicate: bool = False, collective: str = "peer", max_tokens: int = 4096,
                 fused_decode="auto", fused_prefill: bool = True):
        """``collective``: "peer" = the library's all-gather over peer-mapped buffers, "nccl" = ``all_gather_into_tensor``.
        ``fused_decode``: as in ``TPLinear``; "auto" = "deferred_push" from 4 ranks up (shards of a few hundred rows: the fused copy
        costs a handful of CTAs a ticket and saves a launch per linear; measured 1.32 against 1.37 ms per 32-layer step at 8 GPUs)
        and the two-launch form below that (at 2 GPUs the shards' hundreds of CTAs make the tickets dearer than the launch)."""
        self.hidden, self.layers = hidden, []
        multi = dist.is_initialized() and dist.get_world_size(group) > 1 and not replicate
        if fused_decode == "auto":
            fused_decode = "deferred_push" if multi and dist.get_world_size(group) >= 4 else False
        self.collective = collective if multi else "none"
        gather = PeerGather(group, max_tokens * max(hidden, intermediate, qkv), device) if multi and collective == "peer" else None
        self.max_tokens = max_tokens
        self.fused_decode = fused_decode
        self._gather = gather
        from .api import quantize
        for layer in range(layers):
            mods = []
            for j, (rows, cols, glu) in enumerate(((qkv, hidden, False), (hidden, hidden, False), (2 * intermediate, hidden, True),
                                                   (hidden, intermediate, False))):
                gen = torch.Generator(device=device).manual_seed(seed * 1000003 + layer * 4 + j)  # the same weights on every rank
                w = torch.randn((rows, cols), generator=gen, device=device, dtype=torch.float32).mul_(std).to(torch.bfloat16)
                amax = w.abs().amax().float().reshape(1)
                mods.append(TPLinear(quantize(w, amax / (6.0 * 448.0)), group=group, swiglu=glu, replicate=replicate, gather=gather, fused_decode=fused_decode, fused_prefill=fused_prefill))
                del w
            self.layers.append(mods)

    def set_collective(self, collective: str):
        """Switch between the peer-memory all-gather ("peer", if the stack was built with it) and NCCL ("nccl")."""
        if self.collective == "none":
            return
        for layer in self.layers:
            for m in layer:
                m.gather = self._gather if collective == "peer" else None
        self.collective = collective

    def check(self) -> None:
        """Reads the library's kernel status word (this SYNCHRONISES the device: call it at a coarse point such as the end of a
        forward pass, outside stream capture) and raises if a kernel gave up a bounded wait since the last check -- for this
        stack that is a rank that waited longer than the barrier's limit (about a second) for its peers in an all-gather: the
        step's activations are then incomplete on this rank and must not be used."""
        word = ctypes.c_uint(0)
        L.check(L.lib.nvfp4a_b200_kernel_status(ctypes.byref(word), 1))
        if word.value:
            code, launch = word.value & 0xFFF, word.value >> 12
            what = "a tensor-parallel barrier ran out of time waiting for a peer" if code == 0x401 else "a kernel gave up a bounded wait"
            raise RuntimeError(f"{what} (status 0x{code:03x}, launch {launch}): the outputs of that step are incomplete")

    def weight_bytes_local(self) -> int:
        return sum(m.image.numel() for layer in self.layers for m in layer)

    def forward(self, h: torch.Tensor, layers: int | None = None, collect: bool = False):
        """Every layer reads the stack's input ``h`` [T, hidden] and the last layer's output is returned.  (Norms and residuals are
        not part of this path, and without them a chain of SwiGLUs squares the activations' scale layer after layer: BF16's range
        is left within six layers.  Launches, shapes, collectives and their order are those of the chained stack.)
        ``layers``: run only the first that many layers; ``collect``: return a list with a copy of every layer's output."""
        if self.collective == "peer" and h.shape[0] > self.max_tokens:
            raise ValueError(f"{h.shape[0]} tokens exceed the peer buffers ({self.max_tokens})")
        deferred = self.collective == "peer" and h.shape[0] <= 8 and self.fused_decode in ("deferred", "deferred_push")
        outs, y = [], h
        for qkv, o, gate_up, down in self.layers[:layers]:   # the four collectives of a layer alternate between the two peer buffers
            a = qkv(h, 0, close=False)[:, :self.hidden]
            y = down(gate_up(o(a, 1, close=False), 0, close=False), 1, close=False)
            if collect:
                if deferred:
                    self._gather.wait()
                outs.append(y.clone())
        if deferred and not collect:
            self._gather.wait()   # the last gather is complete, and every peer is done with both buffers
        return outs if collect else y

    __call__ = forward
