#!/usr/bin/env python
"""Benchmark of the NVFP4 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload gemm|gemv|quant]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N --steps K --warmup W

Prints ONE JSON line.  Headline metric: W4A4 GEMM M = N = K = 4096 (NVFP4 x NVFP4 -> BF16) in TFLOP/s; a "step" is one
``nvfp4a_gemm`` call on operands already resident in HBM.  Successive steps rotate over buffer sets larger than L2 in
total.  ``extra`` carries the two bandwidth-bound workloads of the same metric (GEMV 8192^2 batch 1, quantization 8192^2)
with their own roofline objects.  ``e2e`` is the same GEMM through the C ABI with HOST operands: pinned host -> device
copies of the quantized operands and the device -> host read of D are inside the timed region, consecutive steps pipelined
over three streams and three device buffer sets (the one-step-at-a-time time is reported beside it).  At N > 1 every rank runs
the same workload on its own GPU (independent GEMMs, no collective on the data path: weak scaling); the time is the
maximum over ranks and ``value`` the sum of all ranks' work divided by it.

``--impl reference`` times the reference's CPU implementation of the path: its host block-sum emulation, restated in
``oracle/`` (the reference ships no CPU library), on all host cores, on a bounded sample of the same workload.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M = N = K = 4096
GEMV_M = GEMV_K = 8192
QUANT_R = QUANT_C = 8192
NOMINAL_FP4_TFLOPS = 9000.0
# the workload of the headline, printed by both arms (the reference arm runs a bounded slab of it on the host and says so in `sample`)
HEADLINE_CONFIG = {"workload": "w4a4_gemm_m4096_n4096_k4096", "entry": "nvfp4a_gemm",
                   "scales": "E4M3 1x16 in the cuBLASLt GEMM-swizzled layout, FP32 decode-factor globals",
                   "l2": "3 rotating operand/output sets (157 MB) > L2", "per_rank": "independent GEMMs, no collective"}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def source_hash(files):
    """SHA-256 (first 16 hex digits) over the named kernel sources: what a DRAM-traffic figure captured under ncu belongs to."""
    import hashlib
    h = hashlib.sha256()
    for f in sorted(files):
        with open(os.path.join(ROOT, "nvfp4effma_b200", "csrc", f), "rb") as fh:
            h.update(f.encode() + b"\0" + fh.read())
    return h.hexdigest()[:16]


def load_traffic():
    """profiles/traffic.json: per kernel {"bytes": DRAM read + write bytes per launch (one ncu capture), "sources": the kernel's
    source files, "hash": source_hash(sources) at the capture}.  A figure whose sources have changed since is stale: the
    roofline then carries null, and `traffic_stamp` in the JSON line says which entries were current."""
    p = os.path.join(ROOT, "profiles", "traffic.json")
    if not os.path.exists(p):
        return {}, {}
    out, stamp = {}, {}
    for key, e in json.load(open(p)).items():
        if not isinstance(e, dict):
            e = {"bytes": e}
        try:
            current = source_hash(e["sources"]) == e["hash"]
        except (OSError, KeyError, TypeError):
            current = False
        out[key] = e.get("bytes") if current else None
        stamp[key] = {"hash": e.get("hash"), "current": current}
    return out, stamp


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            f = [x.strip() for x in line.split(",")]
            if len(f) >= 6:
                self.rows.append(f)

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz = sorted(int(r[0]) for r in self.rows if r[0].isdigit())
        mx = max([int(r[1]) for r in self.rows if r[1].isdigit()] or [0])
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx or None, "reasons": reasons, "samples": len(mhz)}


# ---- the reference arm: CPU block-sum emulation -----------------------------------------------------------------------------
CPU_COLS = 256   # output columns of one host sample of the 4096^3 GEMM (1/16 of the workload)
_cpu_operands = {}


def cpu_gemm_sample(cols, threads):
    """One bounded sample of the W4A4 4096^3 GEMM on the host: `cols` output columns x all 4096 rows, k = 4096, through the
    oracle (the reference's host emulation restated).  The operands are built once, outside the timed call.  Returns seconds."""
    import numpy as np
    import oracle as O
    if cols not in _cpu_operands:
        rng = np.random.default_rng(2)
        A = O.Fp4(M, K, glob=np.array([0.01], np.float32))
        B = O.Fp4(cols, K, glob=np.array([0.01], np.float32))
        for t in (A, B):
            t.data[:] = rng.integers(0, 256, t.data.size, dtype=np.uint8)
            t.scales[:] = rng.integers(0x20, 0x50, t.scales.size).astype(np.uint8)
        _cpu_operands[cols] = (A, B)
    A, B = _cpu_operands[cols]
    t0 = time.perf_counter()
    O.gemm(M, cols, K, A, B, D_dtype=O.BF16, nthreads=threads)
    return time.perf_counter() - t0


def cpu_gemv_baseline(threads):
    """The GEMV workload (8192 x 8192 NVFP4 weights, one BF16 activation vector) in full through the oracle, in the order of
    the reference's GEMV kernel.  Returns (GB/s of weight bytes, seconds)."""
    import numpy as np
    import oracle as O
    rng = np.random.default_rng(3)
    A = O.Fp4(GEMV_M, GEMV_K, glob=np.array([0.01], np.float32))
    A.data[:] = rng.integers(0, 256, A.data.size, dtype=np.uint8)
    A.scales[:] = rng.integers(0x20, 0x50, A.scales.size).astype(np.uint8)
    x = O.Dense(O.BF16, O.from_f32(rng.standard_normal(GEMV_K).astype(np.float32), O.BF16), GEMV_K)
    t0 = time.perf_counter()
    O.gemm(GEMV_M, 1, GEMV_K, A, x, D_dtype=O.BF16, order=1, nthreads=threads)
    t = time.perf_counter() - t0
    return (GEMV_M * GEMV_K // 2 + GEMV_M * GEMV_K // 16) / t / 1e9, t


def cpu_quant_baseline(threads):
    """The quantization workload (8192 x 8192, swizzled scales, amax computed) in full through the oracle.  Returns (GB/s of
    the algorithmic bytes, seconds)."""
    import numpy as np
    import oracle as O
    rng = np.random.default_rng(4)
    x = rng.standard_normal((QUANT_R, QUANT_C)).astype(np.float32)
    dst = O.Fp4(QUANT_R, QUANT_C, flags=O.SWIZZLED | O.GLOBAL_AMAX, glob=0.0)
    t0 = time.perf_counter()
    O.quantize(x, dst, compute_amax=True, nthreads=threads)
    t = time.perf_counter() - t0
    return (QUANT_R * QUANT_C * 2 + QUANT_R * QUANT_C // 2 + QUANT_R * QUANT_C // 16) / t / 1e9, t


def run_reference(args, rank, world):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    cols = CPU_COLS
    cpu_gemm_sample(cols, threads)   # builds the operands, warms the pages
    t_one = cpu_gemm_sample(cols, threads)
    while cols > 32 and t_one * args.steps > 150.0:   # keep the whole run within a few minutes whatever --steps asks
        cols //= 2
        cpu_gemm_sample(cols, threads)
        t_one = cpu_gemm_sample(cols, threads)
    ts = [cpu_gemm_sample(cols, threads) for _ in range(args.steps)]
    ts.sort()
    t = ts[len(ts) // 2]
    tflops = 2.0 * M * cols * K / t / 1e12
    sample = f"{cols} of {N} output columns x {M} rows x k {K} per step (exact block sums), scaled linearly"
    line = {"impl": "reference", "metric": "w4a4_gemm_4096_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": t * 1e3 * (N / cols), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp4 x fp4 -> int32 block sums, fp32 accumulate", "data": "synthetic",
            "config": HEADLINE_CONFIG,
            "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---- our arm ------------------------------------------------------------------------------------------------------------------
def time_steps(fn, steps, warmup, stream, dist, world):
    """W untimed + K timed calls of fn(i); device time by CUDA events on `stream`; returns the max over ranks in ms."""
    import torch
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(steps):
        fn(warmup + i)
    e1.record(stream)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    return ms


def time_groups(fn, steps, warmup, groups, dist, world):
    """The headline timing: `warmup` direct calls, then fn(0..steps-1) captured into one CUDA graph (no host time between the
    kernels), one untimed replay, then `groups` replays, each a group of exactly `steps` steps timed by its own pair of CUDA
    events.  Returns the groups' times in ms (max over ranks per group) and the launches issued on this rank."""
    import torch
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(steps):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(groups):
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    if world > 1:
        t = torch.tensor(ts, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ts = [float(v) for v in t]
    return ts, warmup + steps * (groups + 1)


def time_graph(fn, calls, replays, warmup, dist, world):
    """Kernels of a few microseconds: `calls` launches of fn(i) captured into one CUDA graph (the host's ctypes overhead per
    call would otherwise exceed the kernel), replayed `replays` times after `warmup` direct calls; CUDA events around each
    replay; returns (median ms per call, max over ranks; launches issued on this rank)."""
    import torch
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(calls):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ts = []
    for _ in range(replays):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) / calls)
    ts.sort()
    ms = ts[len(ts) // 2]
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    return ms, warmup + calls * (replays + 2)


def fp4_mma_ceiling(L, dev):
    """TFLOP/s of the bare FP4 MMA stream (CTA pairs, N = 256): one launch of 4 x 4096 MMAs per SM, timed by events."""
    import torch
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    cyc = torch.zeros(2 * sms, dtype=torch.int64, device=dev)
    iters, flags = 4096, 16 | 1   # issued by an elected lane of a converged warp, one commit per four MMAs as a GEMM's main loop
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    best = None
    for i in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        L.check(L.lib.nvfp4a_b200_mma_ceiling(256, 1, iters, flags, ctypes.c_void_p(cyc.data_ptr()), stream))
        e1.record()
        torch.cuda.synchronize()
        if i:
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
    flops = (sms // 2 * 2) * 4 * iters * 2.0 * 128 * 256 * 64
    return flops / (best * 1e-3) / 1e12


def reference_cuda_core(L, W, A, B, D, dev):
    """Context only: the reference library's own nvfp4a_gemm (its CUDA-core DP4A kernel, NVFP4A_DP4A=1) on the same 4096^3
    operands, when the library built from the reference's sources travelled with the repository."""
    import torch
    so = os.path.join(ROOT, "oracle", "_ref", "libnvfp4effma_ref.so")
    if not os.path.exists(so):
        return {"unavailable": "oracle/_ref/libnvfp4effma_ref.so was not built"}
    os.environ["NVFP4A_DP4A"] = "1"
    ref = ctypes.CDLL(so)
    ref.nvfp4a_gemm.restype, ref.nvfp4a_gemm.argtypes = L.lib.nvfp4a_gemm.restype, L.lib.nvfp4a_gemm.argtypes
    tD = W.tensor(D, L.BF16)

    def call():
        st = ref.nvfp4a_gemm(M, N, K, 1.0, ctypes.byref(A), K, ctypes.byref(B), K, 0.0, None, 0, ctypes.byref(tD), M, None, W.stream_ptr())
        if st != 0:
            raise RuntimeError(f"reference nvfp4a_gemm returned {st}")

    try:
        call()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            call()
        e1.record()
        torch.cuda.synchronize()
    except (RuntimeError, OSError) as exc:
        return {"unavailable": str(exc)}
    ms = e0.elapsed_time(e1) / 3
    return {"entry": "the reference library's nvfp4a_gemm, NVFP4A_DP4A=1 (its exact DP4A CUDA-core kernel), built for sm_100 from its own sources",
            "ms_per_call": ms, "tflops": 2.0 * M * N * K / (ms * 1e-3) / 1e12, "calls": 3}


def hbm_entry(name, bytes_per_call, ms, world, peaks, traffic, key, workload, l2, **more):
    gbs = bytes_per_call / (ms * 1e-3) / 1e9
    d = {"metric": name, "value": gbs * world, "unit": "GB/s", "us_per_call": ms * 1e3,
         "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                      "traffic": traffic.get(key)},
         "config": {"workload": workload, "l2": l2}}
    d.update(more)
    return d


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from nvfp4effma_b200 import _lib as L
    from nvfp4effma_b200 import workloads as W

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    stream = torch.cuda.current_stream()
    peaks = load_peaks()
    traffic, traffic_stamp = load_traffic()
    launches = 0
    only = args.only
    if args.pair != -1:
        assert L.lib.nvfp4a_b200_set_pair(args.pair) == 0
    if args.no_pdl:
        L.lib.nvfp4a_b200_set_pdl(0)

    # ---- GEMM W4A4 4096^3: rotating sets (inputs 18.9 MB + D 33.6 MB each; 3 sets > 126 MB of L2) ----
    nsets = 3
    sets = []
    for s in range(nsets):
        A = W.quantize_decode_factor(W.randn_bf16(M, K, 1.0, 200 + 2 * s + 1000 * rank, dev), swizzled=True)
        B = W.quantize_decode_factor(W.randn_bf16(N, K, 1.0, 201 + 2 * s + 1000 * rank, dev), swizzled=True)
        D = torch.empty(N * M, dtype=torch.bfloat16, device=dev)
        sets.append((A, B, D, A.tensor(), B.tensor()))
    torch.cuda.synchronize()

    def gemm_step(i):
        A, B, D, tA, tB = sets[i % nsets]
        W.gemm(M, N, K, tA, tB, D)

    sampler = ClockSampler(local_rank)   # runs until every timed region of this process is over
    if rank == 0:
        sampler.start()
        t_wait = time.perf_counter()
        while not sampler.rows and time.perf_counter() - t_wait < 3.0:   # nvidia-smi needs a moment before its first sample
            time.sleep(0.05)
    groups = 5
    group_ms, n = time_groups(gemm_step, args.steps, args.warmup, groups, dist, world)
    launches += n
    ms = sorted(group_ms)[groups // 2]   # the median group of exactly --steps steps
    ms_step = ms / args.steps
    tflops = 2.0 * M * N * K * world / (ms_step * 1e-3) / 1e12
    peak_fp4 = 4.0 * peaks["bf16_tflops"]
    per_gpu = tflops / world
    ceiling = fp4_mma_ceiling(L, dev)   # what the FP4 MMA instruction itself sustains on this GPU, measured now
    launches += 3
    roofline = {"bound": "tensor", "achieved": per_gpu, "peak": peak_fp4, "unit": "TFLOP/s", "frac": per_gpu / peak_fp4,
                "traffic": traffic.get("w4a4_gemm_4096_dram_bytes"),
                "peak_note": f"4 x {peaks['source']} dense bf16 burst ({peaks['bf16_tflops']:.0f} TF/s): no fp4 figure is in the measured peaks",
                "fp4_mma_ceiling_tflops": ceiling, "frac_of_fp4_mma_ceiling": per_gpu / ceiling if ceiling else None,
                "frac_of_nominal_9000": per_gpu / NOMINAL_FP4_TFLOPS,
                "ceiling_note": "tcgen05.mma kind::mxf4nvf4 cta_group::2 256 x 256 x 64 issued back to back on every SM, no loads, "
                                "no epilogue (nvfp4a_b200_mma_ceiling), timed by CUDA events in this run"}
    timing = {"method": f"CUDA graph of --steps GEMMs; {groups} replays, each timed by its own events; headline = median group",
              "group_ms": group_ms, "min_ms_per_step": min(group_ms) / args.steps, "max_ms_per_step": max(group_ms) / args.steps}

    # ---- e2e: host operands, copies inside the timed region ----
    A, B, D, tA, tB = sets[0]
    hA = [t.cpu().pin_memory() for t in (A.data, A.scales, A.glob)]
    hB = [t.cpu().pin_memory() for t in (B.data, B.scales, B.glob)]
    hD = torch.empty(N * M, dtype=torch.bfloat16).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in hA + hB)
    d2h = hD.numel() * 2

    def e2e_step(i):
        for h, d in zip(hA, (A.data, A.scales, A.glob)):
            d.copy_(h, non_blocking=True)
        for h, d in zip(hB, (B.data, B.scales, B.glob)):
            d.copy_(h, non_blocking=True)
        W.gemm(M, N, K, tA, tB, D)
        hD.copy_(D, non_blocking=True)

    e2e_steps = max(3, min(args.steps, 10)) if only in ("all", "gemm") else 1
    ms_serial = time_steps(e2e_step, e2e_steps, 3 if only in ("all", "gemm") else 0, stream, dist, world) / e2e_steps
    launches += e2e_steps + 3

    # The same steps as a pipeline, the way a caller with a queue of independent GEMMs runs them: three device operand / output
    # sets, host -> device copies, the GEMM and the device -> host read of consecutive steps on three streams.  Every step still
    # copies its operands in from pinned host memory and its whole D out inside the timed region.
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(nsets)]
    ev_gemm = [torch.cuda.Event() for _ in range(nsets)]
    ev_out = [torch.cuda.Event() for _ in range(nsets)]

    def piped_step(i):
        b = i % nsets
        Ab, Bb, Db, tAb, tBb = sets[b]
        with torch.cuda.stream(s_in):
            if i >= nsets:
                s_in.wait_event(ev_out[b])    # the set's previous D has been read out (so its GEMM is done too)
            for h, d in zip(hA, (Ab.data, Ab.scales, Ab.glob)):
                d.copy_(h, non_blocking=True)
            for h, d in zip(hB, (Bb.data, Bb.scales, Bb.glob)):
                d.copy_(h, non_blocking=True)
            ev_in[b].record(s_in)
        stream.wait_event(ev_in[b])
        W.gemm(M, N, K, tAb, tBb, Db)
        ev_gemm[b].record(stream)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_gemm[b])
            hD.copy_(Db, non_blocking=True)
            ev_out[b].record(s_out)

    def time_piped(steps, warmup):
        for i in range(warmup):
            piped_step(i)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        s_in.wait_event(e0)                   # no copy of the timed steps starts before the clock
        for i in range(steps):
            piped_step(i)
        stream.wait_stream(s_out)             # the last D is on the host when the clock stops
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t[0])
        return ms

    piped_steps = 4 * e2e_steps
    ms_e2e = time_piped(piped_steps, 3 if only in ("all", "gemm") else 0) / piped_steps
    launches += piped_steps + 3
    e2e = {"value": 2.0 * M * N * K * world / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "ms_per_step": ms_e2e, "steps": piped_steps,
           "how": f"{nsets} device operand / output sets; the copies in, the GEMM and the read of D of consecutive steps overlap on three streams",
           "one_step_at_a_time": {"ms_per_step": ms_serial, "value": 2.0 * M * N * K * world / (ms_serial * 1e-3) / 1e12}}
    extra = {}
    if rank == 0 and world == 1 and only == "all" and not args.no_cpu:
        extra["reference_cuda_core_b200"] = reference_cuda_core(L, W, tA, tB, D, dev)
        launches += 4 if "ms_per_call" in extra["reference_cuda_core_b200"] else 0
    del sets, hA, hB, hD

    # ---- GEMV 8192^2 batch 1 (W4A16): 8 distinct weights = 302 MB > L2; the image entry is what TCWeight decodes through ----
    if only in ("all", "gemv"):
        nw = 8
        ws = [W.quantize_decode_factor(W.randn_bf16(GEMV_M, GEMV_K, 0.02, 300 + s + 1000 * rank, dev)) for s in range(nw)]
        imgs = [W.weight_image(w) for w in ws]
        x = W.randn_bf16(1, GEMV_K, 1.0, 400 + rank, dev)
        y = torch.empty(GEMV_M, dtype=torch.bfloat16, device=dev)
        tws, tx, ty = [w.tensor() for w in ws], W.tensor(x, L.BF16), W.tensor(y, L.BF16)

        def gemv_image(i):
            L.check(L.lib.nvfp4a_gemv_tc(GEMV_M, 1, GEMV_K, 1.0, ctypes.byref(imgs[i % nw][1]), ctypes.byref(tx), GEMV_K, 0.0, None, 0,
                                         ctypes.byref(ty), GEMV_M, None, W.stream_ptr()))

        def gemv_plain(i):
            L.check(L.lib.nvfp4a_gemm(GEMV_M, 1, GEMV_K, 1.0, ctypes.byref(tws[i % nw]), GEMV_K, ctypes.byref(tx), GEMV_K, 0.0, None, 0,
                                      ctypes.byref(ty), GEMV_M, None, W.stream_ptr()))

        gbytes = GEMV_M * GEMV_K // 2 + GEMV_M * GEMV_K // 16
        ms_gi, n1 = time_graph(gemv_image, 48, 7, 8, dist, world)
        route_image = L.lib.nvfp4a_b200_last_route()
        ms_gp, n2 = time_graph(gemv_plain, 48, 7, 8, dist, world)
        route_plain = L.lib.nvfp4a_b200_last_route()
        launches += n1 + n2
        routes = {2: "mma.sync GEMV", 3: "FP4 tensor-core GEMV (tcgen05)"}
        extra["gemv_8192_b1"] = hbm_entry("gemv_w4a16_8192x8192_b1_gbs", gbytes, ms_gi, world, peaks, traffic, "gemv_8192_dram_bytes",
                                          "gemv_w4a16_m8192_k8192_n1", "8 rotating weights (302 MB) > L2", entry="nvfp4a_gemv_tc (weight image)",
                                          kernel=routes.get(route_image), timing="CUDA graph of 48 calls, median of 7 replays",
                                          plain_operand={"entry": "nvfp4a_gemm (linear scales)", "us_per_call": ms_gp * 1e3,
                                                         "gbs": gbytes / (ms_gp * 1e-3) / 1e9, "kernel": routes.get(route_plain)})
        # W4A8 decode beside it: 4096 x 4096 weights, 8 INT8 activation vectors (gemv_blocked_kernel: exact DP4A block sums)
        m8 = k8 = 4096
        w8 = [W.quantize_decode_factor(W.randn_bf16(m8, k8, 0.02, 330 + s + 1000 * rank, dev)) for s in range(16)]   # 151 MB > L2
        x8 = W.randn_bf16(8, k8, 1.0, 401 + rank, dev)
        xq = torch.empty(8, k8, dtype=torch.int8, device=dev)
        xsc = torch.empty(8, k8 // 16, dtype=torch.float32, device=dev)
        src8, dst8 = W.tensor(x8, L.BF16), W.tensor(xq, L.INT8, xsc, 0)
        L.check(L.lib.nvfp4a_quantize(ctypes.byref(src8), k8, ctypes.byref(dst8), k8, 8, k8, W.stream_ptr()))
        t_xq, t_w8 = W.tensor(xq, L.INT8, xsc, k8 // 16), [w.tensor() for w in w8]
        y8 = torch.empty(8 * m8, dtype=torch.bfloat16, device=dev)
        t_y8 = W.tensor(y8, L.BF16)

        def gemv_int8(i):
            L.check(L.lib.nvfp4a_gemm(m8, 8, k8, 1.0, ctypes.byref(t_w8[i % 16]), k8, ctypes.byref(t_xq), k8, 0.0, None, 0, ctypes.byref(t_y8), m8, None,
                                      W.stream_ptr()))

        ms_g8, n3 = time_graph(gemv_int8, 48, 7, 8, dist, world)
        launches += n3
        b8 = m8 * k8 // 2 + m8 * k8 // 16
        extra["gemv_8192_b1"]["w4a8_4096_b8"] = {"entry": "nvfp4a_gemm, INT8 activations, 8 vectors, 4096 x 4096", "kernel": "gemv_blocked_kernel (DP4A, exact block sums)",
                                                 "us_per_call": ms_g8 * 1e3, "gbs": b8 / (ms_g8 * 1e-3) / 1e9, "frac": b8 / (ms_g8 * 1e-3) / 1e9 / peaks["hbm_gbs"]}
        del ws, tws, imgs, w8, t_w8
    # ---- quantization 8192^2 BF16 -> NVFP4, swizzled scales: 3 inputs = 403 MB > L2 ----
    if only in ("all", "quant"):
        nx = 3
        xs = [W.outlier_input(QUANT_R, QUANT_C, 500 + s + 1000 * rank, dev) for s in range(nx)]
        out = W.QuantizedMatrix(QUANT_R, QUANT_C, True, dev)
        qbytes = QUANT_R * QUANT_C * 2 + QUANT_R * QUANT_C // 2 + QUANT_R * QUANT_C // 16
        ms_q, n1 = time_graph(lambda i: W.quantize_amax_swizzled(xs[i % nx], out), 24, 7, 5, dist, world)
        ms_qg, n2 = time_graph(lambda i: W.quantize_given_amax(xs[i % nx], out), 24, 7, 5, dist, world)
        launches += n1 + n2   # amax computed: one cooperative kernel per call (amax, grid barrier, encode)
        extra["quant_8192"] = hbm_entry("quantize_bf16_nvfp4_8192x8192_gbs", qbytes, ms_q, world, peaks, traffic, "quant_8192_dram_bytes",
                                        "quantize_ex_8192x8192_bf16_swizzled_amax_computed", "3 rotating inputs (403 MB) > L2",
                                        timing="CUDA graph of 24 calls, median of 7 replays",
                                        note="amax computed by the call: the input is read twice, the second read is not credited",
                                        amax_given={"us_per_call": ms_qg * 1e3, "gbs": qbytes / (ms_qg * 1e-3) / 1e9,
                                                    "frac": qbytes / (ms_qg * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                                    "note": "global given (delayed scaling): one read, one write"})
        del xs, out

    # ---- fused transformer-MLP GEMMs (W4A16, extended epilogue) at 2048 tokens ----
    if not args.no_mlp and only in ("all", "mlp"):
        extra["mlp_w4a16"] = bench_mlp(args, L, W, dev, rank, world, dist, stream, peaks, traffic)
        launches += extra["mlp_w4a16"].pop("_launches")
    # ---- tensor-parallel decoder linear stack ----
    if not args.no_tp and only in ("all", "tp"):
        extra["tp_llama8b_linears"] = bench_tp(args, dev, rank, world, dist, stream, peaks, L)
        launches += extra["tp_llama8b_linears"].pop("_launches")

    clocks = sampler.stop() if rank == 0 else None
    # A non-zero status word means a bounded wait inside a tensor-core kernel ran out (about two seconds) and that launch
    # returned early: the line is still printed, with the code in it (`kernel_status`, 0 = healthy), and stderr says so.
    status = W.kernel_status()
    if status:
        print(f"bench: a tensor-core kernel gave up a wait (status 0x{status:x}): one launch returned early", file=sys.stderr)

    # ---- CPU baseline beside it (rank 0, N = 1 only): bounded sample of the same GEMM through the oracle ----
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu and only == "all":
        threads = os.cpu_count() or 1
        cols = CPU_COLS
        cpu_gemm_sample(cols, threads)   # builds the operands, warms the pages
        ts = []
        t0 = time.perf_counter()
        while len(ts) < 3 or (time.perf_counter() - t0 < 12.0 and len(ts) < 40):
            ts.append(cpu_gemm_sample(cols, threads))
        ts.sort()
        t = ts[len(ts) // 2]
        cpu = {"value": 2.0 * M * cols * K / t / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
               "sample": f"median of {len(ts)} x ({cols} of {N} output columns x {M} rows x k {K}) through the oracle's exact block sums; "
                         "operands built outside the timed call"}
        if "gemv_8192_b1" in extra:
            gbs, sec = cpu_gemv_baseline(threads)
            extra["gemv_8192_b1"]["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "seconds": sec,
                                                     "sample": "the whole workload once (8192 x 8192 x 1) through the oracle, in the order of the reference's GEMV kernel"}
        if "quant_8192" in extra:
            gbs, sec = cpu_quant_baseline(threads)
            extra["quant_8192"]["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "seconds": sec,
                                                   "sample": "the whole workload once (8192 x 8192 FP32 -> NVFP4, amax computed, swizzled scales) through the oracle"}

    if rank == 0:
        line = {"metric": "w4a4_gemm_4096_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "fp4 (e2m1, ue4m3 block scales) -> fp32 accumulate -> bf16", "data": "synthetic",
                "config": HEADLINE_CONFIG,
                "roofline": roofline, "timing": timing, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
                "kernel_status": status, "traffic_stamp": traffic_stamp, "extra": extra}
        tp = extra.get("tp_llama8b_linears", {})
        if "tp_efficiency" in tp:
            line["tp_efficiency"] = tp["tp_efficiency"]
        print(json.dumps(line), flush=True)
        parity_failed = tp.get("parity", "bit-exact") != "bit-exact"
    if world > 1:
        dist.destroy_process_group()
    if rank == 0 and parity_failed:
        sys.exit("bench: the sharded linear stack differs from the unsharded one (see extra.tp_llama8b_linears.parity)")


def bench_mlp(args, L, W, dev, rank, world, dist, stream, peaks, traffic):
    """gate / up (RMSNorm column scale + SwiGLU + bias + amax) and down (second output + sums of squares) of a Llama-3-8B MLP
    through nvfp4a_gemm_tc_ex: NVFP4 weights, 2048 BF16 tokens."""
    import torch
    T, H, I = 2048, 4096, 14336
    gu = W.quantize_decode_factor(W.randn_bf16(2 * I, H, 0.02, 600 + rank, dev))
    dn = W.quantize_decode_factor(W.randn_bf16(H, I, 0.02, 601 + rank, dev))
    gu_img, t_gu = W.weight_image(gu)
    dn_img, t_dn = W.weight_image(dn)
    x = W.randn_bf16(T, H, 1.0, 602 + rank, dev)
    parts = torch.rand(T, 256, device=dev) * 0.03 + 0.002
    bias_gu, bias_dn = W.randn_bf16(1, 2 * I, 0.01, 603, dev), W.randn_bf16(1, H, 0.01, 604, dev)
    w2 = (torch.rand(H, device=dev) + 0.5).float()
    h = torch.empty(T * I, dtype=torch.bfloat16, device=dev)
    y = torch.empty(T * H, dtype=torch.bfloat16, device=dev)
    d2 = torch.empty(T * H, dtype=torch.bfloat16, device=dev)
    sq = torch.empty(T * (H // 16), dtype=torch.float32, device=dev)
    amax = torch.zeros(2, dtype=torch.float32, device=dev)
    ws = torch.zeros(L.lib.nvfp4a_tc_workspace_bytes(), dtype=torch.uint8, device=dev)
    ex_gu, ex_dn = L.Epilogue(), L.Epilogue()
    ex_gu.norm_parts, ex_gu.norm_nparts, ex_gu.norm_ld, ex_gu.norm_inv_n, ex_gu.norm_eps = parts.data_ptr(), 256, 256, 1.0 / H, 1e-6
    ex_gu.swiglu = 1
    ex_dn.d2, ex_dn.d2_dtype, ex_dn.ldd2, ex_dn.w2, ex_dn.w2_dtype, ex_dn.sq, ex_dn.ld_sq = d2.data_ptr(), L.BF16, H, w2.data_ptr(), L.FP32, sq.data_ptr(), H // 16

    def image_b(t, rows, k):
        img = torch.empty(L.lib.nvfp4a_tc_image_bytes(L.TC_B, L.BF16, rows, k), dtype=torch.uint8, device=dev)
        tt = W.tensor(t, L.BF16)
        L.check(L.lib.nvfp4a_tc_image(L.TC_B, ctypes.byref(tt), k, rows, k, W.ptr(img), W.stream_ptr()))
        return img

    xi, hi = image_b(x, T, H), None
    t_h, t_y = W.tensor(h, L.BF16, amax=amax[0:1]), W.tensor(y, L.BF16, amax=amax[1:2])
    t_bg, t_bd = W.tensor(bias_gu, L.BF16), W.tensor(bias_dn, L.BF16)
    t_xi = W.tensor(xi, L.BF16)

    def gate_up(i):
        L.check(L.lib.nvfp4a_gemm_tc_ex(2 * I, T, H, 1.0, ctypes.byref(t_gu), ctypes.byref(t_xi), 0.0, None, 0, ctypes.byref(t_h), I, ctypes.byref(t_bg),
                                        ctypes.byref(ex_gu), W.ptr(ws), W.stream_ptr()))

    gate_up(0)
    hi = image_b(h.view(T, I), T, I)
    t_hi = W.tensor(hi, L.BF16)

    def down(i):
        L.check(L.lib.nvfp4a_gemm_tc_ex(H, T, I, 1.0, ctypes.byref(t_dn), ctypes.byref(t_hi), 0.0, None, 0, ctypes.byref(t_y), H, ctypes.byref(t_bd),
                                        ctypes.byref(ex_dn), W.ptr(ws), W.stream_ptr()))

    steps = max(3, min(args.steps, 10))
    ms_gu = time_steps(gate_up, steps, 3, stream, dist, world) / steps
    ms_dn = time_steps(down, steps, 3, stream, dist, world) / steps
    f_gu, f_dn = 2.0 * 2 * I * T * H, 2.0 * H * T * I
    tf = lambda f, ms: f / (ms * 1e-3) / 1e12

    # the same gate / up GEMM with INT8 activations (W4A8): nvfp4a_gemm_ex on plain operands, exact DP4A block sums
    xq = torch.empty(T, H, dtype=torch.int8, device=dev)
    xsc = torch.empty(T, H // 16, dtype=torch.float32, device=dev)
    src, dst = W.tensor(x, L.BF16), W.tensor(xq, L.INT8, xsc, 0)
    L.check(L.lib.nvfp4a_quantize(ctypes.byref(src), H, ctypes.byref(dst), H, T, H, W.stream_ptr()))
    t_xq, t_gu_plain = W.tensor(xq, L.INT8, xsc, H // 16), gu.tensor()

    def gate_up_w4a8(i):
        L.check(L.lib.nvfp4a_gemm_ex(2 * I, T, H, 1.0, ctypes.byref(t_gu_plain), H, ctypes.byref(t_xq), H, 0.0, None, 0, ctypes.byref(t_h), I,
                                     ctypes.byref(t_bg), ctypes.byref(ex_gu), W.stream_ptr()))

    ms_gu8 = time_steps(gate_up_w4a8, 3, 1, stream, dist, world) / 3
    route8 = L.lib.nvfp4a_b200_last_route()
    old = L.lib.nvfp4a_b200_set_route(3)   # the same call on the exact DP4A kernel
    ms_gu8x = time_steps(gate_up_w4a8, 3, 1, stream, dist, world) / 3
    L.lib.nvfp4a_b200_set_route(old)
    return {"metric": "mlp_w4a16_tflops", "unit": "TFLOP/s", "value": tf(f_gu + f_dn, ms_gu + ms_dn) * world, "tokens": T,
            "gate_up": {"m": 2 * I, "k": H, "epilogue": "RMSNorm column scale + bias + SwiGLU + amax", "ms": ms_gu, "tflops": tf(f_gu, ms_gu)},
            "down": {"m": H, "k": I, "epilogue": "bias + second output * w2 + sums of squares + amax", "ms": ms_dn, "tflops": tf(f_dn, ms_dn)},
            "gate_up_w4a8": {"entry": "nvfp4a_gemm_ex, INT8 activations",
                             "kernel": {8: "W4A16 tcgen05 kernel on three BF16 planes of the activations (within the accumulation bound)",
                                        7: "DP4A tiled GEMM (exact block sums, CUDA cores)"}.get(route8, str(route8)),
                             "ms": ms_gu8, "tflops": tf(f_gu, ms_gu8), "includes": "the planes' allocation from the stream's pool and their conversion kernel",
                             "exact_dp4a": {"ms": ms_gu8x, "tflops": tf(f_gu, ms_gu8x), "how": "nvfp4a_b200_set_route(3): bit-identical to the reference's tiled order"}},
            "roofline": {"bound": "tensor", "achieved": tf(f_gu + f_dn, ms_gu + ms_dn), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": tf(f_gu + f_dn, ms_gu + ms_dn) / peaks["bf16_tflops"], "traffic": traffic.get("mlp_w4a16_dram_bytes"),
                         "traffic_note": "one gate / up launch plus one down launch"},
            "config": {"workload": "llama3_8b_mlp_w4a16_2048_tokens", "entry": "nvfp4a_gemm_tc_ex"}, "_launches": 2 * (steps + 3) * 3 + 1 + 5 + 4 + 4}


def bench_tp(args, dev, rank, world, dist, stream, peaks, L):
    """Llama-3-8B-shaped linear stack, weights sharded by output rows over the ranks, NCCL all-gather per layer: decode
    (1 and 8 tokens, the whole step in one CUDA graph when the collectives capture) and prefill (4096 tokens)."""
    import torch
    from nvfp4effma_b200.tp import TPDecoderLinears
    layers = args.tp_layers
    stack = TPDecoderLinears(layers=layers, group=None, seed=4, device=dev)
    weights = 218103808 * layers   # values: QKV 6144 x 4096, O 4096 x 4096, gate / up 28672 x 4096, down 4096 x 14336
    out = {"layers": layers, "world": world, "weight_bytes_per_rank": stack.weight_bytes_local(), "_launches": 0,
           "collective": {"peer": "own all-gather over peer-mapped buffers (nvfp4a_b200_tp_gather)", "nccl": "all_gather_into_tensor",
                          "none": "single rank"}[stack.collective]}

    def decode(T, tag):
        g = torch.Generator(device=dev).manual_seed(40 + T)
        h = torch.randn((T, 4096), generator=g, device=dev).bfloat16()
        for _ in range(2):
            stack(h)
        torch.cuda.synchronize()
        graph = None
        try:
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                stack(h)
            gr.replay()
            torch.cuda.synchronize()
            graph = gr
        except Exception:
            graph = None
        step = (lambda i: graph.replay()) if graph is not None else (lambda i: stack(h))
        steps = 20
        ms = time_steps(step, steps, 3, stream, dist, world) / steps
        gbs = weights * 0.5625 / (ms * 1e-3) / 1e9
        out[tag] = {"ms_per_step": ms, "tokens_per_s": T / (ms * 1e-3), "weight_gbs_all_ranks": gbs, "frac_of_hbm_all_ranks": gbs / (peaks["hbm_gbs"] * world),
                    "cuda_graph": graph is not None}
        out["_launches"] += 4 * layers * (steps + 6)

    if world > 1:
        out["parity"] = tp_parity(stack, dev, dist, L)
    decode(1, "decode_1")
    decode(8, "decode_8")
    if world > 1 and stack.collective == "peer":   # the same step with NCCL all-gathers, for comparison
        stack.set_collective("nccl")
        decode(1, "decode_1_nccl")
        stack.set_collective("peer")
    if not args.no_tp_prefill:
        T = 4096
        g = torch.Generator(device=dev).manual_seed(44)
        h = torch.randn((T, 4096), generator=g, device=dev).bfloat16()
        stack(h)
        steps = 3
        ms = time_steps(lambda i: stack(h), steps, 1, stream, dist, world) / steps
        tfl = 2.0 * weights * T / (ms * 1e-3) / 1e12
        out["prefill_4096"] = {"ms_per_step": ms, "tokens_per_s": T / (ms * 1e-3), "tflops_all_ranks": tfl,
                               "frac_of_bf16_peak_all_ranks": tfl / (peaks["bf16_tflops"] * world)}
        out["_launches"] += 8 * layers * (steps + 2)
    if world > 1:
        # strong scaling of this stack: the same layers unsharded on one GPU (every rank times its own copy; the slowest counts)
        del stack
        torch.cuda.empty_cache()
        solo = TPDecoderLinears(layers=layers, group=None, seed=4, device=dev, replicate=True)
        h1 = torch.randn((1, 4096), generator=torch.Generator(device=dev).manual_seed(41), device=dev).bfloat16()
        for _ in range(2):
            solo(h1)
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            solo(h1)
        gr.replay()
        t1_decode = time_steps(lambda i: gr.replay(), 20, 3, stream, dist, world) / 20
        eff = {"definition": "t_1 / (N * t_N): one GPU running the whole unsharded stack against N GPUs running their shards",
               "decode_1": {"t1_ms": t1_decode, "tN_ms": out["decode_1"]["ms_per_step"], "efficiency": t1_decode / (world * out["decode_1"]["ms_per_step"])}}
        out["_launches"] += 4 * layers * 26
        if "prefill_4096" in out:
            hp = torch.randn((4096, 4096), generator=torch.Generator(device=dev).manual_seed(44), device=dev).bfloat16()
            solo(hp)
            t1_prefill = time_steps(lambda i: solo(hp), 3, 1, stream, dist, world) / 3
            eff["prefill_4096"] = {"t1_ms": t1_prefill, "tN_ms": out["prefill_4096"]["ms_per_step"],
                                   "efficiency": t1_prefill / (world * out["prefill_4096"]["ms_per_step"])}
            out["_launches"] += 8 * layers * 5
        out["tp_efficiency"] = eff
    return out


def tp_parity(stack, dev, dist, L):
    """Sharded against unsharded, bit for bit, on the first two layers of the benchmark's own stack (full Llama-3-8B shapes):
    1, 8 and 64 tokens through the peer-memory all-gather (with the fused prefill GEMM at 64 tokens) and through NCCL.  The
    decode GEMVs are pinned to one kernel for the comparison: left to itself the library gives a 28672-row unsharded layer to
    the FP4 tensor-core GEMV and its shards to the mma.sync GEMV, which add in different orders (both within the accumulation
    bound, not bit-identical to each other).  Returns "bit-exact" or a description of the first difference."""
    import torch
    from nvfp4effma_b200.tp import TPDecoderLinears
    solo = TPDecoderLinears(layers=2, group=None, seed=4, device=dev, replicate=True)
    bad = []
    L.lib.nvfp4a_b200_set_route(2)
    try:
        for T in (1, 8, 64):
            h = torch.randn((T, 4096), generator=torch.Generator(device=dev).manual_seed(70 + T), device=dev).bfloat16()
            want = solo(h, layers=2, collect=True)
            modes = ["peer", "nccl"] if stack.collective == "peer" else [stack.collective]
            for mode in modes:
                stack.set_collective(mode)
                got = stack(h, layers=2, collect=True)
                for li, (g, w) in enumerate(zip(got, want)):
                    if not torch.equal(g, w):
                        bad.append(f"{mode} T={T} layer {li}: {int((g != w).sum())} of {g.numel()} values differ")
            stack.set_collective(modes[0])
    finally:
        L.lib.nvfp4a_b200_set_route(0)
    flag = torch.tensor([len(bad)], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    del solo
    torch.cuda.empty_cache()
    if int(flag[0]) == 0:
        return "bit-exact"
    return "MISMATCH: " + ("; ".join(bad) if bad else "on another rank")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline beside the GPU number")
    ap.add_argument("--no-mlp", action="store_true", help="skip the fused-MLP (W4A16, extended epilogue) extra")
    ap.add_argument("--no-tp", action="store_true", help="skip the tensor-parallel linear stack extra")
    ap.add_argument("--no-tp-prefill", action="store_true", help="tensor-parallel extra: decode only")
    ap.add_argument("--tp-layers", type=int, default=32)
    ap.add_argument("--pair", type=int, default=-1, choices=[-1, 0, 1],
                    help="W4A4 GEMM: -1 automatic, 0 single-CTA tiles only, 1 CTA pairs wherever they apply (tuning aid)")
    ap.add_argument("--no-pdl", action="store_true", help="launch without programmatic stream serialization (tuning aid)")
    ap.add_argument("--only", default="all", choices=["all", "gemm", "gemv", "quant", "mlp", "tp"],
                    help="run one workload only (for profiling captures); the JSON line then lacks the others")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
