#!/usr/bin/env python
"""Benchmark of the Palimpsa operator hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload all|c2|decode|varlen|layer]

Headline workload ("C2"): the 170M-model-shaped layer op, chunked forward + backward in bf16 with fp32 state,
B=8, T=4096, H=6, d_k=d_v=128, seeded synthetic inputs (q,k L2-normalised N(0,1); v ~ N(0,1); b = sigmoid(N);
gt, g = softplus(N); Ip = 1; dO ~ N(0,1)).  One step = one forward and one backward over that batch.  With N > 1
GPUs every rank runs the same per-GPU batch on its own shard of a global batch of 8*N sequences: the op is
independent per (sequence, head), so there is no data-path collective ("weak" scaling); ranks only meet at the
timing barriers.

Prints ONE JSON line (rank 0).  ``value`` is timed with inputs resident in HBM; ``e2e`` is the same step through
the public Python API from pinned HOST buffers, host->device and device->host copies inside the timed region
(``e2e.copy_only_ms``: the same copies with no kernel between them).  ``roofline`` describes the dominant kernel
(the backward main kernel), timed alone with CUDA events through the staged C-ABI entry point.  ``cpu_baseline``
is the naive per-timestep recurrence (float32 port of the reference's ``palimpsa_ref``, forward + autograd
backward) on this box's host cores, on a truncated sample.  ``gpu_baseline`` is the reference's own Triton ops
(unmodified working copy under oracle/_ref) on the same GPU.  ``workloads`` carries the other configurations of
the metric in the same line:

    decode     256 sequences x 12 heads, fp32 (mu, I) cache, single-token bf16 steps: tokens/s and HBM GB/s
    varlen     one packed batch of 32 768 tokens, documents of seeded random length in [128, 4096]
    c5         one 131 072-token sequence, H=12: one GPU with the planner's segments (N=1), or context-parallel
               over the N ranks (boundary states through peer-mapped buffers, and by NCCL send/recv beside it), with the one-GPU time measured in the same run
    c2_strong  the C2 batch (global B=8) sharded over the N ranks by (sequence, head): strong scaling
    model_shapes  chunk fwd+bwd at the head shapes of the reference's shipped model configurations, beside its Triton ops

``--impl reference`` times only the CPU recurrence (the reference has no other CPU path).
"""
from __future__ import annotations

import argparse
import ctypes as C
import hashlib
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

METRIC = "fwd+bwd tokens/s (chunk, bf16, T=4096)"
C2 = dict(B=8, T=4096, H=6, K=128, V=128)
C4 = dict(B=256, H=12, K=128, V=128)
C5 = dict(B=1, T=131072, H=12, K=128, V=128)
L2_BYTES = 126 * 1024 * 1024
NAMES = ("q", "k", "v", "b", "gt", "g", "Ip")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "source": "fallback"}


def make_inputs(B, T, H, K, V, dtype, device, seed=0, pin=False, on_device=False):
    """Seeded synthetic inputs drawn in a fixed order (see module docstring): on the CPU generator, or, for the
    long-sequence workloads where a CPU draw would take longer than the measurement, with ``on_device`` on the
    device's generator (same distributions, same values on every GPU of the box for one seed)."""
    if on_device:
        gen = torch.Generator(device=device).manual_seed(seed)
        rn = lambda *s: torch.randn(*s, generator=gen, dtype=torch.float32, device=device)
    else:
        gen = torch.Generator().manual_seed(seed)
        rn = lambda *s: torch.randn(*s, generator=gen, dtype=torch.float32)
    q = torch.nn.functional.normalize(rn(B, T, H, K), dim=-1)
    k = torch.nn.functional.normalize(rn(B, T, H, K), dim=-1)
    v = rn(B, T, H, V)
    b = torch.sigmoid(rn(B, T, H, V))
    gt = torch.nn.functional.softplus(rn(B, T, H))
    g = torch.nn.functional.softplus(rn(H))
    Ip = torch.ones(H, device=device if on_device else None)
    do = rn(B, T, H, V)
    host = {"q": q.to(dtype), "k": k.to(dtype), "v": v.to(dtype), "b": b.to(dtype), "gt": gt, "g": g, "Ip": Ip,
            "do": do.to(dtype)}
    if on_device:
        return None, host
    if pin:
        host = {n: x.pin_memory() for n, x in host.items()}
    if device is None:
        return host, None
    return host, {n: x.to(device) for n, x in host.items()}


def packed_lengths(T=32768, seed=0):
    """Document lengths of the packed batch: uniform in [128, 4096] until T tokens are reached, last one cut."""
    gen = torch.Generator().manual_seed(seed)
    lens, tot = [], 0
    while tot < T:
        n = min(int(torch.randint(128, 4097, (1,), generator=gen).item()), T - tot)
        lens.append(n)
        tot += n
    return lens


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, val in zip(names, r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# CPU baseline: the naive recurrence (port of the reference's palimpsa_ref), forward + autograd backward
# ------------------------------------------------------------------------------------------------
def cpu_step(inp):
    from oracle.palimpsa_oracle import naive_recurrence_fp32
    leaves = [inp[n].clone().requires_grad_(True) for n in NAMES]
    o = naive_recurrence_fp32(*leaves)
    o.backward(inp["do"].to(o.dtype))
    return o


def cpu_baseline(budget_s, cfg, steps=5, warmup=1):
    """Times the naive recurrence on a truncated sample (same B, H, d_k, d_v; T cut so that the whole call stays
    within ``budget_s`` seconds).  Returns (best tokens/s, description, per-step seconds)."""
    B, H, K, V = cfg["B"], cfg["H"], cfg["K"], cfg["V"]
    torch.set_num_threads(os.cpu_count() or 1)        # launchers pin OMP_NUM_THREADS=1; the baseline gets every core
    probe, _ = make_inputs(B, 4, H, K, V, torch.bfloat16, None, seed=1)
    cpu_step(probe)                                   # first call pays one-time costs
    t0 = time.perf_counter()
    cpu_step(probe)
    per_tok = (time.perf_counter() - t0) / 4
    T = int(max(4, min(256, budget_s / max(per_tok, 1e-6) / max(1, steps + warmup))))
    inp, _ = make_inputs(B, T, H, K, V, torch.bfloat16, None, seed=0)
    for _ in range(warmup):
        cpu_step(inp)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        cpu_step(inp)
        times.append(time.perf_counter() - t0)
    best = min(times)
    return B * T / best, f"B={B} H={H} d_k={K} d_v={V} bf16 inputs, T truncated to {T} (autograd through the " \
                         f"naive loop keeps every step's state); {warmup} warm-up, best of {steps}", times


def spread(times, tokens):
    """Slowest / median / fastest step of a CPU timing, as tokens/s."""
    return {"min": tokens / max(times), "median": tokens / statistics.median(times), "max": tokens / min(times)}


def run_reference(args, rank, world):
    if rank != 0:
        return
    steps = max(5, args.steps)
    val, sample, times = cpu_baseline(150.0, C2, steps=steps, warmup=max(1, args.warmup))
    cores = torch.get_num_threads()                   # as set by cpu_baseline: every host core
    ms = 1e3 * sum(times) / len(times)
    tokens = val * min(times)
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": max(1, args.warmup), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "C2 170M-shaped chunk fwd+bwd B=8 T=4096 H=6 d_k=d_v=128 (CPU sample truncated in T)"},
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample,
                             "spread_tokens_per_s": spread(times, tokens)},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0, "host_cpus": os.cpu_count()}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU arm: helpers
# ------------------------------------------------------------------------------------------------
def fwd_bwd(d, **kw):
    from palimpsa_b200.ops import chunk_palimpsa
    leaves = [d[n].detach().requires_grad_(True) for n in NAMES]
    o = chunk_palimpsa(*leaves, chunk_size=64, **kw)
    o.backward(d["do"])
    return o, [x.grad for x in leaves]


def time_region(fn, steps, warmup, world, dev):
    """``steps`` calls of ``fn`` between CUDA events on the current stream, after ``warmup`` calls; barrier and
    synchronize on both sides; the maximum over ranks.  Returns the total in ms."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def dram_traffic(kernel, source, token_heads):
    """DRAM bytes of one launch of ``kernel``, scaled by token-heads from the ncu capture recorded in
    profiles/dram_traffic.md -- but only if that capture was taken on the kernel source that is running now
    (sha256 of the .cu file); otherwise None."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.md")
    src = os.path.join(ROOT, "palimpsa_b200", "csrc", source)
    if not (os.path.exists(path) and os.path.exists(src)):
        return None, "no capture on record"
    with open(src, "rb") as f:
        sha = hashlib.sha256(f.read()).hexdigest()[:12]
    with open(path) as f:
        for line in f:
            cells = [c.strip().strip("`") for c in line.strip().strip("|").split("|")]
            if len(cells) >= 5 and cells[0] == kernel and cells[1] == sha:
                try:
                    return float(cells[2]) * token_heads / float(cells[3]), f"ncu capture of {cells[4]}; scaled by the units one launch processes"
                except ValueError:
                    continue
    return None, f"no ncu capture of this kernel version ({source} sha256 {sha}) on record"


def kernel_roofline(d, cfg, steps, peaks):
    """Times the backward main kernel alone (CUDA events on its stream) through the C ABI."""
    from palimpsa_b200 import _lib as L
    from palimpsa_b200.ops.palimpsa import _core
    lib = L.lib()
    B, T, H, K, V = cfg["B"], cfg["T"], cfg["H"], cfg["K"], cfg["V"]
    q, k, v, b, gt, g, Ip, do = [d[n] for n in NAMES + ("do",)]
    with torch.no_grad():
        _, _, _, _, ckM, ckI, _, _ = _core.fwd_op(q, k, v, b, gt, g, Ip, None, None, None, K ** -0.5, False, True, False,
                                                  False, 1)
    dq, dk, dv, db = [torch.empty_like(x) for x in (q, k, v, b)]
    dgt = torch.empty(B, T, H, device=q.device)
    dg, dIp = torch.empty(H, device=q.device), torch.empty(H, device=q.device)
    prm = L.BwdParams()
    prm.struct_size = C.sizeof(L.BwdParams)
    prm.p = _core._problem(q, k, v, b, gt, g, Ip, None, None, None, None, K ** -0.5, 0)
    need = lib.palimpsa_bwd_workspace_bytes(C.byref(prm.p))
    ws = torch.empty(need, dtype=torch.uint8, device=q.device)
    prm.d_o, prm.ckpt_M, prm.ckpt_I = do.data_ptr(), ckM.data_ptr(), ckI.data_ptr()
    prm.dq, prm.dk, prm.dv, prm.db = dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), db.data_ptr()
    prm.dgt, prm.dg, prm.dIp = dgt.data_ptr(), dg.data_ptr(), dIp.data_ptr()
    prm.workspace, prm.workspace_bytes = ws.data_ptr(), ws.numel()
    stream = torch.cuda.current_stream()
    sp = C.c_void_p(stream.cuda_stream)
    for _ in range(3):
        L.check(lib.palimpsa_chunk_bwd_stages(C.byref(prm), sp, 1), "bwd main")
    torch.cuda.synchronize()
    times = []
    for _ in range(max(3, steps)):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        L.check(lib.palimpsa_chunk_bwd_stages(C.byref(prm), sp, 1), "bwd main")
        e1.record(stream)
        L.check(lib.palimpsa_chunk_bwd_stages(C.byref(prm), sp, 2), "bwd finish")
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    ms = sum(times) / len(times)
    # the other kernels of a step, each timed alone the same way: finishing kernels, forward (checkpoints on)
    fin = []
    for _ in range(max(3, steps)):
        e0, e1 = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        e0.record(stream)
        L.check(lib.palimpsa_chunk_bwd_stages(C.byref(prm), sp, 2), "bwd finish")
        e1.record(stream)
        torch.cuda.synchronize()
        fin.append(e0.elapsed_time(e1))
    ms_fin = sum(fin) / len(fin)

    # the forward launches back to back (its host side allocates outputs and checkpoints per call, which a single
    # launch timed from an idle GPU would include); one call streams 0.2 GB in and 1.8 GB out, more than L2 holds
    def fwd_once():
        with torch.no_grad():
            _core.fwd_op(q, k, v, b, gt, g, Ip, None, None, None, K ** -0.5, False, True, False, False, 1)
    n_fwd = max(10, steps)
    ms_fwd = time_region(fwd_once, n_fwd, 3, 1, q.device) / n_fwd
    th = B * T * H                                   # token-heads per launch
    es = q.element_size()
    alg_bytes = th * ((2 * K + 3 * V) * es + 4 + (2 * K + 2 * V) * es + 4)   # q,k,v,b,do,gt in; dq,dk,dv,db,dgt out
    flops = 30.0 * K * V * th                        # algorithmic lane-ops of the backward, per the operator's definition
    achieved = alg_bytes / (ms * 1e-3) / 1e9
    traffic, traffic_source = dram_traffic("bwd_kernel", "bwd.cu", th)
    return {"bound": "hbm", "kernel": "bwd_kernel (backward main)", "achieved": achieved, "peak": peaks["hbm_gbs"],
            "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
            "traffic": traffic, "traffic_source": traffic_source,
            "launch_ms": ms, "algorithmic_bytes_per_launch": alg_bytes,
            "workspace_bytes": int(need), "checkpoint_bytes": int(2 * ckM.numel() * 4),
            "note": "the kernel is FP32-pipe bound, not HBM bound: see 'compute'",
            "compute": {"algorithmic_tflops": flops / (ms * 1e-3) / 1e12, "flop_per_token_head": 30 * K * V},
            "other_kernels": {"fwd_kernel": {"launch_ms": ms_fwd, "reciprocals_per_launch": th * K * V,
                                             "trcp_per_s": th * K * V / (ms_fwd * 1e-3) / 1e12},
                              "bwd_finish_rows+heads": {"launch_ms": ms_fin}}}


def fp32_peaks(dev):
    """Measured FP32 FMA and MUFU-reciprocal ceilings of this GPU (register-resident micro-benchmarks)."""
    path = os.path.join(ROOT, "benchmarks", "libpalimpsa_microbench.so")
    if not os.path.exists(path):
        return None
    mb = C.CDLL(path)
    sink = torch.zeros(16, device=dev)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    out = {}
    for kind, name in ((1, "fma_tflops"), (2, "rcp_tops"), (3, "fwd_mix_telem")):
        ms, ops = C.c_float(), C.c_double()
        rc = mb.palimpsa_microbench(kind, sms * 8, 2048, 3, C.c_void_p(sink.data_ptr()), C.byref(ms), C.byref(ops))
        if rc != 0:
            return None
        rate = ops.value / (ms.value * 1e-3) / 1e12
        out[name] = rate * (2.0 if kind == 1 else 1.0)
    return out


def bind_to_gpu_numa_node(local_rank):
    """Runs this process on the CPU cores next to its GPU (as NVML reports them), so that the pinned host
    buffers allocated afterwards land in that socket's memory and uploads / downloads do not cross sockets.
    Reads the topology only; a no-op when NVML or the affinity call is unavailable."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(local_rank)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {64 * w + b for w, m in enumerate(mask) for b in range(64) if (m >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
        return len(cpus)
    except Exception:
        return 0


def copies_only(pipe, host, dev):
    """The host<->device traffic of one end-to-end step with no kernel in between: every slice's inputs up on the
    upload stream, a result-sized set of tensors down on the download stream, same pinned buffers and slice
    bounds as ``HostPipeline.run``.  What the step would cost if compute were free."""
    outs = ("o", "dq", "dk", "dv", "db", "dgt")
    src_of = {"o": "v", "dq": "q", "dk": "k", "dv": "v", "db": "b", "dgt": "gt"}
    for i, (lo, hi) in enumerate(pipe.bounds):
        slot = pipe.slots[i % 2]
        with torch.cuda.stream(pipe.s_in):
            for n in ("q", "k", "v", "b", "gt", "do"):
                slot[n][: hi - lo].copy_(host[n][lo:hi], non_blocking=True)
        with torch.cuda.stream(pipe.s_out):
            for n in outs:
                pipe.out[n][lo:hi].copy_(slot[src_of[n]][: hi - lo], non_blocking=True)
    pipe.s_in.synchronize()
    pipe.s_out.synchronize()


def time_host_region(fn, steps, warmup, world, dev):
    """Wall-clock variant of time_region for work spread over several streams (ends with its own synchronize)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    torch.cuda.synchronize(dev)
    ms = (time.perf_counter() - t0) * 1e3
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    return ms


# ------------------------------------------------------------------------------------------------
# GPU baseline: the reference's own Triton ops on this GPU
# ------------------------------------------------------------------------------------------------
def _load_reference_op(fname, attr):
    path = os.path.join(ROOT, "oracle", "_ref", "palimpsa", "ops", "palimpsa", fname)
    if not os.path.exists(path):
        raise FileNotFoundError("oracle/_ref is absent (python oracle/fetch_reference.py copies the reference there)")
    name = "_bench_reference_" + fname[:-3]
    if name not in sys.modules:
        spec = importlib.util.spec_from_file_location(name, path)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
    return getattr(sys.modules[name], attr)


def gpu_baseline(dev, ours_c2_ms, ours_decode_us, chunk_sizes=(16,), steps=3):
    """The reference's Triton kernels, JIT-compiled here, on the benchmark's shapes: chunk_palimpsa forward +
    backward on C2 (chunk_palimpsa_forgetting_scalar.py:623-667; chunk_size 16 is what its layers pass) and one
    fused_recurrent_palimpsa decode step on C4 (fused_recurrent_palimpsa.py:258-297).  Same inputs, CUDA events,
    warm-up first (it also pays the JIT).  A case that fails to compile or run is reported, not retried."""
    out = {"impl": "reference Triton ops, unmodified (oracle/_ref)", "device": torch.cuda.get_device_name(dev)}
    try:
        import triton
        out["triton"] = triton.__version__
        chunk = _load_reference_op("chunk_palimpsa_forgetting_scalar.py", "chunk_palimpsa")
        fused = _load_reference_op("fused_recurrent_palimpsa.py", "fused_recurrent_palimpsa")
    except Exception as e:                                # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
    B, T, H, K, V = C2["B"], C2["T"], C2["H"], C2["K"], C2["V"]
    _, d = make_inputs(B, T, H, K, V, torch.bfloat16, dev, seed=0)
    for cs in chunk_sizes:
        key = f"c2_chunk{cs}"
        try:
            def step():
                leaves = [d[n].detach().requires_grad_(True) for n in NAMES]
                o = chunk(*leaves, chunk_size=cs)
                o.backward(d["do"])
            t0 = time.perf_counter()
            step()
            torch.cuda.synchronize(dev)
            jit_s = time.perf_counter() - t0
            step()
            torch.cuda.synchronize(dev)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                step()
            e1.record()
            torch.cuda.synchronize(dev)
            ms = e0.elapsed_time(e1) / steps
            out[key] = {"ms_per_step": ms, "tokens_per_s": B * T / (ms * 1e-3), "first_call_s": jit_s,
                        "ours_ms_per_step": ours_c2_ms, "speedup_ours": ms / ours_c2_ms}
        except Exception as e:                            # noqa: BLE001
            out[key] = {"unavailable": f"{type(e).__name__}: {str(e)[:300]}"}
            torch.cuda.synchronize(dev)
    del d
    torch.cuda.empty_cache()
    try:
        Bd, Hd = C4["B"], C4["H"]
        _, t = make_inputs(Bd, 1, Hd, K, V, torch.bfloat16, dev, seed=1)
        mu = torch.randn(Bd, Hd, V, K, device=dev) * 0.1
        I = torch.rand(Bd, Hd, V, K, device=dev) + 1.0

        def dstep(mu, I):
            with torch.no_grad():
                _, mu, I = fused(*[t[n] for n in NAMES], initial_mu_state=mu, initial_I_state=I, output_final_state=True)
            return mu, I
        for _ in range(3):
            mu, I = dstep(mu, I)
        torch.cuda.synchronize(dev)
        n = 50
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            mu, I = dstep(mu, I)
        e1.record()
        torch.cuda.synchronize(dev)
        us = e0.elapsed_time(e1) / n * 1e3
        out["c4_decode_step"] = {"us_per_step": us, "tokens_per_s": Bd / (us * 1e-6), "ours_us_per_step": ours_decode_us,
                                 "speedup_ours": us / ours_decode_us if ours_decode_us else None}
    except Exception as e:                                # noqa: BLE001
        out["c4_decode_step"] = {"unavailable": f"{type(e).__name__}: {str(e)[:300]}"}
    torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------------------------------
# Workloads beside the headline
# ------------------------------------------------------------------------------------------------
def decode_workload(dev, steps):
    """C4: B=256 concurrent sequences with an fp32 (mu, I) state cache each (H=12, d_k=d_v=128), prefilled from a
    random 2048-token context, then ``steps`` single-token bf16 steps on fresh seeded inputs."""
    from palimpsa_b200.ops import DecodeGraph, chunk_palimpsa, decode_step
    B, H, K, V = C4["B"], C4["H"], C4["K"], C4["V"]
    gen = torch.Generator(device=dev).manual_seed(0)
    rn = lambda *s: torch.randn(*s, device=dev, generator=gen)
    g = torch.nn.functional.softplus(rn(H))
    Ip = torch.ones(H, device=dev)

    def tokens(T):
        q = torch.nn.functional.normalize(rn(B, T, H, K), dim=-1).bfloat16()
        k = torch.nn.functional.normalize(rn(B, T, H, K), dim=-1).bfloat16()
        return q, k, rn(B, T, H, V).bfloat16(), torch.sigmoid(rn(B, T, H, V)).bfloat16(), \
            torch.nn.functional.softplus(rn(B, T, H))

    mu = I = None
    with torch.no_grad():
        for _ in range(4):                                   # 2048-token context in four 512-token pieces
            q, k, v, b, gt = tokens(512)
            _, mu, I = chunk_palimpsa(q, k, v, b, gt, g, Ip, initial_mu_state=mu, initial_I_state=I,
                                      output_final_state=True)
        del q, k, v, b, gt
    pool = [tokens(1) for _ in range(32)]                    # fresh inputs per step, cycled
    for i in range(20):
        decode_step(*pool[i % 32], g, Ip, mu, I)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        decode_step(*pool[i % 32], g, Ip, mu, I)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    # the same step replayed from a CUDA graph (inputs copied into the graph's static buffers every step)
    dec = DecodeGraph(g, Ip, mu, I, dtype=torch.bfloat16)
    for i in range(20):
        dec.step(*pool[i % 32])
    torch.cuda.synchronize()
    e0.record()
    for i in range(steps):
        dec.step(*pool[i % 32])
    e1.record()
    torch.cuda.synchronize()
    ms_graph = e0.elapsed_time(e1) / steps
    state_bytes = B * H * V * K * 4 * 2 * 2
    peaks = measured_peaks()
    best = min(ms, ms_graph)
    gbs = state_bytes / (best * 1e-3) / 1e9
    traffic, traffic_source = dram_traffic("decode_kernel", "decode.cu", B * H)
    finite = bool(torch.isfinite(mu).all() and torch.isfinite(I).all())
    del dec, pool, mu, I
    torch.cuda.empty_cache()
    return {"workload": f"C4 decode B={B} H={H} d_k={K} d_v={V}, in-place fp32 state cache, prefill 2048 tokens, bf16 io",
            "steps": steps, "us_per_step_eager": ms * 1e3, "us_per_step_cuda_graph": ms_graph * 1e3,
            "tokens_per_s": B / (best * 1e-3), "gpu_launches": 2 * (steps + 20) + 4,
            "roofline": {"bound": "hbm", "kernel": "decode_kernel", "achieved": gbs, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"], "peak_source": peaks["source"],
                         "algorithmic_bytes_per_launch": state_bytes, "traffic": traffic,
                         "traffic_source": traffic_source},
            "state_finite": finite}


def varlen_workload(dev, steps, warmup):
    """C3: one packed batch of 32 768 tokens made of documents with seeded random lengths in [128, 4096] (H=6,
    d_k=d_v=128, bf16; states reset at every document boundary through ``cu_seqlens``), forward + backward."""
    T, H, K, V = 32768, C2["H"], C2["K"], C2["V"]
    lens = packed_lengths(T)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
    _, d = make_inputs(1, T, H, K, V, torch.bfloat16, dev, seed=0)
    ms = time_region(lambda: fwd_bwd(d, cu_seqlens=cu), steps, max(3, warmup), 1, dev) / steps
    del d
    torch.cuda.empty_cache()
    return {"workload": f"C3 packed batch: {len(lens)} documents, {T} tokens, lengths {min(lens)}..{max(lens)}, H={H} "
                        f"d_k={K} d_v={V} bf16, states reset at document boundaries",
            "ms_per_step": ms, "tokens_per_s": T / (ms * 1e-3), "steps": steps, "gpu_launches": 4 * (steps + max(3, warmup)),
            "limited_by": "the longest documents: one CTA column walks a document serially; the kernels start the "
                          "documents longest first (seq_order), which keeps the tail of the launch short; cutting the "
                          "packed axis into segments was measured and does not pay on this mix"}


MODEL_SHAPES = (  # head shapes of the reference's shipped model configurations: (name, B, T, H, d_k, d_v)
    ("palimpsa_170M (config/palimpsa_170M.json: 16 heads of 48)", 8, 4096, 16, 48, 48),
    ("meta_mamba2_170M (config/meta_mamba2_170M.json: state 48, head 96)", 8, 4096, 16, 48, 96),
    ("not_palimpsa_760M (config/not_palimpsa_760M.json: d_k 96, d_v 192)", 8, 4096, 16, 96, 192),
    ("mqar (zoology/mqar_figure/configs.py: 8 heads, d_k 16, d_v 32)", 64, 512, 8, 16, 32),
)


def model_shapes_workload(dev, steps, with_reference):
    """Chunk forward + backward (bf16, 32 768 tokens per step) at the head shapes the reference's shipped model
    configurations imply, beside the reference's Triton ops (chunk_size 16, as its layers pass) when its working copy
    is present.  ``tflops`` counts the operator's 40 * d_k * d_v flop per token-head."""
    chunk = None
    if with_reference:
        try:
            chunk = _load_reference_op("chunk_palimpsa_forgetting_scalar.py", "chunk_palimpsa")
        except Exception:                                 # noqa: BLE001
            chunk = None
    rows, launches = [], 0
    from palimpsa_b200.ops.palimpsa._core import plan_segments
    for name, B, T, H, K, V in MODEL_SHAPES:
        _, d = make_inputs(B, T, H, K, V, torch.bfloat16, dev, seed=0, on_device=True)
        ms = time_region(lambda: fwd_bwd(d), steps, 3, 1, dev) / steps
        G = plan_segments(B, T, H, K, V, dev, backward=True)
        launches += (8 if G > 1 else 4) * (steps + 3)
        row = {"shape": name, "B": B, "T": T, "H": H, "d_k": K, "d_v": V, "segments": G, "ms_per_step": ms,
               "tokens_per_s": B * T / (ms * 1e-3), "tflops": 40.0 * K * V * B * T * H / (ms * 1e-3) / 1e12}
        if chunk is not None:
            try:
                def step():
                    leaves = [d[n].detach().requires_grad_(True) for n in NAMES]
                    chunk(*leaves, chunk_size=16).backward(d["do"])
                rms = time_region(step, 2, 2, 1, dev) / 2
                row.update(reference_triton_ms_per_step=rms, speedup=rms / ms)
            except Exception as e:                        # noqa: BLE001
                row["reference_triton"] = f"unavailable: {type(e).__name__}: {str(e)[:120]}"
                torch.cuda.synchronize(dev)
        rows.append(row)
        del d
        torch.cuda.empty_cache()
    return {"workload": "chunk fwd+bwd at the head shapes of the reference's shipped configurations, bf16",
            "shapes": rows, "gpu_launches": launches}


def c5_workload(dev, rank, world, steps):
    """C5: one 131 072-token sequence, H=12, d_k=d_v=128, bf16 fwd+bwd.  N=1: the single-GPU op with the planner's
    segments.  N>=2: ``cp_chunk_palimpsa`` over the N ranks (each rank holds T/N contiguous tokens; boundary states
    travel rank to rank through peer-mapped buffers, and once more by NCCL send/recv for comparison); rank 0 also times the whole sequence on its own GPU for the speed-up."""
    from palimpsa_b200.ops.palimpsa._core import padded_k, plan_segments
    B, T, H, K, V = C5["B"], C5["T"], C5["H"], C5["K"], C5["V"]
    out = {"workload": f"C5 long context B={B} T={T} H={H} d_k={K} d_v={V} bf16 chunk fwd+bwd"}
    single_ms = None
    if rank == 0:
        _, d = make_inputs(B, T, H, K, V, torch.bfloat16, dev, seed=0, on_device=True)
        G = plan_segments(B, T, H, K, V, dev, backward=True)
        n1 = max(2, min(steps, 5))
        single_ms = time_region(lambda: fwd_bwd(d), n1, 2, 1, dev) / n1
        out["single_gpu"] = {"ms_per_step": single_ms, "tokens_per_s": T / (single_ms * 1e-3), "segments": G,
                             "gpu_launches_per_step": 8 if G > 1 else 4}
        del d
        torch.cuda.empty_cache()
    if world == 1:
        out.update(ms_per_step=single_ms, tokens_per_s=T / (single_ms * 1e-3), n_gpus=1)
        return out
    from palimpsa_b200.parallel import cp_chunk_palimpsa, shard_bounds
    lo, hi = shard_bounds(T, rank, world)
    _, full = make_inputs(B, T, H, K, V, torch.bfloat16, dev, seed=0, on_device=True)   # the same sequence on every rank
    loc = {n: (x[:, lo:hi] if x.dim() >= 3 else x).contiguous() for n, x in full.items()}
    del full
    torch.cuda.empty_cache()

    def step():
        leaves = [loc[n].detach().requires_grad_(True) for n in NAMES]
        cp_chunk_palimpsa(*leaves).backward(loc["do"])

    def step_nccl():
        leaves = [loc[n].detach().requires_grad_(True) for n in NAMES]
        cp_chunk_palimpsa(*leaves, transport="nccl").backward(loc["do"])

    from palimpsa_b200.parallel import PeerLink
    n = max(3, min(steps, 10))
    ms = time_region(step, n, 3, world, dev) / n                 # transport "auto": peer-mapped buffers where available
    hop = 2 * B * H * V * padded_k(K) * 4
    peer = PeerLink.get(None, hop // 4, dev) is not None
    ms_nccl = time_region(step_nccl, n, 3, world, dev) / n if peer else ms
    out.update(ms_per_step=ms, tokens_per_s=T / (ms * 1e-3), n_gpus=world, tokens_per_rank=hi - lo,
               bytes_per_hop=hop, hops_per_step=2 * (world - 1),
               transport="peer-mapped buffers: the boundary-scan kernel stores into the next rank's memory over "
                         "NVLink, bounded wait / signal kernels order the hand-over" if peer else
                         "torch.distributed send/recv (NCCL)",
               ms_per_step_send_recv=ms_nccl,
               collective="one 1.5 MB boundary state per hop, down in forward and up in backward; all-reduce of dg, "
                          "dIp (2*H floats)",
               limited_by="the rank-to-rank chain is serial: 2*(N-1) hops of wait, relay kernel (decay * in + total) and "
                          "signal; the heavy kernels run on all ranks side by side")
    if single_ms is not None:
        out["speedup_vs_single_gpu"] = single_ms / ms
        out["efficiency"] = single_ms / ms / world
    del loc
    torch.cuda.empty_cache()
    return out


def c2_strong_workload(dev, rank, world, steps, warmup, single_ms):
    """The C2 batch itself (global B=8, H=6: 48 (sequence, head) units) sharded over the N ranks with no
    collective: ranks take contiguous runs of sequences (N <= 8 divides the batch; a rank left with few units cuts
    its sequences into segments to fill its GPU)."""
    from palimpsa_b200.ops.palimpsa._core import plan_segments
    from palimpsa_b200.parallel import shard_bounds
    B, T, H, K, V = C2["B"], C2["T"], C2["H"], C2["K"], C2["V"]
    lo, hi = shard_bounds(B, rank, world)
    host, _ = make_inputs(B, T, H, K, V, torch.bfloat16, None, seed=0)
    d = {n: (x[lo:hi] if x.dim() >= 3 else x).contiguous().to(dev) for n, x in host.items()}
    del host
    if hi > lo:
        step = lambda: fwd_bwd(d)
    else:
        step = lambda: None
    ms = time_region(step, steps, max(3, warmup), world, dev) / steps
    G = plan_segments(max(hi - lo, 1), T, H, K, V, dev, backward=True)
    out = {"workload": f"C2 global batch B={B} T={T} H={H} sharded by (sequence, head) over {world} GPUs, no collective",
           "n_gpus": world, "units_per_gpu": (hi - lo) * H, "segments_per_sequence": G, "ms_per_step": ms,
           "tokens_per_s": B * T / (ms * 1e-3)}
    if single_ms:
        out["speedup_vs_single_gpu"] = single_ms / ms
        out["efficiency"] = single_ms / ms / world
    out["limited_by"] = ("with few (sequence, head) units per GPU the serial walk cannot fill 148 SMs; sequences are cut "
                         "into segments, which adds the summary / boundary-scan / carried-gradient kernels")
    del d
    torch.cuda.empty_cache()
    return out


def cp_parity(dev, rank, world):
    """Context-parallel forward + backward on a small case against the single-GPU op on the whole sequence:
    the largest max|x-ref|/max|ref| over outputs and gradients, over all ranks."""
    from palimpsa_b200.ops import chunk_palimpsa
    from palimpsa_b200.parallel import cp_chunk_palimpsa, shard_bounds

    def rel_err(x, ref):
        x, ref = x.detach().double(), ref.detach().double()
        return ((x - ref).abs().max() / ref.abs().max().clamp_min(1e-30)).item()

    B, T, H, K, V = 1, 1024 * world, 2, 128, 128
    host, d = make_inputs(B, T, H, K, V, torch.bfloat16, dev, seed=3)
    d["gt"] = d["gt"] * 0.05
    full = [d[n].detach().requires_grad_(True) for n in NAMES]
    o_ref = chunk_palimpsa(*full)
    o_ref.backward(d["do"])
    lo, hi = shard_bounds(T, rank, world)
    loc = [(d[n][:, lo:hi] if d[n].dim() >= 3 else d[n]).detach().contiguous().requires_grad_(True) for n in NAMES]
    o = cp_chunk_palimpsa(*loc, num_segments=2)
    o.backward(d["do"][:, lo:hi].contiguous())
    torch.cuda.synchronize(dev)
    errs = [rel_err(o, o_ref[:, lo:hi])]
    for x, y in zip(loc, full):
        errs.append(rel_err(x.grad, y.grad[:, lo:hi] if y.dim() >= 3 else y.grad))
    t = torch.tensor([max(errs)], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# ------------------------------------------------------------------------------------------------
# The run
# ------------------------------------------------------------------------------------------------
def run_ours(args, rank, world, local_rank):
    from palimpsa_b200 import _lib
    _lib.lib()  # fail loudly if the CUDA library is missing
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        bind_to_gpu_numa_node(local_rank)
    cfg = C2
    B, T, H, K, V = cfg["B"], cfg["T"], cfg["H"], cfg["K"], cfg["V"]
    extra = args.workload == "all"
    parity = cp_parity(dev, rank, world) if world > 1 else None
    host, d = make_inputs(B, T, H, K, V, torch.bfloat16, dev, seed=rank, pin=True)
    tokens = B * T
    in_bytes = sum(d[n].numel() * d[n].element_size() for n in ("q", "k", "v", "b", "do", "gt"))

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    ms = time_region(lambda: fwd_bwd(d), args.steps, args.warmup, world, dev)
    clocks = sampler.stop() if sampler else None
    value = world * tokens * args.steps / (ms * 1e-3)

    # end to end: pinned host -> device, fwd+bwd, every result back to pinned host
    names_in = NAMES + ("do",)
    out_host = {}

    from palimpsa_b200.host_pipeline import HostPipeline, ramped_widths
    pipe = HostPipeline(host, dev, slices=ramped_widths(B))

    def e2e_step():
        out_host.update(pipe.run(host))

    e2e_steps = max(3, min(args.steps, 10))
    ms_e2e = time_region(e2e_step, e2e_steps, 3, world, dev)
    e2e_val = world * tokens * e2e_steps / (ms_e2e * 1e-3)
    h2d = sum(host[n].numel() * host[n].element_size() for n in names_in)
    d2h = sum(x.numel() * x.element_size() for x in out_host.values())
    ms_copy = time_host_region(lambda: copies_only(pipe, host, dev), e2e_steps, 2, world, dev) / e2e_steps
    from palimpsa_b200.ops.palimpsa._core import plan_segments
    per_e2e_step = sum(8 if plan_segments(hi - lo, T, H, K, V, dev, backward=True) > 1 else 4 for lo, hi in pipe.bounds)
    slice_widths = [hi - lo for lo, hi in pipe.bounds]
    del pipe, out_host

    peaks = measured_peaks()
    roof = fp = None
    if rank == 0:
        roof = kernel_roofline(d, cfg, args.steps, peaks)
        fp = fp32_peaks(dev)
        if fp:
            roof["compute"].update({"fp32_fma_peak_tflops_measured": fp["fma_tflops"],
                                    "mufu_rcp_peak_tops_measured": fp["rcp_tops"],
                                    "frac_of_fp32_peak": roof["compute"]["algorithmic_tflops"] / fp["fma_tflops"]})
            fk = roof["other_kernels"]["fwd_kernel"]
            fk["frac_of_mufu_peak"] = fk["trcp_per_s"] / fp["rcp_tops"]
    del d, host
    torch.cuda.empty_cache()

    workloads = {}
    launches = 4 * args.steps + per_e2e_step * e2e_steps
    if extra:
        if world > 1:
            dist.barrier()
        # the headline runs the whole C2 batch on every GPU, so its step time IS the one-GPU time of this batch
        workloads["c2_strong"] = c2_strong_workload(dev, rank, world, max(3, min(args.steps, 10)), 3, ms / args.steps)
        workloads["c5"] = c5_workload(dev, rank, world, args.steps)
        if rank == 0 and world == 1:
            workloads["decode"] = decode_workload(dev, args.decode_steps)
            workloads["varlen"] = varlen_workload(dev, max(3, min(args.steps, 10)), 3)
            workloads["model_shapes"] = model_shapes_workload(dev, max(3, min(args.steps, 5)), True)
            launches += (workloads["decode"]["gpu_launches"] + workloads["varlen"]["gpu_launches"] +
                         workloads["model_shapes"]["gpu_launches"])
        elif rank == 0:
            workloads["decode"] = workloads["varlen"] = {"skipped": "measured at n_gpus = 1 (independent per "
                                                                    "sequence: ranks would run disjoint shards)"}
    if rank != 0:
        return
    gpu_line = cpu_line = None                        # CPU port and the reference's Triton ops: beside the one-GPU run
    if world == 1:
        if extra:
            dec_us = workloads["decode"]["us_per_step_eager"] if "decode" in workloads else None
            gpu_line = gpu_baseline(dev, ms / args.steps, dec_us, chunk_sizes=(16, 64) if args.baseline_chunk64 else (16,))
        cb_val, cb_sample, cb_times = cpu_baseline(20.0, cfg, steps=5, warmup=1)
        cpu_line = {"value": cb_val, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                    "sample": cb_sample, "spread_tokens_per_s": spread(cb_times, cb_val * min(cb_times))}
    line = {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "io_dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"C2 170M-shaped layer op: chunk fwd+bwd, bf16 io / fp32 state and arithmetic, "
                                   f"B={B}/GPU T={T} H={H} d_k={K} d_v={V}", "io_dtype": "bf16",
                       "global_batch": B * world, "sharding": "batch x head across GPUs, no collective",
                       "l2": f"inputs per step {in_bytes / 2 ** 20:.0f} MiB > L2 {L2_BYTES // 2 ** 20} MiB (no flush needed)"},
            "e2e": {"value": e2e_val, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": ms_e2e / e2e_steps, "api": "palimpsa_b200.host_pipeline.HostPipeline.run",
                    "slice_widths": slice_widths, "copy_only_ms": ms_copy,
                    "copy_only_gbs_per_rank_per_direction": h2d / (ms_copy * 1e-3) / 1e9,
                    "copy_only_frac_of_e2e": ms_copy / (ms_e2e / e2e_steps),
                    "resident_ms": ms / args.steps},
            "gpu_launches": launches, "clocks": clocks, "roofline": roof, "cpu_baseline": cpu_line,
            "gpu_baseline": gpu_line, "workloads": workloads}
    if parity is not None:
        line["cp_parity_max_rel_err"] = parity
    print(json.dumps(line), flush=True)


def run_layer(args):
    """Extra workload (not the headline): the layer's element-wise prologue and epilogue around the operator on
    the C2 shapes (B=8 T=4096 H=6 d_k=d_v=128, bf16), forward and backward, as four fused kernels.  Each is
    timed alone with CUDA events (inputs 200-600 MB per launch, above L2) and compared with the same lines
    written as the layer writes them, in eager PyTorch on the same GPU.  Prints its own JSON line."""
    import torch.nn.functional as F
    from palimpsa_b200 import _lib
    from palimpsa_b200.layers import layer_epilogue, layer_prologue
    _lib.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B, T, H, K, V = C2["B"], C2["T"], C2["H"], C2["K"], C2["V"]
    gen = torch.Generator(device="cpu").manual_seed(0)
    r = lambda *sh: torch.randn(*sh, generator=gen).to(dev, torch.bfloat16)
    q_raw, k_raw, x, b_raw, gate, o = r(B, T, H, K), r(B, T, H, K), r(B, T, H, V), r(B, T, H, V), r(B, T, H, V), r(B, T, H, V)
    dt_raw, bs_raw = r(B, T, H), r(B, T, H)
    dt_bias, b_scale = torch.randn(H, generator=gen).to(dev), torch.ones(H, device=dev)
    D, weight = torch.ones(H, device=dev), torch.ones(V, device=dev)
    cot = [r(B, T, H, K), r(B, T, H, K), r(B, T, H, V), r(B, T, H, V), torch.randn(B, T, H, generator=gen).to(dev)]
    dy = r(B, T, H, V)
    peaks = measured_peaks()

    def timed(fn, n):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    # the four fused passes, each timed alone through the C ABI (structs built once: no host work in the loop)
    from palimpsa_b200 import layers as LY
    lib = _lib.lib()
    sp = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    pa = LY._prologue_struct(q_raw, k_raw, x, b_raw, dt_raw, bs_raw, dt_bias, b_scale)
    pouts = [torch.empty_like(q_raw), torch.empty_like(k_raw), torch.empty_like(x), torch.empty_like(x),
             torch.empty(B, T, H, device=dev)]
    pa.q, pa.k, pa.v, pa.b, pa.gt = [t.data_ptr() for t in pouts]
    pa.dq, pa.dk, pa.dv, pa.db, pa.dgt = [t.data_ptr() for t in cot]
    pgr = [torch.empty_like(q_raw), torch.empty_like(k_raw), torch.empty_like(x), torch.empty_like(x),
           torch.empty_like(dt_raw), torch.empty_like(bs_raw), torch.empty(H, device=dev), torch.empty(H, device=dev)]
    pa.dq_raw, pa.dk_raw, pa.dx, pa.db_raw, pa.ddt_raw, pa.dbs_raw, pa.d_dt_bias, pa.d_b_scale = \
        [t.data_ptr() for t in pgr]
    ws = LY._workspace(B * T, H, V, dev)
    pa.workspace, pa.workspace_bytes = ws.data_ptr(), ws.numel()
    ea = LY._Epilogue._struct(o, x, D, weight, gate, 1e-5)
    eouts = [torch.empty_like(o) for _ in range(4)]
    egr = [torch.empty(H, device=dev), torch.empty(V, device=dev)]
    ea.y, ea.d_o, ea.dx, ea.dgate = [t.data_ptr() for t in eouts]
    ea.dy, ea.dD, ea.dweight = dy.data_ptr(), egr[0].data_ptr(), egr[1].data_ptr()
    ea.workspace, ea.workspace_bytes = ws.data_ptr(), ws.numel()
    n = max(5, args.steps)
    t_pf = timed(lambda: _lib.check(lib.palimpsa_layer_prologue_fwd(C.byref(pa), sp), "prologue"), n)
    t_pb = timed(lambda: _lib.check(lib.palimpsa_layer_prologue_bwd(C.byref(pa), sp), "prologue bwd"), n)
    t_ef = timed(lambda: _lib.check(lib.palimpsa_layer_epilogue_fwd(C.byref(ea), sp), "epilogue"), n)
    t_eb = timed(lambda: _lib.check(lib.palimpsa_layer_epilogue_bwd(C.byref(ea), sp), "epilogue bwd"), n)

    pin = [t.detach().requires_grad_(True) for t in (q_raw, k_raw, x, b_raw, dt_raw, bs_raw, dt_bias, b_scale)]
    ein = [t.detach().requires_grad_(True) for t in (o, x, D, weight, gate)]

    def ours_fb():                                    # the same work through the public, differentiable API
        for t in pin + ein:
            t.grad = None
        torch.autograd.backward(layer_prologue(*pin), cot)
        layer_epilogue(*ein).backward(dy)

    t_api = timed(ours_fb, n)

    def eager_fb():                                   # the layer's own lines (layers/palimpsa.py:269-281, 337-343)
        for t in pin + ein:
            t.grad = None
        qr, kr, xx, br, dtr, bsr, dtb, bsc = pin
        dt = F.softplus(dtr.float() + dtb)
        q, k = F.normalize(qr, p=2, dim=-1), F.normalize(kr, p=2, dim=-1)
        bs = torch.sigmoid(bsr.float()).to(xx.dtype)
        v = xx * bs.unsqueeze(-1)
        b = torch.sigmoid(br.float()) * F.softplus(bsc.view(1, 1, -1, 1).float())
        b = (b * bs.unsqueeze(-1)).to(xx.dtype)
        torch.autograd.backward([q, k, v, b, dt], cot)
        oo, x2, DD, ww, gg = ein
        z = (oo + x2 * DD[None, None, :, None]).float()
        y = z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + 1e-5) * ww
        y = (y * gg.float() * torch.sigmoid(gg.float())).to(oo.dtype)
        y.backward(dy)

    t_eager = timed(eager_fb, n)
    rows, es = B * T * H, 2
    alg = {"prologue_fwd": rows * ((4 * K + 4 * V) * es + 2 * es + 4),
           "prologue_bwd": rows * ((6 * K + 6 * V) * es + 4 * es + 4 + 8),
           "epilogue_fwd": rows * 4 * V * es,
           "epilogue_bwd": rows * (7 * V * es + 4)}
    ms = {"prologue_fwd": t_pf, "prologue_bwd": t_pb, "epilogue_fwd": t_ef, "epilogue_bwd": t_eb}
    kernels = {k2: {"ms": ms[k2], "algorithmic_bytes": alg[k2], "GB/s": alg[k2] / ms[k2] / 1e6,
                    "frac_of_hbm_peak": alg[k2] / ms[k2] / 1e6 / peaks["hbm_gbs"]} for k2 in ms}
    total = sum(ms.values())
    top = max(ms, key=ms.get)
    line = {"metric": "layer element-wise prologue+epilogue fwd+bwd tokens/s (bf16, T=4096)", "value": B * T / (total * 1e-3),
            "unit": "tokens/s", "n_gpus": 1, "steps": n, "warmup": 3, "ms_per_step": total, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "io_dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"layer element-wise sides on C2 shapes B={B} T={T} H={H} d_k={K} d_v={V} bf16",
                       "l2": "every launch moves 200-600 MB, above L2"},
            "gpu_launches": 4 * (n + 3) + 7 * (n + 3), "kernels": kernels, "public_api_fwd_bwd_ms": t_api,
            "torch_eager_fwd_bwd_ms": t_eager,
            "roofline": {"bound": "hbm", "kernel": top, "achieved": kernels[top]["GB/s"], "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": kernels[top]["frac_of_hbm_peak"], "peak_source": peaks["source"],
                         "traffic": None}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="all", choices=["all", "c2", "decode", "layer", "varlen"],
                    help="all (default): the headline line with every other configuration in its 'workloads' object; "
                         "c2: the headline alone; decode / varlen / layer: that workload's own JSON line")
    ap.add_argument("--decode-steps", type=int, default=1000)
    ap.add_argument("--baseline-chunk64", action="store_true",
                    help="gpu_baseline also times the reference's Triton chunk op at chunk_size=64")
    ap.add_argument("--profile-batch", type=int, default=4, help="batch size of --profile-case")
    ap.add_argument("--profile-segments", type=int, default=1,
                    help="with --profile-case: run one 32768-token sequence (H=12) cut into this many segments")
    ap.add_argument("--profile-heads", default=None, metavar="H,DK,DV",
                    help="with --profile-case: head count and dimensions instead of the benchmark's 6,128,128 "
                         "(e.g. 16,48,48: the reference's 170M configuration)")
    ap.add_argument("--profile-case", action="store_true",
                    help="run a few forward+backward steps of a half-size batch (B=4) and exit: the small case "
                         "that profiler captures are taken on")
    args = ap.parse_args()
    if args.profile_case:
        dev = torch.device("cuda", 0)
        if args.profile_segments > 1:
            # one long sequence cut into segments: exercises the summary (tensor-core) and scan kernels
            _, d = make_inputs(1, 32768, 12, C2["K"], C2["V"], torch.bfloat16, dev)
            for _ in range(3):
                fwd_bwd(d, num_segments=args.profile_segments)
            torch.cuda.synchronize()
            print("profile case (segments) done")
            return
        H, K, V = [int(x) for x in args.profile_heads.split(",")] if args.profile_heads else (C2["H"], C2["K"], C2["V"])
        _, d = make_inputs(args.profile_batch, C2["T"], H, K, V, torch.bfloat16, dev)
        for _ in range(3):
            fwd_bwd(d)
        torch.cuda.synchronize()
        print("profile case done")
        return
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.workload in ("layer", "varlen", "decode"):
        if rank == 0:
            dev = torch.device("cuda", 0)
            torch.cuda.set_device(dev)
            from palimpsa_b200 import _lib
            _lib.lib()
            if args.workload == "layer":
                run_layer(args)
            elif args.workload == "decode":
                w = decode_workload(dev, args.decode_steps)
                print(json.dumps({"metric": "decode tokens/s (fused-recurrent, bf16 io, fp32 state)",
                                  "value": w["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True,
                                  "dtype": "f32", "io_dtype": "bf16", "data": "synthetic",
                                  "config": {"workload": w["workload"]}, **w}), flush=True)
            else:
                w = varlen_workload(dev, args.steps, args.warmup)
                print(json.dumps({"metric": "fwd+bwd tokens/s (chunk, bf16, packed variable-length batch)",
                                  "value": w["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True,
                                  "dtype": "f32", "io_dtype": "bf16", "data": "synthetic",
                                  "config": {"workload": w["workload"], "l2": "inputs 241 MiB > L2"}, **w}), flush=True)
        return
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
