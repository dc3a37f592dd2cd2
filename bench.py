"""Benchmark of the gdn_chunk forward pass.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME] [--path P]

One "step" is one forward pass over one batch of synthetic input.  The default workload is the
one the headline metric is quoted on: B=1, S=8192, Hq=Hk=16, Hv=32, D=128, chunk 64, bf16, with a
random initial state.  With N > 1 (launched by torchrun, one rank per GPU) every rank runs that
workload on its own batch element: the (batch, value-head) sequences are independent, so the path
shards with no communication ("weak" scaling, global batch = N).  `--workload throughput` shards
B=64, S=4096 over the ranks instead.

Prints ONE JSON line (rank 0).  `value` is tokens/s with inputs resident in HBM, timed with CUDA
events around each step, an L2 flush between steps, max over ranks.  `e2e` is the same metric
through the public Python API with pinned HOST buffers: host->device copies of all inputs and
device->host copies of the output and final state inside the timed region.  `cpu_baseline` times
the CPU oracle (the C restatement of the reference's chunked torch function) on this box's host
cores, and the plain torch definition on the small CPU configuration beside it.

`--impl reference` runs the REFERENCE project's own CUDA kernels (its unmodified sources recompiled
for sm_100 by `python -m oracle.reference_cuda`, loaded from oracle/_ref/) through its own dispatch
entry on the same workload, timed the same way, one replica per rank.  When that extension has not
been built the arm falls back to the CPU port and says so in `reference_kind`.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "gdn_chunk_fwd_tokens_per_s"
UNIT = "tokens/s"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
# dram__bytes_read.sum + dram__bytes_write.sum per step of the dominant kernel, from the ncu captures summarised under
# profiles/ (workload, kernel) -> bytes; anything not listed is reported as null
DRAM_TRAFFIC = {
    ("default", "gdn_chain_t_kernel"): 358.0e6,      # 307.1 MB read + 50.9 MB written by the one split launch
    ("default", "gdn_chain_kernel"): 361.8e6,
    ("default", "gdn_coop_kernel"): 328.7e6,
}


_RESULT_STREAM = None


def keep_stdout_for_the_result():
    """The contract is ONE JSON line on stdout.  Libraries write there too (NCCL prints its version banner on stdout at
    some debug levels), so file descriptor 1 is pointed at stderr for the rest of the process and the result line goes
    out through a private copy of the original descriptor."""
    global _RESULT_STREAM
    if _RESULT_STREAM is None:
        sys.stdout.flush()
        _RESULT_STREAM = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit(line):
    out = _RESULT_STREAM or sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def queue_ahead(flush, n=4):
    """A few untimed L2 flushes right after the barrier, before the first timed step: the GPU has work while the host
    enqueues that step, so the CUDA events of the first step bracket device time like those of every later step
    (where the host runs a step ahead anyway) and not the host's launch latency on an idle GPU."""
    for _ in range(n):
        flush.zero_()


def flops_per_token(Hq, Hv, C=64, D=128):
    """Dense products at 64x64x128 tile granularity; Q K^T and K K^T once per qk head."""
    return Hq * 4 * C * D + Hv * (6 * C * D + 6 * D * D)


def bytes_per_token(Hq, Hv, gate_bytes=4):
    """Every input read once, the output written once (state I/O is added per sequence)."""
    return Hq * 512 + Hv * 512 + Hv * 2 * gate_bytes


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"]))}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU while the timed region runs (NVML reads in a thread,
    every ~2 ms; falls back to polling nvidia-smi when NVML is not importable).  Read-only: no setting is changed."""

    SMI_FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                  "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index, interval=0.002):
        self.index = index
        self.interval = interval
        self.sm, self.mx, self.reasons = [], [], set()
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self._max = float(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nvml = None

    def _sample_nvml(self):
        n = self._nvml
        self.sm.append(float(n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM)))
        self.mx.append(self._max)
        try:
            mask = n.nvmlDeviceGetCurrentClocksEventReasons(self._handle)
        except Exception:
            mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
        bits = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
        for name, bit in bits.items():
            if mask & bit:
                self.reasons.add(name)

    def _sample_smi(self):
        r = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.SMI_FIELDS}",
                            "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
        if r.returncode == 0 and r.stdout.strip():
            row = [c.strip() for c in r.stdout.strip().splitlines()[0].split(",")]
            self.sm.append(float(row[0]))
            self.mx.append(float(row[1]))
            for n, val in zip(self.NAMES, row[2:6]):
                if val.lower().startswith("active"):
                    self.reasons.add(n)

    def _run(self):
        while not self._stop.is_set():
            try:
                if self._nvml is not None:
                    self._sample_nvml()
                else:
                    self._sample_smi()
            except Exception:
                pass
            self._stop.wait(self.interval if self._nvml is not None else 0.1)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": max(self.mx) if self.mx else None,
                "reasons": sorted(self.reasons), "samples": len(self.sm),
                "source": "nvml" if self._nvml is not None else "nvidia-smi"}


def cpu_arm(workload, seed, min_seconds=10.0, max_reps=12):
    """Time the CPU oracle (chunked form, all host threads) on the whole workload, repeated."""
    from gdn_qsa_sm80_b200.synthetic import make_inputs
    from oracle import c_oracle
    from gdn_qsa_sm80_b200.synthetic import WORKLOADS
    w = WORKLOADS[workload]
    S = min(w.S, 16384)                       # bounded sample: at most 16384 tokens per run
    B = max(1, min(w.B, 16384 // S))
    whole = (S == w.S and B == w.B)
    q, k, v, g, beta, h0 = make_inputs(w, seed=seed, B=B, S=S)
    x = [t.float().numpy() for t in (q, k, v, g, beta)]
    h = None if h0 is None else h0.numpy()
    # every host core this process may run on, whatever OMP_NUM_THREADS says: torch.distributed.run sets it to 1 for
    # its children, which would time a one-thread run as the CPU arm at N > 1
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    c_oracle.chunk_f32(*x, initial_state=h, nthreads=threads)   # warm-up (page faults, thread pool)
    times = []
    t_start = time.perf_counter()
    while len(times) < max_reps and (time.perf_counter() - t_start < min_seconds or len(times) < 3):
        t0 = time.perf_counter()
        c_oracle.chunk_f32(*x, initial_state=h, nthreads=threads)
        times.append(time.perf_counter() - t0)
    tokens = q.shape[0] * q.shape[1]
    med = statistics.median(times)
    return {"value": tokens / med, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{'whole workload' if whole else f'B={B} S={S} slice of the workload'} ({tokens} tokens) x "
                      f"{len(times)} runs, median; C restatement of the "
                      f"reference's chunked torch function, fp32, OpenMP over (batch, head)",
            "ms_per_step": med * 1e3}


def torch_config0_arm():
    """The plain torch definition of the operator (fp32, chunk 64) on the small CPU configuration
    (B1 S512 Hq4 Hv8, zero initial state): 3 warm-ups, median of 10."""
    import torch
    from gdn_qsa_sm80_b200.synthetic import make_inputs
    from gdn_qsa_sm80_b200.torch_definition import chunk_gated_delta_rule
    q, k, v, g, beta, _ = make_inputs("cpu_small", seed=0)
    q, k = q.repeat_interleave(2, dim=2), k.repeat_interleave(2, dim=2)
    times = []
    for i in range(13):
        t0 = time.perf_counter()
        chunk_gated_delta_rule(q, k, v, g, beta, chunk_size=64)
        if i >= 3:
            times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return {"value": q.shape[0] * q.shape[1] / med, "unit": UNIT, "ms": med * 1e3, "threads": torch.get_num_threads(),
            "cores": os.cpu_count(), "sample": "torch fp32 chunked definition, B1 S512 Hq4 Hv8 chunk 64, median of 10"}


def reference_arm(args, w, cfg, rank, world, local_rank):
    """`--impl reference`: the reference project's own kernels on this GPU when its extension was built, else the
    CPU port.  Same workload, same timing rules, same JSON keys as the main arm."""
    import torch
    mod = None
    why = None
    if torch.cuda.is_available():
        try:
            from oracle import reference_cuda
            mod = reference_cuda.load()
            if mod is None:
                why = "oracle/_ref/_gdn_chunk.so has not been built"
        except Exception as e:      # the built file does not match this torch / driver
            why = f"loading the reference's extension failed: {type(e).__name__}: {e}"
    else:
        why = "no CUDA device"
    if mod is None:
        # CPU arm: the C restatement of the reference's torch function (pinned against it by golden vectors)
        if rank != 0:
            return
        base = cpu_arm(args.workload, args.seed, min_seconds=max(5.0, 0.5 * args.steps))
        cfg = dict(cfg, sharding=f"{world} independent batch elements, one per GPU, no communication")
        emit({"impl": "reference", "reference_kind": f"cpu port ({why})", "metric": METRIC,
                          "value": base["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
                          "warmup": args.warmup, "ms_per_step": base["ms_per_step"], "higher_is_better": True,
                          "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg,
                          "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
                          "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                          "gpu_launches": 0})
        return

    import torch.distributed as dist
    from gdn_qsa_sm80_b200.synthetic import make_inputs
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=dev)
    # the same share of the workload as the main arm; the reference's entry takes bf16 gates and has no initial state
    if args.workload == "default" or w.B < world:
        B_local, total_tokens, scaling = w.B, w.B * w.S * world, "weak"
        cfg["sharding"] = f"{world} independent batch elements, one per GPU, no communication"
    else:
        B_local, total_tokens, scaling = w.B // world, w.B * w.S, "strong"
        cfg["sharding"] = f"batch split {world} ways ({B_local} per GPU), no communication"
    q, k, v, g, beta, _ = make_inputs(w, seed=args.seed + rank, B=B_local)
    host = [t.pin_memory() for t in (q, k, v, g.bfloat16(), beta.bfloat16())]
    d_in = [t.to(dev, non_blocking=True) for t in host]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step(x=d_in):
        r = mod.forward_gdn_chunk_auto(x[0], x[1], x[2], x[3], x[4], True)
        return r[0], r[1]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(args.warmup):
        step()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    queue_ahead(flush)
    with ClockSampler(local_rank) as clocks:
        for a, b in ev:
            flush.zero_()
            a.record()
            step()
            b.record()
        barrier()
    ms_per_step = max_over_ranks(sum(a.elapsed_time(b) for a, b in ev)) / args.steps
    # end to end: pinned host buffers in, results back to pinned host buffers, every step
    out_host = torch.empty((B_local, w.S, w.Hv, 128), dtype=torch.bfloat16).pin_memory()
    st_host = torch.empty((B_local, w.Hv, 128, 128), dtype=torch.bfloat16).pin_memory()
    n_e2e = max(4, min(args.steps, 10))

    def e2e_step():
        o, s = step([t.to(dev, non_blocking=True) for t in host])
        out_host.copy_(o, non_blocking=True)
        st_host.copy_(s, non_blocking=True)

    for _ in range(2):
        e2e_step()
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(n_e2e):
        e2e_step()
    b.record()
    barrier()
    e2e_ms = max_over_ranks(a.elapsed_time(b)) / n_e2e
    if rank == 0:
        peaks, peak_kind = load_peaks()
        fl = flops_per_token(w.Hq, w.Hv) * B_local * w.S
        tf = fl / (ms_per_step * 1e-3) / 1e12
        line = {"impl": "reference",
                "reference_kind": "the reference's own CUDA kernels (csrc/gdn_chunk, unmodified, recompiled with "
                                  "-gencode arch=compute_100,code=sm_100) through forward_gdn_chunk_auto; bf16 gates; "
                                  "zero initial state and bf16 final state (its entry has no others)",
                "metric": METRIC, "value": total_tokens / (ms_per_step * 1e-3), "unit": UNIT, "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": scaling, "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": cfg,
                "clocks": clocks.summary(),
                "e2e": {"value": total_tokens / (e2e_ms * 1e-3), "unit": UNIT,
                        "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in host),
                        "d2h_bytes_per_step": out_host.numel() * 2 + st_host.numel() * 2, "steps": n_e2e,
                        "api": "unpipelined (.to(device) / reference gdn_chunk / .copy_)"},
                "roofline": {"kernel": "whole step (reference kernels)", "bound": "tensor", "achieved": tf,
                             "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": tf / peaks["bf16_tflops"],
                             "traffic": None, "peak_kind": f"{peak_kind} (burst cuBLAS bf16)"}}
        if world == 1 and not args.no_cpu_baseline:
            base = cpu_arm(args.workload, args.seed, min_seconds=max(5.0, 0.5 * args.steps))
            line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        emit(line)
    if world > 1:
        dist.destroy_process_group()


def device_inputs(w, seed, dev, B=None, S=None):
    """A workload's distributions drawn on the GPU generator (the CPU generator takes minutes at the large sizes)."""
    import torch
    F = torch.nn.functional
    B = w.B if B is None else B
    S = w.S if S is None else S
    gen = torch.Generator(device=dev).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=gen, device=dev)
    q = F.normalize(rn(B, S, w.Hq, 128), dim=-1).bfloat16()
    k = F.normalize(rn(B, S, w.Hq, 128), dim=-1).bfloat16()
    v = rn(B, S, w.Hv, 128).bfloat16()
    g = -F.softplus(rn(B, S, w.Hv)) * w.gate_scale
    beta = torch.sigmoid(rn(B, S, w.Hv))
    h0 = 0.1 * rn(B, w.Hv, 128, 128) if w.h0 != "zeros" else None
    return q, k, v, g, beta, h0


def timed_steps(step, steps, warmup, flush, dev, world, barrier_each=False):
    """ms per step: CUDA events around every step on the current stream, an L2 flush before each, max over ranks."""
    import torch
    import torch.distributed as dist
    for _ in range(warmup):
        flush.zero_()
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    total = 0.0
    for _ in range(steps):
        flush.zero_()
        if barrier_each and world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total += float(t.item())
    return total / steps


def sharded_arm(rank, world, dev, flush, seed, steps=5, warmup=3):
    """The throughput workload (B=64 S=4096) split over the ranks by batch, no communication: strong scaling."""
    import torch
    from gdn_qsa_sm80 import gdn_chunk
    from gdn_qsa_sm80_b200.synthetic import WORKLOADS
    w = WORKLOADS["throughput"]
    if w.B % world:
        return None
    Bl = w.B // world
    q, k, v, g, beta, h0 = device_inputs(w, seed + 100 + rank, dev, B=Bl)
    ms = timed_steps(lambda: gdn_chunk(q, k, v, g, beta, output_final_state=True, initial_state=h0), steps, warmup,
                     flush, dev, world)
    del q, k, v, g, beta, h0
    torch.cuda.empty_cache()
    tokens = w.B * w.S
    return {"workload": f"throughput: B={w.B} S={w.S} Hq={w.Hq} Hv={w.Hv} h0={w.h0}, batch split {world} ways "
                        f"({Bl} per GPU), no communication", "scaling": "strong", "value": tokens / (ms * 1e-3),
            "unit": UNIT, "ms_per_step": ms, "steps": steps, "warmup": warmup,
            "frac_of_bf16_peak": tokens * flops_per_token(w.Hq, w.Hv) / (ms * 1e-3) / 1e12 / (load_peaks()[0]["bf16_tflops"] * world)}


def seq_parallel_measure(rank, world, dev, flush, seed, steps=5, warmup=3):
    """The long_context workload (one sequence of 131072 tokens) cut into `world` contiguous segments, boundary
    states exchanged by NCCL send/recv (scan mode with the exact early-out)."""
    import torch
    from gdn_qsa_sm80_b200.distributed import segment_bounds, sequence_parallel_forward
    from gdn_qsa_sm80_b200.synthetic import WORKLOADS
    w = WORKLOADS["long_context"]
    lo, hi = segment_bounds(w.S, world)[rank]
    q, k, v, g, beta, _ = device_inputs(w, seed + 200 + rank, dev, S=hi - lo)
    ms = timed_steps(lambda: sequence_parallel_forward(q, k, v, g, beta, initial_state=None, mode="scan"), steps,
                     warmup, flush, dev, world, barrier_each=True)
    del q, k, v, g, beta
    torch.cuda.empty_cache()
    tokens = w.B * w.S
    return {"workload": f"long_context: B=1 S={w.S} Hq={w.Hq} Hv={w.Hv}, one sequence in {world} contiguous segments, "
                        f"boundary states [Hv,128,128] fp32 by NCCL send/recv, scan mode", "scaling": "strong",
            "value": tokens / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms, "steps": steps, "warmup": warmup}


def link_ceiling(host_in, host_out, dev, world, reps=4):
    """Plain cudaMemcpyAsync of one step's bytes, host->device and device->host at the same time on two streams, on
    every rank at once: what the host link gives with no kernel in the way.  Returns GB/s per direction (this rank,
    min over ranks reported by the caller) and the step time."""
    import torch
    import torch.distributed as dist
    d_in = [torch.empty_like(t, device=dev) for t in host_in]
    d_out = [torch.empty_like(t, device=dev) for t in host_out]
    s1, s2 = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def once():
        with torch.cuda.stream(s1):
            for h, d in zip(host_in, d_in):
                d.copy_(h, non_blocking=True)
        with torch.cuda.stream(s2):
            for h, d in zip(host_out, d_out):
                h.copy_(d, non_blocking=True)

    once()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(reps):
        once()
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / reps
    t = torch.tensor([dt], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def bind_near_gpu(index):
    """Run this process's threads on the CPUs NVML lists as local to the GPU (read-only query; changes only this
    process's own affinity).  Returns a short description for the JSON line."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        n = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, n)
        cpus = {64 * i + b for i, word in enumerate(mask) for b in range(64) if (word >> b) & 1}
        allowed = os.sched_getaffinity(0)
        use = cpus & allowed
        if use and use != allowed:
            os.sched_setaffinity(0, use)
            return f"threads bound to the {len(use)} CPUs local to GPU {index}"
        return f"GPU {index}: every allowed CPU ({len(allowed)}) is local (one NUMA node visible)"
    except Exception as e:       # no NVML / no permission: leave the affinity alone
        return f"affinity unchanged ({type(e).__name__})"


def seq_parallel_arm(args, w, cfg, rank, world, dev):
    """One sequence cut into `world` contiguous segments (multiples of 64 tokens), one per GPU; rank r's segment is
    generated from seed + r (the sequence is the concatenation).  A step = the whole sequence-parallel forward."""
    import torch
    import torch.distributed as dist
    from gdn_qsa_sm80_b200 import _lib
    from gdn_qsa_sm80_b200.distributed import segment_bounds, sequence_parallel_forward
    from gdn_qsa_sm80_b200.synthetic import make_inputs

    lo, hi = segment_bounds(w.S, world)[rank]
    q, k, v, g, beta, h0 = make_inputs(w, seed=args.seed + rank, S=hi - lo)
    d = [t.to(dev) for t in (q, k, v, g, beta)]
    h0 = None if (h0 is None or rank != 0) else h0.to(dev)
    mode = "scan" if args.seq_parallel.startswith("scan") else "pipeline"
    early = args.seq_parallel != "scan_no_early_out"

    def step():
        return sequence_parallel_forward(*d, initial_state=h0, mode=mode, decay_early_out=early)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(args.warmup):     # warm-up steps run exactly like timed ones (flush, barrier, step)
        flush.zero_()
        barrier()
        step()
    launches0 = _lib.kernel_launches()
    barrier()
    total_ms, per_step = 0.0, []
    # a step here is dozens of small launches from Python: sample the clocks sparsely so that the NVML reads do not
    # compete with them for the driver
    with ClockSampler(dev.index, interval=0.01) as clocks:
        for _ in range(args.steps):
            flush.zero_()
            barrier()                                     # every step starts on all ranks together
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            step()
            b.record()
            torch.cuda.synchronize()
            t = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            total_ms += float(t.item())
            per_step.append(round(float(t.item()), 4))
    launches = _lib.kernel_launches() - launches0
    ms = total_ms / args.steps
    tokens = w.B * w.S
    flops = tokens * (w.Hq * 32768 + w.Hv * 147456)
    if rank == 0:
        cfg = dict(cfg, sharding=f"one sequence in {world} contiguous segments, boundary states by send/recv, mode "
                                 f"{args.seq_parallel}")
        emit({
            "metric": METRIC, "value": tokens / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": cfg, "clocks": clocks.summary(),
            "e2e": None, "gpu_launches": int(launches), "step_ms": per_step,
            "roofline": {"bound": "tensor", "achieved": flops / (ms * 1e-3) / 1e12, "peak": load_peaks()[0]["bf16_tflops"] * world,
                         "unit": "TFLOP/s", "frac": flops / (ms * 1e-3) / 1e12 / (load_peaks()[0]["bf16_tflops"] * world),
                         "traffic": None, "note": "whole job over all GPUs; algorithmic flops, redundant passes not counted"}})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="default", choices=["default", "short_batch", "throughput", "long_context"])
    ap.add_argument("--path", default="auto", choices=["auto", "simt", "twopass_nv64", "twopass_nv32", "twopass_t", "coop", "decode"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-multi", action="store_true",
                    help="skip the extra keys \"sharded\" (throughput workload split over the GPUs) and \"seq_parallel\"")
    ap.add_argument("--seq-parallel", default=None, choices=["pipeline", "scan", "scan_no_early_out"],
                    help="with --gpus N > 1: split ONE sequence of the workload into N contiguous segments, one per "
                         "GPU, boundary states exchanged by send/recv (strong scaling)")
    ap.add_argument("--output-gate", action="store_true",
                    help="also time the step with the gated RMS normalisation chained behind it (extra key \"with_output_gate\")")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    keep_stdout_for_the_result()

    from gdn_qsa_sm80_b200.synthetic import WORKLOADS
    w = WORKLOADS[args.workload]
    cfg = {"workload": f"{w.name}: B={w.B} S={w.S} Hq={w.Hq} Hv={w.Hv} D=128 chunk=64 bf16 h0={w.h0}",
           "l2": "flushed between timed steps (256 MiB write)", "path": args.path}

    if args.impl == "reference":
        reference_arm(args, w, cfg, rank, world, local_rank)
        return

    import torch
    import torch.distributed as dist
    from gdn_qsa_sm80 import gdn_chunk
    from gdn_qsa_sm80_b200 import _lib
    from gdn_qsa_sm80_b200.gdn_chunk_interface import check_device_status
    from gdn_qsa_sm80_b200.synthetic import make_inputs

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (sm_100a); there is no CPU path for the operator")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    affinity = bind_near_gpu(local_rank)                 # before the pinned host buffers are allocated
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")   # whatever NCCL logs: not on stdout (one JSON line only)
        dist.init_process_group("nccl", device_id=dev)

    if args.seq_parallel:
        seq_parallel_arm(args, w, cfg, rank, world, dev)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- this rank's share of the workload ------------------------------------------------------------
    if args.workload == "default" or w.B < world:
        B_local, total_tokens, scaling = w.B, w.B * w.S * world, "weak"       # one whole workload per rank
        cfg["sharding"] = f"{world} independent batch elements, one per GPU, no communication"
    else:
        assert w.B % world == 0, "batch must divide over the ranks"
        B_local, total_tokens, scaling = w.B // world, w.B * w.S, "strong"
        cfg["sharding"] = f"batch split {world} ways ({B_local} per GPU), no communication"
    q, k, v, g, beta, h0 = make_inputs(w, seed=args.seed + rank, B=B_local)
    host = [t.pin_memory() for t in (q, k, v, g, beta)] + [None if h0 is None else h0.pin_memory()]
    d_in = [None if t is None else t.to(dev, non_blocking=True) for t in host]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    torch.cuda.synchronize()

    def step():
        return gdn_chunk(d_in[0], d_in[1], d_in[2], d_in[3], d_in[4], output_final_state=True,
                         initial_state=d_in[5], path=args.path)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    check_device_status(dev)

    # ---- device-resident timing ---------------------------------------------------------------------------
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    launches0 = _lib.kernel_launches()
    barrier()
    queue_ahead(flush)
    with ClockSampler(local_rank) as clocks:
        for a, b in ev:
            flush.zero_()
            a.record()
            step()
            b.record()
        barrier()
    launches = _lib.kernel_launches() - launches0
    check_device_status(dev)
    step_ms = [a.elapsed_time(b) for a, b in ev]
    total_ms = sum(step_ms)
    if world > 1:
        t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    value = total_tokens / (ms_per_step * 1e-3)

    # ---- end to end through the public API with host buffers ------------------------------------------------
    e2e = None
    if not args.no_e2e:
        out_host = torch.empty((B_local, w.S, w.Hv, 128), dtype=torch.bfloat16).pin_memory()
        st_host = torch.empty((B_local, w.Hv, 128, 128), dtype=torch.float32).pin_memory()
        h2d = sum(t.numel() * t.element_size() for t in host if t is not None)
        d2h = out_host.numel() * 2 + st_host.numel() * 4

        from gdn_qsa_sm80_b200 import gdn_chunk_host
        outs = [out_host, torch.empty_like(out_host).pin_memory()]
        sts = [st_host, torch.empty_like(st_host).pin_memory()]
        side = [torch.cuda.Stream(dev), torch.cuda.Stream(dev)]
        main = torch.cuda.current_stream(dev)

        def e2e_plain(i):
            # copy everything in, run, copy everything out: one direction of the host link at a time
            dd = [None if t is None else t.to(dev, non_blocking=True) for t in host]
            o, s = gdn_chunk(dd[0], dd[1], dd[2], dd[3], dd[4], output_final_state=True, initial_state=dd[5],
                             path=args.path)
            out_host.copy_(o, non_blocking=True)
            st_host.copy_(s, non_blocking=True)

        def e2e_piped(i):
            # the host-buffer entry point: segments of the sequence in flight in both directions at once
            gdn_chunk_host(host[0], host[1], host[2], host[3], host[4], initial_state=host[5], out=out_host,
                           final_state_out=st_host, synchronize=False)

        def e2e_piped2(i):
            # the same with two calls in flight (a stream, a device arena and result buffers each), as a host
            # that feeds one batch after another would run it
            with torch.cuda.stream(side[i % 2]):
                gdn_chunk_host(host[0], host[1], host[2], host[3], host[4], initial_state=host[5], out=outs[i % 2],
                               final_state_out=sts[i % 2], synchronize=False, arena_slot=1 + i % 2)

        def e2e_piped2_whole(i):
            # two calls in flight, each as ONE segment: the other call's copies fill this call's gaps, and fewer,
            # larger copies use the link better than a call's own segments do
            with torch.cuda.stream(side[i % 2]):
                gdn_chunk_host(host[0], host[1], host[2], host[3], host[4], initial_state=host[5], out=outs[i % 2],
                               final_state_out=sts[i % 2], synchronize=False, arena_slot=1 + i % 2, seg_tokens=w.S)

        n_e2e = max(4, min(args.steps, 10))

        def time_e2e(fn):
            for i in range(2):
                fn(i)
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for s in side:
                s.wait_stream(main)
            a.record()
            for i in range(n_e2e):
                fn(i)
            for s in side:
                main.wait_stream(s)
            b.record()
            barrier()
            ms = a.elapsed_time(b)
            if world > 1:
                t = torch.tensor([ms], dtype=torch.float64, device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            return total_tokens / (ms / n_e2e * 1e-3)

        modes = {"unpipelined (.to(device) / gdn_chunk / .copy_)": time_e2e(e2e_plain)}
        if args.path == "auto":
            modes["gdn_chunk_host, one call at a time"] = time_e2e(e2e_piped)
            modes["gdn_chunk_host, two calls in flight"] = time_e2e(e2e_piped2)
            modes["gdn_chunk_host, two calls in flight, one segment each"] = time_e2e(e2e_piped2_whole)
        best = max(modes, key=modes.get)
        step_s = total_tokens / modes[best] / world          # seconds per step and rank at the best mode
        ceil_s = link_ceiling([t for t in host if t is not None], [out_host, st_host], dev, world)
        e2e = {"value": modes[best], "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "steps": n_e2e, "api": best, "all": modes,
               "achieved_h2d_gbs_per_gpu": h2d / step_s / 1e9, "achieved_d2h_gbs_per_gpu": d2h / step_s / 1e9,
               "link_ceiling": {"what": "the same bytes by plain cudaMemcpyAsync, both directions at once, all ranks at once, "
                                        "no kernel (slowest rank)", "ms_per_step": ceil_s * 1e3,
                                "value": total_tokens / ceil_s, "unit": UNIT,
                                "h2d_gbs_per_gpu": h2d / ceil_s / 1e9, "d2h_gbs_per_gpu": d2h / ceil_s / 1e9},
               "host_affinity": affinity}

    # ---- optional: the layer's next step (gated RMS normalisation of O) chained behind the forward pass ----
    with_gate = None
    if args.output_gate:
        from gdn_qsa_sm80_b200 import rmsnorm_gated
        gen = torch.Generator().manual_seed(args.seed + 1000 + rank)
        zg = (1.5 * torch.randn(B_local, w.S, w.Hv, 128, generator=gen)).bfloat16().to(dev)
        wg = torch.ones(128, dtype=torch.bfloat16, device=dev)

        def timed(fn):
            for _ in range(3):
                fn()
            ts = []
            for _ in range(args.steps):
                flush.zero_()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                torch.cuda.synchronize()
                ts.append(a.elapsed_time(b))
            return sorted(ts)[len(ts) // 2]

        o_dev, _ = step()
        fused_ms = timed(lambda: gdn_chunk(d_in[0], d_in[1], d_in[2], d_in[3], d_in[4], output_final_state=True,
                                           initial_state=d_in[5], path=args.path, output_gate=(zg, wg)))
        alone_cold_ms = timed(lambda: rmsnorm_gated(o_dev, zg, wg, out=o_dev))
        with_gate = {"step_ms_median": fused_ms, "gate_alone_after_l2_flush_ms": alone_cold_ms,
                     "gate_bytes": 3 * o_dev.numel() * 2}

    # ---- the two kernels of a step timed on their own (CUDA events on the launching stream, L2 flushed) ----
    per_kernel = None
    n_sm = torch.cuda.get_device_properties(dev).multi_processor_count
    single_launch = args.path == "coop" or (args.path == "auto" and w.S <= 2048 and 4 * B_local * w.Hv <= n_sm)
    transposed = args.path == "twopass_t" or (args.path == "auto" and not single_launch)
    kernels = ("gdn_coop_kernel (one launch)" if single_launch else
               "gdn_prepare_pair_kernel + gdn_chain_t_kernel (few long sequences are split into warmed-up segments on the device)"
               if transposed else
               "gdn_prepare_kernel + gdn_chain_kernel" if args.path in ("twopass_nv32", "twopass_nv64") else args.path)
    if transposed or args.path in ("twopass_nv32", "twopass_nv64"):
        per_kernel = {}
        step()                                            # leaves a valid workspace for the chain-only launches
        for key, name in (("prepare_only", "prepare_only_t" if transposed else "prepare_only"),
                          ("chain_only", "chain_only_t" if transposed else "chain_only")):
            times = []
            for _ in range(max(3, min(args.steps, 10))):
                flush.zero_()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                gdn_chunk(d_in[0], d_in[1], d_in[2], d_in[3], d_in[4], output_final_state=True,
                          initial_state=d_in[5], path=name)
                b.record()
                torch.cuda.synchronize()
                times.append(a.elapsed_time(b))
            per_kernel[key] = statistics.median(times)
        check_device_status(dev)

    # ---- the two multi-GPU cases of the specification, on the plain line (default workload only) ----------
    sharded = seq_par = None
    if args.workload == "default" and args.path == "auto" and not args.no_multi:
        del d_in
        torch.cuda.empty_cache()
        sharded = sharded_arm(rank, world, dev, flush, args.seed)
        if world > 1:
            seq_par = seq_parallel_measure(rank, world, dev, flush, args.seed)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline: the whole step, and the dominant kernel (the chain) on its own -------------------------
    peaks, peak_kind = load_peaks()
    tokens_local = B_local * w.S
    step_s = statistics.median(step_ms) * 1e-3
    fl = flops_per_token(w.Hq, w.Hv) * tokens_local
    by = bytes_per_token(w.Hq, w.Hv) * tokens_local + B_local * w.Hv * 65536 * (2 if w.h0 != "zeros" else 1)
    whole = {"achieved": fl / step_s / 1e12, "frac": fl / step_s / 1e12 / peaks["bf16_tflops"],
             "algorithmic_flops_per_step": fl, "step_ms_median": step_s * 1e3,
             "hbm": {"achieved": by / step_s / 1e9, "frac": by / step_s / 1e9 / peaks["hbm_gbs"],
                     "algorithmic_bytes_per_step": by, "peak": peaks["hbm_gbs"], "unit": "GB/s"}}
    if per_kernel:
        # flops of the chain kernel: W S, Q S, K^T v~ (2 D D each) and P v_new (2 C D) per value head and token - the
        # transposed chain also forms U = T'' V (2 C D); the prepare kernel has the rest (K K^T, Q K^T per qk head;
        # T K, and T V where the chain does not do it, per value head)
        fl_chain = w.Hv * (6 * 128 * 128 + (4 if transposed else 2) * 64 * 128) * tokens_local
        fl_prep = fl - fl_chain
        k_s = per_kernel["chain_only"] * 1e-3
        tf = fl_chain / k_s / 1e12
        # DRAM bytes of one chain launch on the default workload, from an ncu capture (profiles/): read + write
        traffic = DRAM_TRAFFIC.get((args.workload, "gdn_chain_t_kernel" if transposed else "gdn_chain_kernel")) if world == 1 else None
        roofline = {"kernel": "gdn_chain_t_kernel" if transposed else "gdn_chain_kernel", "bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"],
                    "unit": "TFLOP/s", "frac": tf / peaks["bf16_tflops"], "traffic": traffic,
                    "peak_kind": f"{peak_kind} (burst cuBLAS bf16)", "algorithmic_flops_per_launch": fl_chain,
                    "kernel_ms": per_kernel["chain_only"],
                    "share_of_step": per_kernel["chain_only"] / (per_kernel["chain_only"] + per_kernel["prepare_only"]),
                    "prepare_kernel": {"kernel_ms": per_kernel["prepare_only"], "algorithmic_flops_per_launch": fl_prep,
                                       "achieved": fl_prep / (per_kernel["prepare_only"] * 1e-3) / 1e12,
                                       "frac": fl_prep / (per_kernel["prepare_only"] * 1e-3) / 1e12 / peaks["bf16_tflops"]},
                    "whole_step": whole}
        if traffic:   # the same launch against the HBM roofline, at the DRAM bytes it really moves
            roofline["traffic_hbm"] = {"achieved": traffic / k_s / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                       "frac": traffic / k_s / 1e9 / peaks["hbm_gbs"]}
    elif single_launch:
        # one kernel per step: its duration is the step's (CUDA events around the launch)
        traffic = DRAM_TRAFFIC.get((args.workload, "gdn_coop_kernel")) if world == 1 else None
        roofline = {"kernel": "gdn_coop_kernel", "bound": "tensor", "achieved": whole["achieved"], "peak": peaks["bf16_tflops"],
                    "unit": "TFLOP/s", "frac": whole["frac"], "traffic": traffic,
                    "peak_kind": f"{peak_kind} (burst cuBLAS bf16)", "algorithmic_flops_per_launch": fl,
                    "kernel_ms": step_s * 1e3, "share_of_step": 1.0, "whole_step": whole}
    else:
        roofline = {"kernel": "whole step", "bound": "tensor", "achieved": whole["achieved"], "peak": peaks["bf16_tflops"],
                    "unit": "TFLOP/s", "frac": whole["frac"], "traffic": None,
                    "peak_kind": f"{peak_kind} (burst cuBLAS bf16)", "algorithmic_flops_per_launch": fl,
                    "whole_step": whole}
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": cfg, "clocks": clocks.summary(),
            "e2e": e2e, "gpu_launches": int(launches), "kernels": kernels, "roofline": roofline}
    if sharded is not None:
        line["sharded"] = sharded
    if seq_par is not None:
        line["seq_parallel"] = seq_par
    if with_gate is not None:
        line["with_output_gate"] = with_gate
    if world == 1 and not args.no_cpu_baseline:
        base = cpu_arm(args.workload, args.seed)
        line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        line["cpu_baseline"]["torch_config0"] = torch_config0_arm()
    emit(line)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
