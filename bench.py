#!/usr/bin/env python
"""Benchmark driver for the flash-attention forward path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c3|c4]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" is one forward pass over one batch of synthetic input.  The default
workload is configuration 2 of the baseline: bf16 Q/K/V [B=8,H=16,N=2048,d=128],
N(0,1) from a seed, scale 1/sqrt(128), causal, dropout p=0.1 with Philox seed 42,
offset 0.  With N GPUs every rank runs that workload on its own 128 (batch, head)
units (weak scaling, no data-path collective); the dropout streams use the global
unit index so the job is the same as one [8N,16,2048,128] problem.

Rank 0 prints ONE JSON line.  `value` is device-timed throughput with inputs
resident in HBM; `e2e` is the same metric through the host-buffer entry point
(fa_fwd_host) with the H2D/D2H copies inside the timed region; `roofline` relates
the kernel to the measured bf16 peak; `cpu_baseline` is the reference's own CPU
attention timed on this box's cores on a bounded sample.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: B, H, Nq, Nk, d, causal, window, alibi, p_dropout, splits, description
    "c2": dict(B=8, H=16, Nq=2048, Nk=2048, d=128, causal=True, window=(-1, -1), alibi=False, p=0.1, splits=1,
               desc="config 2: bf16 [8,16,2048,128] causal, dropout 0.1 (Philox seed 42, offset 0)"),
    "c3": dict(B=4, H=32, Nq=8192, Nk=8192, d=128, causal=True, window=(1024, 0), alibi=True, p=0.0, splits=1,
               desc="config 3: bf16 [4,32,8192,128] causal + window(1024,0) + ALiBi 2^(-8(h+1)/32)"),
    "c5": dict(B=1, H=32, Nq=131072, Nk=131072, d=128, causal=True, window=(-1, -1), alibi=False, p=0.0, splits=1,
               desc="config 5: bf16 [1,32,131072,128] causal, N(0,0.5), sequence ring over the ranks (zig-zag chunks, "
                    "NCCL send/recv, LSE merge)"),
    "c4": dict(B=64, H=32, Nq=1, Nk=32768, d=128, causal=False, window=(-1, -1), alibi=False, p=0.0, splits=16,
               desc="config 4: split-KV decode bf16 B=64 H=32 q=1 kv=32768 d=128, 16 splits + LSE combine"),
    # config 4 with grouped-query attention (not a baseline config: the reference has one head count)
    "c4gqa": dict(B=64, H=32, Hk=8, Nq=1, Nk=32768, d=128, causal=False, window=(-1, -1), alibi=False, p=0.0,
                  splits=16, desc="config 4 with 8 K/V heads for the 32 query heads (grouped-query decode): bf16 B=64 "
                                  "q=1 kv=32768 d=128, 16 splits + LSE combine"),
}


def attended_pairs(w):
    """Unmasked (query, key) pairs per (batch, head) unit."""
    Nq, Nk = w["Nq"], w["Nk"]
    wl, wr = w["window"]
    total = 0
    for i in range(Nq):
        lo, hi = 0, Nk - 1
        if w["causal"]:
            hi = min(hi, i)
        if wr >= 0:
            hi = min(hi, i + wr)
        if wl >= 0:
            lo = max(lo, i - wl)
        total += max(0, hi - lo + 1)
    return total


def work_per_step(name, w):
    """(flops, bytes) of one step on one GPU: 4*d FLOP per attended (query, key) pair (causal configs by the
    4*B*H*N^2*d/2 convention), bytes = K + V + Q + O in 16-bit."""
    units = w["B"] * w["H"]
    if name in ("c2", "c5"):
        flops = 4.0 * units * w["Nq"] * w["Nk"] * w["d"] / 2  # causal convention 4*B*H*N^2*d/2
    else:
        flops = 4.0 * units * attended_pairs(w) * w["d"]
    kv_units = w["B"] * w.get("Hk", w["H"])
    nbytes = 2.0 * w["d"] * (2 * kv_units * w["Nk"] + 2 * units * w["Nq"])  # K + V + Q + O, 16-bit
    return flops, nbytes


def pin_to_gpu_node(torch, dev):
    """Keeps this rank's threads, and with them the pages of the pinned host buffers it allocates, on the
    CPUs next to its GPU (the PCI device's local_cpulist): the host-buffer path then crosses no socket
    link.  Returns what was done, for the JSON line."""
    try:
        pr = torch.cuda.get_device_properties(dev)
        bdf = "%04x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
        with open(f"/sys/bus/pci/devices/{bdf}/local_cpulist") as f:
            text = f.read().strip()
        cpus = set()
        for part in text.split(","):
            if "-" in part:
                a, b = part.split("-")
                cpus.update(range(int(a), int(b) + 1))
            elif part:
                cpus.add(int(part))
        allowed = os.sched_getaffinity(0)
        use = cpus & allowed
        if use:
            os.sched_setaffinity(0, use)
            return {"pci": bdf, "local_cpulist": text, "cpus_used": len(use)}
        return {"pci": bdf, "local_cpulist": text, "cpus_used": 0, "note": "no local CPU is allowed to this process"}
    except (OSError, ValueError, AttributeError) as exc:
        return {"error": repr(exc)}


def load_ncu_traffic():
    """DRAM bytes per launch of the dominant kernel per workload, from the ncu captures summarised under
    profiles/ (profiles/ncu_traffic.json names the capture each figure comes from)."""
    path = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    try:
        with open(path) as f:
            return json.load(f)
    except (OSError, ValueError):
        return {}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(tensor=p["bf16_tflops"], tensor_sustained=p.get("bf16_tflops_sustained"), hbm=p["hbm_gbs"],
                    source="measured")
    return dict(tensor=1590.0, tensor_sustained=1400.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML polled from a thread
    (about one sample per 0.3 ms, so that a region of a few milliseconds still gets samples);
    nvidia-smi in loop mode when NVML cannot be loaded."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid):
        self.uuid, self.proc, self.lines = uuid, None, []
        self.samples = []  # (time, sm_mhz, reasons bitmask)
        self.nvml = None
        self.stop_flag = False
        self.t_mark, self.t_end = 0.0, float("inf")

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.handle = pynvml.nvmlDeviceGetHandleByUUID(self.uuid.encode() if hasattr(self.uuid, "encode") else self.uuid)
            self.smax = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", self.uuid, f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _poll(self):
        n = self.nvml
        while not self.stop_flag:
            try:
                mhz = float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                reasons = int(n.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
            except Exception:
                break
            self.samples.append((time.perf_counter(), mhz, reasons))
            time.sleep(0.0003)

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def wait_first_sample(self, limit=10.0):
        t0 = time.perf_counter()
        while (self.nvml is not None or self.proc is not None) and not self.lines and not self.samples \
                and time.perf_counter() - t0 < limit:
            time.sleep(0.01)

    def mark(self):
        """Samples taken before this call (warm-up) are not counted."""
        self.t_mark = time.perf_counter()

    def mark_end(self):
        """Samples taken after this call are not counted."""
        self.t_end = time.perf_counter()

    def window(self, t0, t1):
        """Summary of the samples taken in [t0, t1] (NVML sampler only)."""
        return self._summary([x for x in self.samples if t0 <= x[0] <= t1])

    def _summary(self, rows):
        n = self.nvml
        names = (("hw_slowdown", 0x8), ("sw_thermal_slowdown", 0x20), ("hw_thermal_slowdown", 0x40), ("sw_power_cap", 0x4))
        sm = sorted(r[1] for r in rows)
        reasons = sorted({name for r in rows for name, bit in names if r[2] & bit})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": getattr(self, "smax", None),
                "reasons": reasons, "samples": len(sm)}

    def stop(self):
        if self.nvml is not None:
            self.stop_flag = True
            self.thread.join(timeout=2)
            return self.window(self.t_mark, self.t_end)
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock sampler available"]}
        self.proc.terminate()
        self.thread.join(timeout=2)
        sm, smax, reasons = [], None, set()
        for t, ln in self.lines:
            if t < self.t_mark or t > self.t_end:
                continue
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------ reference CPU arm

def cpu_reference_runner():
    """Returns (kind, fn(q,k,v,scale,causal,window,slopes)->o) for the CPU baseline:
    the reference's attention_forward_cpu compiled from its own sources when that
    library travelled with the repo, else the plain-C port."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib
    if oracle_lib.reference_lib() is not None:
        def run(q, k, v, scale, causal, window, slopes):
            return oracle_lib.reference_cpu_forward(q, k, v, scale, causal=causal, window=window, alibi_slopes=slopes)
        return "reference", run

    def run(q, k, v, scale, causal, window, slopes):
        return oracle_lib.forward(q, k, v, scale, causal=causal, window=(window, window), alibi_slopes=slopes,
                                  num_threads=1)[0]
    return "port", run


def time_cpu_reference(name, w, heads_per_step, steps, warmup):
    """Times the CPU attention on `heads_per_step` (batch, head) units of the
    workload per step, one unit per host thread."""
    import numpy as np
    kind, run = cpu_reference_runner()
    cores = os.cpu_count() or 1
    threads = min(cores, heads_per_step)
    rng = np.random.default_rng(0)
    N, d = w["Nk"], w["d"]
    if w["Nq"] != w["Nk"]:
        raise ValueError("the reference CPU function has one sequence length")
    q = rng.standard_normal((heads_per_step, 1, 1, N, d), dtype=np.float32)
    k = rng.standard_normal((heads_per_step, 1, 1, N, d), dtype=np.float32)
    v = rng.standard_normal((heads_per_step, 1, 1, N, d), dtype=np.float32)
    scale = 1.0 / np.sqrt(d)
    window = w["window"][0] if w["window"][0] >= 0 else -1
    slopes = [np.array([2.0 ** (-8.0 * ((h % w["H"]) + 1) / w["H"])], dtype=np.float32) if w["alibi"] else None
              for h in range(heads_per_step)]

    def one(i):
        run(q[i], k[i], v[i], scale, w["causal"], window, slopes[i])

    def step():
        with ThreadPoolExecutor(max_workers=threads) as ex:
            list(ex.map(one, range(heads_per_step)))

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    flops_unit = work_per_step(name, dict(w, B=1, H=1))[0]
    return dict(kind=kind, cores=threads, seconds_per_step=dt, tflops=flops_unit * heads_per_step / dt / 1e12,
                sample=f"{heads_per_step} of {w['B'] * w['H']} (batch, head) units of the workload per step, "
                       f"fp32, no dropout (the reference CPU path has none), {threads} threads")


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    w = WORKLOADS[args.workload]
    if w["Nq"] != w["Nk"]:
        emit(json.dumps({"impl": "reference", "unavailable": "the reference CPU attention has a single sequence length; "
                          "this workload has seqlen_q != seqlen_k"}))
        return 0
    cores = os.cpu_count() or 1
    heads = max(1, min(w["B"] * w["H"], cores))
    r = time_cpu_reference(args.workload, w, heads, max(1, args.steps), min(args.warmup, 1))
    line = {
        "impl": "reference", "metric": "fwd_attention_tflops", "value": r["tflops"], "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": min(args.warmup, 1),
        "ms_per_step": r["seconds_per_step"] * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": w["desc"], "timed": "reference CPU attention on host cores"},
        "cpu_baseline": {"value": r["tflops"], "unit": "TFLOP/s", "cores": r["cores"], "kind": r["kind"],
                         "sample": r["sample"]},
        "e2e": {"value": r["tflops"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(json.dumps(line))
    return 0


# ------------------------------------------------------------------ our arm

def make_inputs(torch, w, seed, device, copies):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    sets = []
    for _ in range(copies):
        q = torch.randn((w["B"], w["H"], w["Nq"], w["d"]), generator=g, device=device, dtype=torch.float32).bfloat16()
        hk = w.get("Hk", w["H"])
        k = torch.randn((w["B"], hk, w["Nk"], w["d"]), generator=g, device=device, dtype=torch.float32).bfloat16()
        v = torch.randn((w["B"], hk, w["Nk"], w["d"]), generator=g, device=device, dtype=torch.float32).bfloat16()
        sets.append((q, k, v))
    return sets


def time_device(torch, fa, name, w, sets, steps, warmup, rank, barrier, sampler=None, sustain_seconds=0.0, unit0=None):
    """Device-timed steps: returns (seconds per step of this rank, sustained leg or None).  The sustained
    leg repeats the step back to back for `sustain_seconds` (long enough for the power cap to set in and
    for the clock sampler to see it) and reports its own time per step and clocks."""
    units = w["B"] * w["H"]
    dev = sets[0][0].device
    slopes = None
    if w["alibi"]:
        slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / w["H"]) for h in range(w["H"])], device=dev)
    outs = [torch.empty((w["B"], w["H"], w["Nq"], w["d"]), device=dev, dtype=torch.bfloat16) for _ in sets]
    ws = torch.empty(max(16, _workspace_bytes(fa, w)), device=dev, dtype=torch.uint8)
    unit0 = rank * units if unit0 is None else unit0

    def step(i):
        q, k, v = sets[i % len(sets)]
        fa.flash_attn_forward(q, k, v, causal=w["causal"], window=w["window"], alibi_slopes=slopes,
                              p_dropout=w["p"], seed=42, offset=0, num_splits=w["splits"], out=outs[i % len(sets)],
                              unit0=unit0, workspace=ws)

    for i in range(warmup):
        step(i)
    barrier()
    torch.cuda.synchronize()
    # the device idled while the ranks met at the barrier: two untimed steps bring it back to the state
    # the warm-up left (without them the runs with a barrier measured 4 % slower than the run without)
    for i in range(2):
        step(i)
    if sampler is not None:
        sampler.mark()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    if sampler is not None:
        sampler.mark_end()
    barrier()
    sec = e0.elapsed_time(e1) / 1e3 / steps
    sustained = None
    if sustain_seconds > 0:
        n = max(steps, int(sustain_seconds / sec) + 1)
        t0 = time.perf_counter()
        e0.record()
        for i in range(n):
            step(i)
        e1.record()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        sustained = {"steps": n, "seconds": e0.elapsed_time(e1) / 1e3, "ms_per_step": e0.elapsed_time(e1) / n,
                     "clocks": sampler.window(t0, t1) if (sampler is not None and sampler.nvml is not None) else None}
    return sec, sustained


def _workspace_bytes(fa, w):
    if w["splits"] <= 1:
        return 0
    return w["B"] * w["H"] * w["splits"] * w["Nq"] * (w["d"] + 1) * 4 + 1024


def time_e2e(torch, fa, w, steps, warmup, rank):
    """Host-buffer path: pinned host Q/K/V in, O and LSE back, copies inside the timed region."""
    units = w["B"] * w["H"]
    g = torch.Generator()
    g.manual_seed(1234 + rank)
    shape_q = (w["B"], w["H"], w["Nq"], w["d"])
    shape_k = (w["B"], w.get("Hk", w["H"]), w["Nk"], w["d"])
    q = torch.randn(shape_q, generator=g).bfloat16().pin_memory()
    k = torch.randn(shape_k, generator=g).bfloat16().pin_memory()
    v = torch.randn(shape_k, generator=g).bfloat16().pin_memory()
    o = torch.empty(shape_q, dtype=torch.bfloat16).pin_memory()
    slopes = None
    if w["alibi"]:
        slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / w["H"]) for h in range(w["H"])])

    def step():
        return fa.flash_attn_forward_host(q, k, v, causal=w["causal"], window=w["window"], alibi_slopes=slopes,
                                          p_dropout=w["p"], seed=42, offset=0, num_splits=w["splits"], out=o)

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        _, lse = step()
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / steps
    h2d = (q.numel() + k.numel() + v.numel()) * 2
    d2h = o.numel() * 2 + lse.numel() * 4
    return dt, h2d, d2h


def measure_seq_parallel(torch, fa, w, mode, steps, warmup, rank, world, dev, barrier, max_over_ranks, sampler=None):
    """Config 5, ONE problem sharded over the ranks (strong scaling).  mode "ring": each rank holds two
    zig-zag chunks of the sequence, K/V chunks go round the ring (NCCL send/recv) while the forward kernel
    works, every visiting block merged into the running result in the kernel's epilogue.  mode "ulysses":
    head all-to-all.  Returns seconds per step (max over ranks), launches per step and rank, clocks."""
    from flash_attn_b200 import ring, ulysses
    N, C = w["Nq"], w["Nq"] // (2 * world)
    g = torch.Generator(device=dev)
    g.manual_seed(5 + rank)
    if mode == "ulysses":
        # contiguous slice of 2*C rows per rank; two all-to-alls trade it for whole sequences of H/P heads
        mk = lambda: (0.5 * torch.randn((w["B"], w["H"], 2 * C, w["d"]), generator=g, device=dev)).bfloat16()
        q, k, v = mk(), mk(), mk()
        run_step = lambda: ulysses.ulysses_attention_forward(q, k, v, causal=True)
        launches = ulysses._head_groups(w["H"], w["H"], world, 4)
    else:
        mk = lambda: [(0.5 * torch.randn((w["B"], w["H"], C, w["d"]), generator=g, device=dev)).bfloat16() for _ in range(2)]
        q, k, v = mk(), mk(), mk()
        run_step = lambda: ring.ring_attention_forward(q, k, v, causal=True)
        launches = len(ring.ring_schedule(rank, world, C, True))  # one forward launch per visited chunk pair
    for _ in range(warmup):
        run_step()
    barrier()
    torch.cuda.synchronize()
    run_step()  # (the device idled at the barrier)
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        run_step()
    e1.record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    barrier()
    mine = e0.elapsed_time(e1) / 1e3 / steps
    sec = max_over_ranks(mine)
    clocks = sampler.window(t0, t1) if (sampler is not None and sampler.nvml is not None) else None
    del q, k, v
    torch.cuda.empty_cache()
    return {"sec": sec, "launches": launches, "clocks": clocks, "chunk": C}


def c5_entry(w, flops, world, m, peaks, mode):
    value = flops / m["sec"] / 1e12
    e = {"path": "K/V ring (NCCL send/recv, merge in the kernel epilogue)" if mode == "ring" else "head all-to-all (NCCL)",
         "ms_per_step": m["sec"] * 1e3, "tflops": value, "tflops_per_gpu": value / world,
         "frac_of_sustained_tensor_peak": value / world / (peaks["tensor_sustained"] or peaks["tensor"]),
         "launches_per_step_per_rank": m["launches"], "clocks": m["clocks"]}
    if m["clocks"] and m["clocks"].get("sm_mhz"):
        e["tflops_per_gpu_per_mhz"] = value / world / m["clocks"]["sm_mhz"]
    return e


def run_c5(torch, fa, args, w, flops, peaks, rank, world, dev, dist, barrier, max_over_ranks):
    """--workload c5: the line describes the path BASELINE's config 5 names (the ring) unless
    --seq-parallel ulysses asks for the all-to-all; the other path is measured beside it."""
    main_mode = args.seq_parallel
    if main_mode == "ulysses" and w["H"] % world != 0:
        main_mode = "ring"
    other = "ulysses" if main_mode == "ring" else "ring"
    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(dev).uuid)) if rank == 0 else None
    if sampler:
        sampler.start()
        sampler.wait_first_sample()
    m = measure_seq_parallel(torch, fa, w, main_mode, args.steps, args.warmup, rank, world, dev, barrier, max_over_ranks, sampler)
    m2 = None
    if not args.no_secondary and (other == "ring" or w["H"] % world == 0):
        m2 = measure_seq_parallel(torch, fa, w, other, args.steps, args.warmup, rank, world, dev, barrier, max_over_ranks, sampler)
    if sampler:
        sampler.stop()
    value = flops / m["sec"] / 1e12
    N, C = w["Nq"], m["chunk"]
    line = {
        "metric": "fwd_attention_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": m["sec"] * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": ({"workload": w["desc"].replace("sequence ring over the ranks (zig-zag chunks, NCCL send/recv, LSE merge)",
                                                   "head all-to-all over the ranks (NCCL), whole sequences of H/P heads per rank"),
                    "rows_per_rank": 2 * C, "a2a_bytes_sent_per_rank": (4 * w["B"] * w["H"] * 2 * C * w["d"] * 2) * (world - 1) // world,
                    "l2": "each rank reads %d MB of K/V per step (> L2)" % (2 * w["B"] * w["H"] // world * N * w["d"] * 2 // 2 ** 20),
                    "flops_per_step_total": flops} if main_mode == "ulysses" else
                   {"workload": w["desc"], "chunk_rows": C, "kv_bytes_per_ring_step_per_rank": 4 * w["B"] * w["H"] * C * w["d"] * 2,
                    "l2": "each rank streams 2 x %d MB of K/V per ring step (> L2)" % (2 * w["H"] * C * w["d"] * 2 // 2 ** 20),
                    "flops_per_step_total": flops}),
        "clocks": m["clocks"],
        "e2e": {"value": None, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "note": "the sharded sequence lives in device memory; the host-buffer path is measured on config 2"},
        "gpu_launches": m["launches"] * args.steps * world,
        "roofline": {"bound": "tensor", "achieved": value / world, "peak": peaks["tensor_sustained"] or peaks["tensor"],
                     "unit": "TFLOP/s", "frac": value / world / (peaks["tensor_sustained"] or peaks["tensor"]),
                     "peak_source": peaks["source"] + " sustained (seconds-long step)", "traffic": None,
                     "kernel": "fwd_tiled_kernel"},
        "secondary": {main_mode: c5_entry(w, flops, world, m, peaks, main_mode)},
    }
    if m2 is not None:
        line["secondary"][other] = c5_entry(w, flops, world, m2, peaks, other)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        emit(json.dumps(line))
    return 0


_RESULT_OUT = None


def keep_stdout_for_the_result():
    """The process's stdout carries the one JSON line and nothing else: file descriptor 1 is pointed
    at stderr for everything that runs from here on (NCCL prints its version banner to stdout, torchrun
    and other libraries may print too) and the original is kept for emit()."""
    global _RESULT_OUT
    if _RESULT_OUT is None:
        sys.stdout.flush()
        _RESULT_OUT = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit(text):
    out = _RESULT_OUT if _RESULT_OUT is not None else sys.stdout
    out.write(text + "\n")
    out.flush()


def main():
    keep_stdout_for_the_result()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="default: 2000 (c2), 200 (c3), 50 (c4), 5 (c5)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--seq-parallel", default="ring", choices=["ring", "ulysses"],
                    help="config 5: K/V ring with the LSE merge in the kernel epilogue (default: the path the "
                         "baseline's config 5 names) or head all-to-all; the other one is measured beside it")
    ap.add_argument("--no-secondary", action="store_true", help="skip the c3/c4 side measurements")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (for profiler runs)")
    ap.add_argument("--batch", type=int, default=None, help="override the workload's batch size (smaller cases "
                    "for profiler captures; the JSON line then describes the reduced workload)")
    args = ap.parse_args()
    if args.steps is None:
        args.steps = {"c2": 2000, "c3": 200, "c4": 50, "c4gqa": 100, "c5": 5}[args.workload] if args.impl == "ours" else 2
    if args.impl == "reference":
        return run_reference_arm(args)
    args.warmup = max(args.warmup, 3)

    import torch
    import flash_attn_b200 as fa
    from flash_attn_b200 import _lib
    _lib.load()  # fails loudly when the CUDA library is missing: there is no fallback

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    affinity = pin_to_gpu_node(torch, dev)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # NCCL's own stream at high priority: the ring's send/recv kernels must not queue behind the
        # attention launch they overlap
        opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
        dist.init_process_group("nccl", device_id=dev, pg_options=opts)

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(x):
        if dist is None:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def gather_floats(x):
        if dist is None:
            return [x]
        t = torch.zeros(world, device=dev, dtype=torch.float64)
        t[rank] = x
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return [float(v) for v in t.tolist()]

    name = args.workload
    w = dict(WORKLOADS[name])
    if args.batch is not None:
        w["B"] = args.batch
        w["desc"] += f" [batch reduced to {args.batch}]"
    flops, nbytes = work_per_step(name, w)
    peaks = load_peaks()
    if name == "c5":
        return run_c5(torch, fa, args, w, flops, peaks, rank, world, dev, dist, barrier, max_over_ranks)
    # two input sets (2 x 268 MB for config 2) alternate, so no step finds its inputs in the 126 MB L2
    sets = make_inputs(torch, w, 2 + rank, dev, copies=2 if not name.startswith("c4") else 1)

    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(dev).uuid)) if rank == 0 else None
    if sampler:
        sampler.start()
        sampler.wait_first_sample()
    my_sec, sustained = time_device(torch, fa, name, w, sets, args.steps, args.warmup, rank, barrier, sampler,
                                    sustain_seconds=0.0 if args.no_secondary else 0.6)
    clocks = sampler.stop() if sampler else None
    sec = max_over_ranks(my_sec)
    per_rank_ms = gather_floats(my_sec * 1e3)
    del sets
    torch.cuda.empty_cache()

    if args.no_e2e:
        e2e_sec, h2d, d2h = float("inf"), 0, 0
    else:
        e2e_sec, h2d, d2h = time_e2e(torch, fa, w, max(3, min(args.steps, 10)), 2, rank)
        e2e_sec = max_over_ranks(e2e_sec)

    is_decode = name.startswith("c4")
    if is_decode:
        metric, unit = "decode_hbm_gbs", "GB/s"
        value = world * nbytes / sec / 1e9
        e2e_value = world * nbytes / e2e_sec / 1e9
        roof = {"bound": "hbm", "achieved": nbytes / sec / 1e9, "peak": peaks["hbm"], "unit": "GB/s"}
    else:
        metric, unit = "fwd_attention_tflops", "TFLOP/s"
        value = world * flops / sec / 1e12
        e2e_value = world * flops / e2e_sec / 1e12
        roof = {"bound": "tensor", "achieved": flops / sec / 1e12, "peak": peaks["tensor"], "unit": "TFLOP/s"}
    roof["frac"] = roof["achieved"] / roof["peak"]
    if not is_decode and peaks["tensor_sustained"]:
        # the default run is long enough to meet the power cap (see "clocks"): the fraction of the
        # sustained cuBLAS rate, measured under the same cap, is given beside the burst one
        roof["frac_of_sustained_peak"] = roof["achieved"] / peaks["tensor_sustained"]
        roof["sustained_peak"] = peaks["tensor_sustained"]
    roof["peak_source"] = peaks["source"] + (" burst" if not is_decode else " copy")
    # DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the ncu captures summarised
    # under profiles/; null where no capture of the workload exists or the batch was overridden
    traffic = load_ncu_traffic().get(name) if args.batch is None else None
    roof["traffic"] = traffic["bytes_per_launch"] if traffic else None
    roof["traffic_source"] = traffic["source"] if traffic else None
    if is_decode:
        roof["frac_of_nominal_8tbs"] = roof["achieved"] / 8000.0
        roof["peak_note"] = "peak is the measured read+write copy rate; a read-only stream can exceed it, see frac_of_nominal_8tbs"
    roof["kernel"] = "decode_kernel (+ combine_kernel)" if is_decode else "fwd_tiled_kernel"
    launches_per_step = 1 if w["splits"] <= 1 else 2

    line = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": w["desc"], "units_per_gpu": w["B"] * w["H"], "l2": "two input sets alternate; each "
                   "step reads inputs larger than the 126 MB L2" if not is_decode else "%.1f GB streamed per step" % (nbytes / 1e9),
                   "timed_region": "barrier + synchronize, two untimed steps (the device idled at the barrier), "
                                   "K steps between CUDA events, synchronize + barrier",
                   "flops_per_step_per_gpu": flops, "bytes_per_step_per_gpu": nbytes},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_sec * 1e3, "api": "fa_fwd_host (pinned host buffers)",
                "host_gbs_per_gpu": (h2d + d2h) / e2e_sec / 1e9, "host_gbs_all_gpus": world * (h2d + d2h) / e2e_sec / 1e9,
                "cpu_affinity": affinity},
        "gpu_launches": launches_per_step * args.steps * world,
        "roofline": roof,
        "per_rank_ms": per_rank_ms,
    }
    if sustained is not None:
        # the same step repeated back to back for >= 0.6 s: long enough to meet the power cap, with the
        # clocks seen over exactly that stretch
        sv = (nbytes / 1e9 if is_decode else flops / 1e12) / (sustained["ms_per_step"] / 1e3)
        line["sustained"] = {"steps": sustained["steps"], "seconds": sustained["seconds"], "ms_per_step": sustained["ms_per_step"],
                             "value_per_gpu": sv, "unit": unit, "clocks": sustained["clocks"],
                             "frac_of_sustained_peak": (sv / peaks["tensor_sustained"]) if (not is_decode and peaks["tensor_sustained"]) else None}

    if rank == 0 and world == 1 and not args.no_secondary and name == "c2":
        side = {}
        for other in ("c3", "c4", "c4gqa"):
            try:
                ow = WORKLOADS[other]
                osets = make_inputs(torch, ow, 3, dev, copies=1)
                osec, _ = time_device(torch, fa, other, ow, osets, 5 if other == "c4" else 10, 3, 0, lambda: None)
                of, ob = work_per_step(other, ow)
                if other.startswith("c4"):
                    side[other] = {"workload": ow["desc"], "ms": osec * 1e3, "gbs": ob / osec / 1e9,
                                   "frac_of_hbm_peak": ob / osec / 1e9 / peaks["hbm"]}
                else:
                    side[other] = {"workload": ow["desc"], "ms": osec * 1e3, "tflops": of / osec / 1e12,
                                   "frac_of_tensor_peak": of / osec / 1e12 / peaks["tensor"]}
                del osets
                torch.cuda.empty_cache()
            except Exception as exc:  # a side measurement must not lose the main line
                side[other] = {"error": repr(exc)}
        line["secondary"] = side

    if world > 1 and not args.no_secondary and name == "c2":
        # Strong scaling beside the weak-scaling line: ONE config-2/3/4 problem whose (batch, head)
        # units are cut into `world` slices, one per rank, with no communication ("heads sharded"),
        # and config 5, one sequence sharded over the ranks (ring and head all-to-all).
        strong = {}
        for other in ("c2", "c3", "c4"):
            try:
                ow = dict(WORKLOADS[other])
                total_units = ow["B"] * ow["H"]
                lo, hi = (rank * total_units) // world, ((rank + 1) * total_units) // world
                of, ob = work_per_step(other, ow)  # the whole problem
                ow["B"], ow["H"] = 1, hi - lo  # this rank's slice, described as one batch of (hi - lo) heads
                osets = make_inputs(torch, ow, 7 + rank, dev, copies=2 if other == "c2" else 1)
                osec, _ = time_device(torch, fa, other, ow, osets, 5 if other == "c4" else 20, 3, rank, barrier, unit0=lo)
                osec = max_over_ranks(osec)
                e = {"workload": WORKLOADS[other]["desc"], "units_total": total_units, "units_per_rank": hi - lo,
                     "ms": osec * 1e3, "scaling": "strong"}
                if other == "c4":
                    e.update(gbs=ob / osec / 1e9, gbs_per_gpu=ob / osec / 1e9 / world,
                             frac_of_hbm_peak_per_gpu=ob / osec / 1e9 / world / peaks["hbm"])
                else:
                    e.update(tflops=of / osec / 1e12, tflops_per_gpu=of / osec / 1e12 / world,
                             frac_of_tensor_peak_per_gpu=of / osec / 1e12 / world / peaks["tensor"])
                    if other == "c3":
                        e["note"] = "ALiBi slopes follow the slice's own head numbering (same work per head)"
                strong[other] = e
                del osets
                torch.cuda.empty_cache()
            except Exception as exc:
                strong[other] = {"error": repr(exc)}
        side = {"strong": strong}
        try:
            w5 = WORKLOADS["c5"]
            f5, _ = work_per_step("c5", w5)
            smp = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(dev).uuid)) if rank == 0 else None
            if smp:
                smp.start()
                smp.wait_first_sample()
            c5 = {"workload": w5["desc"], "scaling": "strong", "steps": 3}
            m = measure_seq_parallel(torch, fa, w5, "ring", 3, 1, rank, world, dev, barrier, max_over_ranks, smp)
            c5["ring"] = c5_entry(w5, f5, world, m, peaks, "ring")
            if w5["H"] % world == 0:
                m = measure_seq_parallel(torch, fa, w5, "ulysses", 3, 1, rank, world, dev, barrier, max_over_ranks, smp)
                c5["ulysses"] = c5_entry(w5, f5, world, m, peaks, "ulysses")
            if smp:
                smp.stop()
            side["c5"] = c5
        except Exception as exc:
            side["c5"] = {"error": repr(exc)}
        line["secondary"] = side

    if rank == 0 and world == 1 and not args.no_secondary and name == "c2":
        # the C benchmark driver (no Python between the launches) on the same workload, as a cross-check
        # of the time per launch
        try:
            exe = os.path.join(ROOT, "flash_attn_b200", "fa_bench")
            if os.path.exists(exe):
                out = subprocess.run([exe, "--config", "2", "--iters", "200", "--warmup", "10"], capture_output=True,
                                     text=True, timeout=120)
                r = json.loads(out.stdout.strip().splitlines()[-1])
                line.setdefault("secondary", {})["c_driver"] = {"what": "fa_bench --config 2 (C99 over the C ABI), 200 launches",
                                                                "ms_per_launch": r["ms_per_iter"], "tflops": r["tflops"]}
        except Exception as exc:
            line.setdefault("secondary", {})["c_driver"] = {"error": repr(exc)}

    if rank == 0 and world == 1 and not args.no_secondary and name == "c2":
        # the reference's own kernels (fp16, recompiled for sm_100a) on the same shape, for context
        try:
            sys.path.insert(0, os.path.join(ROOT, "tests"))
            import ref_gpu
            if ref_gpu.available():
                qh, kh, vh = (torch.randn((w["B"], w["H"], w["Nq"], w["d"]), device=dev).half() for _ in range(3))
                _, used, us = ref_gpu.forward(qh, kh, vh, w["d"] ** -0.5, causal=True, iters=5)
                line["reference_gpu_kernels"] = {"what": "reference forward_kernel (mma.sync, fp16, causal, no dropout, "
                                                 "fp32 O) recompiled for sm_100a", "ms": us / 1e3,
                                                 "tflops": flops / (us * 1e-6) / 1e12, "splits": used}
                del qh, kh, vh
        except Exception as exc:
            line["reference_gpu_kernels"] = {"error": repr(exc)}

    if rank == 0 and world == 1 and not args.no_cpu:
        try:
            cw = w if w["Nq"] == w["Nk"] else WORKLOADS["c2"]
            cores = os.cpu_count() or 1
            r = time_cpu_reference(name if w["Nq"] == w["Nk"] else "c2", cw, min(cw["B"] * cw["H"], 2 * cores), 1, 0)
            line["cpu_baseline"] = {"value": r["tflops"], "unit": "TFLOP/s", "cores": r["cores"], "kind": r["kind"],
                                    "sample": r["sample"]}
        except Exception as exc:
            line["cpu_baseline"] = {"value": None, "unit": "TFLOP/s", "cores": 0, "kind": "port", "sample": repr(exc)}

    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        emit(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
