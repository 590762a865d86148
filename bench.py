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


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(tensor=p["bf16_tflops"], tensor_sustained=p.get("bf16_tflops_sustained"), hbm=p["hbm_gbs"],
                    source="measured")
    return dict(tensor=1590.0, tensor_sustained=1400.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid):
        self.uuid, self.proc, self.lines = uuid, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", self.uuid, f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def wait_first_sample(self, limit=10.0):
        t0 = time.perf_counter()
        while self.proc is not None and not self.lines and time.perf_counter() - t0 < limit:
            time.sleep(0.01)

    def mark(self):
        """Samples taken before this call (warm-up) are not counted."""
        self.t_mark = time.perf_counter()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.thread.join(timeout=2)
        sm, smax, reasons = [], None, set()
        t_mark = getattr(self, "t_mark", 0.0)
        for t, ln in self.lines:
            if t < t_mark:
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
        print(json.dumps({"impl": "reference", "unavailable": "the reference CPU attention has a single sequence length; "
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
    print(json.dumps(line))
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


def time_device(torch, fa, name, w, sets, steps, warmup, rank, barrier, sampler=None):
    """Device-timed steps: returns seconds per step (this rank)."""
    units = w["B"] * w["H"]
    dev = sets[0][0].device
    slopes = None
    if w["alibi"]:
        slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / w["H"]) for h in range(w["H"])], device=dev)
    outs = [torch.empty((w["B"], w["H"], w["Nq"], w["d"]), device=dev, dtype=torch.bfloat16) for _ in sets]
    ws = torch.empty(max(16, _workspace_bytes(fa, w)), device=dev, dtype=torch.uint8)

    def step(i):
        q, k, v = sets[i % len(sets)]
        fa.flash_attn_forward(q, k, v, causal=w["causal"], window=w["window"], alibi_slopes=slopes,
                              p_dropout=w["p"], seed=42, offset=0, num_splits=w["splits"], out=outs[i % len(sets)],
                              unit0=rank * units, workspace=ws)

    for i in range(warmup):
        step(i)
    barrier()
    torch.cuda.synchronize()
    if sampler is not None:
        sampler.mark()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    barrier()
    return e0.elapsed_time(e1) / 1e3 / steps


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


def run_ring(torch, fa, args, w, flops, peaks, rank, world, dev, dist, barrier, max_over_ranks):
    """Config 5: ONE problem sharded over the ranks (strong scaling): each rank holds two zig-zag
    chunks of the sequence; K/V chunks go round the ring while the forward kernel works."""
    from flash_attn_b200 import ring, ulysses
    use_a2a = args.seq_parallel == "ulysses" and w["H"] % world == 0
    N, C = w["Nq"], w["Nq"] // (2 * world)
    g = torch.Generator(device=dev)
    g.manual_seed(5 + rank)
    if use_a2a:
        # contiguous slice of 2*C rows per rank; two all-to-alls trade it for whole sequences of H/P heads
        mk = lambda: (0.5 * torch.randn((w["B"], w["H"], 2 * C, w["d"]), generator=g, device=dev)).bfloat16()
        run_step = lambda: ulysses.ulysses_attention_forward(q, k, v, causal=True)
    else:
        mk = lambda: [(0.5 * torch.randn((w["B"], w["H"], C, w["d"]), generator=g, device=dev)).bfloat16() for _ in range(2)]
        run_step = lambda: ring.ring_attention_forward(q, k, v, causal=True)
    q, k, v = mk(), mk(), mk()
    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(dev).uuid)) if rank == 0 else None
    if sampler:
        sampler.start()
        sampler.wait_first_sample()
    for _ in range(args.warmup):
        run_step()
    barrier()
    torch.cuda.synchronize()
    if sampler:
        sampler.mark()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run_step()
    e1.record()
    torch.cuda.synchronize()
    barrier()
    sec = max_over_ranks(e0.elapsed_time(e1) / 1e3 / args.steps)
    clocks = sampler.stop() if sampler else None
    value = flops / sec / 1e12
    # kernel launches per step and rank: one forward + one merge per visited (query chunk, key chunk) pair, two casts
    pairs = sum(1 for s in range(world) for a in ring.zigzag_chunks(rank, world)
                for b in ring.zigzag_chunks((rank - s) % world, world) if b <= a)
    line = {
        "metric": "fwd_attention_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": ({"workload": w["desc"].replace("sequence ring over the ranks (zig-zag chunks, NCCL send/recv, LSE merge)",
                                                   "head all-to-all over the ranks (NCCL), whole sequences of H/P heads per rank"),
                    "rows_per_rank": 2 * C, "a2a_bytes_sent_per_rank": (4 * w["B"] * w["H"] * 2 * C * w["d"] * 2) * (world - 1) // world,
                    "l2": "each rank reads %d MB of K/V per step (> L2)" % (2 * w["B"] * w["H"] // world * N * w["d"] * 2 // 2 ** 20),
                    "flops_per_step_total": flops} if use_a2a else
                   {"workload": w["desc"], "chunk_rows": C, "kv_bytes_per_ring_step_per_rank": 4 * w["B"] * w["H"] * C * w["d"] * 2,
                    "l2": "each rank streams 2 x %d MB of K/V per ring step (> L2)" % (2 * w["H"] * C * w["d"] * 2 // 2 ** 20),
                    "flops_per_step_total": flops}),
        "clocks": clocks,
        "e2e": {"value": None, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "note": "the ring works on device-resident shards; the host-buffer path is measured on config 2"},
        # all-to-all: one forward launch per head group; ring: forward + merge per visited pair, two casts
        "gpu_launches": (ulysses._head_groups(w["H"], w["H"], world, 4) if use_a2a else 2 * pairs + 2) * args.steps * world,
        "roofline": {"bound": "tensor", "achieved": value / world, "peak": peaks["tensor_sustained"] or peaks["tensor"],
                     "unit": "TFLOP/s", "frac": value / world / (peaks["tensor_sustained"] or peaks["tensor"]),
                     "peak_source": peaks["source"] + " sustained (seconds-long step)", "traffic": None,
                     "kernel": "fwd_tiled_kernel"},
    }
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="default: 2000 (c2), 200 (c3), 50 (c4), 5 (c5)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--seq-parallel", default="ulysses", choices=["ring", "ulysses"],
                    help="config 5: head all-to-all (default; the faster of the two at 8 GPUs) or K/V ring with "
                         "LSE merge (also taken when the head count is not a multiple of the GPU count)")
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
    if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
        os.environ["NCCL_DEBUG"] = "WARN"  # keeps NCCL's version banner off stdout: rank 0 prints one JSON line
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(x):
        if dist is None:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    name = args.workload
    w = dict(WORKLOADS[name])
    if args.batch is not None:
        w["B"] = args.batch
        w["desc"] += f" [batch reduced to {args.batch}]"
    flops, nbytes = work_per_step(name, w)
    peaks = load_peaks()
    if name == "c5":
        return run_ring(torch, fa, args, w, flops, peaks, rank, world, dev, dist, barrier, max_over_ranks)
    # two input sets (2 x 268 MB for config 2) alternate, so no step finds its inputs in the 126 MB L2
    sets = make_inputs(torch, w, 2 + rank, dev, copies=2 if not name.startswith("c4") else 1)

    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(dev).uuid)) if rank == 0 else None
    if sampler:
        sampler.start()
        sampler.wait_first_sample()
    sec = time_device(torch, fa, name, w, sets, args.steps, args.warmup, rank, barrier, sampler)
    clocks = sampler.stop() if sampler else None
    sec = max_over_ranks(sec)
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
    # DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures
    # summarised under profiles/: config 2 captured at full size, config 4 captured on 128 of the
    # 2048 units and scaled by the units processed; null where no capture of the workload exists
    ncu_traffic = {"c2": 201.42e6 + 47.13e6, "c4": 16 * (2.1476e9 + 5.1e6)}  # no capture of c3 / c4gqa
    roof["traffic"] = ncu_traffic.get(name) if args.batch is None else None
    roof["traffic_source"] = "ncu capture (static figure, not measured in this run)" if roof["traffic"] else None
    roof["kernel"] = "decode_kernel (+ combine_kernel)" if is_decode else "fwd_tiled_kernel"
    launches_per_step = 1 if w["splits"] <= 1 else 2

    line = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": w["desc"], "units_per_gpu": w["B"] * w["H"], "l2": "two input sets alternate; each "
                   "step reads inputs larger than the 126 MB L2" if not is_decode else "%.1f GB streamed per step" % (nbytes / 1e9),
                   "flops_per_step_per_gpu": flops, "bytes_per_step_per_gpu": nbytes},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_sec * 1e3, "api": "fa_fwd_host (pinned host buffers)"},
        "gpu_launches": launches_per_step * args.steps * world,
        "roofline": roof,
    }

    if rank == 0 and world == 1 and not args.no_secondary and name == "c2":
        side = {}
        for other in ("c3", "c4", "c4gqa"):
            try:
                ow = WORKLOADS[other]
                osets = make_inputs(torch, ow, 3, dev, copies=1)
                osec = time_device(torch, fa, other, ow, osets, 5 if other == "c4" else 10, 3, 0, lambda: None)
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
        print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
