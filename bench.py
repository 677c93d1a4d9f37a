#!/usr/bin/env python
"""Benchmark of the nestedtensor hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload pad|unpad|mha] [--impl ours|reference]

One JSON line on stdout (rank 0).  A "step" is one pass of the hot path over one batch of seeded
synthetic input:

  pad    (default) configuration 2: `to_padded_tensor(padding=0)` of 4096 bf16 sequences (L_i, 1024)
         -> (4096, 1024, 1024); metric = HBM GB/s = algorithmic bytes (ragged read once + dense
         written once) / time
  unpad  the inverse with known sizes (2 * valid bytes)
  mha    configuration 5: BERT-large varlen self-attention forward, bf16; metric = valid tokens/s

N > 1 (launched by torch.distributed.run, one rank per GPU): the global job is N batches of the
configuration drawn as one sequence list and cut into N contiguous token-balanced shards; no
collective on the data path (weak scaling).  `value` is whole-job throughput over the slowest rank.
The same line carries a `strong` record: the FIXED configuration lists (4096 / 1024 / 128 sequences) cut
into N token-balanced shards, with the shard outputs all-gathered over NCCL outside the timed region and
compared on rank 0 with the one-GPU result of the whole list.

Every device-timed figure is the MEDIAN of five timed regions of K steps each (the best region is kept
beside it as `best_ms`).

`--impl reference` times the CPU restatement of the reference's own implementation
(oracle/ntref.py; the reference extension cannot be built against this torch) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0


# ----------------------------------------------------------------------------- helpers
def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    except Exception:
        return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS,
                "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.02):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {}
        for n in dir(nv):
            if n.startswith("nvmlClocksThrottleReason") or n.startswith("nvmlClocksEventReason"):
                v = getattr(nv, n)
                if isinstance(v, int) and v not in (0,):
                    names[v] = n.replace("nvmlClocksThrottleReason", "").replace("nvmlClocksEventReason", "")
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in names.items():
                    if bit & (bit - 1) == 0 and mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        med = s[len(s) // 2] if s else None
        ignore = {"GpuIdle", "None", "ApplicationsClocksSetting"}
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "samples": len(s),
                "reasons": sorted(r for r in self.reasons if r not in ignore)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def timed_region(fn, steps, world, device):
    """barrier + synchronize, K steps between two CUDA events on the current stream, synchronize +
    barrier; returns the max over ranks of the elapsed milliseconds."""
    import torch.distributed as dist
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize(device)
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    return ms


def timed_regions(fn, steps, world, device, regions=5):
    """`regions` timed regions of `steps` steps; returns (median ms per step, best ms per step)."""
    ms = sorted(timed_region(fn, steps, world, device) / steps for _ in range(regions))
    return ms[len(ms) // 2], ms[0]


def graph_ms(fn, n, device):
    """Device time per call with the host's launch cost taken out: `n` calls of `fn` captured into ONE CUDA graph,
    replayed once between two events (after a warm-up replay).  For operators of 60-100 us the eager loop leaves a
    few microseconds of idle device between launches; this is the figure to hold against the kernel's roofline.
    Returns None if the call cannot be captured."""
    try:
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize(device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(n):
                fn()
        g.replay()
        torch.cuda.synchronize(device)
        best = None
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize(device)
            ms = e0.elapsed_time(e1) / n
            best = ms if best is None or ms < best else best
        del g
        return best
    except Exception:
        torch.cuda.synchronize(device)
        return None


def all_sum(x, world, device):
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([float(x)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


# --------------------------------------------------------------------------- workloads
SEQUENCE_LIMIT = 0   # --sequences: keep only the first N sequences of each shard (small cases for profiler captures)
KERNEL_ONLY = False  # --kernel-only: skip the end-to-end pass, the CPU baseline and the parity spot check


def _pure_module(name):
    """`nestedtensor_b200.workloads` / `.sharding` loaded by file path: they are plain Python, and importing the
    package instead would load the native libraries, which the reference arm must not touch."""
    import importlib.util
    key = "_ntb200_pure_" + name
    if key in sys.modules:
        return sys.modules[key]
    spec = importlib.util.spec_from_file_location(key, os.path.join(ROOT, "nestedtensor_b200", name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[key] = mod
    spec.loader.exec_module(mod)
    return mod


def shard_lengths(kind, world, rank):
    """Lengths of this rank's shard: N batches of the configuration drawn as ONE list (generator of the
    configuration, batch = N * config batch) and cut token-balanced into N contiguous slices."""
    workloads, sharding = _pure_module("workloads"), _pure_module("sharding")
    if kind in ("pad", "unpad"):
        L = workloads.lengths_c2(workloads._gen(2), 4096 * world)
    else:
        L = workloads.lengths_c5(workloads._gen(5), 1024 * world)
    parts = sharding.token_balanced_partition(L.tolist(), world)
    a, b = parts[rank]
    if SEQUENCE_LIMIT:
        b = min(b, a + SEQUENCE_LIMIT)
    return L[a:b].contiguous(), sharding.imbalance(L.tolist(), parts)


def host_values(n, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    out = torch.empty(n, dtype=dtype)
    chunk = 1 << 26
    for a in range(0, n, chunk):
        b = min(n, a + chunk)
        out[a:b] = torch.randn(b - a, generator=g).to(dtype)
    return out


def cpu_pad_sample(L, hidden, dtype, seqs):
    """The reference's CPU to_padded_tensor (oracle port) on the first `seqs` sequences."""
    from oracle import ntref
    Ls = L[:seqs].tolist()
    g = torch.Generator().manual_seed(11)
    tensors = [torch.randn(l, hidden, generator=g).to(dtype) for l in Ls]
    es = tensors[0].element_size()
    nbytes = es * (sum(Ls) * hidden + len(Ls) * max(Ls) * hidden)
    return tensors, nbytes, (lambda: ntref.to_padded_tensor(tensors, 0))


def cpu_unpad_sample(L, hidden, dtype, seqs):
    from oracle import ntref
    Ls = L[:seqs].tolist()
    g = torch.Generator().manual_seed(11)
    padded = torch.randn(len(Ls), max(Ls), hidden, generator=g).to(dtype)
    sizes = [[l, hidden] for l in Ls]
    nbytes = 2 * padded.element_size() * sum(Ls) * hidden
    return padded, nbytes, (lambda: ntref.from_padded_tensor(padded, sizes))


def time_cpu(fn, warmup, iters):
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        t0 = time.perf_counter()
        fn()
        ts.append(time.perf_counter() - t0)
    ts.sort()
    return ts[len(ts) // 2]


# ------------------------------------------------------------------------- pad / unpad
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per ALGORITHMIC byte of the dominant kernel, from the ncu
# captures summarised under profiles/ (taken on the first 512 sequences of configuration 2 and the first 256 of
# configuration 5, where traffic grows in proportion to the batch: reads equalled the algorithmic bytes, writes fell
# short of them by the lines still dirty in L2 when the kernel ended).  The bench line scales the ratio by the
# algorithmic bytes of the launch it timed, and prints null for a sub-batch run.
NCU_TRAFFIC_PER_ALG_BYTE = {"pad": 10.48 / 10.54, "unpad": 3.85 / 3.90}
NCU_TRAFFIC_GEMM_BYTES_PER_TOKEN = {"mha": 1.20e9 / 151792, "encoder": 1.51e9 / 151792}
NCU_TRAFFIC_SOURCE = "ncu capture summarised in profiles/ (sub-batch, scaled by the units of this launch)"


def copy_values(L, hidden, dtype, world, rank):
    """Values of this rank's shard.  One GPU: the whole configuration-2 buffer from the configuration's own generator
    (lengths first, then all values in one draw).  N > 1: the global list is N batches and only the lengths are drawn
    from that generator on every rank; each rank draws its shard's values from a generator seeded by its rank."""
    if world == 1 and not SEQUENCE_LIMIT:
        w = _pure_module("workloads").config2()
        assert torch.equal(w.sizes[:, 0], L)
        return w.buffer, "workloads.config2 (seed 20242: lengths, then values)"
    return host_values(int(L.sum()) * hidden, dtype, 20242 + 1000 * (rank + 1)), "per-rank generator (seed 20242 + 1000*(rank+1))"


def run_copy(args, kind, rank, world, local):
    import nestedtensor_b200 as nt
    from nestedtensor_b200 import _ops
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    hidden, dtype = 1024, torch.bfloat16
    es = 2
    L, imb = shard_lengths(kind, world, rank)
    B, T, maxL = int(L.numel()), int(L.sum()), int(L.max())
    sizes = torch.stack([L, torch.full_like(L, hidden)], 1).contiguous()
    n_valid, n_pad = T * hidden, B * maxL * hidden
    alg_bytes = es * (n_valid + n_pad) if kind == "pad" else 2 * es * n_valid

    # resident inputs (generated on the host, copied once, outside the timed region)
    host, values_from = copy_values(L, hidden, dtype, world, rank)
    ragged = host.to(device)
    a = nt.NestedTensor(ragged, sizes)
    ops = _ops.ops()
    buf, sz, meta = a._record()
    if kind == "pad":
        step = lambda: ops.to_padded_tensor(buf, sz, meta, 0.0)
    else:
        padded = ops.to_padded_tensor(buf, sz, meta, 0.0)
        step = lambda: ops.from_padded_tensor(padded, sz, meta)
    for _ in range(max(args.warmup, 3)):
        step()
    with ClockSampler(local) as clocks:
        kernel_ms, best_ms = timed_regions(step, args.steps, world, device)
    total_bytes = all_sum(alg_bytes, world, device)
    value = total_bytes / (kernel_ms * 1e-3) / 1e9

    # parity spot check in the same run (size-independent property): round trip is the identity
    parity_ok = None
    if not KERNEL_ONLY:
        chk = ops.from_padded_tensor(ops.to_padded_tensor(buf, sz, meta, 0.0), sz, meta)
        parity_ok = bool(torch.equal(chk.view(torch.int16), ragged.view(torch.int16)))
        del chk

    # the inverse on the same shard, device-timed (sub-record of the pad line)
    inverse = None
    if kind == "pad" and not KERNEL_ONLY:
        padded = ops.to_padded_tensor(buf, sz, meta, 0.0)
        inv = lambda: ops.from_padded_tensor(padded, sz, meta)
        for _ in range(3):
            inv()
        ims, ibest = timed_regions(inv, args.steps, world, device)
        ib = 2 * es * n_valid
        inverse = {"metric": "from_padded_tensor HBM GB/s", "value": all_sum(ib, world, device) / (ims * 1e-3) / 1e9, "unit": "GB/s",
                   "ms_per_step": ims, "best_ms": ibest, "algorithmic_bytes_per_gpu": ib,
                   "roofline": {"bound": "hbm", "achieved": ib / (ims * 1e-3) / 1e9, "peak": measured_peaks()["hbm_gbs"], "unit": "GB/s",
                                "frac": ib / (ims * 1e-3) / 1e9 / measured_peaks()["hbm_gbs"],
                                "traffic": None if SEQUENCE_LIMIT else ib * NCU_TRAFFIC_PER_ALG_BYTE["unpad"],
                                "traffic_source": NCU_TRAFFIC_SOURCE}}
        del padded

    # end to end: pinned host input -> device -> kernel -> pinned host output, every step
    e2e = None
    try:
        import psutil
        avail = psutil.virtual_memory().available
    except Exception:
        avail = 0
    out_elems = n_pad if kind == "pad" else n_valid
    in_elems = n_valid if kind == "pad" else n_pad
    need = es * (out_elems + in_elems)
    if world > 1:  # every rank takes the same branch: the smallest figure any rank saw decides
        import torch.distributed as dist
        t_av = torch.tensor([float(avail)], dtype=torch.float64, device=device)
        dist.all_reduce(t_av, op=dist.ReduceOp.MIN)
        avail = float(t_av.item())
    if KERNEL_ONLY:
        e2e = {"value": None, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0, "sample": "skipped: --kernel-only"}
    elif avail > 3 * need * max(world, 1):
        if kind == "unpad":
            del padded
        torch.cuda.empty_cache()
        bind_note = bind_to_gpu_numa_node(local) if world > 1 else "not bound (single rank)"
        h_in = torch.empty(in_elems, dtype=dtype).pin_memory()
        if kind == "pad":
            h_in.copy_(host)
        else:
            h_in.normal_()
        h_out = torch.empty(out_elems, dtype=dtype).pin_memory()
        d_in = torch.empty(in_elems, dtype=dtype, device=device)

        def serial_step():  # one stream: upload, kernel, download back to back
            d_in.copy_(h_in, non_blocking=True)
            if kind == "pad":
                r = ops.to_padded_tensor(d_in, sz, meta, 0.0)
            else:
                r = ops.from_padded_tensor(d_in.view(B, maxL, hidden), sz, meta)
            h_out.copy_(r.reshape(-1), non_blocking=True)

        def e2e_step():  # the host-buffer entry point of the package: the same three stages, pipelined over ranges
            if kind == "pad":
                nt.to_padded_tensor_host(h_in, sizes, 0.0, out=h_out.view(B, maxL, hidden), device=device)
            else:
                nt.from_padded_tensor_host(h_in.view(B, maxL, hidden), sizes, out=h_out, device=device)

        e2e_steps = max(2, min(args.steps, 5))
        serial_step()
        sms = timed_region(serial_step, e2e_steps, world, device)
        for _ in range(2):
            e2e_step()
        with ClockSampler(local) as clocks2:
            ems = timed_region(e2e_step, e2e_steps, world, device)
        # copy-only legs of the same buffers (what the host side allows with no kernel at all)
        h2d_ms = timed_region(lambda: d_in.copy_(h_in, non_blocking=True), 2, world, device) / 2
        d_out = torch.empty(min(out_elems, 1 << 30), dtype=dtype, device=device)
        d2h_ms = timed_region(lambda: h_out[:d_out.numel()].copy_(d_out, non_blocking=True), 2, world, device) / 2
        e2e = {"value": total_bytes / (ems / e2e_steps * 1e-3) / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": es * in_elems, "d2h_bytes_per_step": es * out_elems,
               "ms_per_step": ems / e2e_steps, "steps": e2e_steps, "sample": "full shard",
               "api": "%s_host (pinned host in/out, 8 ranges pipelined on 3 streams)" %
                      ("to_padded_tensor" if kind == "pad" else "from_padded_tensor"),
               "single_stream_value": total_bytes / (sms / e2e_steps * 1e-3) / 1e9,
               "copy_only": {"h2d_GBps_per_rank": es * in_elems / (h2d_ms * 1e-3) / 1e9,
                             "d2h_GBps_per_rank": es * d_out.numel() / (d2h_ms * 1e-3) / 1e9,
                             "note": "all ranks copy at the same time; max over ranks of the time"},
               "host_binding": bind_note}
        del d_out
        clocks.samples += clocks2.samples
        clocks.reasons |= clocks2.reasons
    else:
        e2e = {"value": None, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
               "sample": "skipped: host has %.1f GB available, needs %.1f GB pinned per rank" % (avail / 1e9, need / 1e9)}

    peaks = measured_peaks()
    line = None
    if rank == 0:
        cpu = {"skipped": "measured at N=1 only (the other ranks would compete for the host cores)"}
        if world == 1 and not KERNEL_ONLY:
            seqs = 512
            if kind == "pad":
                _, nbytes, fn = cpu_pad_sample(L, hidden, dtype, seqs)
            else:
                _, nbytes, fn = cpu_unpad_sample(L, hidden, dtype, seqs)
            torch.set_num_threads(os.cpu_count() or 1)
            t = time_cpu(fn, 1, 3)
            cpu = {"value": nbytes / t / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
                   "sample": "first %d sequences of the shard, median of 3, torch CPU ops of the reference's "
                             "CPU branch (constant_pad_nd + stack)" % seqs if kind == "pad" else
                             "first %d sequences of the shard, median of 3, reference CPU branch (mask + masked_select)" % seqs}
        elif KERNEL_ONLY:
            cpu = {"skipped": "--kernel-only"}
        line = {
            "metric": "to_padded_tensor HBM GB/s" if kind == "pad" else "from_padded_tensor HBM GB/s",
            "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": kernel_ms, "best_ms": best_ms, "timing": "median of 5 timed regions of `steps` steps",
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 (bit copy, u16)", "data": "synthetic",
            "config": {"workload": ("FIRST %d SEQUENCES ONLY of " % SEQUENCE_LIMIT if SEQUENCE_LIMIT else "") +
                                   "config2: %d bf16 sequences (L_i,1024), L_i=clip(round(lognormal(ln200,0.6)),1,1024) "
                                   "per GPU; %s" % (4096, "to_padded_tensor(padding=0)" if kind == "pad" else
                                                    "from_padded_tensor with known sizes"),
                       "batch_per_gpu": B, "tokens_per_gpu": T, "max_len": maxL, "hidden": hidden,
                       "algorithmic_bytes_per_gpu": alg_bytes, "token_imbalance": imb, "values": values_from,
                       "l2": "inputs+outputs (%.1f GB) far larger than the 126 MB L2" % (alg_bytes / 1e9)},
            "roofline": {"bound": "hbm", "achieved": alg_bytes / (kernel_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": alg_bytes / (kernel_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                         "frac_of_nominal_8000": alg_bytes / (kernel_ms * 1e-3) / 1e9 / 8000.0,
                         "peak_source": peaks["source"],
                         "traffic": None if SEQUENCE_LIMIT else alg_bytes * NCU_TRAFFIC_PER_ALG_BYTE[kind],
                         "traffic_source": NCU_TRAFFIC_SOURCE},
            "cpu_baseline": cpu,
            "e2e": e2e,
            "gpu_launches": 5 * args.steps,
            "clocks": clocks.summary(),
            "parity_roundtrip_bit_exact": parity_ok,
        }
        if inverse is not None:
            line["unpad"] = inverse
    return line


def bind_to_gpu_numa_node(local):
    """Pin this process's threads (and, through first touch, the pinned buffers it allocates next) to the CPUs NVML
    reports as local to the GPU.  Returns a note for the bench line.  Reading the affinity changes no GPU setting."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(local)
        n_words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, n_words)
        cpus = [w * 64 + b for w, word in enumerate(mask) for b in range(64) if (int(word) >> b) & 1]
        allowed = sorted(set(cpus) & set(os.sched_getaffinity(0)))
        if not allowed:
            return "no CPU of the GPU's affinity mask is available to this process"
        os.sched_setaffinity(0, allowed)
        torch.set_num_threads(max(1, min(len(allowed), 8)))
        return "threads bound to %d CPUs local to GPU %d (%d..%d)" % (len(allowed), local, allowed[0], allowed[-1])
    except Exception as e:  # NVML absent or affinity not permitted: measure unbound and say so
        return "unbound (%s)" % type(e).__name__


# ---------------------------------------------------------------------- reference arm
def _reference_budget_sequences(est_full_s, steps, warmup, full, fallback):
    """The whole configuration when `steps + warmup` passes of it fit in about three minutes of host time, else the
    stated sub-batch."""
    return full if est_full_s * (steps + warmup) <= 180.0 else fallback


def run_reference(args, kind, rank, world):
    """The reference's own CPU implementation of the path (oracle port) on the host cores; rank 0 only.  Imports
    nothing of the package but its pure-Python length generators, so no native library is loaded."""
    if rank != 0:
        return None
    torch.set_num_threads(os.cpu_count() or 1)
    if kind in ("mha", "encoder"):
        return run_reference_mha(args, world, encoder=(kind == "encoder"))
    L, _ = shard_lengths("pad", 1, 0)
    hidden, dtype = 1024, torch.bfloat16
    steps, warmup = max(1, args.steps), max(1, args.warmup)
    try:
        import psutil
        avail = psutil.virtual_memory().available
    except Exception:
        avail = 0
    # calibrate on 128 sequences, then take the whole configuration if time and host memory allow
    make = cpu_pad_sample if kind == "pad" else cpu_unpad_sample
    _, nb0, fn0 = make(L, hidden, dtype, 128)
    t0 = time_cpu(fn0, 1, 1)
    full_bytes = 2 * (int(L.sum()) * hidden + (int(L.numel()) * int(L.max()) * hidden if kind == "pad" else int(L.sum()) * hidden))
    est_full = t0 * full_bytes / nb0
    seqs = _reference_budget_sequences(est_full, steps, warmup, int(L.numel()), 512)
    if seqs == int(L.numel()) and avail < 4 * 2 * int(L.numel()) * int(L.max()) * hidden:
        seqs = 512  # the dense result, its per-sequence pieces and the stack do not fit in host memory
    _, nbytes, fn = make(L, hidden, dtype, seqs)
    metric = "to_padded_tensor HBM GB/s" if kind == "pad" else "from_padded_tensor HBM GB/s"
    for _ in range(warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    dt = (time.perf_counter() - t0) / steps
    v = nbytes / dt / 1e9
    cores = torch.get_num_threads()
    whole = seqs == int(L.numel())
    sample = ("each step = the whole configuration 2 (%d sequences, %.2f GB algorithmic)" if whole else
              "each step = the first %d sequences of configuration 2 (%.2f GB algorithmic)") % (seqs, nbytes / 1e9)
    return {"impl": "reference", "metric": metric, "value": v, "unit": "GB/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16 (bit copy, u16)", "data": "synthetic",
            "config": {"workload": "config2 on the host cores: " + sample, "whole_configuration": whole},
            "cpu_baseline": {"value": v, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def cpu_mha_sample(L, E, H, dtype, seqs):
    """The reference's generic (CPU-capable) MHA, nestedtensor/csrc/mha.cpp:18-69, on the first `seqs` sequences."""
    from oracle import ntref
    workloads = _pure_module("workloads")
    Ls = L[:seqs].tolist()
    g = torch.Generator().manual_seed(13)
    tensors = [torch.randn(l, E, generator=g).to(dtype) for l in Ls]
    w = workloads._mha_weights(g, E, dtype)
    d = E // H
    fn = lambda: ntref.min_mha(H, d, tensors, tensors, tensors, w["in_proj_weight"], w["in_proj_bias"], float(d) ** -0.5,
                               w["out_proj_weight"], w["out_proj_bias"])
    return sum(Ls), fn


def run_reference_mha(args, world, encoder=False):
    L, _ = shard_lengths("mha", 1, 0)
    E, H, dtype = 1024, 16, torch.bfloat16
    steps, warmup = max(1, args.steps), max(1, args.warmup)

    def make(seqs):
        if encoder:
            from oracle import ntref
            Ls = L[:seqs].tolist()
            g = torch.Generator().manual_seed(13)
            tensors = [torch.randn(l, E, generator=g).to(dtype) for l in Ls]
            params = _layer_params(_bert_large_layer(torch.float32, "cpu"))
            return sum(Ls), (lambda: ntref.encoder_layer(tensors, H, params, "gelu_tanh", False, 1e-5))
        return cpu_mha_sample(L, E, H, dtype, seqs)

    tok0, fn0 = make(16)
    t0 = time_cpu(fn0, 1, 1)
    est_full = t0 * float(L.sum()) / tok0
    seqs = _reference_budget_sequences(est_full, steps, warmup, int(L.numel()), 64)
    tokens, fn = make(seqs)
    for _ in range(warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    dt = (time.perf_counter() - t0) / steps
    v = tokens / dt
    whole = seqs == int(L.numel())
    sample = ("each step = the whole configuration 5 (%d sequences, %d tokens), per-sequence fp32 loop" if whole else
              "each step = the first %d sequences of configuration 5 (%d tokens), per-sequence fp32 loop") % (seqs, tokens)
    return {"impl": "reference", "metric": "varlen encoder layer valid tokens/s" if encoder else "varlen MHA valid tokens/s",
            "value": v, "unit": "tokens/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 inputs, fp32 math", "data": "synthetic",
            "config": {"workload": "config5 on the host cores: " + sample, "whole_configuration": whole},
            "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                             "sample": sample},
            "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def run_mha(args, rank, world, local, brief=False):
    """Configuration 5: BERT-large varlen self-attention forward (bf16, E=1024, 16 heads x 64).  `brief` (or
    --kernel-only) leaves out the end-to-end pass, the sustained loop and the CPU baseline."""
    import ctypes
    import nestedtensor_b200 as nt
    from nestedtensor_b200 import _ops, _cabi, workloads
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    E, H, d, dtype = 1024, 16, 64, torch.bfloat16
    L, imb = shard_lengths("mha", world, rank)
    B, T, maxL = int(L.numel()), int(L.sum()), int(L.max())
    sizes = torch.stack([L, torch.full_like(L, E)], 1).contiguous()
    flops = workloads.mha_flops(L, E)
    attn_flops = 4.0 * E * float((L.double() ** 2).sum())
    if world == 1 and not SEQUENCE_LIMIT:
        w5 = workloads.config5()
        assert torch.equal(w5.sizes[:, 0], L)
        host, w = w5.buffer, w5.weights
    else:
        host = host_values(T * E, dtype, 20245 + 1000 * (rank + 1))
        w = workloads._mha_weights(workloads._gen(5), E, dtype)
    wd = {k: v.to(device) for k, v in w.items()}
    x = nt.NestedTensor(host.to(device), sizes)
    ops = _ops.ops()
    buf, sz, meta = x._record()
    scaling = float(d) ** -0.5
    step = lambda: ops.bt_min_mha(H, d, 0.0, False, buf, sz, meta, wd["in_proj_weight"], wd["in_proj_bias"], scaling,
                                  wd["out_proj_weight"], wd["out_proj_bias"])
    steps = args.steps
    for _ in range(max(args.warmup, 3)):
        step()
    lib = _cabi.load()
    with ClockSampler(local) as clocks:
        step_ms, best_ms = timed_regions(step, steps, world, device)
        # The same three kernels through the C ABI with an event between them, inside a loop of whole steps: per-kernel
        # times that add up to the step (kernels timed alone, after the loop, run at other clocks and overstate it).
        qkv = torch.empty(T, 3 * E, dtype=dtype, device=device)
        attn_out = torch.empty(T, E, dtype=dtype, device=device)
        y = torch.empty(T, E, dtype=dtype, device=device)
        ws_bytes = lib.ntb200_varlen_attention_workspace_bytes(B, T, H, d, 2)
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=device)
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

        def cabi_step(events=None):
            if events is not None:
                events[0].record()
            lib.ntb200_gemm_bias(buf.data_ptr(), wd["in_proj_weight"].data_ptr(), wd["in_proj_bias"].data_ptr(),
                                 qkv.data_ptr(), T, 3 * E, E, 2, 0, stream)
            if events is not None:
                events[1].record()
            lib.ntb200_varlen_attention(qkv.data_ptr(), attn_out.data_ptr(), meta.data_ptr(), B, T, H, d, maxL, scaling, 2, 0,
                                        ws.data_ptr() if ws_bytes else None, ws_bytes, stream)
            if events is not None:
                events[2].record()
            lib.ntb200_gemm_bias(attn_out.data_ptr(), wd["out_proj_weight"].data_ptr(), wd["out_proj_bias"].data_ptr(),
                                 y.data_ptr(), T, E, E, 2, 0, stream)
            if events is not None:
                events[3].record()

        for _ in range(3):
            cabi_step()
        n_inst = max(steps, 10)
        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(n_inst)]
        torch.cuda.synchronize(device)
        for e in evs:
            cabi_step(e)
        torch.cuda.synchronize(device)
        seg = [sorted(e[k].elapsed_time(e[k + 1]) for e in evs) for k in range(3)]
        whole = sorted(e[0].elapsed_time(e[3]) for e in evs)
        med = lambda v: v[len(v) // 2]
        kernels_ms = {"qkv_gemm": med(seg[0]), "attention": med(seg[1]), "out_proj_gemm": med(seg[2]),
                      "sum": med(seg[0]) + med(seg[1]) + med(seg[2]), "instrumented_step": med(whole), "step": step_ms,
                      "how": "CUDA events between the three launches of %d back-to-back steps through the C ABI, median per segment; "
                             "attention includes its work-list kernel and the kernel of the sequences of at most 32 tokens" % n_inst}
    total_tokens = all_sum(T, world, device)
    value = total_tokens / (step_ms * 1e-3)
    flags = lib.ntb200_device_error_flags()

    brief = brief or KERNEL_ONLY
    peaks = measured_peaks()
    sustained = None
    e2e = None
    if not brief:
        # sustained: the step in a loop for >= 2 s, clocks sampled meanwhile (the 20-step regions above are bursts)
        n_sus = max(steps, int(2000.0 / step_ms) + 1)
        with ClockSampler(local) as sclk:
            sus_ms = timed_region(step, n_sus, world, device) / n_sus
        stf = flops / (sus_ms * 1e-3) / 1e12
        sustained = {"value": total_tokens / (sus_ms * 1e-3), "unit": "tokens/s", "ms_per_step": sus_ms, "steps": n_sus,
                     "seconds": sus_ms * n_sus * 1e-3, "step_tflops": stf, "frac_of_bf16_sustained": stf / peaks["bf16_tflops_sustained"],
                     "frac_of_bf16_burst": stf / peaks["bf16_tflops"], "clocks": sclk.summary()}
        clocks.reasons |= sclk.reasons

        bind_note = bind_to_gpu_numa_node(local) if world > 1 else "not bound (single rank)"
        h_in = torch.empty(T * E, dtype=dtype).pin_memory()
        h_in.copy_(host)
        h_out = torch.empty(T * E, dtype=dtype).pin_memory()
        d_in = torch.empty(T * E, dtype=dtype, device=device)

        def serial_step():  # one stream: upload, operator, download back to back
            d_in.copy_(h_in, non_blocking=True)
            r = ops.bt_min_mha(H, d, 0.0, False, d_in, sz, meta, wd["in_proj_weight"], wd["in_proj_bias"], scaling,
                               wd["out_proj_weight"], wd["out_proj_bias"])
            h_out.copy_(r, non_blocking=True)

        def e2e_step():  # the host-buffer entry point of the package: the same three stages, pipelined over ranges
            nt.multi_head_attention_host(h_in, sizes, H, wd["in_proj_weight"], wd["in_proj_bias"], wd["out_proj_weight"],
                                         wd["out_proj_bias"], scaling=scaling, out=h_out)

        e2e_steps = max(3, min(steps, 20))
        serial_step()
        sms = timed_region(serial_step, e2e_steps, world, device) / e2e_steps
        for _ in range(3):
            e2e_step()
        with ClockSampler(local) as clocks2:
            ems = timed_region(e2e_step, e2e_steps, world, device) / e2e_steps
        clocks.samples += clocks2.samples
        clocks.reasons |= clocks2.reasons
        e2e = {"value": total_tokens / (ems * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 2 * T * E,
               "d2h_bytes_per_step": 2 * T * E, "ms_per_step": ems, "steps": e2e_steps,
               "api": "multi_head_attention_host (pinned host in/out, 8 ranges pipelined on 3 streams)",
               "single_stream_value": total_tokens / (sms * 1e-3), "host_binding": bind_note}

    if rank != 0:
        return None
    tf = flops / (step_ms * 1e-3) / 1e12
    gemm_flops = 2.0 * T * 3 * E * E
    gtf = gemm_flops / (kernels_ms["qkv_gemm"] * 1e-3) / 1e12
    atf = attn_flops / (kernels_ms["attention"] * 1e-3) / 1e12
    line = {
        "metric": "varlen MHA valid tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps,
        "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "best_ms": best_ms,
        "timing": "median of 5 timed regions of `steps` steps", "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": ("FIRST %d SEQUENCES ONLY of " % SEQUENCE_LIMIT if SEQUENCE_LIMIT else "") +
                               "config5: BERT-large varlen self-attention forward, batch 1024 per GPU, 70% L~U[16,128] / "
                               "30% L~U[128,512], E=1024, 16 heads x 64, bf16",
                   "batch_per_gpu": B, "tokens_per_gpu": T, "max_len": maxL, "flops_per_gpu": flops,
                   "token_imbalance": imb,
                   "l2": "activations per step (x, qkv, attn, out = %.2f GB) exceed the 126 MB L2" % (12 * T * E / 1e9)},
        "step_tflops": tf, "step_frac_of_bf16_peak": tf / peaks["bf16_tflops"],
        "step_frac_of_bf16_sustained": tf / peaks["bf16_tflops_sustained"],
        "kernels_ms": kernels_ms,
        "attention_tflops_valid": atf, "attention_frac_of_bf16_peak": atf / peaks["bf16_tflops"],
        "roofline": {"bound": "tensor", "kernel": "gemm_bias_tcgen05_pair_kernel (QKV projection, M=%d N=3072 K=1024), timed inside the step" % T,
                     "achieved": gtf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": gtf / peaks["bf16_tflops"],
                     "frac_of_sustained": gtf / peaks["bf16_tflops_sustained"], "peak_source": peaks["source"],
                     "traffic": None if SEQUENCE_LIMIT else T * NCU_TRAFFIC_GEMM_BYTES_PER_TOKEN["mha"],
                     "traffic_source": NCU_TRAFFIC_SOURCE},
        "sustained": sustained,
        "e2e": e2e, "gpu_launches": 5 * 5 * steps, "clocks": clocks.summary(), "device_error_flags": flags,
    }
    if brief:
        line["cpu_baseline"] = {"skipped": "--kernel-only"}
    elif world > 1:
        line["cpu_baseline"] = {"skipped": "measured at N=1 only (the other ranks would compete for the host cores)"}
    else:
        torch.set_num_threads(os.cpu_count() or 1)
        tokens, fn = cpu_mha_sample(L, E, H, dtype, 64)
        t = time_cpu(fn, 1, 3)
        line["cpu_baseline"] = {"value": tokens / t, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                                "sample": "first 64 sequences (%d tokens), median of 3, per-sequence fp32 loop of the "
                                          "reference's generic MHA (nestedtensor/csrc/mha.cpp:18-69)" % tokens}
    return line


def _ref_cuda_lib():
    """oracle/_ref/libntref_cuda.so (the reference's own CUDA files compiled for sm_100a by oracle/build_ref.py), or None."""
    import ctypes
    path = os.path.join(ROOT, "oracle", "_ref", "libntref_cuda.so")
    if not os.path.exists(path):
        return None
    lib = ctypes.CDLL(path)
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.ntref_add_padding.restype = I
    lib.ntref_add_padding.argtypes = [P, P, F, P, P, I, P, I, I, P]
    lib.ntref_remove_padding.restype = I
    lib.ntref_remove_padding.argtypes = [P, P, P, P, P, I, I, I, P]
    if hasattr(lib, "ntref_softmax"):
        lib.ntref_softmax.restype = I
        lib.ntref_softmax.argtypes = [P, P, I, I, I, F, I, P]
    if hasattr(lib, "ntref_add_padding_mask"):
        lib.ntref_add_padding_mask.restype = I
        lib.ntref_add_padding_mask.argtypes = [P, P, P, P, I, I, I, I, P]
    return lib


def reference_kernel_times(sizes, buf, device, n, note=""):
    """The reference's own CUDA padding kernels on `buf` / `sizes` (a batch whose padded tensor has fewer than 2^31
    elements: the reference indexes with `int`), driven as its operators drive them: (L_i, E) batches are collapsed to
    one ragged dimension for the pad (masking.cpp:569-575, add_padding_1) and un-padded in two (remove_padding_2);
    (C, H_i, W_i) batches use add_padding_3 / remove_padding.  16-bit data goes through its half instantiation (a bit
    copy).  A secondary comparator beside the CPU baseline; None when the library is absent."""
    import ctypes
    lib = _ref_cuda_lib()
    B, dim = sizes.shape
    mx = sizes.max(0).values.tolist()
    npad = B
    for v in mx:
        npad *= v
    if lib is None or npad >= 2 ** 31 or buf.element_size() not in (2, 4) or dim < 2 or dim > 3:
        return None
    numel = sizes.prod(1)
    offsets = torch.zeros(B, dtype=torch.int64)
    offsets[1:] = numel.cumsum(0)[:-1]
    d_off = offsets.to(torch.int32).to(device)
    collapse = dim == 2 and bool((sizes[:, 1] == sizes[0, 1]).all())
    pad_sizes = numel[:, None] if collapse else sizes
    pad_dim = pad_sizes.shape[1]
    pad_mx = pad_sizes.max(0).values.tolist()
    d_pad_sizes = pad_sizes.to(torch.int32).contiguous().to(device)
    d_sizes = sizes.to(torch.int32).contiguous().to(device)
    out = torch.empty([B] + mx, dtype=buf.dtype, device=device)
    back = torch.empty_like(buf)
    out_sizes = (ctypes.c_int64 * (pad_dim + 1))(*([B] + pad_mx))
    d_padded_sizes = torch.tensor([B] + mx, dtype=torch.int32, device=device)
    code = 0 if buf.element_size() == 4 else 1
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    pad = lambda: lib.ntref_add_padding(buf.data_ptr(), out.data_ptr(), 0.0, d_off.data_ptr(), d_pad_sizes.data_ptr(), pad_dim, out_sizes, B,
                                        code, stream)
    unpad = lambda: lib.ntref_remove_padding(out.data_ptr(), back.data_ptr(), d_off.data_ptr(), d_padded_sizes.data_ptr(), d_sizes.data_ptr(),
                                             dim, B, code, stream)
    es, nv = buf.element_size(), buf.numel()
    res = {"what": "%s / %s of the reference, grid (B,16) x 256 threads, same inputs, CUDA events%s" %
                   ("add_padding_%d" % pad_dim, "remove_padding_2" if dim == 2 else "remove_padding", note)}
    for name, fn, nbytes in (("to_padded_tensor", pad, es * (nv + npad)), ("from_padded_tensor", unpad, 2 * es * nv)):
        for _ in range(3):
            assert fn() == 0
        ms, _ = timed_regions(fn, n, 1, device)
        res[name] = {"ms": ms, "GB/s": nbytes / ms / 1e6}
    iv = torch.int32 if es == 4 else torch.int16
    res["round_trip_bit_exact"] = bool(torch.equal(back.view(iv), buf.view(iv)))
    return res


def reference_attention_helper_times(lengths, E, H, dtype, device, n):
    """The reference's fused data + mask kernel (add_padding_mask: one thread per sequence) and its masked softmax on
    padded scores [B, H, maxL, maxL], at the lengths of a configuration: what bt_min_mha runs around its batched GEMMs
    (cuda/mha.cpp:57-93).  This library has no counterpart on its MHA path (nothing is padded and no score matrix is
    stored); the times show what that path avoids."""
    import ctypes
    lib = _ref_cuda_lib()
    if lib is None or not hasattr(lib, "ntref_softmax") or not hasattr(lib, "ntref_add_padding_mask"):
        return None
    B, maxL, T = len(lengths), int(max(lengths)), int(sum(lengths))
    if B * H * maxL * maxL >= 2 ** 31 or maxL > 1024:
        return None
    code = 0 if dtype == torch.float32 else 1
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    x = torch.randn(T, E, device=device).to(dtype)
    off = torch.zeros(B + 1, dtype=torch.int32)
    off[1:] = torch.tensor(lengths, dtype=torch.int64).cumsum(0).to(torch.int32)
    d_off = off.to(device)
    padded = torch.zeros(B, maxL, E, dtype=dtype, device=device)
    mask = torch.zeros(B, maxL, dtype=torch.int32, device=device)
    f_mask = lambda: lib.ntref_add_padding_mask(x.data_ptr(), padded.data_ptr(), mask.data_ptr(), d_off.data_ptr(), B, maxL, E, code, stream)
    scores = torch.randn(B, H, maxL, maxL, device=device).to(dtype)
    valid = torch.arange(maxL, device=device)[None, :] < torch.tensor(lengths, device=device)[:, None]
    amask = (valid[:, :, None] & valid[:, None, :]).to(dtype).contiguous()
    f_soft = lambda: lib.ntref_softmax(scores.data_ptr(), amask.data_ptr(), B, H, maxL, 0.125, code, stream)
    res = {"what": "add_padding_mask (grid B x 1 thread) and softmax_kernel_kernelLauncher of the reference at these lengths"}
    for name, fn, reps in (("add_padding_mask", f_mask, min(n, 5)), ("masked_softmax", f_soft, n)):
        for _ in range(2):
            assert fn() == 0
        ms, _ = timed_regions(fn, reps, 1, device, regions=3)
        res[name] = {"ms": ms}
    res["masked_softmax"]["score_bytes"] = scores.numel() * scores.element_size()
    return res


def run_small_configs(args, local):
    """Configurations 3 and 4, device-timed on one GPU (sub-records of the default line): 4-D to_padded_tensor /
    to_tensor_mask / from_padded_tensor on 32 fp32 images, and the BERT-base fp16 MHA step."""
    import nestedtensor_b200 as nt
    from nestedtensor_b200 import _ops, workloads
    device = torch.device("cuda", local)
    ops = _ops.ops()
    peaks = measured_peaks()
    n = max(args.steps, 10)

    def timed(fn):
        for _ in range(3):
            fn()
        return timed_regions(fn, n, 1, device)

    def hbm(ms, nbytes, fn=None):
        g = nbytes / ms / 1e6
        r = {"ms": ms, "GB/s": g, "frac_hbm_measured": g / peaks["hbm_gbs"], "algorithmic_bytes": nbytes}
        gm = graph_ms(fn, n, device) if fn is not None else None
        if gm is not None:  # the same launches replayed from one CUDA graph: no host launch cost between them
            r["graph_ms"] = gm
            r["graph_frac_hbm_measured"] = nbytes / gm / 1e6 / peaks["hbm_gbs"]
        return r

    w = workloads.config3()
    a = nt.NestedTensor(w.buffer.to(device), w.sizes)
    b, sz, meta = a._record()
    nv = w.buffer.numel()
    padded = ops.to_padded_tensor(b, sz, meta, 0.0)
    npad = padded.numel()
    f_pad = lambda: ops.to_padded_tensor(b, sz, meta, 0.0)
    f_mask = lambda: ops.to_tensor_mask(b, sz, meta, None)
    f_unpad = lambda: ops.from_padded_tensor(padded, sz, meta)
    f_scan = lambda: ops.sizes_from_padded(padded, 0.0)
    c3 = {"workload": "config3: 32 fp32 images (3, H_i, W_i), H_i, W_i ~ U[400,1024]",
          "note": "0.6 GB per call; about 1 GB moved in and out: above the 126 MB L2, but part of a call's data is served from it",
          "to_padded_tensor": hbm(timed(f_pad)[0], 4 * (nv + npad), f_pad),
          "to_tensor_mask": hbm(timed(f_mask)[0], 4 * (nv + npad) + npad, f_mask),
          "from_padded_tensor": hbm(timed(f_unpad)[0], 8 * nv, f_unpad),
          "sizes_from_padded": hbm(timed(f_scan)[0], 4 * npad, f_scan)}
    ref = reference_kernel_times(w.sizes, b, device, n)
    if ref is not None:
        c3["reference_kernels_sm100a"] = ref
    del padded, a, b
    w = workloads.config4()
    a = nt.NestedTensor(w.buffer.to(device), w.sizes)
    b, sz, meta = a._record()
    wd = {k: v.to(device) for k, v in w.weights.items()}
    E, H = 768, 12
    d = E // H
    fn = lambda: ops.bt_min_mha(H, d, 0.0, False, b, sz, meta, wd["in_proj_weight"], wd["in_proj_bias"], float(d) ** -0.5,
                                wd["out_proj_weight"], wd["out_proj_bias"])
    ms, best = timed(fn)
    Ls = w.sizes[:, 0]
    fl = workloads.mha_flops(Ls, E)
    c4 = {"workload": "config4: BERT-base varlen self-attention forward, 128 sequences L~U[32,512], E=768, 12 heads x 64, fp16",
          "ms_per_step": ms, "best_ms": best, "tokens": int(Ls.sum()), "tokens_per_s": float(Ls.sum()) / (ms * 1e-3),
          "step_tflops": fl / ms / 1e9, "step_frac_of_bf16_peak": fl / ms / 1e9 / peaks["bf16_tflops"],
          "note": "0.198 TFLOP per step: a step lasts about 0.3 ms, short of filling the GPU for long"}
    ref = reference_kernel_times(w.sizes, b, device, n)
    if ref is not None:  # the same (L_i, 768) fp16 batch through the reference's padding kernels and this library's
        ours = {}
        padded4 = ops.to_padded_tensor(b, sz, meta, 0.0)
        for name, fn in (("to_padded_tensor", lambda: ops.to_padded_tensor(b, sz, meta, 0.0)),
                         ("from_padded_tensor", lambda: ops.from_padded_tensor(padded4, sz, meta))):
            ours[name] = {"ms": timed(fn)[0]}
        ref["this_library_same_batch"] = ours
        helpers = reference_attention_helper_times([int(v) for v in Ls], E, H, torch.float16, device, n)
        if helpers is not None:
            ref["attention_helpers"] = helpers
        c4["reference_kernels_sm100a"] = ref
        del padded4
    del a, b
    torch.cuda.empty_cache()
    # configuration 2 is beyond the reference's int indexing; its first 2047 sequences are not (2047 * 1024 * 1024 < 2^31)
    w2 = workloads.config2(with_values=False)
    sz2 = w2.sizes[:2047].contiguous()
    buf2 = torch.randn(int(sz2.prod(1).sum()), device=device).to(torch.bfloat16)
    c2 = reference_kernel_times(sz2, buf2, device, min(n, 10), note="; first 2047 sequences of configuration 2 (bf16 as a 16-bit copy)")
    out = {"config3": c3, "config4": c4}
    if c2 is not None:
        a2 = nt.NestedTensor(buf2, sz2)
        b2, s2, m2 = a2._record()
        p2 = ops.to_padded_tensor(b2, s2, m2, 0.0)
        c2["this_library_same_batch"] = {"to_padded_tensor": {"ms": timed(lambda: ops.to_padded_tensor(b2, s2, m2, 0.0))[0]},
                                         "from_padded_tensor": {"ms": timed(lambda: ops.from_padded_tensor(p2, s2, m2))[0]}}
        out["config2_subbatch_reference_kernels_sm100a"] = c2
        del a2, b2, p2
    del buf2
    torch.cuda.empty_cache()
    out["next_rows"] = run_next_rows(args, local, peaks, n)
    return out


def run_next_rows(args, local, peaks, n):
    """The rows beside the path (packed LayerNorm, projection with residual, feed-forward up-projection with GELU, ragged
    image transposes) at the configuration-5 token count / a stride-8 feature-map batch, device-timed on one GPU:
    a sub-record of the default line."""
    import nestedtensor_b200 as nt
    from nestedtensor_b200 import _ops
    device = torch.device("cuda", local)
    ops = _ops.ops()
    T, E = 151792, 1024
    g = torch.Generator().manual_seed(20250)
    x = torch.randn(T, E, generator=g).to(torch.bfloat16).to(device)
    res = torch.randn(T, E, generator=g).to(torch.bfloat16).to(device)
    w = (torch.randn(E, E, generator=g) * E ** -0.5).to(torch.bfloat16).to(device)
    w_up = (torch.randn(4 * E, E, generator=g) * E ** -0.5).to(torch.bfloat16).to(device)
    b = torch.randn(E, generator=g).to(torch.bfloat16).to(device)
    b_up = torch.randn(4 * E, generator=g).to(torch.bfloat16).to(device)
    gamma, beta = torch.ones(E, dtype=torch.bfloat16, device=device), torch.zeros(E, dtype=torch.bfloat16, device=device)

    def timed(fn, settle=False):
        """(median ms per call, median SM MHz during the regions).  `settle`: idle for a quarter of a second first, so
        that a row bound by instruction issue or latency is not measured at the clock the power governor still holds
        from the tensor-core work before it (the clock is reported either way)."""
        for _ in range(3):
            fn()
        torch.cuda.synchronize(device)
        if settle:
            time.sleep(0.25)
        with ClockSampler(local, period_s=0.005) as cs:
            ms = timed_regions(fn, n, 1, device)[0]
        return ms, cs.summary().get("sm_mhz")

    def hbm_row(ms, mhz, nbytes):
        return {"ms": ms, "GB/s": nbytes / ms / 1e6, "frac_hbm_measured": nbytes / ms / 1e6 / peaks["hbm_gbs"], "sm_mhz": mhz}

    out = {"workload": "T = 151 792 packed tokens (configuration 5), E = 1024, bf16; transposes: 32 fp16 maps (256, 100-168, 100-168), and the 32 fp32 RGB images of configuration 3",
           "note": "memory-bound rows first, each after 0.25 s of idle; the SM clock seen during each row is beside it"}
    gi = torch.Generator().manual_seed(20248)
    hw = torch.randint(100, 169, (32, 2), generator=gi)
    isz = torch.cat([torch.full((32, 1), 256), hw], 1).contiguous()
    nimg = int((isz[:, 0] * isz[:, 1] * isz[:, 2]).sum())
    img = nt.NestedTensor(torch.randn(nimg, device=device).to(torch.float16), isz)
    nhwc = nt.nn.transpose_nchw_nhwc(img)
    out["transpose_nchw_nhwc"] = hbm_row(*timed(lambda: nt.nn.transpose_nchw_nhwc(img), True), 4.0 * nimg)
    out["transpose_nhwc_nchw"] = hbm_row(*timed(lambda: nt.nn.transpose_nhwc_nchw(nhwc), True), 4.0 * nimg)
    del img, nhwc
    # the images of configuration 3 themselves (32 fp32 RGB images, 400..1024 pixels a side): the small-channel kernel
    from nestedtensor_b200 import workloads as _workloads
    rgb = _workloads.config3()
    rimg = nt.NestedTensor(rgb.buffer.to(device), rgb.sizes)
    rnhwc = nt.nn.transpose_nchw_nhwc(rimg)
    nrgb = int(rimg._buffer.numel())
    out["transpose_rgb_nchw_nhwc"] = hbm_row(*timed(lambda: nt.nn.transpose_nchw_nhwc(rimg), True), 8.0 * nrgb)
    out["transpose_rgb_nhwc_nchw"] = hbm_row(*timed(lambda: nt.nn.transpose_nhwc_nchw(rnhwc), True), 8.0 * nrgb)
    del rimg, rnhwc, rgb
    out["layer_norm"] = hbm_row(*timed(lambda: ops.add_bias_residual_layer_norm(x, None, None, gamma, beta, 1e-5), True), 4.0 * T * E)
    for name, fn, fl in (("out_proj_bias_residual", lambda: ops.packed_linear(x, w, b, 0, res), 2.0 * T * E * E),
                         ("out_proj_bias", lambda: ops.packed_linear(x, w, b, 0, None), 2.0 * T * E * E),
                         ("ffn_up_bias_gelu", lambda: ops.packed_linear(x, w_up, b_up, 1, None), 8.0 * T * E * E)):
        ms, mhz = timed(fn)
        out[name] = {"ms": ms, "TFLOP/s": fl / ms / 1e9, "frac_bf16_burst": fl / ms / 1e9 / peaks["bf16_tflops"], "sm_mhz": mhz}
    return out


def run_strong(args, rank, world, local):
    """Strong scaling of the FIXED configuration lists: configuration 2 (4096 sequences, to_padded_tensor), 5 (1024
    sequences, MHA) and 4 (128 sequences, MHA) cut into `world` contiguous token-balanced shards, no collective on the
    data path.  Rank 0 also runs the whole list alone (the other ranks wait), which gives the one-GPU time and the
    result the shard outputs are compared with after an NCCL all-gather outside the timed region."""
    import torch.distributed as dist
    import nestedtensor_b200 as nt
    from nestedtensor_b200 import _ops, workloads, sharding
    device = torch.device("cuda", local)
    ops = _ops.ops()
    n = max(3, min(args.steps, 20))
    out = {}

    def one(name, wl, kind):
        Ls = wl.sizes[:, 0].tolist()
        parts = sharding.token_balanced_partition(Ls, world)
        a, b = parts[rank]
        sub = wl.slice(a, b)
        E = int(wl.sizes[0, 1])
        if kind == "mha":
            H = wl.num_heads
            d = E // H
            wd = {k: v.to(device) for k, v in wl.weights.items()}
            run = lambda x: ops.bt_min_mha(H, d, 0.0, False, *x._record(), wd["in_proj_weight"], wd["in_proj_bias"], float(d) ** -0.5,
                                           wd["out_proj_weight"], wd["out_proj_bias"])
            work = lambda lens: sum(8.0 * E * E * l + 4.0 * E * l * l for l in lens)
        else:
            run = lambda x: ops.to_padded_tensor(*x._record(), 0.0)
            work = lambda lens: float(sum(lens)) if lens else 0.0
        have = b > a
        xs = nt.NestedTensor(sub.buffer.to(device), sub.sizes) if have else None
        shard_fn = (lambda: run(xs)) if have else (lambda: None)
        for _ in range(3):
            shard_fn()
        t_n = timed_region(shard_fn, n, world, device) / n  # max over ranks
        res = run(xs) if have else torch.empty(0, dtype=wl.dtype, device=device)
        # one GPU, whole list (rank 0 alone; the others wait at the barrier inside the next collective)
        t_1 = torch.zeros(1, dtype=torch.float64, device=device)
        full = None
        if rank == 0:
            xf = nt.NestedTensor(wl.buffer.to(device), wl.sizes)
            for _ in range(3):
                run(xf)
            t_1[0] = timed_region(lambda: run(xf), n, 1, device) / n
            full = run(xf)
        dist.broadcast(t_1, 0)
        # verification, outside every timed region: all-gather the shard outputs over NCCL, compare on rank 0
        if kind == "mha":
            gathered, gsz = sharding.gather_ragged(res.reshape(-1), sub.sizes if have else torch.zeros((0, 2), dtype=torch.int64))
            ok, err = None, None
            if rank == 0:
                err = float((gathered.float() - full.reshape(-1).float()).abs().max())
                ok = bool(torch.equal(gsz, wl.sizes)) and err <= 2e-2
        else:
            shape = torch.tensor([list(res.shape)], dtype=torch.int64) if have else torch.zeros((0, 3), dtype=torch.int64)
            gathered, gsz = sharding.gather_ragged(res.reshape(-1), shape)
            ok, err = None, None
            if rank == 0:
                ok, off, row = True, 0, 0
                for r_b, r_l, r_e in gsz.tolist():
                    piece = gathered[off:off + r_b * r_l * r_e].view(r_b, r_l, r_e)
                    ref = full[row:row + r_b]
                    ok = ok and bool(torch.equal(piece.view(torch.int16), ref[:, :r_l].view(torch.int16)))
                    ok = ok and int(ref[:, r_l:].view(torch.int16).count_nonzero()) == 0
                    off += r_b * r_l * r_e
                    row += r_b
                ok = ok and row == wl.batch
                err = 0.0 if ok else None
        del gathered
        toks = [sum(Ls[x:y]) for x, y in parts]
        wk = [work(Ls[x:y]) for x, y in parts]
        t1 = float(t_1.item())
        out[name] = {"sequences": wl.batch, "tokens": int(sum(Ls)), "ms_1gpu": t1, "ms_%dgpu" % world: t_n,
                     "tokens_per_s": float(sum(Ls)) / (t_n * 1e-3), "speedup": t1 / t_n, "efficiency": t1 / (t_n * world),
                     "token_imbalance": max(toks) / (sum(toks) / world), "work_imbalance": max(wk) / (sum(wk) / world),
                     "sequences_per_rank": [y - x for x, y in parts], "verified": ok, "max_abs_vs_1gpu": err,
                     "verification": "shard outputs all-gathered over NCCL (sharding.gather_ragged), compared on rank 0 with "
                                     "the one-GPU result of the whole list" + (" (max-abs <= 2e-2)" if kind == "mha" else " (bit-exact)")}
        torch.cuda.empty_cache()

    one("config2_pad", workloads.config2(), "pad")
    one("config5_mha", workloads.config5(), "mha")
    one("config4_mha", workloads.config4(), "mha")
    eff = [v["efficiency"] for v in out.values()]
    out["efficiency"] = out["config5_mha"]["efficiency"]
    out["verified"] = all(v["verified"] for k, v in out.items() if isinstance(v, dict)) if rank == 0 else None
    out["note"] = ("fixed lists, contiguous token-balanced shards, no collective on the data path; efficiency = "
                   "t(1 GPU) / (N * t(N GPUs, slowest rank)); `efficiency` at the top is configuration 5's")
    return out


def run_kernels(args, local):
    """Every operator of the path at the configuration that exercises it, CUDA-event timed on one GPU:
    algorithmic bytes (copies, masks) or FLOPs (MHA) per call divided by the mean call time."""
    import nestedtensor_b200 as nt
    from nestedtensor_b200 import _ops, workloads
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    ops = _ops.ops()
    peaks = measured_peaks()
    rows = []

    def timed(fn, n):
        for _ in range(3):
            fn()
        ms = timed_region(fn, n, 1, device) / n
        return ms

    only = args.only

    def add(name, config, ms, nbytes=None, flops=None, graph_fn=None):
        r = {"op": name, "config": config, "ms": ms}
        if nbytes is not None:
            r["GB/s"] = nbytes / ms / 1e6
            r["frac_hbm_measured"] = r["GB/s"] / peaks["hbm_gbs"]
            gm = graph_ms(graph_fn, n, device) if graph_fn is not None else None
            if gm is not None:
                r["graph_ms"] = gm
                r["graph_frac_hbm_measured"] = nbytes / gm / 1e6 / peaks["hbm_gbs"]
        if flops is not None:
            r["TFLOP/s"] = flops / ms / 1e9
            r["frac_bf16_burst"] = r["TFLOP/s"] / peaks["bf16_tflops"]
        rows.append(r)

    n = max(args.steps, 5)

    def image_path():
        # image-shaped path: 32 fp16 feature maps (256, H_i, W_i), H_i, W_i in [100, 168] (a stride-8 backbone level)
        gi = torch.Generator().manual_seed(20248)
        hw = torch.randint(100, 169, (32, 2), generator=gi)
        isz = torch.cat([torch.full((32, 1), 256), hw], 1).contiguous()
        nimg = int((isz[:, 0] * isz[:, 1] * isz[:, 2]).sum())
        img = nt.NestedTensor(torch.randn(nimg, device=device).to(torch.float16), isz)
        add("transpose_nchw_nhwc", "32 x (256, 100-168, 100-168) fp16", timed(lambda: nt.nn.transpose_nchw_nhwc(img), n), 4 * nimg)
        nhwc = nt.nn.transpose_nchw_nhwc(img)
        add("transpose_nhwc_nchw", "same batch", timed(lambda: nt.nn.transpose_nhwc_nchw(nhwc), n), 4 * nimg)
        w11 = (torch.randn(256, 256, 1, 1, device=device) * 0.05).to(torch.float16)
        add("conv2d 1x1 (transpose + packed GEMM + transpose)", "same batch, 256 -> 256 channels",
            timed(lambda: nt.nn.conv2d(img, w11), n), None, 2.0 * (nimg // 256) * 256 * 256)
        del img, nhwc

    def config3_group():
        es = 4
        # configuration 3: 32 fp32 images (3, H_i, W_i)
        w = workloads.config3()
        a = nt.NestedTensor(w.buffer.to(device), w.sizes)
        b, sz, meta = a._record()
        nv = w.buffer.numel()
        padded = ops.to_padded_tensor(b, sz, meta, 0.0)
        npad = padded.numel()
        f_pad = lambda: ops.to_padded_tensor(b, sz, meta, 0.0)
        f_mask = lambda: ops.to_tensor_mask(b, sz, meta, None)
        f_unpad = lambda: ops.from_padded_tensor(padded, sz, meta)
        f_scan = lambda: ops.sizes_from_padded(padded, 0.0)
        add("to_padded_tensor (4-D)", "c3", timed(f_pad, n), es * (nv + npad), graph_fn=f_pad)
        add("to_tensor_mask (4-D uint8 mask)", "c3", timed(f_mask, n), es * (nv + npad) + npad, graph_fn=f_mask)
        add("to_mask(mask_dim=3)", "c3", timed(lambda: ops.to_mask(sz, meta, 3), n), None)
        add("from_padded_tensor (4-D)", "c3", timed(f_unpad, n), 2 * es * nv, graph_fn=f_unpad)
        add("sizes_from_padded (scan)", "c3", timed(f_scan, n), es * npad, graph_fn=f_scan)
        del padded
        add("transpose_nchw_nhwc (3 channels)", "c3", timed(lambda: nt.nn.transpose_nchw_nhwc(a), n), 2 * es * nv)
        a_nhwc = nt.nn.transpose_nchw_nhwc(a)
        add("transpose_nhwc_nchw (3 channels)", "c3", timed(lambda: nt.nn.transpose_nhwc_nchw(a_nhwc), n), 2 * es * nv)
        del a_nhwc

    if only in ("transpose", "c3"):
        image_path() if only == "transpose" else config3_group()
        from nestedtensor_b200 import _cabi
        return {"metric": "per-operator timings (--only %s)" % only, "unit": "ms", "n_gpus": 1, "steps": n, "data": "synthetic",
                "peaks": peaks, "rows": rows, "device_error_flags": _cabi.load().ntb200_device_error_flags()}
    # configuration 1: 64 fp32 (L_i, 256)
    w = workloads.config1()
    a = nt.NestedTensor(w.buffer.to(device), w.sizes)
    b, sz, meta = a._record()
    es, nv = 4, w.buffer.numel()
    padded = ops.to_padded_tensor(b, sz, meta, 0.0)
    npad = padded.numel()
    add("to_padded_tensor", "c1", timed(lambda: ops.to_padded_tensor(b, sz, meta, 0.0), n), es * (nv + npad))
    add("to_tensor_mask(mask_dim=2)", "c1", timed(lambda: ops.to_tensor_mask(b, sz, meta, 2), n), es * (nv + npad) + npad // 256)
    add("from_padded_tensor", "c1", timed(lambda: ops.from_padded_tensor(padded, sz, meta), n), 2 * es * nv)
    add("nested_tensor_from_padded_tensor", "c1 (includes the one host sync of the API)",
        timed(lambda: nt.nested_tensor_from_padded_tensor(padded, padding=0), n), es * (npad + nv))
    config3_group()
    # configuration 2: 4096 bf16 (L_i, 1024)
    L, _ = shard_lengths("pad", 1, 0)
    sizes = torch.stack([L, torch.full_like(L, 1024)], 1).contiguous()
    nv = int(L.sum()) * 1024
    buf = torch.randn(nv // 2, device=device).to(torch.bfloat16).repeat(2)[:nv].contiguous()
    a = nt.NestedTensor(buf, sizes)
    b, sz, meta = a._record()
    padded = ops.to_padded_tensor(b, sz, meta, 0.0)
    npad = padded.numel()
    add("to_padded_tensor", "c2", timed(lambda: ops.to_padded_tensor(b, sz, meta, 0.0), n), 2 * (nv + npad))
    add("from_padded_tensor", "c2", timed(lambda: ops.from_padded_tensor(padded, sz, meta), n), 4 * nv)
    add("to_mask(mask_dim=2)", "c2", timed(lambda: ops.to_mask(sz, meta, 2), n), npad // 1024)
    add("sizes_from_padded (scan)", "c2", timed(lambda: ops.sizes_from_padded(padded, 0.0), n), 2 * npad)
    d_sizes = sizes.to(device)
    add("meta_from_device_sizes (offsets scan)", "c2", timed(lambda: ops.meta_from_device_sizes(d_sizes), n), None)
    del padded, buf, a
    torch.cuda.empty_cache()
    # construction of configuration 2 from 4096 separately allocated device tensors, and a packed embedding lookup
    parts = list(torch.split(b, (sz[:, 0] * sz[:, 1]).tolist()))
    parts = [p.clone() for p in parts]  # separate allocations, as a data loader would hand them over
    shaped = [p.view(int(l), 1024) for p, l in zip(parts, sz[:, 0].tolist())]
    add("nested_tensor(list of device tensors)", "c2 (one gather kernel + one pinned table copy)",
        timed(lambda: ops.pack_list(shaped), n), 4 * nv)
    del parts, shaped
    torch.cuda.empty_cache()
    c5 = workloads.config5()
    T5 = int(c5.sizes[:, 0].sum())
    table = torch.randn(30522, 1024, device=device).to(torch.bfloat16)  # BERT vocabulary x hidden
    idx = torch.randint(0, 30522, (T5,), device=device)
    isz = c5.sizes[:, :1].contiguous()
    from nestedtensor_b200.nested import build_meta
    imeta = build_meta(isz, device)
    add("embedding (packed gather)", "c5 tokens, 30522 x 1024 bf16 table",
        timed(lambda: ops.embedding(table, idx, isz, imeta), n), 2 * 2 * T5 * 1024 + 8 * T5)
    del table, idx
    # configurations 4 and 5: MHA
    for name, wl, dtype, E, H in (("c4", workloads.config4(), torch.float16, 768, 12),
                                  ("c5", workloads.config5(), torch.bfloat16, 1024, 16)):
        a = nt.NestedTensor(wl.buffer.to(device), wl.sizes)
        b, sz, meta = a._record()
        wd = {k: v.to(device) for k, v in wl.weights.items()}
        d = E // H
        fn = lambda: ops.bt_min_mha(H, d, 0.0, False, b, sz, meta, wd["in_proj_weight"], wd["in_proj_bias"], float(d) ** -0.5,
                                    wd["out_proj_weight"], wd["out_proj_bias"])
        ms = timed(fn, n)
        Ls = wl.sizes[:, 0]
        r_flops = workloads.mha_flops(Ls, E)
        add("bt_min_mha", name, ms, None, r_flops)
        rows[-1]["tokens/s"] = float(Ls.sum()) / (ms * 1e-3)
        T = int(Ls.sum())
        bi = lambda: ops.token_index(meta[:wl.batch + 1] // E, T)
        add("token_index", name, timed(bi, n), None)
    # cross-attention of a DETR-style decoder: 100 object queries per image over a ragged memory of 400-1200 tokens
    g = torch.Generator().manual_seed(20247)
    lk = torch.randint(400, 1201, (32,), generator=g)
    for E, H, dtype in ((256, 8, torch.float16), (512, 8, torch.bfloat16)):
        qn = nt.NestedTensor(torch.randn(32 * 100 * E, device=device).to(dtype), torch.tensor([[100, E]] * 32))
        kn = nt.NestedTensor(torch.randn(int(lk.sum()) * E, device=device).to(dtype), torch.stack([lk, torch.full_like(lk, E)], 1))
        mha = torch.nn.MultiheadAttention(E, H).eval().to(dtype).to(device)
        with torch.no_grad():
            fn = lambda: mha(qn, kn, kn, need_weights=False)
            ms = timed(fn, n)
        fl = 4.0 * E * 100 * float(lk.sum()) + 2.0 * E * E * (2 * 3200 + 2 * float(lk.sum()))
        add("MultiheadAttention(query != key)", "DETR-like 32 x (100 queries, 400-1200 keys), E=%d, %d heads x %d" % (E, H, E // H),
            ms, None, fl)
    image_path()
    from nestedtensor_b200 import _cabi
    return {"metric": "per-operator timings", "unit": "ms", "n_gpus": 1, "steps": n, "data": "synthetic",
            "peaks": peaks, "rows": rows, "device_error_flags": _cabi.load().ntb200_device_error_flags()}


# ------------------------------------------------------------------- encoder layer (next row)
def _bert_large_layer(dtype, device):
    torch.manual_seed(20246)
    layer = torch.nn.TransformerEncoderLayer(1024, 16, dim_feedforward=4096, dropout=0.0,
                                             activation=torch.nn.GELU(approximate="tanh"))
    return layer.eval().to(dtype).to(device)


def _layer_params(layer):
    p = {"in_proj_weight": layer.self_attn.in_proj_weight, "in_proj_bias": layer.self_attn.in_proj_bias,
         "out_proj_weight": layer.self_attn.out_proj.weight, "out_proj_bias": layer.self_attn.out_proj.bias,
         "linear1_weight": layer.linear1.weight, "linear1_bias": layer.linear1.bias, "linear2_weight": layer.linear2.weight,
         "linear2_bias": layer.linear2.bias, "norm1_weight": layer.norm1.weight, "norm1_bias": layer.norm1.bias,
         "norm2_weight": layer.norm2.weight, "norm2_bias": layer.norm2.bias}
    return {k: v.detach().float().cpu() for k, v in p.items()}


def run_encoder(args, rank, world, local):
    """Configuration 5 through one BERT-large encoder layer (E=1024, 16 heads x 64, FFN 4096, tanh GELU, post-norm,
    bf16) on packed tokens: the row after MHA in the scope table."""
    import ctypes
    import nestedtensor_b200 as nt
    from nestedtensor_b200 import _cabi
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    E, H, F, dtype = 1024, 16, 4096, torch.bfloat16
    L, imb = shard_lengths("mha", world, rank)
    B, T, maxL = int(L.numel()), int(L.sum()), int(L.max())
    sizes = torch.stack([L, torch.full_like(L, E)], 1).contiguous()
    attn_flops = 4.0 * E * float((L.double() ** 2).sum())
    gemm_flops = 2.0 * T * E * (3 * E + E + 2 * F)
    flops = attn_flops + gemm_flops
    host = host_values(T * E, dtype, 20246 + rank)
    layer = _bert_large_layer(dtype, device)
    x = nt.NestedTensor(host.to(device), sizes)
    x._record()
    step = lambda: nt.nn.transformer_encoder_layer(layer, x)
    steps = args.steps
    for _ in range(max(args.warmup, 3)):
        step()
    lib = _cabi.load()
    with ClockSampler(local) as clocks:
        step_ms, best_ms = timed_regions(step, steps, world, device)
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        # the dominant kernel alone: feed-forward up-projection with the fused bias + GELU epilogue
        a = torch.randn(T, E, device=device).to(dtype)
        h = torch.empty(T, F, dtype=dtype, device=device)
        w1, b1 = layer.linear1.weight, layer.linear1.bias
        ffn1 = lambda: lib.ntb200_gemm_bias_act(a.data_ptr(), w1.data_ptr(), b1.data_ptr(), None, h.data_ptr(), T, F, E, 2, 1, 0, stream)
        for _ in range(3):
            ffn1()
        f1ms = timed_region(ffn1, steps, world, device) / steps
        # the row operator alone: LayerNorm over [T, E]
        o = torch.empty_like(a)
        g, be = layer.norm1.weight, layer.norm1.bias
        ln = lambda: lib.ntb200_layer_norm(a.data_ptr(), g.data_ptr(), be.data_ptr(), 1e-5, o.data_ptr(), T, E, 2, stream)
        for _ in range(3):
            ln()
        lnms = timed_region(ln, steps, world, device) / steps
        del h
    total_tokens = all_sum(T, world, device)
    value = total_tokens / (step_ms * 1e-3)
    flags = lib.ntb200_device_error_flags()

    e2e = None
    if not KERNEL_ONLY:
        h_in = torch.empty(T * E, dtype=dtype).pin_memory()
        h_in.copy_(host)
        h_out = torch.empty(T * E, dtype=dtype).pin_memory()
        e2e_step = lambda: nt.transformer_encoder_layer_host(layer, h_in, sizes, out=h_out)
        e2e_steps = max(3, min(steps, 20))
        for _ in range(3):
            e2e_step()
        with ClockSampler(local) as clocks2:
            ems = timed_region(e2e_step, e2e_steps, world, device) / e2e_steps
        clocks.samples += clocks2.samples
        clocks.reasons |= clocks2.reasons
        e2e = {"value": total_tokens / (ems * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 2 * T * E,
               "d2h_bytes_per_step": 2 * T * E, "ms_per_step": ems, "steps": e2e_steps,
               "api": "transformer_encoder_layer_host (pinned host in/out, 8 ranges pipelined on 3 streams)"}
    if rank != 0:
        return None
    peaks = measured_peaks()
    tf = flops / (step_ms * 1e-3) / 1e12
    f1tf = 2.0 * T * E * F / (f1ms * 1e-3) / 1e12
    ln_gbs = 4.0 * T * E / (lnms * 1e-3) / 1e9
    line = {
        "metric": "varlen encoder layer valid tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps,
        "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "best_ms": best_ms,
        "timing": "median of 5 timed regions of `steps` steps", "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": ("FIRST %d SEQUENCES ONLY of " % SEQUENCE_LIMIT if SEQUENCE_LIMIT else "") +
                               "config5 batch (1024 sequences per GPU, 70% L~U[16,128] / 30% L~U[128,512]) through one BERT-large "
                               "encoder layer: E=1024, 16 heads x 64, FFN 4096, tanh GELU, post-norm, bf16, inference",
                   "batch_per_gpu": B, "tokens_per_gpu": T, "max_len": maxL, "flops_per_gpu": flops, "token_imbalance": imb,
                   "l2": "activations per step (%.2f GB) exceed the 126 MB L2" % (2 * T * (E * 9 + F * 2) / 1e9)},
        "step_tflops": tf, "step_frac_of_bf16_peak": tf / peaks["bf16_tflops"],
        "step_frac_of_bf16_sustained": tf / peaks["bf16_tflops_sustained"],
        "kernels_ms": {"ffn_up_gemm_gelu": f1ms, "layer_norm": lnms, "step": step_ms},
        "layer_norm_hbm": {"achieved": ln_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ln_gbs / peaks["hbm_gbs"],
                           "bytes": 4.0 * T * E},
        "roofline": {"bound": "tensor", "kernel": "gemm_bias_tcgen05_pair_kernel (feed-forward up-projection + bias + GELU, "
                                                  "M=%d N=4096 K=1024)" % T,
                     "achieved": f1tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": f1tf / peaks["bf16_tflops"],
                     "frac_of_sustained": f1tf / peaks["bf16_tflops_sustained"], "peak_source": peaks["source"],
                     "traffic": None if SEQUENCE_LIMIT else T * NCU_TRAFFIC_GEMM_BYTES_PER_TOKEN["encoder"],
                     "traffic_source": NCU_TRAFFIC_SOURCE},
        "e2e": e2e, "gpu_launches": 9 * 5 * steps, "clocks": clocks.summary(), "device_error_flags": flags,
    }
    if not KERNEL_ONLY:
        from oracle import ntref
        torch.set_num_threads(os.cpu_count() or 1)
        seqs = 16
        Ls = L[:seqs].tolist()
        g2 = torch.Generator().manual_seed(13)
        tensors = [torch.randn(l, E, generator=g2).to(dtype) for l in Ls]
        params = _layer_params(layer)
        fn = lambda: ntref.encoder_layer(tensors, H, params, "gelu_tanh", False, 1e-5)
        t = time_cpu(fn, 1, 3)
        line["cpu_baseline"] = {"value": sum(Ls) / t, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                                "sample": "first %d sequences (%d tokens), median of 3, per-sequence fp32 loop (reference's generic "
                                          "MHA + ATen layer_norm / linear per constituent)" % (seqs, sum(Ls))}
    return line


# ------------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="pad", choices=["pad", "unpad", "mha", "kernels", "encoder"])
    ap.add_argument("--no-mha", action="store_true", help="pad workload only: skip the attached MHA measurement")
    ap.add_argument("--sequences", type=int, default=0,
                    help="use only the first N sequences of each GPU's batch (small cases for profiler captures; "
                         "the line then does not describe the named configuration)")
    ap.add_argument("--only", default="", help="kernels workload: run only this group (transpose | c3) so that a profiler capture "
                                               "holds no more than the group's own data on the device")
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the end-to-end pass, the CPU baseline and the parity spot check")
    args = ap.parse_args()
    global SEQUENCE_LIMIT, KERNEL_ONLY
    SEQUENCE_LIMIT, KERNEL_ONLY = max(args.sequences, 0), bool(args.kernel_only)

    rank, world, local = dist_env()
    if world == 1 and args.gpus > 1 and args.impl == "ours":
        # plain invocation with N > 1: re-launch one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(args.gpus),
               "--master-addr", "127.0.0.1", "--master-port", "29517", os.path.abspath(__file__)] + sys.argv[1:]
        os.execv(sys.executable, cmd)

    if args.impl == "reference":
        line = run_reference(args, args.workload, rank, world)
        if line is not None:
            print(json.dumps(line), flush=True)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path in nestedtensor_b200)")
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    try:
        if args.workload == "kernels":
            line = run_kernels(args, local) if rank == 0 else None
        elif args.workload in ("pad", "unpad"):
            line = run_copy(args, args.workload, rank, world, local)
            if args.workload == "pad" and not args.no_mha:
                # the metric has two halves: the same line carries the full MHA (configuration 5) record, the
                # device-timed figures of configurations 3 and 4, and (N > 1) the strong-scaling record
                torch.cuda.empty_cache()
                mha = run_mha(args, rank, world, local)
                if line is not None and mha is not None:
                    line["mha"] = {k: mha[k] for k in ("metric", "value", "unit", "ms_per_step", "best_ms", "step_tflops",
                                                        "step_frac_of_bf16_peak", "step_frac_of_bf16_sustained", "kernels_ms",
                                                        "attention_tflops_valid", "roofline", "sustained", "e2e", "cpu_baseline",
                                                        "config", "device_error_flags")}
                    line["gpu_launches"] += mha["gpu_launches"]
                torch.cuda.empty_cache()
                if rank == 0 and not KERNEL_ONLY and not SEQUENCE_LIMIT:
                    small = run_small_configs(args, local)
                    if line is not None:
                        line.update(small)
                if world > 1 and not KERNEL_ONLY and not SEQUENCE_LIMIT:
                    torch.cuda.empty_cache()
                    strong = run_strong(args, rank, world, local)
                    if line is not None:
                        line["strong"] = strong
        elif args.workload == "encoder":
            line = run_encoder(args, rank, world, local)
        else:
            line = run_mha(args, rank, world, local)
            if world > 1 and not KERNEL_ONLY and not SEQUENCE_LIMIT:
                strong = run_strong(args, rank, world, local)
                if line is not None:
                    line["strong"] = strong
        if rank == 0 and line is not None:
            print(json.dumps(line), flush=True)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
