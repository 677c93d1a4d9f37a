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


def shard_lengths(kind, world, rank):
    """Lengths of this rank's shard: N batches of the configuration drawn as ONE list (generator of the
    configuration, batch = N * config batch) and cut token-balanced into N contiguous slices."""
    from nestedtensor_b200 import workloads, sharding
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
    host = host_values(n_valid, dtype, 20242 + rank)
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
        ms = timed_region(step, args.steps, world, device)
        ms2 = timed_region(step, args.steps, world, device)  # second pass keeps the sampler busy longer
    ms = min(ms, ms2)
    total_bytes = all_sum(alg_bytes, world, device)
    value = total_bytes / (ms / args.steps * 1e-3) / 1e9
    kernel_ms = ms / args.steps

    # parity spot check in the same run (size-independent property): round trip is the identity
    parity_ok = None
    if not KERNEL_ONLY:
        chk = ops.from_padded_tensor(ops.to_padded_tensor(buf, sz, meta, 0.0), sz, meta)
        parity_ok = bool(torch.equal(chk.view(torch.int16), ragged.view(torch.int16)))
        del chk

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
        e2e = {"value": total_bytes / (ems / e2e_steps * 1e-3) / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": es * in_elems, "d2h_bytes_per_step": es * out_elems,
               "ms_per_step": ems / e2e_steps, "steps": e2e_steps, "sample": "full shard",
               "api": "%s_host (pinned host in/out, 8 ranges pipelined on 3 streams)" %
                      ("to_padded_tensor" if kind == "pad" else "from_padded_tensor"),
               "single_stream_value": total_bytes / (sms / e2e_steps * 1e-3) / 1e9}
        clocks.samples += clocks2.samples
        clocks.reasons |= clocks2.reasons
    else:
        e2e = {"value": None, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
               "sample": "skipped: host has %.1f GB available, needs %.1f GB pinned per rank" % (avail / 1e9, need / 1e9)}

    peaks = measured_peaks()
    line = None
    if rank == 0:
        cpu = None
        if world == 1 and not KERNEL_ONLY:  # a single-GPU-run figure; other ranks would compete for the cores
            seqs = 256
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
        line = {
            "metric": "to_padded_tensor HBM GB/s" if kind == "pad" else "from_padded_tensor HBM GB/s",
            "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": kernel_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 (bit copy, u16)", "data": "synthetic",
            "config": {"workload": ("FIRST %d SEQUENCES ONLY of " % SEQUENCE_LIMIT if SEQUENCE_LIMIT else "") +
                                   "config2: %d bf16 sequences (L_i,1024), L_i=clip(round(lognormal(ln200,0.6)),1,1024) "
                                   "per GPU; %s" % (4096, "to_padded_tensor(padding=0)" if kind == "pad" else
                                                    "from_padded_tensor with known sizes"),
                       "batch_per_gpu": B, "tokens_per_gpu": T, "max_len": maxL, "hidden": hidden,
                       "algorithmic_bytes_per_gpu": alg_bytes, "token_imbalance": imb,
                       "l2": "inputs+outputs (%.1f GB) far larger than the 126 MB L2" % (alg_bytes / 1e9)},
            "roofline": {"bound": "hbm", "achieved": alg_bytes / (kernel_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": alg_bytes / (kernel_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                         "frac_of_nominal_8000": alg_bytes / (kernel_ms * 1e-3) / 1e9 / 8000.0,
                         "peak_source": peaks["source"], "traffic": NCU_TRAFFIC.get(kind)},
            "cpu_baseline": cpu,
            "e2e": e2e,
            "gpu_launches": args.steps,
            "clocks": clocks.summary(),
            "parity_roundtrip_bit_exact": parity_ok,
        }
    return line


# Per-launch DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel, from the ncu
# captures summarised under profiles/.  The captures ran on the first 512 (copies) / 256 (MHA) sequences;
# reads equalled the algorithmic bytes and writes fell short of them only by the 50-55 MB still dirty in
# L2 at kernel end, which does not grow with the batch, so the full-size figure is algorithmic - residue:
#   pad   1.950 + 8.590 - 0.055 GB      unpad 1.950 + 1.950 - 0.051 GB
#   QKV projection (A 310.9 MB + W 6.3 MB read, C 932.6 MB written) - 0.052 GB
#   feed-forward up-projection (A 310.9 MB + W 8.4 MB read, C 1243.5 MB written) - 0.05 GB
NCU_TRAFFIC = {"pad": 10.48e9, "unpad": 3.85e9, "mha": 1.20e9, "encoder": 1.51e9}


# ---------------------------------------------------------------------- reference arm
def run_reference(args, kind, rank, world):
    """The reference's own CPU implementation of the path (oracle port) on the host cores; rank 0 only."""
    if rank != 0:
        return None
    torch.set_num_threads(os.cpu_count() or 1)
    L, _ = shard_lengths("pad" if kind in ("pad", "unpad") else "mha", 1, 0)
    hidden, dtype = 1024, torch.bfloat16
    seqs = 256
    if kind == "pad":
        _, nbytes, fn = cpu_pad_sample(L, hidden, dtype, seqs)
        metric = "to_padded_tensor HBM GB/s"
    elif kind == "unpad":
        _, nbytes, fn = cpu_unpad_sample(L, hidden, dtype, seqs)
        metric = "from_padded_tensor HBM GB/s"
    else:
        return run_reference_mha(args, world, encoder=(kind == "encoder"))
    for _ in range(max(1, min(args.warmup, 2))):
        fn()
    steps = max(1, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    dt = (time.perf_counter() - t0) / steps
    v = nbytes / dt / 1e9
    cores = torch.get_num_threads()
    sample = "each step = the first %d sequences of configuration 2 (%.2f GB algorithmic)" % (seqs, nbytes / 1e9)
    return {"impl": "reference", "metric": metric, "value": v, "unit": "GB/s", "n_gpus": world, "steps": steps,
            "warmup": max(1, min(args.warmup, 2)), "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16 (bit copy, u16)", "data": "synthetic",
            "config": {"workload": "config2 (CPU sample): " + sample},
            "cpu_baseline": {"value": v, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def cpu_mha_sample(L, E, H, dtype, seqs):
    """The reference's generic (CPU-capable) MHA, nestedtensor/csrc/mha.cpp:18-69, on the first `seqs` sequences."""
    from oracle import ntref
    from nestedtensor_b200 import workloads
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
    E, H, dtype, seqs = 1024, 16, torch.bfloat16, 64
    if encoder:
        from oracle import ntref
        seqs = 32
        Ls = L[:seqs].tolist()
        g = torch.Generator().manual_seed(13)
        tensors = [torch.randn(l, E, generator=g).to(dtype) for l in Ls]
        params = _layer_params(_bert_large_layer(torch.float32, "cpu"))
        tokens, fn = sum(Ls), (lambda: ntref.encoder_layer(tensors, H, params, "gelu_tanh", False, 1e-5))
    else:
        tokens, fn = cpu_mha_sample(L, E, H, dtype, seqs)
    for _ in range(max(1, min(args.warmup, 2))):
        fn()
    steps = max(1, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    dt = (time.perf_counter() - t0) / steps
    v = tokens / dt
    sample = "each step = the first %d sequences of configuration 5 (%d tokens), per-sequence fp32 loop" % (seqs, tokens)
    return {"impl": "reference", "metric": "varlen encoder layer valid tokens/s" if encoder else "varlen MHA valid tokens/s",
            "value": v, "unit": "tokens/s", "n_gpus": world,
            "steps": steps, "warmup": max(1, min(args.warmup, 2)), "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 inputs, fp32 math", "data": "synthetic",
            "config": {"workload": "config5 (CPU sample): " + sample},
            "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                             "sample": sample},
            "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def run_mha(args, rank, world, local, brief=False):
    """Configuration 5: BERT-large varlen self-attention forward (bf16, E=1024, 16 heads x 64)."""
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
    gemm_flops = 2.0 * T * 3 * E * E
    host = host_values(T * E, dtype, 20245 + rank)
    w = workloads._mha_weights(workloads._gen(5), E, dtype)
    wd = {k: v.to(device) for k, v in w.items()}
    x = nt.NestedTensor(host.to(device), sizes)
    ops = _ops.ops()
    buf, sz, meta = x._record()
    scaling = float(d) ** -0.5
    step = lambda: ops.bt_min_mha(H, d, 0.0, False, buf, sz, meta, wd["in_proj_weight"], wd["in_proj_bias"], scaling,
                                  wd["out_proj_weight"], wd["out_proj_bias"])
    steps = args.steps if not brief else min(args.steps, 20)
    for _ in range(max(args.warmup, 3)):
        step()
    with ClockSampler(local) as clocks:
        ms = timed_region(step, steps, world, device)
        ms = min(ms, timed_region(step, steps, world, device))
        # the dominant kernel alone: QKV projection through the C ABI, same stream, same events
        lib = _cabi.load()
        qkv = torch.empty(T, 3 * E, dtype=dtype, device=device)
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        gemm = lambda: lib.ntb200_gemm_bias(buf.data_ptr(), wd["in_proj_weight"].data_ptr(), wd["in_proj_bias"].data_ptr(),
                                            qkv.data_ptr(), T, 3 * E, E, 2, 0, stream)
        for _ in range(3):
            gemm()
        gms = timed_region(gemm, steps, world, device) / steps
        attn_out = torch.empty(T, E, dtype=dtype, device=device)
        ws_bytes = lib.ntb200_varlen_attention_workspace_bytes(B, T, H, d, 2)
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=device)
        attn = lambda: lib.ntb200_varlen_attention(qkv.data_ptr(), attn_out.data_ptr(), meta.data_ptr(), B, T, H, d, maxL,
                                                   scaling, 2, 0, ws.data_ptr() if ws_bytes else None, ws_bytes, stream)
        for _ in range(3):
            attn()
        ams = timed_region(attn, steps, world, device) / steps
    step_ms = ms / steps
    total_tokens = all_sum(T, world, device)
    value = total_tokens / (step_ms * 1e-3)
    flags = lib.ntb200_device_error_flags()

    brief = brief or KERNEL_ONLY
    e2e = None
    if not brief:
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
               "single_stream_value": total_tokens / (sms * 1e-3)}

    if rank != 0:
        return None
    peaks = measured_peaks()
    tf = flops / (step_ms * 1e-3) / 1e12
    gtf = gemm_flops / (gms * 1e-3) / 1e12
    atf = 4.0 * E * float((L.double() ** 2).sum()) / (ams * 1e-3) / 1e12
    line = {
        "metric": "varlen MHA valid tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps,
        "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": ("FIRST %d SEQUENCES ONLY of " % SEQUENCE_LIMIT if SEQUENCE_LIMIT else "") +
                               "config5: BERT-large varlen self-attention forward, batch 1024 per GPU, 70% L~U[16,128] / "
                               "30% L~U[128,512], E=1024, 16 heads x 64, bf16",
                   "batch_per_gpu": B, "tokens_per_gpu": T, "max_len": maxL, "flops_per_gpu": flops,
                   "token_imbalance": imb,
                   "l2": "activations per step (x, qkv, attn, out = %.2f GB) exceed the 126 MB L2" % (12 * T * E / 1e9)},
        "step_tflops": tf, "step_frac_of_bf16_peak": tf / peaks["bf16_tflops"],
        "step_frac_of_bf16_sustained": tf / peaks["bf16_tflops_sustained"],
        "kernels_ms": {"qkv_gemm": gms, "attention": ams, "step": step_ms},
        "attention_tflops_valid": atf,
        "roofline": {"bound": "tensor", "kernel": "gemm_bias_tcgen05_pair_kernel (QKV projection, M=%d N=3072 K=1024)" % T,
                     "achieved": gtf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": gtf / peaks["bf16_tflops"],
                     "frac_of_sustained": gtf / peaks["bf16_tflops_sustained"], "peak_source": peaks["source"],
                     "traffic": NCU_TRAFFIC.get("mha")},
        "e2e": e2e, "gpu_launches": 4 * steps, "clocks": clocks.summary(), "device_error_flags": flags,
    }
    if not brief:
        torch.set_num_threads(os.cpu_count() or 1)
        tokens, fn = cpu_mha_sample(L, E, H, dtype, 32)
        t = time_cpu(fn, 1, 3)
        line["cpu_baseline"] = {"value": tokens / t, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                                "sample": "first 32 sequences (%d tokens), median of 3, per-sequence fp32 loop of the "
                                          "reference's generic MHA" % tokens}
    return line


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

    def add(name, config, ms, nbytes=None, flops=None):
        r = {"op": name, "config": config, "ms": ms}
        if nbytes is not None:
            r["GB/s"] = nbytes / ms / 1e6
            r["frac_hbm_measured"] = r["GB/s"] / peaks["hbm_gbs"]
        if flops is not None:
            r["TFLOP/s"] = flops / ms / 1e9
            r["frac_bf16_burst"] = r["TFLOP/s"] / peaks["bf16_tflops"]
        rows.append(r)

    n = max(args.steps, 5)
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
    # configuration 3: 32 fp32 images (3, H_i, W_i)
    w = workloads.config3()
    a = nt.NestedTensor(w.buffer.to(device), w.sizes)
    b, sz, meta = a._record()
    nv = w.buffer.numel()
    padded = ops.to_padded_tensor(b, sz, meta, 0.0)
    npad = padded.numel()
    add("to_padded_tensor (4-D)", "c3", timed(lambda: ops.to_padded_tensor(b, sz, meta, 0.0), n), es * (nv + npad))
    add("to_tensor_mask (4-D uint8 mask)", "c3", timed(lambda: ops.to_tensor_mask(b, sz, meta, None), n), es * (nv + npad) + npad)
    add("to_mask(mask_dim=3)", "c3", timed(lambda: ops.to_mask(sz, meta, 3), n), None)
    add("from_padded_tensor (4-D)", "c3", timed(lambda: ops.from_padded_tensor(padded, sz, meta), n), 2 * es * nv)
    add("sizes_from_padded (scan)", "c3", timed(lambda: ops.sizes_from_padded(padded, 0.0), n), es * npad)
    del padded
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
    # image-shaped path: 32 fp16 feature maps (256, H_i, W_i), H_i, W_i in [100, 168] (a stride-8 backbone level)
    hw = torch.randint(100, 169, (32, 2), generator=g)
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
        ms = timed_region(step, steps, world, device)
        ms = min(ms, timed_region(step, steps, world, device))
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
    step_ms = ms / steps
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
        "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak",
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
                     "traffic": NCU_TRAFFIC.get("encoder")},
        "e2e": e2e, "gpu_launches": 8 * steps, "clocks": clocks.summary(), "device_error_flags": flags,
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
                # the metric has two halves; attach a short MHA (configuration 5) measurement to the same line
                torch.cuda.empty_cache()
                mha = run_mha(args, rank, world, local, brief=True)
                if line is not None and mha is not None:
                    line["mha"] = {k: mha[k] for k in ("metric", "value", "unit", "ms_per_step", "step_tflops",
                                                        "step_frac_of_bf16_peak", "kernels_ms", "roofline", "config")}
        elif args.workload == "encoder":
            line = run_encoder(args, rank, world, local)
        else:
            line = run_mha(args, rank, world, local)
        if rank == 0 and line is not None:
            print(json.dumps(line), flush=True)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
