"""Token-balanced contiguous partition of a sequence list across GPUs.

The path has no inter-sequence dependency, so multi-GPU runs give every rank a contiguous
slice of the batch holding about the same number of tokens; no collective is needed on the
data path (the reference itself has no multi-GPU mode at all)."""
from __future__ import annotations

from typing import List, Sequence, Tuple


def token_balanced_partition(lengths: Sequence[int], world_size: int) -> List[Tuple[int, int]]:
    """Split ``range(len(lengths))`` into ``world_size`` contiguous ``[start, end)`` slices.

    With prefix sums ``P_i`` of the lengths and ``T = P_n``, rank ``r`` starts at the index whose
    prefix sum is closest to ``r * T / world_size``.  Deterministic from the lengths alone, keeps
    the order (re-assembly is concatenation) and never yields a negative-size slice; a slice may
    be empty when there are fewer sequences than ranks."""
    n = len(lengths)
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    prefix = [0] * (n + 1)
    for i, v in enumerate(lengths):
        if v < 0:
            raise ValueError("negative length")
        prefix[i + 1] = prefix[i] + int(v)
    total = prefix[n]
    cuts = [0]
    lo = 0
    for r in range(1, world_size):
        target = r * total / world_size
        # first index with prefix >= target, then pick the closer of it and its predecessor
        i = lo
        while i < n and prefix[i] < target:
            i += 1
        if i > lo and abs(prefix[i - 1] - target) <= abs(prefix[i] - target):
            i -= 1
        cuts.append(i)
        lo = i
    cuts.append(n)
    return [(cuts[r], cuts[r + 1]) for r in range(world_size)]


def imbalance(lengths: Sequence[int], parts: Sequence[Tuple[int, int]]) -> float:
    """max over ranks of tokens / mean tokens per rank (1.0 = perfectly balanced)."""
    toks = [sum(int(v) for v in lengths[a:b]) for a, b in parts]
    mean = sum(toks) / max(len(toks), 1)
    return max(toks) / mean if mean > 0 else 1.0


def gather_ragged(local_buffer, local_sizes, group=None):
    """All-gather the per-rank pieces of a sharded nested tensor for VERIFICATION (never on the data
    path): every rank contributes its 1-D buffer and its CPU int64 sizes matrix; returns
    (buffer, sizes) of the whole batch in rank order.  Buffers are padded to the largest per-rank
    element count for the fixed-size collective.  Works with NCCL (device buffers) and gloo (CPU)."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    dev = local_buffer.device
    tdim = local_sizes.size(1)
    counts = torch.tensor([local_buffer.numel(), local_sizes.size(0)], dtype=torch.int64, device=dev)
    all_counts = [torch.zeros_like(counts) for _ in range(world)]
    dist.all_gather(all_counts, counts, group=group)
    all_counts = [c.cpu().tolist() for c in all_counts]
    max_elems = max(c[0] for c in all_counts)
    max_rows = max(c[1] for c in all_counts)
    pad_buf = torch.zeros(max(max_elems, 1), dtype=local_buffer.dtype, device=dev)
    pad_buf[:local_buffer.numel()] = local_buffer
    bufs = [torch.empty_like(pad_buf) for _ in range(world)]
    dist.all_gather(bufs, pad_buf, group=group)
    pad_sz = torch.zeros((max(max_rows, 1), max(tdim, 1)), dtype=torch.int64, device=dev)
    if local_sizes.numel():
        pad_sz[:local_sizes.size(0), :tdim] = local_sizes.to(dev)
    szs = [torch.empty_like(pad_sz) for _ in range(world)]
    dist.all_gather(szs, pad_sz, group=group)
    buffer = torch.cat([b[:c[0]] for b, c in zip(bufs, all_counts)])
    sizes = torch.cat([s[:c[1], :tdim].cpu() for s, c in zip(szs, all_counts)]).contiguous()
    return buffer, sizes
