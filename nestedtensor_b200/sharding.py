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
