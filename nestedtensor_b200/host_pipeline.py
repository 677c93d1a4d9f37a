"""Host-buffer entry points: ragged data in pinned host memory on both sides of the operator.

A caller whose batches live in host memory pays a host->device copy of the input and a device->host
copy of the result around every operator call; done back to back on one stream, the two copies and the
kernel add up.  Here the batch is cut into a few contiguous ranges of sequences (sequences are
independent on this path) and the three stages run as a software pipeline on three CUDA streams with
double-buffered device slots: while range c is computed, range c+1 is uploaded and range c-1 is drained,
so that a step costs about max(upload, download) instead of their sum.

    to_padded_tensor_host(h_ragged, sizes, padding)   -> pinned dense tensor (B, max_1, ..., max_k)
    from_padded_tensor_host(h_padded, sizes)          -> pinned 1-D ragged buffer
    multi_head_attention_host(h_x, sizes, ...)        -> pinned packed [T, E] output of bt_min_mha
    transformer_encoder_layer_host(layer, h_x, sizes) -> pinned packed [T, E] output of an encoder layer

The kernels are the ones behind ``torch.ops.nestedtensor.to_padded_tensor`` / ``bt_min_mha``; there is no
CPU path.  The reference has no host-buffer API (its operators take device tensors only).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch

from . import _ops
from .nested import build_meta
from .sharding import token_balanced_partition


def plan_ranges(weights: Sequence[int], n_ranges: int) -> List[Tuple[int, int]]:
    """Contiguous, non-empty ``[start, end)`` ranges of the batch with about equal total weight."""
    n_ranges = max(1, min(int(n_ranges), len(weights)))
    parts = token_balanced_partition(list(weights), n_ranges)
    return [(a, b) for a, b in parts if b > a]


_STREAMS = {}


def _streams(device: torch.device):
    """The upload / compute / download streams of a device, created once: the caching allocator keeps one
    pool of blocks per stream, so fresh streams on every call would mean fresh device allocations on every
    call."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _STREAMS:
        _STREAMS[key] = tuple(torch.cuda.Stream(torch.device("cuda", key)) for _ in range(3))
    return _STREAMS[key]


def run_pipeline(n: int, upload: Callable[[int, int], None], compute: Callable[[int, int], None],
                 download: Callable[[int, int], None], device: torch.device, slots: int = 2) -> None:
    """Three-stage pipeline over ranges ``0..n-1``; stage callbacks get ``(range index, slot)`` and enqueue
    on the current stream.  Slot ``c % slots`` of the upload buffers is reused once range ``c - slots`` has
    been computed, of the download buffers once it has been drained.  On return the caller's stream waits
    for everything enqueued here (nothing is synchronised on the host)."""
    caller = torch.cuda.current_stream(device)
    s_up, s_comp, s_down = _streams(device)
    start = torch.cuda.Event()
    start.record(caller)
    for s in (s_up, s_comp, s_down):
        s.wait_event(start)
    ev_up = [torch.cuda.Event() for _ in range(n)]
    ev_comp = [torch.cuda.Event() for _ in range(n)]
    ev_down = [torch.cuda.Event() for _ in range(n)]
    for c in range(n):
        slot = c % slots
        with torch.cuda.stream(s_up):
            if c >= slots:
                s_up.wait_event(ev_comp[c - slots])
            upload(c, slot)
            ev_up[c].record(s_up)
        with torch.cuda.stream(s_comp):
            s_comp.wait_event(ev_up[c])
            if c >= slots:
                s_comp.wait_event(ev_down[c - slots])
            compute(c, slot)
            ev_comp[c].record(s_comp)
        with torch.cuda.stream(s_down):
            s_down.wait_event(ev_comp[c])
            download(c, slot)
            ev_down[c].record(s_down)
    for c in range(max(0, n - slots), n):
        caller.wait_event(ev_down[c])
        s_comp.wait_event(ev_down[c])  # memory that compute callbacks allocated may be released after this point


def _check_host(t: torch.Tensor, name: str) -> None:
    if t.device.type != "cpu" or not t.is_pinned() or not t.is_contiguous():
        raise ValueError("%s must be a contiguous tensor in pinned host memory" % name)


def _check_sizes(sizes: torch.Tensor) -> None:
    if sizes.dtype != torch.int64 or sizes.dim() != 2 or sizes.device.type != "cpu":
        raise TypeError("sizes must be a CPU int64 [B, tensor_dim] tensor")


def to_padded_tensor_host(h_ragged: torch.Tensor, sizes: torch.Tensor, padding=0, out: Optional[torch.Tensor] = None,
                          device="cuda", ranges: int = 8) -> torch.Tensor:
    """``to_padded_tensor`` (nestedtensor/csrc/masking.cpp:558-650) for a nested tensor whose buffer is the
    pinned 1-D host tensor ``h_ragged`` with constituent shapes ``sizes``; returns the pinned dense tensor
    ``(B, max_1, ..., max_k)``.  The copies are asynchronous: synchronise the current stream before
    reading the result on the host."""
    _check_host(h_ragged, "h_ragged")
    _check_sizes(sizes)
    device = torch.device(device)
    B, tdim = sizes.shape
    if B == 0 or tdim == 0:
        raise ValueError("to_padded_tensor_host needs a non-empty batch of tensors with at least one dimension")
    numel = sizes.prod(1)
    if int(numel.sum()) != h_ragged.numel() or h_ragged.dim() != 1:
        raise ValueError("h_ragged must be 1-D with sum(numel) elements")
    maxes = [int(v) for v in sizes.max(0).values]
    slab = 1
    for v in maxes:
        slab *= v
    shape = [B] + maxes
    if out is None:
        out = torch.empty(shape, dtype=h_ragged.dtype).pin_memory()
    else:
        _check_host(out, "out")
        if list(out.shape) != shape or out.dtype != h_ragged.dtype:
            raise ValueError("out must have shape %s and dtype %s" % (shape, h_ragged.dtype))
    if slab == 0:
        return out
    parts = plan_ranges([int(v) + slab for v in numel], ranges)
    offs = torch.zeros(B + 1, dtype=torch.int64)
    torch.cumsum(numel, 0, out=offs[1:])
    ops = _ops.ops()
    with torch.cuda.device(device):
        metas = [build_meta(sizes[a:b], device) for a, b in parts]
        subs = [sizes[a:b].contiguous() for a, b in parts]
        in_max = max(int(offs[b] - offs[a]) for a, b in parts)
        b_max = max(b - a for a, b in parts)
        d_in = [torch.empty(max(in_max, 1), dtype=h_ragged.dtype, device=device) for _ in range(2)]
        d_out = [torch.empty([b_max] + maxes, dtype=h_ragged.dtype, device=device) for _ in range(2)]

        def upload(c, slot):
            a, b = parts[c]
            n = int(offs[b] - offs[a])
            d_in[slot][:n].copy_(h_ragged[int(offs[a]):int(offs[b])], non_blocking=True)

        def compute(c, slot):
            a, b = parts[c]
            n = int(offs[b] - offs[a])
            ops.to_padded_tensor_out(d_in[slot][:n], subs[c], metas[c], float(padding), d_out[slot][:b - a])

        def download(c, slot):
            a, b = parts[c]
            out[a:b].copy_(d_out[slot][:b - a], non_blocking=True)

        run_pipeline(len(parts), upload, compute, download, device)
        # the device slots go back to the allocator when this frame ends; the caller's stream has been made
        # to wait for the pipeline, and the slots were allocated on that stream, so reuse is ordered
    return out


def from_padded_tensor_host(h_padded: torch.Tensor, sizes: torch.Tensor, out: Optional[torch.Tensor] = None,
                            device="cuda", ranges: int = 8) -> torch.Tensor:
    """``from_padded_tensor`` (nestedtensor/csrc/masking.cpp:459-533) for a pinned dense host tensor
    ``(B, d_1, ..., d_k)`` and known constituent shapes ``sizes``; returns the pinned 1-D ragged buffer
    (asynchronous, as above)."""
    _check_host(h_padded, "h_padded")
    _check_sizes(sizes)
    device = torch.device(device)
    B, tdim = sizes.shape
    if B == 0 or tdim == 0 or h_padded.dim() != tdim + 1 or h_padded.size(0) != B:
        raise ValueError("h_padded must have shape (batch, extents...) matching sizes")
    numel = sizes.prod(1)
    total = int(numel.sum())
    if out is None:
        out = torch.empty(total, dtype=h_padded.dtype).pin_memory()
    else:
        _check_host(out, "out")
        if out.dim() != 1 or out.numel() != total or out.dtype != h_padded.dtype:
            raise ValueError("out must be 1-D with sum(numel) elements of the input dtype")
    slab = h_padded[0].numel()
    if total == 0:
        return out
    parts = plan_ranges([int(v) + slab for v in numel], ranges)
    offs = torch.zeros(B + 1, dtype=torch.int64)
    torch.cumsum(numel, 0, out=offs[1:])
    ops = _ops.ops()
    with torch.cuda.device(device):
        metas = [build_meta(sizes[a:b], device) for a, b in parts]
        subs = [sizes[a:b].contiguous() for a, b in parts]
        b_max = max(b - a for a, b in parts)
        d_in = [torch.empty([b_max] + list(h_padded.shape[1:]), dtype=h_padded.dtype, device=device) for _ in range(2)]
        results = [None, None]

        def upload(c, slot):
            a, b = parts[c]
            d_in[slot][:b - a].copy_(h_padded[a:b], non_blocking=True)

        def compute(c, slot):
            a, b = parts[c]
            results[slot] = ops.from_padded_tensor(d_in[slot][:b - a], subs[c], metas[c])

        def download(c, slot):
            a, b = parts[c]
            # results[slot] stays referenced until range c + 2 replaces it, which the compute stream does only
            # after waiting for this download: its memory cannot be handed out again before the copy has run
            out[int(offs[a]):int(offs[b])].copy_(results[slot], non_blocking=True)

        run_pipeline(len(parts), upload, compute, download, device)
    return out


def multi_head_attention_host(h_x: torch.Tensor, sizes: torch.Tensor, num_heads: int, in_proj_weight: torch.Tensor,
                              in_proj_bias: torch.Tensor, out_proj_weight: torch.Tensor,
                              out_proj_bias: Optional[torch.Tensor], scaling: Optional[float] = None,
                              out: Optional[torch.Tensor] = None, ranges: int = 8) -> torch.Tensor:
    """Self-attention ``bt_min_mha`` (nestedtensor/csrc/cuda/mha.cpp:25-107) over a packed token matrix held
    in pinned host memory: ``h_x`` is ``[T, E]`` (or its 1-D buffer), ``sizes`` the ``(L_i, E)`` rows; the
    weights are CUDA tensors and pick the device.  Returns the pinned ``[T, E]`` output (asynchronous, as
    above)."""
    _check_host(h_x, "h_x")
    _check_sizes(sizes)
    device = in_proj_weight.device
    if device.type != "cuda":
        raise ValueError("the projection weights must be CUDA tensors (this build has no CPU implementation)")
    B, tdim = sizes.shape
    if tdim != 2 or B == 0:
        raise ValueError("query needs to be 3 dim.")
    E = int(sizes[0, 1])
    if bool((sizes[:, 1] != E).any()):
        raise ValueError("query's third dimension must be regular.")
    if E % num_heads != 0:
        raise ValueError("embed_dim must be divisible by num_heads")
    head_dim = E // num_heads
    lengths = sizes[:, 0]
    T = int(lengths.sum())
    if h_x.numel() != T * E:
        raise ValueError("h_x must hold sum(L_i) * E elements")
    x = h_x.reshape(T, E)
    if out is None:
        out = torch.empty((T, E), dtype=h_x.dtype).pin_memory()
    else:
        _check_host(out, "out")
        if out.numel() != T * E or out.dtype != h_x.dtype:
            raise ValueError("out must hold sum(L_i) * E elements of the input dtype")
    o2 = out.reshape(T, E)
    if scaling is None:
        scaling = float(head_dim) ** -0.5
    parts = plan_ranges([int(v) for v in lengths], ranges)
    toff = torch.zeros(B + 1, dtype=torch.int64)
    torch.cumsum(lengths, 0, out=toff[1:])
    ops = _ops.ops()
    with torch.cuda.device(device):
        metas = [build_meta(sizes[a:b], device) for a, b in parts]
        subs = [sizes[a:b].contiguous() for a, b in parts]
        t_max = max(int(toff[b] - toff[a]) for a, b in parts)
        d_in = [torch.empty((max(t_max, 1), E), dtype=h_x.dtype, device=device) for _ in range(2)]
        results = [None, None]

        def upload(c, slot):
            a, b = parts[c]
            n = int(toff[b] - toff[a])
            d_in[slot][:n].copy_(x[int(toff[a]):int(toff[b])], non_blocking=True)

        def compute(c, slot):
            a, b = parts[c]
            n = int(toff[b] - toff[a])
            results[slot] = ops.bt_min_mha(num_heads, head_dim, 0.0, False, d_in[slot][:n].reshape(-1), subs[c], metas[c],
                                           in_proj_weight, in_proj_bias, float(scaling), out_proj_weight, out_proj_bias)

        def download(c, slot):
            a, b = parts[c]
            # results[slot] stays referenced until range c + 2 replaces it, which the compute stream does only
            # after waiting for this download: its memory cannot be handed out again before the copy has run
            o2[int(toff[a]):int(toff[b])].copy_(results[slot].reshape(-1, E), non_blocking=True)

        run_pipeline(len(parts), upload, compute, download, device)
    return out


def transformer_encoder_layer_host(layer: torch.nn.TransformerEncoderLayer, h_x: torch.Tensor, sizes: torch.Tensor,
                                   activation: Optional[str] = None, out: Optional[torch.Tensor] = None,
                                   ranges: int = 8) -> torch.Tensor:
    """``nn.transformer_encoder_layer`` over a packed token matrix held in pinned host memory (``h_x`` is
    ``[T, E]`` or its 1-D buffer, ``sizes`` the ``(L_i, E)`` rows); the layer's parameters pick the device.
    Returns the pinned ``[T, E]`` output (asynchronous, as above)."""
    from .nested import NestedTensor
    from .nn import transformer_encoder_layer
    _check_host(h_x, "h_x")
    _check_sizes(sizes)
    device = layer.linear1.weight.device
    if device.type != "cuda":
        raise ValueError("the layer must be on a CUDA device (this build has no CPU implementation)")
    B, tdim = sizes.shape
    if tdim != 2 or B == 0:
        raise ValueError("query needs to be 3 dim.")
    E = int(sizes[0, 1])
    if bool((sizes[:, 1] != E).any()):
        raise ValueError("query's third dimension must be regular.")
    lengths = sizes[:, 0]
    T = int(lengths.sum())
    if h_x.numel() != T * E:
        raise ValueError("h_x must hold sum(L_i) * E elements")
    x = h_x.reshape(T, E)
    if out is None:
        out = torch.empty((T, E), dtype=h_x.dtype).pin_memory()
    else:
        _check_host(out, "out")
        if out.numel() != T * E or out.dtype != h_x.dtype:
            raise ValueError("out must hold sum(L_i) * E elements of the input dtype")
    o2 = out.reshape(T, E)
    parts = plan_ranges([int(v) for v in lengths], ranges)
    toff = torch.zeros(B + 1, dtype=torch.int64)
    torch.cumsum(lengths, 0, out=toff[1:])
    with torch.cuda.device(device):
        metas = [build_meta(sizes[a:b], device) for a, b in parts]
        subs = [sizes[a:b].contiguous() for a, b in parts]
        t_max = max(int(toff[b] - toff[a]) for a, b in parts)
        d_in = [torch.empty((max(t_max, 1), E), dtype=h_x.dtype, device=device) for _ in range(2)]
        results = [None, None]

        def upload(c, slot):
            a, b = parts[c]
            d_in[slot][:int(toff[b] - toff[a])].copy_(x[int(toff[a]):int(toff[b])], non_blocking=True)

        def compute(c, slot):
            a, b = parts[c]
            n = int(toff[b] - toff[a])
            src = NestedTensor(d_in[slot][:n].reshape(-1), subs[c], metas[c])
            results[slot] = transformer_encoder_layer(layer, src, activation)._buffer

        def download(c, slot):
            a, b = parts[c]
            # (kept alive by stream order, as in multi_head_attention_host)
            o2[int(toff[a]):int(toff[b])].copy_(results[slot].reshape(-1, E), non_blocking=True)

        run_pipeline(len(parts), upload, compute, download, device)
    return out
