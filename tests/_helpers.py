"""Shared helpers for the parity tests: raw C-ABI calls on torch-owned device memory and
bit-exact comparison."""
import ctypes
import math

import torch

from nestedtensor_b200 import _cabi
from nestedtensor_b200.nested import build_meta


def bits_of(value, dtype):
    t = torch.full((1,), value, dtype=dtype)
    raw = t.view(torch.uint8).tolist()
    out = 0
    for i, b in enumerate(raw):
        out |= b << (8 * i)
    return out


def sizes_of(tensors):
    if len(tensors) == 0:
        return torch.zeros((0, 0), dtype=torch.int64)
    return torch.tensor([list(t.shape) for t in tensors], dtype=torch.int64).reshape(len(tensors), tensors[0].dim())


def fold(sizes, dense_dims=None):
    """(nd, inner): trailing regular dims folded into the last ragged one."""
    B, tdim = sizes.shape
    mx = sizes.max(0).values.tolist() if B else [0] * tdim
    k, inner = tdim, 1
    while k > 1:
        j = k - 1
        reg = bool((sizes[:, j] == sizes[0, j]).all())
        if not (reg and mx[j] > 0 and (dense_dims is None or dense_dims[j] == mx[j])):
            break
        inner *= mx[j]
        k -= 1
    return k, inner


def stream_ptr():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def cabi_pad(tensors, padding, device):
    """to_padded_tensor through ntb200_pad_nd; returns the dense tensor."""
    lib = _cabi.load()
    dtype = tensors[0].dtype
    sizes = sizes_of(tensors)
    B, tdim = sizes.shape
    buf = torch.cat([t.reshape(-1) for t in tensors]).to(device)
    meta = build_meta(sizes, device)
    mx = sizes.max(0).values.tolist()
    out = torch.empty([B] + mx, dtype=dtype, device=device)
    nd, inner = fold(sizes)
    rc = lib.ntb200_pad_nd(buf.data_ptr(), out.data_ptr(), meta.data_ptr(), meta.data_ptr() + 8 * (B + 1), tdim, nd,
                           inner, B, _cabi.host_i64(mx), buf.element_size(), bits_of(padding, dtype), stream_ptr())
    _cabi.check("ntb200_pad_nd", rc)
    torch.cuda.synchronize()
    return out


def cabi_unpad(padded, sizes):
    """from_padded_tensor through ntb200_unpad_nd; returns the ragged buffer."""
    lib = _cabi.load()
    B, tdim = sizes.shape
    meta = build_meta(sizes, padded.device)
    total = int(sizes.prod(1).sum())
    out = torch.empty(total, dtype=padded.dtype, device=padded.device)
    dims = list(padded.shape[1:])
    nd, inner = fold(sizes, dims)
    rc = lib.ntb200_unpad_nd(padded.data_ptr(), out.data_ptr(), meta.data_ptr(), meta.data_ptr() + 8 * (B + 1), tdim,
                             nd, inner, B, _cabi.host_i64(dims), total, padded.element_size(), stream_ptr())
    _cabi.check("ntb200_unpad_nd", rc)
    torch.cuda.synchronize()
    return out


def cabi_mask(sizes, mask_nd, device):
    lib = _cabi.load()
    B, tdim = sizes.shape
    meta = build_meta(sizes, device)
    mx = sizes.max(0).values.tolist()[:mask_nd]
    out = torch.empty([B] + mx, dtype=torch.uint8, device=device)
    rc = lib.ntb200_mask_from_sizes(out.data_ptr(), meta.data_ptr() + 8 * (B + 1), tdim, mask_nd, B,
                                    _cabi.host_i64(mx), stream_ptr())
    _cabi.check("ntb200_mask_from_sizes", rc)
    torch.cuda.synchronize()
    return out


def int_view(t):
    """Reinterpret as integers of the same width so that comparisons are bit-exact
    (distinguishes -0.0 from 0.0 and compares NaN payloads)."""
    t = t.contiguous()
    return t.view({1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[t.element_size()])


def assert_bit_equal(a, b, what=""):
    a, b = a.cpu(), b.cpu()
    assert a.shape == b.shape, "%s shape %s vs %s" % (what, tuple(a.shape), tuple(b.shape))
    assert a.dtype == b.dtype, "%s dtype %s vs %s" % (what, a.dtype, b.dtype)
    if a.numel() == 0:
        return
    ia, ib = int_view(a), int_view(b)
    if not torch.equal(ia, ib):
        bad = (ia != ib).nonzero()
        raise AssertionError("%s: %d of %d elements differ, first at %s" % (what, bad.size(0), a.numel(), bad[0].tolist()))


def random_list(gen, batch, tdim, lo, hi, dtype, regular_last=None, int_values=False):
    """``batch`` tensors of ``tdim`` dims with extents in [lo, hi]; optionally a regular last dim."""
    out = []
    for _ in range(batch):
        shape = [int(torch.randint(lo, hi + 1, (1,), generator=gen)) for _ in range(tdim)]
        if regular_last is not None:
            shape[-1] = regular_last
        x = torch.randn(shape, generator=gen)
        if dtype in (torch.int64, torch.int32, torch.int16, torch.uint8, torch.int8):
            x = (x * 50).to(dtype)
        elif dtype == torch.bool:
            x = x > 0
        else:
            x = x.to(dtype)
        out.append(x)
    return out
