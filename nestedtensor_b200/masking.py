"""Dense -> nested constructors (nestedtensor/nested/masking.py:12-50 over
nt_from_tensor_mask, nestedtensor/csrc/masking.cpp:181-249).

The reference walks the mask on the host with one ``.item()`` per element.  Here one kernel
pass recovers every constituent's extents from the mask (or straight from ``tensor != padding``
without materialising a mask), the host checks that they describe a padding mask, and the
unpad kernel gathers the data.  A constituent is the leading box ``tensor[b, :s_1, :s_2, ...]``;
a mask with holes (a valid element equal to the padding value, or an arbitrary selection
mask) is rejected with a RuntimeError where the reference would either fail inside
``stack`` or silently shorten rows."""
from __future__ import annotations

import collections

import torch

from . import _ops
from .nested import NestedTensor, build_meta

TensorMask = collections.namedtuple("TensorMask", "tensor mask")


def _require_cuda(t, what):
    if not t.is_cuda:
        raise RuntimeError("nestedtensor_b200: %s needs a CUDA tensor (this build has no CPU implementation)" % what)


def _from_sizes(tensor, sizes_dev, counts_dev, lead_dims):
    """Validate device-computed extents on the host and gather the constituents."""
    B = tensor.size(0)
    both = torch.cat([sizes_dev, counts_dev.unsqueeze(1)], 1).cpu()  # the one synchronising copy
    lead = both[:, :lead_dims]
    counts = both[:, lead_dims]
    box = lead.prod(1)
    bad = (counts != box).nonzero()
    if bad.numel() > 0:
        b = int(bad[0])
        raise RuntimeError(
            "nestedtensor_b200: entry %d of the mask is not a padding mask (%d valid elements do not fill the "
            "%s leading box); only masks that keep a leading box of every entry are supported"
            % (b, int(counts[b]), tuple(lead[b].tolist())))
    trail = list(tensor.shape[1 + lead_dims:])
    sizes = torch.cat([lead, torch.tensor(trail, dtype=torch.int64).expand(B, len(trail))], 1).contiguous()
    # an all-false entry keeps its outer extents and gets an empty innermost one, as the
    # reference's all_zero branch does (masking.cpp:203-216)
    empty = counts == 0
    if bool(empty.any()):
        full_outer = torch.tensor(list(tensor.shape[1:lead_dims]), dtype=torch.int64)
        sizes[empty, :max(lead_dims - 1, 0)] = full_outer
        sizes[empty, lead_dims - 1] = 0
    meta = build_meta(sizes, tensor.device)
    buffer = _ops.ops().from_padded_tensor(tensor, sizes, meta)
    return NestedTensor(buffer, sizes, meta)


def nested_tensor_from_padded_tensor(tensor, nested_dim=1, padding=-1):
    """Every ``tensor[b]`` minus its padding becomes a constituent
    (nestedtensor/nested/masking.py:12-14)."""
    _check_args(tensor, tensor, nested_dim)
    if nested_dim != 1:
        raise RuntimeError("Only nested_dim of 1 is currently supported.")
    _require_cuda(tensor, "nested_tensor_from_padded_tensor")
    if tensor.dim() == 1:
        keep = tensor != padding
        sel = tensor[keep]
        return NestedTensor(sel.reshape(-1).clone(), torch.zeros((sel.numel(), 0), dtype=torch.int64))
    sizes_dev, counts_dev = _ops.ops().sizes_from_padded(tensor, padding)
    return _from_sizes(tensor, sizes_dev, counts_dev, tensor.dim() - 1)


def _check_args(tensor, mask, nested_dim):
    """nestedtensor/nested/masking.py:19-41"""
    if tensor is None:
        raise RuntimeError("Tensor can't be undefined (None).")
    if mask is None:
        raise RuntimeError("Mask can't be undefined (None).")
    if tensor.dim() == 0:
        raise RuntimeError("Can't construct nested tensor from a scalar.")
    if nested_dim == 0:
        raise RuntimeError("Nested dimension can't be 0.")
    if nested_dim is not None and nested_dim > tensor.dim():
        raise RuntimeError("Nested dimension ({0}) can't be bigger than data tensor dimension ({1}).".format(
            nested_dim, tensor.dim()))
    if tensor.numel() == 0 and mask.numel() != 0:
        raise RuntimeError("Data tensor can't be emtpy if a mask has values.")
    if tensor.numel() != 0 and mask.numel() == 0:
        raise RuntimeError("Mask tensor can't be emtpy if a data tensor has values.")


def nested_tensor_from_tensor_mask(tensor, mask, nested_dim=1):
    _check_args(tensor, mask, nested_dim)
    return nt_from_tensor_mask(tensor, mask, nested_dim)


def nt_from_tensor_mask(tensor, mask, nested_dim):
    """``torch.ops.nestedtensor.nt_from_tensor_mask`` (nestedtensor/csrc/masking.cpp:223-249, nested_dim 1) with its
    record wrapped in a NestedTensor."""
    if nested_dim != 1:
        raise RuntimeError("Only nested_dim of 1 is currently supported.")
    buffer, sizes, meta = _ops.ops().nt_from_tensor_mask(tensor, mask, nested_dim)
    return NestedTensor(buffer, sizes, meta if meta.numel() == (sizes.size(0) + 1) + sizes.numel() and meta.device == buffer.device else None)


def merge_tensor_mask(tensor, mask, mask_dim=None):
    """``torch.ops.nestedtensor.merge_tensor_mask`` (nestedtensor/csrc/masking.cpp:12-43): drop trailing mask
    dimensions whose slices are all-0 or all-1."""
    return _ops.ops().merge_tensor_mask(tensor, mask, mask_dim)
