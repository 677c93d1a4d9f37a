"""``nested_tensor`` / ``as_nested_tensor`` (nestedtensor/nested/creation.py:9-26 and the
constructor nestedtensor/csrc/creation.cpp:191-222)."""
from __future__ import annotations

import torch

from .nested import NestedTensor, _sizes_from_list, build_meta

_ADVICE = ("To form a valid NestedTensor all Tensor / NestedTensor constiuents of the given list must be of the same "
           "dimension, layout, device, scalar type and either all or none require gradients.")


def _verify(tensors):
    """nestedtensor/csrc/creation.cpp:28-171"""
    first = tensors[0]
    for t in tensors:
        if t.dim() != first.dim():
            raise RuntimeError("Given Tensor / NestedTensor constiuent of dimension {} doesn't match another constiuent "
                               "of dimension {}. {}".format(t.dim(), first.dim(), _ADVICE))
        if t.layout != first.layout:
            raise RuntimeError("Given Tensor / NestedTensor constiuent of layout {} doesn't match another constiuent "
                               "of layout {}. {}".format(t.layout, first.layout, _ADVICE))
        if t.device != first.device:
            raise RuntimeError("Given Tensor / NestedTensor constiuent of device {} doesn't match another constiuent "
                               "of device {}. ".format(t.device, first.device))
        if t.dtype != first.dtype:
            raise RuntimeError("Given Tensor / NestedTensor constiuent of scalar type {} doesn't match another "
                               "constiuent of scalar type {}. ".format(t.dtype, first.dtype))
        if t.requires_grad != first.requires_grad:
            raise RuntimeError("Given Tensor / NestedTensor constiuent requires gradient in contrast to another "
                               "constiuent. " + _ADVICE)


def nested_tensor(data, dtype=None, device=None, requires_grad=False, pin_memory=False, channels_last=False):
    """Arguments match ``torch.tensor``.  The constituents are copied into one buffer
    (storage/Packed.h:75-98) with a single concatenation, then moved/cast once."""
    if requires_grad:
        raise RuntimeError(
            "This version of nestedtensor currently does not support autograd. Please open an issue on "
            "https://github.com/pytorch/nestedtensor if you need this.")
    if dtype is None:
        dtype = torch.get_default_dtype()
    if device is None:
        device = torch.device("cpu")
    device = torch.device(device)
    if not isinstance(data, (list, tuple)):
        raise RuntimeError("Currently only supporting a flat sequence of Tensors.")
    tensors = list(data)
    for t in tensors:
        if isinstance(t, NestedTensor):
            raise RuntimeError("Currently do not support NestedTensor entries.")
        if not torch.is_tensor(t):
            raise RuntimeError("Currently only supporting a sequence of Tensors.")
    if len(tensors) > 0:
        _verify(tensors)
    sizes = _sizes_from_list(tensors)
    meta = None
    if len(tensors) == 0:
        buffer = torch.empty(0, dtype=dtype, device=device)
    elif tensors[0].is_cuda and device.type == "cuda" and tensors[0].element_size() in (1, 2, 4, 8) \
            and tensors[0].device.index == (device.index if device.index is not None else torch.cuda.current_device()) \
            and not tensors[0].is_complex():
        # constituents already on the target GPU: one pointer-array gather kernel packs them (and the same host
        # copy that carries the pointer table carries the offsets and sizes, i.e. meta)
        from . import _ops
        buffer, sizes, meta = _ops.ops().pack_list([t.detach() for t in tensors])
        if buffer.dtype != dtype:
            buffer = buffer.to(dtype)
    elif device.type == "cuda" and not tensors[0].is_cuda:
        # host constituents: concatenated straight into pinned memory, then one asynchronous copy
        src_dtype = tensors[0].dtype
        total = int(sum(t.numel() for t in tensors))
        staging = torch.empty(total, dtype=src_dtype).pin_memory()
        torch.cat([t.detach().reshape(-1) for t in tensors], out=staging)
        buffer = staging.to(device, non_blocking=True)
        if buffer.dtype != dtype:
            buffer = buffer.to(dtype)
        # the pinned block goes back to torch's host allocator, which hands it out again only after the copy
        # recorded on this stream has completed
    else:
        buffer = torch.cat([t.detach().reshape(-1) for t in tensors]).to(device=device, dtype=dtype)
        if buffer.data_ptr() == tensors[0].data_ptr():  # single contiguous constituent already in place
            buffer = buffer.clone()
    if pin_memory:
        buffer = buffer.pin_memory()
    if meta is None and device.type == "cuda":
        meta = build_meta(sizes, device)
    result = NestedTensor(buffer, sizes, meta)
    if channels_last:  # nestedtensor/csrc/creation.cpp:217-220
        result = result.contiguous(memory_format=torch.channels_last)
    return result


def as_nested_tensor(data, dtype=None, device=None, requires_grad=False, pin_memory=False):
    if not isinstance(data, NestedTensor):
        return nested_tensor(data, dtype, device, requires_grad, pin_memory)
    return data
