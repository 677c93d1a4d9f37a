"""The ``NestedTensor`` wrapper: a list of tensors of equal dimension stored as one ragged buffer.

Mirrors the user-facing class of the reference (nestedtensor/nested/nested.py:200-514) for the
ragged<->dense / mask / attention path.  Instead of wrapping an ``at::Tensor`` whose TensorImpl
is a NestedTensorImpl (nestedtensor/csrc/nested_tensor_impl.h:46-173), it holds the record the
kernels consume:

    _buffer  1-D tensor, constituents concatenated row-major            (nested_tensor_impl.h:167)
    _sizes   CPU int64 [B, tensor_dim], one row per constituent          (storage/EfficientSizeNode.h:53-138)
    _meta    device int64 [(B+1) + B*tensor_dim]: element offsets then sizes, built once and cached

Only nested_dim == 1 exists, as in the reference (nestedtensor/csrc/creation.cpp:182-188).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from . import _ops


def _sizes_from_list(tensors) -> torch.Tensor:
    if len(tensors) == 0:
        return torch.zeros((0, 0), dtype=torch.int64)
    return torch.tensor([list(t.shape) for t in tensors], dtype=torch.int64).reshape(len(tensors), tensors[0].dim())


def build_meta(sizes: torch.Tensor, device) -> torch.Tensor:
    """[offsets | sizes] as one int64 tensor on ``device`` (one pinned, asynchronous H2D copy).
    Host counterpart of batch_offsets_from_efficient_size (nestedtensor/csrc/masking.cpp:110-125),
    done once per nested tensor instead of once per operator call."""
    B = sizes.size(0)
    numel = sizes.prod(1) if sizes.size(1) > 0 else torch.ones(B, dtype=torch.int64)
    host = torch.empty((B + 1) + sizes.numel(), dtype=torch.int64)
    host[0] = 0
    torch.cumsum(numel, 0, out=host[1:B + 1])
    host[B + 1:] = sizes.reshape(-1)
    device = torch.device(device)
    if device.type == "cuda":
        return host.pin_memory().to(device, non_blocking=True)
    return host


class NestedTensor(object):
    def __init__(self, buffer: torch.Tensor, sizes: torch.Tensor, meta: Optional[torch.Tensor] = None,
                 channels_last: bool = False):
        if not torch.is_tensor(buffer) or buffer.dim() != 1:
            raise TypeError("Got unexpected type " + str(type(buffer)))
        if sizes.dtype != torch.int64 or sizes.dim() != 2 or sizes.device.type != "cpu":
            raise TypeError("sizes must be a CPU int64 [B, tensor_dim] tensor")
        if channels_last and sizes.size(1) != 3:
            raise RuntimeError("channels_last needs constituents of shape (C, H_i, W_i)")
        self._buffer = buffer
        self._sizes = sizes.contiguous()
        self._meta = meta
        # channels_last (nestedtensor/csrc/nested_tensor_impl.cpp:46, storage_is_contiguous_channels_last): the sizes are
        # the logical (C, H_i, W_i), every constituent is STORED as (H_i, W_i, C), i.e. with strides (1, W_i*C, C).
        self._channels_last = bool(channels_last)
        self._nchw = None  # cached contiguous copy of a channels_last tensor, made on first use by an operator

    # ---- record access -------------------------------------------------------------------
    def _record(self):
        """(buffer, sizes, meta) in the contiguous layout every operator works on; a channels_last tensor is brought
        there once (one transpose kernel) and the result is kept."""
        if self._channels_last:
            if self._nchw is None:
                self._nchw = self.contiguous()
            return self._nchw._record()
        if self._meta is None or self._meta.device != self._buffer.device:
            self._meta = build_meta(self._sizes, self._buffer.device)
        return self._buffer, self._sizes, self._meta

    def _stored_sizes(self):
        """Constituent shapes as they lie in the buffer."""
        return self._sizes[:, [1, 2, 0]].contiguous() if self._channels_last else self._sizes

    # ---- attributes ----------------------------------------------------------------------
    @property
    def dtype(self):
        return self._buffer.dtype

    @property
    def device(self):
        return self._buffer.device

    @property
    def layout(self):
        return self._buffer.layout

    @property
    def requires_grad(self):
        return False

    @property
    def is_cuda(self):
        return self._buffer.is_cuda

    @property
    def is_nested(self):
        # not a core torch.nested tensor: stock modules must not take their torch.nested branches
        return False

    @property
    def shape(self):
        return self.size()

    def is_pinned(self):
        return self._buffer.is_pinned()

    def numel(self):
        return self._buffer.numel()

    def nested_dim(self):
        return 1

    def tensor_dim(self):
        return int(self._sizes.size(1))

    def dim(self):
        return 1 + self.tensor_dim()

    def __len__(self):
        return int(self._sizes.size(0))

    def size(self, dim=None):
        """``None`` for ragged dimensions (nestedtensor/csrc/py_init.cpp:169-172)."""
        if dim is not None:
            return self.size()[dim]
        out = [len(self)]
        for j in range(self.tensor_dim()):
            col = self._sizes[:, j]
            out.append(int(col[0]) if len(self) > 0 and bool((col == col[0]).all()) else None)
        return tuple(out)

    def nested_size(self, dim=None):
        sizes = tuple(torch.Size(row) for row in self._sizes.tolist())
        if dim is None:
            return sizes
        if dim == 0:
            return len(self)
        return tuple(s[dim - 1] for s in sizes)

    def nested_stride(self, dim=None):
        strides = []
        for row in self._sizes.tolist():
            if self._channels_last:
                c, _, w = row
                strides.append((1, w * c, c))
                continue
            st, acc = [], 1
            for s in reversed(row):
                st.append(acc)
                acc *= s
            strides.append(tuple(reversed(st)))
        if dim is None:
            return tuple(strides)
        return tuple(s[dim - 1] for s in strides)

    def is_contiguous(self, memory_format=torch.contiguous_format):
        """nestedtensor/csrc/nested_tensor_impl.h (get_is_contiguous): row-major or channels_last storage."""
        if memory_format == torch.contiguous_format:
            return not self._channels_last
        if memory_format == torch.channels_last:
            return self._channels_last
        raise RuntimeError("Given memory format " + str(memory_format) + " not supported.")

    def contiguous(self, memory_format=torch.contiguous_format):
        """NestedTensor_contiguous (nestedtensor/csrc/nested_tensor_impl.cpp, transpose.cpp:87-202): to and from
        channels_last storage with one ragged transpose kernel over the whole batch."""
        if memory_format not in (torch.contiguous_format, torch.channels_last):
            raise RuntimeError("Given memory format " + str(memory_format) + " not supported.")
        want_cl = memory_format == torch.channels_last
        if want_cl == self._channels_last:
            return self
        if self.dim() != 4:
            raise RuntimeError("transpose_nchw_nhwc needs 4d input.")
        if len(self) > 0 and bool((self._sizes[:, 0] != self._sizes[0, 0]).any()):
            raise RuntimeError("Expected first dimension to be regular.")
        if not self._buffer.is_cuda:
            raise RuntimeError("nestedtensor_b200: channels_last conversion needs a CUDA nested tensor (this build has no CPU implementation)")
        ops = _ops.ops()
        if want_cl:
            buf, sizes, meta = self._record()
            return NestedTensor(ops.transpose_nchw_nhwc(buf, sizes, meta), sizes, meta, channels_last=True)
        stored = self._stored_sizes()
        out = ops.transpose_nhwc_nchw(self._buffer, stored, build_meta(stored, self._buffer.device))
        return NestedTensor(out, self._sizes)

    # ---- views of the constituents -------------------------------------------------------
    def unbind(self, dim=0):
        if dim != 0:
            raise NotImplementedError("nestedtensor_b200: unbind is only implemented for dim 0")
        out, off = [], 0
        for row in self._sizes.tolist():
            n = 1
            for s in row:
                n *= s
            piece = self._buffer[off:off + n]
            out.append(piece.reshape(row[1], row[2], row[0]).permute(2, 0, 1) if self._channels_last else piece.reshape(row))
            off += n
        return tuple(out)

    def to_tensor_list(self):
        return list(self.unbind())

    def __iter__(self):
        return iter(self.unbind())

    def __getitem__(self, key):
        if isinstance(key, int):
            return self.unbind()[key]
        raise NotImplementedError("nestedtensor_b200: only integer indexing of constituents is implemented")

    def to(self, *args, **kwargs):
        buf = self._buffer.to(*args, **kwargs)
        meta = self._meta if (self._meta is not None and self._meta.device == buf.device) else None
        return NestedTensor(buf, self._sizes, meta, channels_last=self._channels_last)

    def cuda(self, device=None):
        return self.to(torch.device("cuda") if device is None else device)

    def cpu(self):
        return self.to("cpu")

    def __str__(self):
        body = ",\n".join("  " + str(t).replace("\n", "\n  ") for t in self.unbind())
        return "nested_tensor([\n" + body + "\n])"

    __repr__ = __str__

    def __bool__(self):
        raise NotImplementedError("NestedTensor doesn't support function __bool__")

    # ---- the hot path --------------------------------------------------------------------
    def to_padded_tensor(self, padding=-1):
        """nestedtensor/nested/nested.py:509-511"""
        padding = float(padding)
        return _ops.ops().to_padded_tensor(self, padding)

    def to_tensor_mask(self, mask_dim=None):
        """(zero-padded tensor, validity mask); nestedtensor/nested/nested.py:490-507"""
        return _ops.ops().to_tensor_mask(self, mask_dim)

    # ---- operator routing ----------------------------------------------------------------
    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        """Routes ``torch.ops.nestedtensor.*`` calls made with the wrapper, and stock
        ``torch.nn.functional.multi_head_attention_forward``, to this package
        (nestedtensor/nested/nested.py:444-465).  Anything else is outside the path this
        package accelerates."""
        kwargs = kwargs or {}
        name = _packet_name(func)
        if name is not None and name in _RECORD_OPS:
            return _RECORD_OPS[name](*args, **kwargs)
        if func is torch.nn.functional.multi_head_attention_forward:
            from .nn import multi_head_attention_forward
            return multi_head_attention_forward(*args, **kwargs)
        if func is torch.nn.functional.conv2d or func is torch.conv2d:
            from .nn import conv2d
            return conv2d(*args, **kwargs)
        if func is torch.nn.functional.max_pool2d or func is torch.max_pool2d:
            from .nn import max_pool2d
            return max_pool2d(*args, **kwargs)
        if func is torch.nn.functional.embedding:
            from .nn import embedding
            return embedding(*args, **kwargs)
        if func is torch.nn.functional.layer_norm or func is torch.layer_norm:
            from .nn import layer_norm
            if func is torch.layer_norm:  # (input, normalized_shape, weight, bias, eps, cudnn_enable)
                args = args[:5]
                kwargs = {k: v for k, v in kwargs.items() if k != "cudnn_enable"}
            return layer_norm(*args, **kwargs)
        raise NotImplementedError(
            "nestedtensor_b200 implements the construction / padding / mask / attention / layer-norm path only; %s is not supported on a "
            "NestedTensor" % getattr(func, "__name__", str(func)))


def _packet_name(func):
    qual = getattr(func, "_qualified_op_name", None)  # OpOverloadPacket
    if qual is None:
        qual = getattr(func, "name", None)
        qual = qual() if callable(qual) else None  # OpOverload
    if isinstance(qual, str) and qual.startswith("nestedtensor::"):
        return qual.split("::", 1)[1].split(".")[0]
    return None


def _wrap(buffer, sizes, meta=None):
    return NestedTensor(buffer, sizes, meta)


def _op_to_padded_tensor(nt, padding):
    buf, sizes, meta = nt._record()
    return _ops.ops().to_padded_tensor(buf, sizes, meta, float(padding))


def _op_to_tensor_mask(nt, mask_dim=None):
    buf, sizes, meta = nt._record()
    return _ops.ops().to_tensor_mask(buf, sizes, meta, mask_dim)


def _op_to_mask(nt, mask_dim=None):
    _, sizes, meta = nt._record()
    return _ops.ops().to_mask(sizes, meta, mask_dim)


def _op_from_padded_tensor(padded, target):
    """``from_padded_tensor(padded, sizes-of(target))`` (nestedtensor/csrc/masking.cpp:459-533)."""
    _, sizes, meta = target._record()
    if meta.device != padded.device:
        meta = build_meta(sizes, padded.device)
    return NestedTensor(_ops.ops().from_padded_tensor(padded, sizes, meta), sizes, meta)


def _op_bt_min_mha(num_heads, head_dim, dropout_p, training, query, key, value, attr_kernel, attr_bias, scaling,
                   out_proj_weight, out_proj_bias):
    from .nn import mha
    return mha.bt_min_mha(num_heads, head_dim, dropout_p, training, query, key, value, attr_kernel, attr_bias,
                          scaling, out_proj_weight, out_proj_bias)


def _op_transpose_nchw_nhwc(nt):
    from .nn import transpose_nchw_nhwc
    return transpose_nchw_nhwc(nt)


def _op_transpose_nhwc_nchw(nt):
    from .nn import transpose_nhwc_nchw
    return transpose_nhwc_nchw(nt)


def _op_get_max_size(nt):
    """``torch.ops.nestedtensor.get_max_size`` (nestedtensor/csrc/masking.cpp:105-108)."""
    return list(_ops.ops().get_max_size(nt._sizes))


def _op_pad_nt(nt, shape):
    """``torch.ops.nestedtensor.pad_nt`` (nestedtensor/csrc/masking.cpp:138-179)."""
    buf, sizes, meta = nt._record()
    return _ops.ops().pad_nt(buf, sizes, meta, list(shape))


_RECORD_OPS = {
    "get_max_size": _op_get_max_size,
    "pad_nt": _op_pad_nt,
    "min_mha": _op_bt_min_mha,
    "transpose_nchw_nhwc": _op_transpose_nchw_nhwc,
    "transpose_nhwc_nchw": _op_transpose_nhwc_nchw,
    "to_padded_tensor": _op_to_padded_tensor,
    "to_tensor_mask": _op_to_tensor_mask,
    "to_mask": _op_to_mask,
    "from_padded_tensor": _op_from_padded_tensor,
    "bt_min_mha": _op_bt_min_mha,
}
