"""Image-shaped nested tensors: ragged NCHW <-> NHWC transposes and the convolution / pooling callers of the
padding path (nestedtensor/csrc/transpose.cpp:87-202, nestedtensor/csrc/conv2d.cpp:19-106,
nestedtensor/csrc/pooling.cpp:33-71).

A batch of images ``(C, H_i, W_i)`` goes through

* a 1x1 convolution as transpose -> ONE packed GEMM over all pixels of all images -> transpose (no padding);
* any other convolution, and max pooling, as ``to_padded_tensor`` -> the dense library operator ->
  ``from_padded_tensor`` with the per-image output sizes.
"""
from __future__ import annotations

import torch

from .. import _ops
from ..nested import NestedTensor, build_meta


def _pair(v):
    return (int(v), int(v)) if isinstance(v, int) else (int(v[0]), int(v[1]))


def transpose_nchw_nhwc(input: NestedTensor) -> NestedTensor:
    """``(C, H_i, W_i)`` constituents to ``(H_i, W_i, C)`` (nestedtensor/csrc/transpose.cpp:124-150)."""
    buf, sizes, meta = input._record()
    out = _ops.ops().transpose_nchw_nhwc(buf, sizes, meta)
    return NestedTensor(out, sizes[:, [1, 2, 0]].contiguous())


def transpose_nhwc_nchw(input: NestedTensor) -> NestedTensor:
    """``(H_i, W_i, C)`` constituents to ``(C, H_i, W_i)`` (nestedtensor/csrc/transpose.cpp:186-202)."""
    buf, sizes, meta = input._record()
    out = _ops.ops().transpose_nhwc_nchw(buf, sizes, meta)
    return NestedTensor(out, sizes[:, [2, 0, 1]].contiguous())


def _window_out(n, pad, dil, k, stride):
    return (n + 2 * pad - dil * (k - 1) - 1) // stride + 1


def conv2d(input: NestedTensor, weight, bias=None, stride=1, padding=0, dilation=1, groups=1) -> NestedTensor:
    """``torch.nn.functional.conv2d`` on a NestedTensor of ``(C, H_i, W_i)`` images
    (nestedtensor/csrc/conv2d.cpp:19-106)."""
    if input.dim() != 4:
        raise RuntimeError("Expected input to be dim 4, but got %d." % input.dim())
    if isinstance(padding, str):
        raise NotImplementedError("nestedtensor_b200: string padding modes are not supported")
    stride, padding, dilation = _pair(stride), _pair(padding), _pair(dilation)
    sizes = input._sizes
    if bool((sizes[:, 0] != sizes[0, 0]).any()):
        raise RuntimeError("Expected first dimension to be regular.")
    ops = _ops.ops()
    cout, _, kh, kw = weight.shape
    if (bias is None and kh == 1 and kw == 1 and stride == (1, 1) and padding == (0, 0) and dilation == (1, 1) and groups == 1
            and input.dtype in (torch.float16, torch.bfloat16, torch.float32)):
        # pointwise convolution: every pixel of every image is one row of a single packed GEMM.  A channels_last input is
        # stored pixel-major already and the result stays channels_last: no transpose on either side.
        cl = input._channels_last
        pixels = input._buffer if cl else transpose_nchw_nhwc(input)._buffer
        cin = int(sizes[0, 0])
        y = ops.packed_linear(pixels.view(-1, cin), weight.reshape(cout, cin), None, 0, None)
        if cl:
            out_sizes = sizes.clone()
            out_sizes[:, 0] = cout
            return NestedTensor(y.reshape(-1), out_sizes, channels_last=True)
        nhwc = sizes[:, [1, 2, 0]].contiguous()
        nhwc[:, 2] = cout
        return transpose_nhwc_nchw(NestedTensor(y.reshape(-1), nhwc))
    buf, sizes, meta = input._record()
    dense = ops.to_padded_tensor(buf, sizes, meta, 0.0)
    res = torch.nn.functional.conv2d(dense, weight, bias, stride, padding, dilation, groups)
    new_sizes = sizes.clone()
    new_sizes[:, 0] = cout
    new_sizes[:, 1] = torch.div(sizes[:, 1] + 2 * padding[0] - dilation[0] * (kh - 1) - 1, stride[0], rounding_mode="floor") + 1
    new_sizes[:, 2] = torch.div(sizes[:, 2] + 2 * padding[1] - dilation[1] * (kw - 1) - 1, stride[1], rounding_mode="floor") + 1
    new_meta = build_meta(new_sizes, buf.device)
    return NestedTensor(ops.from_padded_tensor(res.contiguous(), new_sizes, new_meta), new_sizes, new_meta)


def max_pool2d(input: NestedTensor, kernel_size, stride=None, padding=0, dilation=1, ceil_mode=False,
               return_indices=False) -> NestedTensor:
    """``torch.nn.functional.max_pool2d`` on a NestedTensor of ``(C, H_i, W_i)`` images
    (nestedtensor/csrc/pooling.cpp:33-71).  The batch is padded with -inf, not 0, so that windows reaching past
    an image see what the dense operator's own implicit padding would show them."""
    if input.dim() != 4:
        raise RuntimeError("Input must be 4 dimensional.")
    if ceil_mode or return_indices:
        raise NotImplementedError("nestedtensor_b200: max_pool2d with ceil_mode / return_indices is not supported")
    kernel_size = _pair(kernel_size)
    stride = kernel_size if stride is None or stride == [] else _pair(stride)
    padding, dilation = _pair(padding), _pair(dilation)
    buf, sizes, meta = input._record()
    ops = _ops.ops()
    dense = ops.to_padded_tensor(buf, sizes, meta, float("-inf"))
    res = torch.nn.functional.max_pool2d(dense, kernel_size, stride, padding, dilation, False)
    new_sizes = sizes.clone()
    new_sizes[:, 1] = torch.div(sizes[:, 1] + 2 * padding[0] - dilation[0] * (kernel_size[0] - 1) - 1, stride[0],
                                rounding_mode="floor") + 1
    new_sizes[:, 2] = torch.div(sizes[:, 2] + 2 * padding[1] - dilation[1] * (kernel_size[1] - 1) - 1, stride[1],
                                rounding_mode="floor") + 1
    new_meta = build_meta(new_sizes, buf.device)
    return NestedTensor(ops.from_padded_tensor(res.contiguous(), new_sizes, new_meta), new_sizes, new_meta)
