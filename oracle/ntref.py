"""CPU restatement of the reference's ragged<->dense / mask / MHA path.

TEST INFRASTRUCTURE ONLY: this module is the checker.  The product package never
imports it; the only callers are the test-suite, the smoke check and the
benchmark's CPU-baseline / reference arm.

A nested tensor is represented here as a plain Python ``list`` of CPU tensors
(nested_dim 1, the only nesting depth the reference enables,
nestedtensor/csrc/creation.cpp:182-188).  Every function names the reference
lines it restates.  The arithmetic the reference delegates to ATen
(``constant_pad_nd``, ``stack``, ``masked_select``, ``matmul``, ``softmax``) is
delegated to the same ATen operators of the installed torch.

Parity status: PINNED.  tests/test_oracle_golden.py replays the literal
input/output tensors of the reference's own tests
(test/test_nested_tensor_masking.py) against these functions, and checks
``min_mha`` against stock ``torch.nn.functional.multi_head_attention_forward``
with ``key_padding_mask`` exactly as test/test_nested_tensor_functional.py:648-667
and :1040-1161 do.  The functions added for the rows around the core path are
pinned the same way: ``layer_norm`` against ``torch.nn.LayerNorm`` applied to each
constituent (the reference's own check, test/test_nested_tensor_functional.py:895-957),
``encoder_layer`` against stock ``torch.nn.TransformerEncoderLayer`` evaluated per
sequence, ``embedding`` / ``conv2d`` / ``max_pool2d`` / the NCHW<->NHWC transposes are
the per-constituent ATen calls of the reference's generic branches themselves.

Deliberate differences from the reference (its defects are not reproduced):
  * a scalar constituent is appended twice by the reference's CPU
    ``to_padded_tensor`` (masking.cpp:643-646); here it is appended once;
  * ``from_padded_tensor`` pads its masks to the padded tensor's own trailing
    shape instead of the per-dimension maximum of the target sizes
    (masking.cpp:511-512), so a padded tensor wider than the largest constituent
    is accepted like on the reference's CUDA path (masking.cpp:463-509).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

NTList = List[torch.Tensor]


# --------------------------------------------------------------------------- sizes
def nt_dim(tensors: NTList) -> int:
    """dim of the nested tensor = 1 + dim of a constituent (nested_tensor_impl.h:201-280)."""
    if len(tensors) == 0:
        return 1
    return 1 + tensors[0].dim()


def get_max_size(tensors: NTList) -> List[int]:
    """Per-dimension maximum over constituents (masking.cpp:60-108)."""
    if len(tensors) == 0:
        return []
    result = list(tensors[0].shape)
    for t in tensors[1:]:
        for j, s in enumerate(t.shape):
            if s > result[j]:
                result[j] = s
    return result


def opt_sizes(tensors: NTList) -> List[Optional[int]]:
    """``nt.size()``: common size per dim or None (storage/EfficientSizeNode.h:27-49)."""
    out: List[Optional[int]] = [len(tensors)]
    if len(tensors) == 0:
        return out
    for j in range(tensors[0].dim()):
        vals = {int(t.shape[j]) for t in tensors}
        out.append(vals.pop() if len(vals) == 1 else None)
    return out


def pad_tensor_to_shape(t: torch.Tensor, goal_shape: Sequence[int], value=0) -> torch.Tensor:
    """masking.cpp:45-58 — right-pad every dimension up to ``goal_shape``."""
    if t.dim() != len(goal_shape):
        raise RuntimeError("dimension doesn't match length of goal shape.")
    padd = []
    for i in range(t.dim() - 1, -1, -1):
        padd.append(0)
        padd.append(int(goal_shape[i]) - int(t.shape[i]))
    new_tensor = F.pad(t, padd, mode="constant", value=value) if padd else t
    return new_tensor.reshape(list(goal_shape))


# ----------------------------------------------------------------- to_padded_tensor
def to_padded_tensor(tensors: NTList, padding: float) -> torch.Tensor:
    """CPU branch of ``to_padded_tensor`` (masking.cpp:624-649)."""
    osz = opt_sizes(tensors)
    if len(osz) == 1 and osz[0] == 1:
        return tensors[0].reshape(-1)
    max_size = get_max_size(tensors)
    if len(tensors) == 0:
        return torch.tensor([float(padding)], dtype=torch.float64)
    res = []
    for t in tensors:
        if t.numel() == 0:
            raise RuntimeError("Empty tensors are not yet supported.")
        res.append(pad_tensor_to_shape(t, max_size, padding))
    return torch.stack(res)


# -------------------------------------------------------------------- to_tensor_mask
def pad_nt(tensors: NTList, shape: Sequence[int]) -> Tuple[torch.Tensor, torch.Tensor]:
    """masking.cpp:138-179 — zero-padded data and a uint8 validity mask, stacked."""
    if len(tensors) == 0:
        return torch.tensor([0]), torch.tensor([False], dtype=torch.uint8)
    res_t, res_m = [], []
    for t in tensors:
        if t.numel() == 0:
            raise RuntimeError("Empty tensors are not yet supported.")
        if t.dim() == 0:
            res_t.append(t)
            res_m.append(torch.tensor(True))
            continue
        res_t.append(pad_tensor_to_shape(t, shape))
        res_m.append(pad_tensor_to_shape(torch.full(t.shape, 1, dtype=torch.uint8), shape))
    return torch.stack(res_t), torch.stack(res_m)


def merge_tensor_mask(tensor: torch.Tensor, mask: torch.Tensor, mask_dim: Optional[int]):
    """masking.cpp:12-43 — drop trailing mask dims whose slices are all-0 or all-1."""
    if mask_dim is not None and mask.dim() == mask_dim:
        return tensor, mask
    if mask.dim() == 0:
        return tensor, mask
    last_size = mask.size(-1)
    collapsed = mask.sum(-1)
    is_last_size_sum = int((collapsed == last_size).sum().item())
    is_zero_sum = int((collapsed == 0).sum().item())
    if is_last_size_sum + is_zero_sum == collapsed.numel():
        return merge_tensor_mask(tensor, collapsed.to(torch.bool), mask_dim)
    if mask_dim is not None and mask_dim != mask.dim():
        raise RuntimeError("Mask dimension is too small to represent data tensor.")
    return tensor.contiguous(), mask.contiguous()


def to_tensor_mask(tensors: NTList, mask_dim: Optional[int] = None):
    """Generic branch of ``to_tensor_mask`` (masking.cpp:297-319)."""
    d = nt_dim(tensors)
    if mask_dim is not None and mask_dim > d:
        raise RuntimeError(
            "Requested mask dimension {} is bigger than dimension {} of given NestedTensor.".format(mask_dim, d))
    osz = opt_sizes(tensors)
    if len(osz) == 1 and osz[0] == 1:
        buf = tensors[0].reshape(-1)
        m = torch.tensor(True) if (mask_dim is None or mask_dim == 0) else torch.tensor([True])
        return buf, m
    max_size = get_max_size(tensors)
    t, m = pad_nt(tensors, max_size)
    return merge_tensor_mask(t, m, mask_dim)


# --------------------------------------------------------------------------- to_mask
def merge_mask(mask: torch.Tensor, mask_dim: Optional[int]) -> torch.Tensor:
    """masking.cpp:322-351."""
    return merge_tensor_mask(mask, mask, mask_dim)[1]


def _create_nt_mask(sizes: Sequence[int], shape: Sequence[int]) -> torch.Tensor:
    """masking.cpp:353-372."""
    numel = 1
    for s in sizes:
        numel *= int(s)
    if not numel > 0:
        raise RuntimeError("Empty tensors are not yet supported.")
    if len(sizes) == 0:
        return torch.tensor(True)
    return pad_tensor_to_shape(torch.full(list(sizes), 1, dtype=torch.uint8), shape)


def to_mask(tensors: NTList, mask_dim: Optional[int]) -> torch.Tensor:
    """masking.cpp:408-457 — the mask alone, from sizes only."""
    d = nt_dim(tensors)
    if mask_dim is not None and mask_dim > d:
        raise RuntimeError(
            "Requested mask dimension {} is bigger than dimension {} of given NestedTensor.".format(mask_dim, d))
    osz = opt_sizes(tensors)
    if len(osz) == 1 and osz[0] == 1:
        return torch.tensor(True) if (mask_dim is None or mask_dim == 0) else torch.tensor([True])
    if d > 1 and mask_dim is not None and mask_dim > 1:
        tmp_max = get_max_size(tensors)
        max_size = [tmp_max[i - 1] for i in range(1, mask_dim)]
        if mask_dim == 2 and d == 3:
            # literal host double loop of masking.cpp:436-451
            result = torch.zeros((osz[0], tmp_max[0]), dtype=torch.uint8)
            for i, t in enumerate(tensors):
                for j in range(int(t.shape[0])):
                    result[i, j] = 1
            return result
        masks = [_create_nt_mask(list(t.shape[: len(max_size)]), max_size) for t in tensors]
        return torch.stack(masks)
    max_size = get_max_size(tensors)
    if len(tensors) == 0:
        return merge_mask(torch.tensor([False], dtype=torch.uint8), mask_dim)
    masks = [_create_nt_mask(list(t.shape), max_size) for t in tensors]
    return merge_mask(torch.stack(masks), mask_dim)


# ---------------------------------------------------------------- from_padded_tensor
def from_padded_tensor(padded: torch.Tensor, sizes: Sequence[Sequence[int]]) -> NTList:
    """CPU branch of ``from_padded_tensor`` (masking.cpp:511-532): per-constituent
    ones-mask padded to the dense shape, ``stack``, ``masked_select``; then the flat
    buffer is cut back into constituents (storage/Packed.h:21-64)."""
    if len(sizes) > 0 and padded.dim() != 1 + len(sizes[0]):
        raise RuntimeError("Target size has different dimension as input padded Tensor.")
    goal = list(padded.shape[1:])
    masks = []
    for s in sizes:
        m = torch.full(list(s), 1, dtype=torch.uint8)
        masks.append(pad_tensor_to_shape(m, goal))
    final_mask = torch.stack(masks).to(torch.bool)
    buf = padded.masked_select(final_mask)
    out, off = [], 0
    for s in sizes:
        n = int(math.prod(s))
        out.append(buf[off:off + n].reshape(list(s)))
        off += n
    return out


def _nt_from_tensor_mask_nd0(tensor: torch.Tensor, mask: torch.Tensor):
    """nested_dim == 0 branch of masking.cpp:185-222 (one host sync per mask element)."""
    if mask.numel() == 0 or (mask.numel() == 1 and bool(mask.item())):
        return tensor
    if mask.dim() == 1:
        keep = [tensor[i] for i in range(mask.size(0)) if bool(mask[i].item())]
        if len(keep) == 0:
            return torch.tensor([]).to(tensor)
        return torch.stack(keep)
    if mask.dim() > 1:
        keep, all_zero = [], True
        for i in range(mask.size(0)):
            tmp = _nt_from_tensor_mask_nd0(tensor[i], mask[i])
            if tmp.numel() > 0:
                all_zero = False
                keep.append(tmp)
        if all_zero:
            for i in range(mask.size(0)):
                keep.append(_nt_from_tensor_mask_nd0(tensor[i], mask[i]))
        if len(keep) == 0:
            return torch.tensor([]).to(tensor)
        return torch.stack(keep)
    return None


def nt_from_tensor_mask(tensor: torch.Tensor, mask: torch.Tensor, nested_dim: int) -> NTList:
    """masking.cpp:181-249 for nested_dim == 1; returns the list of constituents."""
    if nested_dim != 1:
        raise RuntimeError("Only nested_dim of 1 is currently supported.")
    inner = []
    if mask.numel() == 0 or (mask.numel() == 1 and bool(mask.item())):
        for i in range(tensor.size(0)):
            inner.append(_nt_from_tensor_mask_nd0(tensor[i], mask))
    elif mask.numel() == 1 and not bool(mask.item()):
        inner.append(None)
    else:
        for i in range(tensor.size(0)):
            inner.append(_nt_from_tensor_mask_nd0(tensor[i], mask[i]))
    return [t for t in inner if t is not None]


def nested_tensor_from_tensor_mask(tensor, mask, nested_dim=1) -> NTList:
    """Argument checks of nestedtensor/nested/masking.py:18-43, then the op."""
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
    return nt_from_tensor_mask(tensor, mask, nested_dim)


def nested_tensor_from_padded_tensor(tensor, nested_dim=1, padding=-1) -> NTList:
    """nestedtensor/nested/masking.py:12-14."""
    return nested_tensor_from_tensor_mask(tensor, tensor != padding, nested_dim)


def from_padded_by_value_fast(tensor: torch.Tensor, padding) -> NTList:
    """Vectorised equivalent of ``nested_tensor_from_padded_tensor`` for the case the
    literal per-element recursion cannot finish (anything beyond a few thousand
    elements): constituent b is ``tensor[b, :s_1, :s_2, ...]`` with s_j one past the
    last index along dim j that holds a non-padding element.  Identical to
    masking.cpp:181-249 whenever no valid element equals ``padding``."""
    out = []
    for b in range(tensor.size(0)):
        nz = (tensor[b] != padding).nonzero()
        if nz.numel() == 0:
            out.append(torch.tensor([]).to(tensor))
            continue
        hi = nz.max(0).values + 1
        sl = tuple(slice(0, int(h)) for h in hi)
        out.append(tensor[b][sl].contiguous())
    return out


# ------------------------------------------------------------------------------ MHA
def min_mha(num_heads: int, head_dim: int, query: NTList, key: NTList, value: NTList,
            in_proj_weight: torch.Tensor, in_proj_bias: torch.Tensor, scaling: float,
            out_proj_weight: torch.Tensor, out_proj_bias: torch.Tensor) -> NTList:
    """nestedtensor/csrc/mha.cpp:18-69, evaluated per constituent in fp32
    (dropout is the identity at inference, :63)."""
    E = num_heads * head_dim
    W = in_proj_weight.float()
    bias = in_proj_bias.float()
    Wq, Wk, Wv = W[:E].t().contiguous(), W[E:2 * E].t().contiguous(), W[2 * E:].t().contiguous()
    bq, bk, bv = bias[:E], bias[E:2 * E], bias[2 * E:]
    Wo = out_proj_weight.float().t()
    bo = out_proj_bias.float()
    out = []
    for xq, xk, xv in zip(query, key, value):
        q = (xq.float() @ Wq + bq) * scaling
        k = xk.float() @ Wk + bk
        v = xv.float() @ Wv + bv
        q = q.reshape(-1, num_heads, head_dim).transpose(0, 1)
        k = k.reshape(-1, num_heads, head_dim).transpose(0, 1)
        v = v.reshape(-1, num_heads, head_dim).transpose(0, 1)
        w = torch.softmax(q @ k.transpose(1, 2), -1)
        o = (w @ v).transpose(0, 1).reshape(-1, E)
        out.append(o @ Wo + bo)
    return out


def mha_weights(num_heads: int, head_dim: int, query: NTList, key: NTList, in_proj_weight: torch.Tensor,
                in_proj_bias: torch.Tensor, scaling: float, average: bool = True) -> NTList:
    """The attention probabilities inside min_mha (nestedtensor/csrc/mha.cpp:55-62: softmax of the scaled q k^T of
    every constituent), which the reference computes and discards - its Python layer returns None for the weights
    (nestedtensor/nn/mha.py:57-83).  One (L_q, L_k) matrix per constituent averaged over the heads, as
    torch.nn.MultiheadAttention(need_weights=True) does, or (H, L_q, L_k)."""
    E = num_heads * head_dim
    W = in_proj_weight.float()
    bias = in_proj_bias.float()
    Wq, Wk = W[:E].t().contiguous(), W[E:2 * E].t().contiguous()
    bq, bk = bias[:E], bias[E:2 * E]
    out = []
    for xq, xk in zip(query, key):
        q = ((xq.float() @ Wq + bq) * scaling).reshape(-1, num_heads, head_dim).transpose(0, 1)
        k = (xk.float() @ Wk + bk).reshape(-1, num_heads, head_dim).transpose(0, 1)
        w = torch.softmax(q @ k.transpose(1, 2), -1)
        out.append(w.mean(0) if average else w)
    return out


def masked_softmax(scores: torch.Tensor, mask: torch.Tensor, scaling: float) -> torch.Tensor:
    """The live softmax of the reference's CUDA MHA
    (nestedtensor/csrc/cuda/attention.cu:182-225): ``softmax(S*scaling + (1-mask)*-10000)``
    over the last dim with ``1e-6`` added to the row sum; scores (B,H,L,L), mask (B,L,L)."""
    s = scores.float() * scaling + (1.0 - mask.float()).unsqueeze(1) * -10000.0
    s = s - s.max(-1, keepdim=True).values
    e = torch.exp(s)
    return e / (e.sum(-1, keepdim=True) + 1e-6)


# ------------------------------------------------------- layer norm and the encoder layer
def layer_norm(tensors: NTList, normalized_shape, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor],
               eps: float = 1e-5) -> NTList:
    """nestedtensor/csrc/functions.cpp:65-110 (CPU branch: ``at::layer_norm`` mapped over the constituents),
    with its checks; evaluated in fp32."""
    if isinstance(normalized_shape, int):
        normalized_shape = (normalized_shape,)
    if len(normalized_shape) != 1:
        raise RuntimeError("Currently only singleton tuples of integers supported for layer_norm.")
    if len(tensors) == 0:
        return []
    last = tensors[0].dim()  # index of the last dimension of the nested tensor
    if any(t.size(-1) != tensors[0].size(-1) for t in tensors):
        raise RuntimeError("Cannot normalize across irregular dimension %d" % last)
    if tensors[0].size(-1) != normalized_shape[0]:
        raise RuntimeError("Normalized shape [%d] does not match the size of the last dimension (%d) of input."
                           % (normalized_shape[0], tensors[0].size(-1)))
    if (weight is None) != (bias is None):
        raise RuntimeError("Either both weight and bias are used or not.")
    w = None if weight is None else weight.float()
    b = None if bias is None else bias.float()
    return [F.layer_norm(t.float(), tuple(normalized_shape), w, b, eps) for t in tensors]


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    """The GELU of the reference's fused kernels (nestedtensor/csrc/cuda/cuda_kernels.cu:29-36)."""
    x = x.float()
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)))


def encoder_layer(tensors: NTList, num_heads: int, p: dict, activation: str = "gelu_tanh", norm_first: bool = False,
                  eps: float = 1e-5) -> NTList:
    """One transformer encoder layer (self-attention + feed-forward, inference) per constituent in fp32, built
    from ``min_mha`` (nestedtensor/csrc/mha.cpp:18-69) and ``layer_norm`` above, in the order of
    ``torch.nn.TransformerEncoderLayer``.  ``p`` holds in_proj_weight/bias, out_proj_weight/bias,
    linear1_weight/bias, linear2_weight/bias, norm1_weight/bias, norm2_weight/bias."""
    f = {k: v.float() for k, v in p.items()}
    E = f["out_proj_weight"].size(0)
    head_dim = E // num_heads
    act = {"gelu_tanh": gelu_tanh, "relu": torch.relu}[activation]

    def sa(xs):
        return min_mha(num_heads, head_dim, xs, xs, xs, f["in_proj_weight"], f["in_proj_bias"], float(head_dim) ** -0.5,
                       f["out_proj_weight"], f["out_proj_bias"])

    def ff(xs):
        return [act(x @ f["linear1_weight"].t() + f["linear1_bias"]) @ f["linear2_weight"].t() + f["linear2_bias"] for x in xs]

    def ln(xs, which):
        return layer_norm(xs, (E,), f[which + "_weight"], f[which + "_bias"], eps)

    xs = [t.float() for t in tensors]
    if norm_first:
        xs = [x + a for x, a in zip(xs, sa(ln(xs, "norm1")))]
        return [x + h for x, h in zip(xs, ff(ln(xs, "norm2")))]
    xs = ln([x + a for x, a in zip(xs, sa(xs))], "norm1")
    return ln([x + h for x, h in zip(xs, ff(xs))], "norm2")


def embedding(indices: NTList, weight: torch.Tensor) -> NTList:
    """nestedtensor/csrc/functions.cpp:57-63 (``at::embedding`` mapped over the constituents; the packed fast
    path :29-56 is the same gather on the concatenated indices)."""
    return [F.embedding(i.long(), weight) for i in indices]


# ---------------------------------------------------------------- image-shaped nested tensors
def transpose_nchw_nhwc(tensors: NTList) -> NTList:
    """nestedtensor/csrc/transpose.cpp:124-150: each (C, H, W) constituent as (H, W, C)."""
    return [t.permute(1, 2, 0).contiguous() for t in tensors]


def transpose_nhwc_nchw(tensors: NTList) -> NTList:
    """nestedtensor/csrc/transpose.cpp:186-202: each (H, W, C) constituent as (C, H, W)."""
    return [t.permute(2, 0, 1).contiguous() for t in tensors]


def conv2d(tensors: NTList, weight, bias=None, stride=1, padding=0, dilation=1, groups=1) -> NTList:
    """nestedtensor/csrc/conv2d.cpp:91-105: ``at::conv2d`` on each constituent, in fp32."""
    b = None if bias is None else bias.float()
    return [F.conv2d(t.float().unsqueeze(0), weight.float(), b, stride, padding, dilation, groups).squeeze(0) for t in tensors]


def max_pool2d(tensors: NTList, kernel_size, stride=None, padding=0, dilation=1) -> NTList:
    """nestedtensor/csrc/pooling.cpp:58-70: ``at::max_pool2d`` on each constituent."""
    return [F.max_pool2d(t.unsqueeze(0), kernel_size, stride, padding, dilation, False).squeeze(0) for t in tensors]
