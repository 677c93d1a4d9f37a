"""Self-attention on nested tensors (nestedtensor/nn/mha.py:7-83 over bt_min_mha,
nestedtensor/csrc/cuda/mha.cpp:22-107)."""
from __future__ import annotations

import torch

from .. import _ops
from ..nested import NestedTensor


def bt_min_mha(num_heads, head_dim, dropout_p, training, query, key, value, attr_kernel, attr_bias, scaling,
               out_proj_weight, out_proj_bias):
    """``torch.ops.nestedtensor.bt_min_mha`` with the reference's argument list; returns a NestedTensor with the
    query's nested size.  query is key is value: the packed self-attention path; otherwise the general form of
    ``min_mha`` (queries of sequence b over the keys / values of sequence b)."""
    if query.dim() != 3:
        raise RuntimeError("query needs to be 3 dim.")
    if not (query is key and key is value):
        # the general form (nestedtensor/csrc/mha.cpp:18-69): queries of sequence b over the keys / values of
        # sequence b of other nested tensors, e.g. a decoder's cross-attention
        if key.dim() != 3 or value.dim() != 3:
            raise RuntimeError("key and value need to be 3 dim.")
        if not torch.equal(key._sizes, value._sizes):
            raise RuntimeError("nestedtensor_b200: key and value must have the same nested size")
        qb, qs, qm = query._record()
        kb, ks, km = key._record()
        vb = kb if value is key else value._record()[0]
        out = _ops.ops().min_mha_cross(num_heads, head_dim, qb, qs, qm, kb, ks, km, vb, attr_kernel, attr_bias, float(scaling),
                                       out_proj_weight, out_proj_bias)
        return NestedTensor(out, qs, qm)
    buf, sizes, meta = query._record()
    out = _ops.ops().bt_min_mha(num_heads, head_dim, float(dropout_p), bool(training), buf, sizes, meta, attr_kernel,
                                attr_bias, float(scaling), out_proj_weight, out_proj_bias)
    return NestedTensor(out, sizes, meta)


def multi_head_attention_forward(query,
                                 key,
                                 value,
                                 embed_dim_to_check,
                                 num_heads,
                                 in_proj_weight,
                                 in_proj_bias,
                                 bias_k,
                                 bias_v,
                                 add_zero_attn,
                                 dropout_p,
                                 out_proj_weight,
                                 out_proj_bias,
                                 training=True,
                                 key_padding_mask=None,
                                 need_weights=True,
                                 attn_mask=None,
                                 use_separate_proj_weight=False,
                                 q_proj_weight=None,
                                 k_proj_weight=None,
                                 v_proj_weight=None,
                                 static_k=None,
                                 static_v=None,
                                 average_attn_weights=True,
                                 is_causal=False):
    """Stock signature; the unsupported options are rejected exactly as the reference does
    (nestedtensor/nn/mha.py:37-45).  Returns ``(output, weights)``: with ``need_weights`` the attention
    probabilities as a nested tensor of one ``(L_q,i, L_k,i)`` matrix per sequence (averaged over the heads, or
    ``(H, L_q,i, L_k,i)`` with ``average_attn_weights=False``), computed by a separate kernel; without it ``None``,
    which is what the reference returns in every case (nestedtensor/nn/mha.py:57-83).  The output projection bias is
    applied (the reference's CUDA path drops it, nestedtensor/csrc/cuda/mha.cpp:106 and nn/mha.py:69; its generic
    path adds it, nestedtensor/csrc/mha.cpp:66-67)."""
    assert isinstance(query, NestedTensor)
    assert isinstance(key, NestedTensor)
    assert isinstance(value, NestedTensor)
    assert torch.is_tensor(out_proj_weight)
    assert torch.is_tensor(out_proj_bias)
    assert not use_separate_proj_weight
    assert attn_mask is None
    assert key_padding_mask is None
    assert bias_k is None
    assert bias_v is None
    assert static_k is None
    assert static_v is None
    assert not add_zero_attn
    assert not is_causal

    bsz, tgt_len, embed_dim = query.size()
    assert embed_dim == embed_dim_to_check
    assert key.size(0) == value.size(0) and key.size(1) == value.size(1)
    head_dim = embed_dim // num_heads
    assert head_dim * num_heads == embed_dim, "embed_dim must be divisible by num_heads"
    scaling = float(head_dim) ** -0.5

    if not in_proj_weight.is_cuda:
        raise RuntimeError("nestedtensor_b200: attention needs CUDA weights (this build has no CPU implementation)")
    # self-attention runs on the tcgen05 kernels; query != key (a decoder's cross-attention, which the reference
    # leaves to its per-sequence loop, nestedtensor/nn/mha.py:57-83) on the general kernels
    out = bt_min_mha(num_heads, head_dim, dropout_p, False, query, key, value, in_proj_weight, in_proj_bias,
                     scaling, out_proj_weight, out_proj_bias)
    return out, (attention_weights(num_heads, head_dim, query, key, in_proj_weight, in_proj_bias, scaling,
                                   average_attn_weights) if need_weights else None)


def attention_weights(num_heads, head_dim, query, key, in_proj_weight, in_proj_bias, scaling, average=True):
    """softmax(scaling * q k^T) of every sequence as a nested tensor: ``(L_q,i, L_k,i)`` per sequence averaged over the
    heads, or ``(H, L_q,i, L_k,i)``.  What ``torch.nn.MultiheadAttention(need_weights=True)`` returns per sequence."""
    qb, qs, qm = query._record()
    kb, ks, km = key._record()
    w, wsizes = _ops.ops().attention_weights(num_heads, head_dim, qb, qs, qm, kb, ks, km, in_proj_weight, in_proj_bias,
                                             float(scaling), bool(average))
    return NestedTensor(w, wsizes)


class MultiheadAttention(torch.nn.MultiheadAttention):
    """``torch.nn.MultiheadAttention`` whose forward accepts NestedTensor inputs.  The reference relies on
    the stock module plus ``NestedTensor.__torch_function__``; this subclass makes the route explicit so
    that it does not depend on the stock forward's pre-checks."""

    def forward(self, query, key, value, key_padding_mask=None, need_weights=True, attn_mask=None,
                average_attn_weights=True, is_causal=False):
        if isinstance(query, NestedTensor):
            return multi_head_attention_forward(
                query, key, value, self.embed_dim, self.num_heads, self.in_proj_weight, self.in_proj_bias, self.bias_k,
                self.bias_v, self.add_zero_attn, self.dropout, self.out_proj.weight, self.out_proj.bias,
                training=self.training, key_padding_mask=key_padding_mask, need_weights=need_weights,
                attn_mask=attn_mask, average_attn_weights=average_attn_weights, is_causal=is_causal)
        return super().forward(query, key, value, key_padding_mask=key_padding_mask, need_weights=need_weights,
                               attn_mask=attn_mask, average_attn_weights=average_attn_weights, is_causal=is_causal)
