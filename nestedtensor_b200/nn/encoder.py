"""A transformer encoder layer on nested tensors, tokens packed (never padded) from end to end.

    x  ->  QKV projection  ->  varlen self-attention  ->  output projection (+ bias + residual, fused)
       ->  LayerNorm  ->  linear1 (+ bias + activation, fused)  ->  linear2 (+ bias + residual, fused)  ->  LayerNorm

Seven kernels per layer (four tcgen05 GEMMs with fused epilogues, the attention kernel with its work list,
two row-wise LayerNorms); the reference has the building blocks (bt_min_mha,
nestedtensor/csrc/cuda/mha.cpp:22-107; NestedTensor_layer_norm, nestedtensor/csrc/cuda/layernorm.cpp:14-76;
add_bias_act / add_bias_input_layernorm, nestedtensor/csrc/cuda/cuda_kernels.cu:73-159) and runs the
feed-forward part through per-sequence ATen calls.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _ops
from ..nested import NestedTensor

ACTIVATIONS = {"none": 0, "gelu_tanh": 1, "relu": 2}


def layer_norm(input: NestedTensor, normalized_shape, weight=None, bias=None, eps: float = 1e-5) -> NestedTensor:
    """``torch.nn.functional.layer_norm`` on a NestedTensor (nestedtensor/csrc/functions.cpp:65-110): the
    last dimension must be regular and equal ``normalized_shape``, a singleton."""
    if isinstance(normalized_shape, int):
        normalized_shape = (normalized_shape,)
    buf, sizes, meta = input._record()
    out = _ops.ops().layer_norm(buf, sizes, meta, list(normalized_shape), weight, bias, float(eps))
    return NestedTensor(out, sizes, meta)


def _activation_code(layer: torch.nn.TransformerEncoderLayer, activation: Optional[str]) -> int:
    if activation is None:
        fn = getattr(layer, "activation", None)
        if fn is torch.nn.functional.relu or isinstance(fn, torch.nn.ReLU):
            activation = "relu"
        elif isinstance(fn, torch.nn.GELU) and getattr(fn, "approximate", "none") == "tanh":
            activation = "gelu_tanh"
        else:
            raise NotImplementedError(
                "nestedtensor_b200: the fused feed-forward epilogue implements relu and the tanh form of gelu "
                "(torch.nn.GELU(approximate='tanh')); pass activation='relu' or 'gelu_tanh' explicitly to override")
    if activation not in ("relu", "gelu_tanh"):
        raise ValueError("activation must be 'relu' or 'gelu_tanh'")
    return ACTIVATIONS[activation]


def transformer_encoder_layer(layer: torch.nn.TransformerEncoderLayer, src: NestedTensor,
                              activation: Optional[str] = None) -> NestedTensor:
    """Forward of a stock ``torch.nn.TransformerEncoderLayer`` (inference; dropout is the identity) on a
    NestedTensor of ``(L_i, E)`` sequences, post-norm or pre-norm (``norm_first``)."""
    if not isinstance(src, NestedTensor):
        raise TypeError("src must be a NestedTensor")
    if src.dim() != 3:
        raise RuntimeError("query needs to be 3 dim.")
    if layer.training:
        raise NotImplementedError("nestedtensor_b200: inference only (call layer.eval())")
    attn = layer.self_attn
    if not getattr(attn, "_qkv_same_embed_dim", True) or attn.in_proj_bias is None or attn.bias_k is not None or attn.add_zero_attn:
        raise NotImplementedError("nestedtensor_b200: the packed self-attention needs one in_proj weight with bias")
    act = _activation_code(layer, activation)
    ops = _ops.ops()
    buf, sizes, meta = src._record()
    E, H = attn.embed_dim, attn.num_heads
    d = E // H
    T = buf.numel() // E
    x = buf.view(T, E)

    def self_attention(inp, residual):
        a = ops.bt_min_mha_core(H, d, inp.reshape(-1), sizes, meta, attn.in_proj_weight, attn.in_proj_bias, float(d) ** -0.5)
        return ops.packed_linear(a.view(T, E), attn.out_proj.weight, attn.out_proj.bias, 0, residual)

    def feed_forward(inp, residual):
        h = ops.packed_linear(inp, layer.linear1.weight, layer.linear1.bias, act, None)
        return ops.packed_linear(h, layer.linear2.weight, layer.linear2.bias, 0, residual)

    def norm(m, inp):
        return ops.add_bias_residual_layer_norm(inp, None, None, m.weight, m.bias, float(m.eps))

    if getattr(layer, "norm_first", False):
        x1 = self_attention(norm(layer.norm1, x), x)
        out = feed_forward(norm(layer.norm2, x1), x1)
    else:
        x1 = norm(layer.norm1, self_attention(x, x))
        out = norm(layer.norm2, feed_forward(x1, x1))
    return NestedTensor(out.reshape(-1), sizes, meta)


def transformer_encoder(encoder: torch.nn.TransformerEncoder, src: NestedTensor, activation: Optional[str] = None) -> NestedTensor:
    """Forward of a stock ``torch.nn.TransformerEncoder`` (its layers in turn, then its final norm if it has one) on
    a NestedTensor; the tokens stay packed from the first layer to the last."""
    out = src
    for layer in encoder.layers:
        out = transformer_encoder_layer(layer, out, activation)
    if encoder.norm is not None:
        out = layer_norm(out, encoder.norm.normalized_shape, encoder.norm.weight, encoder.norm.bias, encoder.norm.eps)
    return out


def embedding(input: NestedTensor, weight: torch.Tensor, padding_idx=None, max_norm=None, norm_type=2.0,
              scale_grad_by_freq=False, sparse=False) -> NestedTensor:
    """``torch.nn.functional.embedding`` on a NestedTensor of 1-D index sequences
    (nestedtensor/csrc/functions.cpp:29-56): one gather on the packed index buffer; the result holds
    ``(L_i, embedding_dim)`` constituents.  ``padding_idx``, ``scale_grad_by_freq`` and ``sparse`` only
    affect gradients and are ignored at inference; ``max_norm`` (which rewrites the weight) is not supported."""
    if max_norm is not None:
        raise NotImplementedError("nestedtensor_b200: embedding with max_norm is not supported")
    if input.dim() != 2:
        raise NotImplementedError("nestedtensor_b200: embedding expects a nested tensor of 1-D index sequences")
    buf, sizes, meta = input._record()
    out = _ops.ops().embedding(weight, buf, sizes, meta)
    E = weight.size(1)
    new_sizes = torch.cat([sizes, torch.full((sizes.size(0), 1), E, dtype=torch.int64)], 1).contiguous()
    return NestedTensor(out, new_sizes)
