"""Self-attention on nested tensors (nestedtensor/nn/mha.py:7-83, nestedtensor/csrc/cuda/mha.cpp:22-107)."""
from __future__ import annotations

import torch


def bt_min_mha(num_heads, head_dim, dropout_p, training, query, key, value, attr_kernel, attr_bias, scaling,
               out_proj_weight, out_proj_bias):
    raise NotImplementedError("nestedtensor_b200: the attention kernels are not built yet")


def multi_head_attention_forward(*args, **kwargs):
    raise NotImplementedError("nestedtensor_b200: the attention kernels are not built yet")


class MultiheadAttention(torch.nn.MultiheadAttention):
    """Stock ``torch.nn.MultiheadAttention``; called with NestedTensor inputs its forward reaches
    ``multi_head_attention_forward`` above through ``NestedTensor.__torch_function__``."""
