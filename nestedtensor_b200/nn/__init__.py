from .mha import multi_head_attention_forward, MultiheadAttention, bt_min_mha
