from .mha import multi_head_attention_forward, MultiheadAttention, bt_min_mha
from .encoder import layer_norm, transformer_encoder_layer, embedding
