from .mha import multi_head_attention_forward, MultiheadAttention, bt_min_mha
from .encoder import layer_norm, transformer_encoder_layer, transformer_encoder, embedding
from .vision import transpose_nchw_nhwc, transpose_nhwc_nchw, conv2d, max_pool2d
