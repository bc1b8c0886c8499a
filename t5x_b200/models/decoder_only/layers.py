"""Layer library of the decoder-only family: the T5 layers, shared
(t5x/examples/decoder_only/layers.py holds a copy of the T5 layer set)."""
from t5x_b200.models.t5.layers import *  # noqa: F401,F403
from t5x_b200.models.t5.layers import (  # noqa: F401
    DenseGeneral, Embed, LayerNorm, MlpBlock, MultiHeadDotProductAttention,
    RelativePositionBiases, combine_biases, combine_masks, dot_product_attention,
    make_attention_mask, make_causal_mask, make_decoder_mask)
