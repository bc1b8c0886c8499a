"""Layer library of the scalable T5 family: the T5 layers, shared
(t5x/examples/scalable_t5/layers.py differs from the T5 set only in how parameters are
annotated for scanning and in its 3-D attention kernels; see `network.py` for how those
layouts are produced here)."""
from t5x_b200.models.t5.layers import *  # noqa: F401,F403
from t5x_b200.models.t5.layers import (  # noqa: F401
    DenseGeneral, Embed, LayerNorm, MlpBlock, MultiHeadDotProductAttention,
    RelativePositionBiases)
