"""Model API (names of t5x/models.py) and network definitions (sub-packages)."""
from t5x_b200.models.base import (  # noqa: F401
    BaseModel, BaseTransformerModel, DecoderParams, EncoderDecoderModel, MetricsMap,
    compute_base_metrics, count_packed_examples, get_input_vocabulary, get_output_vocabulary,
    module_param_axes, module_param_tree, remove_prefix)
from t5x_b200.models.decoder_only_model import DecoderOnlyModel  # noqa: F401
