"""T5.1.1 model configs as buildables (t5x/fiddle_configs/models/t5_1_1.py; the gin form is
t5x/examples/t5/t5_1_1/{small,base,...}.gin)."""
from __future__ import annotations

from typing import Optional

from t5x_b200 import adafactor, fdl, models
from t5x_b200.data import vocabularies
from t5x_b200.models.t5 import network

# loss hyper-parameters of the published T5.1.1 recipes
Z_LOSS = 0.0001
LABEL_SMOOTHING = 0.0
LOSS_NORMALIZING_FACTOR = None
VOCABULARY_FILE = "gs://t5-data/vocabs/cc_all.32000.100extra/sentencepiece.model"

# (emb_dim, num_heads, layers, mlp_dim) per size; head_dim is 64 throughout
SIZES = {
    "small": (512, 6, 8, 1024),
    "base": (768, 12, 12, 2048),
    "large": (1024, 16, 24, 2816),
    "xl": (2048, 32, 24, 5120),
    "xxl": (4096, 64, 24, 10240),
}


def vocabulary(sentencepiece_model_file: str = VOCABULARY_FILE) -> fdl.Buildable:
  return fdl.Config(vocabularies.SentencePieceVocabulary,
                    sentencepiece_model_file=sentencepiece_model_file)


def optimizer() -> fdl.Buildable:
  return fdl.Config(adafactor.Adafactor, decay_rate=0.8, step_offset=0,
                    logical_factor_rules=fdl.Config(adafactor.standard_logical_factor_rules))


def sized_config(size: str, dropout_rate: Optional[float]) -> fdl.Buildable:
  emb_dim, num_heads, layers, mlp_dim = SIZES[size]
  return fdl.Config(network.T5Config, vocab_size=32128, dtype="bfloat16", emb_dim=emb_dim,
                    num_heads=num_heads, num_encoder_layers=layers, num_decoder_layers=layers,
                    head_dim=64, mlp_dim=mlp_dim, mlp_activations=("gelu", "linear"),
                    dropout_rate=dropout_rate, logits_via_embedding=False)


def base_config(dropout_rate: Optional[float]) -> fdl.Buildable:
  return sized_config("base", dropout_rate)


def small_config(dropout_rate: Optional[float]) -> fdl.Buildable:
  return sized_config("small", dropout_rate)


def model(config: fdl.Buildable, z_loss: float = Z_LOSS,
          label_smoothing: float = LABEL_SMOOTHING,
          loss_normalizing_factor: Optional[float] = LOSS_NORMALIZING_FACTOR,
          vocab: Optional[fdl.Buildable] = None) -> fdl.Buildable:
  """EncoderDecoderModel over `config`; one vocabulary config serves inputs and outputs."""
  vocab = vocab if vocab is not None else vocabulary()
  return fdl.Config(models.EncoderDecoderModel,
                    module=fdl.Config(network.Transformer, config=config),
                    input_vocabulary=vocab, output_vocabulary=vocab, optimizer_def=optimizer(),
                    z_loss=z_loss, label_smoothing=label_smoothing,
                    loss_normalizing_factor=loss_normalizing_factor)
