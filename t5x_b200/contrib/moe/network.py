"""T5 encoder-decoder whose feed-forward blocks are, at chosen layers, mixtures of experts
(the Switch / ST-MoE layouts the reference's MoE contrib trains through Flaxformer).

`sparse_layout`: 'every_other' puts an expert layer at layers 1, 3, 5, ... (Switch);
'all' at every layer; a tuple of indices selects layers explicitly. Dense layers keep the
standard T5 `mlp`; expert layers have `mlp/router/...` and `mlp/expert/...` parameters."""
from __future__ import annotations

import dataclasses
from typing import Sequence, Tuple, Union

from torch import nn

from t5x_b200.contrib.moe import layers as moe_layers
from t5x_b200.models.t5 import layers as t5_layers
from t5x_b200.models.t5 import network as t5_network


@dataclasses.dataclass
class MoeT5Config(t5_network.T5Config):
  num_experts: int = 8
  num_selected_experts: int = 1
  train_capacity_factor: float = 1.25
  eval_capacity_factor: float = 2.0
  min_expert_capacity: int = 4
  router_jitter_noise: float = 0.0
  sparse_layout: Union[str, Tuple[int, ...]] = "every_other"
  expert_mlp_dim: int = 0  # 0: same as mlp_dim
  router_type: str = "tokens_choose"  # or "experts_choose"


def is_sparse_layer(config: MoeT5Config, index: int) -> bool:
  lay = config.sparse_layout
  if lay == "all":
    return True
  if lay == "every_other":
    return index % 2 == 1
  if lay in (None, "none"):
    return False
  return index in tuple(lay)


def _moe(config: MoeT5Config, device):
  c = config
  return moe_layers.MoeLayer(
      c.emb_dim, c.expert_mlp_dim or c.mlp_dim, c.num_experts, c.mlp_activations,
      c.num_selected_experts, c.train_capacity_factor, c.eval_capacity_factor,
      c.min_expert_capacity, c.dropout_rate, c.router_jitter_noise, c.dtype, device=device,
      router_type=c.router_type)


class Transformer(t5_network.Transformer):
  """`t5.network.Transformer` with `mlp` swapped for `MoeLayer` at the sparse layers."""

  def __init__(self, config: MoeT5Config, device=None):
    super().__init__(config, device=device)
    for i in range(config.num_encoder_layers):
      if is_sparse_layer(config, i):
        getattr(self.encoder, f"layers_{i}").mlp = _moe(config, device)
    for i in range(config.num_decoder_layers):
      if is_sparse_layer(config, i):
        getattr(self.decoder, f"layers_{i}").mlp = _moe(config, device)
