"""Model wrappers that add the MoE auxiliary losses and metrics
(t5x/contrib/moe/models.py:49-425)."""
from __future__ import annotations

from typing import Dict, Mapping, Tuple

import torch

from t5x_b200 import decoding
from t5x_b200 import losses
from t5x_b200 import metrics as metrics_lib
from t5x_b200.contrib.moe import layers as moe_layers
from t5x_b200.models import base as base_models
from t5x_b200.models import decoder_only_model

AveragePerStep = metrics_lib.AveragePerStep
MOE_METRICS = moe_layers.MOE_METRICS


def _extract_diversity_metrics(collected) -> Dict[str, torch.Tensor]:
  """Per-layer router metrics averaged over the MoE layers of one forward pass."""
  avg = {}
  for name in MOE_METRICS:
    vals = [m[name] for m in collected if name in m]
    if not vals:
      raise ValueError(f"Unable to find expert metric: {name}. Please check that MoE metrics "
                       "and losses are correctly sown.")
    avg[name] = torch.stack([torch.as_tensor(v, dtype=torch.float32) for v in vals]).mean()
  return avg


def _expert_losses(diversity_metrics, auxiliary_loss_factor: float, router_z_loss_factor: float):
  aux = auxiliary_loss_factor * diversity_metrics["auxiliary_loss"].mean()
  rz = router_z_loss_factor * diversity_metrics["router_z_loss"].mean()
  return aux, rz


def _expert_metrics(diversity_metrics, total_loss, z_loss, auxiliary_loss, router_z_loss,
                    num_tokens: int):
  """Expert metrics plus cross-entropy metrics corrected for the auxiliary losses."""
  cross_ent_loss = total_loss - z_loss - auxiliary_loss - router_z_loss
  det = lambda v: v.detach() if isinstance(v, torch.Tensor) else torch.as_tensor(v)
  return {
      "experts/auxiliary_loss": AveragePerStep.from_model_output(det(auxiliary_loss)),
      "experts/router_z_loss": AveragePerStep.from_model_output(det(router_z_loss)),
      "experts/fraction_tokens_left_behind": AveragePerStep.from_model_output(
          det(diversity_metrics["fraction_tokens_left_behind"].mean())),
      "experts/expert_usage": AveragePerStep.from_model_output(
          det(diversity_metrics["expert_usage"].mean())),
      "experts/router_confidence": AveragePerStep.from_model_output(
          det(diversity_metrics["router_confidence"].mean())),
      "cross_ent_loss": metrics_lib.AveragePerStep(total=det(cross_ent_loss)),
      "cross_ent_loss_per_all_target_tokens": AveragePerStep.from_model_output(
          det(cross_ent_loss) / num_tokens),
  }


def _moe_loss_fn(model, params, batch, dropout_rng, aux_loss_factor, router_z_loss_factor):
  lnf, weights = losses.get_loss_normalizing_factor_and_weights(model._loss_normalizing_factor,
                                                                batch)
  targets = batch["decoder_target_tokens"].long()
  moe_layers.reset_collected_metrics()
  fused = model._compute_hidden(params, batch, dropout_rng)
  if fused is not None:
    hidden, weight, scale = fused
    tok_loss, tok_z, correct = model._token_losses(hidden, weight, scale, targets)
    total_loss, z_loss, _ = losses.weight_and_normalize(tok_loss, tok_z, targets, weights, lnf)
    logits = None
  else:
    logits = model._compute_logits(params, batch, dropout_rng)
    total_loss, z_loss, _ = losses.compute_weighted_cross_entropy(
        logits, targets=targets, weights=weights, label_smoothing=model._label_smoothing,
        z_loss=model._z_loss, loss_normalizing_factor=lnf)
    correct = None
  diversity = _extract_diversity_metrics(moe_layers.collected_metrics())
  aux_loss, router_z = _expert_losses(diversity, aux_loss_factor, router_z_loss_factor)
  total_loss = total_loss + aux_loss + router_z
  metrics = base_models.compute_base_metrics(logits=logits, targets=targets, mask=weights,
                                             loss=total_loss, z_loss=z_loss, correct=correct)
  metrics.update(_expert_metrics(diversity, total_loss, z_loss, aux_loss, router_z,
                                 num_tokens=targets.numel()))
  return total_loss, metrics


class MoeEncoderDecoderModel(base_models.EncoderDecoderModel):
  """Encoder-decoder that propagates the MoE auxiliary losses and metrics."""

  def __init__(self, module, input_vocabulary, output_vocabulary, optimizer_def,
               decode_fn=decoding.beam_search, feature_converter_cls=None,
               label_smoothing: float = 0.0, z_loss: float = 0.0, loss_normalizing_factor=None,
               aux_loss_factor: float = 0.0, router_z_loss_factor: float = 0.0):
    super().__init__(module=module, input_vocabulary=input_vocabulary,
                     output_vocabulary=output_vocabulary, optimizer_def=optimizer_def,
                     decode_fn=decode_fn, feature_converter_cls=feature_converter_cls,
                     label_smoothing=label_smoothing, z_loss=z_loss,
                     loss_normalizing_factor=loss_normalizing_factor)
    self._aux_loss_factor = aux_loss_factor
    self._router_z_loss_factor = router_z_loss_factor

  def loss_fn(self, params, batch, dropout_rng):
    return _moe_loss_fn(self, params, batch, dropout_rng, self._aux_loss_factor,
                        self._router_z_loss_factor)

  def _graph_decoder(self, *args, **kwargs):
    return None  # the captured decode step covers dense feed-forward blocks only


class MoeDecoderOnlyModel(decoder_only_model.DecoderOnlyModel):
  """Decoder-only model that propagates the MoE auxiliary losses and metrics."""

  def __init__(self, module, vocabulary, optimizer_def, decode_fn=decoding.temperature_sample,
               inputs_bidirectional_attention: bool = False, feature_converter_cls=None,
               label_smoothing: float = 0.0, z_loss: float = 0.0, loss_normalizing_factor=None,
               aux_loss_factor: float = 0.0, router_z_loss_factor: float = 0.0):
    super().__init__(module=module, vocabulary=vocabulary, optimizer_def=optimizer_def,
                     decode_fn=decode_fn,
                     inputs_bidirectional_attention=inputs_bidirectional_attention,
                     feature_converter_cls=feature_converter_cls, label_smoothing=label_smoothing,
                     z_loss=z_loss, loss_normalizing_factor=loss_normalizing_factor)
    self._aux_loss_factor = aux_loss_factor
    self._router_z_loss_factor = router_z_loss_factor

  def loss_fn(self, params, batch, dropout_rng):
    return _moe_loss_fn(self, params, batch, dropout_rng, self._aux_loss_factor,
                        self._router_z_loss_factor)
