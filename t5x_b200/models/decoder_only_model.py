"""`DecoderOnlyModel`: language-model / prefix-LM wrapper (t5x/models.py:814-1240).

Accepts batches made of 'targets' only or of 'inputs' + 'targets' concatenated by the
decoder feature converter; with `inputs_bidirectional_attention=True` the inputs region is
attended bidirectionally (prefix LM). Generation prefills the key/value cache with the
prompt in one pass and then samples from per-example positions.
"""
from __future__ import annotations

from typing import Any, Mapping, MutableMapping, Optional, Tuple

import numpy as np
import torch

from t5x_b200 import decoding
from t5x_b200 import losses
from t5x_b200.models import base
from t5x_b200.models.t5 import layers as t5_layers
from t5x_b200.ops import reference as ref


class DecoderOnlyModel(base.BaseTransformerModel):
  """Model class for decoder-only modules."""

  FEATURE_CONVERTER_CLS = None  # DecoderFeatureConverter unless overridden

  def __init__(self, module, vocabulary, optimizer_def, decode_fn=decoding.temperature_sample,
               inputs_bidirectional_attention: bool = False, feature_converter_cls=None,
               label_smoothing: float = 0.0, z_loss: float = 0.0, loss_normalizing_factor=None):
    if feature_converter_cls is not None:
      self.FEATURE_CONVERTER_CLS = feature_converter_cls
    elif self.FEATURE_CONVERTER_CLS is None:
      from t5x_b200.data import feature_converters
      self.FEATURE_CONVERTER_CLS = feature_converters.DecoderFeatureConverter
    self._inputs_bidirectional_attention = inputs_bidirectional_attention
    super().__init__(module, input_vocabulary=vocabulary, output_vocabulary=vocabulary,
                     optimizer_def=optimizer_def, decode_fn=decode_fn,
                     label_smoothing=label_smoothing, z_loss=z_loss,
                     loss_normalizing_factor=loss_normalizing_factor)

  def get_initial_variables(self, rng, input_shapes, input_types=None):
    if "decoder_input_tokens" not in input_shapes:
      raise KeyError("input_shapes needs 'decoder_input_tokens'")
    if rng is not None and not isinstance(rng, torch.Generator):
      t5_layers.reinitialize(self.module, int(rng))
    return {"params": base.module_param_tree(self.module),
            "params_axes": base.module_param_axes(self.module)}

  def _get_decoder_causal_attention(self, batch):
    if not self._inputs_bidirectional_attention:
      return None
    if "decoder_causal_attention" not in batch:
      raise ValueError('`inputs_bidirectional_attention` mode requires '
                       '"decoder_causal_attention" feature in the batch')
    return batch["decoder_causal_attention"]

  def _run(self, params, batch, dropout_rng, return_hidden):
    if dropout_rng is not None:
      ref.set_dropout_seed(int(dropout_rng))
    return base.call_module(
        self.module, params, None, batch["decoder_input_tokens"],
        batch["decoder_target_tokens"],
        decoder_segment_ids=batch.get("decoder_segment_ids"),
        decoder_positions=batch.get("decoder_positions"),
        decoder_causal_attention=self._get_decoder_causal_attention(batch),
        enable_dropout=dropout_rng is not None, decode=False, return_hidden=return_hidden)

  def _compute_logits(self, params, batch, dropout_rng=None, mutable=None, other_variables=None):
    return self._run(params, batch, dropout_rng, False)

  def _compute_hidden(self, params, batch, dropout_rng=None):
    dec = getattr(self.module, "decoder", None)
    if dec is None or not hasattr(dec, "logits_weight_and_scale"):
      return None
    hidden = self._run(params, batch, dropout_rng, True)
    if params is not None and not base._owns(self.module, params):
      c = self.module.config
      if c.logits_via_embedding:
        weight = params["decoder"]["token_embedder"]["embedding"]
        scale = 1.0 / np.sqrt(c.emb_dim)
      else:
        weight, scale = params["decoder"]["logits_dense"]["kernel"], 1.0
    else:
      weight, scale = dec.logits_weight_and_scale()
    return hidden, weight, scale

  def _compute_logits_from_slice(self, decoding_state: decoding.DecodingState, params,
                                 max_decode_length: int):
    """Token ids [rows, 1] -> (logits [rows, vocab], cache) for one decode step."""
    flat_ids = decoding_state.cur_token
    cache = decoding_state.cache
    logits = base.call_module(self.module, params, None, flat_ids, flat_ids,
                              enable_dropout=False, decode=True,
                              max_decode_length=max_decode_length, cache=cache)
    return logits[:, 0, :], cache

  def score_batch(self, params, batch, return_intermediates: bool = False):
    targets = batch["decoder_target_tokens"].long()
    weights = batch["decoder_loss_weights"]
    with torch.no_grad():
      logits = self._compute_logits(params, batch, None)
      onehot = torch.nn.functional.one_hot(targets, logits.shape[-1]).float()
      token_scores = -losses.cross_entropy_with_logits(logits, onehot, z_loss=0.0)[0] * weights
    sequence_scores = token_scores.sum(-1)
    if return_intermediates:
      return sequence_scores, {"decoder": {"target_tokens": (targets,),
                                           "loss_weights": (weights,),
                                           "token_scores": (token_scores,)}}
    return sequence_scores

  def _compute_kv_cache(self, params, inputs: torch.Tensor,
                        causal_attention_mask: torch.Tensor) -> Tuple[Any, torch.Tensor]:
    """Prefills the cache with the prompt. Returns (cache, index of the next position)."""
    inputs_lengths = (inputs[:, 1:] != 0).sum(-1)
    b, l = inputs.shape
    cache = self.module.init_cache(b, l, device=inputs.device)
    maybe_ca = self._get_decoder_causal_attention(
        {"decoder_causal_attention": causal_attention_mask})
    base.call_module(self.module, params, None, inputs, causal_attention_mask,
                     decoder_causal_attention=maybe_ca, enable_dropout=False, decode=True,
                     prefill=True, prefill_lengths=inputs_lengths, cache=cache,
                     return_hidden=True)
    return cache, inputs_lengths

  def predict_batch_with_aux(self, params, batch, rng=None, *, return_all_decodes: bool = False,
                             num_decodes: int = 1,
                             decoder_params: Optional[MutableMapping[str, Any]] = None):
    """Samples continuations of the inputs region (t5x/models.py:1057-1240): the targets part
    of `decoder_input_tokens` is zeroed by `decoder_causal_attention` and filled with samples."""
    if "decoder_causal_attention" not in batch:
      raise ValueError("Batch does not have the right format for text generation: probably "
                       "because `task_feature_lengths` passed to the feature converter does "
                       "not have both `inputs` and `targets`.")
    inputs = batch["decoder_input_tokens"] * batch["decoder_causal_attention"]
    with torch.no_grad():
      cache, initial_index = self._compute_kv_cache(params, inputs,
                                                    batch["decoder_causal_attention"])
      max_decode_length = batch["decoder_input_tokens"].shape[1]

      def tokens_ids_to_logits(state):
        return self._compute_logits_from_slice(state, params=params,
                                               max_decode_length=max_decode_length)

      decoder_params = dict(decoder_params or {})
      if rng is not None:
        if decoder_params.get("decode_rng") is not None:
          raise ValueError("Got RNG both from the `rng` argument and "
                           "`decoder_params['decode_rng']`. Please specify one or the other.")
        decoder_params["decode_rng"] = rng
      scanned = bool(getattr(self.module, "scan_layers", False))
      if "eos_id" not in decoder_params:
        decoder_params["eos_id"] = getattr(self.output_vocabulary, "eos_id", None) or 1
      decoded, scores = self._decode_fn(
          inputs=inputs, cache=cache, tokens_to_logits=tokens_ids_to_logits,
          num_decodes=num_decodes, initial_index=initial_index,
          cache_offset=1 if scanned else 0, **decoder_params)
    if not return_all_decodes:
      decoded = decoded[:, -1, :]
      aux = {"scores": scores[:, -1]}
    else:
      aux = {"scores": scores}
    return base.remove_prefix(decoded, initial_index), aux

  def predict_batch(self, params, batch, rng=None):
    return self.predict_batch_with_aux(params, batch, rng)[0]
