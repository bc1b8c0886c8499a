"""Early-exit ("anytime") encoder-decoder model (role of t5x/contrib/calm/models.py).

Training: the loss is a weighted average of the cross-entropies of the logits after every
decoder layer (`loss_fn`, models.py:446-537), or, with `train_meta_cls`, the loss of a small
classifier that predicts from a layer's hidden state whether its top token already equals the
last layer's (`loss_fn_meta_cls`, `loss_fn_meta_cls_geom_like`, :237-444).

Decoding: each token runs the decoder only up to the first exit whose confidence reaches the
threshold (`_compute_logits_from_slice_early_exit`, :539-856); the hidden state at the exit is
then written into the key/value caches of the layers that were skipped, so that later tokens
which do reach those layers can attend to this position. Needs a module with the
`decode(start_idx, end_idx, ...)` / `compute_logits` interface of
`t5x_b200.contrib.calm.network.Transformer`.
"""
from __future__ import annotations

import copy
import math
from typing import Any, Callable, Mapping, MutableMapping, Optional, Tuple

import torch

from t5x_b200 import decoding
from t5x_b200 import losses
from t5x_b200 import metrics as metrics_lib
from t5x_b200 import models
from t5x_b200.contrib.calm import decoding as calm_decoding
from t5x_b200.models.base import call_module


class EncoderDecoderModel(models.EncoderDecoderModel):
  """`models.EncoderDecoderModel` with CALM's anytime losses and early-exit inference."""

  def __init__(self, module, input_vocabulary, output_vocabulary, optimizer_def,
               decode_fn: Callable = calm_decoding.temperature_sample,
               feature_converter_cls=None, label_smoothing: float = 0.0, z_loss: float = 0.0,
               loss_normalizing_factor: Optional[float] = None,
               apply_early_inference: bool = False, decoder_layers: int = 12,
               conf_threshold: float = 1.0, min_exit: int = 0, first_exit: int = 0,
               exit_interval: int = 1, aggregation_weights: int = 1,
               oracle_tok_consistency: bool = False, oracle_cache: bool = False,
               oracle_tok_noisy_cache: bool = False, conf_method: str = "softmax_max",
               train_meta_cls: bool = False, geomlike_loss: bool = False,
               position_adjusted_threshold: bool = False, position_temp: int = 4):
    self.apply_early_inference = apply_early_inference
    self.decoder_layers = decoder_layers
    self.conf_threshold = conf_threshold
    self.min_exit = min_exit
    self.first_exit = first_exit
    self.exit_interval = exit_interval
    self.aggregation_weights = aggregation_weights
    self.oracle_tok_consistency = oracle_tok_consistency
    self.oracle_cache = oracle_cache
    self.oracle_tok_noisy_cache = oracle_tok_noisy_cache
    self.conf_method = conf_method
    self.train_meta_cls = train_meta_cls
    self.geomlike_loss = geomlike_loss
    self.position_adjusted_threshold = position_adjusted_threshold
    self.position_temp = position_temp
    super().__init__(module=module, input_vocabulary=input_vocabulary,
                     output_vocabulary=output_vocabulary, optimizer_def=optimizer_def,
                     decode_fn=decode_fn, feature_converter_cls=feature_converter_cls,
                     label_smoothing=label_smoothing, z_loss=z_loss,
                     loss_normalizing_factor=loss_normalizing_factor)

  # ---- confidence ------------------------------------------------------------------------
  def get_pred_confidence(self, logits: Optional[torch.Tensor] = None,
                          prev_state: Optional[torch.Tensor] = None,
                          new_state: Optional[torch.Tensor] = None,
                          meta_score: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-row confidence of the current prediction (t5x/contrib/calm/models.py:177-235)."""
    if self.conf_method in ("softmax_diff", "softmax_diff_approx"):
      assert logits is not None
      top2 = torch.topk(torch.softmax(logits.float(), dim=-1), 2, dim=-1).values
      return top2[..., 0] - top2[..., 1]
    if self.conf_method == "softmax_max":
      assert logits is not None
      return torch.softmax(logits.float(), dim=-1).max(dim=-1).values
    if self.conf_method == "state":
      assert prev_state is not None and new_state is not None
      a, b = prev_state.float(), new_state.float()
      conf = (a * b).sum(dim=-1) / (torch.linalg.norm(a, dim=-1) * torch.linalg.norm(b, dim=-1))
      return conf.squeeze()
    if self.conf_method == "meta":
      assert meta_score is not None
      return meta_score
    raise NotImplementedError(f"Confidence method {self.conf_method} is not implemented.")

  # ---- training --------------------------------------------------------------------------
  def _compute_hidden(self, params, batch, dropout_rng=None):
    return None  # the anytime losses need the logits of every layer, not only the last

  def _layer_weights(self, n: int, device) -> torch.Tensor:
    if self.aggregation_weights == -1:
      w = torch.tensor([2.0 ** i for i in range(n)], device=device)  # geometric, a=1, r=2
    elif self.aggregation_weights == 0:
      w = torch.ones(n, device=device)
    else:
      w = torch.arange(1, self.aggregation_weights * n + 1, self.aggregation_weights,
                       device=device, dtype=torch.float32)
    return w / w.sum()

  def loss_fn(self, params, batch, dropout_rng) -> Tuple[torch.Tensor, Mapping[str, Any]]:
    """Weighted average over the decoder layers of the usual loss; the module must return
    the logits of all layers (`return_all_logits`)."""
    if self.train_meta_cls:
      if self.geomlike_loss:
        return self.loss_fn_meta_cls_geom_like(params, batch, dropout_rng)
      return self.loss_fn_meta_cls(params, batch, dropout_rng)
    lnf, weights = losses.get_loss_normalizing_factor_and_weights(self._loss_normalizing_factor,
                                                                  batch)
    all_logits = self._compute_logits(params, batch, dropout_rng)
    if isinstance(all_logits, tuple):
      all_logits = all_logits[0]
    targets = batch["decoder_target_tokens"].long()
    all_loss, all_z = [], []
    for logits in all_logits:
      loss_i, z_i, _ = losses.compute_weighted_cross_entropy(
          logits, targets=targets, weights=weights, label_smoothing=self._label_smoothing,
          z_loss=self._z_loss, loss_normalizing_factor=lnf)
      all_loss.append(loss_i)
      all_z.append(z_i)
    w = self._layer_weights(len(all_loss), all_loss[0].device)
    loss = (torch.stack(all_loss) * w).sum()
    total_z = (torch.stack(all_z) * w).sum()
    metrics = dict(self._compute_metrics(logits=all_logits[-1], targets=targets, mask=weights,
                                         loss=loss, z_loss=total_z))
    for i, logits in enumerate(all_logits[:-1]):
      metrics[f"accuracy_per_layer/layer_{i}"] = metrics_lib.Accuracy.from_model_output(
          logits=logits, labels=targets, mask=weights)
      metrics[f"loss_per_layer/layer_{i}"] = metrics_lib.AveragePerStep(total=all_loss[i].detach())
    return loss, metrics

  def _meta_inputs(self, params, batch, dropout_rng):
    all_logits = self._compute_logits(params, batch, dropout_rng)
    assert isinstance(all_logits, tuple), "Verify that meta_cls was initialized in decoder."
    all_logits, all_meta_logits = all_logits
    predictions = all_logits.argmax(-1)
    labels = (predictions[-1][None] == predictions).long()   # [layers, batch, len]
    return all_logits, all_meta_logits, labels

  def loss_fn_meta_cls(self, params, batch, dropout_rng):
    """Independent per-layer exit classifiers with class-balanced weights."""
    lnf, weights = losses.get_loss_normalizing_factor_and_weights(self._loss_normalizing_factor,
                                                                  batch)
    if weights is None:
      weights = (batch["decoder_target_tokens"] > 0).float()
    all_logits, all_meta_logits, all_labels = self._meta_inputs(params, batch, dropout_rng)
    targets = batch["decoder_target_tokens"].long()
    all_loss, all_z = [], []
    for meta_logits, labels in zip(all_meta_logits[:-1], all_labels[:-1]):
      lab = labels.float()
      pos = ((lab * weights) == 1).sum().float()
      neg = (((1 - lab) * weights) == 1).sum().float()
      tot = torch.clamp(pos + neg, min=1.0)
      balanced = weights * lab * (1 - pos / tot) + weights * (1 - lab) * (1 - neg / tot)
      loss_i, z_i, _ = losses.compute_weighted_cross_entropy(
          meta_logits, targets=labels, weights=balanced, label_smoothing=self._label_smoothing,
          z_loss=self._z_loss, loss_normalizing_factor=lnf)
      all_loss.append(loss_i)
      all_z.append(z_i)
    loss = torch.stack(all_loss).mean()
    total_z = torch.stack(all_z).mean()
    metrics = dict(self._compute_metrics(logits=all_logits[-1], targets=targets, mask=weights,
                                         loss=loss, z_loss=total_z))
    for i, (meta_logits, labels) in enumerate(zip(all_meta_logits[:-1], all_labels[:-1])):
      metrics[f"meta_accuracy/layer_{i}"] = metrics_lib.Accuracy.from_model_output(
          logits=meta_logits, labels=labels, mask=weights)
      metrics[f"meta_loss/layer_{i}"] = metrics_lib.AveragePerStep(total=all_loss[i].detach())
    return loss, metrics

  def loss_fn_meta_cls_geom_like(self, params, batch, dropout_rng):
    """The exit classifiers as one sequence of decisions: the probability of stopping at
    layer i is P(stop at i) * prod_{j<i} P(continue at j); the target is the first layer
    that agrees with the last one."""
    lnf, weights = losses.get_loss_normalizing_factor_and_weights(self._loss_normalizing_factor,
                                                                  batch)
    all_logits, all_meta_logits, all_labels = self._meta_inputs(params, batch, dropout_rng)
    targets = batch["decoder_target_tokens"].long()
    multiclass = all_labels.argmax(0)          # first agreeing layer
    scores = torch.log_softmax(all_meta_logits.float(), dim=-1)
    pos, neg = scores[..., 1], scores[..., 0]
    non_stop = neg.cumsum(0) - neg
    geom = (non_stop + pos).movedim(0, -1)     # [batch, len, layers]
    loss, _, _ = losses.compute_weighted_cross_entropy(
        geom, targets=multiclass, weights=weights, label_smoothing=self._label_smoothing,
        z_loss=self._z_loss, loss_normalizing_factor=lnf)
    metrics = dict(self._compute_metrics(logits=all_logits[-1], targets=targets, mask=weights,
                                         loss=loss, z_loss=torch.zeros_like(loss)))
    for i, (meta_logits, labels) in enumerate(zip(all_meta_logits[:-1], all_labels[:-1])):
      metrics[f"meta_accuracy/layer_{i}"] = metrics_lib.Accuracy.from_model_output(
          logits=meta_logits, labels=labels, mask=weights)
    metrics["meta_accuracy/multiclass"] = metrics_lib.Accuracy.from_model_output(
        logits=geom, labels=multiclass, mask=weights)
    return loss, metrics

  # ---- inference -------------------------------------------------------------------------
  def _split(self, out):
    """(hidden or logits, meta score or None) of a module output that may carry meta logits."""
    if isinstance(out, tuple):
      return out[0], torch.softmax(out[1].float(), dim=-1)[..., 1]
    return out, None

  def _compute_logits_from_slice_early_exit(self, decoding_state: decoding.DecodingState, params,
                                            encoded_inputs, raw_inputs, max_decode_length: int,
                                            conf_threshold: float, pos: Any = 0):
    """One decode step with early exit: -> (logits [rows, vocab], cache, confidence, layers).

    The decoder runs segment by segment (first `first_exit + 1` layers, then `exit_interval`
    at a time) and stops at the first exit where the least confident row of the batch
    reaches the threshold, but never before `min_exit` layers."""
    n = self.decoder_layers
    flat_ids = decoding_state.cur_token
    cache = decoding_state.cache
    mod = self.module

    def run(start, end, hidden=None, propagate=False, use_cache=cache):
      return call_module(mod, params, "decode", encoded_inputs, raw_inputs, flat_ids, flat_ids,
                         enable_dropout=False, decode=True, max_decode_length=max_decode_length,
                         cache=use_cache, start_idx=start, end_idx=end,
                         decoder_embedded_input=hidden, return_prelogits=True,
                         only_propagate_state=propagate)

    def logits_of(hidden):
      return self._split(call_module(mod, params, "compute_logits", hidden))

    oracle_logits = None
    if self.oracle_tok_consistency or self.oracle_tok_noisy_cache:
      # the full model's prediction, on a copy of the cache
      full = run(0, n, use_cache=copy.deepcopy(cache))
      oracle_logits, _ = logits_of(full)

    keep = list(range(self.first_exit + 1, n, self.exit_interval))
    intervals = [(0, self.first_exit + 1)] + list(zip(keep, keep[1:] + [n]))

    hidden = run(*intervals[0])
    logits, meta_score = (logits_of(hidden) if ("softmax" in self.conf_method or
                                                self.conf_method == "meta") else (None, None))
    if self.conf_method == "state":
      conf = torch.zeros((), device=hidden.device)  # no previous state at the first exit
    else:
      conf = self.get_pred_confidence(logits=logits, meta_score=meta_score)
    interval, layer = 1, intervals[0][1]

    if self.position_adjusted_threshold:
      p0 = float(torch.as_tensor(pos).min())
      threshold = (conf_threshold * math.exp(-self.position_temp * p0 / max_decode_length) / 10
                   + 9 * conf_threshold / 10)
    else:
      threshold = conf_threshold

    def keep_going():
      if self.oracle_tok_consistency:
        same = bool((logits.argmax(-1) == oracle_logits.argmax(-1)).all())
        return (not same) and layer < n
      return (float(conf.min()) < threshold and layer < n) or layer < self.min_exit

    while keep_going() and interval < len(intervals):
      new_hidden = run(*intervals[interval], hidden=hidden)
      if "softmax" in self.conf_method or self.conf_method == "meta":
        logits, meta_score = logits_of(new_hidden)
      conf = self.get_pred_confidence(logits=logits, prev_state=hidden, new_state=new_hidden,
                                      meta_score=meta_score)
      hidden = new_hidden
      interval += 1
      layer = min(layer + self.exit_interval, n)

    if logits is None or not ("softmax" in self.conf_method or self.conf_method == "meta"):
      logits, _ = logits_of(hidden)  # only after the exit

    if layer < n:
      if self.oracle_cache:
        h = hidden  # run the remaining layers for their true keys / values
        for iv in intervals[interval:]:
          h = run(*iv, hidden=h)
      else:
        # the skipped layers project their keys / values from the state at the exit
        run(intervals[interval][0], n, hidden=hidden, propagate=True)

    if self.oracle_tok_noisy_cache:
      logits = oracle_logits
    conf_rows = conf.reshape(-1) if conf.numel() > 1 else conf.reshape(()).expand(
        flat_ids.shape[0])
    return logits[:, 0, :], cache, conf_rows, layer

  def predict_batch_with_aux(self, params, batch, rng=None,
                             decoder_params: Optional[MutableMapping[str, Any]] = None,
                             return_all_decodes: bool = False, num_decodes: int = 1,
                             prompt_with_targets: bool = False):
    """Sampling (or the configured decode function) with optional early exit; the auxiliary
    dictionary also holds `exits` and `confidences` per generated position."""
    if not self.apply_early_inference:
      decodes, aux = self._predict_plain(params, batch, rng, decoder_params, return_all_decodes,
                                         num_decodes, prompt_with_targets)
      return decodes, {**aux, "exits": [], "confidences": []}
    inputs = batch["encoder_input_tokens"]
    dec_in = batch["decoder_input_tokens"]
    b, l = dec_in.shape
    with torch.no_grad():
      encoded = decoding.flat_batch_beam_expand(
          call_module(self.module, params, "encode", inputs, enable_dropout=False), num_decodes)
      raw_inputs = decoding.flat_batch_beam_expand(inputs, num_decodes)
      cache = self.module.init_cache(b, l + 1, device=encoded.device)

      def tokens_ids_to_logits(state):
        return self._compute_logits_from_slice_early_exit(
            state, params=params, encoded_inputs=encoded, raw_inputs=raw_inputs,
            max_decode_length=l, conf_threshold=self.conf_threshold, pos=state.cur_index)

      decoder_params = dict(decoder_params or {})
      if rng is not None:
        if decoder_params.get("decode_rng") is not None:
          raise ValueError("Got RNG both from the `rng` argument and "
                           "`decoder_params['decode_rng']`. Please specify one or the other.")
        decoder_params["decode_rng"] = rng
      eos = getattr(self.output_vocabulary, "eos_id", None) or 1
      prompt = dec_in * (dec_in != eos) if prompt_with_targets else torch.zeros_like(dec_in)
      decoder_params.setdefault("eos_id", eos)
      scanned = bool(getattr(self.module, "scan_layers", False))
      decodes, (scores, exits, confidences) = self._decode_fn(
          inputs=prompt, cache=cache, tokens_to_logits=tokens_ids_to_logits,
          num_decodes=num_decodes, cache_offset=1 if scanned else 0, **decoder_params)
    if return_all_decodes:
      return decodes, {"scores": scores, "exits": exits, "confidences": confidences}
    return decodes[:, -1, :], {"scores": scores[:, -1], "exits": exits[:, -1, :],
                               "confidences": confidences[:, -1, :]}

  def _predict_plain(self, params, batch, rng, decoder_params, return_all_decodes, num_decodes,
                     prompt_with_targets):
    """All layers for every token, through the shared decode loop."""
    saved = self._decode_fn
    if saved is calm_decoding.temperature_sample:
      self._decode_fn = decoding.temperature_sample
    try:
      return super().predict_batch_with_aux(params, batch, rng, decoder_params,
                                            return_all_decodes, num_decodes,
                                            prompt_with_targets)
    finally:
      self._decode_fn = saved
