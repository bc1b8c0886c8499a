"""Model API (parity target: t5x/models.py): loss/eval/predict/score over a network module.

A model wraps a `torch.nn.Module` network whose parameters form a tree with the reference's
names. `params` arguments are nested dicts of tensors; when they are the module's own
parameters (the normal case: the train state holds them) the module runs directly, otherwise
the call goes through `torch.func.functional_call`.
"""
from __future__ import annotations

import abc
import dataclasses
import inspect
from typing import Any, Callable, Mapping, MutableMapping, Optional, Tuple, Union

import numpy as np
import torch

from t5x_b200 import decoding
from t5x_b200 import losses
from t5x_b200 import metrics as metrics_lib
from t5x_b200 import optimizers
from t5x_b200.models.t5 import layers as t5_layers
from t5x_b200.ops import functional as F
from t5x_b200.ops import reference as ref
from t5x_b200.parallel import state as pstate
from t5x_b200.utils import tree as tree_utils

MetricsMap = Mapping[str, metrics_lib.Metric]
PyTree = Any


@dataclasses.dataclass
class DecoderParams:
  return_all_decodes: bool = False
  num_decodes: int = 1


# ----------------------------------------------------------------------------
# Module <-> param tree helpers
# ----------------------------------------------------------------------------
def module_param_tree(module: torch.nn.Module) -> dict:
  """Nested dict of the module's parameters keyed like the reference's param tree."""
  return tree_utils.unflatten_dict({n.replace(".", "/"): p for n, p in module.named_parameters()})


def module_param_axes(module: torch.nn.Module) -> dict:
  return tree_utils.unflatten_dict(
      {n.replace(".", "/"): tuple(getattr(p, "axes", (None,) * p.dim()))
       for n, p in module.named_parameters()})


def _owns(module: torch.nn.Module, params) -> bool:
  flat = tree_utils.flatten_dict(params)
  own = dict(module.named_parameters())
  for k, v in flat.items():
    if own.get(k.replace("/", ".")) is not v:
      return False
  return True


def call_module(module: torch.nn.Module, params, method: Optional[str], *args, **kwargs):
  """module.<method>(*args) evaluated with `params` as its parameters."""
  fn_name = method or "forward"
  if params is None or _owns(module, params):
    return getattr(module, fn_name)(*args, **kwargs)
  flat = {k.replace("/", "."): v for k, v in tree_utils.flatten_dict(params).items()}
  if fn_name == "forward":
    return torch.func.functional_call(module, flat, args, kwargs)
  # functional_call drives forward(); route other methods through a thin dispatcher.
  orig_forward = module.forward
  try:
    module.forward = getattr(module, fn_name)
    return torch.func.functional_call(module, flat, args, kwargs)
  finally:
    module.forward = orig_forward


class BaseModel(abc.ABC):
  """Abstract model: loss_fn, eval_fn, predict_batch(_with_aux), score_batch,
  get_initial_variables (t5x/models.py:113-233)."""

  FEATURE_CONVERTER_CLS: Callable[..., Any]

  def __init__(self, optimizer_def: optimizers.OptimizerDef):
    self.optimizer_def = optimizer_def

  @abc.abstractmethod
  def loss_fn(self, params, batch, dropout_rng) -> Tuple[torch.Tensor, MetricsMap]:
    ...

  def eval_fn(self, params, batch) -> Tuple[torch.Tensor, MetricsMap]:
    with torch.no_grad():
      return self.loss_fn(params=params, batch=batch, dropout_rng=None)

  def predict_batch(self, params, batch, rng=None):
    return self.predict_batch_with_aux(params=params, batch=batch, rng=rng)[0]

  @abc.abstractmethod
  def predict_batch_with_aux(self, params, batch, rng=None):
    ...

  @abc.abstractmethod
  def score_batch(self, params, batch, return_intermediates: bool = False):
    ...

  @abc.abstractmethod
  def get_initial_variables(self, rng, input_shapes, input_types=None):
    ...


class BaseTransformerModel(BaseModel):
  """Cross-entropy loss + standard metrics on top of `_compute_logits`
  (t5x/models.py:236-355)."""

  def __init__(self, module: torch.nn.Module, input_vocabulary, output_vocabulary,
               optimizer_def: optimizers.OptimizerDef, decode_fn=None,
               label_smoothing: float = 0.0, z_loss: float = 0.0,
               loss_normalizing_factor=None):
    self.module = module
    self._input_vocabulary = input_vocabulary
    self._output_vocabulary = output_vocabulary
    self._decode_fn = decode_fn
    self._label_smoothing = label_smoothing
    self._z_loss = z_loss
    self._loss_normalizing_factor = loss_normalizing_factor
    super().__init__(optimizer_def=optimizer_def)

  @property
  def input_vocabulary(self):
    return self._input_vocabulary

  @property
  def output_vocabulary(self):
    return self._output_vocabulary

  @property
  def decode_fn(self):
    return self._decode_fn

  def _compute_logits(self, params, batch, dropout_rng=None):
    raise NotImplementedError

  def _compute_hidden(self, params, batch, dropout_rng=None):
    """Decoder output before the vocabulary projection, plus (weight, scale) of the projection.
    Models that provide it get the fused projection+cross-entropy path."""
    return None

  def loss_fn(self, params, batch, dropout_rng):
    lnf, weights = losses.get_loss_normalizing_factor_and_weights(self._loss_normalizing_factor,
                                                                  batch)
    targets = batch["decoder_target_tokens"].long()
    fused = self._compute_hidden(params, batch, dropout_rng)
    if fused is not None:
      hidden, weight, scale = fused
      tok_loss, tok_z, correct = self._token_losses(hidden, weight, scale, targets)
      loss, z_loss, _ = losses.weight_and_normalize(tok_loss, tok_z, targets, weights, lnf)
      logits = None
    else:
      logits = self._compute_logits(params, batch, dropout_rng)
      loss, z_loss, _ = losses.compute_weighted_cross_entropy(
          logits, targets=targets, weights=weights, label_smoothing=self._label_smoothing,
          z_loss=self._z_loss, loss_normalizing_factor=lnf)
      correct = None
    segment_ids = {k[:-len("_segment_ids")]: v for k, v in batch.items()
                   if k.endswith("_segment_ids")}
    if not segment_ids:
      segment_ids = {k: v != 0 for k, v in batch.items()
                     if k in ("encoder_input_tokens", "decoder_target_tokens")}
    metrics = self._compute_metrics(logits=logits, targets=targets, mask=weights, loss=loss,
                                    z_loss=z_loss, segment_ids=segment_ids, correct=correct)
    return loss, metrics

  def _token_losses(self, hidden, weight, scale, targets):
    """Per-token (loss, z-loss, correct). Vocab-parallel when the projection is sharded."""
    st = pstate.get()
    if st.model_size > 1 and getattr(weight, "shard_dim", None) is not None:
      from t5x_b200.parallel import vocab_parallel
      return vocab_parallel.logits_cross_entropy(
          hidden, weight, targets, z_loss=self._z_loss, label_smoothing=self._label_smoothing,
          logits_scale=scale)
    return F.logits_cross_entropy(hidden, weight, targets, z_loss=self._z_loss,
                                  label_smoothing=self._label_smoothing, logits_scale=scale)

  def _compute_metrics(self, logits, targets, mask, loss, z_loss=None, segment_ids=None,
                       correct=None):
    return compute_base_metrics(logits=logits, targets=targets, mask=mask, loss=loss,
                                z_loss=z_loss, segment_ids=segment_ids, correct=correct)


class EncoderDecoderModel(BaseTransformerModel):
  """Encoder-decoder wrapper (t5x/models.py:364-812)."""

  FEATURE_CONVERTER_CLS = None  # set lazily to the seqio-style EncDecFeatureConverter

  def __init__(self, module, input_vocabulary, output_vocabulary, optimizer_def,
               decode_fn=decoding.beam_search, feature_converter_cls=None,
               label_smoothing: float = 0.0, z_loss: float = 0.0, loss_normalizing_factor=None,
               default_decoder_params: Optional[DecoderParams] = None):
    if feature_converter_cls is not None:
      self.FEATURE_CONVERTER_CLS = feature_converter_cls
    elif self.FEATURE_CONVERTER_CLS is None:
      from t5x_b200.data import feature_converters
      self.FEATURE_CONVERTER_CLS = feature_converters.EncDecFeatureConverter
    self._default_decoder_params = default_decoder_params or DecoderParams()
    super().__init__(module=module, input_vocabulary=input_vocabulary,
                     output_vocabulary=output_vocabulary, optimizer_def=optimizer_def,
                     decode_fn=decode_fn, label_smoothing=label_smoothing, z_loss=z_loss,
                     loss_normalizing_factor=loss_normalizing_factor)

  def get_initial_variables(self, rng, input_shapes, input_types=None):
    """{'params', 'params_axes'} of the module, re-drawn under `rng` when it is an int seed
    (t5x/models.py:400-454; shapes only serve validation here: the module owns its shapes)."""
    if rng is not None and not isinstance(rng, torch.Generator):
      t5_layers.reinitialize(self.module, int(rng))
    return {"params": module_param_tree(self.module),
            "params_axes": module_param_axes(self.module)}

  @staticmethod
  def _module_kwargs(batch):
    kw = {}
    for name in ("encoder_segment_ids", "decoder_segment_ids", "encoder_positions",
                 "decoder_positions"):
      if name in batch:
        kw[name] = batch[name]
    return kw

  def _seed_dropout(self, dropout_rng):
    if dropout_rng is not None:
      ref.set_dropout_seed(int(dropout_rng))

  def _compute_logits(self, params, batch, dropout_rng=None, mutable=None, other_variables=None):
    self._seed_dropout(dropout_rng)
    return call_module(self.module, params, None, batch["encoder_input_tokens"],
                       batch["decoder_input_tokens"], batch["decoder_target_tokens"],
                       enable_dropout=dropout_rng is not None, decode=False,
                       **self._module_kwargs(batch))

  def _compute_hidden(self, params, batch, dropout_rng=None):
    if not hasattr(self.module, "decoder") or not hasattr(self.module.decoder,
                                                          "logits_weight_and_scale"):
      return None
    self._seed_dropout(dropout_rng)
    hidden = call_module(self.module, params, None, batch["encoder_input_tokens"],
                         batch["decoder_input_tokens"], batch["decoder_target_tokens"],
                         enable_dropout=dropout_rng is not None, decode=False, return_hidden=True,
                         **self._module_kwargs(batch))
    if params is not None and not _owns(self.module, params):
      c = self.module.config
      if c.logits_via_embedding:
        weight, scale = params["token_embedder"]["embedding"], 1.0 / np.sqrt(c.emb_dim)
      else:
        weight, scale = params["decoder"]["logits_dense"]["kernel"], 1.0
    else:
      weight, scale = self.module.decoder.logits_weight_and_scale()
    return hidden, weight, scale

  def _compute_logits_from_slice(self, decoding_state: decoding.DecodingState, params,
                                 encoded_inputs, raw_inputs, max_decode_length,
                                 beams_per_kv: int = 1):
    """One decode step: token ids [batch*beam, 1] -> logits [batch*beam, vocab]
    (t5x/models.py:484-515). The encoder output is NOT expanded by beams: cross-attention
    keys/values are projected once per example and shared by its beams."""
    flat_ids = decoding_state.cur_token
    cache = decoding_state.cache
    hidden = call_module(self.module, params, "decode_hidden", encoded_inputs, raw_inputs,
                         flat_ids, flat_ids, enable_dropout=False, decode=True,
                         max_decode_length=max_decode_length, cache=cache,
                         beams_per_kv=beams_per_kv)
    logits = self.module.decoder.logits(hidden)
    return logits[:, 0, :], cache

  def _compute_kv_cache(self, params, encoded_inputs, encoder_input_tokens,
                        decoder_input_tokens, prefill_decoder_prompt: bool = False):
    b, l = decoder_input_tokens.shape
    cache = self.module.init_cache(b, l, device=encoded_inputs.device)
    return cache, None

  def predict_batch_with_aux(self, params, batch, rng=None,
                             decoder_params: Optional[MutableMapping[str, Any]] = None,
                             return_all_decodes: bool = None, num_decodes: int = None,
                             prompt_with_targets: bool = False):
    """Beam search (or the configured decode fn) over a batch (t5x/models.py:584-758)."""
    if return_all_decodes is None:
      return_all_decodes = self._default_decoder_params.return_all_decodes
    if num_decodes is None:
      num_decodes = self._default_decoder_params.num_decodes
    encoder_input_tokens = batch["encoder_input_tokens"]
    decoder_input_tokens = batch["decoder_input_tokens"]
    eos = getattr(self.output_vocabulary, "eos_id", None) or 1
    if prompt_with_targets:
      decoder_prompt_inputs = decoder_input_tokens * (decoder_input_tokens != eos)
    else:
      decoder_prompt_inputs = torch.zeros_like(decoder_input_tokens)
    fast = self._graph_decoder(params, decoder_input_tokens, num_decodes, eos, decoder_params,
                               rng, prompt_with_targets)
    if fast is not None:
      decodes, scores = fast.decode(encoder_input_tokens)
      if return_all_decodes:
        return decodes, {"scores": scores}
      return decodes[:, -1, :], {"scores": scores[:, -1]}
    with torch.no_grad():
      encoded_inputs = call_module(self.module, params, "encode", encoder_input_tokens,
                                   enable_dropout=False)
      # The cache holds batch*num_decodes rows for self-attention; cross-attention K/V stay
      # per example ([batch, ...]) and are shared by the beams.
      b, l = decoder_input_tokens.shape
      cache = self.module.init_cache(b, l + 1, device=encoded_inputs.device)

      def tokens_ids_to_logits(state: decoding.DecodingState):
        rows = state.cur_token.shape[0]
        return self._compute_logits_from_slice(
            state, params=params, encoded_inputs=encoded_inputs,
            raw_inputs=encoder_input_tokens, max_decode_length=l,
            beams_per_kv=rows // encoder_input_tokens.shape[0])

      decoder_params = dict(decoder_params or {})
      if rng is not None:
        if decoder_params.get("decode_rng") is not None:
          raise ValueError("Got RNG both from the `rng` argument and "
                           "`decoder_params['decode_rng']`. Please specify one or the other.")
        decoder_params["decode_rng"] = rng
      scanned = bool(getattr(self.module, "scan_layers", False))
      if "eos_id" not in decoder_params:
        decoder_params["eos_id"] = eos
      decodes, scores = self._decode_fn(
          inputs=decoder_prompt_inputs, cache=cache, tokens_to_logits=tokens_ids_to_logits,
          num_decodes=num_decodes, cache_offset=1 if scanned else 0, **decoder_params)
    if return_all_decodes:
      return decodes, {"scores": scores}
    return decodes[:, -1, :], {"scores": scores[:, -1]}

  def _graph_decoder(self, params, decoder_input_tokens, num_decodes, eos, decoder_params, rng,
                     prompt_with_targets):
    """The CUDA-graph beam decoder when it covers this call (bf16 T5 network on a GPU, beam
    search without a prompt and with default search options), else None."""
    import os
    if prompt_with_targets or rng is not None or os.environ.get("T5X_B200_GRAPH_DECODE") == "0":
      return None
    if params is not None and not _owns(self.module, params):
      return None
    extra = set(decoder_params or {}) - {"eos_id", "alpha"}
    if extra:
      return None
    from t5x_b200 import decoding_fast
    if not decoding_fast.supported(self.module, decoder_input_tokens, self._decode_fn):
      return None
    dp = decoder_params or {}
    key = (decoder_input_tokens.shape[0], num_decodes, decoder_input_tokens.shape[1],
           dp.get("eos_id", eos), dp.get("alpha", 0.6))
    cache = self.__dict__.setdefault("_graph_decoders", {})
    if key not in cache:
      cache.clear()  # one set of static buffers at a time
      cache[key] = decoding_fast.GraphBeamDecoder(self.module, key[0], key[1], key[2], key[3],
                                                  alpha=key[4])
    return cache[key]

  def score_batch(self, params, batch, return_intermediates: bool = False):
    """Sequence log-likelihoods (t5x/models.py:760-812)."""
    weights = batch["decoder_loss_weights"]
    targets = batch["decoder_target_tokens"].long()
    with torch.no_grad():
      fused = self._compute_hidden(params, batch, None)
      if fused is not None:
        hidden, weight, scale = fused
        saved = (self._z_loss, self._label_smoothing)
        self._z_loss, self._label_smoothing = 0.0, 0.0
        try:
          tok_loss, _, _ = self._token_losses(hidden, weight, scale, targets)
        finally:
          self._z_loss, self._label_smoothing = saved
        token_scores = -tok_loss * weights
      else:
        logits = self._compute_logits(params, batch)
        onehot = torch.nn.functional.one_hot(targets, logits.shape[-1]).float()
        token_scores = -losses.cross_entropy_with_logits(logits, onehot, z_loss=0.0)[0] * weights
      if token_scores.is_cuda:
        from t5x_b200.parallel import tp_fused
        tp_fused.end_step()
    sequence_scores = token_scores.sum(-1)
    if return_intermediates:
      intermediates = {"decoder": {"target_tokens": (targets,), "loss_weights": (weights,),
                                   "token_scores": (token_scores,)}}
      return sequence_scores, intermediates
    return sequence_scores


def remove_prefix(sequence: torch.Tensor, prefix_length: torch.Tensor) -> torch.Tensor:
  """Shifts each row left by its prefix length, zero-filling (t5x/models.py:1248-1282).
  `sequence` is [batch, len] or [batch, num_decodes, len]."""
  if sequence.dim() == 3:
    b, n, l = sequence.shape
    out = remove_prefix(sequence.reshape(b * n, l), prefix_length.repeat_interleave(n))
    return out.view(b, n, l)
  b, l = sequence.shape
  idx = torch.arange(l, device=sequence.device)[None, :] + prefix_length[:, None].long()
  valid = idx < l
  out = sequence.gather(1, idx.clamp(max=l - 1))
  return torch.where(valid, out, torch.zeros_like(out))


def count_packed_examples(segment_ids: torch.Tensor) -> torch.Tensor:
  """Number of packed examples in a [batch, length] segment-id array
  (t5x/models.py:1337-1368)."""
  seg = segment_ids.long()
  first = torch.cat([seg[:, :1], seg[:, 1:] - seg[:, :-1]], dim=-1)
  return (first > 0).sum()


def compute_base_metrics(logits, targets, mask, loss, z_loss=None, segment_ids=None,
                         correct=None) -> MetricsMap:
  """The standard train/eval metric set (t5x/models.py:1371-1469)."""
  num_examples = targets.shape[0]
  num_tokens = targets.numel()
  num_devices = max(1, pstate.get().world_size)
  nonpadding_tokens = mask.sum() if mask is not None else num_tokens
  if correct is not None:
    acc = metrics_lib.Accuracy.from_model_output(correct=correct, mask=mask)
  else:
    acc = metrics_lib.Accuracy.from_model_output(logits=logits, labels=targets, mask=mask)
  loss_d = loss.detach()
  metrics = {
      "accuracy": acc,
      "loss": metrics_lib.AveragePerStep(total=loss_d),
      "loss_per_nonpadding_target_token": metrics_lib.Average(total=loss_d,
                                                              count=nonpadding_tokens),
      "loss_per_all_target_tokens": metrics_lib.Average(total=loss_d, count=num_tokens),
      "timing/seqs_per_second": metrics_lib.TimeRate.from_model_output(numerator=num_examples),
      "timing/steps_per_second": metrics_lib.StepsPerTime.from_model_output(),
      "timing/seconds": metrics_lib.Time(),
      "timing/seqs": metrics_lib.Sum(num_examples),
      "timing/seqs_per_second_per_core": metrics_lib.TimeRate.from_model_output(
          numerator=num_examples / num_devices),
      "timing/target_tokens_per_second": metrics_lib.TimeRate.from_model_output(
          numerator=num_tokens),
      "timing/target_tokens_per_second_per_core": metrics_lib.TimeRate.from_model_output(
          numerator=num_tokens / num_devices),
      "non_padding_fraction/loss_weights": metrics_lib.Average(total=nonpadding_tokens,
                                                               count=num_tokens),
  }
  if z_loss is not None:
    z_d = z_loss.detach()
    metrics.update({
        "z_loss": metrics_lib.AveragePerStep(total=z_d),
        "z_loss_per_all_target_tokens": metrics_lib.Average(total=z_d, count=num_tokens),
        "cross_ent_loss": metrics_lib.AveragePerStep(total=loss_d - z_d),
        "cross_ent_loss_per_all_target_tokens": metrics_lib.Average(total=loss_d - z_d,
                                                                    count=num_tokens),
    })
  if segment_ids is not None:
    total_tokens = 0
    total_non_padding = 0
    for feature, seg in segment_ids.items():
      if seg is None or seg.shape[1] == 0:
        continue
      metrics[f"effective_batch_size/{feature}"] = metrics_lib.AveragePerStep(
          total=count_packed_examples(seg))
      non_pad = (seg != 0).sum()
      size = seg.numel()
      total_tokens += size
      total_non_padding = total_non_padding + non_pad
      metrics[f"non_padding_fraction/{feature}"] = metrics_lib.Average(total=non_pad, count=size)
    metrics["non_padding_fraction/overall"] = metrics_lib.Average(total=total_non_padding,
                                                                  count=total_tokens)
  return metrics


def get_input_vocabulary(model):
  return model.input_vocabulary


def get_output_vocabulary(model):
  return model.output_vocabulary
