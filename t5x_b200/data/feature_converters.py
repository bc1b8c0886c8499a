"""Feature converters: task features -> model features (the seqio.FeatureConverter contract
the reference models rely on, t5x/models.py:367,829 and the worked example at :1105-1148).
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Sequence

import numpy as np


def _pad(x: np.ndarray, length: int) -> np.ndarray:
  x = np.asarray(x)[:length]
  out = np.zeros((length,), dtype=np.int32)
  out[:len(x)] = x
  return out


def _shift_right_by_segment(targets: np.ndarray, segment_ids: Optional[np.ndarray]) -> np.ndarray:
  """Autoregressive inputs: shift right; position 0 of every packed segment becomes 0."""
  shifted = np.concatenate([[0], targets[:-1]]).astype(np.int32)
  if segment_ids is not None:
    starts = np.concatenate([[True], segment_ids[1:] != segment_ids[:-1]])
    shifted = np.where(starts, 0, shifted).astype(np.int32)
  return shifted


class FeatureConverter:
  """Base: `__call__(examples, task_feature_lengths)` yields model-feature dicts."""
  TASK_FEATURES: Sequence[str] = ()
  MODEL_FEATURES: Sequence[str] = ()
  PACKING_FEATURE_DTYPES = {}

  def __init__(self, pack: bool = True, use_custom_packing_ops: bool = False,
               apply_length_check: bool = True, bos_id: int = 0):
    self.pack = pack
    self.apply_length_check = apply_length_check
    self.bos_id = bos_id

  def get_model_feature_lengths(self, task_feature_lengths: Mapping[str, int]) -> Dict[str, int]:
    raise NotImplementedError

  def _pack(self, examples, lengths: Mapping[str, int], keys: Sequence[str]):
    """Greedy first-fit packing of consecutive examples into rows of `lengths`."""
    cur = None
    def new():
      return {k: [] for k in keys} | {k + "_seg": [] for k in keys} | {k + "_pos": [] for k in keys} | {"n": 0}
    for ex in examples:
      if cur is None:
        cur = new()
      fits = all(len(cur[k]) + min(len(ex[k]), lengths[k]) <= lengths[k] for k in keys)
      if not fits and cur["n"] > 0:
        yield cur
        cur = new()
      cur["n"] += 1
      for k in keys:
        v = list(ex[k])[:lengths[k]]
        cur[k].extend(v)
        cur[k + "_seg"].extend([cur["n"]] * len(v))
        cur[k + "_pos"].extend(range(len(v)))
    if cur is not None and cur["n"] > 0:
      yield cur

  def __call__(self, examples, task_feature_lengths: Mapping[str, int]):
    raise NotImplementedError


class EncDecFeatureConverter(FeatureConverter):
  """inputs/targets -> encoder_input_tokens, decoder_target_tokens, decoder_input_tokens,
  decoder_loss_weights (+ segment ids / positions when packing)."""
  TASK_FEATURES = ("inputs", "targets")
  MODEL_FEATURES = ("encoder_input_tokens", "decoder_target_tokens", "decoder_input_tokens",
                    "decoder_loss_weights")

  def get_model_feature_lengths(self, task_feature_lengths):
    el, dl = task_feature_lengths["inputs"], task_feature_lengths["targets"]
    out = {"encoder_input_tokens": el, "decoder_target_tokens": dl, "decoder_input_tokens": dl,
           "decoder_loss_weights": dl}
    if self.pack:
      out.update({"encoder_segment_ids": el, "decoder_segment_ids": dl, "encoder_positions": el,
                  "decoder_positions": dl})
    return out

  def __call__(self, examples, task_feature_lengths):
    el, dl = task_feature_lengths["inputs"], task_feature_lengths["targets"]
    if not self.pack:
      for ex in examples:
        tgt = _pad(ex["targets"], dl)
        yield {"encoder_input_tokens": _pad(ex["inputs"], el),
               "decoder_target_tokens": tgt,
               "decoder_input_tokens": _shift_right_by_segment(tgt, None),
               "decoder_loss_weights": (tgt > 0).astype(np.int32)}
      return
    for row in self._pack(examples, {"inputs": el, "targets": dl}, ("inputs", "targets")):
      tgt = _pad(row["targets"], dl)
      dseg = _pad(row["targets_seg"], dl)
      yield {"encoder_input_tokens": _pad(row["inputs"], el),
             "decoder_target_tokens": tgt,
             "decoder_input_tokens": _shift_right_by_segment(tgt, dseg),
             "decoder_loss_weights": (tgt > 0).astype(np.int32),
             "encoder_segment_ids": _pad(row["inputs_seg"], el),
             "decoder_segment_ids": dseg,
             "encoder_positions": _pad(row["inputs_pos"], el),
             "decoder_positions": _pad(row["targets_pos"], dl)}


class DecoderFeatureConverter(FeatureConverter):
  """Decoder-only LM: targets (optionally inputs as a prefix) -> decoder_* features.
  With `loss_on_targets_only` the prefix carries zero loss weight."""
  TASK_FEATURES = ("targets",)
  MODEL_FEATURES = ("decoder_target_tokens", "decoder_input_tokens", "decoder_loss_weights")

  def __init__(self, loss_on_targets_only: bool = True, pack: bool = True, **kw):
    super().__init__(pack=pack, **kw)
    self.loss_on_targets_only = loss_on_targets_only

  def get_model_feature_lengths(self, task_feature_lengths):
    dl = sum(task_feature_lengths.get(k, 0) for k in ("inputs", "targets"))
    out = {"decoder_target_tokens": dl, "decoder_input_tokens": dl, "decoder_loss_weights": dl}
    if "inputs" in task_feature_lengths:
      out["decoder_causal_attention"] = dl
    if self.pack:
      out.update({"decoder_segment_ids": dl, "decoder_positions": dl})
    return out

  def _concat(self, ex, task_feature_lengths):
    if "inputs" in ex and "inputs" in task_feature_lengths:
      inp = list(ex["inputs"])[:task_feature_lengths["inputs"]]
      tgt = list(ex["targets"])[:task_feature_lengths["targets"]]
      tokens = inp + tgt
      # inputs_width counts the prefix positions plus one (the reference's convention:
      # the position that predicts the first target still sees the inputs bidirectionally)
      causal = [1] * (len(inp) + 1) + [0] * max(0, len(tgt) - 1)
      weights = [0] * len(inp) + [1] * len(tgt) if self.loss_on_targets_only else [1] * len(tokens)
      return tokens, causal[:len(tokens)], weights
    tokens = list(ex["targets"])[:task_feature_lengths["targets"]]
    return tokens, None, [1] * len(tokens)

  def __call__(self, examples, task_feature_lengths):
    dl = sum(task_feature_lengths.get(k, 0) for k in ("inputs", "targets"))
    has_inputs = "inputs" in task_feature_lengths

    def rows():
      cur = {"t": [], "c": [], "w": [], "seg": [], "pos": [], "n": 0}
      for ex in examples:
        tokens, causal, weights = self._concat(ex, task_feature_lengths)
        if self.pack and cur["n"] > 0 and len(cur["t"]) + len(tokens) > dl:
          yield cur
          cur = {"t": [], "c": [], "w": [], "seg": [], "pos": [], "n": 0}
        cur["n"] += 1
        cur["t"] += tokens
        cur["c"] += (causal or [0] * len(tokens))
        cur["w"] += weights
        cur["seg"] += [cur["n"]] * len(tokens)
        cur["pos"] += list(range(len(tokens)))
        if not self.pack:
          yield cur
          cur = {"t": [], "c": [], "w": [], "seg": [], "pos": [], "n": 0}
      if cur["n"] > 0:
        yield cur

    for row in rows():
      tgt = _pad(row["t"], dl)
      seg = _pad(row["seg"], dl) if self.pack else None
      out = {"decoder_target_tokens": tgt,
             "decoder_input_tokens": _shift_right_by_segment(tgt, seg),
             "decoder_loss_weights": _pad(row["w"], dl) * (tgt > 0)}
      if has_inputs:
        out["decoder_causal_attention"] = _pad(row["c"], dl)
      if self.pack:
        out["decoder_segment_ids"] = seg
        out["decoder_positions"] = _pad(row["pos"], dl)
      yield out


class PrefixLMFeatureConverter(DecoderFeatureConverter):
  """inputs + targets concatenated for a prefix LM; inputs attend bidirectionally."""
  TASK_FEATURES = ("inputs", "targets")
  MODEL_FEATURES = ("decoder_target_tokens", "decoder_input_tokens", "decoder_loss_weights",
                    "decoder_causal_attention")


class LMFeatureConverter(DecoderFeatureConverter):
  TASK_FEATURES = ("targets",)
