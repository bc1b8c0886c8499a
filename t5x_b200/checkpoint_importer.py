"""Import of Mesh-TensorFlow T5 checkpoints (API of t5x/checkpoint_importer.py).

A checkpoint is read as a flat `{name: LazyArray}` mapping, renamed by a `CheckpointTranslator`
(regular-expression rules -> T5X state-dict keys) and merged into the optimizer state dict.
The default translator covers T5 encoder-decoder and decoder-only ("transformer/") variables
together with their Adafactor slots (`_slot_v`, `_slot_vr`, `_slot_vc`).

Reading does not need TensorFlow: `io/tf_bundle.py` parses the tensor-bundle files directly.
"""
from __future__ import annotations

import concurrent.futures
import re
from typing import Any, Callable, Mapping, MutableMapping, Optional

import numpy as np

from t5x_b200.checkpoints import LazyArray  # noqa: F401  (re-export, reference name)
from t5x_b200.utils import tree as tree_utils


class LazyThreadPoolArray(LazyArray):
  """LazyArray whose `get_async` runs the read on a shared thread pool
  (t5x/checkpoint_importer.py:102-131)."""

  executor = concurrent.futures.ThreadPoolExecutor(max_workers=8)

  def get_async(self) -> concurrent.futures.Future:
    return self.executor.submit(self.get)


class LazyAwaitableArray(LazyArray):
  """LazyArray built from a function that returns either the array or a future of it
  (t5x/checkpoint_importer.py:134-186)."""

  def get_async(self) -> concurrent.futures.Future:
    fut = concurrent.futures.Future()
    try:
      res = self._get_fn()
      if isinstance(res, concurrent.futures.Future):
        return res
      fut.set_result(res)
    except Exception as e:  # pylint: disable=broad-except
      fut.set_exception(e)
    return fut

  def get(self):
    return self.get_async().result()

  @classmethod
  def from_array(cls, array, get_fn, dtype=None):
    return cls(array.shape, dtype or array.dtype, get_fn)

  @classmethod
  def from_tensor_store_spec_or_array(cls, maybe_spec, get_fn, dtype=None):
    if hasattr(maybe_spec, "shape"):
      return cls.from_array(maybe_spec, get_fn, dtype)
    return cls(tuple(maybe_spec.get("metadata", {}).get("shape", ())),
               dtype or maybe_spec.get("dtype", np.float32), get_fn)


class CheckpointTranslator:
  """Ordered regex rules from one flat-key dictionary to another. A rule function receives
  `(opts, key, value, *regex_groups)` and returns `(new_key, new_value)`; a `None` key drops
  the entry. Every pattern must match the whole key."""

  def __init__(self):
    self.rules = []

  def add(self, pattern: str):
    def register(fn):
      self.rules.append((re.compile(pattern + "$"), fn))
      return fn
    return register

  def apply(self, flatdict: Mapping[str, Any], **opts) -> dict:
    out, unmatched = {}, {}
    for key, value in flatdict.items():
      for pattern, fn in self.rules:
        m = pattern.match(key)
        if m:
          new_key, new_value = fn(opts, key, value, *m.groups())
          if new_key is not None:
            out[new_key] = new_value
          break
      else:
        unmatched[key] = value
    if unmatched:
      raise ValueError(f"Unmapped tensor keys exist: {unmatched}")
    return out


# ----------------------------------------------------------------------------
# T5 rules
# ----------------------------------------------------------------------------
SLOT_MAP = {"_slot_vc": "v_col", "_slot_vr": "v_row", "_slot_v": "v"}
TOWER_MAP = {"transformer": "decoder"}
_TOWER = r"(encoder|decoder|transformer)"
_QKVO = {"q": "query", "k": "key", "v": "value", "o": "out"}
_NORMS = {
    "encoder": ("pre_attention_layer_norm", "pre_mlp_layer_norm"),
    "decoder": ("pre_self_attention_layer_norm", "pre_cross_attention_layer_norm",
                "pre_mlp_layer_norm"),
    "transformer": ("pre_self_attention_layer_norm", "pre_mlp_layer_norm"),
}
_FINAL_NORM = {"encoder": "encoder_norm", "decoder": "decoder_norm", "transformer": "decoder_norm"}


def _placed(slot: str, path: str) -> str:
  """`target/<path>` for a variable, `state/param_states/<path>/<slot name>` for a slot."""
  if slot:
    return f"state/param_states/{path}/{SLOT_MAP[slot]}"
  return f"target/{path}"


def _tower(name: str) -> str:
  return TOWER_MAP.get(name, name)


def _build_t5_importer() -> CheckpointTranslator:
  tr = CheckpointTranslator()

  @tr.add(r"global_step")
  def _step(opts, key, val):
    return "state/step", (val.astype(np.int32).get() if isinstance(val, LazyArray) else val)

  @tr.add(r"shared/embedding(\w*)")
  def _shared(opts, key, val, slot):
    return _placed(slot, "token_embedder/embedding"), val

  @tr.add(_TOWER + r"/embedding(\w*)")
  def _separate(opts, key, val, tower, slot):
    return _placed(slot, f"{_tower(tower)}/token_embedder/embedding"), val

  @tr.add(_TOWER + r"/block_(\d+)/layer_000/SelfAttention/relative_attention_bias(\w*)")
  def _relpos(opts, key, val, tower, block, slot):
    # kept per layer here; collapsed afterwards when only block 0 carries one
    return _placed(slot, f"{_tower(tower)}/layers_{int(block)}/relpos_bias/rel_embedding"), val

  @tr.add(_TOWER + r"/block_(\d+)/layer_\d+/(SelfAttention|EncDecAttention)/(q|k|v|o)(\w*)")
  def _attention(opts, key, val, tower, block, kind, which, slot):
    if tower == "encoder":
      name = "attention"
    else:
      name = "self_attention" if kind == "SelfAttention" else "encoder_decoder_attention"
    return _placed(slot, f"{_tower(tower)}/layers_{int(block)}/{name}/{_QKVO[which]}/kernel"), val

  @tr.add(_TOWER + r"/block_(\d+)/layer_\d+/DenseReluDense/(wi|wo)(?:_(\d+))?/kernel(\w*)")
  def _mlp(opts, key, val, tower, block, io_name, io_num, slot):
    dense = io_name + (f"_{io_num}" if io_num else "")
    return _placed(slot, f"{_tower(tower)}/layers_{int(block)}/mlp/{dense}/kernel"), val

  @tr.add(_TOWER + r"/block_(\d+)/layer_(\d+)/(?:layer|rms)_norm/scale(\w*)")
  def _norm(opts, key, val, tower, block, layer, slot):
    name = _NORMS[tower][int(layer)]
    return _placed(slot, f"{_tower(tower)}/layers_{int(block)}/{name}/scale"), val

  @tr.add(_TOWER + r"/(?:final_layer|rms)_norm/scale(\w*)")
  def _final_norm(opts, key, val, tower, slot):
    return _placed(slot, f"{_tower(tower)}/{_FINAL_NORM[tower]}/scale"), val

  @tr.add(r"(?:decoder|transformer)/logits/kernel(\w*)")
  def _logits(opts, key, val, slot):
    return _placed(slot, "decoder/logits_dense/kernel"), val

  return tr


t5_importer = _build_t5_importer()


def _add_missing_param_states(t5_data: MutableMapping[str, Any]) -> MutableMapping[str, Any]:
  """The (1,)-shaped placeholders T5X's Adafactor state carries for the slots a parameter does
  not use (momentum always; `v` or `v_row`/`v_col` depending on factoring)."""
  extra = {}
  one = lambda: np.zeros((1,), np.float32)
  for k in t5_data:
    if not k.startswith("target"):
      continue
    leaf = "state/param_states" + k[len("target"):]
    extra[leaf + "/m"] = one()
    if leaf + "/v" in t5_data:
      extra[leaf + "/v_row"] = one()
      extra[leaf + "/v_col"] = one()
    elif leaf + "/v_row" in t5_data:
      extra[leaf + "/v"] = one()
  t5_data.update(extra)
  return t5_data


def _maybe_correct_relpos_bias(t5_data: Mapping[str, Any]) -> Mapping[str, Any]:
  """When only layer 0 has a relative-position bias it is the one shared by the whole stack:
  `.../layers_0/relpos_bias` -> `.../relpos_bias`."""
  layers = [int(m.group(1)) for k in t5_data
            for m in [re.search(r"layers_(\d+)/relpos_bias", k)] if m]
  if layers and max(layers) > 0:
    return t5_data
  return {re.sub(r"layers_\d+/relpos_bias", "relpos_bias", k): v for k, v in t5_data.items()}


def load_tf_ckpt(path: str) -> dict:
  """A TensorFlow checkpoint as `{variable name: LazyThreadPoolArray}`."""
  from t5x_b200.io import tf_bundle
  reader = tf_bundle.BundleReader(path)
  return {name: LazyThreadPoolArray(entry.shape, entry.dtype,
                                    lambda n=name: reader.get_tensor(n))
          for name, entry in reader.entries.items()}


def _update_state_dict(state_dict: Mapping[str, Any], t5_data: MutableMapping[str, Any],
                       strict: bool = True) -> Mapping[str, Any]:
  flat = tree_utils.flatten_dict(state_dict, keep_empty_nodes=True)
  if not strict:
    for k in list(t5_data):
      if k not in flat:
        t5_data.pop(k)
  for k, v in t5_data.items():
    if k not in flat:
      raise KeyError(f"Variable {k} of the checkpoint is not part of the model state")
    want = tuple(getattr(flat[k], "shape", ()))
    if want != tuple(v.shape):
      raise ValueError(f"Variable {k} has shape {tuple(v.shape)} != {want}")
  return tree_utils.unflatten_dict(dict(t5_data))


def restore_from_t5_checkpoint(state_dict: Mapping[str, Any], path: str,
                               lazy_parameters: bool = False, strict: bool = True,
                               translator: Optional[CheckpointTranslator] = None):
  """State dict (target + Adafactor state) filled from a Mesh-TensorFlow T5 checkpoint; its
  structure must match the model's up to the shapes of the leaves
  (t5x/checkpoint_importer.py:522-566)."""
  translator = translator or t5_importer
  t5_data = translator.apply(load_tf_ckpt(path))
  t5_data = _add_missing_param_states(t5_data)
  t5_data = _maybe_correct_relpos_bias(t5_data)
  new_state = _update_state_dict(state_dict, dict(t5_data), strict=strict)
  if not lazy_parameters:
    new_state = tree_utils.tree_map(lambda x: x.get() if isinstance(x, LazyArray) else x,
                                    new_state)
  return new_state
