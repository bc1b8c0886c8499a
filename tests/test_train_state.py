"""`FlaxOptimTrainState` and `InferenceState`: creation with axis names and mutable collections,
validation errors, step / parameter replacement, gradient application, logical axes, state
dicts and restoring (the behaviours of t5x/train_state_test.py)."""
import numpy as np
import pytest
import torch

from t5x_b200 import adafactor, optimizers
from t5x_b200 import train_state as ts_lib
from t5x_b200.utils import tree


def _variables(with_mutables=False):
  v = {"params": {"dense": {"kernel": torch.ones(128, 256), "bias": torch.zeros(256)},
                  "embedding": torch.full((256, 128), 2.0)},
       "params_axes": {"dense": {"kernel": ("embed", "mlp"), "bias": ("mlp",)},
                       "embedding": ("vocab", "embed")}}
  if with_mutables:
    v["cache"] = {"index": torch.zeros((), dtype=torch.int32)}
    v["cache_axes"] = {"index": ()}
  return v


def _adafactor():
  return adafactor.Adafactor(decay_rate=0.8, step_offset=0, factored=True,
                             logical_factor_rules=adafactor.standard_logical_factor_rules())


def test_create_keeps_params_axes_and_mutables():
  state = ts_lib.FlaxOptimTrainState.create(_adafactor(), _variables(with_mutables=True))
  assert int(state.step) == 0
  assert state.params["dense"]["kernel"].shape == (128, 256)
  assert state.params_axes["embedding"] == ("vocab", "embed")
  assert set(state.flax_mutables) == {"cache"}
  assert state.flax_mutables_axes == {"cache": {"index": ()}}
  # a factored slot per matrix, an unfactored one for the vector
  slots = tree.flatten_dict(state.param_states)
  assert slots["dense/kernel/v_row"].shape == (128,) and slots["dense/kernel/v_col"].shape == (256,)
  assert slots["dense/bias/v"].shape == (256,)


def test_create_rejects_missing_or_mismatched_axes():
  v = _variables()
  del v["params_axes"]["embedding"]
  with pytest.raises(ValueError, match="Missing axis names.*embedding"):
    ts_lib.FlaxOptimTrainState.create(_adafactor(), v)
  v = _variables()
  v["params_axes"]["dense"]["kernel"] = ("embed",)
  with pytest.raises(ValueError, match="do not match the rank"):
    ts_lib.FlaxOptimTrainState.create(_adafactor(), v)
  v = _variables()
  del v["params_axes"]
  with pytest.raises(ValueError, match="not emitting them"):
    ts_lib.FlaxOptimTrainState.create(_adafactor(), v)   # Adafactor factors by axis name
  with pytest.raises(ValueError, match="not emitting them"):
    ts_lib.FlaxOptimTrainState.create(optimizers.sgd(0.1), v)   # the wrappers derive axes too


def test_replace_step_and_params():
  state = ts_lib.FlaxOptimTrainState.create(_adafactor(), _variables())
  later = state.replace_step(7)
  assert int(later.step) == 7 and int(state.step) == 0
  new = {"dense": {"kernel": torch.full((128, 256), 3.0), "bias": torch.ones(256)},
         "embedding": torch.zeros(256, 128)}
  kernel = state.params["dense"]["kernel"]
  state.replace_params(new)
  assert kernel is state.params["dense"]["kernel"]       # values change, storage stays
  assert float(kernel.sum()) == 3.0 * 128 * 256
  with pytest.raises(ValueError, match="Shape mismatch"):
    state.replace_params({**new, "embedding": torch.zeros(256, 5)})
  with pytest.raises(ValueError, match="do not match"):
    state.replace_params({"dense": new["dense"]})


def test_apply_gradient_steps_the_optimizer_and_swaps_mutables():
  state = ts_lib.FlaxOptimTrainState.create(optimizers.sgd(0.5), _variables(with_mutables=True))
  grads = tree.tree_map(torch.ones_like, state.params)
  new = state.apply_gradient(grads, learning_rate=0.5,
                             flax_mutables={"cache": {"index": torch.tensor(3)}})
  assert int(new.step) == 1
  torch.testing.assert_close(new.params["dense"]["kernel"], torch.full((128, 256), 0.5))
  torch.testing.assert_close(new.params["embedding"], torch.full((256, 128), 1.5))
  assert int(new.flax_mutables["cache"]["index"]) == 3


def test_as_logical_axes_follow_the_factoring():
  state = ts_lib.FlaxOptimTrainState.create(_adafactor(), _variables(with_mutables=True))
  axes = state.as_logical_axes()
  assert axes.params["dense"]["kernel"] == ("embed", "mlp")
  slot_axes = tree.flatten_dict(axes.param_states, is_leaf=lambda x: not isinstance(x, dict))
  # factored statistics are small and stay replicated; an unfactored second moment and the
  # momentum (when there is one) are laid out like their parameter
  assert slot_axes["dense/kernel/v_row"] is None and slot_axes["dense/kernel/v_col"] is None
  assert slot_axes["dense/kernel/v"] is None
  assert tuple(slot_axes["dense/bias/v"]) == ("mlp",)
  assert slot_axes["dense/kernel/m"] is None
  with_momentum = adafactor.Adafactor(
      decay_rate=0.8, step_offset=0, beta1=0.9,
      logical_factor_rules=adafactor.standard_logical_factor_rules())
  m_axes = tree.flatten_dict(
      ts_lib.FlaxOptimTrainState.create(with_momentum, _variables()).as_logical_axes().param_states,
      is_leaf=lambda x: not isinstance(x, dict))
  assert tuple(m_axes["dense/kernel/m"]) == ("embed", "mlp")
  assert axes.flax_mutables == {"cache": {"index": ()}}
  plain = ts_lib.FlaxOptimTrainState.create(_adafactor(), _variables())
  assert plain.as_logical_axes().flax_mutables == {}


def test_state_dict_layout_and_restore_round_trip():
  state = ts_lib.FlaxOptimTrainState.create(_adafactor(), _variables(with_mutables=True))
  sd = state.state_dict()
  assert set(sd) == {"target", "state", "flax_mutables"}
  assert set(sd["state"]) == {"step", "param_states"}
  assert set(tree.flatten_dict(sd["target"])) == {"dense/kernel", "dense/bias", "embedding"}
  # a checkpoint-like dict of numpy arrays with other values
  new_sd = {
      "target": {"dense": {"kernel": np.full((128, 256), 5.0, np.float32),
                           "bias": np.arange(256, dtype=np.float32)},
                 "embedding": np.full((256, 128), -1.0, np.float32)},
      "state": {"step": np.int32(12),
                "param_states": tree.tree_map(lambda t: np.full(tuple(t.shape), 0.25, np.float32),
                                              sd["state"]["param_states"])},
      "flax_mutables": {"cache": {"index": np.int32(9)}}}
  restored = state.restore_state(new_sd)
  assert int(restored.step) == 12
  assert float(restored.params["dense"]["kernel"][0, 0]) == 5.0
  assert restored.params["dense"]["bias"].tolist() == list(range(256))
  assert all(float(v.flatten()[0]) == 0.25
             for v in tree.flatten_dict(restored.param_states).values() if v.numel())
  assert int(restored.flax_mutables["cache"]["index"]) == 9
  broken = {**new_sd, "target": {"embedding": new_sd["target"]["embedding"]}}
  with pytest.raises(ValueError, match="do not match at 'target'"):
    state.restore_state(broken)
  # without the mutables the dict has no such key
  assert "flax_mutables" not in ts_lib.FlaxOptimTrainState.create(
      _adafactor(), _variables()).state_dict()


# ---- InferenceState -----------------------------------------------------------------------------
def test_inference_state():
  state = ts_lib.InferenceState.create(_variables(with_mutables=True))
  assert int(state.step) == 0 and state.params_axes["embedding"] == ("vocab", "embed")
  assert set(state.flax_mutables) == {"cache"}
  with pytest.raises(NotImplementedError):
    state.param_states
  with pytest.raises(NotImplementedError):
    state.apply_gradient({}, 0.1)
  assert int(state.replace_step(4).step) == 4
  sd = state.state_dict()
  assert set(sd) == {"target", "state", "flax_mutables"} and set(sd["state"]) == {"step"}
  axes = state.as_logical_axes()
  assert axes.params["dense"]["bias"] == ("mlp",) and axes.step is None
  restored = state.restore_state({
      "target": tree.tree_map(lambda t: np.zeros(tuple(t.shape), np.float32), sd["target"]),
      "state": {"step": np.int32(3)}})
  assert int(restored.step) == 3 and float(restored.params["embedding"].abs().sum()) == 0.0
  assert restored.flax_mutables == {}
  v = _variables()
  v["params_axes"]["embedding"] = ("vocab",)
  with pytest.raises(ValueError, match="do not match the rank"):
    ts_lib.InferenceState.create(v)
  bare = ts_lib.InferenceState.create({"params": {"w": torch.ones(2)}})
  assert bare.params_axes is None and "flax_mutables" not in bare.state_dict()
