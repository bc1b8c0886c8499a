"""Train state objects (API of t5x/train_state.py).

`FlaxOptimTrainState` keeps the legacy name and `state_dict()` layout
`{'target', 'state': {'step', 'param_states'}[, 'flax_mutables']}` that the checkpoint
format is built on. Parameters are the live `torch.nn.Parameter`s of the model's module, so
restoring a state dict copies values INTO them (identity is preserved, the bf16 working
copies and gradient buffers attached to each parameter stay valid).
"""
from __future__ import annotations

import dataclasses
from typing import Any, Mapping, Optional

import numpy as np
import torch

from t5x_b200 import optimizers
from t5x_b200.utils import tree as tree_utils

EMPTY_DICT: dict = {}


def _leaf_axes(x) -> bool:
  return not isinstance(x, Mapping)


def _validate_params_axes(params_axes, params):
  """Checks that every parameter has axis names of matching rank
  (t5x/train_state.py:88-97)."""
  flat_axes = tree_utils.flatten_dict(params_axes, is_leaf=_leaf_axes)
  flat_params = tree_utils.flatten_dict(params)
  missing = set(flat_params) - set(flat_axes)
  if missing:
    raise ValueError(f"Missing axis names for parameters: {sorted(missing)}")
  for k, axes in flat_axes.items():
    if k in flat_params and axes is not None and len(axes) != flat_params[k].dim():
      raise ValueError(f"Axis names {axes} do not match the rank of parameter {k} "
                       f"{tuple(flat_params[k].shape)}")


def _as_tensor(value) -> torch.Tensor:
  if hasattr(value, "get") and not isinstance(value, Mapping):  # LazyArray
    value = value.get()
  arr = np.asarray(value)
  if arr.dtype.name == "bfloat16":
    return torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16)
  return torch.as_tensor(arr)


def _copy_into(target, value, path=""):
  """Recursively copies `value` leaves into `target` tensors in place."""
  if isinstance(target, Mapping):
    if not isinstance(value, Mapping) or set(target.keys()) != set(value.keys()):
      tk = set(target.keys())
      vk = set(value.keys()) if isinstance(value, Mapping) else set()
      raise ValueError(f"The target dict keys and state dict keys do not match at '{path}': "
                       f"missing {sorted(tk - vk)}, unexpected {sorted(vk - tk)}")
    return {k: _copy_into(target[k], value[k], f"{path}/{k}" if path else k) for k in target}
  if isinstance(target, torch.Tensor):
    src = value if isinstance(value, torch.Tensor) else _as_tensor(value)
    if tuple(src.shape) != tuple(target.shape):
      raise ValueError(f"Shape mismatch restoring '{path}': checkpoint {tuple(src.shape)} vs "
                       f"state {tuple(target.shape)}")
    with torch.no_grad():
      target.copy_(src.to(device=target.device, dtype=target.dtype))
      bf = getattr(target, "bf16", None)
      if bf is not None:
        bf.copy_(target)
    return target
  return value


@dataclasses.dataclass
class FlaxOptimTrainState:
  """Parameters + optimizer state + step (t5x/train_state.py:115-231)."""
  _optimizer: optimizers.Optimizer
  params_axes: Optional[Mapping[str, Any]] = None
  flax_mutables: Mapping[str, Any] = dataclasses.field(default_factory=dict)
  flax_mutables_axes: Optional[Mapping[str, Any]] = None

  @classmethod
  def create(cls, optimizer_def: optimizers.OptimizerDef,
             model_variables: Mapping[str, Any]) -> "FlaxOptimTrainState":
    other = dict(model_variables)
    params = other.pop("params")
    params_axes = other.pop("params_axes", None)
    if params_axes is not None:
      _validate_params_axes(params_axes, params)
    mutables = {k: v for k, v in other.items() if not k.endswith("_axes")}
    mutables_axes = {k[:-5]: v for k, v in other.items() if k.endswith("_axes")}
    if hasattr(optimizer_def, "set_param_axes"):
      if params_axes is None:
        raise ValueError("The optimizer supports params_axes for model-based partitioning, "
                         "but the model is not emitting them.")
      optimizer_def.set_param_axes(params_axes)
    optimizer = optimizer_def.create(params)
    return cls(optimizer, params_axes=params_axes, flax_mutables=mutables,
               flax_mutables_axes=mutables_axes or None)

  def replace(self, **kw):
    return dataclasses.replace(self, **kw)

  @property
  def step(self):
    return self._optimizer.state.step

  @property
  def params(self):
    return self._optimizer.target

  @property
  def param_states(self):
    return self._optimizer.state.param_states

  def state_dict(self):
    sd = self._optimizer.state_dict()
    if self.flax_mutables:
      sd["flax_mutables"] = dict(self.flax_mutables)
    return sd

  def apply_gradient(self, grads, learning_rate, flax_mutables=EMPTY_DICT):
    new_opt = self._optimizer.apply_gradient(grads, learning_rate=learning_rate)
    return self.replace(_optimizer=new_opt, flax_mutables=flax_mutables or {})

  def replace_params(self, params):
    _copy_into(self._optimizer.target, params)
    return self

  def replace_flax_mutables(self, flax_mutables):
    return self.replace(flax_mutables=flax_mutables)

  def replace_step(self, step):
    st = self._optimizer.state
    new_step = torch.as_tensor(step, dtype=torch.int32)
    return self.replace(_optimizer=self._optimizer.replace(state=st.replace(step=new_step)))

  def restore_state(self, state_dict):
    opt = self._optimizer
    _copy_into(opt.target, state_dict["target"], "target")
    new_ps = _copy_into(opt.state.param_states, state_dict["state"]["param_states"],
                        "state/param_states")
    step = torch.as_tensor(np.asarray(state_dict["state"]["step"]), dtype=torch.int32)
    new_opt = opt.replace(state=optimizers.OptimizerState(step=step, param_states=new_ps))
    return self.replace(_optimizer=new_opt,
                        flax_mutables=dict(state_dict.get("flax_mutables", {})))

  def as_logical_axes(self):
    od = self._optimizer.optimizer_def
    if not hasattr(od, "derive_logical_axes"):
      raise ValueError(f"Optimizer '{od.__class__.__name__}' requires a `derive_logical_axes` "
                       "method to be used with named axis partitioning.")
    return FlaxOptimTrainState(
        _optimizer=od.derive_logical_axes(self._optimizer, self.params_axes),
        flax_mutables=self.flax_mutables_axes or {})


@dataclasses.dataclass
class InferenceState:
  """Parameters and step only (t5x/train_state.py:234-318)."""
  step: Any
  params: Mapping[str, Any]
  params_axes: Optional[Mapping[str, Any]] = None
  flax_mutables: Mapping[str, Any] = dataclasses.field(default_factory=dict)
  flax_mutables_axes: Optional[Mapping[str, Any]] = None

  @classmethod
  def create(cls, model_variables: Mapping[str, Any]) -> "InferenceState":
    other = dict(model_variables)
    params = other.pop("params")
    params_axes = other.pop("params_axes", None)
    if params_axes is not None:
      _validate_params_axes(params_axes, params)
    mutables = {k: v for k, v in other.items() if not k.endswith("_axes")}
    mutables_axes = {k[:-5]: v for k, v in other.items() if k.endswith("_axes")}
    return cls(step=torch.zeros((), dtype=torch.int32), params=params, params_axes=params_axes,
               flax_mutables=mutables, flax_mutables_axes=mutables_axes or None)

  def replace(self, **kw):
    return dataclasses.replace(self, **kw)

  @property
  def param_states(self):
    raise NotImplementedError("InferenceState has no optimizer states.")

  def apply_gradient(self, *args, **kwargs):
    raise NotImplementedError("InferenceState does not support `apply_gradient`.")

  def state_dict(self):
    sd = {"target": self.params, "state": {"step": self.step}}
    if self.flax_mutables:
      sd["flax_mutables"] = dict(self.flax_mutables)
    return sd

  def replace_step(self, step):
    return self.replace(step=torch.as_tensor(step, dtype=torch.int32))

  def replace_params(self, params):
    _copy_into(self.params, params)
    return self

  def replace_flax_mutables(self, flax_mutables):
    return self.replace(flax_mutables=flax_mutables)

  def restore_state(self, state_dict):
    _copy_into(self.params, state_dict["target"], "target")
    step = torch.as_tensor(np.asarray(state_dict["state"]["step"]), dtype=torch.int32)
    return self.replace(step=step, flax_mutables=dict(state_dict.get("flax_mutables", {})))

  def as_logical_axes(self):
    return InferenceState(step=None, params=self.params_axes,
                          flax_mutables=self.flax_mutables_axes or {})


TrainState = FlaxOptimTrainState  # the protocol's canonical implementation
