"""Optimizer framework (API of t5x/optimizers.py).

`OptimizerDef` / `Optimizer` / `OptimizerState` keep the legacy Flax contract that the
train state and checkpoints rely on: `state_dict()` is
`{'target': params, 'state': {'step': int, 'param_states': tree}}`.
Parameters are updated IN PLACE (PyTorch idiom; the "new" optimizer returned by
`apply_gradient` shares the updated tensors), which is what lets the CUDA optimizer
kernels also refresh the bf16 working copies in the same pass.

The optax-style constructors (`adam`, `adamw`, `lion`, `sgd`, ... , `chain`) are small
gradient transformations written here (optax itself is not a dependency) and wrapped by
`OptaxWrapper` so they expose the same OptimizerDef interface and a serialisable state.
"""
from __future__ import annotations

import dataclasses
import math
import re
from typing import Any, Callable, Dict, Mapping, NamedTuple, Optional, Sequence, Tuple, Union

import torch

from t5x_b200.utils import tree as tree_utils

flatten = tree_utils.flatten_dict
unflatten = tree_utils.unflatten_dict


@dataclasses.dataclass
class OptimizerState:
  step: Any
  param_states: Any

  def replace(self, **kw):
    return dataclasses.replace(self, **kw)


def _to_state_dict(x):
  if dataclasses.is_dataclass(x) and not isinstance(x, type):
    return {f.name: _to_state_dict(getattr(x, f.name)) for f in dataclasses.fields(x)}
  if isinstance(x, Mapping):
    return {k: _to_state_dict(v) for k, v in x.items()}
  if isinstance(x, (list, tuple)):
    if all(v is None or isinstance(v, (str, tuple)) for v in x):
      return x  # a tuple of axis names is a leaf
    return {str(i): _to_state_dict(v) for i, v in enumerate(x)}
  return x


def _from_state_dict(target, state):
  """Restores `state` into the structure of `target` (flax.serialization.from_state_dict)."""
  if dataclasses.is_dataclass(target) and not isinstance(target, type):
    vals = {f.name: _from_state_dict(getattr(target, f.name), state[f.name])
            for f in dataclasses.fields(target)}
    return dataclasses.replace(target, **vals)
  if isinstance(target, Mapping):
    missing = set(target.keys()) ^ set(state.keys())
    if missing:
      raise ValueError(f"The target dict keys and state dict keys do not match: {sorted(missing)}")
    return {k: _from_state_dict(v, state[k]) for k, v in target.items()}
  if isinstance(target, (list, tuple)):
    vals = [_from_state_dict(v, state[str(i)]) for i, v in enumerate(target)]
    return type(target)(vals)
  return state


to_state_dict = _to_state_dict
from_state_dict = _from_state_dict


class OptimizerDef:
  """Base class for an optimizer definition (t5x/optimizers.py:52-118)."""

  def __init__(self, hyper_params):
    self.hyper_params = hyper_params

  def apply_gradient(self, hyper_params, params, state, grads):
    raise NotImplementedError()

  def init_state(self, params):
    raise NotImplementedError()

  def update_hyper_params(self, **hyper_param_overrides):
    hp = hyper_param_overrides.pop("hyper_params", self.hyper_params)
    if hyper_param_overrides:
      hp = dataclasses.replace(hp, **hyper_param_overrides)
    return hp

  def create(self, target):
    return Optimizer(self, self.init_state(target), target)

  def state_dict(self, target, state):
    return {"target": _to_state_dict(target), "state": _to_state_dict(state)}

  def restore_state(self, opt_target, opt_state, state_dict):
    opt_target = _from_state_dict(opt_target, state_dict["target"])
    opt_state = _from_state_dict(opt_state, state_dict["state"])
    return opt_target, opt_state

  # Hooks used by the train state / partitioner.
  def set_param_axes(self, param_logical_axes) -> None:
    pass

  def derive_logical_axes(self, optimizer, param_logical_axes):
    raise NotImplementedError()


@dataclasses.dataclass
class Optimizer:
  """Target + optimizer state (t5x/optimizers.py:121-164)."""
  optimizer_def: OptimizerDef
  state: Any
  target: Any

  def replace(self, **kw):
    return dataclasses.replace(self, **kw)

  def apply_gradient(self, grads, **hyper_param_overrides):
    hyper_params = self.optimizer_def.update_hyper_params(**hyper_param_overrides)
    new_target, new_state = self.optimizer_def.apply_gradient(hyper_params, self.target,
                                                              self.state, grads)
    return self.replace(target=new_target, state=new_state)

  def state_dict(self):
    return self.optimizer_def.state_dict(self.target, self.state)

  def restore_state(self, state):
    target, state = self.optimizer_def.restore_state(self.target, self.state, state)
    return self.replace(target=target, state=state)


OptimizerType = Optimizer
OptimizerStateType = Union[OptimizerState, Mapping[str, Any]]
OptimizerDefType = OptimizerDef


# ----------------------------------------------------------------------------
# Gradient transformations (the subset of optax that the reference wraps)
# ----------------------------------------------------------------------------
class GradientTransformation(NamedTuple):
  init: Callable[[Dict[str, torch.Tensor]], Any]
  update: Callable[..., Tuple[Dict[str, torch.Tensor], Any]]
  name: str = "transform"
  # what the transformation was built with (read by OptaxWrapper to recognise chains that a
  # fused kernel covers); for a chain: {"transforms": [...]}
  hparams: Mapping[str, Any] = {}


def _zeros_like_tree(params):
  return {k: torch.zeros_like(v, dtype=torch.float32) for k, v in params.items()}


# Learning rate handed in by the caller of `Optimizer.apply_gradient(learning_rate=...)` for the
# duration of one OptaxWrapper update; transformations built with `learning_rate=None` use it.
_STEP_LEARNING_RATE = [None]


def _lr(learning_rate, count):
  if learning_rate is None:
    if _STEP_LEARNING_RATE[0] is None:
      raise ValueError("This optimizer was built with learning_rate=None: pass "
                       "`learning_rate=` to apply_gradient (the trainer does).")
    return float(_STEP_LEARNING_RATE[0])
  return learning_rate(count) if callable(learning_rate) else learning_rate


def scale(step_size: float) -> GradientTransformation:
  return GradientTransformation(lambda p: {}, lambda u, s, p=None: (
      {k: v * step_size for k, v in u.items()}, s), "scale")


def scale_by_learning_rate(learning_rate, flip_sign=True) -> GradientTransformation:
  sign = -1.0 if flip_sign else 1.0

  def init(params):
    return {"count": torch.zeros((), dtype=torch.int32)}

  def update(updates, state, params=None):
    lr = _lr(learning_rate, int(state["count"]))
    return {k: v * (sign * lr) for k, v in updates.items()}, {"count": state["count"] + 1}

  return GradientTransformation(init, update, "scale_by_schedule",
                                {"learning_rate": learning_rate, "flip_sign": flip_sign})


def clip(max_delta: float) -> GradientTransformation:
  return GradientTransformation(lambda p: {}, lambda u, s, p=None: (
      {k: v.clamp(-max_delta, max_delta) for k, v in u.items()}, s), "clip")


def clip_by_global_norm(max_norm: float) -> GradientTransformation:
  def update(updates, state, params=None):
    if not updates:
      return updates, state
    g = torch.sqrt(sum((v.float() ** 2).sum() for v in updates.values()))
    factor = torch.clamp(max_norm / (g + 1e-16), max=1.0)
    # optax: scale only when g >= max_norm, i.e. factor = min(1, max_norm/g)
    return {k: v * factor for k, v in updates.items()}, state

  return GradientTransformation(lambda p: {}, update, "clip_by_global_norm",
                                {"max_norm": max_norm})


def trace(decay: float, nesterov: bool = False) -> GradientTransformation:
  def init(params):
    return {"trace": _zeros_like_tree(params)}

  def update(updates, state, params=None):
    new_trace = {k: updates[k] + decay * state["trace"][k] for k in updates}
    out = ({k: updates[k] + decay * new_trace[k] for k in updates} if nesterov else new_trace)
    return out, {"trace": new_trace}

  return GradientTransformation(init, update, "trace")


def scale_by_adam(b1=0.9, b2=0.999, eps=1e-8, eps_root=0.0) -> GradientTransformation:
  def init(params):
    return {"count": torch.zeros((), dtype=torch.int32), "mu": _zeros_like_tree(params),
            "nu": _zeros_like_tree(params)}

  def update(updates, state, params=None):
    count = state["count"] + 1
    c = int(count)
    mu = {k: b1 * state["mu"][k] + (1 - b1) * g for k, g in updates.items()}
    nu = {k: b2 * state["nu"][k] + (1 - b2) * g * g for k, g in updates.items()}
    bc1, bc2 = 1 - b1 ** c, 1 - b2 ** c
    out = {k: (mu[k] / bc1) / (torch.sqrt(nu[k] / bc2 + eps_root) + eps) for k in updates}
    return out, {"count": count, "mu": mu, "nu": nu}

  return GradientTransformation(init, update, "scale_by_adam",
                                {"b1": b1, "b2": b2, "eps": eps, "eps_root": eps_root})


def scale_by_belief(b1=0.9, b2=0.999, eps=1e-16, eps_root=1e-16) -> GradientTransformation:
  def init(params):
    return {"count": torch.zeros((), dtype=torch.int32), "mu": _zeros_like_tree(params),
            "nu": _zeros_like_tree(params)}

  def update(updates, state, params=None):
    count = state["count"] + 1
    c = int(count)
    mu = {k: b1 * state["mu"][k] + (1 - b1) * g for k, g in updates.items()}
    nu = {k: b2 * state["nu"][k] + (1 - b2) * (g - mu[k]) ** 2 + eps_root
          for k, g in updates.items()}
    bc1, bc2 = 1 - b1 ** c, 1 - b2 ** c
    out = {k: (mu[k] / bc1) / (torch.sqrt(nu[k] / bc2) + eps) for k in updates}
    return out, {"count": count, "mu": mu, "nu": nu}

  return GradientTransformation(init, update, "scale_by_belief")


def scale_by_yogi(b1=0.9, b2=0.999, eps=1e-3, initial_accumulator_value=1e-6):
  def init(params):
    return {"count": torch.zeros((), dtype=torch.int32), "mu": _zeros_like_tree(params),
            "nu": {k: torch.full_like(v, initial_accumulator_value, dtype=torch.float32)
                   for k, v in params.items()}}

  def update(updates, state, params=None):
    count = state["count"] + 1
    c = int(count)
    mu = {k: b1 * state["mu"][k] + (1 - b1) * g for k, g in updates.items()}
    nu = {k: state["nu"][k] - (1 - b2) * torch.sign(state["nu"][k] - g * g) * g * g
          for k, g in updates.items()}
    bc1, bc2 = 1 - b1 ** c, 1 - b2 ** c
    out = {k: (mu[k] / bc1) / (torch.sqrt(nu[k] / bc2) + eps) for k in updates}
    return out, {"count": count, "mu": mu, "nu": nu}

  return GradientTransformation(init, update, "scale_by_yogi")


def scale_by_radam(b1=0.9, b2=0.999, eps=1e-8, threshold=5.0):
  ro_inf = 2.0 / (1 - b2) - 1

  def init(params):
    return {"count": torch.zeros((), dtype=torch.int32), "mu": _zeros_like_tree(params),
            "nu": _zeros_like_tree(params)}

  def update(updates, state, params=None):
    count = state["count"] + 1
    c = int(count)
    mu = {k: b1 * state["mu"][k] + (1 - b1) * g for k, g in updates.items()}
    nu = {k: b2 * state["nu"][k] + (1 - b2) * g * g for k, g in updates.items()}
    bc1, bc2 = 1 - b1 ** c, 1 - b2 ** c
    b2t = b2 ** c
    ro = ro_inf - 2 * c * b2t / (1 - b2t)
    if ro >= threshold:
      r = math.sqrt((ro - 4) * (ro - 2) * ro_inf / ((ro_inf - 4) * (ro_inf - 2) * ro))
      out = {k: r * (mu[k] / bc1) / (torch.sqrt(nu[k] / bc2) + eps) for k in updates}
    else:
      out = {k: mu[k] / bc1 for k in updates}
    return out, {"count": count, "mu": mu, "nu": nu}

  return GradientTransformation(init, update, "scale_by_radam")


def scale_by_rms(decay=0.9, eps=1e-8, initial_scale=0.0):
  def init(params):
    return {"nu": {k: torch.full_like(v, initial_scale, dtype=torch.float32)
                   for k, v in params.items()}}

  def update(updates, state, params=None):
    nu = {k: decay * state["nu"][k] + (1 - decay) * g * g for k, g in updates.items()}
    return {k: g / (torch.sqrt(nu[k]) + eps) for k, g in updates.items()}, {"nu": nu}

  return GradientTransformation(init, update, "scale_by_rms")


def scale_by_rss(initial_accumulator_value=0.1, eps=1e-7):
  def init(params):
    return {"sum_of_squares": {k: torch.full_like(v, initial_accumulator_value,
                                                  dtype=torch.float32)
                               for k, v in params.items()}}

  def update(updates, state, params=None):
    ss = {k: state["sum_of_squares"][k] + g * g for k, g in updates.items()}
    out = {k: torch.where(ss[k] > 0, g / torch.sqrt(ss[k] + eps), torch.zeros_like(g))
           for k, g in updates.items()}
    return out, {"sum_of_squares": ss}

  return GradientTransformation(init, update, "scale_by_rss")


def scale_by_lion(b1=0.9, b2=0.99):
  def init(params):
    return {"count": torch.zeros((), dtype=torch.int32), "mu": _zeros_like_tree(params)}

  def update(updates, state, params=None):
    out = {k: torch.sign(b1 * state["mu"][k] + (1 - b1) * g) for k, g in updates.items()}
    mu = {k: b2 * state["mu"][k] + (1 - b2) * g for k, g in updates.items()}
    return out, {"count": state["count"] + 1, "mu": mu}

  return GradientTransformation(init, update, "scale_by_lion")


def add_decayed_weights(weight_decay: float, mask=None):
  """`mask`: None (decay everything), a tree of booleans shaped like the parameters, or a
  callable that maps the parameter tree to such a tree; only entries that are true decay."""
  def selected(params):
    if mask is None:
      return None
    m = mask(tree_utils.unflatten_dict(dict(params))) if callable(mask) else mask
    flat = tree_utils.flatten_dict(m) if isinstance(m, Mapping) else m
    return {k: bool(v) for k, v in flat.items()}

  def update(updates, state, params=None):
    if params is None:
      raise ValueError("add_decayed_weights needs params")
    keep = selected(params)
    return {k: (g + weight_decay * params[k].float()) if keep is None or keep.get(k, False) else g
            for k, g in updates.items()}, state

  return GradientTransformation(lambda p: {}, update, "add_decayed_weights",
                                {"weight_decay": weight_decay, "mask": mask})


def scale_by_trust_ratio(min_norm=0.0, trust_coefficient=1.0, eps=0.0):
  def update(updates, state, params=None):
    out = {}
    for k, g in updates.items():
      pn = torch.clamp(params[k].float().norm(), min=min_norm)
      un = torch.clamp(g.norm(), min=min_norm)
      ratio = trust_coefficient * pn / (un + eps)
      ratio = torch.where((pn == 0) | (un == 0), torch.ones_like(ratio), ratio)
      out[k] = g * ratio
    return out, state

  return GradientTransformation(lambda p: {}, update, "scale_by_trust_ratio")


def add_noise(eta: float, gamma: float, seed: int):
  def init(params):
    return {"count": torch.zeros((), dtype=torch.int32)}

  def update(updates, state, params=None):
    count = state["count"] + 1
    gen = torch.Generator().manual_seed(seed + int(count))
    var = eta / (int(count) ** gamma)
    out = {k: g + math.sqrt(var) * torch.randn(g.shape, generator=gen).to(g.device)
           for k, g in updates.items()}
    return out, {"count": count}

  return GradientTransformation(init, update, "add_noise")


def chain_transforms(*transforms: GradientTransformation) -> GradientTransformation:
  def init(params):
    return {str(i): t.init(params) for i, t in enumerate(transforms)}

  def update(updates, state, params=None):
    new_state = {}
    for i, t in enumerate(transforms):
      updates, new_state[str(i)] = t.update(updates, state[str(i)], params)
    return updates, new_state

  return GradientTransformation(init, update, "chain", {"transforms": list(transforms)})


# --- aliases with optax's signatures ------------------------------------------------------
def _sgd(learning_rate, momentum=None, nesterov=False):
  parts = [trace(momentum, nesterov)] if momentum is not None else []
  return chain_transforms(*parts, scale_by_learning_rate(learning_rate))


def _adam(learning_rate, b1=0.9, b2=0.999, eps=1e-8, eps_root=0.0):
  return chain_transforms(scale_by_adam(b1, b2, eps, eps_root),
                          scale_by_learning_rate(learning_rate))


def _adamw(learning_rate, b1=0.9, b2=0.999, eps=1e-8, eps_root=0.0, weight_decay=1e-4,
           mask=None):
  return chain_transforms(scale_by_adam(b1, b2, eps, eps_root),
                          add_decayed_weights(weight_decay, mask),
                          scale_by_learning_rate(learning_rate))


def _lion(learning_rate, b1=0.9, b2=0.99, weight_decay=1e-3, mask=None):
  return chain_transforms(scale_by_lion(b1, b2), add_decayed_weights(weight_decay, mask),
                          scale_by_learning_rate(learning_rate))


def _lamb(learning_rate, b1=0.9, b2=0.999, eps=1e-6, eps_root=0.0, weight_decay=0.0, mask=None):
  return chain_transforms(scale_by_adam(b1, b2, eps, eps_root),
                          add_decayed_weights(weight_decay, mask), scale_by_trust_ratio(),
                          scale_by_learning_rate(learning_rate))


def _lars(learning_rate, weight_decay=0.0, trust_coefficient=0.001, eps=0.0, momentum=0.9,
          nesterov=False):
  return chain_transforms(add_decayed_weights(weight_decay),
                          scale_by_trust_ratio(trust_coefficient=trust_coefficient, eps=eps),
                          scale_by_learning_rate(learning_rate), trace(momentum, nesterov))


def _adagrad(learning_rate, initial_accumulator_value=0.1, eps=1e-7):
  return chain_transforms(scale_by_rss(initial_accumulator_value, eps),
                          scale_by_learning_rate(learning_rate))


def _adabelief(learning_rate, b1=0.9, b2=0.999, eps=1e-16, eps_root=1e-16):
  return chain_transforms(scale_by_belief(b1, b2, eps, eps_root),
                          scale_by_learning_rate(learning_rate))


def _radam(learning_rate, b1=0.9, b2=0.999, eps=1e-8, threshold=5.0):
  return chain_transforms(scale_by_radam(b1, b2, eps, threshold),
                          scale_by_learning_rate(learning_rate))


def _rmsprop(learning_rate, decay=0.9, eps=1e-8, initial_scale=0.0, momentum=None,
             nesterov=False):
  parts = [scale_by_rms(decay, eps, initial_scale), scale_by_learning_rate(learning_rate)]
  if momentum is not None:
    parts.append(trace(momentum, nesterov))
  return chain_transforms(*parts)


def _yogi(learning_rate, b1=0.9, b2=0.999, eps=1e-3):
  return chain_transforms(scale_by_yogi(b1, b2, eps), scale_by_learning_rate(learning_rate))


def _noisy_sgd(learning_rate, eta=0.01, gamma=0.55, seed=0):
  return chain_transforms(add_noise(eta, gamma, seed), scale_by_learning_rate(learning_rate))


def _fromage(learning_rate, min_norm=1e-6):
  mult = 1.0 / math.sqrt(1.0 + learning_rate ** 2)
  def shrink(updates, state, params=None):
    return {k: g + (mult - 1.0) * params[k].float() / 1.0 for k, g in updates.items()}, state
  return chain_transforms(scale_by_trust_ratio(min_norm), scale(-learning_rate * mult),
                          GradientTransformation(lambda p: {}, shrink, "fromage_shrink"))


# ----------------------------------------------------------------------------
# OptaxWrapper
# ----------------------------------------------------------------------------
class OptaxWrapper(OptimizerDef):
  """Wraps a GradientTransformation as an OptimizerDef (t5x/optimizers.py:377-523)."""

  def __init__(self, optax_optimizer: GradientTransformation):
    self.optax_optimizer = optax_optimizer
    self.fused_plan = _fused_adamw_plan(optax_optimizer)
    super().__init__(hyper_params=None)

  def init_state(self, params):
    flat = tree_utils.flatten_dict(params)
    state = self.optax_optimizer.init(flat)
    return OptimizerState(step=torch.zeros((), dtype=torch.int32),
                          param_states=self._nest(state))

  @staticmethod
  def _nest(state):
    """Per-parameter flat dicts inside the transform state become nested trees."""
    def conv(node):
      if isinstance(node, dict):
        if node and all(isinstance(v, torch.Tensor) for v in node.values()) and any(
            "/" in k for k in node):
          return tree_utils.unflatten_dict(node)
        return {k: conv(v) for k, v in node.items()}
      return node
    return conv(state)

  @staticmethod
  def _flat(state, param_keys):
    keyset = set(param_keys)
    def conv(node):
      if isinstance(node, dict):
        fl = tree_utils.flatten_dict(node)
        if fl and set(fl.keys()) == keyset:
          return fl
        return {k: conv(v) for k, v in node.items()}
      return node
    return conv(state)

  def update_hyper_params(self, **hyper_param_overrides):
    """The wrapped transformation owns its hyper-parameters (a learning rate given at
    construction, possibly a schedule, wins); only a `learning_rate` override is kept, for
    transformations that were built with `learning_rate=None` (t5x/optimizers.py:493-500)."""
    return {"learning_rate": hyper_param_overrides.get("learning_rate")}

  def apply_gradient(self, hyper_params, params, state, grads):
    flat_p = tree_utils.flatten_dict(params)
    if self.fused_plan is not None and _fused_adamw_usable(flat_p, grads):
      return self._apply_fused_adamw(hyper_params, params, state, grads)
    flat_g = {k: v.float() for k, v in tree_utils.flatten_dict(grads).items()}
    opt_state = self._flat(state.param_states, flat_p.keys())
    _STEP_LEARNING_RATE[0] = (hyper_params or {}).get("learning_rate")
    with torch.no_grad():
      try:
        updates, new_opt_state = self.optax_optimizer.update(
            flat_g, opt_state, {k: v.detach() for k, v in flat_p.items()})
      finally:
        _STEP_LEARNING_RATE[0] = None
      for k, p in flat_p.items():
        p.add_(updates[k].to(p.dtype))
        bf = getattr(p, "bf16", None)
        if bf is not None:
          bf.copy_(p)
    return params, OptimizerState(step=state.step + 1, param_states=self._nest(new_opt_state))

  def _apply_fused_adamw(self, hyper_params, params, state, grads):
    """[clip_by_global_norm ->] scale_by_adam [-> add_decayed_weights] -> scale_by_learning_rate
    as one native kernel per parameter (csrc/adamw.cu), with the same state layout as the
    generic path. With the optimizer sharded over the data axis (`parallel/zero.py`) the owner
    of a parameter first sums the replicas' gradients over NVLink, the clip factor is taken
    from the norm of the summed gradients of all owners, and the update kernel stores the new
    bf16 weights into every replica's working copy."""
    from t5x_b200.ops import comm, native
    from t5x_b200.parallel import state as pstate
    plan = self.fused_plan
    flat_p = tree_utils.flatten_dict(params)
    flat_g = tree_utils.flatten_dict(grads)
    opt_state = self._flat(state.param_states, flat_p.keys())
    def at(path):
      node = opt_state
      for i in path:
        node = node[str(i)]
      return node

    adam_state, lr_state = at(plan["adam_path"]), at(plan["lr_path"])
    _STEP_LEARNING_RATE[0] = (hyper_params or {}).get("learning_rate")
    try:
      lr = float(_lr(plan["learning_rate"], int(lr_state["count"])))
    finally:
      _STEP_LEARNING_RATE[0] = None
    step = int(adam_state["count"]) + 1
    st = pstate.get()
    with torch.no_grad():
      mine, replicated = [], []
      for k, p in flat_p.items():
        z = getattr(p, "zero", None)
        if z is None:
          replicated.append(k)
        elif z.mine:
          comm.peer_reduce_f32_(flat_g[k], z.grad_ptrs(), z.numel)
          mine.append(k)
      clip_scale = None
      if plan["max_norm"] is not None:
        def sumsq(keys):
          if not keys:
            return torch.zeros((), dtype=torch.float32, device=st.device)
          norms = torch._foreach_norm([flat_g[k] for k in keys])
          return torch.stack(norms).float().pow(2).sum()
        total = sumsq(mine)
        if any(getattr(p, "zero", None) is not None for p in flat_p.values()):
          import torch.distributed as dist
          dist.all_reduce(total, group=st.data_group)
        total = total + sumsq(replicated)
        gnorm = torch.sqrt(total)
        clip_scale = torch.clamp(plan["max_norm"] / (gnorm + 1e-16), max=1.0).float().reshape(1)
      for k in mine + replicated:
        p, g = flat_p[k], flat_g[k]
        z = getattr(p, "zero", None)
        bf = getattr(p, "bf16", None)
        if z is not None:
          outs, mc = z.bf16_ptrs(), z.bf16_mc()
        elif bf is not None:
          outs, mc = comm._ptr_array([bf.data_ptr()]), 0
        else:
          outs, mc = comm._ptr_array([]), 0
        native.adamw_step_(p, g, adam_state["mu"][k], adam_state["nu"][k], outs, mc, lr=lr,
                           b1=plan["b1"], b2=plan["b2"], eps=plan["eps"],
                           eps_root=plan["eps_root"], weight_decay=plan["weight_decay"],
                           step=step, clip_scale=clip_scale)
    adam_state["count"] = adam_state["count"] + 1
    lr_state["count"] = lr_state["count"] + 1
    return params, OptimizerState(step=state.step + 1, param_states=self._nest(opt_state))

  def derive_logical_axes(self, optimizer, param_logical_axes):
    """Per-parameter moments inherit the parameter's axes; counters are replicated."""
    flat_axes = tree_utils.flatten_dict(param_logical_axes, is_leaf=lambda x: not isinstance(x, dict))
    keyset = set(flat_axes.keys())

    def conv(node):
      if isinstance(node, dict):
        fl = tree_utils.flatten_dict(node)
        if fl and set(fl.keys()) == keyset:
          return tree_utils.unflatten_dict({k: flat_axes[k] for k in fl})
        return {k: conv(v) for k, v in node.items()}
      return None

    state_axes = OptimizerState(step=None, param_states=conv(optimizer.state.param_states))
    return Optimizer(optimizer.optimizer_def, state_axes, param_logical_axes)


def _fused_adamw_plan(t: GradientTransformation):
  """The hyper-parameters of an Adam / AdamW chain that the native kernel covers, or None:
  [clip_by_global_norm,] scale_by_adam, [add_decayed_weights without a mask,]
  scale_by_learning_rate (descending), possibly nested one level (`chain([clip, adamw(...)])`)."""
  def flatten(x):
    if x.name == "chain":
      out = []
      for sub in x.hparams.get("transforms", []):
        out.extend(flatten(sub))
      return out
    return [x]

  def index_paths(x, prefix=()):
    if x.name == "chain":
      out = []
      for i, sub in enumerate(x.hparams.get("transforms", [])):
        out.extend(index_paths(sub, prefix + (i,)))
      return out
    return [prefix]

  if t.name != "chain":
    return None
  parts, paths = flatten(t), index_paths(t)
  names = [x.name for x in parts]
  want = [n for n in names if n != "clip_by_global_norm"]
  if want not in (["scale_by_adam", "scale_by_schedule"],
                  ["scale_by_adam", "add_decayed_weights", "scale_by_schedule"]):
    return None
  if names.count("clip_by_global_norm") > 1 or \
      ("clip_by_global_norm" in names and names[0] != "clip_by_global_norm"):
    return None
  by = {x.name: x for x in parts}
  wd = by.get("add_decayed_weights")
  if wd is not None and wd.hparams.get("mask") is not None:
    return None
  if not by["scale_by_schedule"].hparams.get("flip_sign", True):
    return None
  adam = by["scale_by_adam"].hparams
  return {"adam_path": paths[names.index("scale_by_adam")],
          "lr_path": paths[names.index("scale_by_schedule")],
          "learning_rate": by["scale_by_schedule"].hparams["learning_rate"],
          "b1": adam["b1"], "b2": adam["b2"], "eps": adam["eps"], "eps_root": adam["eps_root"],
          "weight_decay": wd.hparams["weight_decay"] if wd is not None else 0.0,
          "max_norm": by["clip_by_global_norm"].hparams["max_norm"]
          if "clip_by_global_norm" in by else None}


def _fused_adamw_usable(flat_p, grads) -> bool:
  flat_g = tree_utils.flatten_dict(grads)
  for k, p in flat_p.items():
    g = flat_g.get(k)
    if not (isinstance(p, torch.Tensor) and p.is_cuda and p.dtype == torch.float32 and
            isinstance(g, torch.Tensor) and g.is_cuda and g.dtype == torch.float32 and
            g.is_contiguous()):
      return False
    z = getattr(p, "zero", None)
    if (z is None or z.mine) and not p.is_contiguous():
      return False
  return True


def wrap_optax_optimizer(optax_optimizer_fn):
  """Makes `fn(*args) -> OptaxWrapper(fn(*args))` (t5x/optimizers.py:529-546)."""
  def wrapped(*args, **kwargs) -> OptimizerDef:
    return OptaxWrapper(optax_optimizer_fn(*args, **kwargs))
  wrapped.__name__ = getattr(optax_optimizer_fn, "__name__", "optimizer").lstrip("_")
  return wrapped


def chain(transformations: Sequence[GradientTransformation]) -> OptimizerDef:
  return OptaxWrapper(chain_transforms(*transformations))


adabelief = wrap_optax_optimizer(_adabelief)
adagrad = wrap_optax_optimizer(_adagrad)
adam = wrap_optax_optimizer(_adam)
adamw = wrap_optax_optimizer(_adamw)
fromage = wrap_optax_optimizer(_fromage)
lamb = wrap_optax_optimizer(_lamb)
lars = wrap_optax_optimizer(_lars)
lion = wrap_optax_optimizer(_lion)
noisy_sgd = wrap_optax_optimizer(_noisy_sgd)
radam = wrap_optax_optimizer(_radam)
rmsprop = wrap_optax_optimizer(_rmsprop)
sgd = wrap_optax_optimizer(_sgd)
yogi = wrap_optax_optimizer(_yogi)


def warmup_cosine_decay_schedule(init_value, peak_value, warmup_steps, decay_steps,
                                 end_value=0.0):
  def schedule(count):
    if count < warmup_steps:
      return init_value + (peak_value - init_value) * count / max(1, warmup_steps)
    t = min(1.0, (count - warmup_steps) / max(1, decay_steps - warmup_steps))
    return end_value + 0.5 * (peak_value - end_value) * (1 + math.cos(math.pi * t))
  return schedule


# ----------------------------------------------------------------------------
# MultiOptimizer
# ----------------------------------------------------------------------------
class ModelParamTraversal:
  """Selects parameters whose '/'-joined path passes `filter_fn(path, value)`."""

  def __init__(self, filter_fn: Callable[[str, Any], bool]):
    self._filter_fn = filter_fn

  def keys(self, flat_params: Mapping[str, Any]):
    return [k for k, v in flat_params.items() if self._filter_fn("/" + k, v)]


class MultiOptimizer(OptimizerDef):
  """Different optimizers for disjoint parameter subsets (t5x/optimizers.py:634-791).
  Parameters matched by no traversal are left untouched (frozen)."""

  def __init__(self, traversals_and_optimizers: Sequence[Tuple[ModelParamTraversal, OptimizerDef]]):
    self.traversals, self.sub_optimizers = zip(*traversals_and_optimizers)
    super().__init__(hyper_params=[o.hyper_params for o in self.sub_optimizers])

  def _subsets(self, flat):
    seen = set()
    out = []
    for t in self.traversals:
      ks = t.keys(flat)
      dup = seen.intersection(ks)
      if dup:
        raise ValueError(f"Multiple optimizers match the same leaves: {sorted(dup)}")
      seen.update(ks)
      out.append(ks)
    return out

  def init_state(self, params):
    flat = tree_utils.flatten_dict(params)
    param_states = {k: None for k in flat}
    for ks, opt in zip(self._subsets(flat), self.sub_optimizers):
      sub = opt.init_state(tree_utils.unflatten_dict({k: flat[k] for k in ks}))
      sub_flat = tree_utils.flatten_dict(sub.param_states, is_leaf=lambda x: _is_param_state(x))
      for k in ks:
        param_states[k] = sub_flat.get(k)
    return OptimizerState(step=torch.zeros((), dtype=torch.int32),
                          param_states=tree_utils.unflatten_dict(param_states))

  def apply_gradient(self, hyper_params, params, state, grads):
    flat_p = tree_utils.flatten_dict(params)
    flat_g = tree_utils.flatten_dict(grads)
    flat_s = tree_utils.flatten_dict(state.param_states, is_leaf=lambda x: _is_param_state(x))
    new_s = dict(flat_s)
    for ks, opt, hp in zip(self._subsets(flat_p), self.sub_optimizers, hyper_params):
      if not ks:
        continue
      sub_p = tree_utils.unflatten_dict({k: flat_p[k] for k in ks})
      sub_g = tree_utils.unflatten_dict({k: flat_g[k] for k in ks})
      sub_state = OptimizerState(step=state.step, param_states=tree_utils.unflatten_dict(
          {k: flat_s[k] for k in ks}))
      _, ns = opt.apply_gradient(hp, sub_p, sub_state, sub_g)
      nf = tree_utils.flatten_dict(ns.param_states, is_leaf=lambda x: _is_param_state(x))
      for k in ks:
        new_s[k] = nf[k]
    return params, OptimizerState(step=state.step + 1,
                                  param_states=tree_utils.unflatten_dict(new_s))

  def update_hyper_params(self, **hyper_param_overrides):
    hps = hyper_param_overrides.pop("hyper_params", self.hyper_params)
    if hyper_param_overrides:
      hps = [dataclasses.replace(hp, **hyper_param_overrides) if hp is not None else None
             for hp in hps]
    return hps

  def set_param_axes(self, param_logical_axes):
    for opt in self.sub_optimizers:
      opt.set_param_axes(param_logical_axes)


def _is_param_state(x) -> bool:
  return x is None or not isinstance(x, Mapping) or (
      isinstance(x, Mapping) and set(x.keys()) <= {"v_row", "v_col", "v", "m"} and len(x) > 0)
