"""Adafactor with T5X semantics (API of t5x/adafactor.py).

Factored second moments with per-axis `FactorDim` rules derived from logical axis names,
the rank<=2 heuristic fallback, `(1,)` placeholders for unused state slots, RMS update
clipping, parameter-scale multiplication, optional momentum / weight decay / global-norm
clipping / NaN skipping.

Parameters are updated in place. On CUDA, 2-D (and leading-batch-dim) fp32 parameters go
through the fused kernels in `csrc/adafactor.cu`, which also write the bf16 working copy;
when the parameter is a tensor-parallel shard the partial row/column sums and RMS scalars
are summed over the `model` axis between kernel phases, so a sharded run takes the same
update as an unsharded one. Everything else runs the PyTorch statement of the same math.
"""
from __future__ import annotations

import dataclasses
import enum
import re
from typing import Any, Mapping, Optional, Sequence, Tuple, Union

import numpy as np
import torch
import torch.distributed as dist

from t5x_b200.optimizers import OptimizerDef, OptimizerState
from t5x_b200.parallel import state as pstate
from t5x_b200.utils import tree as tree_utils


class FactorDim(enum.Enum):
  NONE = None      # do not factorize this dimension
  BATCH = 1        # batch-like dimension that is never averaged over
  ROW = 2
  COLUMN = 3


class HeuristicRule(enum.Enum):
  token = 1


HEURISTIC_RULE = HeuristicRule.token
FactorRule = Union[HeuristicRule, Tuple[FactorDim, ...]]


def standard_logical_factor_rules():
  """Logical axis name -> FactorDim (t5x/adafactor.py:104-122)."""
  return {
      "vocab": FactorDim.COLUMN,
      "embed": FactorDim.ROW,
      "mlp": FactorDim.COLUMN,
      "heads": FactorDim.COLUMN,
      "kv": FactorDim.COLUMN,
      "joined_kv": FactorDim.COLUMN,
      "relpos_buckets": FactorDim.NONE,
      "layers": FactorDim.BATCH,
      "stack": FactorDim.BATCH,
      "q_wi_fused": FactorDim.COLUMN,
      "o_wo_fused": FactorDim.COLUMN,
      "multiquery_heads": FactorDim.COLUMN,
      "kv_fused": FactorDim.COLUMN,
      "layer_norm_scale": FactorDim.NONE,
      "mlp_activations": FactorDim.COLUMN,
  }


def factor_name_to_factordim(name):
  if not isinstance(name, str):
    return name
  return {
      "row": FactorDim.ROW, "col": FactorDim.COLUMN, "column": FactorDim.COLUMN,
      "batch": FactorDim.BATCH, "none": FactorDim.NONE, "unfactorized": FactorDim.NONE,
  }[name.lower()]


class HParamMap:
  """Maps '/'-joined parameter paths to hyper-parameters by first matching regex."""

  def __init__(self, rules):
    self._rules = [(re.compile(r), p) for r, p in rules]

  def __getitem__(self, key: str) -> Any:
    for r, p in self._rules:
      if r.search(key):
        return p
    raise KeyError(f"No factor rule found for parameter: {key}")

  def __call__(self, params):
    flat = tree_utils.flatten_dict(params)
    return tree_utils.unflatten_dict({k: self[k] for k in flat})


@dataclasses.dataclass
class _AdafactorHyperParams:
  learning_rate: Optional[float]
  factored: bool
  multiply_by_parameter_scale: Union[bool, HParamMap]
  beta1: Optional[float]
  decay_rate: float
  step_offset: int
  clipping_threshold: Optional[float]
  weight_decay_rate: Optional[float]
  min_dim_size_to_factor: int
  epsilon1: float
  epsilon2: float
  factor_map: Optional[Any] = None
  logical_factor_rules: Any = None
  weight_decay_rate_lr_exponent: Optional[float] = None
  global_norm_clip_threshold: Optional[float] = None
  max_parameter_scale: Optional[float] = None
  skip_nan_updates: Optional[bool] = False

  def replace(self, **kw):
    return dataclasses.replace(self, **kw)


_STATE_KEYS = ("v_row", "v_col", "v", "m")


def _placeholder(device):
  return torch.zeros((1,), dtype=torch.float32, device=device)


class Adafactor(OptimizerDef):
  """Adafactor (https://arxiv.org/abs/1804.04235), T5X flavour (t5x/adafactor.py:193-683)."""

  def __init__(self, learning_rate: Optional[float] = None, factored: bool = True,
               multiply_by_parameter_scale: Union[bool, HParamMap] = True,
               beta1: Optional[float] = None, decay_rate: float = 0.8, step_offset: int = 0,
               clipping_threshold: Optional[float] = 1.0,
               weight_decay_rate: Optional[float] = None, min_dim_size_to_factor: int = 128,
               epsilon1: float = 1e-30, epsilon2: float = 1e-3,
               dtype_momentum: Any = torch.float32, factor_map: Optional[HParamMap] = None,
               logical_factor_rules: Optional[Mapping[str, FactorDim]] = None,
               weight_decay_rate_lr_exponent: Optional[float] = None,
               global_norm_clip_threshold: Optional[float] = None,
               max_parameter_scale: Optional[float] = None,
               skip_nan_updates: Optional[bool] = False):
    if not factored and factor_map is not None:
      raise ValueError("Adafactor factored is False but factorization rules have been provided.")
    if not isinstance(multiply_by_parameter_scale, (bool, HParamMap)):
      raise TypeError("`multiply_by_parameter_scale` must be either bool or `HParamMap` type.")
    if logical_factor_rules is not None and factor_map is not None:
      raise ValueError("Adafactor received both logical_factor_rules and factor_map.")
    if isinstance(dtype_momentum, str):
      dtype_momentum = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype_momentum]
    self.dtype_momentum = dtype_momentum
    super().__init__(_AdafactorHyperParams(
        learning_rate, factored, multiply_by_parameter_scale, beta1, decay_rate, step_offset,
        clipping_threshold, weight_decay_rate, min_dim_size_to_factor, epsilon1, epsilon2,
        factor_map, logical_factor_rules, weight_decay_rate_lr_exponent,
        global_norm_clip_threshold, max_parameter_scale, skip_nan_updates))

  # ---- rule handling ---------------------------------------------------------------------
  @staticmethod
  def _decay_rate_pow(i: int, exponent: float = 0.8) -> float:
    return 1.0 - float(i + 1.0) ** (-exponent)

  @staticmethod
  def _parse_rule(rule, shape, path, fallback_to_heuristics=True):
    """-> (dims to average over, factored dims | HEURISTIC_RULE | None)
    (t5x/adafactor.py:318-395)."""
    nd = len(shape)
    if rule is None:
      return tuple(range(nd)), None
    if rule is HEURISTIC_RULE:
      if nd > 2:
        raise ValueError("A parameter with rank strictly higher than 2 must have an explicit "
                         f"factorization rule: {path}, {tuple(shape)}")
      return tuple(range(nd)), HEURISTIC_RULE
    if len(rule) != nd:
      raise ValueError(f"Factorization rule {rule} has incorrect rank for param of rank {nd}: "
                       f"{path}, {tuple(shape)}")
    row_dims = tuple(i for i, d in enumerate(rule) if d == FactorDim.ROW)
    col_dims = tuple(i for i, d in enumerate(rule) if d == FactorDim.COLUMN)
    batched = tuple(i for i, d in enumerate(rule) if d == FactorDim.BATCH)
    averaging = tuple(i for i in range(nd) if i not in batched)
    factor_dims = (row_dims, col_dims)
    if factor_dims == ((), ()):
      factor_dims = None
    if fallback_to_heuristics and nd <= 2 and not batched:
      return tuple(range(nd)), HEURISTIC_RULE
    return averaging, factor_dims

  def _factored_dims(self, shape):
    """Heuristic: factor over the two largest dims if both >= min_dim_size_to_factor."""
    if not self.hyper_params.factored or len(shape) < 2:
      return None
    sorted_dims = np.argsort(np.asarray(shape), kind="stable")
    if shape[sorted_dims[-2]] < self.hyper_params.min_dim_size_to_factor:
      return None
    return (int(sorted_dims[-2]),), (int(sorted_dims[-1]),)

  def _rule_for(self, path):
    if not self.hyper_params.factored:
      return None
    fm = self.hyper_params.factor_map
    return fm[path] if fm else HEURISTIC_RULE

  def _resolve(self, shape, path):
    averaging, factored = self._parse_rule(self._rule_for(path), shape, path)
    if factored is HEURISTIC_RULE:
      factored = self._factored_dims(shape)
    return averaging, factored

  @staticmethod
  def _global_shape(param):
    return tuple(getattr(param, "global_shape", None) or param.shape)

  # ---- state -----------------------------------------------------------------------------
  def init_param_state(self, param, path):
    shape = self._global_shape(param)
    local = tuple(param.shape)
    dev = param.device
    state = {k: _placeholder(dev) for k in _STATE_KEYS}
    _, factored = self._resolve(shape, path)
    if factored is not None:
      d1, d0 = factored
      state["v_row"] = torch.zeros(tuple(np.delete(local, d0)), dtype=torch.float32, device=dev)
      state["v_col"] = torch.zeros(tuple(np.delete(local, d1)), dtype=torch.float32, device=dev)
    else:
      state["v"] = torch.zeros(local, dtype=torch.float32, device=dev)
    if self.hyper_params.beta1 is not None:
      state["m"] = torch.zeros(local, dtype=self.dtype_momentum, device=dev)
    return state

  def init_state(self, params):
    flat = tree_utils.flatten_dict(params)
    states = {k: self.init_param_state(p, k) for k, p in flat.items()}
    return OptimizerState(torch.zeros((), dtype=torch.int32),
                          tree_utils.unflatten_dict(states))

  # ---- update ----------------------------------------------------------------------------
  def apply_param_gradient(self, step, hyper_params, param, state, grad, path,
                           pre_reduced: bool = False):
    """Updates `param` and `state` in place; returns them. `pre_reduced`: with the optimizer
    sharded over the data axis, `grad` already holds the sum over replicas (global-norm
    clipping needed it first), so the update only pushes the new weights."""
    hp = hyper_params
    assert hp.learning_rate is not None, "no learning rate provided."
    lr = float(hp.learning_rate)
    weight_decay_rate = hp.weight_decay_rate
    if hp.weight_decay_rate_lr_exponent:
      weight_decay_rate = (weight_decay_rate or 1.0) * lr ** hp.weight_decay_rate_lr_exponent
    gshape = self._global_shape(param)
    averaging_dims, factored_dims = self._resolve(gshape, path)
    decay = self._decay_rate_pow(int(step) - hp.step_offset, exponent=hp.decay_rate)
    mbps = hp.multiply_by_parameter_scale
    if isinstance(mbps, HParamMap):
      mbps = mbps[path]
    zinfo = getattr(param, "zero", None)
    if zinfo is not None and not pre_reduced and \
        self._fused_sharded_ok(param, state, grad, averaging_dims, factored_dims):
      # gradient reduction and weight broadcast happen inside the update kernels
      done = self._try_native(param, state, grad, path, lr, decay, bool(mbps),
                              weight_decay_rate, averaging_dims, factored_dims, zinfo=zinfo)
      assert done
      return param, state
    if zinfo is not None:
      from t5x_b200.ops import comm
      if not pre_reduced:
        comm.peer_reduce_f32_(grad, zinfo.grad_ptrs(), zinfo.numel)
    if not self._try_native(param, state, grad, path, lr, decay, bool(mbps), weight_decay_rate,
                            averaging_dims, factored_dims):
      self._apply_torch(param, state, grad, lr, decay, bool(mbps), weight_decay_rate,
                        averaging_dims, factored_dims)
    if zinfo is not None:
      comm.peer_push_bf16_(zinfo.bf16_ptrs(), param.bf16, zinfo.numel,
                           skip_rank=zinfo.push_skip_rank())
    return param, state

  def _fused_sharded_ok(self, param, state, grad, averaging_dims, factored_dims) -> bool:
    """True when the NVLink-fused kernels cover this parameter: a factored [batch, R, C]
    fp32 matrix with C % 4 == 0 that is not also tensor-parallel sharded."""
    if factored_dims is None or param.dtype != torch.float32 or not param.is_contiguous():
      return False
    st = pstate.get()
    if getattr(param, "shard_dim", None) is not None and st.model_size > 1:
      return False
    if self.hyper_params.beta1 is not None and self.dtype_momentum != torch.float32:
      return False
    nd = param.dim()
    batch_dims = tuple(i for i in range(nd) if i not in averaging_dims)
    nb = len(batch_dims)
    if batch_dims != tuple(range(nb)):
      return False
    d1, d0 = factored_dims
    rest = tuple(range(nb, nd))
    if tuple(d1) + tuple(d0) == rest:
      col_dims = d0
    elif tuple(d0) + tuple(d1) == rest:
      col_dims = d1
    else:
      return False
    return int(np.prod([param.shape[d] for d in col_dims])) % 4 == 0

  # PyTorch statement (any rank, any rule). Sharded dims are reduced over the model axis.
  def _apply_torch(self, param, state, grad, lr, decay, mbps, weight_decay_rate,
                   averaging_dims, factored_dims):
    hp = self.hyper_params if not hasattr(self, "_hp_override") else self._hp_override
    shard_dim = getattr(param, "shard_dim", None)
    st = pstate.get()
    sharded = shard_dim is not None and st.model_size > 1
    gshape = self._global_shape(param)

    def mean(x, dims, keepdim=False):
      """Mean over `dims` of the GLOBAL tensor when one of them is the sharded dim."""
      dims = tuple(dims)
      s = x.sum(dim=dims, keepdim=keepdim)
      cnt = 1
      for d in dims:
        cnt *= gshape[d]
      if sharded and shard_dim in dims:
        dist.all_reduce(s, group=st.model_group)
      return s / cnt

    with torch.no_grad():
      g = grad.float()
      p = param.data
      update_scale = lr
      if mbps:
        ps = torch.sqrt(mean(p.float() * p.float(), averaging_dims, keepdim=True))
        ps = torch.clamp(ps, min=hp.epsilon2)
        if hp.max_parameter_scale is not None:
          ps = torch.clamp(ps, max=hp.max_parameter_scale)
        update_scale = update_scale * ps
      mixing = 1.0 - decay
      gsq = g * g + hp.epsilon1
      if factored_dims is not None:
        d1, d0 = factored_dims
        new_v_row = decay * state["v_row"] + mixing * mean(gsq, d0)
        new_v_col = decay * state["v_col"] + mixing * mean(gsq, d1)
        reduced_d1 = tuple(d - len([e for e in d0 if e < d]) for d in d1)
        # mean over the d1 positions of v_row (global when d1 holds the sharded dim)
        s = new_v_row.sum(dim=reduced_d1, keepdim=True)
        cnt = 1
        for d in d1:
          cnt *= gshape[d]
        if sharded and shard_dim in d1:
          dist.all_reduce(s, group=st.model_group)
        row_col_mean = s / cnt
        row_factor = (new_v_row / row_col_mean) ** -0.5
        col_factor = new_v_col ** -0.5
        rf, cf = row_factor, col_factor
        for d in sorted(d0):
          rf = rf.unsqueeze(d)
        for d in sorted(d1):
          cf = cf.unsqueeze(d)
        y = g * rf * cf
        new_state = {"v_row": new_v_row, "v_col": new_v_col}
      else:
        new_v = decay * state["v"] + mixing * gsq
        y = g * new_v ** -0.5
        new_state = {"v": new_v}
      if hp.clipping_threshold is not None:
        denom = torch.clamp(torch.sqrt(mean(y * y, averaging_dims, keepdim=True)) /
                            hp.clipping_threshold, min=1.0)
        y = y / denom
      sub = update_scale * y
      if hp.beta1 is not None:
        new_m = hp.beta1 * state["m"].float() + (1.0 - hp.beta1) * sub
        sub = new_m
        new_state["m"] = new_m.to(self.dtype_momentum)
      if weight_decay_rate is not None:
        new_p = (1.0 - weight_decay_rate) * p - sub
      else:
        new_p = p - sub
      if hp.skip_nan_updates:
        for k in list(new_state):
          new_state[k] = torch.where(torch.isnan(new_state[k]), state[k], new_state[k])
        new_p = torch.where(torch.isnan(new_p), p, new_p)
      p.copy_(new_p.to(p.dtype))
      for k, v in new_state.items():
        state[k].copy_(v)
      bf = getattr(param, "bf16", None)
      if bf is not None:
        bf.copy_(p)
    return param, state

  # Fused CUDA path for fp32 parameters laid out [batch..., rows, cols].
  def _try_native(self, param, state, grad, path, lr, decay, mbps, weight_decay_rate,
                  averaging_dims, factored_dims, zinfo=None) -> bool:
    if not (param.is_cuda and param.dtype == torch.float32 and grad.dtype == torch.float32 and
            param.is_contiguous() and grad.is_contiguous()):
      return False
    hp = self.hyper_params
    nd = param.dim()
    batch_dims = tuple(i for i in range(nd) if i not in averaging_dims)
    if batch_dims != tuple(range(len(batch_dims))):
      return False  # batch dims must lead
    nb = len(batch_dims)
    from t5x_b200.ops import native
    st = pstate.get()
    shard_dim = getattr(param, "shard_dim", None)
    sharded = shard_dim is not None and st.model_size > 1
    gshape = self._global_shape(param)
    batch = int(np.prod(param.shape[:nb])) if nb else 1
    flags = 0
    if mbps:
      flags |= native.AF_PARAM_SCALE
    if hp.clipping_threshold is not None:
      flags |= native.AF_CLIP
    if weight_decay_rate is not None:
      flags |= native.AF_WD
    if hp.beta1 is not None:
      if self.dtype_momentum != torch.float32:
        return False
      flags |= native.AF_MOMENTUM
    if hp.max_parameter_scale is not None:
      flags |= native.AF_MAX_SCALE
    if hp.skip_nan_updates:
      flags |= native.AF_SKIP_NAN
    common = dict(lr=lr, eps2=hp.epsilon2, clip_threshold=hp.clipping_threshold or 1.0,
                  weight_decay=weight_decay_rate or 0.0, beta1=hp.beta1 or 0.0,
                  max_param_scale=hp.max_parameter_scale or 0.0, flags=flags)
    bf = getattr(param, "bf16", None)
    m = state["m"] if hp.beta1 is not None else None
    n_global = int(np.prod(gshape[nb:])) if nd > nb else 1

    if factored_dims is None:
      rows = 1 if nd - nb <= 1 else int(np.prod(param.shape[nb:-1]))
      cols = int(param.shape[-1]) if nd > nb else 1
      n_local = rows * cols
      ld_bf16, bbs = (0, 0)
      if bf is not None:
        if not bf.is_contiguous():
          return False
        ld_bf16, bbs = cols, n_local
      scratch = _scratch(param.device, 4 * batch)
      native.adafactor_unfactored_stats_(param, grad, state["v"], scratch, batch, n_local, decay,
                                         hp.epsilon1, bool(hp.skip_nan_updates))
      if sharded:
        dist.all_reduce(scratch[:4 * batch], group=st.model_group)
      native.adafactor_unfactored_apply_(param, grad, state["v"], m, bf, scratch, batch, rows,
                                         cols, n_global, ld_bf16=ld_bf16, bf16_batch_stride=bbs,
                                         **common)
      return True

    d1, d0 = factored_dims  # v_row reduces d0; v_col reduces d1
    rest = tuple(range(nb, nd))
    # The non-batch dims must split into a leading group and a trailing group that are exactly
    # (d0, d1) in one of the two orders, so the tensor is a [batch, R, C] matrix.
    if tuple(sorted(d0 + d1)) != rest:
      return False
    if tuple(d1) + tuple(d0) == rest:
      row_dims, col_dims, row_is_normalized = d1, d0, True    # v_row indexed by rows (= d1)
    elif tuple(d0) + tuple(d1) == rest:
      row_dims, col_dims, row_is_normalized = d0, d1, False   # v_row indexed by cols (= d1)
    else:
      return False
    R = int(np.prod([param.shape[d] for d in row_dims]))
    C = int(np.prod([param.shape[d] for d in col_dims]))
    gR = int(np.prod([gshape[d] for d in row_dims]))
    gC = int(np.prod([gshape[d] for d in col_dims]))
    # state vectors: the one indexed by matrix rows has the column dims removed.
    v_rvec = state["v_row"] if row_is_normalized else state["v_col"]
    v_cvec = state["v_col"] if row_is_normalized else state["v_row"]
    ld_bf16, bbs = (0, 0)
    if bf is not None:
      if bf.dim() != param.dim() or bf.stride(-1) != 1:
        return False
      if len(col_dims) != 1 or (len(row_dims) != 1) or nb > 1:
        if not bf.is_contiguous():
          return False
        ld_bf16, bbs = C, R * C
      else:
        ld_bf16 = bf.stride(-2)
        bbs = bf.stride(0) if nb == 1 else 0
    scratch = _scratch(param.device, native.adafactor_scratch_floats(batch, R, C))
    if zinfo is not None:
      from t5x_b200.ops import comm
      comm.dist_adafactor_stats_(param, zinfo.grad_ptrs(), grad, scratch, batch, R, C,
                                 hp.epsilon1, grad_mc=zinfo.grad_mc())
    else:
      native.adafactor_stats_(param, grad, scratch, batch, R, C, hp.epsilon1)
    rows_sharded = sharded and shard_dim in row_dims
    cols_sharded = sharded and shard_dim in col_dims
    o_row, o_col = 0, batch * R
    o_scal = 2 * batch * (R + C)
    if sharded:
      # Row sums run over columns: they are partial when columns are sharded (and vice versa).
      if cols_sharded:
        dist.all_reduce(scratch[o_row:o_row + batch * R], group=st.model_group)
      if rows_sharded:
        dist.all_reduce(scratch[o_col:o_col + batch * C], group=st.model_group)
      dist.all_reduce(scratch[o_scal:o_scal + 4 * batch], group=st.model_group)
    native.adafactor_ema_(v_rvec, v_cvec, scratch, batch, R, C, gR, gC, row_is_normalized, decay,
                          bool(hp.skip_nan_updates))
    if sharded:
      norm_sharded = rows_sharded if row_is_normalized else cols_sharded
      if norm_sharded:
        vs = scratch[o_scal:o_scal + 4 * batch].view(batch, 4)[:, 2].contiguous()
        dist.all_reduce(vs, group=st.model_group)
        scratch[o_scal:o_scal + 4 * batch].view(batch, 4)[:, 2] = vs
    native.adafactor_usq_(grad, v_rvec, v_cvec, scratch, batch, R, C, gR, gC, row_is_normalized,
                          hp.clipping_threshold is not None)
    if sharded and hp.clipping_threshold is not None:
      us = scratch[o_scal:o_scal + 4 * batch].view(batch, 4)[:, 1].contiguous()
      dist.all_reduce(us, group=st.model_group)
      scratch[o_scal:o_scal + 4 * batch].view(batch, 4)[:, 1] = us
    if zinfo is not None:
      comm.dist_adafactor_apply_(param, grad, m, zinfo.bf16_ptrs(), scratch, batch, R, C,
                                 n_global, bf16_mc=zinfo.bf16_mc(), **common)
    else:
      native.adafactor_apply_(param, grad, m, bf, scratch, batch, R, C, n_global,
                              ld_bf16=ld_bf16, bf16_batch_stride=bbs, **common)
    return True

  def apply_gradient(self, hyper_params, params, state, grads):
    step = state.step
    flat_p = tree_utils.flatten_dict(params)
    flat_s = tree_utils.flatten_dict(state.param_states, is_leaf=_is_state_leaf)
    flat_g = tree_utils.flatten_dict(grads)
    saved_hp = self.hyper_params
    self.hyper_params = hyper_params
    try:
      pre_reduced = False
      if hyper_params.global_norm_clip_threshold:
        # The norm is that of the gradient summed over replicas. With the optimizer sharded
        # over the data axis that sum exists on a parameter's owner only, so owners reduce
        # their gradients here (the update below then skips its own reduction) and the
        # squared norms are summed over the data axis; tensor-parallel shards are summed over
        # the model axis, replicated parameters are counted once.
        thr = hyper_params.global_norm_clip_threshold
        st = pstate.get()
        counted = []
        sums = torch.zeros(4, dtype=torch.float32, device=next(iter(flat_g.values())).device)
        for k, p in flat_p.items():
          zinfo = getattr(p, "zero", None)
          if zinfo is not None:
            if not zinfo.mine:
              continue
            from t5x_b200.ops import comm
            comm.peer_reduce_f32_(flat_g[k], zinfo.grad_ptrs(), zinfo.numel)
            pre_reduced = True
          counted.append(k)
          slot = 2 * (zinfo is not None) + (getattr(p, "shard_dim", None) is not None)
          sums[slot] += (flat_g[k].float() ** 2).sum()
        if any(getattr(p, "zero", None) is not None for p in flat_p.values()):
          pre_reduced = True
          dist.all_reduce(sums[2:], group=st.data_group)
        if st.model_size > 1:
          sharded = sums[1] + sums[3]
          dist.all_reduce(sharded, group=st.model_group)
          total = sums[0] + sums[2] + sharded
        else:
          total = sums.sum()
        gn = torch.sqrt(total)
        scale = thr * torch.minimum(torch.tensor(1.0 / thr, device=gn.device), 1.0 / gn)
        for k in counted:
          flat_g[k].mul_(scale.to(flat_g[k].dtype))
      from t5x_b200.parallel import zero
      done = zero.done_this_step()
      for k, p in flat_p.items():
        zinfo = getattr(p, "zero", None)
        if zinfo is not None and not zinfo.mine:
          continue  # its owner updates it and pushes the new bf16 weights here
        if k in done:
          continue  # already updated while the backward pass was running
        self.apply_param_gradient(step, hyper_params, p, flat_s[k], flat_g[k], k,
                                  pre_reduced=pre_reduced)
    finally:
      self.hyper_params = saved_hp
    return params, OptimizerState(step + 1, state.param_states)

  # ---- axes ------------------------------------------------------------------------------
  def set_param_axes(self, param_logical_axes):
    """Builds the factor map from logical axis names (t5x/adafactor.py:629-660)."""
    rules = self.hyper_params.logical_factor_rules
    if rules is None:
      return
    NONE, COLUMN, ROW = FactorDim.NONE, FactorDim.COLUMN, FactorDim.ROW

    def apply_rules(axes):
      axis_rules = tuple(factor_name_to_factordim(rules[x]) for x in axes)
      if ROW in axis_rules and COLUMN in axis_rules and NONE in axis_rules:
        raise ValueError(f"Incomplete adafactor spec {axis_rules} for {axes}!")
      if ROW not in axis_rules or COLUMN not in axis_rules:
        axis_rules = tuple(NONE if x in (ROW, COLUMN) else x for x in axis_rules)
      return axis_rules

    flat = tree_utils.flatten_dict(param_logical_axes,
                                   is_leaf=lambda x: not isinstance(x, Mapping))
    self.hyper_params = self.hyper_params.replace(
        factor_map={k: apply_rules(tuple(v)) for k, v in flat.items()})

  def derive_logical_axes(self, optimizer, param_logical_axes):
    """Only unfactored `v` and `m` inherit the parameter's axes (t5x/adafactor.py:662-683)."""
    from t5x_b200.optimizers import Optimizer
    flat_axes = tree_utils.flatten_dict(param_logical_axes,
                                        is_leaf=lambda x: not isinstance(x, Mapping))
    flat_states = tree_utils.flatten_dict(optimizer.state.param_states, is_leaf=_is_state_leaf)
    out = {}
    for k, axes in flat_axes.items():
      leaf = flat_states[k]
      out[k] = dict(v_row=None, v_col=None,
                    v=axes if tuple(leaf["v"].shape) != (1,) else None,
                    m=axes if self.hyper_params.beta1 else None)
    state_axes = OptimizerState(step=None, param_states=tree_utils.unflatten_dict(out))
    return Optimizer(optimizer.optimizer_def, state_axes, param_logical_axes)


def _is_state_leaf(x) -> bool:
  return not isinstance(x, Mapping) or (len(x) > 0 and set(x.keys()) <= set(_STATE_KEYS))


_SCRATCH = {}


def _scratch(device, n_floats: int) -> torch.Tensor:
  """Grow-only fp32 scratch per device for the kernel phases."""
  buf = _SCRATCH.get(device)
  if buf is None or buf.numel() < n_floats:
    buf = torch.empty(max(n_floats, 1 << 16), dtype=torch.float32, device=device)
    _SCRATCH[device] = buf
  return buf[:n_floats]
