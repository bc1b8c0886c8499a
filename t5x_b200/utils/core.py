"""Run-level utilities (API of t5x/utils.py, first half): checkpoint/dataset config
dataclasses, restore-path resolution, `TrainStateInitializer`, checkpoint-manager factories,
host barriers and broadcast helpers, `log_model_info`."""
from __future__ import annotations

import dataclasses
import functools
import logging
import os
import time
from typing import Any, Callable, Iterable, Mapping, Optional, Sequence, Tuple, Type, Union

import numpy as np
import torch
import torch.distributed as dist

from t5x_b200 import checkpoints
from t5x_b200 import partitioning
from t5x_b200 import state_utils
from t5x_b200 import train_state as train_state_lib
from t5x_b200.parallel import state as pstate
from t5x_b200.utils import tree as tree_utils

Array = Any
PartitionSpec = partitioning.PartitionSpec
DType = Any
Shape = Tuple[int, ...]


# ----------------------------------------------------------------------------
# Checkpoint configs
# ----------------------------------------------------------------------------
@dataclasses.dataclass
class SaveCheckpointConfig:
  """How and when to save checkpoints (t5x/utils.py:128-162)."""
  dtype: Optional[str] = "float32"
  period: Optional[int] = None
  checkpoint_steps: Optional[Sequence[int]] = None
  keep: Optional[int] = None
  keep_dataset_checkpoints: Optional[int] = None
  save_dataset: bool = False
  checkpointer_cls: Callable[..., Any] = checkpoints.Checkpointer
  state_transformation_fns: Sequence[Callable] = dataclasses.field(default_factory=list)
  checkpoint_manager_cls: Callable[..., Any] = checkpoints.OrbaxCheckpointManagerInterface

  def __post_init__(self):
    if self.dtype not in (None, "float32", "bfloat16"):
      raise ValueError("`SaveCheckpointConfig.dtype` must be one of None, 'float32' or "
                       f"'bfloat16'. Got {self.dtype}.")


@dataclasses.dataclass
class RestoreCheckpointConfig:
  """What to restore from (t5x/utils.py:166-225)."""
  path: Union[str, Sequence[str]]
  mode: str = "latest"
  assignment_map: Optional[Sequence[Tuple[str, Optional[str]]]] = None
  strict: bool = True
  fallback_to_scratch: bool = False
  dtype: Optional[str] = None
  restore_dataset: bool = False
  checkpointer_cls: Callable[..., Any] = checkpoints.Checkpointer
  state_transformation_fns: Sequence[Callable] = ()
  checkpoint_manager_cls: Callable[..., Any] = checkpoints.OrbaxCheckpointManagerInterface

  def __post_init__(self):
    if self.mode not in ("specific", "latest", "all"):
      raise ValueError("`RestoreCheckpointConfig.mode` must be one of 'specific', 'latest', "
                       f"or 'all'. Got {self.mode}.")
    if self.dtype not in (None, "float32", "bfloat16", "float16"):
      raise ValueError("`RestoreCheckpointConfig.dtype` must be one of `None`, 'float32', "
                       f"'float16' or 'bfloat16'. Got {self.dtype}.")
    if self.assignment_map is not None:
      fn = functools.partial(state_utils.apply_assignment_map,
                             assignment_map=self.assignment_map)
      self.state_transformation_fns = (fn, *self.state_transformation_fns)


@dataclasses.dataclass
class CheckpointConfig:
  save: Optional[SaveCheckpointConfig] = None
  restore: Optional[RestoreCheckpointConfig] = None


@dataclasses.dataclass
class DatasetConfig:
  """A dataset for train / eval / infer (t5x/utils.py:530-564)."""
  mixture_or_task_name: Union[str, Any]
  task_feature_lengths: Mapping[str, int]
  split: str
  batch_size: int
  shuffle: bool
  seed: Optional[int]
  use_cached: bool = False
  pack: bool = False
  use_custom_packing_ops: bool = False
  module: Optional[str] = None
  use_memory_cache: bool = True
  trim_output_features: bool = True
  runtime_preprocessors: Optional[Sequence[Callable]] = None
  num_prefetch_threads: Optional[int] = None
  num_workers: int = 0


# ----------------------------------------------------------------------------
# Host-level collectives (the role of jax.experimental.multihost_utils)
# ----------------------------------------------------------------------------
def _dist_on() -> bool:
  return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def sync_global_devices(name: str) -> None:
  """Barrier across all ranks (t5x/utils.py:760-769), on the host and with a timeout: see
  `parallel.state.host_barrier`."""
  pstate.host_barrier(name)


def broadcast_one_to_all(value, is_source: Optional[bool] = None):
  """Value of rank 0 on every rank."""
  if not _dist_on():
    return value
  obj = [value]
  dist.broadcast_object_list(obj, src=0)
  return obj[0]


def multihost_assert_equal(value, fail_message: str = "") -> None:
  """Raises on every rank if `value` differs between ranks."""
  if not _dist_on():
    return
  gathered = [None] * dist.get_world_size()
  dist.all_gather_object(gathered, value)
  ref = gathered[0]
  for r, g in enumerate(gathered):
    same = np.array_equal(np.asarray(g), np.asarray(ref)) if not isinstance(g, (dict, str)) \
        else g == ref
    if not same:
      raise AssertionError(f"{fail_message}: rank {r} has {g!r}, rank 0 has {ref!r}")


def get_local_data(x):
  if isinstance(x, torch.Tensor):
    return x.detach().cpu().numpy()
  return x


def set_hardware_rng_ops():
  """Kept for API parity: the CUDA Philox generators are already the fast path."""
  logging.info("Hardware RNG is the default (Philox); nothing to switch.")


# ----------------------------------------------------------------------------
# Restore-config resolution
# ----------------------------------------------------------------------------
def get_first_valid_restore_config_and_paths(restore_cfgs: Sequence[RestoreCheckpointConfig]):
  """First config that points at existing checkpoints, with the paths to restore
  (t5x/utils.py:926-977)."""
  for cfg in restore_cfgs:
    paths = [cfg.path] if isinstance(cfg.path, str) else list(cfg.path)
    if cfg.mode == "specific":
      return cfg, paths
    if cfg.mode in ("all", "latest"):
      for ckpt_dir in paths:
        if not os.path.isdir(ckpt_dir):
          raise ValueError("Checkpoint path(s) must be valid directories when using restore "
                           "mode 'all' or 'latest'.")
        ckpt_paths = [os.path.join(ckpt_dir, f"checkpoint_{s}")
                      for s in checkpoints.all_steps(ckpt_dir)]
        if not ckpt_paths:
          logging.info("No checkpoints found in specified directory: %s", ckpt_dir)
          continue
        if cfg.mode == "latest":
          ckpt_paths = ckpt_paths[-1:]
        return cfg, ckpt_paths
    else:
      logging.error("Unsupported checkpoint restore mode: %s", cfg.mode)
  return None, []


def get_fallback_state(restore_cfg, init_fn: Callable[[Any], Mapping[str, Any]], init_rng):
  """State used for leaves the checkpoint lacks (t5x/utils.py:980-1003)."""
  if restore_cfg is None:
    return None
  if restore_cfg.fallback_to_scratch:
    if not restore_cfg.state_transformation_fns:
      raise ValueError("`state_transformation_fns` must be provided with `fallback_to_scratch`")
    if init_rng is None:
      raise ValueError("An `init_rng` must be provided with `fallback_to_scratch`")
    return init_fn(init_rng)
  return None


# ----------------------------------------------------------------------------
# Train-state initialisation
# ----------------------------------------------------------------------------
class TrainStateInitializer:
  """Creates the (sharded) train state from scratch or from checkpoints
  (t5x/utils.py:1006-1202)."""

  def __init__(self, optimizer_def, init_fn: Callable[..., Mapping[str, Any]],
               input_shapes: Mapping[str, Shape], partitioner,
               input_types: Optional[Mapping[str, DType]] = None):
    self._optimizer_def = optimizer_def
    self._init_fn = init_fn
    self._input_shapes = input_shapes
    self._input_types = input_types
    self._partitioner = partitioner
    self._state = None

    def initialize_train_state(rng):
      variables = init_fn(rng, input_shapes, input_types)
      if optimizer_def:
        return train_state_lib.FlaxOptimTrainState.create(optimizer_def, variables)
      return train_state_lib.InferenceState.create(variables)

    self._initialize_train_state = initialize_train_state
    # The "shape" state: parameters live in the model's module, so the state object built once
    # here is also the one every later restore copies values into.
    self.global_train_state_shape = initialize_train_state(None)
    self.train_state_axes = (partitioner.get_mesh_axes(self.global_train_state_shape)
                             if partitioner is not None else None)

  def from_scratch(self, init_rng):
    logging.info("Initializing parameters from scratch.")
    return self._initialize_train_state(init_rng)

  def from_checkpoints(self, restore_cfgs: Sequence[RestoreCheckpointConfig], ds_iter=None,
                       init_rng=None) -> Iterable[Tuple[Any, str]]:
    def restore_path(path, cfg):
      if cfg is None:
        raise ValueError("Expected valid `RestoreCheckpointConfig`.")
      ck = cfg.checkpointer_cls(train_state=self.global_train_state_shape,
                                partitioner=self._partitioner, checkpoints_dir="",
                                dataset_iterator=ds_iter if cfg.restore_dataset else None,
                                restore_dtype=cfg.dtype if cfg.dtype else None)
      from_tensorflow = os.path.exists(path + ".index")
      if from_tensorflow and cfg.state_transformation_fns:
        raise ValueError("Cannot initialize from a TensorFlow checkpoint using "
                         "`state_transformation_fns`.")
      if from_tensorflow:
        return ck.restore_from_tf_checkpoint(path, strict=cfg.strict)
      fallback = get_fallback_state(cfg, lambda rng: self.from_scratch(rng).state_dict(),
                                    init_rng)
      return ck.restore(path=path, state_transformation_fns=cfg.state_transformation_fns,
                        fallback_state=fallback)

    cfg, paths = get_first_valid_restore_config_and_paths(restore_cfgs)
    for path in paths:
      yield restore_path(path, cfg), path

  def from_checkpoint(self, ckpt_cfgs, *, ds_iter=None, init_rng=None):
    states = [s for s, _ in self.from_checkpoints(ckpt_cfgs, ds_iter=ds_iter, init_rng=init_rng)]
    if len(states) > 1:
      raise ValueError(f"Expected at most 1 checkpoint but got {len(states)} for config(s): "
                       f"{ckpt_cfgs}")
    return states[0] if states else None

  def from_checkpoint_or_scratch(self, ckpt_cfgs, *, init_rng, ds_iter=None):
    return (self.from_checkpoint(ckpt_cfgs, ds_iter=ds_iter, init_rng=init_rng) or
            self.from_scratch(init_rng))


# ----------------------------------------------------------------------------
# Checkpoint-manager factories
# ----------------------------------------------------------------------------
def create_checkpoint_manager(*, save_cfg: Optional[SaveCheckpointConfig],
                              restore_cfg: Optional[RestoreCheckpointConfig], train_state,
                              partitioner, ds_iter=None, model_dir: Optional[str] = None):
  """Checkpoint manager for the run directory (t5x/utils.py:1205-1270)."""
  save_dtype = restore_dtype = None
  period = keep = keep_ds = None
  checkpoint_steps = None
  cls = checkpoints.OrbaxCheckpointManagerInterface
  if save_cfg is not None:
    save_dtype, period, keep = save_cfg.dtype, save_cfg.period, save_cfg.keep
    keep_ds, checkpoint_steps = save_cfg.keep_dataset_checkpoints, save_cfg.checkpoint_steps
    cls = save_cfg.checkpoint_manager_cls or cls
    if not save_cfg.save_dataset:
      ds_iter = None
  if restore_cfg is not None:
    restore_dtype = restore_cfg.dtype
  return cls(directory=model_dir, train_state=train_state, partitioner=partitioner,
             dataset_iterator=ds_iter, save_dtype=save_dtype, restore_dtype=restore_dtype,
             keep=keep, period=period or 1, checkpoint_steps=checkpoint_steps,
             keep_dataset_checkpoints=keep_ds)


def restore(checkpoint_manager, paths: Sequence[str], restore_cfg: RestoreCheckpointConfig,
            fallback_state=None):
  """Restores one train state (or a list for several paths) (t5x/utils.py:469-526)."""
  fns = restore_cfg.state_transformation_fns

  def one(path):
    # When the newest checkpoint of a run directory is asked for and it turns out to be
    # unreadable (the job was killed while a later process was still flushing it, a disk
    # filled up), fall back to the one before it rather than refuse to resume. All ranks take
    # the decision together: a rank whose shards happened to be intact follows the others.
    from t5x_b200 import checkpoints
    candidates = [path]
    if getattr(restore_cfg, "mode", None) == "latest" and os.path.isdir(path):
      from t5x_b200 import checkpoints_utils
      try:
        parent, step = checkpoints_utils.get_step_from_checkpoint_dir(path)
        candidates += [checkpoints_utils.get_checkpoint_dir(parent, s)
                       for s in reversed(checkpoints_utils.all_steps(parent)) if s < step]
      except ValueError:
        pass
    last_error = None
    for cand in candidates:
      state, error = None, None
      try:
        state = checkpoint_manager.restore(path=cand, fallback_state=fallback_state,
                                           state_transformation_fns=fns)
      except checkpoints.CheckpointReadError as e:
        error = e
      if not pstate.host_any(error is not None):
        return state
      last_error = error or last_error
      logging.warning("Checkpoint %s is unreadable on some rank (%s); trying the previous one.",
                      cand, error)
    raise last_error or checkpoints.CheckpointReadError(f"no readable checkpoint at {path}")

  if len(paths) == 1:
    return one(paths[0])
  return [one(p) for p in paths]


def create_checkpoint_manager_and_restore(train_state_initializer: TrainStateInitializer,
                                          partitioner, restore_checkpoint_cfg,
                                          restore_path: Optional[str], fallback_init_rng,
                                          save_checkpoint_cfg=None, model_dir=None, ds_iter=None,
                                          use_orbax: bool = True):
  """Manager for `model_dir` plus the state restored from `restore_path` (or None)
  (t5x/utils.py:1273-1379)."""
  state = train_state_initializer.global_train_state_shape
  manager = create_checkpoint_manager(save_cfg=save_checkpoint_cfg,
                                      restore_cfg=restore_checkpoint_cfg, train_state=state,
                                      partitioner=partitioner, ds_iter=ds_iter,
                                      model_dir=model_dir)
  train_state = None
  if restore_path and restore_checkpoint_cfg is not None:
    fallback = get_fallback_state(
        restore_checkpoint_cfg,
        lambda rng: train_state_initializer.from_scratch(rng).state_dict(), fallback_init_rng)
    train_state = restore(manager, [restore_path], restore_checkpoint_cfg, fallback)
  return train_state, manager


# ----------------------------------------------------------------------------
# Model info
# ----------------------------------------------------------------------------
def log_model_info(log_file: Optional[str], full_train_state, partitioner) -> None:
  """One line per variable (name, size, shape with axis names, partition spec) and the total
  parameter count, to the log and to `log_file` (t5x/utils.py:1387-1473)."""
  if pstate.get().rank != 0:
    return
  sd = full_train_state.state_dict()
  flat = tree_utils.flatten_dict(sd.get("target", {}))
  axes = {}
  if getattr(full_train_state, "params_axes", None):
    axes = tree_utils.flatten_dict(full_train_state.params_axes,
                                   is_leaf=lambda x: not isinstance(x, Mapping))
  mesh_axes = {}
  if partitioner is not None:
    try:
      ma = partitioner.get_mesh_axes(full_train_state).state_dict().get("target", {})
      mesh_axes = tree_utils.flatten_dict(
          ma, is_leaf=lambda x: not isinstance(x, Mapping) or isinstance(x, PartitionSpec))
    except Exception:  # logging must never break a run
      mesh_axes = {}
  lines = []
  total = 0
  for name, p in flat.items():
    shape = tuple(getattr(p, "global_shape", None) or p.shape)
    n = int(np.prod(shape)) if shape else 1
    total += n
    names = axes.get(name)
    shape_str = (", ".join(f"{a}={s}" for a, s in zip(names, shape)) if names
                 else ", ".join(str(s) for s in shape))
    lines.append(f"Variable {name:<70} size {n:<12} shape ({shape_str}) "
                 f"partition spec {mesh_axes.get(name)}")
  lines.append(f"Total number of parameters: {total}")
  states = sd.get("state", {}).get("param_states")
  if states:
    for name, v in tree_utils.flatten_dict(states).items():
      if hasattr(v, "shape"):
        lines.append(f"Variable param_states/{name:<57} size {int(np.prod(v.shape)):<12} "
                     f"shape {tuple(v.shape)}")
  for l in lines:
    logging.info(l)
  if log_file:
    os.makedirs(os.path.dirname(log_file) or ".", exist_ok=True)
    with open(log_file, "w") as f:
      f.write("\n".join(lines) + "\n")


def round_vocab_size_to_multiple(vocabulary, divisor: int = 128) -> int:
  """Vocabulary size rounded up to a multiple of `divisor` (t5x/utils.py:2188-2193)."""
  size = vocabulary.vocab_size
  return size + -size % divisor


def flatten_dict_string_keys(x):
  return tree_utils.flatten_dict(x, sep="/")


def flatten_lists(lsts):
  out = []
  for l in lsts:
    out.extend(l)
  return out
