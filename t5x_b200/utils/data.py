"""Run-level utilities (API of t5x/utils.py, second half): dataset construction, host batch
iterators, zero batches, `get_infer_fn`, vocabulary checks, checkpoint-step arithmetic."""
from __future__ import annotations

import logging
from typing import Any, Callable, Iterable, Mapping, Optional, Sequence, Tuple

import numpy as np
import torch

from t5x_b200 import data as data_lib
from t5x_b200.data.dataset import Dataset, PrefetchIterator, ShardInfo
from t5x_b200.parallel import state as pstate
from t5x_b200.utils import tree as tree_utils

_INDEX_PAD = -1


# ----------------------------------------------------------------------------
# Datasets
# ----------------------------------------------------------------------------
def import_module(module: Optional[str]) -> None:
  if module:
    import importlib
    importlib.import_module(module)


def get_vocabulary(cfg) -> Tuple[Any, Any]:
  """(input vocabulary, output vocabulary) of a dataset config's task (t5x/utils.py:1843-1914)."""
  import_module(cfg.module)
  provider = data_lib.get_mixture_or_task(cfg.mixture_or_task_name)
  features = provider.output_features
  if "inputs" in features and "targets" in features:
    return features["inputs"].vocabulary, features["targets"].vocabulary
  if "targets" in features:
    v = features["targets"].vocabulary
    return v, v
  raise ValueError('"targets" must be defined in the task features.')


def verify_matching_vocabs(cfg, model) -> None:
  """Model and task vocabularies must agree (t5x/utils.py:1917-1949)."""
  ds_in, ds_out = get_vocabulary(cfg)
  if (ds_in != model.input_vocabulary) or (ds_out != model.output_vocabulary):
    raise ValueError(f"Model and Task vocabularies do not match:\n  task={cfg.mixture_or_task_name}"
                     f"\n  ds_vocabs=({ds_in}, {ds_out})\n  model.input_vocabulary="
                     f"{model.input_vocabulary}\n  model.output_vocabulary="
                     f"{model.output_vocabulary}")


def get_dataset(cfg, shard_id: int, num_shards: int, feature_converter_cls,
                num_epochs: Optional[int] = None, continue_from_last_checkpoint: bool = False):
  """Batched, converted dataset for this host's shard (t5x/utils.py:1952-2073)."""
  if continue_from_last_checkpoint:
    raise ValueError("`continue_from_last_checkpoint` must be set to False as this is not "
                     "supported by this dataset fn.")
  del continue_from_last_checkpoint
  if cfg.module:
    import_module(cfg.module)
  if cfg.batch_size % num_shards:
    raise ValueError(f"Batch size ({cfg.batch_size}) must be divisible by number of shards "
                     f"({num_shards}).")
  seed = cfg.seed
  if seed is None:
    import time
    from t5x_b200.utils import core
    seed = int(core.broadcast_one_to_all(np.int32(time.time())))
    logging.info("Dataset seed not set; using time-based seed %d from rank 0", seed)
  from t5x_b200.utils import core
  core.multihost_assert_equal(int(seed), "`seed` is not same across hosts")
  return get_dataset_inner(cfg, ShardInfo(index=shard_id, num_shards=num_shards),
                           feature_converter_cls, seed, num_epochs)


def get_dataset_inner(cfg, shard_info: ShardInfo, feature_converter_cls, seed=None,
                      num_epochs=None):
  batch_size = cfg.batch_size // shard_info.num_shards
  converter = feature_converter_cls(pack=cfg.pack)
  ds = data_lib.get_dataset(
      mixture_or_task_name=cfg.mixture_or_task_name,
      task_feature_lengths=cfg.task_feature_lengths, dataset_split=cfg.split,
      shuffle=cfg.shuffle, num_epochs=num_epochs, feature_converter=converter,
      shard_info=shard_info, use_cached=cfg.use_cached, seed=seed,
      trim_output_features=cfg.trim_output_features)
  return ds.batch(batch_size, drop_remainder=True)


def get_training_eval_datasets(cfg, shard_id: int, num_shards: int, eval_steps: int,
                               feature_converter_cls, deterministic: bool = False,
                               model_dir: Optional[str] = None, start_step: int = 0
                               ) -> Mapping[str, Dataset]:
  """{task name: dataset of `eval_steps` batches} for teacher-forced evaluation
  (t5x/utils.py:2076-2185)."""
  if isinstance(cfg.mixture_or_task_name, str):
    provider = data_lib.get_mixture_or_task(cfg.mixture_or_task_name)
  else:
    provider = cfg.mixture_or_task_name
  tasks = provider.tasks if hasattr(provider, "tasks") else [provider]
  datasets = {}
  import dataclasses
  for task in tasks:
    if cfg.split not in task.splits:
      logging.info("Task %s has no '%s' split; skipping training evaluation.", task.name,
                   cfg.split)
      continue
    task_cfg = dataclasses.replace(cfg, mixture_or_task_name=task.name, batch_size=cfg.batch_size)
    ds = get_dataset(task_cfg, shard_id, num_shards, feature_converter_cls, num_epochs=None)
    datasets[task.name] = ds.take(eval_steps) if eval_steps > 0 else ds
  if len(tasks) > 1 and isinstance(cfg.mixture_or_task_name, str):
    ds = get_dataset(cfg, shard_id, num_shards, feature_converter_cls, num_epochs=None)
    datasets[cfg.mixture_or_task_name] = ds.take(eval_steps) if eval_steps > 0 else ds
  return datasets


class ShardedDatasetIterator:
  """Host batches -> pinned torch tensors, prefetched on a background thread; positions can
  be saved / restored through the wrapped iterator (t5x/utils.py:693-728)."""

  def __init__(self, iterator, partitioner=None, global_shapes=None, prefetch: int = 2):
    self._iterator = iterator
    self._pin = torch.cuda.is_available()
    self._prefetch = PrefetchIterator(iterator, depth=prefetch, transform=self._convert)

  def _convert(self, batch):
    out = {}
    for k, v in batch.items():
      a = np.asarray(v)
      t = torch.from_numpy(a.astype(np.int64) if a.dtype.kind in "iu" else a)
      out[k] = t.pin_memory() if self._pin else t
    return out

  def __iter__(self):
    return self

  def __next__(self):
    return next(self._prefetch)

  @property
  def element_spec(self):
    return self._iterator.element_spec

  def peek(self):
    return self._iterator.peek()

  def peek_async(self):
    return self._iterator.peek_async()

  def save(self, filename: str):
    return self._iterator.save(filename)

  def restore(self, filename: str):
    return self._iterator.restore(filename)


def prepare_train_iter(train_iter, *, partitioner=None, checkpoint_cfg=None, data_layout=None):
  """Wraps a dataset (iterator) for the train loop (t5x/utils.py:731-757)."""
  if isinstance(train_iter, Dataset):
    train_iter = iter(train_iter)
  return train_iter


def get_zeros_batch_like_spec(batch_spec: Mapping[str, Any]) -> Mapping[str, np.ndarray]:
  return {k: np.zeros(t.shape, t.dtype) for k, t in batch_spec.items()}


def get_zeros_batch_like_dataset(dataset, batch_size=None) -> Mapping[str, np.ndarray]:
  spec = dataset.element_spec
  out = {}
  for k, t in spec.items():
    shape = list(t.shape)
    if batch_size is not None:
      shape[0] = batch_size
    out[k] = np.zeros(shape, t.dtype)
  return out


# ----------------------------------------------------------------------------
# Inference function
# ----------------------------------------------------------------------------
def get_infer_fn(infer_step: Callable, batch_size: int, train_state_axes, partitioner,
                 keep_aux_as_numpy: bool = False) -> Callable:
  """Builds `infer_fn(ds, train_state, rng=None)` that runs `infer_step(params, batch, rng)`
  over an enumerated dataset and returns `[(index, output), ...]` (plus aux) in dataset order.

  The dataset is padded to a multiple of the batch size with copies of its first example
  tagged index -1, examples are dealt round-robin to the data shards, and the padded rows are
  dropped from the result (t5x/utils.py:1543-1817)."""
  layout = partitioner.get_data_layout(batch_size) if partitioner is not None else None
  num_shards = layout.num_shards if layout else 1
  shard_id = layout.shard_id if layout else 0
  per_shard_batch = batch_size // num_shards
  device = pstate.get().device

  def infer_fn(ds, train_state, rng=None):
    examples = list(ds)
    if not examples:
      return []
    n = len(examples)
    first_idx, first_ex = examples[0]
    pad = (-n) % batch_size
    examples = examples + [(_INDEX_PAD, first_ex)] * pad
    mine = examples[shard_id::num_shards]
    all_indices, all_outputs, all_aux = [], [], []
    for start in range(0, len(mine), per_shard_batch):
      chunk = mine[start:start + per_shard_batch]
      idx = np.asarray([i for i, _ in chunk], dtype=np.int64)
      batch = {k: torch.from_numpy(np.stack([np.asarray(ex[k]) for _, ex in chunk]).astype(
          np.int64 if np.asarray(chunk[0][1][k]).dtype.kind in "iu" else np.float32)).to(device)
               for k in chunk[0][1]}
      step_rng = None if rng is None else (int(rng) * 1000003 + start) % (2 ** 31)
      with torch.no_grad():
        out = infer_step(train_state.params, batch, step_rng)
      aux = None
      if isinstance(out, tuple):
        out, aux = out
      all_indices.append(idx)
      all_outputs.append(tree_utils.tree_map(_to_numpy, out))
      if aux is not None:
        all_aux.append(tree_utils.tree_map(_to_numpy, aux))
    indices = np.concatenate(all_indices)
    outputs = _concat(all_outputs)
    aux = _concat(all_aux) if all_aux else None
    # gather the shards of every data-parallel replica
    if num_shards > 1:
      import torch.distributed as dist
      gathered = [None] * dist.get_world_size()
      dist.all_gather_object(gathered, (shard_id, indices, outputs, aux))
      seen = {}
      for sid, i, o, a in gathered:
        seen.setdefault(sid, (i, o, a))
      parts = [seen[s] for s in sorted(seen)]
      indices = np.concatenate([p[0] for p in parts])
      outputs = _concat([p[1] for p in parts])
      aux = _concat([p[2] for p in parts]) if aux is not None else None
    keep = indices != _INDEX_PAD
    order = np.argsort(indices[keep], kind="stable")

    def select(x):
      return x[keep][order]

    idx_sorted = indices[keep][order]
    outputs = tree_utils.tree_map(select, outputs)
    result = list(zip(idx_sorted.tolist(), _unstack(outputs, len(idx_sorted))))
    if aux is None:
      return result
    aux = tree_utils.tree_map(select, aux)
    if not keep_aux_as_numpy:
      aux = tree_utils.tree_map(lambda x: x.tolist(), aux)
    return result, aux

  return infer_fn


def _to_numpy(x):
  if isinstance(x, torch.Tensor):
    x = x.detach()
    if x.dtype == torch.bfloat16:
      x = x.float()
    return x.cpu().numpy()
  return np.asarray(x)


def _concat(parts):
  first = parts[0]
  if isinstance(first, Mapping):
    return {k: _concat([p[k] for p in parts]) for k in first}
  return np.concatenate(parts, axis=0)


def _unstack(tree, n):
  if isinstance(tree, Mapping):
    cols = {k: _unstack(v, n) for k, v in tree.items()}
    return [{k: cols[k][i] for k in cols} for i in range(n)]
  return [tree[i] for i in range(n)]


# ----------------------------------------------------------------------------
# Misc
# ----------------------------------------------------------------------------
def override_params_axes_names(model_variables, params_axes_names_override=()):
  """Replaces the logical axis names of parameters whose path fully matches a regex
  (t5x/utils.py:2220-2281)."""
  import re
  if "params_axes" not in model_variables:
    raise ValueError("Model variables do not contain a 'params_axes' collection to apply an "
                     "override to.")
  flat_params = tree_utils.flatten_dict(model_variables["params"])
  flat_axes = tree_utils.flatten_dict(model_variables["params_axes"],
                                      is_leaf=lambda x: not isinstance(x, Mapping))
  for key, param in flat_params.items():
    for pattern, names in params_axes_names_override:
      if re.fullmatch(pattern, key):
        if len(names) != param.dim():
          raise ValueError(f"Provided axis name override for {key} does not match param rank "
                           f"({param.dim()}): {names}")
        flat_axes[key] = tuple(names)
        if isinstance(param, torch.Tensor):
          param.axes = tuple(names)
        break
  out = dict(model_variables)
  out["params_axes"] = tree_utils.unflatten_dict(flat_axes)
  return out


def find_next_checkpoint_step(step: int, period: Optional[int],
                              checkpoint_steps_index: int,
                              checkpoint_steps: Optional[Sequence[int]]
                              ) -> Tuple[Optional[int], Optional[int], int]:
  """(next periodic step, next explicit step, new index) after `step`
  (t5x/utils.py:2284-2350)."""
  next_periodic = None
  if period:
    next_periodic = (step // period + 1) * period
  next_explicit = None
  steps = sorted(checkpoint_steps) if checkpoint_steps else []
  idx = checkpoint_steps_index
  while idx < len(steps) and steps[idx] <= step:
    idx += 1
  if idx < len(steps):
    next_explicit = steps[idx]
  return next_periodic, next_explicit, idx


def find_first_checkpoint_step(host_step: int, checkpoint_steps: Optional[Sequence[int]]
                               ) -> Tuple[Optional[int], int]:
  """First explicit checkpoint step >= host_step and its index (t5x/utils.py:2353-2382)."""
  if not checkpoint_steps:
    return None, 0
  steps = sorted(checkpoint_steps)
  for i, s in enumerate(steps):
    if s >= host_step:
      return s, i
  return None, len(steps)
