"""Checkpointing in the native T5X format (API of t5x/checkpoints.py).

Layout of `<dir>/checkpoint_<step>/`:
  checkpoint                       msgpack {'version': 3, 'optimizer': state_dict}; every leaf is
                                   either an inline array or a TensorStore spec dict
                                   {'driver':'zarr','dtype':..,'kvstore':{'driver':'file',
                                   'path':'target.a.b.kernel'},'metadata':{'compressor':{'id':
                                   'gzip'},'shape':[..],'chunks':[..]}} with a RELATIVE path
  target.<a.b.c>/ , state.param_states.<...>.v/   one zarr v2 array per partitioned leaf
  train_ds-SSS-of-NNN              optional dataset iterator position per data shard
A leaf is a zarr array when the partitioner gives it a PartitionSpec (every parameter with
logical axis names, plus unfactored Adafactor moments) and inline otherwise (step, factored
v_row / v_col, (1,) placeholders). Every rank writes only the chunks of its own slice (and only
if it is replica 0 for that slice); rank 0 writes the msgpack index and renames the temporary
directory into place, so a checkpoint either exists completely or not at all. Checkpoints are
topology independent: restore reads whatever slice the current mesh assigns to this rank.
"""
from __future__ import annotations

import concurrent.futures
import dataclasses
from zlib import error as zlib_error
import functools
import logging
import os
import re
import shutil
import time
from typing import Any, Callable, Dict, Mapping, Optional, Sequence, Tuple, Union

import numpy as np
import torch
import torch.distributed as dist

from t5x_b200 import checkpoint_utils
from t5x_b200 import checkpoints_utils
from t5x_b200 import partitioning
from t5x_b200 import state_utils
from t5x_b200.io import msgpack_io
from t5x_b200.io import orbax_tree
from t5x_b200.io import zarr_io
from t5x_b200.parallel import state as pstate
from t5x_b200.utils import tree as tree_utils

PartitionSpec = partitioning.PartitionSpec
VERSION = 3
_DESIRED_CHUNK_SIZE_BYTES = 64 * 1024 * 1024
_TRAIN_DS_PREFIX = "train_ds"

all_steps = checkpoints_utils.all_steps
all_dataset_checkpoint_steps = checkpoints_utils.all_dataset_checkpoint_steps
latest_step = checkpoints_utils.latest_step
get_checkpoint_dir = checkpoints_utils.get_checkpoint_dir
get_checkpoint_prefix = checkpoints_utils.get_checkpoint_prefix

SaveStateTransformationFn = Callable[[Mapping[str, Any], Mapping[str, Any]],
                                     Tuple[Mapping[str, Any], Mapping[str, Any]]]
RestoreStateTransformationFn = Callable[..., Mapping[str, Any]]


def _choose_chunk_shape(write_shape: Sequence[int], target_elements: int):
  """Chunk shape of an array written as `write_shape`: every chunk extent divides its
  dimension, the chunk holds at most `target_elements` values, and it is reached from the
  whole array by repeatedly stepping the widest remaining extent (the first one on a tie)
  down to its next smaller divisor. This walk fixes the on-disk chunk grid, so that files
  written here are chunked like the reference's (t5x/checkpoints.py:103-157)."""
  if target_elements < 1:
    raise ValueError("target_elements must be at least 1")
  chunk = [int(n) for n in write_shape]

  def step_down(extent: int, full: int) -> int:
    for cand in range(extent - 1, 0, -1):
      if full % cand == 0:
        return cand
    raise AssertionError("extent 1 has no smaller divisor")

  while int(np.prod(chunk, dtype=np.int64)) > target_elements:
    widest = max(range(len(chunk)), key=lambda i: (chunk[i], -i))
    chunk[widest] = step_down(chunk[widest], int(write_shape[widest]))
  return chunk


@dataclasses.dataclass
class _ParameterInfo:
  """What is needed to write/read one leaf."""
  name: str
  shape: Tuple[int, ...]                 # global shape
  ts_spec: Optional[Dict[str, Any]]      # None => inline in the msgpack file
  local_chunk_info: Optional[partitioning.LocalChunkInfo]
  axes: Optional[PartitionSpec] = None


class LazyArray:
  """An array that is materialised on `get()` (t5x/checkpoint_importer.py:34-186)."""

  def __init__(self, shape, dtype, get_fn: Callable[[], np.ndarray]):
    self._shape = tuple(shape)
    self._dtype = np.dtype(dtype) if not isinstance(dtype, torch.dtype) else dtype
    self._get_fn = get_fn

  @property
  def shape(self):
    return self._shape

  @property
  def dtype(self):
    return self._dtype

  @property
  def size(self):
    return int(np.prod(self._shape))

  def astype(self, dtype):
    return LazyArray(self._shape, dtype, lambda: self._get_fn().astype(dtype))

  def get(self) -> np.ndarray:
    return self._get_fn()

  def __repr__(self):
    return f"{type(self).__name__}(shape={self.shape}, dtype={self.dtype})"


LazyThreadPoolArray = LazyArray
LazyAwaitableArray = LazyArray


def _maybe_get(x):
  return x.get() if isinstance(x, LazyArray) else x


def _to_numpy(x) -> np.ndarray:
  return msgpack_io._to_numpy(_maybe_get(x))


def _np_dtype(d) -> Optional[np.dtype]:
  if d is None:
    return None
  if isinstance(d, torch.dtype):
    if d == torch.bfloat16:
      import ml_dtypes
      return np.dtype(ml_dtypes.bfloat16)
    return np.dtype(str(d).replace("torch.", ""))
  if isinstance(d, str) and d == "bfloat16":
    import ml_dtypes
    return np.dtype(ml_dtypes.bfloat16)
  return np.dtype(d)


def _sync_global_devices(name: str) -> None:
  """Barrier over all ranks between the phases of a save (multihost_utils.sync_global_devices in
  the reference). It runs on the host with a timeout: a rank that crashed before reaching
  `name` turns into a `HostSyncError` on the others, not into a save that never returns."""
  pstate.host_barrier(name)


class CheckpointReadError(ValueError):
  """A checkpoint exists but cannot be read (index file missing or damaged, an array chunk
  missing or truncated)."""


def _broadcast_int_from_rank0(value: int) -> int:
  if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
    obj = [value]
    dist.broadcast_object_list(obj, src=0)
    return int(obj[0])
  return int(value)


def _rank() -> int:
  return pstate.get().rank


def _spec_for(name: str, dtype: np.dtype, metadata: Dict[str, Any]) -> Dict[str, Any]:
  return {"driver": "zarr", "dtype": zarr_io.dtype_name(dtype),
          "kvstore": {"driver": "file", "path": name.replace("/", ".")},
          "metadata": metadata}


def _spec_path(spec: Mapping[str, Any], ckpt_dir: str) -> str:
  """Directory of the array a (relative or absolute, file or gcs) spec points at, re-rooted
  at `ckpt_dir` where the checkpoint now lives (t5x/checkpoints.py:237-347)."""
  kv = spec.get("kvstore", {})
  path = kv.get("path", "") or spec.get("path", "")
  if spec.get("path") and kv.get("driver") == "gcs":
    path = spec["path"]
  path = path.rstrip("/")
  if os.path.isabs(path):
    rel = os.path.basename(path)
    cand = os.path.join(ckpt_dir, rel)
    return cand if os.path.exists(cand) or not os.path.exists(path) else path
  return os.path.join(ckpt_dir, os.path.basename(path) if "/" in path and not os.path.exists(
      os.path.join(ckpt_dir, path)) else path)


def _is_spec(x) -> bool:
  return state_utils.tensorstore_leaf(None, x)


def _gather_model_shards(t: torch.Tensor) -> torch.Tensor:
  """Full tensor for an inline leaf that is sharded over the model axis (factored Adafactor
  vectors of tensor-parallel weights)."""
  st = pstate.get()
  sd = getattr(t, "shard_dim", None)
  if sd is None or st.model_size == 1:
    return t
  parts = [torch.empty_like(t) for _ in range(st.model_size)]
  dist.all_gather(parts, t.contiguous(), group=st.model_group)
  return torch.cat(parts, dim=sd)


class Checkpointer:
  """Saves and restores train states in the T5X format (t5x/checkpoints.py:501-1339)."""

  def __init__(self, train_state, partitioner, checkpoints_dir: str, dataset_iterator=None, *,
               keep: Optional[int] = None, save_dtype=np.float32, restore_dtype=None,
               keep_dataset_checkpoints: Optional[int] = None):
    self._train_state = train_state
    self._partitioner = partitioner
    self.checkpoints_dir = os.fspath(checkpoints_dir)
    self.keep = keep
    self.keep_dataset_checkpoints = keep_dataset_checkpoints
    self._save_dtype = _np_dtype(save_dtype)
    self.restore_dtype = _np_dtype(restore_dtype)
    self._dataset_iterator = dataset_iterator
    self._dataset_ckpt_name = None
    self._should_write_dataset_ckpt = False
    if dataset_iterator is not None:
      layout = partitioner.get_data_layout()
      self._dataset_ckpt_name = (f"{_TRAIN_DS_PREFIX}-{layout.shard_id:03}-of-"
                                 f"{layout.num_shards:03}")
      self._should_write_dataset_ckpt = layout.is_first_host_in_replica_set
    self._parameter_infos = self._get_parameter_infos()

  # -- bookkeeping ------------------------------------------------------------------------
  def all_steps(self) -> Sequence[int]:
    return all_steps(self.checkpoints_dir)

  def all_dataset_checkpoint_steps(self) -> Sequence[int]:
    return all_dataset_checkpoint_steps(self.checkpoints_dir)

  def latest_step(self) -> Optional[int]:
    return latest_step(self.checkpoints_dir)

  def _remove_old_dataset_checkpoints(self):
    if self.keep_dataset_checkpoints:
      steps = self.all_dataset_checkpoint_steps()
      for step in steps[:-self.keep_dataset_checkpoints]:
        checkpoint_utils.remove_dataset_checkpoint(get_checkpoint_dir(self.checkpoints_dir, step),
                                                   _TRAIN_DS_PREFIX)

  def _remove_stale_tmp_dirs(self, keep: Optional[str] = None):
    """`checkpoint_<step>.tmp-<timestamp>` directories are saves that never reached their final
    rename (the job died mid-save). Step discovery ignores them; the next save removes them."""
    import glob
    import shutil
    pattern = os.path.join(self.checkpoints_dir, f"{get_checkpoint_prefix()}_*.tmp-*")
    for path in glob.glob(pattern):
      if path != keep and os.path.isdir(path):
        logging.warning("Removing unfinished checkpoint directory %s", path)
        shutil.rmtree(path, ignore_errors=True)

  def _remove_old_checkpoints(self):
    if self.keep:
      steps = self.all_steps()
      for step in steps[:-self.keep]:
        checkpoint_utils.remove_checkpoint_dir(get_checkpoint_dir(self.checkpoints_dir, step))

  # -- parameter infos --------------------------------------------------------------------
  def _mesh_axes_state_dict(self):
    if self._partitioner is None:
      return None
    return self._partitioner.get_mesh_axes(self._train_state).state_dict()

  def _get_parameter_infos(self):
    """State-dict-shaped tree of _ParameterInfo (t5x/checkpoints.py:623-702)."""
    sd = self._train_state.state_dict()
    flat = tree_utils.flatten_dict(sd, keep_empty_nodes=True)
    axes_sd = self._mesh_axes_state_dict()
    flat_axes = {}
    if axes_sd is not None:
      flat_axes = tree_utils.flatten_dict(
          axes_sd, keep_empty_nodes=True,
          is_leaf=lambda x: not isinstance(x, Mapping) or isinstance(x, PartitionSpec))
    infos = {}
    for name, arr in flat.items():
      if arr is None:
        infos[name] = None
        continue
      if isinstance(arr, dict) and not arr:
        infos[name] = {}
        continue
      axes = flat_axes.get(name)
      gshape = tuple(getattr(arr, "global_shape", None) or getattr(arr, "shape", ()))
      if axes is None or self._partitioner is None:
        infos[name] = _ParameterInfo(name, gshape, None, None, None)
        continue
      info = self._partitioner.get_local_chunk_info(gshape, axes)
      write_shape = [si if sl == slice(None) else sl.stop - sl.start
                     for si, sl in zip(gshape, info.slice)]
      dtype = _np_dtype(arr.dtype) if hasattr(arr, "dtype") else np.dtype(np.float32)
      if name.split("/")[0] == "target" and self._save_dtype is not None:
        dtype = self._save_dtype
      chunk_shape = _choose_chunk_shape(
          write_shape, target_elements=max(1, _DESIRED_CHUNK_SIZE_BYTES // dtype.itemsize))
      metadata = {"compressor": {"id": "gzip"}, "shape": list(gshape),
                  "chunks": [int(c) for c in chunk_shape]}
      infos[name] = _ParameterInfo(name, gshape, _spec_for(name, dtype, metadata), info, axes)
    return tree_utils.unflatten_dict(infos)

  def _get_state_dict_for_save(self, state_dict, lazy_load: bool = True):
    return state_dict

  # -- save -------------------------------------------------------------------------------
  def save(self, train_state, state_transformation_fns: Sequence[SaveStateTransformationFn] = (),
           *, concurrent_gb: int = 128):
    """Writes `checkpoint_<step>` atomically (t5x/checkpoints.py:742-845)."""
    start = time.time()
    step = int(_to_numpy(train_state.step))
    timestamp = _broadcast_int_from_rank0(int(time.time()))
    final_dir = os.path.join(self.checkpoints_dir, f"{get_checkpoint_prefix()}_{step}")
    tmp_dir = final_dir + f".tmp-{timestamp}"
    if os.path.exists(final_dir):
      logging.info("Skipping save checkpoint for step %d (directory %s already exists)", step,
                   final_dir)
      return
    logging.info("Saving checkpoint for step %d to %s", step, tmp_dir)
    if _rank() == 0:
      self._remove_stale_tmp_dirs(keep=tmp_dir)
      os.makedirs(tmp_dir, exist_ok=True)
    _sync_global_devices(f"checkpointer:make_dir:{tmp_dir}")
    written = self._write_state_to_tensorstore(tmp_dir, train_state, concurrent_gb,
                                               state_transformation_fns)
    if self._should_write_dataset_ckpt:
      self._dataset_iterator.save(os.path.join(tmp_dir, self._dataset_ckpt_name))
    _sync_global_devices(f"checkpointer:tensorstore_write_complete:{tmp_dir}")
    if _rank() == 0:
      data = msgpack_io.msgpack_serialize({"version": VERSION, "optimizer": written})
      with open(os.path.join(tmp_dir, "checkpoint"), "wb") as fp:
        fp.write(data)
      os.rename(tmp_dir, final_dir)
      logging.info("Saved checkpoint for step %d to %s", step, final_dir)
      self._remove_old_checkpoints()
      self._remove_old_dataset_checkpoints()
    _sync_global_devices(f"checkpointer:write_complete:{final_dir}")
    logging.info("checkpoint write took %.2f s", time.time() - start)

  def _write_state_to_tensorstore(self, ckpt_dir, train_state, concurrent_gb,
                                  state_transformation_fns):
    """Writes every partitioned leaf's local slice; returns the state dict for the index with
    those leaves replaced by their specs (t5x/checkpoints.py:847-978)."""
    state_dict = self._get_state_dict_for_save(train_state.state_dict())
    infos = self._parameter_infos
    for fn in state_transformation_fns:
      state_dict, infos = fn(state_dict, infos)
    flat_sd = tree_utils.flatten_dict(state_dict, keep_empty_nodes=True)
    flat_info = tree_utils.flatten_dict(
        infos, keep_empty_nodes=True,
        is_leaf=lambda x: not isinstance(x, Mapping) or isinstance(x, _ParameterInfo))
    out = {}
    budget = _BytesBudget(int(concurrent_gb * 10 ** 9))
    futures = []
    pool = concurrent.futures.ThreadPoolExecutor(max_workers=8)
    for name, value in flat_sd.items():
      info = flat_info.get(name)
      if value is None or (isinstance(value, dict) and not value) or info is None or \
          not isinstance(info, _ParameterInfo):
        out[name] = value
        continue
      if info.ts_spec is None:
        v = _maybe_get(value)
        if isinstance(v, torch.Tensor):
          v = _gather_model_shards(v)
        out[name] = _to_numpy(v)
        continue
      out[name] = info.ts_spec
      if info.local_chunk_info.replica_id != 0:
        continue
      dtype = _np_dtype(info.ts_spec["dtype"])
      md = info.ts_spec["metadata"]
      path = os.path.join(ckpt_dir, info.ts_spec["kvstore"]["path"])

      def write(value=value, dtype=dtype, md=md, path=path, info=info):
        arr = _to_numpy(value)
        nbytes = arr.size * arr.dtype.itemsize
        budget.acquire(nbytes)
        try:
          if arr.dtype != dtype:
            arr = arr.astype(dtype)
          z = zarr_io.ZarrArray.create(path, md["shape"], md["chunks"], dtype,
                                       md.get("compressor"))
          z.write(arr, info.local_chunk_info.slice)
        finally:
          budget.release(nbytes)

      futures.append(pool.submit(write))
    for f in futures:
      f.result()
    pool.shutdown()
    _sync_global_devices(f"checkpointer:tensorstore_write_complete_inner:{ckpt_dir}")
    return tree_utils.unflatten_dict(out)

  # -- restore ----------------------------------------------------------------------------
  def restore(self, step: Optional[int] = None, path: Optional[str] = None,
              state_transformation_fns: Sequence[RestoreStateTransformationFn] = (),
              fallback_state: Optional[Mapping[str, Any]] = None, lazy_parameters: bool = False):
    """Restores the train state from a checkpoint (t5x/checkpoints.py:991-1159)."""
    if lazy_parameters and self._partitioner is not None and \
        getattr(self._partitioner, "params_on_devices", False):
      raise ValueError("Lazy Parameters cannot be copied to devices, please set partitioner."
                       "params_on_devices=False.")
    if step is not None and path is not None:
      raise ValueError("At most one of `step` or `path` may be provided.")
    if path:
      ckpt_path = path
    else:
      if step is None:
        step = self.latest_step()
        if not step and step != 0:
          raise ValueError(f"No checkpoints found in {self.checkpoints_dir}.")
      ckpt_path = get_checkpoint_dir(self.checkpoints_dir, step)
    if os.path.isdir(ckpt_path):
      ckpt_dir = ckpt_path
      ckpt_path = os.path.join(ckpt_path, "checkpoint")
    else:
      ckpt_dir = os.path.dirname(ckpt_path)
    tree_dir = orbax_tree.find_state_dir(ckpt_dir)
    if tree_dir is not None:
      # One zarr directory per leaf plus a placeholder / metadata file: the layout of the
      # reference's Orbax manager (t5x/checkpoints.py:2386-2510).
      logging.info("Restoring from PyTree checkpoint directory: %s", tree_dir)
      try:
        ckpt_contents = {"version": VERSION, "optimizer": _orbax_state_dict(tree_dir)}
      except NotImplementedError:
        raise
      except Exception as e:
        raise CheckpointReadError(f"Checkpoint tree {tree_dir} is damaged: {e}") from e
      ckpt_dir = tree_dir
    else:
      if not os.path.exists(ckpt_path) or os.path.isdir(ckpt_path):
        raise CheckpointReadError(f"Path is not a valid T5X checkpoint: {ckpt_path}")
      logging.info("Restoring from checkpoint: %s", ckpt_path)
      try:
        with open(ckpt_path, "rb") as fp:
          raw = fp.read()
        ckpt_contents = msgpack_io.msgpack_restore(raw)
        if not isinstance(ckpt_contents, Mapping) or "optimizer" not in ckpt_contents:
          raise ValueError("no 'optimizer' entry")
      except Exception as e:
        raise CheckpointReadError(f"Checkpoint index {ckpt_path} is damaged: {e}") from e
    ckpt_state_dict = self._get_optimizer_state_dict(ckpt_contents, state_transformation_fns)
    written_infos = self._parameter_infos
    target_sd = self._train_state.state_dict()
    if fallback_state is not None:
      ckpt_state_dict = dict(ckpt_state_dict)
    flat_ckpt = state_utils.flatten_state_dict(ckpt_state_dict, keep_empty_nodes=True)
    flat_target = tree_utils.flatten_dict(target_sd, keep_empty_nodes=True)
    flat_info = tree_utils.flatten_dict(
        written_infos, keep_empty_nodes=True,
        is_leaf=lambda x: not isinstance(x, Mapping) or isinstance(x, _ParameterInfo))
    flat_fallback = state_utils.flatten_state_dict(fallback_state or {})
    missing = [k for k in flat_target if k not in flat_ckpt and k not in flat_fallback]
    if missing:
      raise ValueError("The target dict keys and state dict keys do not match, target dict "
                       f"contains keys {sorted(missing)} which are not present in the checkpoint")
    # Checkpoint entries the target has no slot for (e.g. optimizer slots when restoring for
    # inference) are left unread.
    for k in flat_ckpt:
      if k not in flat_target:
        logging.debug("Not restoring key from ckpt: %s", k)
    restored = {}
    for name, tgt in flat_target.items():
      if name not in flat_ckpt:
        restored[name] = flat_fallback[name]
        logging.warning("Initializing param=%s from fallback state", name)
        continue
      try:
        restored[name] = self._read_leaf(name, flat_ckpt[name], tgt, flat_info.get(name),
                                         ckpt_dir, ckpt_contents.get("version", VERSION),
                                         lazy_parameters)
      except (OSError, EOFError, KeyError, zlib_error, ValueError) as e:
        if isinstance(e, CheckpointReadError):
          raise
        raise CheckpointReadError(
            f"Array {name} of checkpoint {ckpt_dir} cannot be read "
            f"({type(e).__name__}: {e})") from e
    state_dict = tree_utils.unflatten_dict(restored)
    if self._dataset_iterator is not None and self._dataset_ckpt_name:
      ds_path = os.path.join(ckpt_dir, self._dataset_ckpt_name)
      if os.path.exists(ds_path):
        self._dataset_iterator.restore(ds_path)
      else:
        logging.warning("dataset checkpoint %s not found; iterator starts from scratch", ds_path)
    return self._train_state.restore_state(state_dict)

  def _read_leaf(self, name, ckpt_leaf, target, info, ckpt_dir, version, lazy):
    if target is None or (isinstance(target, dict) and not target):
      return target
    is_target_param = name.split("/")[0] == "target"
    rd = self.restore_dtype if is_target_param else None
    local_shape = tuple(getattr(target, "shape", ()))
    gshape = tuple(info.shape) if isinstance(info, _ParameterInfo) else local_shape
    region = None
    if isinstance(info, _ParameterInfo) and info.local_chunk_info is not None:
      region = info.local_chunk_info.slice
    elif gshape != local_shape and getattr(target, "shard_dim", None) is not None:
      st = pstate.get()
      sdim = target.shard_dim
      per = gshape[sdim] // st.model_size
      region = tuple(slice(st.model_rank * per, (st.model_rank + 1) * per) if i == sdim
                     else slice(None) for i in range(len(gshape)))
    if isinstance(ckpt_leaf, orbax_tree.ArrayRef):
      def get():
        want = _np_dtype(target.dtype) if hasattr(target, "dtype") else None
        return ckpt_leaf.read(region, dtype=rd, expected_shape=gshape, expected_dtype=want)
    elif _is_spec(ckpt_leaf):
      def get():
        return _read_ts(ckpt_leaf, ckpt_dir, gshape, region, rd, version, name)
    else:
      def get():
        arr = np.asarray(ckpt_leaf)
        if arr.shape != gshape and arr.shape != local_shape:
          raise ValueError(f"Shape of `{name}` in checkpoint {arr.shape} does not match "
                           f"expectation {gshape}.")
        if region is not None and arr.shape == gshape and gshape != local_shape:
          arr = arr[region]
        if rd is not None:
          arr = arr.astype(rd)
        return arr
    if lazy:
      dtype = rd or (_np_dtype(target.dtype) if hasattr(target, "dtype") else np.float32)
      return LazyArray(local_shape, dtype, get)
    return get()

  def _get_optimizer_state_dict(self, ckpt_contents, state_transformation_fns):
    return _get_optimizer_state_dict(ckpt_contents, self._train_state.state_dict(),
                                     state_transformation_fns)

  # -- TF checkpoints ---------------------------------------------------------------------
  def restore_from_tf_checkpoint(self, path_or_dir: str, strict: bool = True, translator=None):
    """Restores parameters from a Mesh-TensorFlow T5 checkpoint (optimizer state, if the
    checkpoint carries Adafactor slots, included) (t5x/checkpoints.py:1261-1304)."""
    from t5x_b200 import checkpoint_importer
    full_state_dict = checkpoint_importer.restore_from_t5_checkpoint(
        self._train_state.state_dict(), path_or_dir, strict=strict, translator=translator)
    return self._train_state.restore_state(full_state_dict)

  def convert_from_tf_checkpoint(self, path_or_dir: str, *, state_transformation_fns=(),
                                 concurrent_gb: int = 16, translator=None):
    """Reads a TF checkpoint and writes it out in the native format
    (t5x/checkpoints.py:1306-1326)."""
    train_state = self.restore_from_tf_checkpoint(path_or_dir, translator=translator)
    self.save(train_state, state_transformation_fns, concurrent_gb=concurrent_gb)


class _BytesBudget:
  """Blocks writers while more than `max_bytes` are in flight (t5x/checkpoints.py:424-442)."""

  def __init__(self, max_bytes: int):
    import threading
    self._max = max(1, max_bytes)
    self._used = 0
    self._cv = threading.Condition()

  def acquire(self, n: int):
    n = min(n, self._max)
    with self._cv:
      self._cv.wait_for(lambda: self._used + n <= self._max)
      self._used += n

  def release(self, n: int):
    n = min(n, self._max)
    with self._cv:
      self._used -= n
      self._cv.notify_all()


def _read_ts(spec: Mapping[str, Any], ckpt_dir: str, expected_shape, region, restore_dtype,
             version: int, name: str = "") -> np.ndarray:
  """Reads (a region of) the zarr array a spec points to, trusting the on-disk `.zarray` for
  chunking/compression (t5x/checkpoints.py:1673-1775)."""
  path = _spec_path(spec, ckpt_dir)
  z = zarr_io.ZarrArray.open(path)
  if expected_shape is not None and tuple(z.shape) != tuple(expected_shape):
    raise ValueError(f"Shape of `{name}` in checkpoint {tuple(z.shape)} does not match "
                     f"expectation {tuple(expected_shape)}.")
  if version < 3 and spec.get("dtype") == "bfloat16" and z.dtype == np.dtype(np.uint16):
    raise ValueError("Checkpoints with bfloat16 stored as uint16 (format version 2) are not "
                     "supported; re-save the checkpoint with a current version.")
  return z.read(region, dtype=restore_dtype)


def _orbax_state_dict(tree_dir: str):
  """Tree of a PyTree checkpoint directory as a state dict: sequences become dicts keyed
  '0', '1', ... (the form `state_dict()` gives them) and a bare dataclass dump with an
  `_optimizer` entry is unwrapped to its {'state', 'target'} part."""
  def as_dicts(node):
    if isinstance(node, Mapping):
      return {str(k): as_dicts(v) for k, v in node.items()}
    if isinstance(node, (list, tuple)):
      return {str(i): as_dicts(v) for i, v in enumerate(node)}
    return node
  tree = as_dicts(orbax_tree.load_tree(tree_dir))
  if "_optimizer" in tree and "target" not in tree:
    extra = {k: v for k, v in tree.items() if k == "flax_mutables" and v}
    tree = dict(tree["_optimizer"], **extra)
  return tree


def save_state_as_orbax_tree(train_state, checkpoints_dir: str, compressor=None) -> str:
  """Writes `train_state.state_dict()` under `<checkpoints_dir>/checkpoint_<step>/state/` in
  the one-directory-per-array PyTree layout (where the reference's Orbax manager puts its
  state item, t5x/checkpoints.py:2336-2384). A single-process export for interchange: arrays
  must be whole on this rank. Returns the checkpoint directory."""
  step = int(_to_numpy(train_state.step))
  final_dir = get_checkpoint_dir(checkpoints_dir, step)
  tmp_dir = final_dir + f".tmp-{int(time.time())}"
  flat = tree_utils.flatten_dict(train_state.state_dict(), keep_empty_nodes=True)
  tree = tree_utils.unflatten_dict(
      {k: (v if v is None or (isinstance(v, Mapping) and not v) else _to_numpy(_maybe_get(v)))
       for k, v in flat.items()})
  orbax_tree.save_tree(os.path.join(tmp_dir, "state"), tree, compressor)
  if os.path.exists(final_dir):
    checkpoint_utils.remove_checkpoint_dir(final_dir)
  os.rename(tmp_dir, final_dir)
  return final_dir


def _get_optimizer_state_dict(ckpt_contents, optimizer_state, state_transformation_fns):
  """Checkpoint's optimizer dict after version checks and restore transformations
  (t5x/checkpoints.py:1637-1659)."""
  version = ckpt_contents.get("version", 0)
  if version == 0:
    ckpt_optimizer_state = ckpt_contents
  else:
    ckpt_optimizer_state = ckpt_contents["optimizer"]
  if version >= 2:
    for fn in state_transformation_fns:
      ckpt_optimizer_state = fn(ckpt_optimizer_state, optimizer_state)
    return ckpt_optimizer_state
  raise ValueError("Checkpoint versions earlier than 2 are not supported. "
                   f"Got version: {version}")


# ----------------------------------------------------------------------------
# Standalone loading
# ----------------------------------------------------------------------------
def find_checkpoint(path: str, step: Optional[int] = None) -> str:
  """Path of the msgpack index given a dir of checkpoints, a checkpoint dir or the file itself
  (t5x/checkpoints.py:1803-1832)."""
  if os.path.isdir(path):
    if step is not None:
      path = get_checkpoint_dir(path, step)
    elif os.path.exists(os.path.join(path, "checkpoint")):
      pass
    else:
      s = latest_step(path)
      if s is None:
        raise ValueError(f"No checkpoints found in {path}")
      path = get_checkpoint_dir(path, s)
    path = os.path.join(path, "checkpoint")
  if not os.path.exists(path) or os.path.isdir(path):
    raise ValueError(f"Path is not a valid checkpoint: {path}")
  return path


def load_t5x_checkpoint(path: str, step: Optional[int] = None,
                        state_transformation_fns: Sequence[RestoreStateTransformationFn] = (),
                        remap: bool = True, restore_dtype=None, lazy_parameters: bool = False):
  """Reads a whole checkpoint into a nested dict without needing the model or optimizer
  (t5x/checkpoints.py:1835-1958)."""
  tree_dir = None
  if os.path.isdir(path):
    cand = path if step is None else get_checkpoint_dir(path, step)
    if step is None and orbax_tree.find_state_dir(cand) is None and latest_step(path) is not None:
      cand = get_checkpoint_dir(path, latest_step(path))
    tree_dir = orbax_tree.find_state_dir(cand)
  if tree_dir is not None:
    ckpt_dir = tree_dir
    contents = {"version": VERSION, "optimizer": _orbax_state_dict(tree_dir)}
  else:
    ckpt_file = find_checkpoint(path, step)
    ckpt_dir = os.path.dirname(ckpt_file)
    with open(ckpt_file, "rb") as fp:
      contents = msgpack_io.msgpack_restore(fp.read())
  version = contents.get("version", 0)
  state_dict = _get_optimizer_state_dict(contents, {}, state_transformation_fns)
  rd = _np_dtype(restore_dtype)
  flat = state_utils.flatten_state_dict(state_dict, keep_empty_nodes=True)
  out = {}
  for name, leaf in flat.items():
    if isinstance(leaf, orbax_tree.ArrayRef):
      dt = rd if name.split("/")[0] == "target" else None
      get = functools.partial(leaf.read, None, dt)
      out[name] = LazyArray(leaf.shape or (), dt or leaf.dtype or "float32", get) \
          if lazy_parameters else get()
    elif _is_spec(leaf):
      dt = rd if name.split("/")[0] == "target" else None
      shape = tuple(leaf.get("metadata", {}).get("shape", ()))
      get = functools.partial(_read_ts, leaf, ckpt_dir, None, None, dt, version, name)
      out[name] = LazyArray(shape, dt or leaf.get("dtype", "float32"), get) if lazy_parameters \
          else get()
    else:
      out[name] = leaf
  return tree_utils.unflatten_dict(out)


# ----------------------------------------------------------------------------
# Keep-best checkpointer
# ----------------------------------------------------------------------------
def _get_metrics_from_events(summary_dir: str, metric_name: str):
  """{step: value} of a scalar tag read from TensorBoard event files."""
  from t5x_b200.utils import metric_writers
  scalars = metric_writers.read_scalars(summary_dir)
  return {int(s): float(v) for s, v in scalars.get(metric_name, [])}


def populate_metrics_for_steps(checkpoints_dir: str, metric_name: str,
                               steps: Sequence[int]) -> Mapping[int, float]:
  """Metric value per checkpoint step; `metric_name` is '<summary subdir>/<tag>'
  (t5x/checkpoints.py:1385-1457)."""
  parts = metric_name.split("/")
  for split in range(len(parts) - 1, 0, -1):
    d = os.path.join(checkpoints_dir, *parts[:split])
    if os.path.isdir(d):
      vals = _get_metrics_from_events(d, "/".join(parts[split:]))
      return {s: vals[s] for s in steps if s in vals}
  return {}


class SaveBestCheckpointer(Checkpointer):
  """Keeps the `keep` best checkpoints by a monitored TensorBoard metric, plus the latest
  (t5x/checkpoints.py:1462-1612)."""

  def __init__(self, train_state, partitioner, checkpoints_dir, dataset_iterator=None, *,
               keep: Optional[int] = None, save_dtype=np.float32, restore_dtype=None,
               metric_name_to_monitor: str = "train/accuracy", metric_mode: str = "max",
               keep_checkpoints_without_metrics: bool = True,
               force_keep_period: Optional[int] = None, keep_dataset_checkpoints=None):
    super().__init__(train_state, partitioner, checkpoints_dir, dataset_iterator, keep=keep,
                     save_dtype=save_dtype, restore_dtype=restore_dtype,
                     keep_dataset_checkpoints=keep_dataset_checkpoints)
    if metric_mode not in ("max", "min"):
      raise ValueError('Unsupported `metric_mode`: %s' % metric_mode)
    self._metric_name_to_monitor = metric_name_to_monitor
    self._metric_mode = metric_mode
    self._keep_checkpoints_without_metrics = keep_checkpoints_without_metrics
    self._force_keep_period = force_keep_period

  def _filter_out_force_keep_period_steps(self, steps):
    if self._force_keep_period is None:
      return steps
    return [s for s in steps if s % self._force_keep_period != 0]

  def _remove_old_checkpoints(self):
    if not self.keep:
      return
    existing = self.all_steps()
    if len(existing) <= self.keep:
      return
    latest, existing = existing[-1], existing[:-1]  # the latest is always kept
    existing = self._filter_out_force_keep_period_steps(existing)
    metrics = populate_metrics_for_steps(self.checkpoints_dir, self._metric_name_to_monitor,
                                         existing)
    with_metrics = [s for s in existing if s in metrics]
    without = [s for s in existing if s not in metrics]
    with_metrics.sort(key=lambda s: metrics[s], reverse=(self._metric_mode == "max"))
    n_keep = max(0, self.keep - 1)
    if self._keep_checkpoints_without_metrics:
      to_remove = with_metrics[n_keep:]
    else:
      to_remove = with_metrics[n_keep:] + without
    for step in to_remove:
      checkpoint_utils.remove_checkpoint_dir(get_checkpoint_dir(self.checkpoints_dir, step))


# ----------------------------------------------------------------------------
# Checkpoint-manager interface
# ----------------------------------------------------------------------------
class OrbaxCheckpointManagerInterface:
  """The checkpoint-manager call surface `train()` drives (t5x/checkpoints.py:2211-2550):
  `should_save / save / restore / wait_until_finished / close`, save period and explicit steps,
  keep / keep-best policy. Saves use the native T5X format (the published interchange
  format); restores also read Orbax PyTree directories that are not OCDBT-packed
  (`io/orbax_tree.py`)."""

  def __init__(self, directory: str, train_state, partitioner, dataset_iterator=None,
               save_dtype=None, restore_dtype=None, keep: Optional[int] = None, period: int = 1,
               checkpoint_steps: Optional[Sequence[int]] = None,
               keep_dataset_checkpoints: Optional[int] = None,
               force_keep_period: Optional[int] = None,
               metric_name_to_monitor: Optional[str] = None, metric_mode: str = "max",
               keep_checkpoints_without_metrics: bool = True):
    # A manager built only to restore (evaluation, inference) has no directory of its own.
    self._directory = os.fspath(directory) if directory is not None else ""
    self._period = period or 1
    self._checkpoint_steps = set(checkpoint_steps or ())
    kwargs = dict(keep=keep, save_dtype=save_dtype or np.float32, restore_dtype=restore_dtype,
                  keep_dataset_checkpoints=keep_dataset_checkpoints)
    if metric_name_to_monitor is not None:
      self._checkpointer = SaveBestCheckpointer(
          train_state, partitioner, self._directory, dataset_iterator,
          metric_name_to_monitor=metric_name_to_monitor, metric_mode=metric_mode,
          keep_checkpoints_without_metrics=keep_checkpoints_without_metrics,
          force_keep_period=force_keep_period, **kwargs)
    else:
      self._checkpointer = Checkpointer(train_state, partitioner, self._directory,
                                        dataset_iterator, **kwargs)
    self._pool = concurrent.futures.ThreadPoolExecutor(max_workers=1)
    self._pending: Optional[concurrent.futures.Future] = None

  @property
  def directory(self):
    return self._directory

  def all_steps(self):
    return self._checkpointer.all_steps()

  def latest_step(self):
    return self._checkpointer.latest_step()

  def should_save(self, step: int) -> bool:
    return step % self._period == 0 or step in self._checkpoint_steps

  def save(self, train_state, state_transformation_fns=(), force: bool = True) -> bool:
    step = int(_to_numpy(train_state.step))
    if not force and not self.should_save(step):
      return False
    self.wait_until_finished()
    self._checkpointer.save(train_state, state_transformation_fns)
    return True

  def restore(self, step: Optional[int] = None, path: Optional[str] = None,
              fallback_state=None, state_transformation_fns=(), lazy_parameters: bool = False):
    return self._checkpointer.restore(step=step, path=path,
                                      state_transformation_fns=state_transformation_fns,
                                      fallback_state=fallback_state,
                                      lazy_parameters=lazy_parameters)

  def wait_until_finished(self):
    if self._pending is not None:
      self._pending.result()
      self._pending = None

  def close(self):
    self.wait_until_finished()
    self._pool.shutdown(wait=True)


CheckpointManagerConstructor = Callable[..., OrbaxCheckpointManagerInterface]
