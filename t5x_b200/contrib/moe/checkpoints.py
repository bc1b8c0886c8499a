"""Sparse upcycling: initialise a mixture-of-experts model from a dense checkpoint
(t5x/contrib/moe/checkpoints.py:38-320).

`UpcycleCheckpointer` behaves like `Checkpointer` except that a checkpoint array whose shape
equals the target's shape without its leading expert dimension is repeated over that
dimension: every expert starts as a copy of the dense MLP (and of its optimizer slots). The
mapping of names (`.../mlp/expert/wi_0/kernel` <- `.../mlp/wi_0/kernel`) is the usual
`assignment_map` of the restore config; router weights, which a dense checkpoint does not
have, come from `fallback_to_scratch`. Each expert-parallel rank materialises only the
experts it owns."""
from __future__ import annotations

from typing import Any, Optional

import numpy as np

from t5x_b200 import checkpoints
from t5x_b200.io import orbax_tree
from t5x_b200.parallel import state as pstate


class UpcycleCheckpointer(checkpoints.Checkpointer):
  """Checkpointer for dense-to-sparse restores."""

  def __init__(self, train_state, partitioner, checkpoints_dir: str, num_experts: int,
               dataset_iterator=None, *, keep: Optional[int] = None, save_dtype=np.float32,
               restore_dtype=None, keep_dataset_checkpoints: Optional[int] = None):
    super().__init__(train_state, partitioner, checkpoints_dir, dataset_iterator, keep=keep,
                     save_dtype=save_dtype, restore_dtype=restore_dtype,
                     keep_dataset_checkpoints=keep_dataset_checkpoints)
    self._num_experts = num_experts

  def _read_leaf(self, name, ckpt_leaf, target, info, ckpt_dir, version, lazy):
    local_shape = tuple(getattr(target, "shape", ()))
    gshape = tuple(info.shape) if isinstance(info, checkpoints._ParameterInfo) else local_shape
    stored = _stored_shape(ckpt_leaf, ckpt_dir)
    if stored is None or not _needs_broadcast(stored, gshape, self._num_experts):
      return super()._read_leaf(name, ckpt_leaf, target, info, ckpt_dir, version, lazy)
    # dense array: read it whole, then repeat it over this rank's experts
    is_target_param = name.split("/")[0] == "target"
    rd = self.restore_dtype if is_target_param else None
    n_local = local_shape[0]

    def get():
      if isinstance(ckpt_leaf, orbax_tree.ArrayRef):
        dense = ckpt_leaf.read(None, dtype=rd, expected_shape=stored)
      elif checkpoints._is_spec(ckpt_leaf):
        dense = checkpoints._read_ts(ckpt_leaf, ckpt_dir, stored, None, rd, version, name)
      else:
        dense = np.asarray(ckpt_leaf)
        if rd is not None:
          dense = dense.astype(rd)
      return np.repeat(dense[None], n_local, axis=0)

    if lazy:
      dtype = rd or (checkpoints._np_dtype(target.dtype) if hasattr(target, "dtype")
                     else np.float32)
      return checkpoints.LazyArray(local_shape, dtype, get)
    return get()


def _stored_shape(ckpt_leaf, ckpt_dir):
  if isinstance(ckpt_leaf, orbax_tree.ArrayRef):
    return ckpt_leaf.shape
  if checkpoints._is_spec(ckpt_leaf):
    from t5x_b200.io import zarr_io
    return tuple(zarr_io.ZarrArray.open(checkpoints._spec_path(ckpt_leaf, ckpt_dir)).shape)
  if hasattr(ckpt_leaf, "shape"):
    return tuple(ckpt_leaf.shape)
  return None


def _needs_broadcast(stored_shape, global_shape, num_experts: int) -> bool:
  """True when the target is [num_experts, *stored_shape]."""
  return (len(global_shape) == len(stored_shape) + 1 and global_shape[0] == num_experts and
          tuple(global_shape[1:]) == tuple(stored_shape))
