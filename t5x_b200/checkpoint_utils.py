"""Pinned checkpoints and checkpoint-type detection (API of t5x/checkpoint_utils.py)."""
from __future__ import annotations

import enum
import glob
import logging
import os
import shutil
from typing import Any, Optional

from t5x_b200.io import msgpack_io
from t5x_b200.io import orbax_tree

_PINNED_CHECKPOINT_FILENAME = "PINNED"
_TS_KEYS = {"driver", "kvstore", "metadata"}


def pinned_checkpoint_filepath(ckpt_dir: str) -> str:
  return os.path.join(ckpt_dir, _PINNED_CHECKPOINT_FILENAME)


def is_pinned_checkpoint(ckpt_dir: str) -> bool:
  """A pinned checkpoint is exempt from the keep-N garbage collection."""
  return os.path.exists(pinned_checkpoint_filepath(ckpt_dir))


def pin_checkpoint(ckpt_dir: str, txt: str = "1") -> None:
  with open(pinned_checkpoint_filepath(ckpt_dir), "w") as f:
    f.write(txt)


def unpin_checkpoint(ckpt_dir: str) -> None:
  if not is_pinned_checkpoint(ckpt_dir):
    return
  try:
    os.remove(pinned_checkpoint_filepath(ckpt_dir))
  except OSError:
    logging.exception("Failed to unpin %s", ckpt_dir)


def remove_checkpoint_dir(ckpt_dir: str) -> None:
  if not is_pinned_checkpoint(ckpt_dir):
    logging.info("Deleting checkpoint: %s", ckpt_dir)
    shutil.rmtree(ckpt_dir, ignore_errors=True)
  else:
    logging.info("Keeping pinned checkpoint: %s", ckpt_dir)


def remove_dataset_checkpoint(ckpt_dir: str, train_ds_prefix: str) -> None:
  if not is_pinned_checkpoint(ckpt_dir):
    for fn in glob.glob(os.path.join(ckpt_dir, train_ds_prefix + "*")):
      os.remove(fn)
  else:
    logging.info("Keeping pinned checkpoint: %s", ckpt_dir)


class CheckpointTypes(enum.Enum):
  ORBAX = "ORBAX"
  T5X = "T5X"
  T5X_TF = "T5X_TF"


def _contains_ts_spec(tree: Any) -> bool:
  """True when any subtree looks like a serialised TensorStore spec."""
  if isinstance(tree, dict):
    if set(tree.keys()) >= _TS_KEYS:
      return True
    return any(_contains_ts_spec(v) for v in tree.values())
  return False


def _contains_ocdbt(path: str) -> bool:
  d = path if os.path.isdir(path) else os.path.dirname(path)
  return any(os.path.exists(os.path.join(d, n)) for n in ("manifest.ocdbt", "_METADATA",
                                                          "_CHECKPOINT_METADATA"))


def detect_checkpoint_type(checkpoint_path: str,
                           expected: Optional[CheckpointTypes] = None) -> CheckpointTypes:
  """Sniffs the on-disk format: an Orbax directory, a native T5X checkpoint (msgpack index with
  TensorStore specs) or a TensorFlow checkpoint (t5x/checkpoint_utils.py:101-250)."""
  found = None
  d = checkpoint_path if os.path.isdir(checkpoint_path) else os.path.dirname(checkpoint_path)
  if _contains_ocdbt(checkpoint_path) or os.path.isdir(os.path.join(d, "state")) or \
      orbax_tree.find_state_dir(d) is not None:
    found = CheckpointTypes.ORBAX
  else:
    f = checkpoint_path if os.path.isfile(checkpoint_path) else os.path.join(d, "checkpoint")
    try:
      with open(f, "rb") as fp:
        tree = msgpack_io.msgpack_restore(fp.read())
      if isinstance(tree, dict) and ("optimizer" in tree or _contains_ts_spec(tree)):
        found = CheckpointTypes.T5X
    except Exception:  # not msgpack: a TF checkpoint's text `checkpoint` file or data shards
      found = None
    if found is None:
      if glob.glob(os.path.join(d, "*.index")) or glob.glob(checkpoint_path + ".index"):
        found = CheckpointTypes.T5X_TF
      else:
        found = expected or CheckpointTypes.T5X
  if expected is not None and found != expected:
    logging.warning("Expected the checkpoint at %s to be %s format, but detected %s.",
                    checkpoint_path, expected, found)
  return found
