"""Checkpoint directory naming and step discovery (API of t5x/checkpoints_utils.py)."""
from __future__ import annotations

import glob
import os
import re
from typing import Optional, Sequence, Tuple

_TRAIN_DS_PREFIX = "train_ds"
_CHECKPOINT_PREFIX = "checkpoint"


def get_checkpoint_prefix(prefix: str = _CHECKPOINT_PREFIX) -> str:
  return prefix


def all_steps(checkpoints_dir: str) -> Sequence[int]:
  """Available step numbers, ascending."""
  pat = re.compile(r".*/checkpoint_(\d+)$")
  matches = [pat.match(p) for p in glob.glob(os.path.join(checkpoints_dir, "checkpoint_*"))]
  return sorted(int(m.group(1)) for m in matches if m)


def all_dataset_checkpoint_steps(checkpoints_dir: str) -> Sequence[int]:
  pat = re.compile(r".*/checkpoint_(\d+)/.*$")
  paths = glob.glob(os.path.join(checkpoints_dir, "checkpoint_*", f"{_TRAIN_DS_PREFIX}-*"))
  return sorted({int(m.group(1)) for m in (pat.match(p) for p in paths) if m})


def latest_step(checkpoints_dir: str) -> Optional[int]:
  steps = all_steps(checkpoints_dir)
  return steps[-1] if steps else None


def get_checkpoint_dir(checkpoints_dir: str, step: int,
                       step_format_fixed_length: Optional[int] = None) -> str:
  step_str = f"{step:0{step_format_fixed_length}d}" if step_format_fixed_length else str(step)
  return os.path.join(checkpoints_dir, f"{get_checkpoint_prefix()}_{step_str}")


def get_step_from_checkpoint_dir(checkpoints_dir: str) -> Tuple[str, int]:
  if checkpoints_dir.endswith("/"):
    checkpoints_dir = checkpoints_dir[:-1]
  parent, checkpoint = os.path.split(checkpoints_dir)
  if get_checkpoint_prefix() not in checkpoint:
    raise ValueError("Found improperly formatted checkpoint directory.")
  return parent, int(checkpoint.replace(f"{get_checkpoint_prefix()}_", ""))
