"""Utilities for restructuring optimizer state dicts (API of t5x/state_utils.py)."""
from __future__ import annotations

import logging
import re
from typing import Any, Mapping, Optional, Sequence, Tuple

from t5x_b200.utils import tree as tree_utils


def tensorstore_leaf(_, value) -> bool:
  """True when `value` is a serialised TensorStore spec dict (a leaf, not a subtree)."""
  return isinstance(value, Mapping) and set(value.keys()) >= {"driver", "kvstore", "metadata"}


def _is_leaf(x) -> bool:
  return not isinstance(x, Mapping) or tensorstore_leaf(None, x)


def flatten_state_dict(state_dict, keep_empty_nodes: bool = False):
  """Flattens to '/'-joined keys, stopping at arrays and TensorStore specs."""
  return tree_utils.flatten_dict(state_dict, sep="/", keep_empty_nodes=keep_empty_nodes,
                                 is_leaf=_is_leaf)


def get_name_tree(state_dict, keep_empty_nodes: bool = False):
  """Same tree with every leaf replaced by its '/'-joined path."""
  flat = tree_utils.flatten_dict(state_dict, keep_empty_nodes=keep_empty_nodes)
  return tree_utils.unflatten_dict({k: k for k in flat})


def intersect_state(state_dict: Mapping[str, Any], intersect_state_dict: Mapping[str, Any]):
  """Drops entries of `state_dict` that are absent from `intersect_state_dict`."""
  flat = flatten_state_dict(state_dict)
  keep = flatten_state_dict(intersect_state_dict)
  for k in list(flat):
    if k not in keep:
      flat.pop(k)
      logging.warning("Not restoring param=%s because it's missing in the checkpoint", k)
  return tree_utils.unflatten_dict(flat)


def merge_state(state_dict: Mapping[str, Any], from_scratch_state: Mapping[str, Any],
                overwrite: bool = False):
  """Inserts entries of `from_scratch_state` that `state_dict` lacks (or all, if overwrite)."""
  flat = flatten_state_dict(state_dict)
  scratch = flatten_state_dict(from_scratch_state)
  for k, v in scratch.items():
    if k not in flat or overwrite:
      logging.warning("Initializing param=%s from scratch", k)
      flat[k] = v
  return tree_utils.unflatten_dict(flat)


def apply_assignment_map(ckpt_optimizer_state, optimizer_state,
                         assignment_map: Sequence[Tuple[str, Optional[str]]],
                         require_all_rules_match: bool = True, *, is_resuming: bool = False):
  """Renames checkpoint entries to the current model's names by regex rules.

  For each key of the current optimizer state, the first rule whose pattern fully matches it
  decides: a `None` replacement drops the key, otherwise the expanded replacement names the
  checkpoint entry to take. Checkpoint keys not consumed by any rule are kept; current keys
  without a rule are copied when the checkpoint has them (t5x/state_utils.py:128-238).
  """
  if is_resuming:
    return ckpt_optimizer_state
  flat_ckpt = flatten_state_dict(ckpt_optimizer_state)
  unmapped_old = dict(flat_ckpt)
  result = {}
  skipped = set()
  flat_opt = flatten_state_dict(optimizer_state)
  used = set()
  for k in flat_opt:
    for pattern, repl in assignment_map:
      m = re.fullmatch(pattern, k)
      if not m:
        continue
      used.add(pattern)
      if repl is None:
        skipped.add(k)
        break
      old_k = m.expand(repl)
      unmapped_old.pop(old_k, None)
      if old_k not in flat_ckpt:
        raise ValueError(f"Parameter '{old_k}' does not exist in restore checkpoint. "
                         f"Must be one of: {sorted(flat_ckpt.keys())}")
      result[k] = flat_ckpt[old_k]
      break
  for key, v in unmapped_old.items():
    if key not in skipped:
      result[key] = v
  for key in set(flat_opt) - set(result):
    if key in skipped:
      continue
    if key in flat_ckpt:
      result[key] = flat_ckpt[key]
    else:
      logging.warning("Skipping key=%s which did not match assignment map or checkpoint.", key)
  if require_all_rules_match and len(assignment_map) != len(used):
    unused = ", ".join(f"'{p}'" for p, _ in assignment_map if p not in used)
    raise ValueError("Unused patterns in `assignment_map`: {" + unused + "}")
  return tree_utils.unflatten_dict(result)
