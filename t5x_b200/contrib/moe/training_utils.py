"""Helpers for expert-parallel training (t5x/contrib/moe/training_utils.py)."""
from __future__ import annotations

import re
from typing import Any, Callable, Mapping, Optional

from t5x_b200.utils import tree as tree_utils


def match_fn(prefix: Optional[str]) -> Callable[[str], bool]:
  """Predicate over '/'-joined parameter names: full regex match of `prefix`; a missing
  prefix matches nothing."""
  if not prefix:
    return lambda name: False
  params_regex = re.compile(f"^{prefix}$" if not prefix.startswith("^") else prefix)
  return lambda name: params_regex.match(name) is not None


def tree_map_with_names(f, param_tree, match_name_fn=lambda name: True):
  """Applies `f` to the leaves whose '/'-joined name satisfies `match_name_fn`."""
  flat = tree_utils.flatten_dict(param_tree)
  out = {k: (f(v) if match_name_fn(k) else v) for k, v in flat.items()}
  return tree_utils.unflatten_dict(out)


def scale_sharded_grads(grads: Mapping[str, Any], sharded_match_fn: Optional[Callable[[str], bool]],
                        scale_factor: float):
  """Multiplies the gradients of the matching (expert) parameters by `scale_factor`.

  The reference needs this because a mean over the whole data axis is taken for every
  gradient while expert weights only see the tokens of one expert partition
  (t5x/contrib/moe/training_utils.py:49-73). Here gradients are summed explicitly over the
  groups that replicate a parameter, so the trainer passes a factor of 1 unless asked."""
  if sharded_match_fn is None or scale_factor == 1.0:
    return grads
  return tree_map_with_names(lambda x: x * scale_factor, grads, sharded_match_fn)
