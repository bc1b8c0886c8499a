"""Nested-dict ("pytree") helpers: the containers for params, optimizer state and caches."""
from __future__ import annotations

from typing import Any, Callable, Dict, Mapping, Tuple


def is_leaf_default(x) -> bool:
  return not isinstance(x, Mapping)


def flatten_dict(tree: Mapping[str, Any], sep: str = "/", keep_empty_nodes: bool = False,
                 is_leaf: Callable[[Any], bool] = is_leaf_default) -> Dict[str, Any]:
  """{'a': {'b': x}} -> {'a/b': x} (flax.traverse_util.flatten_dict with a separator)."""
  out: Dict[str, Any] = {}

  def rec(prefix, node):
    if isinstance(node, Mapping) and not is_leaf(node):
      if not node and keep_empty_nodes and prefix:
        out[prefix] = {}
      for k, v in node.items():
        rec(f"{prefix}{sep}{k}" if prefix else str(k), v)
    else:
      out[prefix] = node

  rec("", tree)
  return out


def unflatten_dict(flat: Mapping[str, Any], sep: str = "/") -> Dict[str, Any]:
  out: Dict[str, Any] = {}
  for path, v in flat.items():
    keys = path.split(sep) if isinstance(path, str) else list(path)
    node = out
    for k in keys[:-1]:
      node = node.setdefault(k, {})
    node[keys[-1]] = v
  return out


def tree_map(fn: Callable, tree, *rest, is_leaf: Callable[[Any], bool] = is_leaf_default):
  """Maps over nested dicts (lists/tuples are treated as containers too)."""
  if isinstance(tree, Mapping) and not is_leaf(tree):
    return {k: tree_map(fn, v, *[r[k] for r in rest], is_leaf=is_leaf) for k, v in tree.items()}
  if isinstance(tree, (list, tuple)) and not is_leaf(tree):
    vals = [tree_map(fn, v, *[r[i] for r in rest], is_leaf=is_leaf) for i, v in enumerate(tree)]
    return type(tree)(vals) if not hasattr(tree, "_fields") else type(tree)(*vals)
  return fn(tree, *rest)


def tree_leaves(tree, is_leaf: Callable[[Any], bool] = is_leaf_default):
  out = []
  tree_map(lambda x: out.append(x), tree, is_leaf=is_leaf)
  return out


def flatten_dict_string_keys(x):
  """Flattens with '/'-joined keys (t5x/utils.py flatten_dict_string_keys)."""
  return flatten_dict(x, sep="/")
