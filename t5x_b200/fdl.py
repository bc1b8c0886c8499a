"""Buildable configuration objects: the Fiddle-style alternative to gin for the launchers
(role of the `fiddle` package as the reference uses it: t5x/config_utils.py,
t5x/fiddle_configs/**).

A `Config(fn_or_cls, **arguments)` is a mutable description of a call; `build(config)` makes the
call, building nested configs first (a config object that appears in several places is built
once and shared). `Partial` builds to a callable that still accepts arguments. An `ArgFactory`
is only meaningful inside a `Partial`: it is called anew on every call of the built partial
(a fresh learning-rate schedule per trainer, say).

    cfg = fdl.Config(train, model=fdl.Config(EncoderDecoderModel, ...), total_steps=10)
    cfg.total_steps = 20
    cfg.model.z_loss = 1e-4
    fdl.build(cfg)        # train(model=EncoderDecoderModel(...), total_steps=20)

This is an independent, small implementation of that interface (no dependency on the fiddle
package): argument names are checked against the callable's signature, values can be read,
set and deleted as attributes, configs compare, copy, print and round-trip through JSON when
their leaves are plain values.
"""
from __future__ import annotations

import copy
import functools
import importlib
import inspect
import json
from typing import Any, Callable, Dict, Mapping

_RESERVED = ("__fn_or_cls__", "__arguments__", "__signature__")


class UnserializableValueError(ValueError):
  """A config holds a value that has no JSON form (a lambda, a tensor, an open file...)."""


class Buildable:
  """Arguments bound to a callable, not yet called."""

  def __init__(self, fn_or_cls: Callable[..., Any], *args, **kwargs):
    if isinstance(fn_or_cls, Buildable):
      raise TypeError("the first argument is the function or class to configure, not a config; "
                      "use fdl.cast() to change the kind of an existing config")
    object.__setattr__(self, "__fn_or_cls__", fn_or_cls)
    try:
      sig = inspect.signature(fn_or_cls)
    except (TypeError, ValueError):
      sig = None
    object.__setattr__(self, "__signature__", sig)
    arguments: Dict[str, Any] = {}
    if sig is not None:
      bound = sig.bind_partial(*args, **kwargs)
      for name, value in bound.arguments.items():
        kind = sig.parameters[name].kind
        if kind is inspect.Parameter.VAR_KEYWORD:
          arguments.update(value)
        elif kind is inspect.Parameter.VAR_POSITIONAL:
          raise TypeError("variadic positional arguments cannot be configured")
        else:
          arguments[name] = value
    else:
      if args:
        raise TypeError(f"{fn_or_cls!r} has no inspectable signature: pass keyword arguments")
      arguments.update(kwargs)
    object.__setattr__(self, "__arguments__", arguments)

  # -- attribute access -----------------------------------------------------------------------
  def _check_name(self, name: str) -> None:
    sig = self.__signature__
    if sig is None or name in sig.parameters:
      if sig is not None and sig.parameters[name].kind in (inspect.Parameter.VAR_POSITIONAL,
                                                           inspect.Parameter.VAR_KEYWORD):
        raise AttributeError(f"{name!r} is a variadic parameter of {_name(self.__fn_or_cls__)}")
      return
    if any(p.kind is inspect.Parameter.VAR_KEYWORD for p in sig.parameters.values()):
      return
    raise AttributeError(f"{_name(self.__fn_or_cls__)} has no parameter {name!r}; it takes "
                         f"{list(sig.parameters)}")

  def __getattr__(self, name: str) -> Any:
    if name in _RESERVED or name.startswith("__"):
      raise AttributeError(name)
    arguments = object.__getattribute__(self, "__arguments__")
    if name in arguments:
      return arguments[name]
    self._check_name(name)
    default = self.__signature__.parameters[name].default if self.__signature__ is not None and \
        name in self.__signature__.parameters else inspect.Parameter.empty
    if default is inspect.Parameter.empty:
      raise AttributeError(f"no value has been set for {name!r} of "
                           f"{_name(self.__fn_or_cls__)} and it has no default")
    return default

  def __setattr__(self, name: str, value: Any) -> None:
    self._check_name(name)
    self.__arguments__[name] = value

  def __delattr__(self, name: str) -> None:
    try:
      del self.__arguments__[name]
    except KeyError:
      raise AttributeError(f"{name!r} has not been set") from None

  # -- value semantics ------------------------------------------------------------------------
  def __eq__(self, other: Any) -> bool:
    return (type(self) is type(other) and self.__fn_or_cls__ is other.__fn_or_cls__ and
            self.__arguments__ == other.__arguments__)

  __hash__ = object.__hash__

  def __deepcopy__(self, memo):
    new = type(self).__new__(type(self))
    memo[id(self)] = new
    object.__setattr__(new, "__fn_or_cls__", self.__fn_or_cls__)
    object.__setattr__(new, "__signature__", self.__signature__)
    object.__setattr__(new, "__arguments__", copy.deepcopy(self.__arguments__, memo))
    return new

  def __copy__(self):
    new = type(self).__new__(type(self))
    object.__setattr__(new, "__fn_or_cls__", self.__fn_or_cls__)
    object.__setattr__(new, "__signature__", self.__signature__)
    object.__setattr__(new, "__arguments__", dict(self.__arguments__))
    return new

  def __repr__(self) -> str:
    return _format(self, 0)


class Config(Buildable):
  """Builds to the result of the call."""


class Partial(Buildable):
  """Builds to a callable: `functools.partial` of the callable over the built arguments, with
  `ArgFactory` arguments evaluated on every call."""


class ArgFactory(Buildable):
  """Inside a `Partial` (at any depth of its containers): a value made fresh per call."""


Buildable_ = Buildable  # alias for annotations in configs


def _name(fn: Any) -> str:
  return getattr(fn, "__qualname__", None) or getattr(fn, "__name__", None) or repr(fn)


def _format(value: Any, indent: int) -> str:
  pad = "  " * (indent + 1)
  if isinstance(value, Buildable):
    if not value.__arguments__:
      return f"<{type(value).__name__}[{_name(value.__fn_or_cls__)}()]>"
    lines = [f"<{type(value).__name__}[{_name(value.__fn_or_cls__)}("]
    for k, v in value.__arguments__.items():
      lines.append(f"{pad}{k}={_format(v, indent + 1)},")
    lines.append("  " * indent + ")]>")
    return "\n".join(lines)
  if isinstance(value, Mapping) and any(isinstance(v, Buildable) for v in value.values()):
    inner = ", ".join(f"{k!r}: {_format(v, indent + 1)}" for k, v in value.items())
    return "{" + inner + "}"
  if isinstance(value, (list, tuple)) and any(isinstance(v, Buildable) for v in value):
    inner = ", ".join(_format(v, indent + 1) for v in value)
    return ("[" + inner + "]") if isinstance(value, list) else ("(" + inner + ",)")
  return repr(value)


# ----------------------------------------------------------------------------
# build
# ----------------------------------------------------------------------------
class _PartialWithFactories:
  """The callable a `Partial` with `ArgFactory` arguments builds to."""

  def __init__(self, fn, arguments: Dict[str, Any]):
    self.func, self._arguments = fn, arguments
    functools.update_wrapper(self, fn, updated=())

  def __call__(self, *args, **kwargs):
    made = {k: _call_factories(v) for k, v in self._arguments.items()}
    made.update(kwargs)
    return self.func(*args, **made)


class _Factory:
  def __init__(self, fn, arguments):
    self.fn, self.arguments = fn, arguments

  def __call__(self):
    return self.fn(**{k: _call_factories(v) for k, v in self.arguments.items()})


def _call_factories(value: Any) -> Any:
  if isinstance(value, _Factory):
    return value()
  if isinstance(value, dict):
    return {k: _call_factories(v) for k, v in value.items()}
  if isinstance(value, list):
    return [_call_factories(v) for v in value]
  if isinstance(value, tuple):
    return tuple(_call_factories(v) for v in value)
  return value


def _has_factory(value: Any) -> bool:
  if isinstance(value, _Factory):
    return True
  if isinstance(value, dict):
    return any(_has_factory(v) for v in value.values())
  if isinstance(value, (list, tuple)):
    return any(_has_factory(v) for v in value)
  return False


def build(value: Any, _memo: Dict[int, Any] = None) -> Any:
  """Builds a config (or every config inside a dict / list / tuple). A config object reached
  twice is built once; its result is shared."""
  memo = {} if _memo is None else _memo
  if isinstance(value, Buildable):
    if id(value) in memo:
      return memo[id(value)]
    arguments = {k: build(v, memo) for k, v in value.__arguments__.items()}
    fn = value.__fn_or_cls__
    if isinstance(value, ArgFactory):
      out = _Factory(fn, arguments)
    elif isinstance(value, Partial):
      out = (_PartialWithFactories(fn, arguments) if _has_factory(arguments)
             else functools.partial(fn, **arguments))
    else:
      if _has_factory(arguments):
        raise ValueError(f"ArgFactory inside Config[{_name(fn)}]: factories are only evaluated "
                         "by a Partial that contains them")
      try:
        out = fn(**arguments)
      except TypeError as e:
        raise TypeError(f"while building {_name(fn)}: {e}") from e
    memo[id(value)] = out
    return out
  if isinstance(value, dict):
    return {k: build(v, memo) for k, v in value.items()}
  if isinstance(value, list):
    return [build(v, memo) for v in value]
  if isinstance(value, tuple) and not hasattr(value, "_fields"):
    return tuple(build(v, memo) for v in value)
  return value


def cast(kind: type, buildable: Buildable) -> Buildable:
  """The same callable and arguments as another kind of buildable (Config <-> Partial)."""
  if not (isinstance(kind, type) and issubclass(kind, Buildable)):
    raise TypeError(f"{kind!r} is not a kind of buildable")
  new = kind.__new__(kind)
  object.__setattr__(new, "__fn_or_cls__", buildable.__fn_or_cls__)
  object.__setattr__(new, "__signature__", buildable.__signature__)
  object.__setattr__(new, "__arguments__", dict(buildable.__arguments__))
  return new


def get_callable(buildable: Buildable) -> Callable[..., Any]:
  return buildable.__fn_or_cls__


def select(root: Any, fn_or_cls: Callable[..., Any]):
  """Every buildable under `root` (inclusive) that configures `fn_or_cls`."""
  found, seen = [], set()

  def walk(v):
    if id(v) in seen:
      return
    seen.add(id(v))
    if isinstance(v, Buildable):
      if v.__fn_or_cls__ is fn_or_cls:
        found.append(v)
      for a in v.__arguments__.values():
        walk(a)
    elif isinstance(v, dict):
      for a in v.values():
        walk(a)
    elif isinstance(v, (list, tuple)):
      for a in v:
        walk(a)
  walk(root)
  return found


def set_by_path(root: Buildable, path: str, value: Any) -> None:
  """`set_by_path(cfg, "model.optimizer_def.decay_rate", 0.9)`; `[i]` / `['k']` index
  containers."""
  import re
  tokens = re.findall(r"\.?([A-Za-z_][A-Za-z_0-9]*)|\[([^\]]+)\]", path)
  if not tokens:
    raise ValueError(f"empty path {path!r}")
  node = root
  steps = [(name, None) if name else (None, _literal(idx)) for name, idx in tokens]
  for name, idx in steps[:-1]:
    node = getattr(node, name) if name is not None else node[idx]
  name, idx = steps[-1]
  if name is not None:
    setattr(node, name, value)
  else:
    node[idx] = value


def _literal(text: str) -> Any:
  import ast
  try:
    return ast.literal_eval(text)
  except (ValueError, SyntaxError):
    return text


# ----------------------------------------------------------------------------
# JSON
# ----------------------------------------------------------------------------
def _importable(fn: Any) -> str:
  module, qual = getattr(fn, "__module__", None), getattr(fn, "__qualname__", None)
  if not module or not qual or "<" in qual:
    raise UnserializableValueError(f"{fn!r} cannot be named as module:qualname")
  return f"{module}:{qual}"


def _resolve(name: str) -> Any:
  module, _, qual = name.partition(":")
  obj = importlib.import_module(module)
  for part in qual.split("."):
    obj = getattr(obj, part)
  return obj


def _to_jsonable(value: Any) -> Any:
  if isinstance(value, Buildable):
    return {"__fdl__": type(value).__name__, "fn": _importable(value.__fn_or_cls__),
            "args": {k: _to_jsonable(v) for k, v in value.__arguments__.items()}}
  if value is None or isinstance(value, (bool, int, float, str)):
    return value
  if isinstance(value, (list, tuple)):
    return {"__seq__": "tuple" if isinstance(value, tuple) else "list",
            "items": [_to_jsonable(v) for v in value]}
  if isinstance(value, dict):
    if not all(isinstance(k, str) for k in value):
      raise UnserializableValueError("only string keys have a JSON form")
    return {"__dict__": {k: _to_jsonable(v) for k, v in value.items()}}
  if callable(value) and hasattr(value, "__qualname__"):
    return {"__ref__": _importable(value)}
  raise UnserializableValueError(f"no JSON form for {type(value).__name__}: {value!r}")


def _from_jsonable(value: Any) -> Any:
  if isinstance(value, dict):
    if "__fdl__" in value:
      kind = {"Config": Config, "Partial": Partial, "ArgFactory": ArgFactory}[value["__fdl__"]]
      return kind(_resolve(value["fn"]),
                  **{k: _from_jsonable(v) for k, v in value["args"].items()})
    if "__seq__" in value:
      items = [_from_jsonable(v) for v in value["items"]]
      return tuple(items) if value["__seq__"] == "tuple" else items
    if "__dict__" in value:
      return {k: _from_jsonable(v) for k, v in value["__dict__"].items()}
    if "__ref__" in value:
      return _resolve(value["__ref__"])
  return value


def dump_json(config: Buildable, indent: int = 2) -> str:
  return json.dumps(_to_jsonable(config), indent=indent)


def load_json(text: str) -> Any:
  return _from_jsonable(json.loads(text))


def copy_with(buildable: Buildable, **overrides) -> Buildable:
  """A shallow copy with some arguments replaced."""
  new = copy.copy(buildable)
  for k, v in overrides.items():
    setattr(new, k, v)
  return new
