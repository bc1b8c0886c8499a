"""Configuration helpers shared by the entry points (role of t5x/config_utils.py).

A launcher is configured either by gin (`--gin_file`, `--gin.NAME=value`) or by buildable
configs (`t5x_b200.fdl`, the Fiddle-style interface):

  --fdl_config=package.module:function        call `function()` -> a config of the launcher
  --fdl_config='package.module:function(a=1)' the same with literal keyword arguments
  --fdl_config_file=path.json                  a config written by `fdl.dump_json`
  --fdl_set=path.to.argument=value             any number of literal overrides, applied in order
  --fdl_help                                   print the resolved config and exit

`config_with_fiddle(function, flags)` turns those flags into an `fdl.Partial` of `function`
(building it gives the launcher call without running it); `run(main)` is the launcher used by
the entry points' `__main__` blocks.
"""
from __future__ import annotations

import ast
import copy
import importlib
import logging
import os
from typing import Any, Callable, Optional, Sequence

from t5x_b200 import fdl
from t5x_b200 import gin_utils


def add_flags(parser) -> None:
  """The buildable-config flags, added to an argparse parser of an entry point."""
  parser.add_argument("--fdl_config", default=None,
                      help="module:function returning the launcher's config.")
  parser.add_argument("--fdl_config_file", default=None, help="JSON file written by fdl.dump_json.")
  parser.add_argument("--fdl_set", action="append", default=[],
                      help="path.to.argument=value override (repeatable).")
  parser.add_argument("--fdl_help", action="store_true", help="Print the config and exit.")


def using_fdl(flags=None) -> bool:
  """True if any buildable-config flag is set."""
  if flags is None:
    return False
  return bool(getattr(flags, "fdl_config", None) or getattr(flags, "fdl_config_file", None) or
              getattr(flags, "fdl_help", False))


def _select_summarizers(config):
  return fdl.select(config, direct_summarize_fiddle_config)


def prepare_to_summarize(config: fdl.Buildable) -> fdl.Buildable:
  """A copy of `config` whose `summarize_fiddle_config` partials can reach the config they
  are part of (through a getter, so the config does not contain itself)."""
  new_config = copy.deepcopy(config)
  for node in _select_summarizers(new_config):
    node.get_current_fiddle_config = lambda: config
  return new_config


def sanitize_summary_getter(config: fdl.Buildable) -> fdl.Buildable:
  """A copy of `config` without those getters (for printing and serialising)."""
  new_config = copy.deepcopy(config)
  for node in _select_summarizers(new_config):
    node.get_current_fiddle_config = None
  return new_config


def direct_summarize_fiddle_config(model_dir: str, summary_writer: Optional[Any], step: int,
                                   get_current_fiddle_config: Optional[Callable[[], Any]] = None
                                   ) -> None:
  """Writes the config to `<model_dir>/fiddle_config.txt` (and `.json` when every leaf has a
  JSON form) and to the summary writer (t5x/config_utils.py:67-118). Pass the `fdl.Partial`
  `summarize_fiddle_config` as a launcher's `summarize_config_fn`."""
  from t5x_b200.parallel import state as pstate
  if pstate.get().rank != 0:
    return
  if not get_current_fiddle_config:
    raise ValueError("get_current_fiddle_config() not provided. Pass the config through "
                     "config_utils.prepare_to_summarize before building it.")
  config = sanitize_summary_getter(get_current_fiddle_config())
  config_str = str(config)
  os.makedirs(model_dir, exist_ok=True)
  with open(os.path.join(model_dir, "fiddle_config.txt"), "w") as f:
    f.write(config_str)
  try:
    with open(os.path.join(model_dir, "fiddle_config.json"), "w") as f:
      f.write(fdl.dump_json(config))
  except fdl.UnserializableValueError as e:
    os.remove(os.path.join(model_dir, "fiddle_config.json"))
    logging.warning("Unable to serialise the config to JSON, skipping. Error: %s", e)
  if summary_writer is not None:
    summary_writer.write_texts(step, {"fiddle_config": config_str})
    summary_writer.flush()


summarize_fiddle_config = fdl.Partial(direct_summarize_fiddle_config)


def _config_from_spec(spec: str) -> Any:
  """'pkg.module:fn', 'pkg.module.fn' or either with '(k=literal, ...)' -> fn(**kwargs)."""
  call_args = {}
  if spec.rstrip().endswith(")") and "(" in spec:
    spec, _, arg_text = spec.rstrip()[:-1].partition("(")
    tree = ast.parse(f"f({arg_text})", mode="eval").body
    if tree.args:
      raise ValueError(f"--fdl_config takes keyword arguments only, got {arg_text!r}")
    call_args = {kw.arg: ast.literal_eval(kw.value) for kw in tree.keywords}
  if ":" in spec:
    module_name, _, attr = spec.partition(":")
  else:
    module_name, _, attr = spec.rpartition(".")
  if not module_name or not attr:
    raise ValueError(f"--fdl_config wants module:function, got {spec!r}")
  obj = importlib.import_module(module_name)
  for part in attr.split("."):
    obj = getattr(obj, part)
  return obj(**call_args) if callable(obj) and not isinstance(obj, fdl.Buildable) else obj


def config_with_fiddle(function: Callable[..., Any], flags) -> fdl.Buildable:
  """An `fdl.Partial` of `function` from the buildable-config flags
  (t5x/config_utils.py:125-201). Raises ValueError if gin flags are mixed in, if both a config
  function and a config file are given, or if the config configures another function."""
  assert using_fdl(flags), "No buildable-config command line flags found"
  has_gin = bool(getattr(flags, "gin_file", None) or getattr(flags, "gin_bindings", None))
  if (flags.fdl_config_file or flags.fdl_config) and has_gin:
    raise ValueError("Must pass exactly one of `--fdl_config_file`, `--fdl_config`, or "
                     f"`--gin_file` / `--gin_bindings`. Got: --fdl_config_file="
                     f"{flags.fdl_config_file} --fdl_config={flags.fdl_config} "
                     f"--gin_file={flags.gin_file} --gin_bindings={flags.gin_bindings}.")
  if flags.fdl_config_file and flags.fdl_config:
    raise ValueError("Must pass exactly one of `--fdl_config_file` or `--fdl_config`. Got: "
                     f"--fdl_config_file={flags.fdl_config_file} "
                     f"--fdl_config={flags.fdl_config}.")
  if flags.fdl_config_file:
    with open(flags.fdl_config_file) as f:
      config = fdl.load_json(f.read())
  elif flags.fdl_config:
    config = _config_from_spec(flags.fdl_config)
  else:
    raise ValueError("--fdl_help needs --fdl_config or --fdl_config_file to have a config to "
                     "show")
  if not isinstance(config, fdl.Buildable):
    raise ValueError(f"the configured object is {type(config).__name__}, not a buildable config")
  for assignment in flags.fdl_set:
    path, eq, text = assignment.partition("=")
    if not eq:
      raise ValueError(f"--fdl_set wants path=value, got {assignment!r}")
    try:
      value = ast.literal_eval(text)
    except (ValueError, SyntaxError):
      value = text
    fdl.set_by_path(config, path.strip(), value)
  # Config[function] would run the launcher when built: make it a Partial
  config = fdl.cast(fdl.Partial, config)
  got, want = fdl.get_callable(config), function
  if getattr(got, "__qualname__", None) != getattr(want, "__qualname__", None) or \
      getattr(got, "__module__", None) not in (getattr(want, "__module__", None), "__main__") and \
      getattr(want, "__module__", None) != "__main__":
    name = lambda fn: ".".join((getattr(fn, "__module__", "?"), getattr(fn, "__qualname__", "?")))
    raise ValueError(f"Expected the flags to configure function {name(want)} but they "
                     f"configured {name(got)}.\n\nConfig: {config}")
  return prepare_to_summarize(config)


def run_with_fiddle(function: Callable[..., Any], flags) -> Any:
  """Resolves the flags and runs the launcher (or prints the config for `--fdl_help`)."""
  config = config_with_fiddle(function, flags)
  if flags.fdl_help:
    print(sanitize_summary_getter(config))
    return None
  return fdl.build(config)()


def run(main: Callable[[Sequence[str]], None]) -> None:
  """Runs `main(argv)` after rewriting `--gin.NAME=value` flags into gin bindings."""
  gin_utils.run(main)
