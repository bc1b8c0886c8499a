"""Gin plumbing for the entry points (API of t5x/gin_utils.py)."""
from __future__ import annotations

import logging
import os
from typing import Optional, Sequence, Union

from t5x_b200 import gin
from t5x_b200.parallel import state as pstate


def get_gin_config_str() -> str:
  """Operative config if anything has been used yet, else the full parsed config."""
  op = gin.operative_config_str()
  full = gin.config_str()
  return full if len(full) >= len(op) else op


def parse_gin_flags(gin_search_paths: Sequence[str], gin_files: Sequence[str],
                    gin_bindings: Sequence[str], skip_unknown: Union[bool, Sequence[str]] = False,
                    finalize_config: bool = True) -> None:
  """Parses gin files (later overriding earlier) and then the bindings
  (t5x/gin_utils.py:52-90)."""
  for p in gin_search_paths:
    gin.add_config_file_search_path(p)
  gin.parse_config_files_and_bindings(gin_files, gin_bindings, skip_unknown=bool(skip_unknown),
                                      finalize_config=finalize_config)
  logging.info("Gin Configuration:")
  for line in get_gin_config_str().splitlines():
    logging.info("%s", line)


def rewrite_gin_args(args: Sequence[str]) -> Sequence[str]:
  """`--gin.NAME=VALUE` -> `--gin_bindings=NAME = VALUE` (t5x/gin_utils.py:93-111)."""
  def rewrite(arg):
    if not arg.startswith("--gin."):
      return arg
    if "=" not in arg:
      raise ValueError("Gin bindings must be of the form '--gin.<param>=<value>', got: " + arg)
    name, value = arg[6:].split("=", maxsplit=1)
    return f"--gin_bindings={name} = {value}"
  return [rewrite(a) for a in args]


@gin.register
def summarize_gin_config(model_dir: str, summary_writer, step: int) -> None:
  """Writes `config.gin` into the model dir and the config as a TensorBoard text summary
  (t5x/gin_utils.py:114-130)."""
  if pstate.get().rank != 0:
    return
  config_str = get_gin_config_str()
  os.makedirs(model_dir, exist_ok=True)
  with open(os.path.join(model_dir, "config.gin"), "w") as f:
    f.write(config_str)
  if summary_writer is not None:
    summary_writer.write_texts(step, {"config": gin.markdown(config_str)})
    summary_writer.flush()


def run(main):
  """Runs `main(argv)` after rewriting `--gin.X=Y` flags (t5x/gin_utils.py:133-143)."""
  import sys
  main(rewrite_gin_args(sys.argv))


# ---- gin helper configurables (t5x/gin_utils.py:146-167) ----
@gin.configurable
def sum_fn(var1=gin.REQUIRED, var2=gin.REQUIRED):
  """`@gin_utils.sum_fn()` adds two configured values."""
  return var1 + var2


@gin.configurable
def bool_fn(var1=gin.REQUIRED):
  return bool(var1)


@gin.configurable
def string_split_fn(text=gin.REQUIRED, separator=",", maxsplit=-1, index=None):
  values = text.split(separator, maxsplit)
  return values[index] if index is not None else values
