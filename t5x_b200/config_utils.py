"""Configuration helpers shared by the entry points (role of t5x/config_utils.py).

The reference can be configured either by gin or by Fiddle. Fiddle is not a dependency here:
`using_fdl()` is always False and `config_with_fiddle` raises with a message pointing at gin.
`run(main)` is the single launcher used by the entry points' `__main__` blocks.
"""
from __future__ import annotations

import sys
from typing import Any, Callable, Optional, Sequence

from t5x_b200 import gin_utils


def using_fdl() -> bool:
  return False


def prepare_to_summarize(config: Any) -> Any:
  return config


def sanitize_summary_getter(config: Any) -> Any:
  return config


def direct_summarize_fiddle_config(model_dir: str, summary_writer: Optional[Any], step: int,
                                   get_current_fiddle_config: Callable[[], Any]) -> None:
  raise NotImplementedError("Fiddle configuration is not supported; use gin "
                            "(--gin_file / --gin.NAME=value).")


def config_with_fiddle(function: Callable[..., Any]) -> Any:
  raise NotImplementedError("Fiddle configuration is not supported; use gin "
                            "(--gin_file / --gin.NAME=value).")


def run(main: Callable[[Sequence[str]], None]) -> None:
  """Runs `main(argv)` after rewriting `--gin.NAME=value` flags into gin bindings."""
  gin_utils.run(main)
