r"""One entry point for every run mode (API of t5x/main.py).

  python -m t5x_b200.main --run_mode=train --gin_file=... --gin.MODEL_DIR=\"/tmp/m\"

`--run_mode` selects the function that gin configures: train, eval, infer, precompile, export.
"""
from __future__ import annotations

import enum
import importlib
import logging
import sys
from typing import Optional, Sequence

from t5x_b200 import gin
from t5x_b200 import gin_utils


@enum.unique
class RunMode(enum.Enum):
  TRAIN = "train"
  EVAL = "eval"
  INFER = "infer"
  PRECOMPILE = "precompile"
  EXPORT = "export"


_MODULE_BY_RUN_MODE = {RunMode.TRAIN: "t5x_b200.train", RunMode.EVAL: "t5x_b200.eval",
                       RunMode.INFER: "t5x_b200.infer", RunMode.PRECOMPILE: "t5x_b200.precompile",
                       RunMode.EXPORT: "t5x_b200.export_lib"}
_ATTR_BY_RUN_MODE = {RunMode.TRAIN: "train", RunMode.EVAL: "evaluate", RunMode.INFER: "infer",
                     RunMode.PRECOMPILE: "precompile", RunMode.EXPORT: "save"}


def main(argv: Optional[Sequence[str]] = None) -> None:
  from t5x_b200 import train as train_lib
  logging.basicConfig(level=logging.INFO)
  argv = gin_utils.rewrite_gin_args(list(sys.argv[1:] if argv is None else argv))
  ap = train_lib.build_flag_parser(__doc__)
  ap.add_argument("--run_mode", required=True, choices=[m.value for m in RunMode],
                  help="The mode to run under.")
  flags = ap.parse_args(argv)
  mode = RunMode(flags.run_mode)
  module = importlib.import_module(_MODULE_BY_RUN_MODE[mode])
  fn = getattr(module, _ATTR_BY_RUN_MODE[mode])
  train_lib.init_distributed_from_flags(flags)
  gin.set_main_module(module)
  train_lib.parse_gin_from_flags(flags, train_lib._DEFAULT_GIN_SEARCH_PATHS)
  if flags.dry_run:
    logging.info("Dry run for mode %s: configuration parsed.\n%s", mode.value, gin.config_str())
    return
  gin.get_configurable(fn)()


if __name__ == "__main__":
  main()
