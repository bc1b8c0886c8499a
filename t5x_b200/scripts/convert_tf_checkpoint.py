"""Converts a Mesh-TensorFlow T5 checkpoint to the native T5X format
(role of t5x/scripts/convert_tf_checkpoint.py:41-84).

  python -m t5x_b200.scripts.convert_tf_checkpoint \\
      --gin_file=t5x/examples/t5/t5_1_0/small.gin \\
      --gin.convert_checkpoint.model=%MODEL \\
      --gin.convert_checkpoint.tf_checkpoint_path=\\"/path/to/model.ckpt-1000000\\" \\
      --gin.convert_checkpoint.output_dir=\\"/tmp/t5x_checkpoints/t5_small\\"

The TensorFlow checkpoint is read by the tensor-bundle reader in `t5x_b200.io.tf_bundle`
(no TensorFlow needed); variable names are mapped by `t5x_b200.checkpoint_importer`.
"""
from __future__ import annotations

import logging
import sys
from typing import Optional, Sequence

import numpy as np

from t5x_b200 import checkpoints
from t5x_b200 import gin
from t5x_b200 import gin_utils
from t5x_b200 import models
from t5x_b200 import partitioning
from t5x_b200 import train_state as train_state_lib


def convert_checkpoint(model: models.BaseModel, tf_checkpoint_path: str, output_dir: str,
                       save_dtype="float32", concurrent_gb: int = 16) -> None:
  """Builds the model's train state (for its names and shapes), fills it from the TensorFlow
  checkpoint and writes it to `output_dir` in the native format, parameters as `save_dtype`."""
  variables = model.get_initial_variables(
      rng=0, input_shapes={"encoder_input_tokens": (1, 1), "decoder_input_tokens": (1, 1)})
  train_state = train_state_lib.FlaxOptimTrainState.create(model.optimizer_def, variables)
  partitioner = partitioning.PjitPartitioner(1)
  checkpointer = checkpoints.Checkpointer(train_state, partitioner, output_dir,
                                          save_dtype=np.dtype(save_dtype))
  checkpointer.convert_from_tf_checkpoint(tf_checkpoint_path, concurrent_gb=concurrent_gb)


def main(argv: Optional[Sequence[str]] = None) -> None:
  from t5x_b200 import train as train_lib
  logging.basicConfig(level=logging.INFO)
  argv = gin_utils.rewrite_gin_args(list(sys.argv[1:] if argv is None else argv))
  flags = train_lib.build_flag_parser(__doc__).parse_args(argv)
  gin.set_main_module(sys.modules[__name__])
  train_lib.parse_gin_from_flags(flags, train_lib._DEFAULT_GIN_SEARCH_PATHS)
  gin.get_configurable(convert_checkpoint)()


if __name__ == "__main__":
  main()
