r"""Ahead-of-time preparation of a training run (role of t5x/precompile.py).

The reference lowers and compiles the partitioned train step and dumps its HLO. Here nothing is
traced: the kernels are sm_100a binaries. "Precompiling" therefore means (1) building the native
library if its binary is stale, (2) constructing the train state shape and its partition specs,
(3) on a GPU, running one throw-away train step on a dummy batch so that TMA tensor maps,
allocator pools and NCCL communicators exist before the first real step, and (4) writing the
launch plan: every parameter with its shape, shard and the GEMM problem sizes of a step.
"""
from __future__ import annotations

import logging
import os
import time
from typing import Callable, Optional

import numpy as np
import torch

from t5x_b200 import models
from t5x_b200 import partitioning
from t5x_b200 import trainer as trainer_lib
from t5x_b200 import utils
from t5x_b200.parallel import state as pstate
from t5x_b200.utils import tree as tree_utils


def precompile(*, model: models.BaseTransformerModel, train_dataset_cfg: utils.DatasetConfig,
               partitioner: partitioning.BasePartitioner, model_dir: str,
               random_seed: Optional[int], get_dataset_fn=utils.get_dataset,
               verify_matching_vocabs_fn: Optional[Callable] = utils.verify_matching_vocabs,
               backend: Optional[str] = None):
  """Builds kernels, warms one step and writes `<model_dir>/launch_plan.txt`."""
  del backend
  from t5x_b200.ops import build as build_lib
  tick = time.time()
  build_lib.build()
  build_seconds = time.time() - tick
  layout = partitioner.get_data_layout(train_dataset_cfg.batch_size)
  if verify_matching_vocabs_fn is not None:
    verify_matching_vocabs_fn(train_dataset_cfg, model)
  ds = get_dataset_fn(train_dataset_cfg, layout.shard_id, layout.num_shards,
                      model.FEATURE_CONVERTER_CLS)
  spec = ds.element_spec
  input_shapes = {k: (layout.batch_size, *v.shape[1:]) for k, v in spec.items()}
  input_types = {k: v.dtype for k, v in spec.items()}
  dummy = {k: np.ones((v.shape[0], *v.shape[1:]), v.dtype) for k, v in spec.items()}
  init = utils.TrainStateInitializer(optimizer_def=model.optimizer_def,
                                     init_fn=model.get_initial_variables,
                                     input_shapes=input_shapes, input_types=input_types,
                                     partitioner=partitioner)
  state = init.from_scratch(random_seed or 42)
  axes = init.train_state_axes
  lines = [f"# native build: {build_seconds:.2f} s", f"# world size: {pstate.get().world_size}",
           f"# per-rank batch: { {k: tuple(v.shape) for k, v in dummy.items()} }", ""]
  flat = tree_utils.flatten_dict(state.params) if isinstance(state.params, dict) else {}
  tokens = int(np.prod(next(iter(dummy.values())).shape[:2]))
  total = 0
  for name, p in sorted(flat.items()):
    shape = tuple(p.shape)
    total += int(np.prod(shape))
    gemm = ""
    if len(shape) == 2:
      gemm = f"  gemm fwd M={tokens} K={shape[0]} N={shape[1]}"
    lines.append(f"{'/'.join(name):<70} {str(shape):<18} shard_dim="
                 f"{getattr(p, 'shard_dim', None)}{gemm}")
  lines.append(f"\n# local parameters: {total}")
  step_seconds = None
  if torch.cuda.is_available():
    trainer_lib.attach_compute_buffers(state.params, bf16_copy=True, main_grad=True)
    batch = {k: torch.from_numpy(v).to(pstate.get().device) for k, v in dummy.items()}
    tick = time.time()
    trainer_lib.train_with_lr(state, batch, learning_rate=0.0, dropout_rng=0, model=model,
                              num_microbatches=None, weight_metrics_computer=None)
    torch.cuda.synchronize()
    step_seconds = time.time() - tick
    lines.append(f"# warm-up step: {step_seconds:.3f} s")
  if pstate.get().rank == 0:
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "launch_plan.txt"), "w") as f:
      f.write("\n".join(lines) + "\n")
  logging.info("Precompile done (build %.2fs, step %s).", build_seconds, step_seconds)
  return {"build_seconds": build_seconds, "step_seconds": step_seconds, "axes": axes}


def main(argv=None) -> None:
  import sys
  from t5x_b200 import gin, gin_utils
  from t5x_b200 import train as train_lib
  logging.basicConfig(level=logging.INFO)
  argv = gin_utils.rewrite_gin_args(list(sys.argv[1:] if argv is None else argv))
  flags = train_lib.build_flag_parser(__doc__).parse_args(argv)
  train_lib.init_distributed_from_flags(flags)
  gin.set_main_module(sys.modules[__name__])
  train_lib.parse_gin_from_flags(flags, train_lib._DEFAULT_GIN_SEARCH_PATHS)
  gin.get_configurable(precompile)()


if __name__ == "__main__":
  main()
