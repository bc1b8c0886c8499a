"""Fine-tuning run as a buildable (t5x/fiddle_configs/configs/finetune.py; gin form:
t5x/configs/runs/finetune.gin): restores a specific checkpoint, constant learning rate,
inference evaluation on the validation split."""
from __future__ import annotations

from typing import Mapping, Optional

from t5x_b200 import config_utils, fdl
from t5x_b200 import train as train_lib
from t5x_b200.data import evaluation
from t5x_b200.fiddle_configs.configs import common

BATCH_SIZE = 128
EVAL_STEPS = 20
EVAL_PERIOD = 1000
RANDOM_SEED = None
USE_CACHED_TASKS = True
USE_HARDWARE_RNG = False
JSON_WRITE_N_RESULTS = None  # write every inference result


def train(model: fdl.Buildable, model_dir: Optional[str], train_steps: int,
          mixture_or_task_name: common.MixtureOrTask, task_feature_lengths: Mapping[str, int],
          initial_checkpoint_path: str, eval_steps: int = EVAL_STEPS,
          eval_period: int = EVAL_PERIOD, relative_steps: Optional[int] = None,
          random_seed: Optional[int] = RANDOM_SEED, mixture_or_task_module: Optional[str] = None,
          use_hardware_rng: bool = USE_HARDWARE_RNG, batch_size: int = BATCH_SIZE,
          use_cached_tasks: bool = USE_CACHED_TASKS) -> fdl.Buildable:
  """A configuration of the `train()` launcher for fine-tuning."""
  data = (mixture_or_task_name, task_feature_lengths, batch_size, use_cached_tasks,
          mixture_or_task_module)
  return fdl.Config(
      train_lib.train, model=model, model_dir=model_dir,
      train_dataset_cfg=common.dataset_config("train", *data, shuffle=True, seed=None),
      train_eval_dataset_cfg=common.dataset_config("validation", *data, shuffle=False, seed=42),
      # full-length inference evaluation: lengths are computed from the data, no packing
      infer_eval_dataset_cfg=common.dataset_config(
          "validation", mixture_or_task_name, None, batch_size, use_cached_tasks,
          mixture_or_task_module, shuffle=False, seed=42, pack=False),
      inference_evaluator_cls=fdl.Partial(evaluation.Evaluator, num_examples=None,
                                          use_memory_cache=True),
      checkpoint_cfg=common.checkpoint_config(initial_checkpoint_path, "specific", period=5000,
                                              save_dataset=False),
      partitioner=common.partitioner(),
      trainer_cls=common.trainer_cls("constant", 0.001, 1000),
      total_steps=train_steps, eval_steps=eval_steps, eval_period=eval_period,
      relative_steps=relative_steps, random_seed=random_seed, use_hardware_rng=use_hardware_rng,
      summarize_config_fn=config_utils.summarize_fiddle_config)
