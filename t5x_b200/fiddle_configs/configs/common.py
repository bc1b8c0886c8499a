"""Pieces shared by the run configs."""
from __future__ import annotations

import copy
from typing import Mapping, Optional, Sequence, Union

from t5x_b200 import fdl, partitioning, trainer, utils

MixtureOrTask = Union[str, object]


def dataset_config(split: str, mixture_or_task_name: MixtureOrTask,
                   task_feature_lengths: Optional[Mapping[str, int]], batch_size: int,
                   use_cached_tasks: bool, mixture_or_task_module: Optional[str], *,
                   shuffle: bool, seed: Optional[int], pack: bool = True) -> fdl.Buildable:
  lengths = copy.copy(task_feature_lengths) if task_feature_lengths is not None else None
  return fdl.Config(utils.DatasetConfig, mixture_or_task_name=mixture_or_task_name,
                    task_feature_lengths=lengths, split=split, batch_size=batch_size,
                    shuffle=shuffle, seed=seed, use_cached=use_cached_tasks, pack=pack,
                    module=mixture_or_task_module)


def partitioner(num_partitions: int = 1) -> fdl.Buildable:
  return fdl.Config(partitioning.PjitPartitioner, num_partitions=num_partitions,
                    model_parallel_submesh=None,
                    logical_axis_rules=fdl.Config(partitioning.standard_logical_axis_rules))


def trainer_cls(factors: str, base_learning_rate: float, warmup_steps: int) -> fdl.Buildable:
  """`Trainer` with a learning-rate schedule made anew for every trainer that is built."""
  return fdl.Partial(trainer.Trainer, num_microbatches=None,
                     learning_rate_fn=fdl.ArgFactory(utils.create_learning_rate_scheduler,
                                                     factors=factors,
                                                     base_learning_rate=base_learning_rate,
                                                     warmup_steps=warmup_steps))


def checkpoint_config(restore_path: Union[str, Sequence[str]] = (), restore_mode: str = "latest",
                      period: int = 1000, save_dataset: bool = False) -> fdl.Buildable:
  restore = fdl.Config(utils.RestoreCheckpointConfig, path=list(restore_path)
                       if not isinstance(restore_path, str) else restore_path)
  if restore_path:
    restore.mode = restore_mode
    restore.dtype = "float32"
  return fdl.Config(utils.CheckpointConfig, restore=restore,
                    save=fdl.Config(utils.SaveCheckpointConfig, period=period, dtype="float32",
                                    keep=None, save_dataset=save_dataset))
