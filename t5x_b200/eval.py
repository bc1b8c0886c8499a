r"""Evaluation entry point (API of t5x/eval.py).

  python -m t5x_b200.eval --gin_file=t5x/configs/runs/eval.gin --gin.CHECKPOINT_PATH=... \
      --gin.EVAL_OUTPUT_DIR=...

`InferenceEvaluator` wraps a seqio-style evaluator with the model's predict / score steps;
`evaluate()` walks one or all checkpoints of a directory, skipping those already evaluated.
"""
from __future__ import annotations

import functools
import logging
import os
import re
import sys
from typing import Callable, Collection, Mapping, Optional, Sequence, Set, Tuple, Type

from t5x_b200 import checkpoints
from t5x_b200 import gin
from t5x_b200 import gin_utils
from t5x_b200 import models
from t5x_b200 import partitioning
from t5x_b200 import trainer as trainer_lib
from t5x_b200 import utils
from t5x_b200.data import seqio_api as seqio
from t5x_b200.parallel import state as pstate


class InferenceEvaluator:
  """Metric evaluation through decoding and scoring (t5x/eval.py:62-180)."""

  def __init__(self, infer_eval_dataset_cfg: utils.DatasetConfig, inference_evaluator_cls,
               model: models.BaseModel, partitioner: partitioning.BasePartitioner,
               log_dir: Optional[str] = None,
               verify_matching_vocabs_fn: Optional[Callable] = utils.verify_matching_vocabs):
    if verify_matching_vocabs_fn and isinstance(model, models.BaseTransformerModel):
      verify_matching_vocabs_fn(infer_eval_dataset_cfg, model)
    self._model = model
    self._partitioner = partitioner
    self._cfg = infer_eval_dataset_cfg
    kwargs = {}
    if log_dir:
      kwargs["log_dir"] = os.path.join(log_dir, "inference_eval")
    else:
      kwargs["logger_cls"] = ()
    self._evaluator = inference_evaluator_cls(
        mixture_or_task_name=infer_eval_dataset_cfg.mixture_or_task_name,
        feature_converter=model.FEATURE_CONVERTER_CLS(pack=False),
        eval_split=infer_eval_dataset_cfg.split, use_cached=infer_eval_dataset_cfg.use_cached,
        seed=infer_eval_dataset_cfg.seed,
        sequence_length=infer_eval_dataset_cfg.task_feature_lengths,
        use_memory_cache=infer_eval_dataset_cfg.use_memory_cache, **kwargs)
    self._predict_fn = self._predict_with_aux_fn = self._score_fn = None

  @property
  def model_feature_shapes(self) -> Mapping[str, Tuple[int, ...]]:
    return self._evaluator.model_feature_shapes

  @property
  def eval_tasks(self):
    return self._evaluator.eval_tasks

  def close(self):
    self._evaluator.close()

  def evaluate(self, train_state, train_state_axes):
    """-> future of {task: {metric: value}}; metrics are computed on rank 0 only."""
    if self._predict_fn is None:
      mk = functools.partial(utils.get_infer_fn, batch_size=self._cfg.batch_size,
                             train_state_axes=train_state_axes, partitioner=self._partitioner)
      self._predict_fn = mk(infer_step=self._model.predict_batch)
      self._predict_with_aux_fn = mk(infer_step=self._model.predict_batch_with_aux)
      self._score_fn = mk(infer_step=self._model.score_batch)
    all_metrics, _ = self._evaluator.evaluate(
        compute_metrics=pstate.get().rank == 0,
        step=int(utils.get_local_data(train_state.step)),
        predict_fn=functools.partial(self._predict_fn, train_state=train_state, rng=0),
        score_fn=functools.partial(self._score_fn, train_state=train_state),
        predict_with_aux_fn=functools.partial(self._predict_with_aux_fn,
                                              train_state=train_state, rng=0))
    return all_metrics


def _sorted_ckpt_paths(ckpt_paths: Collection[str]) -> Sequence[str]:
  def step_of(path):
    m = re.search(r"checkpoint_(\d+)", os.path.basename(path.rstrip("/")))
    return int(m.group(1)) if m else -1
  return sorted(ckpt_paths, key=step_of)


def _load_evaluated_ckpt_paths(eval_ckpt_path: str) -> Set[str]:
  if not os.path.exists(eval_ckpt_path):
    return set()
  with open(eval_ckpt_path) as f:
    return {line.strip() for line in f if line.strip()}


def evaluate(*, model: models.BaseTransformerModel, dataset_cfg: utils.DatasetConfig,
             restore_checkpoint_cfg: utils.RestoreCheckpointConfig,
             partitioner: partitioning.BasePartitioner, output_dir: str,
             inference_evaluator_cls=seqio.Evaluator,
             training_evaluator_cls: Optional[Type[trainer_lib.Trainer]] = None,
             summarize_config_fn: Callable = gin_utils.summarize_gin_config,
             train_state_initializer_cls=utils.TrainStateInitializer,
             train_eval_get_dataset_fn=utils.get_training_eval_datasets,
             fallback_init_rng: Optional[int] = None, use_orbax: bool = True):
  """Evaluates one or all checkpoints on a task or mixture (t5x/eval.py:202-424)."""
  logging.info("Process ID: %d", pstate.get().rank)
  if dataset_cfg.module:
    utils.import_module(dataset_cfg.module)
  batch_size = dataset_cfg.batch_size
  os.makedirs(output_dir, exist_ok=True)
  summarize_config_fn(model_dir=output_dir, summary_writer=None, step=0)

  evaluator = InferenceEvaluator(dataset_cfg, inference_evaluator_cls, model, partitioner,
                                 log_dir=output_dir)
  if not evaluator.eval_tasks:
    raise ValueError(f"'{dataset_cfg.mixture_or_task_name}' has no metrics for evaluation, "
                     "or this mixture/task doesn't have provided split.")
  input_shapes = {k: (batch_size,) + tuple(s) for k, s in evaluator.model_feature_shapes.items()}
  initializer = train_state_initializer_cls(optimizer_def=None,
                                            init_fn=model.get_initial_variables,
                                            input_shapes=input_shapes, partitioner=partitioner)
  train_state_axes = initializer.train_state_axes
  utils.log_model_info(os.path.join(output_dir, "model-info.txt"),
                       initializer.global_train_state_shape, partitioner)

  train_evaluator = None
  train_eval_datasets = {}
  if training_evaluator_cls:
    layout = partitioner.get_data_layout(dataset_cfg.batch_size)
    train_eval_datasets = train_eval_get_dataset_fn(
        dataset_cfg, layout.shard_id, layout.num_shards,
        feature_converter_cls=model.FEATURE_CONVERTER_CLS)
    train_evaluator = training_evaluator_cls(
        model=model, train_state=None, partitioner=partitioner,
        train_state_axes=train_state_axes, eval_names=list(train_eval_datasets.keys()),
        summary_dir=output_dir, rng=0, learning_rate_fn=None, num_microbatches=None)

  restore_checkpoint_cfg.strict = False  # the optimizer state is dropped
  eval_ckpt_path = os.path.join(output_dir, f"eval.{dataset_cfg.mixture_or_task_name}.ckpt")
  if restore_checkpoint_cfg.mode == "all" and os.path.exists(eval_ckpt_path):
    dirs = ([restore_checkpoint_cfg.path] if isinstance(restore_checkpoint_cfg.path, str)
            else list(restore_checkpoint_cfg.path))
    ckpt_paths = set()
    for d in dirs:
      if not os.path.isdir(d):
        raise ValueError(f"Checkpoint path '{d}' must be a valid directory when using "
                         "restore mode 'all'.")
      ckpt_paths.update(checkpoints.get_checkpoint_dir(d, s) for s in checkpoints.all_steps(d))
    done = _load_evaluated_ckpt_paths(eval_ckpt_path)
    logging.info("Skipping evaluated checkpoints:\n %s",
                 "\n ".join(_sorted_ckpt_paths(ckpt_paths & done)))
    ckpt_paths = _sorted_ckpt_paths(ckpt_paths - done)
    restore_cfg = restore_checkpoint_cfg
    restore_cfg.mode = "specific"
  else:
    restore_cfg, ckpt_paths = utils.get_first_valid_restore_config_and_paths(
        [restore_checkpoint_cfg])

  results = {}
  for ckpt_path in ckpt_paths:
    train_state, manager = utils.create_checkpoint_manager_and_restore(
        initializer, partitioner, restore_cfg, ckpt_path, fallback_init_rng, use_orbax=use_orbax)
    if train_state is None:
      raise ValueError("Failed to restore checkpoint.")
    host_step = int(utils.get_local_data(train_state.step))
    if train_evaluator is not None:
      train_evaluator.train_state = train_state
      train_evaluator.eval({t: iter(ds) for t, ds in train_eval_datasets.items()})
    all_metrics = evaluator.evaluate(train_state, train_state_axes)
    results[host_step] = all_metrics.result()
    utils.sync_global_devices(f"step_{host_step}:complete")
    if pstate.get().rank == 0:
      # read / replace rather than append, so that a crash cannot leave a torn line
      done = _load_evaluated_ckpt_paths(eval_ckpt_path)
      done.add(ckpt_path)
      tmp = eval_ckpt_path + ".tmp"
      with open(tmp, "w") as f:
        f.write("\n".join(_sorted_ckpt_paths(done)))
      os.replace(tmp, eval_ckpt_path)
    manager.close()
  evaluator.close()
  if train_evaluator is not None:
    train_evaluator.close()
  logging.info("Finished.")
  return results


def main(argv: Optional[Sequence[str]] = None) -> None:
  from t5x_b200 import train as train_lib
  logging.basicConfig(level=logging.INFO)
  argv = gin_utils.rewrite_gin_args(list(sys.argv[1:] if argv is None else argv))
  flags = train_lib.build_flag_parser(__doc__).parse_args(argv)
  train_lib.init_distributed_from_flags(flags)
  from t5x_b200 import config_utils
  if config_utils.using_fdl(flags):
    config_utils.run_with_fiddle(evaluate, flags)
    return
  gin.set_main_module(sys.modules[__name__])
  train_lib.parse_gin_from_flags(flags, train_lib._DEFAULT_GIN_SEARCH_PATHS)
  gin.get_configurable(evaluate)()


if __name__ == "__main__":
  main()
