"""Inference-based evaluation over registered tasks (the seqio.Evaluator contract used by
t5x/eval.py:62-180 and t5x/train.py:455-466) and its metric loggers."""
from __future__ import annotations

import concurrent.futures
import json
import logging
import os
import time
from typing import Any, Callable, Dict, Mapping, Optional, Sequence

import numpy as np

from t5x_b200.data import tasks as tasks_lib
from t5x_b200.data.dataset import Dataset


class Logger:
  def __init__(self, output_dir: Optional[str] = None):
    self.output_dir = output_dir

  def __call__(self, task_name: str, step: Optional[int], metrics: Mapping[str, Any],
               dataset=None, inferences=None, targets=None) -> None:
    raise NotImplementedError


class PyLoggingLogger(Logger):
  def __call__(self, task_name, step, metrics, dataset=None, inferences=None, targets=None):
    for k, v in metrics.items():
      logging.info("%s/%s at step %s: %s", task_name, k, step, v)


class JSONLogger(Logger):
  """Appends one JSON line per evaluation to `<dir>/<task>-metrics.jsonl`."""

  def __call__(self, task_name, step, metrics, dataset=None, inferences=None, targets=None):
    if not self.output_dir:
      return
    os.makedirs(self.output_dir, exist_ok=True)
    rec = {"step": step}
    rec.update({k: (float(v) if np.isscalar(v) or isinstance(v, np.generic) else v)
                for k, v in metrics.items()})
    with open(os.path.join(self.output_dir, f"{task_name}-metrics.jsonl"), "a") as f:
      f.write(json.dumps(rec) + "\n")


class TensorBoardLogger(Logger):
  def __init__(self, output_dir=None):
    super().__init__(output_dir)
    self._writers = {}

  def __call__(self, task_name, step, metrics, dataset=None, inferences=None, targets=None):
    if not self.output_dir:
      return
    from t5x_b200.utils import metric_writers
    w = self._writers.get(task_name)
    if w is None:
      w = metric_writers.TensorBoardWriter(os.path.join(self.output_dir, task_name))
      self._writers[task_name] = w
    w.write_scalars(step or 0, {f"eval/{k}": v for k, v in metrics.items()
                                if np.isscalar(v) or isinstance(v, np.generic)})
    w.flush()


class Evaluator:
  """Runs model inference over the evaluation split of every task of a mixture and computes
  the tasks' metric functions on the decoded predictions (and scores)."""

  def __init__(self, mixture_or_task_name: str, feature_converter, eval_split: str = "validation",
               use_cached: bool = False, seed: Optional[int] = 42,
               sequence_length: Optional[Mapping[str, int]] = None, num_examples: Optional[int] = None,
               shuffle: bool = False, logger_cls: Sequence[Callable[..., Logger]] = (),
               log_dir: Optional[str] = None, use_memory_cache: bool = True,
               target_field_name: str = "targets"):
    mt = tasks_lib.get_mixture_or_task(mixture_or_task_name)
    all_tasks = mt.tasks if isinstance(mt, tasks_lib.Mixture) else [mt]
    self._eval_tasks = [t for t in all_tasks if t.metric_fns and eval_split in t.splits]
    self._feature_converter = feature_converter
    self._split = eval_split
    self._seed = seed
    self._num_examples = num_examples if num_examples is not None else 64
    self._sequence_length = dict(sequence_length) if sequence_length else None
    self._loggers = [cls(output_dir=log_dir) for cls in logger_cls]
    self._target_field = target_field_name
    self._cached: Dict[str, Dict[str, Any]] = {}
    self._pool = concurrent.futures.ThreadPoolExecutor(max_workers=1)
    for t in self._eval_tasks:
      examples = []
      ds = t.get_dataset(self._sequence_length, split=eval_split, seed=seed, shuffle=False)
      for i, ex in enumerate(ds):
        if i >= self._num_examples:
          break
        examples.append(ex)
      if self._sequence_length is None:
        lens = {}
        for ex in examples:
          for k, v in ex.items():
            if isinstance(v, np.ndarray):
              lens[k] = max(lens.get(k, 0), len(v))
        self._sequence_length = lens
      self._cached[t.name] = {"examples": examples}

  @property
  def eval_tasks(self):
    return self._eval_tasks

  @property
  def model_feature_shapes(self) -> Mapping[str, tuple]:
    if not self._sequence_length:
      return {}
    lens = self._feature_converter.get_model_feature_lengths(self._sequence_length)
    return {k: (v,) for k, v in lens.items()}

  def close(self):
    self._pool.shutdown(wait=True)

  def evaluate(self, *, compute_metrics: bool = True, step: Optional[int] = None,
               predict_fn: Callable, score_fn: Callable,
               predict_with_aux_fn: Optional[Callable] = None):
    """-> (future of {task: metrics}, all outputs). predict_fn(ds) returns a list of
    (index, token array); score_fn(ds) a list of (index, score)."""
    all_metrics, all_outputs = {}, {}
    for t in self._eval_tasks:
      examples = self._cached[t.name]["examples"]
      ds = Dataset.from_examples(examples).convert(
          type(self._feature_converter)(pack=False), self._sequence_length)
      vocab = t.output_features[self._target_field].vocabulary
      targets = [t.postprocess(vocab.decode(list(ex[self._target_field])), example=ex,
                               is_target=True) for ex in examples]
      metrics = {}
      outputs = {}
      if t.predict_metric_fns:
        res = (predict_with_aux_fn or predict_fn)(ds.enumerate())
        aux = None
        if isinstance(res, tuple):
          res, aux = res
        preds_tokens = [np.asarray(p) for _, p in sorted(res, key=lambda x: x[0])]
        preds = [t.postprocess(vocab.decode(list(p)), example=ex, is_target=False)
                 for p, ex in zip(preds_tokens, examples)]
        outputs["prediction"] = preds
        if compute_metrics:
          for fn in t.predict_metric_fns:
            metrics.update(fn(targets, preds))
      if t.score_metric_fns:
        scores = [s for _, s in sorted(score_fn(ds.enumerate()), key=lambda x: x[0])]
        outputs["score"] = scores
        if compute_metrics:
          for fn in t.score_metric_fns:
            metrics.update(fn(targets, scores))
      all_metrics[t.name] = metrics
      all_outputs[t.name] = outputs
      for lg in self._loggers:
        lg(t.name, step, metrics)
    fut = concurrent.futures.Future()
    fut.set_result(all_metrics)
    return fut, all_outputs
