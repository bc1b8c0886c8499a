"""Notebook-friendly wrapper around a model: construct, restore or initialise, then call
`train_step`, `predict`, `predict_with_aux`, `score`, `evaluate`, `train_loop` on plain Python
examples (API of t5x/interactive_model.py:66-1250).

Examples are strings (inputs only) or dicts `{"input": ..., "target": ...}`; they are
tokenised with the model's vocabularies and run through the model's feature converter, so
what the model sees is exactly what the batch entry points would feed it.
"""
from __future__ import annotations

import abc
import enum
import logging
import os
from typing import Any, Callable, Dict, Iterator, List, Mapping, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from t5x_b200 import checkpoints
from t5x_b200 import models
from t5x_b200 import partitioning
from t5x_b200 import trainer as trainer_lib
from t5x_b200 import utils
from t5x_b200.data import dataset as dataset_lib
from t5x_b200.parallel import state as pstate

BatchesType = Union[Sequence[Mapping[str, str]], Sequence[Sequence[Mapping[str, str]]]]


class InferenceType(enum.Enum):
  PREDICT_WITH_AUX = 1
  SCORE = 2


class T5XScriptType(enum.Enum):
  FINETUNING = 1
  INFERENCE = 2
  EVALUATION = 3
  PRETRAINING = 4


class InteractiveModel(abc.ABC):
  """Wrapper around a T5X-style model for interactive use."""

  def __init__(self, batch_size: int, task_feature_lengths: Mapping[str, int], output_dir: str,
               partitioner: partitioning.BasePartitioner, model: models.BaseTransformerModel,
               dtype: Optional[str], restore_mode: str, checkpoint_path: str,
               input_shapes: Mapping[str, Any],
               input_types: Optional[Mapping[str, Any]] = None, init_random_seed: int = 42,
               add_eos: bool = True, eval_names: Optional[Sequence[str]] = None):
    self._batch_size = batch_size
    self._task_feature_lengths = dict(task_feature_lengths)
    self._output_dir = output_dir
    self._partitioner = partitioner
    self._model = model
    self._add_eos = add_eos
    self._init_random_seed = init_random_seed
    self._checkpoint_path = checkpoint_path
    self._restore_mode = restore_mode
    self._dtype = dtype
    os.makedirs(output_dir, exist_ok=True)
    data_layout = partitioner.get_data_layout(batch_size)
    if data_layout.shard_id != 0 or data_layout.num_shards != 1:
      raise ValueError("This wrapper feeds the whole batch from one process: use a partitioner "
                       "with a single data shard.")
    self._input_shapes = dict(input_shapes)
    self._input_types = dict(input_types) if input_types else None
    self._initializer = utils.TrainStateInitializer(
        optimizer_def=model.optimizer_def, init_fn=model.get_initial_variables,
        input_shapes=self._input_shapes, input_types=self._input_types, partitioner=partitioner)
    self._train_state_axes = self._initializer.train_state_axes
    restore_cfg = None
    if checkpoint_path:
      restore_cfg = utils.RestoreCheckpointConfig(path=checkpoint_path, mode=restore_mode,
                                                  dtype=dtype)
    save_cfg = utils.SaveCheckpointConfig(dtype="float32", period=1, keep=None,
                                          save_dataset=False)
    valid_cfg, paths = (utils.get_first_valid_restore_config_and_paths([restore_cfg])
                        if restore_cfg else (None, []))
    if len(paths) > 1:
      raise ValueError("Expected a single checkpoint to restore, got several.")
    self._train_state, self._checkpoint_manager = utils.create_checkpoint_manager_and_restore(
        self._initializer, partitioner, valid_cfg, paths[0] if paths else None,
        init_random_seed, save_checkpoint_cfg=save_cfg, model_dir=output_dir)
    if self._train_state is None:
      self._train_state = self._initializer.from_scratch(init_random_seed)
    self._eval_names = list(eval_names or [])
    self._trainer = trainer_lib.Trainer(
        model=model, train_state=self._train_state, partitioner=partitioner,
        eval_names=self._eval_names, summary_dir=output_dir,
        train_state_axes=self._train_state_axes, rng=init_random_seed + 1,
        learning_rate_fn=utils.create_learning_rate_scheduler(), num_microbatches=None)
    self._train_summary = None
    self._cached_infer_fns: Dict[Any, Callable] = {}

  # ---- properties ------------------------------------------------------------------------
  @property
  def trainer(self):
    return self._trainer

  @property
  def partitioner(self):
    return self._partitioner

  @property
  def model(self):
    return self._model

  @property
  def train_state(self):
    return self._trainer.train_state

  @property
  def train_state_axes(self):
    return self._train_state_axes

  @property
  def train_summary(self):
    return self._train_summary.result() if self._train_summary is not None else None

  @property
  def step(self) -> int:
    return int(utils.get_local_data(self.train_state.step))

  # ---- training --------------------------------------------------------------------------
  def train_step(self, examples: Sequence[Union[str, Mapping[str, str]]]) -> None:
    """One train step on `examples` (padded / cut to the batch size by repetition)."""
    self.train_step_with_preprocessors(examples, preprocessors=())

  def train_step_with_preprocessors(self, examples, preprocessors: Sequence[Callable] = ()):
    if len(examples) < self._batch_size:
      logging.warning("Fewer examples (%d) than the batch size (%d): repeating examples.",
                      len(examples), self._batch_size)
    batches = get_batches_from_seqio(
        "interactive_train", self._task_feature_lengths, self._batch_size, examples,
        feature_converter=self._model.FEATURE_CONVERTER_CLS(pack=False),
        vocabularies=(self._model.input_vocabulary, self._model.output_vocabulary),
        add_eos=self._add_eos, preprocessors=preprocessors, fill=True)
    self.train_step_from_batch_iterator(iter(batches[:1]))

  def train_step_from_batch_iterator(self, iterator: Iterator[Mapping[str, np.ndarray]]) -> None:
    self._train_summary = self._trainer.train(iterator, 1, start_step=self.step)
    if hasattr(self._trainer, "sync_replicas"):
      self._trainer.sync_replicas()

  def save_checkpoint(self) -> None:
    self._checkpoint_manager.save(self.train_state, force=True)
    self._checkpoint_manager.wait_until_finished()

  # ---- inference -------------------------------------------------------------------------
  def infer_with_preprocessors(self, mode: InferenceType, examples,
                               preprocessors: Sequence[Callable] = (), **inference_kwargs):
    """Runs prediction or scoring; returns (per-example outputs, aux)."""
    batches = get_batches_from_seqio(
        "interactive_infer", self._task_feature_lengths, self._batch_size, examples,
        feature_converter=self._model.FEATURE_CONVERTER_CLS(pack=False),
        vocabularies=(self._model.input_vocabulary, self._model.output_vocabulary),
        add_eos=self._add_eos, preprocessors=preprocessors, fill=False)
    dev = pstate.get().device
    outputs, aux_all = [], []
    for batch in batches:
      n = next(iter(batch.values())).shape[0]
      tb = {k: torch.from_numpy(np.asarray(v)).to(dev) for k, v in batch.items()}
      with torch.no_grad():
        if mode == InferenceType.PREDICT_WITH_AUX:
          out, aux = self._model.predict_batch_with_aux(self.train_state.params, tb,
                                                        **inference_kwargs)
          aux_all.append({k: v.cpu().numpy()[:n] for k, v in aux.items()})
        elif mode == InferenceType.SCORE:
          out = self._model.score_batch(self.train_state.params, tb)
        else:
          raise ValueError(f"Mode must be `predict_with_aux` or `score`, got {mode}.")
      outputs.extend(list(out.cpu().numpy()[:n]))
    outputs = outputs[:len(examples)]
    aux = {}
    if aux_all:
      aux = {k: np.concatenate([a[k] for a in aux_all])[:len(examples)] for k in aux_all[0]}
    return outputs, aux

  def predict(self, examples) -> List[str]:
    return self.predict_with_aux(examples)[0]

  def predict_with_aux(self, examples, **kwargs) -> Tuple[List[str], Mapping[str, Any]]:
    """Decoded predictions (text) and the model's aux values (e.g. scores)."""
    tokens, aux = self.infer_with_preprocessors(InferenceType.PREDICT_WITH_AUX, examples,
                                                **kwargs)
    vocab = self._model.output_vocabulary
    return [vocab.decode([int(t) for t in row]) for row in tokens], aux

  def score(self, examples) -> Sequence[float]:
    """Log-likelihood of each example's target given its input."""
    scores, _ = self.infer_with_preprocessors(InferenceType.SCORE, examples)
    return [float(s) for s in scores]

  # ---- evaluation ------------------------------------------------------------------------
  def _compute_metrics(self, targets: Sequence[Any], predictions: Sequence[Any],
                       aux_values: Mapping[str, Any], scores: Sequence[Any],
                       predict_metric_fns: Sequence[Callable],
                       predict_with_aux_metric_fns: Sequence[Callable],
                       score_metric_fns: Sequence[Callable]) -> Mapping[str, Any]:
    results = {}
    for fn in predict_metric_fns:
      results.update(fn(targets, predictions))
    for fn in predict_with_aux_metric_fns:
      results.update(fn(targets, predictions, aux_values))
    for fn in score_metric_fns:
      results.update(fn(targets, scores))
    return results

  def evaluate(self, examples, metric_fns: Sequence[Callable]) -> Mapping[str, Any]:
    """Metrics of predictions against the examples' targets. A metric function takes
    (targets, predictions); one with a `scores` argument takes (targets, scores)."""
    return self.evaluate_with_preprocessors(examples, (), metric_fns)

  def evaluate_with_preprocessors(self, examples, preprocessors, metric_fns,
                                  postprocessor: Optional[Callable] = None):
    import inspect
    targets = [ex["target"] if isinstance(ex, Mapping) else "" for ex in examples]
    if postprocessor:
      targets = [postprocessor(t, example=ex, is_target=True) for t, ex in zip(targets, examples)]
    predict_fns, aux_fns, score_fns = [], [], []
    for fn in metric_fns:
      names = list(inspect.signature(fn).parameters)
      if "scores" in names:
        score_fns.append(fn)
      elif "aux_values" in names:
        aux_fns.append(fn)
      else:
        predict_fns.append(fn)
    predictions, aux, scores = [], {}, []
    if predict_fns or aux_fns:
      predictions, aux = self.predict_with_aux(examples)
      if postprocessor:
        predictions = [postprocessor(p, example=ex, is_target=False)
                       for p, ex in zip(predictions, examples)]
    if score_fns:
      scores = self.score(examples)
    return self._compute_metrics(targets, predictions, aux, scores, predict_fns, aux_fns,
                                 score_fns)

  def train_loop(self, num_steps: int, eval_period: Optional[int] = 1,
                 train_batches: Optional[BatchesType] = None,
                 predict_batches: Optional[BatchesType] = None,
                 score_batches: Optional[BatchesType] = None,
                 eval_batches: Optional[BatchesType] = None,
                 metrics_fns: Optional[Sequence[Callable]] = None):
    """Trains for `num_steps` steps, cycling through `train_batches`; every `eval_period`
    steps runs prediction / scoring / evaluation on the corresponding batches. Returns the
    last (predictions, scores, metrics)."""
    train_batches = list(train_batches or [])
    if not train_batches:
      raise ValueError("train_loop needs `train_batches`.")
    if train_batches and not isinstance(train_batches[0], (list, tuple)):
      train_batches = [train_batches]
    last = (None, None, None)
    for i in range(num_steps):
      self.train_step(train_batches[i % len(train_batches)])
      if eval_period and (i + 1) % eval_period == 0:
        preds = [self.predict(b) for b in _as_batches(predict_batches)]
        scs = [self.score(b) for b in _as_batches(score_batches)]
        mets = [self.evaluate(b, metrics_fns or ()) for b in _as_batches(eval_batches)]
        last = (preds, scs, mets)
    return last


def _as_batches(batches):
  if not batches:
    return []
  if isinstance(batches[0], (list, tuple)):
    return list(batches)
  return [batches]


# ----------------------------------------------------------------------------
# Text examples -> model batches
# ----------------------------------------------------------------------------
def get_dataset_from_natural_text_examples(
    examples: Sequence[Union[str, Mapping[str, str]]], preprocessors: Sequence[Callable],
    task_feature_lengths: Mapping[str, int], features: Mapping[str, Any]) -> List[dict]:
  """Tokenised examples: `{"inputs", "targets", "inputs_pretokenized", "targets_pretokenized"}`
  (t5x/interactive_model.py:891-990). `features[name]` provides `.vocabulary` and `.add_eos`."""
  out = []
  for ex in examples:
    if isinstance(ex, str):
      ex = {"input": ex, "target": ""}
    rec = {"inputs_pretokenized": ex.get("input", ex.get("inputs", "")),
           "targets_pretokenized": ex.get("target", ex.get("targets", ""))}
    for prep in preprocessors:
      rec = prep(rec)
    for name in ("inputs", "targets"):
      feat = features[name]
      ids = list(feat.vocabulary.encode(rec[f"{name}_pretokenized"]))
      if getattr(feat, "add_eos", True):
        ids.append(feat.vocabulary.eos_id)
      limit = task_feature_lengths.get(name)
      if limit:
        ids = ids[:limit]
      rec[name] = np.asarray(ids, np.int32)
    out.append(rec)
  return out


def _get_equal_length_batches(examples: Sequence[Any], batch_size: int, fill: bool):
  """Batches of exactly `batch_size` examples; the last one is filled by repeating examples."""
  examples = list(examples)
  if not examples:
    return []
  batches = [examples[i:i + batch_size] for i in range(0, len(examples), batch_size)]
  last = batches[-1]
  i = 0
  while len(last) < batch_size:
    last.append(examples[i % len(examples)])
    i += 1
  return batches


def get_batches_from_seqio(task_or_mixture_name: str, task_feature_lengths: Mapping[str, int],
                           batch_size: int, examples, feature_converter, vocabularies,
                           add_eos: bool = True, preprocessors: Sequence[Callable] = (),
                           fill: bool = False, **_) -> List[Dict[str, np.ndarray]]:
  """Model-feature batches (numpy) for `examples` (t5x/interactive_model.py:1026-1106)."""
  from t5x_b200.data import tasks as tasks_lib
  in_vocab, out_vocab = vocabularies
  features = {"inputs": tasks_lib.Feature(in_vocab, add_eos=add_eos),
              "targets": tasks_lib.Feature(out_vocab, add_eos=add_eos)}
  tok = get_dataset_from_natural_text_examples(examples, preprocessors, task_feature_lengths,
                                               features)
  batches = []
  for group in _get_equal_length_batches(tok, batch_size, fill):
    ds = dataset_lib.Dataset.from_examples(group).convert(feature_converter, task_feature_lengths)
    rows = list(ds)
    batches.append({k: np.stack([np.asarray(r[k]) for r in rows]) for k in rows[0]})
  return batches


def get_seqio_task_from_examples(task_name: str, examples, preprocessors, add_eos: bool,
                                 vocabularies=None):
  """Registers (or replaces) an ad-hoc task over in-memory examples."""
  from t5x_b200.data import tasks as tasks_lib
  in_vocab, out_vocab = vocabularies
  features = {"inputs": tasks_lib.Feature(in_vocab, add_eos=add_eos),
              "targets": tasks_lib.Feature(out_vocab, add_eos=add_eos)}

  def source(split, shard_info=None, seed=None, sequence_length=None, **_):
    return iter(get_dataset_from_natural_text_examples(examples, preprocessors,
                                                       sequence_length or {}, features))

  if task_name in tasks_lib.TaskRegistry:
    tasks_lib.TaskRegistry.remove(task_name)
  return tasks_lib.TaskRegistry.add(task_name, source, features, splits=("interactive",))


def get_gin_config_from_interactive_model(interactive_model: InteractiveModel,
                                          script_type: T5XScriptType, task_name: str,
                                          partitioner_config_str: str, model_config_str: str,
                                          train_steps: int = 1, imports_str: str = "") -> str:
  """A gin file that reproduces the interactive session as a batch run."""
  m = interactive_model
  restore = (f'utils.RestoreCheckpointConfig.path = "{m._checkpoint_path}"\n'
             f'utils.RestoreCheckpointConfig.mode = "{m._restore_mode}"\n'
             f'utils.RestoreCheckpointConfig.dtype = "{m._dtype or "float32"}"')
  run = {T5XScriptType.FINETUNING: "finetune", T5XScriptType.PRETRAINING: "pretrain",
         T5XScriptType.INFERENCE: "infer", T5XScriptType.EVALUATION: "eval"}[script_type]
  return f"""from __gin__ import dynamic_registration
{imports_str}
include 't5x/configs/runs/{run}.gin'

MODEL_DIR = "{m._output_dir}"
MIXTURE_OR_TASK_NAME = "{task_name}"
TASK_FEATURE_LENGTHS = {dict(m._task_feature_lengths)}
BATCH_SIZE = {m._batch_size}
TRAIN_STEPS = {m.step + train_steps}
RANDOM_SEED = {m._init_random_seed}

{model_config_str}
{partitioner_config_str}
{restore}
"""
