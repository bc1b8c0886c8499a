"""Task / mixture registry and dataset construction (the seqio surface used by t5x/utils.py
`get_dataset`, `get_vocabulary`, and the gin run configs' MIXTURE_OR_TASK_NAME)."""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Dict, Mapping, Optional, Sequence, Union

import numpy as np

from t5x_b200.data import synthetic
from t5x_b200.data import vocabularies
from t5x_b200.data.dataset import Dataset, ShardInfo


@dataclasses.dataclass
class Feature:
  vocabulary: vocabularies.Vocabulary
  add_eos: bool = True
  required: bool = True
  dtype: Any = np.int32
  rank: int = 1


class Task:
  """A named source of tokenised examples with output features and metric functions.

  `source(split, shard_info, seed) -> iterable of dict(str -> array)`.
  """

  def __init__(self, name: str, source: Callable[..., Any], output_features: Mapping[str, Feature],
               metric_fns: Sequence[Callable] = (), postprocess_fn: Optional[Callable] = None,
               splits: Sequence[str] = ("train", "validation"),
               num_input_examples: Optional[Mapping[str, int]] = None):
    self.name = name
    self._source = source
    self.output_features = dict(output_features)
    self.metric_fns = list(metric_fns)
    self.postprocess_fn = postprocess_fn
    self.splits = tuple(splits)
    self._num_input_examples = dict(num_input_examples or {})
    self.predict_metric_fns = [f for f in self.metric_fns
                               if "scores" not in f.__code__.co_varnames[:f.__code__.co_argcount]]
    self.score_metric_fns = [f for f in self.metric_fns if f not in self.predict_metric_fns]

  def num_input_examples(self, split):
    return self._num_input_examples.get(split)

  def get_dataset(self, sequence_length=None, split="train", use_cached=False, shuffle=True,
                  seed=None, shard_info: Optional[ShardInfo] = None, num_epochs=1,
                  trim_output_features=True, **_) -> Dataset:
    shard_info = shard_info or ShardInfo(0, 1)
    seed = 0 if seed is None else seed

    def make(start):
      it = iter(self._source(split=split, shard_info=shard_info, seed=seed,
                             sequence_length=sequence_length))
      import itertools
      it = itertools.islice(it, start, None)
      for ex in it:
        if trim_output_features and sequence_length:
          ex = {k: (np.asarray(v)[:sequence_length[k]] if k in sequence_length and
                    isinstance(v, (np.ndarray, list)) else v) for k, v in ex.items()}
        yield ex

    n = self.num_input_examples(split)
    card = None if n is None else (n - shard_info.index + shard_info.num_shards - 1) // shard_info.num_shards
    ds = Dataset(make, cardinality=card)
    if num_epochs is None and card is not None:
      ds = ds.repeat()
    return ds

  def postprocess(self, x, **kw):
    return self.postprocess_fn(x, **kw) if self.postprocess_fn else x


class Mixture:
  """A rate-weighted mixture of tasks (examples are interleaved deterministically by seed)."""

  def __init__(self, name: str, tasks_and_rates: Sequence):
    self.name = name
    self._tasks = []
    self._rates = []
    for item in tasks_and_rates:
      if isinstance(item, (tuple, list)):
        t, r = item
      else:
        t, r = item, 1.0
      self._tasks.append(TaskRegistry.get(t) if isinstance(t, str) else t)
      self._rates.append(float(r))

  @property
  def tasks(self):
    return list(self._tasks)

  @property
  def output_features(self):
    return self._tasks[0].output_features

  def get_dataset(self, sequence_length=None, split="train", seed=None, shard_info=None,
                  num_epochs=1, **kw) -> Dataset:
    seed = 0 if seed is None else seed
    probs = np.asarray(self._rates) / np.sum(self._rates)
    dss = [t.get_dataset(sequence_length, split=split, seed=seed, shard_info=shard_info,
                         num_epochs=None, **kw) for t in self._tasks]

    def make(start):
      rng = np.random.default_rng([seed, 7919])
      its = [iter(d) for d in dss]
      i = 0
      while True:
        k = int(rng.choice(len(its), p=probs))
        ex = next(its[k])
        if i >= start:
          yield ex
        i += 1

    return Dataset(make)


class _Registry:
  def __init__(self):
    self._items: Dict[str, Any] = {}

  def add(self, name, *args, **kwargs):
    raise NotImplementedError

  def add_provider(self, name, obj):
    self._items[name] = obj
    return obj

  def get(self, name):
    if name not in self._items:
      raise ValueError(f"'{name}' is not registered; known: {sorted(self._items)}")
    return self._items[name]

  def names(self):
    return list(self._items)

  def remove(self, name):
    self._items.pop(name, None)

  def __contains__(self, name):
    return name in self._items


class _TaskRegistry(_Registry):
  def add(self, name, source, output_features, **kwargs):
    return self.add_provider(name, Task(name, source, output_features, **kwargs))


class _MixtureRegistry(_Registry):
  def add(self, name, tasks_and_rates):
    return self.add_provider(name, Mixture(name, tasks_and_rates))


TaskRegistry = _TaskRegistry()
MixtureRegistry = _MixtureRegistry()


def get_mixture_or_task(name: str):
  if name in MixtureRegistry:
    return MixtureRegistry.get(name)
  return TaskRegistry.get(name)


def get_dataset(mixture_or_task_name, task_feature_lengths, feature_converter, dataset_split="train",
                use_cached=False, shuffle=False, num_epochs=1, shard_info=None, verbose=True,
                seed=None, batch_size=None, trim_output_features=True, **_) -> Dataset:
  """Task examples -> converted (optionally packed) model features -> optional batches."""
  mt = (get_mixture_or_task(mixture_or_task_name) if isinstance(mixture_or_task_name, str)
        else mixture_or_task_name)
  ds = mt.get_dataset(task_feature_lengths, split=dataset_split, use_cached=use_cached,
                      shuffle=shuffle, seed=seed, shard_info=shard_info, num_epochs=num_epochs,
                      trim_output_features=trim_output_features)
  ds = ds.convert(feature_converter, task_feature_lengths)
  if batch_size is not None:
    ds = ds.batch(batch_size, drop_remainder=True)
  return ds


# ----------------------------------------------------------------------------
# Built-in synthetic tasks
# ----------------------------------------------------------------------------
def _span_corruption_source(split, shard_info, seed, sequence_length=None, **_):
  sl = sequence_length or {"inputs": 512, "targets": 114}
  off = {"train": 0, "validation": 1_000_003, "test": 2_000_003}.get(split, 0)
  stream = synthetic.span_corruption_stream(seed + off, sl["inputs"], sl["targets"],
                                            shard_id=shard_info.index,
                                            num_shards=shard_info.num_shards)
  if split == "train":
    return stream
  # held-out splits are finite so that evaluation and batch inference terminate
  import itertools
  per_shard = -(-_HELD_OUT_EXAMPLES // shard_info.num_shards)
  return itertools.islice(stream, per_shard)


_HELD_OUT_EXAMPLES = 64


def _token_accuracy(targets, predictions):
  t = [str(x) for x in targets]
  p = [str(x) for x in predictions]
  return {"sequence_accuracy": 100.0 * float(np.mean([a == b for a, b in zip(t, p)])) if t else 0.0}


def register_synthetic_tasks(vocab_size: int = 32128) -> None:
  vocab = vocabularies.PassThroughVocabulary(vocab_size)
  feats = {"inputs": Feature(vocab), "targets": Feature(vocab)}
  for name in ("synthetic_span_corruption", "c4_v220_span_corruption"):
    if name not in TaskRegistry:
      TaskRegistry.add(name, _span_corruption_source, feats, metric_fns=[_token_accuracy],
                       splits=("train", "validation", "test"))


register_synthetic_tasks()
