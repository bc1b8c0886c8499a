"""A small checkpointable dataset abstraction (the role tf.data plays for the reference).

`Dataset` wraps a factory `make(start_index) -> iterator` so that the position of an iterator
can be saved and restored exactly (dataset checkpoints `train_ds-XXX-of-YYY`), batched,
sharded by `ShardInfo`, prefetched on a background thread, and peeked asynchronously.
"""
from __future__ import annotations

import concurrent.futures
import dataclasses
import itertools
import json
import os
import queue
import threading
from typing import Any, Callable, Dict, Iterable, Iterator, Mapping, Optional, Sequence

import numpy as np


@dataclasses.dataclass
class ShardInfo:
  index: int
  num_shards: int


class Dataset:
  """An iterable of dict-of-ndarray examples built from a restartable factory."""

  def __init__(self, make: Callable[[int], Iterator[Dict[str, np.ndarray]]],
               element_spec: Optional[Mapping[str, Any]] = None, cardinality: Optional[int] = None):
    self._make = make
    self._element_spec = element_spec
    self._cardinality = cardinality

  @classmethod
  def from_examples(cls, examples: Sequence[Mapping[str, Any]]) -> "Dataset":
    examples = list(examples)
    return cls(lambda start: iter(examples[start:]), cardinality=len(examples))

  @classmethod
  def from_generator_fn(cls, fn: Callable[[], Iterable], cardinality=None) -> "Dataset":
    return cls(lambda start: itertools.islice(iter(fn()), start, None), cardinality=cardinality)

  # -- transformations ---------------------------------------------------------------------
  def map(self, fn) -> "Dataset":
    return Dataset(lambda start: (fn(x) for x in self._make(start)), cardinality=self._cardinality)

  def enumerate(self) -> "Dataset":
    return Dataset(lambda start: ((start + i, x) for i, x in enumerate(self._make(start))),
                   cardinality=self._cardinality)

  def take(self, n: int) -> "Dataset":
    card = n if self._cardinality is None else min(n, self._cardinality)
    return Dataset(lambda start: itertools.islice(self._make(start), max(0, n - start)),
                   cardinality=card)

  def skip(self, n: int) -> "Dataset":
    card = None if self._cardinality is None else max(0, self._cardinality - n)
    return Dataset(lambda start: self._make(start + n), cardinality=card)

  def repeat(self) -> "Dataset":
    if self._cardinality is None:
      return self
    n = self._cardinality

    def make(start):
      epoch, off = divmod(start, max(1, n))
      it = self._make(off)
      while True:
        yield from it
        it = self._make(0)
    return Dataset(make, cardinality=None)

  def shard(self, num_shards: int, index: int) -> "Dataset":
    card = None if self._cardinality is None else (
        (self._cardinality - index + num_shards - 1) // num_shards)
    return Dataset(lambda start: itertools.islice(self._make(0), index + start * num_shards, None,
                                                  num_shards), cardinality=card)

  def batch(self, batch_size: int, drop_remainder: bool = True) -> "Dataset":
    def make(start):
      it = self._make(start * batch_size)
      while True:
        items = list(itertools.islice(it, batch_size))
        if not items or (len(items) < batch_size and drop_remainder):
          return
        yield _stack(items)
    card = None
    if self._cardinality is not None:
      card = (self._cardinality // batch_size if drop_remainder
              else -(-self._cardinality // batch_size))
    return Dataset(make, cardinality=card)

  def padded_batch(self, batch_size: int) -> "Dataset":
    return self.batch(batch_size, drop_remainder=False)

  def convert(self, converter, task_feature_lengths) -> "Dataset":
    """Applies a feature converter (which may pack several examples into one row)."""
    if getattr(converter, "pack", False):
      # Packing changes the example count; positions restart from the beginning on restore.
      def make(start):
        return itertools.islice(converter(self._make(0), task_feature_lengths), start, None)
      return Dataset(make)
    return Dataset(lambda start: converter(self._make(start), task_feature_lengths),
                   cardinality=self._cardinality)

  # -- consumption -------------------------------------------------------------------------
  def cardinality(self) -> Optional[int]:
    return self._cardinality

  def __len__(self):
    if self._cardinality is None:
      raise TypeError("dataset has unknown / infinite length")
    return self._cardinality

  def __iter__(self) -> "DatasetIterator":
    return DatasetIterator(self)

  def as_numpy_iterator(self):
    return iter(self)

  @property
  def element_spec(self):
    if self._element_spec is None:
      first = next(self._make(0))
      self._element_spec = _spec_of(first)
    return self._element_spec


def _spec_of(x):
  if isinstance(x, Mapping):
    return {k: _spec_of(v) for k, v in x.items()}
  if isinstance(x, tuple):
    return tuple(_spec_of(v) for v in x)
  a = np.asarray(x)
  return TensorSpec(tuple(a.shape), a.dtype)


@dataclasses.dataclass(frozen=True)
class TensorSpec:
  shape: tuple
  dtype: Any


def _stack(items):
  first = items[0]
  if isinstance(first, Mapping):
    return {k: _stack([it[k] for it in items]) for k in first}
  if isinstance(first, tuple):
    return tuple(_stack([it[i] for it in items]) for i in range(len(first)))
  if isinstance(first, (str, bytes)):
    return np.asarray(items, dtype=object)
  return np.stack([np.asarray(i) for i in items])


class DatasetIterator:
  """Iterator with an exact position that can be saved / restored, `peek`, and `peek_async`
  (the clu DatasetIterator contract used by t5x/train.py:385 and t5x/checkpoints.py:793-806)."""

  def __init__(self, dataset: Dataset, start: int = 0):
    self._dataset = dataset
    self._index = start
    self._it = dataset._make(start)
    self._peeked = []
    self._lock = threading.Lock()
    self._pool = None

  @property
  def element_spec(self):
    return self._dataset.element_spec

  def __iter__(self):
    return self

  def __next__(self):
    with self._lock:
      if self._peeked:
        item = self._peeked.pop(0)
      else:
        item = next(self._it)
      self._index += 1
      return item

  def peek(self):
    with self._lock:
      if not self._peeked:
        self._peeked.append(next(self._it))
      return self._peeked[0]

  def peek_async(self) -> concurrent.futures.Future:
    if self._pool is None:
      self._pool = concurrent.futures.ThreadPoolExecutor(max_workers=1)
    return self._pool.submit(self.peek)

  def reset(self):
    self.set_position(0)

  def set_position(self, index: int):
    with self._lock:
      self._index = index
      self._it = self._dataset._make(index)
      self._peeked = []

  def save(self, filename: str) -> None:
    os.makedirs(os.path.dirname(filename) or ".", exist_ok=True)
    tmp = filename + ".tmp"
    with open(tmp, "w") as f:
      json.dump({"index": self._index}, f)
    os.replace(tmp, filename)

  def restore(self, filename: str) -> None:
    with open(filename) as f:
      self.set_position(int(json.load(f)["index"]))

  # aliases used by the checkpointer
  def get_state(self) -> dict:
    return {"index": self._index}

  def set_state(self, state: Mapping[str, Any]) -> None:
    self.set_position(int(state["index"]))


class PrefetchIterator:
  """Runs the wrapped iterator on a background thread, `depth` batches ahead. Each element may
  be post-processed on that thread (e.g. copied into pinned memory)."""

  _END = object()

  def __init__(self, it, depth: int = 2, transform: Optional[Callable] = None):
    self._it = it
    self._q: "queue.Queue" = queue.Queue(maxsize=depth)
    self._transform = transform
    self._thread = threading.Thread(target=self._run, daemon=True)
    self._error = None
    self._thread.start()

  def _run(self):
    try:
      for x in self._it:
        self._q.put(self._transform(x) if self._transform else x)
    except BaseException as e:  # surfaced on the consumer side
      self._error = e
    self._q.put(self._END)

  def __iter__(self):
    return self

  def __next__(self):
    x = self._q.get()
    if x is self._END:
      if self._error is not None:
        raise self._error
      raise StopIteration
    return x
