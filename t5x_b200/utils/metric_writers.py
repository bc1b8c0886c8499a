"""Metric values and writers (the clu.values / clu.metric_writers surface the trainer uses).

`TensorBoardWriter` emits standard event files via the tensorboard package's own record
writer and protos; `LoggingWriter` prints; `MultiWriter` fans out; `AsyncWriter` serialises
all calls on one background thread.
"""
from __future__ import annotations

import concurrent.futures
import dataclasses
import logging
import os
import time
from typing import Any, Mapping, Optional, Sequence

import numpy as np


@dataclasses.dataclass
class Scalar:
  value: Any


@dataclasses.dataclass
class Text:
  value: str


@dataclasses.dataclass
class Histogram:
  value: Any
  num_buckets: Optional[int] = None


def to_float(v) -> float:
  if isinstance(v, Scalar):
    v = v.value
  if hasattr(v, "detach"):
    v = v.detach().float().cpu().item() if v.numel() == 1 else v.detach().float().cpu().numpy()
  return float(np.asarray(v))


class MetricWriter:
  def write_scalars(self, step: int, scalars: Mapping[str, Any]) -> None:
    raise NotImplementedError

  def write_texts(self, step: int, texts: Mapping[str, str]) -> None:
    pass

  def write_hparams(self, hparams: Mapping[str, Any]) -> None:
    pass

  def write_histograms(self, step, arrays, num_buckets=None) -> None:
    pass

  def flush(self) -> None:
    pass

  def close(self) -> None:
    self.flush()


class LoggingWriter(MetricWriter):
  def __init__(self, collection: Optional[str] = None):
    self._prefix = f"[{collection}] " if collection else ""

  def write_scalars(self, step, scalars):
    vals = ", ".join(f"{k}={to_float(v):.6g}" for k, v in sorted(scalars.items()))
    logging.info("%s[%d] %s", self._prefix, step, vals)

  def write_texts(self, step, texts):
    for k, v in texts.items():
      logging.info("%s[%d] %s=%s", self._prefix, step, k, v[:2000])


class TensorBoardWriter(MetricWriter):
  """Writes scalars / texts as TensorBoard event files under `logdir`."""

  def __init__(self, logdir: str):
    from tensorboard.summary.writer.event_file_writer import EventFileWriter
    os.makedirs(logdir, exist_ok=True)
    self._writer = EventFileWriter(logdir)
    self.logdir = logdir

  def _add(self, step, summary):
    from tensorboard.compat.proto import event_pb2
    self._writer.add_event(event_pb2.Event(wall_time=time.time(), step=int(step),
                                           summary=summary))

  def write_scalars(self, step, scalars):
    from tensorboard.compat.proto import summary_pb2
    values = [summary_pb2.Summary.Value(tag=k, simple_value=to_float(v))
              for k, v in scalars.items()]
    self._add(step, summary_pb2.Summary(value=values))

  def write_texts(self, step, texts):
    from tensorboard.compat.proto import summary_pb2, tensor_pb2, tensor_shape_pb2, types_pb2
    vals = []
    for k, v in texts.items():
      meta = summary_pb2.SummaryMetadata(
          plugin_data=summary_pb2.SummaryMetadata.PluginData(plugin_name="text"))
      tensor = tensor_pb2.TensorProto(dtype=types_pb2.DT_STRING,
                                      string_val=[v.encode("utf-8")],
                                      tensor_shape=tensor_shape_pb2.TensorShapeProto())
      vals.append(summary_pb2.Summary.Value(tag=k, metadata=meta, tensor=tensor))
    self._add(step, summary_pb2.Summary(value=vals))

  def flush(self):
    self._writer.flush()

  def close(self):
    self._writer.close()


class MultiWriter(MetricWriter):
  def __init__(self, writers: Sequence[MetricWriter]):
    self._writers = list(writers)

  def write_scalars(self, step, scalars):
    for w in self._writers:
      w.write_scalars(step, scalars)

  def write_texts(self, step, texts):
    for w in self._writers:
      w.write_texts(step, texts)

  def write_hparams(self, hparams):
    for w in self._writers:
      w.write_hparams(hparams)

  def flush(self):
    for w in self._writers:
      w.flush()

  def close(self):
    for w in self._writers:
      w.close()


class AsyncWriter(MetricWriter):
  """Runs every call of the wrapped writer on a single worker thread, in order."""

  def __init__(self, writer: MetricWriter):
    self._writer = writer
    self._pool = concurrent.futures.ThreadPoolExecutor(max_workers=1)
    self._futures = []

  def _submit(self, fn, *a):
    self._futures.append(self._pool.submit(fn, *a))

  def write_scalars(self, step, scalars):
    self._submit(self._writer.write_scalars, step, dict(scalars))

  def write_texts(self, step, texts):
    self._submit(self._writer.write_texts, step, dict(texts))

  def write_hparams(self, hparams):
    self._submit(self._writer.write_hparams, dict(hparams))

  def flush(self):
    for f in self._futures:
      f.result()
    self._futures = []
    self._writer.flush()

  def close(self):
    self.flush()
    self._pool.shutdown(wait=True)
    self._writer.close()


def create_default_writer(logdir: Optional[str] = None, *, just_logging: bool = False,
                          asynchronous: bool = True, collection: Optional[str] = None):
  """Logging + TensorBoard on the writing host; logging only elsewhere."""
  if logdir is not None and collection is not None:
    logdir = os.path.join(logdir, collection)
  writers = [LoggingWriter(collection)]
  if not just_logging and logdir is not None:
    writers.append(TensorBoardWriter(logdir))
  w = MultiWriter(writers)
  return AsyncWriter(w) if asynchronous else w


def read_scalars(logdir: str):
  """{tag: [(step, value), ...]} from the event files of `logdir` (for SaveBestCheckpointer
  and tests)."""
  from tensorboard.backend.event_processing import event_file_loader
  out = {}
  if not os.path.isdir(logdir):
    return out
  for fn in sorted(os.listdir(logdir)):
    if "tfevents" not in fn:
      continue
    for ev in event_file_loader.LegacyEventFileLoader(os.path.join(logdir, fn)).Load():
      for v in ev.summary.value:
        if v.HasField("simple_value"):
          out.setdefault(v.tag, []).append((ev.step, v.simple_value))
  return out
