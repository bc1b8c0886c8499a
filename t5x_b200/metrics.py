"""Metric objects (API of t5x/metrics.py plus the few CLU base classes it builds on).

A metric is an immutable dataclass with `merge` and `compute`. Values may be device
tensors: merging stays on the device and nothing synchronises until `compute` results
are turned into Python floats by the writer thread.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Mapping, Optional

import numpy as np
import torch

Scalar = Any


def _asarray(v):
  if isinstance(v, torch.Tensor):
    return v.detach()
  return torch.as_tensor(v)


@dataclasses.dataclass(frozen=True)
class Metric:
  """Base class: `from_model_output`, `merge`, `compute` (clu.metrics.Metric contract)."""

  @classmethod
  def from_model_output(cls, *args, **kwargs) -> "Metric":
    raise NotImplementedError

  def merge(self, other: "Metric") -> "Metric":
    raise NotImplementedError

  def compute(self):
    raise NotImplementedError

  def compute_value(self):
    from t5x_b200.utils import metric_writers
    return metric_writers.Scalar(self.compute())

  def replace(self, **kw):
    return dataclasses.replace(self, **kw)


@dataclasses.dataclass(frozen=True)
class Average(Metric):
  total: Scalar = 0.0
  count: Scalar = 0

  @classmethod
  def from_model_output(cls, values, mask=None, **_):
    values = _asarray(values).float()
    if values.dim() == 0:
      values = values[None]
    if mask is None:
      return cls(total=values.sum(), count=float(values.numel()))
    mask = _asarray(mask).to(values.dtype)
    while mask.dim() < values.dim():
      mask = mask[..., None]
    mask = mask.expand_as(values)
    return cls(total=(values * mask).sum(), count=mask.sum())

  def merge(self, other):
    return type(self)(total=self.total + other.total, count=self.count + other.count)

  def compute(self):
    return self.total / self.count


@dataclasses.dataclass(frozen=True)
class Accuracy(Average):
  """Fraction of positions where argmax(logits) == labels, under an optional mask."""

  @classmethod
  def from_model_output(cls, logits=None, labels=None, mask=None, correct=None, **_):
    if correct is None:
      correct = (logits.argmax(-1) == labels)
    return super().from_model_output(values=_asarray(correct).float(), mask=mask)


@dataclasses.dataclass(frozen=True)
class LastValue(Metric):
  value: Scalar = 0.0

  @classmethod
  def from_model_output(cls, value, **_):
    return cls(value=_asarray(value))

  def merge(self, other):
    return other

  def compute(self):
    return self.value


@dataclasses.dataclass(frozen=True)
class Sum(Metric):
  """Sum of a scalar or a batch of values (t5x/metrics.py:52-81)."""
  total: Scalar = 0.0

  @classmethod
  def from_model_output(cls, values, **_):
    values = _asarray(values)
    if values.dim() == 0:
      values = values[None]
    return cls(total=values.sum())

  def merge(self, other):
    return type(self)(total=self.total + other.total)

  def compute(self):
    return self.total


@dataclasses.dataclass(frozen=True)
class Step(Metric):
  """Tracks a step count that the trainer sets after the (micro-batched) step
  (t5x/metrics.py:84-107)."""
  steps: Optional[int] = 1

  def replace_steps(self, steps):
    return self.replace(steps=steps)

  def compute(self):
    if self.steps is None:
      raise ValueError("`steps` must be set by calling `replace_steps` before computing metric.")
    return self.steps


@dataclasses.dataclass(frozen=True)
class AveragePerStep(Step):
  """total / number of steps (t5x/metrics.py:110-147)."""
  total: Optional[Scalar] = None

  @classmethod
  def from_model_output(cls, values, steps: Optional[int] = 1, **_):
    values = _asarray(values)
    if values.dim() == 0:
      values = values[None]
    return cls(total=values.sum(), steps=steps)

  def merge(self, other):
    assert type(self) is type(other)
    return type(self)(total=self.total + other.total, steps=self.steps + other.steps)

  def compute(self):
    steps = Step.compute(self)
    if self.total is None:
      raise ValueError("`AveragePerStep` `total` cannot be None.")
    return self.total / steps


@dataclasses.dataclass(frozen=True)
class Time(Metric):
  """A duration set on the host after the step ran (t5x/metrics.py:150-186)."""
  duration: Optional[Scalar] = None

  def merge(self, other):
    return self

  def compute(self):
    if self.duration is None:
      raise ValueError(
          "`Time` `duration` must be set by calling `replace_duration` before computing.")
    return self.duration

  def replace_duration(self, duration):
    return self.replace(duration=duration)


@dataclasses.dataclass(frozen=True)
class TimeRate(Time):
  """numerator / duration (t5x/metrics.py:189-221)."""
  numerator: Optional[Scalar] = None

  @classmethod
  def from_model_output(cls, numerator, **_):
    return cls(numerator=numerator)

  def merge(self, other):
    assert self.duration is None and other.duration is None, (
        "Merging with non-None durations is currently not supported.")
    return type(self)(numerator=self.numerator + other.numerator)

  def compute(self):
    return self.numerator / Time.compute(self)


@dataclasses.dataclass(frozen=True)
class StepsPerTime(Step, Time):
  """steps / duration (t5x/metrics.py:224-250)."""

  @classmethod
  def from_model_output(cls, steps: Optional[int] = 1, **_):
    return cls(steps=steps)

  def merge(self, other):
    assert type(self) is type(other)
    return type(self)(steps=self.steps + other.steps)

  def compute(self):
    return Step.compute(self) / Time.compute(self)


def is_metric_obj(obj) -> bool:
  return isinstance(obj, Metric)


def is_time_metric(obj) -> bool:
  return isinstance(obj, Time)


def create_metrics_dict(float_metrics_dict: Mapping[str, Any]):
  return {k: Sum(v) for k, v in float_metrics_dict.items()}


def shape_obj_to_defined_obj(obj: Metric) -> Metric:
  """Zero-valued metric of the same class/shape (t5x/metrics.py:262-289)."""
  vals = {}
  for f in dataclasses.fields(obj):
    a = getattr(obj, f.name)
    if isinstance(a, Metric):
      vals[f.name] = shape_obj_to_defined_obj(a)
    elif hasattr(a, "shape"):
      vals[f.name] = torch.zeros(tuple(a.shape), dtype=getattr(a, "dtype", torch.float32))
    else:
      vals[f.name] = a
  return obj.__class__(**vals)


def set_time_metrics_duration(metrics, duration):
  return {k: (m.replace_duration(duration) if isinstance(m, Time) else m)
          for k, m in metrics.items()}


def set_step_metrics_num_steps(metrics, num_steps):
  return {k: (m.replace_steps(num_steps) if isinstance(m, Step) else m)
          for k, m in metrics.items()}


def merge_metrics(a, b):
  """Key-wise merge of two metric dicts (t5x/trainer.py:69-84)."""
  if a is None:
    return b
  if b is None:
    return a
  return {k: a[k].merge(b[k]) for k in a}
