"""Metric classes (the contracts of t5x/metrics.py): sums over any rank, time and rate metrics
that refuse to compute before a duration is set, per-step averages and step rates."""
import numpy as np
import pytest
import torch

from t5x_b200 import metrics


@pytest.mark.parametrize("values, expected", [
    (2.0, 2.0),
    ([1, 2, 3], 6.0),
    ([[1, 2], [2, 3], [3, 4]], 15.0),
    ([[[1, 2], [2, 3]], [[2, 1], [3, 4]], [[3, 1], [4, 1]]], 27.0),
])
def test_sum(values, expected):
  assert float(metrics.Sum.from_model_output(values).compute()) == pytest.approx(expected)
  assert float(metrics.Sum.from_model_output(torch.tensor(values)).compute()) == pytest.approx(expected)
  assert float(metrics.Sum.from_model_output(np.asarray(values)).compute()) == pytest.approx(expected)


def test_sum_merge_adds():
  a = metrics.Sum.from_model_output([1, 2])
  b = metrics.Sum.from_model_output(4.5)
  assert float(a.merge(b).compute()) == pytest.approx(7.5)


def test_time_rate():
  metric = metrics.TimeRate.from_model_output(np.array([3.0])).replace_duration(2.0)
  assert float(metric.compute()) == pytest.approx(1.5)
  with pytest.raises(ValueError):
    metrics.TimeRate.from_model_output(np.array([3.0])).compute()


def test_time():
  assert float(metrics.Time().replace_duration(2.0).compute()) == pytest.approx(2.0)
  with pytest.raises(ValueError):
    metrics.Time().compute()


@pytest.mark.parametrize("values, expected", [(2.0, 2.0), ([1, 2, 3], 6.0)])
def test_average_per_step(values, expected):
  a = metrics.AveragePerStep.from_model_output(values)
  m = metrics.set_step_metrics_num_steps({"a": a}, 1)
  assert float(m["a"].compute()) == pytest.approx(expected)
  b = metrics.AveragePerStep.from_model_output(values, steps=5)
  m = metrics.set_step_metrics_num_steps({"b": b}, 5)
  assert float(m["b"].compute()) == pytest.approx(expected / 5)


def test_steps_per_time():
  metric = metrics.StepsPerTime.from_model_output(steps=8.0).replace_duration(2.0)
  out = metrics.set_step_metrics_num_steps({"metric": metric}, 8.0)
  assert float(out["metric"].compute()) == pytest.approx(4.0)


def test_duration_and_step_setters_touch_only_their_kind():
  tree = {"loss": metrics.Sum.from_model_output(3.0),
          "rate": metrics.TimeRate.from_model_output(10.0),
          "time": metrics.Time(),
          "per_step": metrics.AveragePerStep.from_model_output(6.0),
          "steps_per_s": metrics.StepsPerTime.from_model_output()}
  tree = metrics.set_time_metrics_duration(tree, 4.0)
  tree = metrics.set_step_metrics_num_steps(tree, 3)
  assert float(tree["loss"].compute()) == pytest.approx(3.0)
  assert float(tree["rate"].compute()) == pytest.approx(2.5)
  assert float(tree["time"].compute()) == pytest.approx(4.0)
  assert float(tree["per_step"].compute()) == pytest.approx(2.0)
  assert float(tree["steps_per_s"].compute()) == pytest.approx(0.75)
