"""Metrics manager, duration timer and the stop actions of the trainer
(the behaviours exercised by t5x/trainer_test.py besides the train loop itself)."""
import os
import time

import pytest
import torch

from t5x_b200 import metrics as metrics_lib
from t5x_b200 import trainer as trainer_lib
from t5x_b200.utils import metric_writers


class _Recorder(metric_writers.MetricWriter):
  def __init__(self):
    self.scalars = []

  def write_scalars(self, step, scalars):
    self.scalars.append((step, {k: metric_writers.to_float(v) for k, v in scalars.items()}))

  def flush(self):
    pass

  def close(self):
    pass


def _manager(monkeypatch, name="train", summary_dir=None):
  rec = _Recorder()
  monkeypatch.setattr(trainer_lib.MetricsManager, "_create_writer", lambda self, n, d=None: rec)
  return trainer_lib.MetricsManager(name, summary_dir=summary_dir), rec


def test_summary_dir_is_a_subdirectory_named_after_the_manager(tmp_path):
  mm = trainer_lib.MetricsManager("eval", summary_dir=str(tmp_path))
  try:
    assert mm.summary_dir == os.path.join(str(tmp_path), "eval")
    mm.write_scalar("loss", 1.5, 3)
    mm.flush()
    assert any(f.startswith("events.out.tfevents") for f in os.listdir(mm.summary_dir))
  finally:
    mm.close()
  assert trainer_lib.MetricsManager("eval", summary_dir=None).summary_dir is None


def test_write_scalar_reaches_the_writer_with_its_step(monkeypatch):
  mm, rec = _manager(monkeypatch)
  mm.write_scalar("loss", torch.tensor(1.0), 1)
  mm.write_scalars(2, {"loss": 0.5, "accuracy": torch.tensor(0.25)})
  mm.close()
  assert rec.scalars == [(1, {"loss": 1.0}), (2, {"loss": 0.5, "accuracy": 0.25})]


def test_write_metrics_summary_fills_in_duration_and_step_count(monkeypatch):
  mm, rec = _manager(monkeypatch)
  accumulated = {
      "loss": metrics_lib.Sum(40.0),
      "accuracy": metrics_lib.Average(total=torch.tensor(20.0), count=torch.tensor(10)),
      "steps_per_second": metrics_lib.StepsPerTime(),
      "seqs_per_second": metrics_lib.TimeRate(numerator=64.0),
      "timing/seconds": metrics_lib.Time(),
      "lr": metrics_lib.AveragePerStep(total=1.0),
  }
  mm.start_duration_timer()
  time.sleep(0.05)
  summary = mm.write_metrics_summary(accumulated, step=4, num_steps=2).result()
  mm.close()
  assert summary["loss"].value == 40.0
  assert float(summary["accuracy"].value) == 2.0
  assert summary["lr"].value == pytest.approx(0.5)       # per step
  seconds = summary["timing/seconds"].value
  assert 0.04 < seconds < 5.0
  assert summary["steps_per_second"].value == pytest.approx(2 / seconds)
  assert summary["seqs_per_second"].value == pytest.approx(64 / seconds)
  (step, written), = rec.scalars
  assert step == 4 and set(written) == set(accumulated)


def test_duration_timer_needs_a_start_and_measures_wall_time():
  timer = trainer_lib._AsyncTimer()
  with pytest.raises(ValueError, match="hasn't been started"):
    timer.stop()
  timer.start()
  time.sleep(0.03)
  first = timer.stop().result()
  time.sleep(0.03)
  second = timer.stop().result()   # the same start serves several stops
  timer.close()
  assert 0.02 < first < second < 5.0


def test_summaries_are_written_in_submission_order(monkeypatch):
  mm, rec = _manager(monkeypatch)
  futures = []
  for step in range(1, 6):
    mm.start_duration_timer()
    futures.append(mm.write_metrics_summary({"loss": metrics_lib.Sum(float(step))}, step, 1))
  mm.flush()
  mm.close()
  assert [f.result()["loss"].value for f in futures] == [1.0, 2.0, 3.0, 4.0, 5.0]
  assert [s for s, _ in rec.scalars] == [1, 2, 3, 4, 5]


# ---- actions ------------------------------------------------------------------------------------
def _run(action, values, task="task", metric="loss"):
  return [action.run(None, {task: {metric: metric_writers.Scalar(v)}}) for v in values]


@pytest.mark.parametrize("mode,values,atol,rtol,expect", [
    ("min", [5.0, 4.0, 3.0, 2.0], 0.0, 0.0, [False] * 4),                 # keeps improving
    ("min", [1.0, 1.0, 1.0], 0.0, 0.0, [False, False, True]),             # flat for `patience`
    ("min", [1.0, 0.95, 0.91], 0.1, 0.0, [False, False, True]),           # gains within atol
    ("min", [1.0, 0.8, 0.6], 0.1, 0.0, [False, False, False]),            # gains beyond atol
    ("min", [10.0, 9.5, 9.1], 0.0, 0.1, [False, False, True]),            # gains within rtol
    ("max", [0.1, 0.2, 0.3, 0.4], 0.0, 0.0, [False] * 4),
    ("max", [0.5, 0.4, 0.3], 0.0, 0.0, [False, False, True]),             # getting worse
    ("max", [0.5, 0.4, 0.45, 0.3], 0.0, 0.0, [False, False, False, False]),  # one gain in window
])
def test_early_stopping_variants(mode, values, atol, rtol, expect):
  action = trainer_lib.EarlyStoppingAction(("task", "loss"), mode=mode, patience=3, atol=atol,
                                           rtol=rtol)
  assert _run(action, values) == expect


def test_early_stopping_ignores_what_it_cannot_read():
  action = trainer_lib.EarlyStoppingAction(("task", "loss"), mode="min", patience=2)
  assert action.run(None, {"other_task": {"loss": metric_writers.Scalar(1.0)}}) is False
  assert action.run(None, {"task": {"accuracy": metric_writers.Scalar(1.0)}}) is False
  assert action.run(None, {"task": {"loss": metric_writers.Text("n/a")}}) is False
  # none of those entered the window
  assert _run(action, [1.0, 1.0]) == [False, True]
  with pytest.raises(ValueError):
    trainer_lib.EarlyStoppingAction(("task", "loss"), mode="min", atol=-1.0)


@pytest.mark.parametrize("value,stop", [(1.0, False), (float("nan"), True), (float("inf"), True),
                                        (-float("inf"), True), (0.0, False)])
def test_terminate_on_nan_variants(value, stop):
  action = trainer_lib.TerminateOnNanAction(task="task", metric="loss")
  assert action.run(None, {"task": {"loss": metric_writers.Scalar(value)}}) is stop
  assert action.run(None, {"task": {"loss": value}}) is stop           # plain floats too
  assert action.run(None, {"task": {"other": metric_writers.Scalar(value)}}) is False
  assert action.run(None, {"elsewhere": {"loss": metric_writers.Scalar(value)}}) is False
