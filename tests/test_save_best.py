"""SaveBestCheckpointer: retention by a monitored TensorBoard metric
(t5x/checkpoints.py:1462-1612; the cases of t5x/checkpoints_test.py's save-best tests)."""
import os

import pytest
import torch

from t5x_b200 import adafactor, checkpoints, models, partitioning
from t5x_b200 import train_state as ts_lib
from t5x_b200.data import vocabularies
from t5x_b200.models.t5 import network
from t5x_b200.utils import metric_writers


def _state():
  cfg = network.T5Config(vocab_size=64, dtype="float32", emb_dim=32, num_heads=2,
                         num_encoder_layers=1, num_decoder_layers=1, head_dim=16, mlp_dim=32,
                         mlp_activations=("gelu", "linear"), dropout_rate=0.0)
  module = network.Transformer(cfg)
  vocab = vocabularies.PassThroughVocabulary(64)
  model = models.EncoderDecoderModel(module, vocab, vocab, adafactor.Adafactor())
  return ts_lib.FlaxOptimTrainState.create(model.optimizer_def,
                                           model.get_initial_variables(0, None))


def _write_metric(ckpt_dir, subdir, tag, values):
  w = metric_writers.TensorBoardWriter(os.path.join(ckpt_dir, subdir))
  for step, v in values.items():
    w.write_scalars(step, {tag: v})
  w.flush()
  w.close()


def _steps(d):
  return list(checkpoints.all_steps(str(d)))


@pytest.mark.parametrize("mode,expect", [("max", [30, 40, 50]), ("min", [10, 20, 50])])
def test_keeps_the_best_by_metric_plus_the_latest(tmp_path, mode, expect):
  part = partitioning.PjitPartitioner(num_partitions=1)
  state = _state()
  _write_metric(str(tmp_path), "train", "accuracy", {10: 0.1, 20: 0.2, 30: 0.5, 40: 0.4, 50: 0.05})
  ck = checkpoints.SaveBestCheckpointer(state, part, str(tmp_path), keep=3,
                                        metric_name_to_monitor="train/accuracy",
                                        metric_mode=mode)
  for step in (10, 20, 30, 40, 50):
    ck.save(state.replace_step(step))
  # two best of the earlier ones + the latest
  assert _steps(tmp_path) == expect


def test_checkpoints_without_a_metric_and_forced_periods(tmp_path):
  part = partitioning.PjitPartitioner(num_partitions=1)
  state = _state()
  _write_metric(str(tmp_path), "training_eval/val", "loss", {10: 3.0, 20: 1.0, 30: 2.0})
  ck = checkpoints.SaveBestCheckpointer(state, part, str(tmp_path), keep=2,
                                        metric_name_to_monitor="training_eval/val/loss",
                                        metric_mode="min")
  for step in (10, 20, 30, 35, 40):
    ck.save(state.replace_step(step))
  # 35 has no metric and is kept by default; of 10/20/30 only the best (20) stays; 40 is latest
  assert _steps(tmp_path) == [20, 35, 40]
  strict = tmp_path / "strict"
  strict.mkdir()
  _write_metric(str(strict), "train", "accuracy", {10: 0.3, 20: 0.1})
  ck = checkpoints.SaveBestCheckpointer(state, part, str(strict), keep=2,
                                        keep_checkpoints_without_metrics=False,
                                        force_keep_period=15)
  for step in (10, 15, 20, 25, 30):
    ck.save(state.replace_step(step))
  # 15 and 30 are multiples of the forced period (30 is also the latest); 25 has no metric
  # and goes; of 10 / 20 the better one stays
  assert _steps(strict) == [10, 15, 30]
  with pytest.raises(ValueError, match="metric_mode"):
    checkpoints.SaveBestCheckpointer(state, part, str(tmp_path), metric_mode="median")


def test_metric_lookup_splits_directory_from_tag(tmp_path):
  _write_metric(str(tmp_path), "training_eval/task_a", "nested/accuracy", {5: 0.5, 7: 0.7})
  got = checkpoints.populate_metrics_for_steps(str(tmp_path),
                                               "training_eval/task_a/nested/accuracy", [5, 6, 7])
  assert got == {5: 0.5, 7: pytest.approx(0.7)}
  assert checkpoints.populate_metrics_for_steps(str(tmp_path), "nowhere/accuracy", [5]) == {}
