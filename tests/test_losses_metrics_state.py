"""Losses, metrics, state-dict utilities and checkpoint bookkeeping helpers
(cases after t5x/losses_test.py, t5x/metrics_test.py, t5x/state_utils_test.py,
t5x/checkpoint_utils_test.py)."""
import os

import numpy as np
import pytest
import torch

from t5x_b200 import checkpoint_utils, checkpoints_utils, losses, metrics, state_utils


# ---- losses ---------------------------------------------------------------------------------
def test_cross_entropy_with_z_loss_value_and_gradient():
  torch.manual_seed(0)
  logits = torch.randn(2, 4, 8, dtype=torch.float64, requires_grad=True)
  targets = torch.nn.functional.one_hot(torch.randint(0, 8, (2, 4)), 8).double()
  z = 0.1
  loss, z_loss = losses.cross_entropy_with_logits(logits, targets, z_loss=z)
  lse = torch.logsumexp(logits, -1)
  expect = lse - (logits * targets).sum(-1) + z * lse ** 2
  torch.testing.assert_close(loss, expect.detach())
  torch.testing.assert_close(z_loss.double(), (z * lse ** 2).detach(), rtol=1e-5, atol=1e-6)
  (g,) = torch.autograd.grad(loss.sum(), logits)
  (g_ref,) = torch.autograd.grad(expect.sum(), logits)
  torch.testing.assert_close(g, g_ref)


def test_weighted_cross_entropy_label_smoothing_and_normalisation():
  torch.manual_seed(1)
  logits = torch.randn(2, 3, 5)
  targets = torch.tensor([[1, 2, 0], [4, 0, 0]])
  weights = (targets > 0).float()
  loss, z_loss, wsum = losses.compute_weighted_cross_entropy(
      logits, targets, weights, label_smoothing=0.1, z_loss=0.0, loss_normalizing_factor=2.0)
  conf, low = 0.9, 0.1 / 4
  soft = torch.full((2, 3, 5), low).scatter_(-1, targets[..., None], conf)
  lp = torch.log_softmax(logits, -1)
  # the constant that makes a perfect prediction score zero is subtracted
  const = -(conf * np.log(conf) + 4 * low * np.log(low + 1e-20))
  expect = ((-(soft * lp).sum(-1) - const) * weights).sum() / 2.0
  assert float(loss) == pytest.approx(float(expect), rel=1e-5)
  assert float(wsum) == 3.0 and float(z_loss) == 0.0


def test_special_loss_normalizing_factors():
  batch = {"decoder_target_tokens": torch.tensor([[1, 2, 3, 4, 0], [5, 6, 0, 0, 0]])}
  lnf, w = losses.get_loss_normalizing_factor_and_weights(
      losses.SpecialLossNormalizingFactor.NUM_REAL_TARGET_TOKENS, batch)
  assert float(lnf) == 6.0
  assert w.tolist() == [[1, 1, 1, 1, 0], [1, 1, 0, 0, 0]]
  lnf, _ = losses.get_loss_normalizing_factor_and_weights("NUM_TOTAL_TARGET_TOKENS", batch)
  assert float(lnf) == 10.0
  batch["decoder_segment_ids"] = torch.tensor([[1, 1, 2, 2, 0], [1, 1, 0, 0, 0]])
  batch["decoder_positions"] = torch.tensor([[0, 1, 0, 1, 0], [0, 1, 0, 0, 0]])
  lnf, w = losses.get_loss_normalizing_factor_and_weights("AVERAGE_PER_SEQUENCE", batch)
  # three packed sequences of two tokens each: every token weighs 1/2
  assert float(lnf) == 3.0
  np.testing.assert_allclose(w.numpy(), [[.5, .5, .5, .5, 0], [.5, .5, 0, 0, 0]])
  lnf, w = losses.get_loss_normalizing_factor_and_weights(7.0, batch)
  assert lnf == 7.0 and w is None or float(lnf) == 7.0


# ---- metrics --------------------------------------------------------------------------------
def test_metric_algebra():
  s = metrics.Sum.from_model_output(torch.tensor([1.0, 2.0])).merge(
      metrics.Sum.from_model_output(torch.tensor([3.0])))
  assert float(s.compute()) == 6.0
  a = metrics.AveragePerStep.from_model_output(torch.tensor(4.0)).merge(
      metrics.AveragePerStep.from_model_output(torch.tensor(8.0)))
  assert float(a.compute()) == 6.0  # (4 + 8) / 2 steps
  assert float(a.replace_steps(4).compute()) == 3.0
  rate = metrics.TimeRate.from_model_output(numerator=torch.tensor(100.0)).replace_duration(4.0)
  assert float(rate.compute()) == 25.0
  with pytest.raises(ValueError):
    metrics.TimeRate.from_model_output(numerator=torch.tensor(1.0)).compute()
  spt = metrics.StepsPerTime.from_model_output().merge(metrics.StepsPerTime.from_model_output())
  assert float(spt.replace_duration(0.5).compute()) == 4.0
  acc = metrics.Accuracy.from_model_output(
      logits=torch.tensor([[[0.1, 0.9], [0.8, 0.2]]]), labels=torch.tensor([[1, 1]]),
      mask=torch.tensor([[1.0, 1.0]]))
  assert float(acc.compute()) == 0.5
  d = {"t": metrics.Time(), "r": metrics.TimeRate.from_model_output(numerator=torch.tensor(6.0)),
       "s": metrics.Sum(total=torch.tensor(2.0))}
  d = metrics.set_time_metrics_duration(d, 3.0)
  assert float(d["r"].compute()) == 2.0 and float(d["t"].compute()) == 3.0
  merged = metrics.merge_metrics({"s": metrics.Sum(total=torch.tensor(1.0))},
                                 {"s": metrics.Sum(total=torch.tensor(2.0))})
  assert float(merged["s"].compute()) == 3.0


# ---- state utils ----------------------------------------------------------------------------
def test_intersect_and_merge_state():
  assert state_utils.intersect_state({"a": {"b": 2, "c": 3}}, {"a": {"b": 4}, "d": 5}) == \
      {"a": {"b": 2}}
  assert state_utils.merge_state({"a": {"b": 2, "c": 3}}, {"a": {"b": 4}, "d": 5}) == \
      {"a": {"b": 2, "c": 3}, "d": 5}


def test_tensorstore_leaf_detection_and_flatten():
  spec = {"driver": "zarr", "kvstore": {"driver": "file", "path": "target.bias"},
          "metadata": {"chunks": [4, 1], "dtype": "<f4", "shape": [4, 1]}}
  assert state_utils.tensorstore_leaf(None, spec)
  assert not state_utils.tensorstore_leaf(None, {"driver": np.ones((4, 4))})
  flat = state_utils.flatten_state_dict({"target": {"a": {"b": 3}}, "ts": spec})
  assert flat == {"target/a/b": 3, "ts": spec}
  assert state_utils.get_name_tree({"a": {"b": 1}, "c": 2}) == {"a": {"b": "a/b"}, "c": "c"}


def test_assignment_map():
  # new keys foo/bar and foo/baz both read the checkpoint's `fandangle`; unmapped model keys
  # that exist in the checkpoint keep their own value
  result = state_utils.apply_assignment_map(
      ckpt_optimizer_state={"fandangle": 1234, "food": 31},
      optimizer_state={"foo": {"bar": 0, "baz": 0}, "food": 0},
      assignment_map=[(r"foo/bar", "fandangle"), (r"foo/baz", "fandangle")])
  assert result["foo"] == {"bar": 1234, "baz": 1234} and result["food"] == 31
  # capture groups, and None to leave a key to its initial value
  result = state_utils.apply_assignment_map(
      ckpt_optimizer_state={"old": {"w0": 1, "w1": 2}},
      optimizer_state={"new": {"w0": 0, "w1": 0, "extra": 0}},
      assignment_map=[(r"new/(w\d)", r"old/\1"), (r"new/extra", None)])
  assert result["new"]["w0"] == 1 and result["new"]["w1"] == 2 and "extra" not in result["new"]
  with pytest.raises(ValueError):
    state_utils.apply_assignment_map({"a": 1}, {"b": 0}, [(r"b", "missing")])
  # a resuming run ignores the map entirely
  same = state_utils.apply_assignment_map({"a": 1}, {"b": 0}, [(r"b", "a")], is_resuming=True)
  assert same == {"a": 1}


# ---- checkpoint bookkeeping -----------------------------------------------------------------
def test_pinning_and_step_listing(tmp_path):
  for s in (10, 2, 300):
    os.makedirs(tmp_path / f"checkpoint_{s}")
  os.makedirs(tmp_path / "checkpoint_7.tmp-123")
  os.makedirs(tmp_path / "train_ds-5")
  assert list(checkpoints_utils.all_steps(str(tmp_path))) == [2, 10, 300]
  assert checkpoints_utils.latest_step(str(tmp_path)) == 300
  assert checkpoints_utils.get_checkpoint_dir(str(tmp_path), 10).endswith("checkpoint_10")
  d = str(tmp_path / "checkpoint_10")
  assert not checkpoint_utils.is_pinned_checkpoint(d)
  checkpoint_utils.pin_checkpoint(d)
  assert checkpoint_utils.is_pinned_checkpoint(d)
  checkpoint_utils.remove_checkpoint_dir(d)      # pinned: kept
  assert os.path.isdir(d)
  checkpoint_utils.unpin_checkpoint(d)
  checkpoint_utils.remove_checkpoint_dir(d)
  assert not os.path.isdir(d)
