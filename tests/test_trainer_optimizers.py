"""Trainer loop, microbatching, RNG fold-in, actions, schedules and the optax-style optimizers
(cases after t5x/trainer_test.py, t5x/optimizers_test.py, t5x/utils_test.py)."""
import os

import numpy as np
import pytest
import torch

from t5x_b200 import adafactor, metrics as metrics_lib, models, optimizers
from t5x_b200 import train_state as ts, trainer as trainer_lib
from t5x_b200.utils import metric_writers, schedules


class _LinearModel(models.BaseModel):
  """y = x @ w; loss = sum of squared errors (a sum, as in the reference: global = sum of shards)."""

  def __init__(self, optimizer_def):
    super().__init__(optimizer_def)
    self.w = torch.nn.Parameter(torch.zeros(4, 2))
    self.w.axes = ("embed", "mlp")

  def get_initial_variables(self, rng, input_shapes, input_types=None):
    return {"params": {"w": self.w}, "params_axes": {"w": ("embed", "mlp")}}

  def loss_fn(self, params, batch, dropout_rng):
    err = batch["x"].float() @ params["w"] - batch["y"].float()
    loss = (err ** 2).sum()
    rng_val = torch.tensor(float(dropout_rng if dropout_rng is not None else -1))
    return loss, {"loss": metrics_lib.Sum(total=loss.detach()),
                  "rng": metrics_lib.LastValue(value=rng_val),
                  "examples": metrics_lib.Sum(total=torch.tensor(float(batch["x"].shape[0])))}

  def eval_fn(self, params, batch):
    return self.loss_fn(params, batch, None)

  def predict_batch_with_aux(self, params, batch, rng=None):
    return batch["x"].float() @ params["w"], {}

  def score_batch(self, params, batch, return_intermediates=False):
    return -((batch["x"].float() @ params["w"] - batch["y"].float()) ** 2).sum(-1)


def _batches(n, bs=8, seed=0):
  g = torch.Generator().manual_seed(seed)
  w_true = torch.tensor([[1.0, -1.0], [0.5, 2.0], [0.0, 1.0], [-2.0, 0.3]])
  out = []
  for _ in range(n):
    x = torch.randn(bs, 4, generator=g)
    out.append({"x": x.numpy(), "y": (x @ w_true).numpy()})
  return out


def _trainer(tmp_path, num_microbatches=None, opt=None, lr=0.05):
  model = _LinearModel(opt or optimizers.sgd(learning_rate=None))
  state = ts.FlaxOptimTrainState.create(model.optimizer_def,
                                        model.get_initial_variables(None, None))
  return trainer_lib.Trainer(model, state, None, ["val"], str(tmp_path), None, rng=17,
                             learning_rate_fn=lambda step: lr,
                             num_microbatches=num_microbatches), model


def test_train_loop_reduces_loss_and_counts_steps(tmp_path):
  tr, model = _trainer(tmp_path)
  data = _batches(30)
  first = tr.train(iter(data[:10]), 10).result()
  last = tr.train(iter(data[10:]), 20).result()
  assert int(tr.train_state.step) == 30
  assert float(last["loss"].value) < float(first["loss"].value)
  assert float(last["examples"].value) == 160.0
  assert float(last["learning_rate"].value) == pytest.approx(0.05)
  tr.close()
  assert any(f.startswith("events") or f.endswith(".jsonl") or os.path.isdir(os.path.join(tmp_path, f))
             for f in os.listdir(tmp_path))


def test_microbatching_matches_full_batch(tmp_path):
  data = _batches(3)
  tr1, m1 = _trainer(tmp_path / "a", num_microbatches=None)
  tr4, m4 = _trainer(tmp_path / "b", num_microbatches=4)
  s1 = tr1.train(iter(data), 3).result()
  s4 = tr4.train(iter(data), 3).result()
  torch.testing.assert_close(m1.w.detach(), m4.w.detach(), rtol=1e-5, atol=1e-6)
  assert float(s1["loss"].value) == pytest.approx(float(s4["loss"].value), rel=1e-5)
  with pytest.raises(ValueError):
    _trainer(tmp_path / "c", num_microbatches=3)[0].train(iter(data), 1)


def test_step_rng_is_folded_from_base_and_step(tmp_path):
  tr, _ = _trainer(tmp_path)
  a = tr.train(iter(_batches(1)), 1, start_step=5).result()
  tr2, _ = _trainer(tmp_path / "again")
  b = tr2.train(iter(_batches(1)), 1, start_step=5).result()
  c = tr2.train(iter(_batches(1)), 1, start_step=6).result()
  assert float(a["rng"].value) == float(b["rng"].value) != float(c["rng"].value)
  assert trainer_lib.fold_in_seed(17, 5) == trainer_lib.fold_in_seed(17, 5)
  assert trainer_lib.fold_in_seed(17, 5) != trainer_lib.fold_in_seed(18, 5)


def test_eval_summaries(tmp_path):
  tr, _ = _trainer(tmp_path)
  out = tr.eval({"val": iter(_batches(4, seed=3))})
  assert float(out["val"]["examples"].value) == 32.0 and "loss" in out["val"]


def test_actions():
  early = trainer_lib.EarlyStoppingAction(("task", "loss"), mode="min", patience=3, atol=0.0)
  vals = [3.0, 2.0, 2.5, 2.6]
  stops = [early.run(None, {"task": {"loss": metric_writers.Scalar(v)}}) for v in vals]
  # stops once the last `patience` values show no improvement from one to the next
  assert stops == [False, False, False, True]
  assert early.run(None, {"other": {}}) is False
  nan = trainer_lib.TerminateOnNanAction(task="task", metric="loss")
  assert nan.run(None, {"task": {"loss": metric_writers.Scalar(1.0)}}) is False
  assert nan.run(None, {"task": {"loss": metric_writers.Scalar(float("nan"))}}) is True
  with pytest.raises(ValueError):
    trainer_lib.EarlyStoppingAction(("task", "loss"), mode="sideways")


def test_learning_rate_schedules():
  f = schedules.create_learning_rate_scheduler("constant * linear_warmup * rsqrt_decay", 2.0, 100)
  assert f(0) == pytest.approx(1e-8) and f(50) == pytest.approx(2.0 * 0.5 / 10.0)
  assert f(400) == pytest.approx(2.0 / 20.0)
  g = schedules.create_learning_rate_scheduler("constant * rsqrt_decay", 1.0, 10000)
  assert g(0) == pytest.approx(0.01) and g(40000) == pytest.approx(0.005)
  h = schedules.create_learning_rate_scheduler("constant * decay_every", 1.0, decay_factor=0.5,
                                               steps_per_decay=10)
  assert h(25) == pytest.approx(0.25)
  with pytest.raises(ValueError):
    schedules.create_learning_rate_scheduler("constant * nope")


# ---- optimizers -----------------------------------------------------------------------------
def _run(opt_def, steps=3, lr=0.1):
  torch.manual_seed(0)
  p = {"a": torch.randn(3, 2), "b": {"c": torch.randn(4)}}
  opt = opt_def.create(p)
  for i in range(steps):
    g = {"a": torch.full((3, 2), 0.5 + i), "b": {"c": torch.arange(4.0) - i}}
    opt = opt.apply_gradient(g, learning_rate=lr)
  return opt


def test_sgd_and_adam_match_torch_optim():
  for mine, theirs in [(optimizers.sgd(None, momentum=0.9),
                        lambda ps: torch.optim.SGD(ps, lr=0.1, momentum=0.9)),
                       (optimizers.adam(None, b1=0.9, b2=0.999, eps=1e-8),
                        lambda ps: torch.optim.Adam(ps, lr=0.1, betas=(0.9, 0.999), eps=1e-8)),
                       (optimizers.adamw(None, weight_decay=0.01),
                        lambda ps: torch.optim.AdamW(ps, lr=0.1, weight_decay=0.01))]:
    torch.manual_seed(0)
    a = torch.nn.Parameter(torch.randn(3, 2))
    c = torch.nn.Parameter(torch.randn(4))
    ref = theirs([a, c])
    for i in range(3):
      a.grad = torch.full((3, 2), 0.5 + i)
      c.grad = torch.arange(4.0) - i
      ref.step()
    opt = _run(mine)
    torch.testing.assert_close(opt.target["a"], a.detach(), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(opt.target["b"]["c"], c.detach(), rtol=1e-4, atol=1e-5)
    assert int(opt.state.step) == 3


def test_optimizer_state_dict_round_trip_and_chain():
  opt = _run(optimizers.adam(None))
  sd = opt.state_dict()
  assert set(sd) == {"target", "state"} and int(sd["state"]["step"]) == 3
  fresh = optimizers.adam(None).create({"a": torch.zeros(3, 2), "b": {"c": torch.zeros(4)}})
  restored = fresh.restore_state(sd)
  torch.testing.assert_close(restored.target["a"], opt.target["a"])
  assert int(restored.state.step) == 3
  chained = optimizers.chain([optimizers.clip_by_global_norm(1.0), optimizers.scale(-0.1)])
  out = chained.create({"w": torch.zeros(2)}).apply_gradient({"w": torch.tensor([3.0, 4.0])})
  torch.testing.assert_close(out.target["w"], torch.tensor([-0.06, -0.08]))


def test_multi_optimizer_routes_parameters():
  """Two Adafactor variants over disjoint parameter sets (parameter scaling on / off), the
  arrangement the reference uses to exclude some variables from scaling."""
  sel_a = optimizers.ModelParamTraversal(lambda path, _: "a" in path.split("/"))
  sel_rest = optimizers.ModelParamTraversal(lambda path, _: "a" not in path.split("/"))
  scaled = adafactor.Adafactor(min_dim_size_to_factor=0)
  unscaled = adafactor.Adafactor(min_dim_size_to_factor=0, multiply_by_parameter_scale=False)
  mo = optimizers.MultiOptimizer(((sel_a, scaled), (sel_rest, unscaled)))
  p = {"a": 2.0 * torch.ones(4, 4), "b": {"c": 2.0 * torch.ones(4, 4)}}
  g = {"a": torch.ones(4, 4), "b": {"c": torch.ones(4, 4)}}
  opt = mo.create(p).apply_gradient(g, learning_rate=0.5)
  # identical gradients: the scaled update is RMS(p) = 2 times the unscaled one
  da = 2.0 - opt.target["a"]
  dc = 2.0 - opt.target["b"]["c"]
  torch.testing.assert_close(da, 2.0 * dc, rtol=1e-5, atol=1e-6)
  sd = opt.state_dict()
  assert "v_row" in sd["state"]["param_states"]["b"]["c"] and int(sd["state"]["step"]) == 1
  with pytest.raises(ValueError):
    optimizers.MultiOptimizer(((sel_a, scaled), (sel_a, unscaled))).create(p)
