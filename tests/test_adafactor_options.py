"""Adafactor options on the CPU against an independent numpy statement of the update:
momentum, weight decay (with the learning-rate exponent), parameter-scale switches and caps,
unfactored statistics, step offsets, NaN skipping and per-parameter hyper-parameter maps
(the equivalences checked by t5x/adafactor_test.py)."""
import numpy as np
import pytest
import torch

from t5x_b200 import adafactor
from t5x_b200.utils import tree


def _reference_step(p, g, state, step, *, lr, factored, mbps=True, beta1=None, decay_rate=0.8,
                    step_offset=0, clip=1.0, wd=None, wd_lr_exp=None, eps1=1e-30, eps2=1e-3,
                    max_scale=None):
  """One Adafactor update of a matrix in float64 numpy."""
  t = step - step_offset + 1.0
  decay = 1.0 - t ** (-decay_rate)
  mixing = 1.0 - decay
  scale = lr
  if mbps:
    ps = max(np.sqrt(np.mean(p * p)), eps2)
    if max_scale is not None:
      ps = min(ps, max_scale)
    scale = scale * ps
  gsq = g * g + eps1
  new = {}
  if factored:
    v_row = decay * state["v_row"] + mixing * gsq.mean(axis=1)
    v_col = decay * state["v_col"] + mixing * gsq.mean(axis=0)
    y = g * ((v_row / v_row.mean()) ** -0.5)[:, None] * (v_col ** -0.5)[None, :]
    new.update(v_row=v_row, v_col=v_col)
  else:
    v = decay * state["v"] + mixing * gsq
    y = g * v ** -0.5
    new.update(v=v)
  if clip is not None:
    y = y / max(1.0, np.sqrt(np.mean(y * y)) / clip)
  sub = scale * y
  if beta1 is not None:
    m = beta1 * state["m"] + (1 - beta1) * sub
    sub = m
    new.update(m=m)
  if wd is not None:
    rate = wd * lr ** wd_lr_exp if wd_lr_exp else wd
    return (1 - rate) * p - sub, new
  return p - sub, new


CASES = {
    "factored": dict(),
    "unfactored": dict(factored=False),
    "momentum": dict(beta1=0.9),
    "momentum_unfactored": dict(beta1=0.5, factored=False),
    "no_parameter_scale": dict(multiply_by_parameter_scale=False),
    "capped_parameter_scale": dict(max_parameter_scale=0.05),
    "weight_decay": dict(weight_decay_rate=0.01),
    "weight_decay_lr_exponent": dict(weight_decay_rate=0.5, weight_decay_rate_lr_exponent=1.0),
    "no_clipping": dict(clipping_threshold=None),
    "step_offset": dict(step_offset=3),
    "decay_rate": dict(decay_rate=0.5),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_three_steps_match_the_numpy_statement(name):
  kw = dict(CASES[name])
  factored = kw.pop("factored", True)
  opt_def = adafactor.Adafactor(factored=factored, min_dim_size_to_factor=4, **kw)
  rng = np.random.default_rng(0)
  p0 = rng.normal(size=(6, 8)).astype(np.float32)
  opt = opt_def.create({"w": torch.from_numpy(p0.copy())})
  start = kw.get("step_offset", 0)
  if start:
    opt = opt.replace(state=opt.state.replace(step=torch.tensor(start, dtype=torch.int32)))
  p = p0.astype(np.float64)
  state = {"v_row": np.zeros(6), "v_col": np.zeros(8), "v": np.zeros((6, 8)), "m": np.zeros((6, 8))}
  for i in range(3):
    g = rng.normal(size=(6, 8)).astype(np.float32)
    opt = opt.apply_gradient({"w": torch.from_numpy(g)}, learning_rate=0.1)
    p, new = _reference_step(
        p, g.astype(np.float64), state, start + i, lr=0.1, factored=factored,
        mbps=kw.get("multiply_by_parameter_scale", True), beta1=kw.get("beta1"),
        decay_rate=kw.get("decay_rate", 0.8), step_offset=kw.get("step_offset", 0),
        clip=kw.get("clipping_threshold", 1.0), wd=kw.get("weight_decay_rate"),
        wd_lr_exp=kw.get("weight_decay_rate_lr_exponent"), max_scale=kw.get("max_parameter_scale"))
    state.update(new)
    np.testing.assert_allclose(opt.target["w"].numpy(), p, rtol=2e-5, atol=2e-6, err_msg=f"step {i}")
  slots = opt.state.param_states["w"]
  if factored:
    np.testing.assert_allclose(slots["v_row"].numpy(), state["v_row"], rtol=1e-5)
    np.testing.assert_allclose(slots["v_col"].numpy(), state["v_col"], rtol=1e-5)
    assert tuple(slots["v"].shape) == (1,)
  else:
    np.testing.assert_allclose(slots["v"].numpy(), state["v"], rtol=1e-5)
    assert tuple(slots["v_row"].shape) == (1,) and tuple(slots["v_col"].shape) == (1,)
  if kw.get("beta1") is not None:
    np.testing.assert_allclose(slots["m"].numpy(), state["m"], rtol=1e-4, atol=1e-7)
  else:
    assert tuple(slots["m"].shape) == (1,)
  assert int(opt.state.step) == start + 3


def test_skip_nan_updates_leaves_parameter_and_statistics():
  params = {"good": torch.ones(4, 8), "bad": torch.ones(4, 8)}
  grads = {"good": torch.full((4, 8), 0.5), "bad": torch.full((4, 8), float("nan"))}
  skipping = adafactor.Adafactor(min_dim_size_to_factor=4, skip_nan_updates=True).create(
      tree.tree_map(torch.clone, params))
  out = skipping.apply_gradient(grads, learning_rate=0.1)
  assert torch.equal(out.target["bad"], params["bad"])
  assert not torch.isnan(out.state.param_states["bad"]["v_row"]).any()
  assert not torch.equal(out.target["good"], params["good"])
  plain = adafactor.Adafactor(min_dim_size_to_factor=4).create(tree.tree_map(torch.clone, params))
  assert torch.isnan(plain.apply_gradient(grads, learning_rate=0.1).target["bad"]).all()


def test_per_parameter_scale_switch_through_an_hparam_map():
  scale_map = adafactor.HParamMap([("embedding", False), (".*", True)])
  opt_def = adafactor.Adafactor(min_dim_size_to_factor=4, multiply_by_parameter_scale=scale_map)
  params = {"embedding": 3.0 * torch.ones(4, 8), "dense": {"kernel": 3.0 * torch.ones(4, 8)}}
  grads = tree.tree_map(torch.ones_like, params)
  out = opt_def.create(params).apply_gradient(grads, learning_rate=0.1)
  moved_emb = float((3.0 - out.target["embedding"]).mean())
  moved_dense = float((3.0 - out.target["dense"]["kernel"]).mean())
  assert moved_dense == pytest.approx(3.0 * moved_emb, rel=1e-5)   # scaled by RMS(p) = 3
  assert scale_map["decoder/embedding"] is False and scale_map["anything"] is True
  assert scale_map({"embedding": 0, "x": {"y": 0}}) == {"embedding": False, "x": {"y": True}}
  with pytest.raises(KeyError, match="No factor rule"):
    adafactor.HParamMap([("only_this", 1)])["something_else"]


def test_factor_names_and_learning_rate_requirement():
  f = adafactor.factor_name_to_factordim
  assert f("row") is adafactor.FactorDim.ROW and f("Column") is adafactor.FactorDim.COLUMN
  assert f("col") is adafactor.FactorDim.COLUMN and f("batch") is adafactor.FactorDim.BATCH
  assert f("none") is adafactor.FactorDim.NONE and f("unfactorized") is adafactor.FactorDim.NONE
  assert f(adafactor.FactorDim.ROW) is adafactor.FactorDim.ROW
  opt = adafactor.Adafactor(min_dim_size_to_factor=4).create({"w": torch.ones(4, 8)})
  with pytest.raises((ValueError, AssertionError, TypeError)):
    opt.apply_gradient({"w": torch.ones(4, 8)})          # no learning rate anywhere
  fixed = adafactor.Adafactor(learning_rate=0.2, min_dim_size_to_factor=4).create(
      {"w": torch.ones(4, 8)})
  assert not torch.equal(fixed.apply_gradient({"w": torch.ones(4, 8)}).target["w"],
                         torch.ones(4, 8))
