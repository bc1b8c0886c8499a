"""Adafactor: state shapes under heuristic and manual factor rules, golden update values,
factored-rule equivalences, native vs PyTorch path (cases and expected numbers after
t5x/adafactor_test.py)."""
import numpy as np
import pytest
import torch

from t5x_b200 import adafactor
from t5x_b200.optimizers import OptimizerState
from t5x_b200.utils import tree as tree_utils

ROW, COL, BATCH, NONE = (adafactor.FactorDim.ROW, adafactor.FactorDim.COLUMN,
                         adafactor.FactorDim.BATCH, adafactor.FactorDim.NONE)


def _shapes(opt_def, params):
  state = opt_def.init_state(params)
  return {k: tuple(v.shape) for k, v in tree_utils.flatten_dict(state.param_states).items()}


def test_2d_heuristic_shapes():
  x = {"a": torch.ones(24, 16)}
  assert _shapes(adafactor.Adafactor(min_dim_size_to_factor=8), x) == \
      {"a/m": (1,), "a/v": (1,), "a/v_col": (24,), "a/v_row": (16,)}
  assert _shapes(adafactor.Adafactor(min_dim_size_to_factor=32), x) == \
      {"a/m": (1,), "a/v": (24, 16), "a/v_col": (1,), "a/v_row": (1,)}
  assert _shapes(adafactor.Adafactor(min_dim_size_to_factor=32, beta1=0.1), x) == \
      {"a/m": (24, 16), "a/v": (24, 16), "a/v_col": (1,), "a/v_row": (1,)}


@pytest.mark.parametrize("rule,v_col,v_row", [
    ((COL, BATCH, ROW), (24, 4), (4, 16)),
    ((ROW, BATCH, COL), (4, 16), (24, 4)),
    ((COL, ROW, ROW), (24,), (4, 16)),
    ((COL, COL, ROW), (24, 4), (16,)),
])
def test_3d_manual_rules(rule, v_col, v_row):
  x = {"a": torch.ones(24, 4, 16)}
  opt = adafactor.Adafactor(min_dim_size_to_factor=8,
                            factor_map=adafactor.HParamMap((("a", rule),)))
  assert _shapes(opt, x) == {"a/m": (1,), "a/v": (1,), "a/v_col": v_col, "a/v_row": v_row}


@pytest.mark.parametrize("rule", [(ROW, COL), (COL, ROW)])
def test_2d_ignores_manual_rule(rule):
  # a 2-D parameter always falls back to the heuristic: v_row indexes the smaller dim
  x = {"a": torch.ones(24, 16)}
  opt = adafactor.Adafactor(min_dim_size_to_factor=8,
                            factor_map=adafactor.HParamMap((("a", rule),)))
  assert _shapes(opt, x) == {"a/m": (1,), "a/v": (1,), "a/v_col": (24,), "a/v_row": (16,)}


def test_factoring_threshold():
  opt = adafactor.Adafactor(learning_rate=0.1, min_dim_size_to_factor=32)
  assert _shapes(opt, {"x": torch.zeros(64, 64)})["x/v_row"] == (64,)
  assert _shapes(opt, {"x": torch.zeros(31, 64)})["x/v"] == (31, 64)


def test_apply_gradient_golden_values():
  opt = adafactor.Adafactor(learning_rate=0.1, decay_rate=0.8, min_dim_size_to_factor=0)
  params = {"x": torch.ones(3, 2)}
  state = OptimizerState(torch.tensor(1), {"x": {
      "v_row": torch.tensor([0.9, 0.9]), "v_col": torch.tensor([0.1, 0.1, 0.1]),
      "v": torch.zeros(1), "m": torch.zeros(1)}})
  new_params, new_state = opt.apply_gradient(opt.hyper_params, params, state,
                                             {"x": torch.ones(3, 2)})
  np.testing.assert_allclose(new_params["x"].numpy(), 0.9 * np.ones((3, 2)), rtol=1e-6)
  np.testing.assert_allclose(new_state.param_states["x"]["v_row"].numpy(), [0.9574349] * 2,
                             rtol=1e-6)
  np.testing.assert_allclose(new_state.param_states["x"]["v_col"].numpy(), [0.6169143] * 3,
                             rtol=1e-6)
  assert int(new_state.step) == 2
  # unfactored with momentum
  opt = adafactor.Adafactor(learning_rate=0.1, beta1=0.0, decay_rate=0.8,
                            min_dim_size_to_factor=32)
  params = {"x": torch.ones(3, 2)}
  state = OptimizerState(torch.tensor(1), {"x": {
      "v_row": torch.zeros(1), "v_col": torch.zeros(1), "v": 0.5 * torch.ones(3, 2),
      "m": torch.zeros(3, 2)}})
  new_params, new_state = opt.apply_gradient(opt.hyper_params, params, state,
                                             {"x": torch.ones(3, 2)})
  np.testing.assert_allclose(new_params["x"].numpy(), 0.9 * np.ones((3, 2)), rtol=1e-6)
  np.testing.assert_allclose(new_state.param_states["x"]["v"].numpy(),
                             0.787174 * np.ones((3, 2)), rtol=1e-6)
  np.testing.assert_allclose(new_state.param_states["x"]["m"].numpy(), 0.1 * np.ones((3, 2)),
                             rtol=1e-6)


def test_global_norm_clipping_scales_gradients():
  opt = adafactor.Adafactor(learning_rate=0.1, decay_rate=0.8, min_dim_size_to_factor=0,
                            global_norm_clip_threshold=1.0, multiply_by_parameter_scale=False,
                            clipping_threshold=None)
  params = {"x": torch.ones(3, 2)}
  g = {"x": 10.0 * torch.ones(3, 2)}
  st0 = opt.init_state(params)
  p_clip, _ = opt.apply_gradient(opt.hyper_params, {"x": torch.ones(3, 2)}, st0, g)
  opt2 = adafactor.Adafactor(learning_rate=0.1, decay_rate=0.8, min_dim_size_to_factor=0,
                             multiply_by_parameter_scale=False, clipping_threshold=None)
  unit = {"x": 10.0 * torch.ones(3, 2) / (10.0 * np.sqrt(6.0))}
  p_ref, _ = opt2.apply_gradient(opt2.hyper_params, {"x": torch.ones(3, 2)},
                                 opt2.init_state(params), unit)
  torch.testing.assert_close(p_clip["x"], p_ref["x"])


@pytest.mark.parametrize("shape,rule", [((64, 64), (ROW, COL)), ((64, 32), (COL, ROW)),
                                        ((8, 64, 32), (BATCH, ROW, COL))])
def test_rule_based_update_matches_per_matrix_heuristic(shape, rule):
  """Leading BATCH dims are independent matrices; a (ROW, COL) rule is the classic update."""
  torch.manual_seed(0)
  p0 = torch.randn(shape)
  g = torch.randn(shape)
  opt_rule = adafactor.Adafactor(learning_rate=0.01, min_dim_size_to_factor=8,
                                 factor_map=adafactor.HParamMap((("x", rule),)))
  p_rule, _ = opt_rule.apply_gradient(opt_rule.hyper_params, {"x": p0.clone()},
                                      opt_rule.init_state({"x": p0}), {"x": g.clone()})
  opt_h = adafactor.Adafactor(learning_rate=0.01, min_dim_size_to_factor=8)
  if len(shape) == 2:
    p_h, _ = opt_h.apply_gradient(opt_h.hyper_params, {"x": p0.clone()},
                                  opt_h.init_state({"x": p0}), {"x": g.clone()})
    torch.testing.assert_close(p_rule["x"], p_h["x"], rtol=1e-5, atol=1e-6)
  else:
    for b in range(shape[0]):
      p_h, _ = opt_h.apply_gradient(opt_h.hyper_params, {"x": p0[b].clone()},
                                    opt_h.init_state({"x": p0[b]}), {"x": g[b].clone()})
      torch.testing.assert_close(p_rule["x"][b], p_h["x"], rtol=1e-5, atol=1e-6)


def test_standard_logical_rules_cover_model_axes():
  rules = adafactor.standard_logical_factor_rules()
  for axis in ("vocab", "embed", "mlp", "heads", "kv", "joined_kv", "relpos_buckets", "layers",
               "stack"):
    assert axis in rules
  assert rules["layers"] == BATCH and rules["stack"] == BATCH
  opt = adafactor.Adafactor(logical_factor_rules=rules)
  opt.set_param_axes({"k": ("embed", "mlp"), "s": ("embed",)})
  # 2-D parameters use the size heuristic whatever the rules say (min_dim_size_to_factor=128)
  shapes = _shapes(opt, {"k": torch.zeros(128, 256), "s": torch.zeros(16)})
  assert shapes["k/v"] == (1,) and shapes["s/v"] == (16,)
  assert sorted([shapes["k/v_row"], shapes["k/v_col"]]) == [(128,), (256,)]
  assert _shapes(opt, {"k": torch.zeros(16, 32), "s": torch.zeros(16)})["k/v"] == (16, 32)
  with pytest.raises(ValueError):
    adafactor.Adafactor(factored=False, factor_map=adafactor.HParamMap((("a", (ROW, COL)),)))
