"""The MoE partitioner on simulated ranks: mesh factoring, model-partition arithmetic, logical
axis rules, data specs and their overrides, optimizer-slot axes of expert kernels and the
inferred state filter (the cases of t5x/contrib/moe/partitioning_test.py)."""
import pytest
import torch

from t5x_b200 import adafactor, optimizers, partitioning
from t5x_b200 import train_state as ts_lib
from t5x_b200.contrib.moe import adafactor_utils
from t5x_b200.contrib.moe import partitioning as moe_partitioning
from t5x_b200.partitioning import PartitionSpec
from t5x_b200.utils import tree


@pytest.mark.parametrize("world,experts_wanted,model,expect", [
    (8, 8, 1, {"data": 1, "expert": 8, "model": 1}),
    (8, 4, 1, {"data": 2, "expert": 4, "model": 1}),
    (8, 8, 2, {"data": 1, "expert": 4, "model": 2}),
    (8, 3, 1, {"data": 4, "expert": 2, "model": 1}),   # 3 does not divide 8: next smaller that does
    (4, 16, 1, {"data": 1, "expert": 4, "model": 1}),
])
def test_mesh_factors_the_data_axis(world, experts_wanted, model, expect):
  mesh = moe_partitioning.default_moe_mesh(experts_wanted, num_partitions=model,
                                           world_size=world, local_rank=0)
  assert dict(mesh.shape) == expect
  assert list(mesh.axis_names) == ["data", "expert", "model"]


def test_compute_num_model_partitions():
  f = moe_partitioning.compute_num_model_partitions
  assert f(4, None) == 4
  assert f(None, (2, 2, 1, 1)) == 4
  assert f(4, (2, 2, 1, 1)) == 4
  with pytest.raises(ValueError, match="inconsistent"):
    f(3, (2, 2, 1, 1))
  with pytest.raises(ValueError, match="At least one"):
    f(None, None)


def test_logical_axis_rules_add_the_moe_axes_and_reshard_the_batch():
  rules = moe_partitioning.standard_logical_axis_rules()
  as_dict = {}
  for k, v in rules:
    as_dict.setdefault(k, v)
  assert as_dict["batch"] == ("expert", "data")
  assert as_dict["expert"] == "expert" and as_dict["expert_mlp"] == "model"
  assert as_dict["expert_replicas"] == "data" and as_dict["unmodeled"] is None
  assert as_dict["mlp"] == "model" and as_dict["vocab"] == "model"
  extra = moe_partitioning.standard_logical_axis_rules(additional_rules=[("my_axis", "model")])
  assert ("my_axis", "model") in extra
  base = dict(partitioning.standard_logical_axis_rules())
  assert base["batch"] == "data"   # the base rules are left alone


def test_data_partition_spec_and_overrides():
  part = moe_partitioning.MoePjitPartitioner(num_expert_partitions=4, num_partitions=1,
                                             world_size=8, local_rank=3)
  assert part.data_partition_spec == PartitionSpec(("expert", "data"),)
  assert part.num_expert_partitions == 4
  fix = moe_partitioning.override_partition_specs
  assert fix(PartitionSpec("data",)) == PartitionSpec(("expert", "data"),)
  assert fix(PartitionSpec("model",)) == PartitionSpec("model",)
  mixed = fix((PartitionSpec("data",), None, PartitionSpec("data", "model")))
  assert mixed == (PartitionSpec(("expert", "data"),), None, PartitionSpec("data", "model"))
  assert fix(None) is None and fix("data") == "data"


def _moe_state(opt_def):
  params = {"encoder": {"layers_0": {"mlp": {"expert": {"wi": {"kernel": torch.zeros(4, 128, 256)}},
                                             "router": {"w": {"kernel": torch.zeros(128, 4)}}},
                                     "attention": {"query": {"kernel": torch.zeros(128, 128)}}}}}
  axes = {"encoder": {"layers_0": {"mlp": {"expert": {"wi": {"kernel": ("expert", "embed", "expert_mlp")}},
                                           "router": {"w": {"kernel": ("embed", "unmodeled")}}},
                                   "attention": {"query": {"kernel": ("embed", "joined_kv")}}}}}
  return ts_lib.FlaxOptimTrainState.create(opt_def, {"params": params, "params_axes": axes})


def test_factored_slots_of_expert_kernels_get_the_expert_axis():
  opt = adafactor.Adafactor(decay_rate=0.8, step_offset=0, factored=True,
                            logical_factor_rules=adafactor_utils.logical_factor_rules())
  state = _moe_state(opt)
  part = moe_partitioning.MoePjitPartitioner(num_expert_partitions=4, num_partitions=1,
                                             world_size=4, local_rank=0)
  axes = tree.flatten_dict(part.get_logical_axes(state).param_states,
                           is_leaf=lambda x: not isinstance(x, dict))
  expert = "encoder/layers_0/mlp/expert/wi/kernel"
  assert tuple(axes[f"{expert}/v_row"])[0] == "expert"
  assert tuple(axes[f"{expert}/v_col"])[0] == "expert"
  # dense kernels and the router are untouched
  assert axes["encoder/layers_0/attention/query/kernel/v_row"] is None
  assert axes["encoder/layers_0/mlp/router/w/kernel/v_row"] is None
  # parameters keep their own names
  p_axes = tree.flatten_dict(part.get_logical_axes(state).params,
                             is_leaf=lambda x: not isinstance(x, dict))
  assert tuple(p_axes[expert]) == ("expert", "embed", "expert_mlp")
  # an explicit filter wins over the inferred one
  only_rows = moe_partitioning.MoePjitPartitioner(
      num_expert_partitions=4, num_partitions=1, world_size=4, local_rank=0,
      state_filter_fn=lambda name: name.endswith("expert/wi/kernel/v_row"))
  axes = tree.flatten_dict(only_rows.get_logical_axes(state).param_states,
                           is_leaf=lambda x: not isinstance(x, dict))
  assert tuple(axes[f"{expert}/v_row"])[0] == "expert" and axes[f"{expert}/v_col"] is None


def test_inferred_state_filter_by_optimizer_kind():
  infer = moe_partitioning._infer_state_filter_fn
  rules = adafactor_utils.logical_factor_rules()
  factored = infer(_moe_state(adafactor.Adafactor(factored=True, logical_factor_rules=rules)))
  assert factored("encoder/layers_0/mlp/expert/wi/kernel/v_row")
  assert factored("decoder/layers_3/mlp/expert/wo/kernel/v_col")
  assert not factored("encoder/layers_0/mlp/expert/wi/kernel/m")
  assert not factored("encoder/layers_0/attention/query/kernel/v_row")
  assert infer(_moe_state(adafactor.Adafactor(factored=False, logical_factor_rules=rules))) is None
  assert infer(_moe_state(optimizers.adamw(None))) is None
  # MultiOptimizer: one kind of sub-optimizer, one factoring
  everything = optimizers.ModelParamTraversal(lambda path, _: True)
  nothing = optimizers.ModelParamTraversal(lambda path, _: False)
  multi = optimizers.MultiOptimizer(((everything, adafactor.Adafactor(factored=True, logical_factor_rules=rules)),
                                     (nothing, adafactor.Adafactor(factored=True, logical_factor_rules=rules))))
  assert infer(_moe_state(multi))("x/expert/wi/kernel/v_row")
  mixed = optimizers.MultiOptimizer(((everything, adafactor.Adafactor(factored=True, logical_factor_rules=rules)),
                                     (nothing, adafactor.Adafactor(factored=False, logical_factor_rules=rules))))
  with pytest.raises(ValueError, match="mixed factoring"):
    infer(_moe_state(mixed))


def test_inference_state_axes_pass_through():
  part = moe_partitioning.MoePjitPartitioner(num_expert_partitions=2, num_partitions=1,
                                             world_size=2, local_rank=0)
  state = ts_lib.InferenceState.create({
      "params": {"expert": {"wi": {"kernel": torch.zeros(2, 8, 16)}}},
      "params_axes": {"expert": {"wi": {"kernel": ("expert", "embed", "expert_mlp")}}}})
  axes = part.get_logical_axes(state)
  assert axes.params["expert"]["wi"]["kernel"] == ("expert", "embed", "expert_mlp")
