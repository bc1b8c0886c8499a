"""Mesh construction, local chunks, logical-axis resolution and the partitioner's view of a
train state, with ranks simulated by `world_size` / `local_rank`
(cases after t5x/partitioning_test.py)."""
import numpy as np
import pytest
import torch

from t5x_b200 import adafactor, partitioning, train_state as ts

P = partitioning.PartitionSpec


def test_gpu_mesh_fills_model_axis_first():
  mesh = partitioning.get_gpu_mesh(num_partitions=4, world_size=8, local_rank=6)
  assert dict(mesh.shape) == {"data": 2, "model": 4}
  assert dict(mesh.coords()) == {"data": 1, "model": 2}     # rank 6 = data 1, model 2
  assert np.asarray(mesh.devices).tolist() == [[0, 1, 2, 3], [4, 5, 6, 7]]
  with pytest.raises(ValueError):
    partitioning.get_gpu_mesh(num_partitions=3, world_size=8, local_rank=0)
  cpu = partitioning.get_cpu_mesh(world_size=2, local_rank=1)
  assert dict(cpu.shape) == {"data": 2, "model": 1}


def test_default_mesh_with_submesh_and_ici_dcn():
  mesh = partitioning.default_mesh(1, model_parallel_submesh=(1, 2, 1, 2), world_size=8,
                                   local_rank=0)
  assert dict(mesh.shape) == {"data": 2, "model": 4}
  mesh = partitioning.default_mesh(1, ici_mesh_shape=(1, 4, 2), dcn_mesh_shape=(1, 1, 1),
                                   world_size=8, local_rank=3)
  assert dict(mesh.shape) == {"replica": 1, "data": 4, "model": 2}


@pytest.mark.parametrize("rank", range(8))
def test_local_chunker(rank):
  mesh = partitioning.get_gpu_mesh(num_partitions=2, world_size=8, local_rank=rank)
  ch = partitioning.LocalChunker(mesh)
  assert ch.num_chunks["data"] == 4 and ch.num_chunks["model"] == 2
  d, m = rank // 2, rank % 2
  assert ch.chunk_ids["data"] == d and ch.chunk_ids["model"] == m
  info = ch.get_local_chunk_info((128, 16), ["data", "model"])
  assert info.replica_id == 0
  assert info.slice == (slice(32 * d, 32 * (d + 1)), slice(8 * m, 8 * (m + 1)))
  info = ch.get_local_chunk_info((128, 16), [None, "model"])
  assert info.replica_id == d and info.slice == (slice(None), slice(8 * m, 8 * (m + 1)))
  info = ch.get_local_chunk_info((128, 16), [None, None])
  assert info.replica_id == rank


def test_logical_to_mesh_axes_priority_and_conflicts():
  rules = partitioning.standard_logical_axis_rules(2, 2)
  # 'embed' prefers 'model', but 'mlp' (earlier rule) already took it: falls to 'data'
  assert partitioning.logical_to_mesh_axes(("embed", "mlp"), rules) == P("data", "model")
  assert partitioning.logical_to_mesh_axes(("batch", "length", "embed"), rules) == \
      P("data", None, "model")
  assert partitioning.logical_to_mesh_axes(None, rules) is None
  with pytest.raises(ValueError, match="Unmatched"):
    partitioning.logical_to_mesh_axes(("no_such_axis",), rules)


@pytest.mark.parametrize("a,p", [(1, 1), (2, 1), (1, 2), (2, 2)])
def test_standard_rules_presets(a, p):
  rules = partitioning.standard_logical_axis_rules(a, p)
  d = {}
  for k, v in rules:
    d.setdefault(k, []).append(v)
  assert d["batch"] == ["data"] and d["vocab"] == ["model"] and d["mlp"] == ["model"]
  expect = {(1, 1): [None], (2, 1): ["model"], (1, 2): ["data"], (2, 2): ["model", "data"]}
  assert d["embed"] == expect[(a, p)]
  extra = (("my-new-axis", "data"), ("another-axis", None))
  longer = partitioning.standard_logical_axis_rules(a, p, additional_rules=extra)
  assert list(longer[-2:]) == list(extra) and list(longer[:-2]) == list(rules)
  with pytest.raises(ValueError):
    partitioning.standard_logical_axis_rules(3, 1)


def _axes_spec(factored, momentum):
  part = partitioning.PjitPartitioner(
      num_partitions=1, world_size=1, local_rank=0,
      logical_axis_rules=(("batch", "data"), ("embed", None), ("vocab", "model"),
                          ("mlp", "model")))
  opt = adafactor.Adafactor(
      learning_rate=0.1, factored=factored, min_dim_size_to_factor=8,
      beta1=0.1 if momentum else None,
      logical_factor_rules={"batch": adafactor.FactorDim.NONE, "embed": adafactor.FactorDim.ROW,
                            "vocab": adafactor.FactorDim.COLUMN,
                            "mlp": adafactor.FactorDim.COLUMN})
  state = ts.FlaxOptimTrainState.create(opt, {
      "params": {"logits_dense": torch.ones(16, 16), "mlp": {"wo": {"kernel": torch.ones(32, 16)}}},
      "params_axes": {"logits_dense": ("vocab", "embed"),
                      "mlp": {"wo": {"kernel": ("embed", "mlp")}}}})
  return part.get_mesh_axes(state).state_dict()


@pytest.mark.parametrize("factored", [True, False])
@pytest.mark.parametrize("momentum", [True, False])
def test_get_mesh_axes_for_optimizer_state(factored, momentum):
  """Parameters get their resolved specs; of the optimizer slots only unfactored `v` and the
  momentum inherit them, factored vectors stay replicated."""
  sd = _axes_spec(factored, momentum)
  p0, p1 = P("model", None), P(None, "model")
  assert sd["target"]["logits_dense"] == p0
  assert sd["target"]["mlp"]["wo"]["kernel"] == p1
  s0 = sd["state"]["param_states"]["logits_dense"]
  s1 = sd["state"]["param_states"]["mlp"]["wo"]["kernel"]
  assert s0["v_row"] is None and s0["v_col"] is None and s1["v_row"] is None
  assert s0["m"] == (p0 if momentum else None) and s1["m"] == (p1 if momentum else None)
  assert s0["v"] == (None if factored else p0) and s1["v"] == (None if factored else p1)


def test_data_layout():
  part = partitioning.PjitPartitioner(num_partitions=2, world_size=8, local_rank=5)
  lay = part.get_data_layout(32)
  # rank 5 = data row 2 of 4, model column 1: reads shard 2, and is not the first replica
  assert (lay.batch_size, lay.shard_id, lay.num_shards) == (32, 2, 4)
  assert lay.is_first_host_in_replica_set is False
  assert partitioning.PjitPartitioner(num_partitions=2, world_size=8, local_rank=4) \
      .get_data_layout(32).is_first_host_in_replica_set is True
  with pytest.raises(ValueError):
    part.get_data_layout(30)
  assert part.data_partition_spec == P("data")


def test_parameter_partitioning_over_data_is_visible_to_the_trainer():
  """`parameter_partitioning_dims=2` puts 'embed' on the data axis: the partitioner reports it,
  and the trainer turns that into optimizer sharding over the data axis."""
  from t5x_b200 import partitioning
  one = partitioning.PjitPartitioner(
      num_partitions=1, logical_axis_rules=partitioning.standard_logical_axis_rules(
          parameter_partitioning_dims=1))
  two = partitioning.PjitPartitioner(
      num_partitions=1, logical_axis_rules=partitioning.standard_logical_axis_rules(
          parameter_partitioning_dims=2))
  assert not one.partitions_parameters_over_data
  assert two.partitions_parameters_over_data


def _mesh_worker(rank, world, port, out_dir):
  import json
  import os
  import torch.distributed as dist
  from t5x_b200.parallel import state as pstate
  os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                    WORLD_SIZE=str(world))
  dist.init_process_group("gloo", rank=rank, world_size=world)
  st = pstate.setup_mesh(model_size=2)
  import torch
  one = torch.tensor([float(rank)])
  model_sum, data_sum = one.clone(), one.clone()
  dist.all_reduce(model_sum, group=st.model_group)
  dist.all_reduce(data_sum, group=st.data_group)
  with open(os.path.join(out_dir, f"{rank}.json"), "w") as f:
    json.dump({"data": [st.data_size, st.data_rank], "model": [st.model_size, st.model_rank],
               "model_ranks": dist.get_process_group_ranks(st.model_group),
               "data_ranks": dist.get_process_group_ranks(st.data_group),
               "model_sum": float(model_sum), "data_sum": float(data_sum)}, f)
  dist.destroy_process_group()


def test_four_ranks_as_data2_x_model2(tmp_path):
  """Model groups are consecutive ranks, data groups stride over them; collectives on one
  axis touch only that axis."""
  import json
  import socket
  import torch.multiprocessing as mp
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
  mp.spawn(_mesh_worker, args=(4, port, str(tmp_path)), nprocs=4, join=True)
  got = [json.load(open(tmp_path / f"{r}.json")) for r in range(4)]
  assert [g["model_ranks"] for g in got] == [[0, 1], [0, 1], [2, 3], [2, 3]]
  assert [g["data_ranks"] for g in got] == [[0, 2], [1, 3], [0, 2], [1, 3]]
  assert [g["data"] for g in got] == [[2, 0], [2, 0], [2, 1], [2, 1]]
  assert [g["model"] for g in got] == [[2, 0], [2, 1], [2, 0], [2, 1]]
  assert [g["model_sum"] for g in got] == [1.0, 1.0, 5.0, 5.0]
  assert [g["data_sum"] for g in got] == [2.0, 4.0, 2.0, 4.0]
