"""Partitioning for mixture-of-experts models: a ('data', 'expert', 'model') mesh
(t5x/contrib/moe/partitioning.py).

Ranks are laid out model-fastest, then expert, then data, the same order
`parallel.state.setup_mesh(model_size, expert_size)` uses for its process groups: the batch is
split over ('expert', 'data'), expert weights over 'expert', and dense weights are replicated
over both."""
from __future__ import annotations

import logging
from typing import Any, Optional, Sequence

import numpy as np

from t5x_b200 import partitioning as base_partitioning
from t5x_b200.parallel import state as pstate

Mesh = base_partitioning.Mesh
PartitionSpec = base_partitioning.PartitionSpec
HardwareMesh = base_partitioning.HardwareMesh
LogicalAxisRules = base_partitioning.LogicalAxisRules


def get_cpu_mesh(world_size: Optional[int] = None, local_rank: Optional[int] = None) -> Mesh:
  """Trivial (data, expert, model) mesh for CPU testing."""
  world = pstate.get().world_size if world_size is None else world_size
  return Mesh(np.arange(world).reshape(world, 1, 1), ["data", "expert", "model"], local_rank)


def get_gpu_mesh(world_size: Optional[int] = None, local_rank: Optional[int] = None) -> Mesh:
  """Simple (data, expert, model) mesh with all devices on the data axis."""
  return get_cpu_mesh(world_size, local_rank)


def default_moe_mesh(num_expert_partitions: int, num_partitions: Optional[int] = None,
                     model_parallel_submesh: Optional[HardwareMesh] = None,
                     backend: Optional[str] = None, world_size: Optional[int] = None,
                     local_rank: Optional[int] = None) -> Mesh:
  """(data, expert, model) mesh: the vanilla (data, model) mesh with its data axis factored
  into data x expert. The expert axis is the largest size <= `num_expert_partitions` that
  divides the data axis (t5x/contrib/moe/partitioning.py:59-118)."""
  base = base_partitioning.default_mesh(num_partitions or 1, model_parallel_submesh, backend,
                                        world_size=world_size, local_rank=local_rank)
  data_axis_size, model_axis_size = (base.shape["data"], base.shape["model"])
  expert_axis_size = num_expert_partitions
  while data_axis_size % expert_axis_size != 0:
    expert_axis_size -= 1
  devices = np.asarray(base.devices).reshape(-1, expert_axis_size, model_axis_size)
  mesh = Mesh(devices, ["data", "expert", "model"], base.local_rank)
  logging.info("MoE mesh shape: %s", dict(mesh.shape))
  return mesh


def compute_num_model_partitions(num_model_partitions: Optional[int],
                                 model_parallel_submesh: Optional[HardwareMesh]) -> int:
  if num_model_partitions is None and model_parallel_submesh is None:
    raise ValueError("At least one of num_model_partitions and model_parallel_submesh must be "
                     "specified.")
  if num_model_partitions is not None:
    if model_parallel_submesh is not None and \
        num_model_partitions != int(np.prod(model_parallel_submesh)):
      raise ValueError("num_model_partitions and model_parallel_submesh are inconsistent. "
                       f"Received: {num_model_partitions} and {model_parallel_submesh}")
    return num_model_partitions
  return int(np.prod(model_parallel_submesh))


def standard_logical_axis_rules(activation_partitioning_dims: int = 2,
                                parameter_partitioning_dims: int = 1,
                                additional_rules: Optional[LogicalAxisRules] = None):
  """The base rules plus the MoE axes; `batch` is sharded over ('expert', 'data')."""
  if parameter_partitioning_dims == 2:
    logging.warning("2D parameter sharding (`parameter_partitioning_dims=2`) is supported but "
                    "untested for MoE.")
  rules = list(base_partitioning.standard_logical_axis_rules(activation_partitioning_dims,
                                                             parameter_partitioning_dims))
  rules += [("expert", "expert"), ("expert_mlp", "model"), ("expert_replicas", "data"),
            ("unmodeled", None)]
  if additional_rules:
    rules.extend(additional_rules)
  return [(k, ("expert", "data") if k == "batch" else v) for k, v in rules]


def override_partition_specs(resources: Any):
  """PartitionSpec('data') -> PartitionSpec(('expert', 'data')) wherever a raw data spec is
  hard-coded; everything else is left alone."""
  def fix(r):
    return PartitionSpec(("expert", "data"),) if r == PartitionSpec("data",) else r
  if isinstance(resources, PartitionSpec):
    return fix(resources)
  if isinstance(resources, Sequence) and not isinstance(resources, str):
    return tuple(fix(r) for r in resources)
  return resources


class MoePjitPartitioner(base_partitioning.PjitPartitioner):
  """Partitioner over the (data, expert, model) mesh."""

  def __init__(self, num_expert_partitions: int, num_partitions: Optional[int] = None,
               model_parallel_submesh: Optional[HardwareMesh] = None,
               params_on_devices: bool = True,
               logical_axis_rules: Optional[LogicalAxisRules] = None,
               state_filter_fn=None, world_size: Optional[int] = None,
               local_rank: Optional[int] = None):
    if logical_axis_rules is None:
      logical_axis_rules = standard_logical_axis_rules()
    super().__init__(num_partitions=num_partitions or 1,
                     model_parallel_submesh=model_parallel_submesh,
                     params_on_devices=params_on_devices, logical_axis_rules=logical_axis_rules,
                     world_size=world_size, local_rank=local_rank)
    self._num_expert_partitions = num_expert_partitions
    self._state_filter_fn = state_filter_fn
    self._data_axis = ("expert", "data")

  @property
  def num_expert_partitions(self) -> int:
    return self.mesh.shape["expert"]

  @property
  def data_partition_spec(self) -> PartitionSpec:
    return PartitionSpec(("expert", "data"),)

  @property
  def mesh(self) -> Mesh:
    if self._mesh_cache is None:
      self._mesh_cache = default_moe_mesh(self._num_expert_partitions, self._num_partitions,
                                          self._model_parallel_submesh, self._backend,
                                          self._world_size, self._local_rank)
    return self._mesh_cache

  def partition(self, fn, in_axis_resources, out_axis_resources, static_argnums=(),
                donate_argnums=()):
    return super().partition(fn, override_partition_specs(in_axis_resources),
                             override_partition_specs(out_axis_resources), static_argnums,
                             donate_argnums)
