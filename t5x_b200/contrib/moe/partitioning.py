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

  def get_data_layout(self, batch_size: Optional[int] = None,
                      host_index: Optional[int] = None) -> base_partitioning.DataLayout:
    """Data layout with both 'expert' and 'data' acting as data axes: shards are numbered
    expert-major (shard id = data chunk + expert chunk * data chunks), and a process reads data
    when it is the first replica of its (expert, data) block
    (t5x/contrib/moe/partitioning.py:205-262)."""
    if host_index is not None:
      raise NotImplementedError("Explicit host_index is not yet implemented.")
    chunker = self._local_chunker
    mesh_shape = chunker.global_mesh.shape
    data_mesh_size = mesh_shape["data"] * mesh_shape["expert"]
    batch_size = batch_size or data_mesh_size
    if batch_size % data_mesh_size:
      raise ValueError(
          f"Batch size ({batch_size}) must be divisible by entire data mesh size "
          f"({data_mesh_size}). Note that for MoE, the data mesh spans both the \"expert\" and "
          "\"data\" virtual mesh axes.")
    num_shards = chunker.num_chunks["data"] * chunker.num_chunks["expert"]
    if batch_size % num_shards:
      raise ValueError(f"Batch size ({batch_size}) must be divisible by total number of shards "
                       f"({num_shards}) across \"data\" and \"expert\" mesh axes.")
    block = chunker.get_local_chunk_info(
        (mesh_shape["expert"], batch_size // mesh_shape["expert"]), ("expert", "data"))
    return base_partitioning.DataLayout(
        batch_size=int(batch_size),
        shard_id=int(chunker.chunk_ids["data"] +
                     chunker.chunk_ids["expert"] * chunker.num_chunks["data"]),
        num_shards=int(num_shards), is_first_host_in_replica_set=(block.replica_id == 0))

  def get_logical_axes(self, train_state):
    """Logical axes of the train state with 'expert' prepended to the optimizer slots that
    the state filter names. Factored Adafactor does not carry the parameter's axis names over
    to its `v_row` / `v_col` vectors, so for expert kernels (stacked [experts, ...]) those
    vectors would otherwise look replicated although they have one slice per expert
    (t5x/contrib/moe/partitioning.py:264-317)."""
    logical_axes = train_state.as_logical_axes()
    if not hasattr(train_state, "_optimizer"):
      return logical_axes  # inference state: no optimizer slots
    state_filter_fn = self._state_filter_fn or _infer_state_filter_fn(train_state)
    if state_filter_fn is None:
      return logical_axes
    from t5x_b200 import optimizers
    from t5x_b200.utils import tree as tree_utils
    axes_opt = logical_axes._optimizer  # pylint: disable=protected-access
    slots = tree_utils.flatten_dict(axes_opt.state.param_states,
                                    is_leaf=lambda x: not isinstance(x, dict))
    for path, axes in slots.items():
      name = path if isinstance(path, str) else "/".join(str(k) for k in path)
      if state_filter_fn(name):
        slots[path] = ("expert",) + tuple(axes) if axes else ("expert",)
    new_state = optimizers.OptimizerState(step=axes_opt.state.step,
                                          param_states=tree_utils.unflatten_dict(slots))
    return logical_axes.replace(_optimizer=axes_opt.replace(state=new_state))

  def partition(self, fn, in_axis_resources, out_axis_resources, static_argnums=(),
                donate_argnums=()):
    return super().partition(fn, override_partition_specs(in_axis_resources),
                             override_partition_specs(out_axis_resources), static_argnums,
                             donate_argnums)



def _infer_state_filter_fn(train_state):
  """Which optimizer slots are sharded along 'expert' without saying so in their axis names:
  for factored Adafactor the `v_row` / `v_col` vectors of expert kernels; for unfactored
  Adafactor and for wrapped optax optimizers the slots inherit the parameter's names and
  nothing needs overriding (t5x/contrib/moe/partitioning.py:506-581)."""
  from t5x_b200 import adafactor, optimizers
  from t5x_b200.contrib.moe import training_utils
  opt_def = train_state._optimizer.optimizer_def  # pylint: disable=protected-access
  if isinstance(opt_def, optimizers.MultiOptimizer):
    subs = list(opt_def.sub_optimizers)
    if not subs:
      return None
    if any(type(o) is not type(subs[0]) for o in subs):
      raise ValueError("optimizers.MultiOptimizer is only supported in cases where all "
                       "suboptimizers are of the same type.")
    if isinstance(subs[0], adafactor.Adafactor) and \
        any(o.hyper_params.factored != subs[0].hyper_params.factored for o in subs):
      raise ValueError("If using adafactor.Adafactor as the suboptimizer in "
                       "optimizers.MultiOptimizer, all suboptimizers must be either factored or "
                       "unfactored (cannot use mixed factoring).")
    opt_def = subs[0]
  if isinstance(opt_def, optimizers.OptaxWrapper):
    return None
  if not isinstance(opt_def, adafactor.Adafactor):
    raise ValueError("Unrecognized optimizer type. Expecting optimizers.OptaxWrapper or "
                     f"adafactor.Adafactor. Received: {opt_def}")
  if opt_def.hyper_params.factored:
    return training_utils.match_fn(r".*expert.*/kernel/v_.*")
  return None
