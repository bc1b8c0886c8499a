"""Partitioning: device mesh, logical-axis rules, local chunks, partitioner classes
(API of t5x/partitioning.py).

The reference hands shardings to pjit and lets GSPMD insert collectives. Here every process
owns exactly one GPU ("one host = one device"), parameters are created already sharded along
the `model` axis by the layer library, and collectives are explicit (NCCL or the fused peer-
memory kernels). What this module keeps from the reference is everything that other layers
observe: the mesh and its axis names, the rule tables and the logical -> mesh axis resolution,
`PartitionSpec`s for every train-state leaf (they decide which checkpoint leaves are sharded
arrays and which rank writes which chunk), the data layout for the input pipeline, and the
`partition()/compile()` call shape used by the trainer and `get_infer_fn`.
"""
from __future__ import annotations

import abc
import collections
import dataclasses
import logging
from typing import Any, Callable, Mapping, Optional, Sequence, Set, Tuple, Union

import numpy as np
import torch

from t5x_b200.parallel import state as pstate
from t5x_b200.utils import tree as tree_utils

LogicalAxisRules = Sequence[Tuple[str, Optional[str]]]
HardwareMesh = Tuple[int, ...]


class PartitionSpec(tuple):
  """Tuple of mesh-axis names (or None, or tuples of names) per array dimension."""

  def __new__(cls, *partitions):
    return super().__new__(cls, partitions)

  def __repr__(self):
    return "PartitionSpec%s" % (tuple(self),)


P = PartitionSpec


class AxisNames(tuple):
  """Tuple of logical axis names for one array (t5x/partitioning.py:53-65)."""

  def __new__(cls, *names):
    return super().__new__(cls, names)

  def __repr__(self):
    return "AxisNames%s" % (tuple(self),)


def with_sharding_constraint(x, axis_resources):
  """Activation sharding hint. Shardings are explicit in this framework, so this is the
  identity (as it is on CPU in the reference, t5x/partitioning.py:68-73)."""
  return x


# ----------------------------------------------------------------------------
# Mesh
# ----------------------------------------------------------------------------
class Mesh:
  """An n-d grid of ranks with named axes. `local_rank` is the rank this process (or the
  simulated host under test) owns."""

  def __init__(self, devices, axis_names: Sequence[str], local_rank: Optional[int] = None):
    self.devices = np.asarray(devices)
    self.axis_names = tuple(axis_names)
    assert self.devices.ndim == len(self.axis_names)
    self.local_rank = pstate.get().rank if local_rank is None else local_rank

  @property
  def shape(self) -> "collections.OrderedDict[str, int]":
    return collections.OrderedDict(zip(self.axis_names, self.devices.shape))

  @property
  def size(self) -> int:
    return int(self.devices.size)

  def coords(self, rank: Optional[int] = None) -> "collections.OrderedDict[str, int]":
    rank = self.local_rank if rank is None else rank
    loc = np.argwhere(self.devices == rank)
    if len(loc) == 0:
      raise ValueError(f"rank {rank} is not part of the mesh")
    return collections.OrderedDict(zip(self.axis_names, (int(i) for i in loc[0])))

  @property
  def local_mesh(self) -> "Mesh":
    c = self.coords()
    idx = tuple(slice(c[a], c[a] + 1) for a in self.axis_names)
    return Mesh(self.devices[idx], self.axis_names, self.local_rank)

  def __repr__(self):
    return f"Mesh({dict(self.shape)}, local_rank={self.local_rank})"


def bounds_from_last_device(last_device) -> HardwareMesh:
  """Kept for API parity: (x, y, z, cores) bounds of a TPU slice."""
  if hasattr(last_device, "coords"):
    x, y, z = last_device.coords
    return x + 1, y + 1, z + 1, last_device.core_on_chip + 1
  return int(last_device) + 1, 1


def get_coords(device) -> HardwareMesh:
  if hasattr(device, "coords"):
    return (*device.coords, device.core_on_chip)
  return (int(device), 0)


def get_gpu_mesh(num_partitions: int, world_size: Optional[int] = None,
                 local_rank: Optional[int] = None) -> Mesh:
  """`model` axis filled first from consecutive (NVLink-adjacent) ranks, the rest is `data`
  (t5x/partitioning.py:272-291)."""
  world = pstate.get().world_size if world_size is None else world_size
  if world % num_partitions:
    raise ValueError(f"world size {world} is not divisible by num_partitions {num_partitions}")
  devices = np.arange(world).reshape(world // num_partitions, num_partitions)
  return Mesh(devices, ("data", "model"), local_rank)


def get_cpu_mesh(world_size: Optional[int] = None, local_rank: Optional[int] = None) -> Mesh:
  world = pstate.get().world_size if world_size is None else world_size
  return Mesh(np.arange(world).reshape(world, 1), ("data", "model"), local_rank)


def get_mesh(model_parallel_submesh: HardwareMesh, input_devices: Sequence[Any] = (),
             input_local_devices: Sequence[Any] = (), tile_by_host_if_needed: bool = True,
             backend: Optional[str] = None, world_size: Optional[int] = None,
             local_rank: Optional[int] = None) -> Mesh:
  """Mesh from a model-parallel submesh: its volume is the size of the `model` axis."""
  return get_gpu_mesh(int(np.prod(model_parallel_submesh)), world_size, local_rank)


def default_mesh(num_partitions: int, model_parallel_submesh: Optional[HardwareMesh] = None,
                 backend: Optional[str] = None, ici_mesh_shape: Optional[HardwareMesh] = None,
                 dcn_mesh_shape: Optional[HardwareMesh] = None, world_size: Optional[int] = None,
                 local_rank: Optional[int] = None) -> Mesh:
  """The mesh for this job (t5x/partitioning.py:294-411). With ici/dcn mesh shapes the result
  has axes (`replica`, `data`, `model`); a single box only ever has replica = 1."""
  if ici_mesh_shape is not None and dcn_mesh_shape is not None:
    shape = tuple(int(i) * int(d) for i, d in zip(ici_mesh_shape, dcn_mesh_shape))
    world = pstate.get().world_size if world_size is None else world_size
    if int(np.prod(shape)) != world:
      raise ValueError(f"ici x dcn mesh {shape} does not cover {world} devices")
    names = ("replica", "data", "model")[-len(shape):]
    return Mesh(np.arange(world).reshape(shape), names, local_rank)
  if model_parallel_submesh is not None:
    return get_mesh(model_parallel_submesh, backend=backend, world_size=world_size,
                    local_rank=local_rank)
  return get_gpu_mesh(num_partitions, world_size, local_rank)


# ----------------------------------------------------------------------------
# Local chunks
# ----------------------------------------------------------------------------
@dataclasses.dataclass
class LocalChunkInfo:
  slice: Tuple[slice, ...]
  replica_id: int


class LocalChunker:
  """Answers, for this process, "which block of a sharded global array is mine, and which
  copy of that block am I?" (the role of t5x/partitioning.py:424-542).

  Along every mesh axis the devices of one process form one chunk; `num_chunks[axis]` is how
  many such chunks the axis has and `chunk_ids[axis]` which of them this process is. A block
  index over several mesh axes, and the replica index over the axes an array is NOT sharded
  on, are both mixed-radix numbers in those digits, most significant axis first."""

  def __init__(self, global_mesh: Mesh):
    self.global_mesh = global_mesh
    per_process = global_mesh.local_mesh.shape
    here = global_mesh.coords()
    self.mesh_axes = list(global_mesh.shape.keys())
    self.num_chunks = collections.OrderedDict(
        (a, global_mesh.shape[a] // per_process[a]) for a in self.mesh_axes)
    self.chunk_ids = collections.OrderedDict(
        (a, here[a] // per_process[a]) for a in self.mesh_axes)

  def _mixed_radix(self, axes) -> Tuple[int, int]:
    """(value, radix product) of this process's chunk digits along `axes`, in that order."""
    value, span = 0, 1
    for a in axes:
      value = value * self.num_chunks[a] + self.chunk_ids[a]
      span *= self.num_chunks[a]
    return value, span

  @staticmethod
  def _as_axes(spec) -> Tuple[str, ...]:
    if not spec:
      return ()
    return (spec,) if isinstance(spec, str) else tuple(a for a in spec if a)

  def get_local_chunk_info(self, global_shape: Tuple[int, ...],
                           mesh_axes: Sequence[Optional[str]]) -> LocalChunkInfo:
    block, used = [], set()
    # a spec shorter than the array's rank leaves the trailing dimensions whole
    specs = list(mesh_axes) + [None] * (len(global_shape) - len(mesh_axes))
    for extent, spec in zip(global_shape, specs):
      axes = self._as_axes(spec)
      if not axes:
        block.append(slice(None))
        continue
      used.update(axes)
      index, count = self._mixed_radix(axes)
      width = extent // count
      block.append(slice(index * width, (index + 1) * width))
    return LocalChunkInfo(tuple(block), self.get_replica_id(used))

  def get_shard_id(self, sharded_mesh_axes: Union[str, Set[Optional[str]], Sequence]) -> int:
    return self._mixed_radix(self._as_axes(sharded_mesh_axes))[0]

  def get_replica_id(self, sharded_mesh_axes: Union[str, Set[Optional[str]], Sequence]) -> int:
    sharded = set(self._as_axes(sharded_mesh_axes))
    return self._mixed_radix([a for a in self.mesh_axes if a not in sharded])[0]


# ----------------------------------------------------------------------------
# Logical axis rules
# ----------------------------------------------------------------------------
def standard_logical_axis_rules(activation_partitioning_dims: int = 1,
                                parameter_partitioning_dims: int = 1,
                                additional_rules: Optional[LogicalAxisRules] = None
                                ) -> LogicalAxisRules:
  """The four rule presets keyed by (activation, parameter) partitioning dims
  (t5x/partitioning.py:545-625)."""
  a, p = activation_partitioning_dims, parameter_partitioning_dims
  base = [("batch", "data"), ("vocab", "model")]
  tail = [("mlp", "model"), ("heads", "model"), ("kv", None), ("joined_kv", "model")]
  if a == 1 and p == 1:
    rules = base + [("embed", None)] + tail
  elif a == 2 and p == 1:
    rules = base + tail + [("embed", "model")]
  elif a == 1 and p == 2:
    rules = base + tail + [("embed", "data")]
  elif a == 2 and p == 2:
    rules = base + tail + [("embed", "model"), ("embed", "data")]
  else:
    raise ValueError(f"`activation_partitioning_dims` = {a} `parameter_partitioning_dims` = "
                     f"{p} is not supported.")
  rules.extend([("relpos_buckets", None), ("abspos_buckets", None), ("length", None),
                ("layers", None), ("stack", None), ("mlp_activations", None)])
  if additional_rules:
    rules.extend(additional_rules)
  return rules


def logical_to_mesh_axes(array_dim_names: Optional[Sequence[Optional[str]]],
                         rules: LogicalAxisRules) -> Optional[PartitionSpec]:
  """Resolves logical names to mesh axes: rules are tried in priority order; a rule applies to
  a dimension that is still unassigned if its mesh axis is not yet used by another dimension
  of the same array; a name with no rule at all is an error (flax
  `logical_to_mesh_axes` semantics, docs/usage/partitioning.md:159-187)."""
  if array_dim_names is None:
    return None
  result = [_UNASSIGNED] * len(array_dim_names)
  for rule_name, rule_mesh in rules:
    if rule_name in array_dim_names:
      pos = array_dim_names.index(rule_name)
      used = [r for r in result if r is not _UNASSIGNED and r is not None]
      flat_used = set()
      for r in used:
        flat_used.update((r,) if isinstance(r, str) else r)
      mesh_set = set() if rule_mesh is None else set(
          (rule_mesh,) if isinstance(rule_mesh, str) else rule_mesh)
      if result[pos] is _UNASSIGNED and not (mesh_set & flat_used):
        result[pos] = rule_mesh
  for i, name in enumerate(array_dim_names):
    if result[i] is _UNASSIGNED:
      if name is None:
        result[i] = None
      elif any(name == r for r, _ in rules):
        result[i] = None  # every rule for this name was blocked by an earlier assignment
      else:
        raise ValueError(f"Unmatched logical axis name '{name}' in {tuple(array_dim_names)} "
                         f"with rules {list(rules)}")
  return PartitionSpec(*result)


class _Unassigned:
  def __repr__(self):
    return "UNASSIGNED"


_UNASSIGNED = _Unassigned()


# ----------------------------------------------------------------------------
# Partitioners
# ----------------------------------------------------------------------------
@dataclasses.dataclass
class DataLayout:
  """Which shard of the global batch this host reads (t5x/partitioning.py:637-643)."""
  batch_size: int
  shard_id: int
  num_shards: int
  is_first_host_in_replica_set: bool


PartitionedCallable = Callable[..., Any]
CompiledPartitionedCallable = Callable[..., Any]


class PjittedFnWithContext:
  """A function bound to a mesh and axis rules (t5x/partitioning.py:943-964). Calling it runs
  the function eagerly on this rank's shards; `lower().compile()` returns it unchanged."""

  def __init__(self, fn: Callable, partition_mesh: Mesh,
               logical_axis_rules: LogicalAxisRules = (), in_axis_resources=None,
               out_axis_resources=None, static_argnums=(), donate_argnums=()):
    self._fn = fn
    self._mesh = partition_mesh
    self._logical_axis_rules = logical_axis_rules
    self.in_axis_resources = in_axis_resources
    self.out_axis_resources = out_axis_resources
    self.static_argnums = static_argnums
    self.donate_argnums = donate_argnums

  def __call__(self, *args, **kwargs):
    return self._fn(*args, **kwargs)

  def lower(self, *args, **kwargs):
    return self

  def compile(self):
    return self


class BasePartitioner(metaclass=abc.ABCMeta):
  """Interface for partitioning computations across hardware devices
  (t5x/partitioning.py:650-940)."""

  def __init__(self, num_partitions: Optional[int] = None,
               model_parallel_submesh: Optional[HardwareMesh] = None,
               params_on_devices: bool = True, backend: Optional[str] = None,
               ici_mesh_shape: Optional[HardwareMesh] = None,
               dcn_mesh_shape: Optional[HardwareMesh] = None, world_size: Optional[int] = None,
               local_rank: Optional[int] = None):
    if not num_partitions and model_parallel_submesh is None and ici_mesh_shape is None:
      raise ValueError("At least one of `num_partitions`, `model_parallel_submesh` or "
                       "`ici_mesh_shape` must be set.")
    if model_parallel_submesh is not None and len(model_parallel_submesh) != 4:
      logging.warning("`model_parallel_submesh` should be a 4-tuple; using its volume.")
    self._num_partitions = num_partitions
    self._model_parallel_submesh = model_parallel_submesh
    self._params_on_devices = params_on_devices
    self._data_axis = "data"
    self._backend = backend
    self._ici_mesh_shape = ici_mesh_shape
    self._dcn_mesh_shape = dcn_mesh_shape
    self._world_size = world_size
    self._local_rank = local_rank
    self._mesh_cache = None
    self._chunker_cache = None

  @property
  def mesh(self) -> Mesh:
    if self._mesh_cache is None:
      self._mesh_cache = default_mesh(self._num_partitions or 1, self._model_parallel_submesh,
                                      self._backend, self._ici_mesh_shape, self._dcn_mesh_shape,
                                      self._world_size, self._local_rank)
    return self._mesh_cache

  @property
  def _local_chunker(self) -> LocalChunker:
    if self._chunker_cache is None:
      self._chunker_cache = LocalChunker(self.mesh)
    return self._chunker_cache

  @property
  def data_partition_spec(self) -> PartitionSpec:
    return PartitionSpec(self._data_axis)

  @property
  def data_mesh_size(self) -> int:
    axes = (self._data_axis,) if isinstance(self._data_axis, str) else self._data_axis
    return int(np.prod([self.mesh.shape[a] for a in axes]))

  @property
  def data_shards(self) -> int:
    axes = (self._data_axis,) if isinstance(self._data_axis, str) else self._data_axis
    return int(np.prod([self._local_chunker.num_chunks[a] for a in axes]))

  @property
  def data_shard_id(self) -> int:
    return self._local_chunker.get_shard_id(self._data_axis)

  def get_data_layout(self, batch_size: Optional[int] = None,
                      host_index: Optional[int] = None) -> DataLayout:
    if host_index is not None:
      raise NotImplementedError("Explicit host_index is not yet implemented.")
    if self._data_axis is None:
      return DataLayout(batch_size=batch_size, shard_id=0, num_shards=1,
                        is_first_host_in_replica_set=(self.mesh.local_rank == 0))
    batch_size = batch_size or self.data_mesh_size
    if batch_size % self.data_mesh_size:
      raise ValueError(f"Batch size ({batch_size}) must be divisible by corresponding data mesh "
                       f"size ({self.data_mesh_size}).")
    if batch_size % self.data_shards:
      raise ValueError(f"Batch size ({batch_size}) must be divisible by number of data shards "
                       f"({self.data_shards}).")
    replica_id = self._local_chunker.get_replica_id(self._data_axis)
    return DataLayout(batch_size=int(batch_size), shard_id=int(self.data_shard_id),
                      num_shards=int(self.data_shards),
                      is_first_host_in_replica_set=(replica_id == 0))

  def get_local_chunk_info(self, global_shape: Tuple[int, ...],
                           mesh_axes: Sequence[Optional[str]]) -> LocalChunkInfo:
    return self._local_chunker.get_local_chunk_info(global_shape, mesh_axes)

  @property
  def params_on_devices(self):
    return self._params_on_devices

  def move_params_to_devices(self, train_state, train_state_axes):
    """Parameters are created on their devices, already sharded; nothing to move."""
    return train_state

  @abc.abstractmethod
  def get_mesh_axes(self, train_state):
    ...

  def get_logical_axes(self, train_state):
    """None for every leaf: this partitioner has no logical names."""
    return tree_utils.tree_map(lambda _: None, train_state.state_dict())

  @abc.abstractmethod
  def partition(self, fn: Callable, in_axis_resources, out_axis_resources,
                static_argnums: Union[int, Sequence[int]] = (),
                donate_argnums: Union[int, Sequence[int]] = ()) -> PartitionedCallable:
    ...

  @abc.abstractmethod
  def compile(self, partitioned_fn: PartitionedCallable, *args) -> CompiledPartitionedCallable:
    ...


class BasePjitPartitioner(BasePartitioner):
  """Partitioner that binds functions to the mesh (t5x/partitioning.py:967-1004)."""

  def partition(self, fn, in_axis_resources, out_axis_resources, static_argnums=(),
                donate_argnums=()):
    return PjittedFnWithContext(fn, self.mesh, (), in_axis_resources, out_axis_resources,
                                static_argnums, donate_argnums)

  def compile(self, partitioned_fn, *args):
    return partitioned_fn.lower(*args).compile()


class PjitPartitioner(BasePjitPartitioner):
  """Partitioner that resolves logical axis names with rule tables
  (t5x/partitioning.py:1007-1149)."""

  def __init__(self, num_partitions: Optional[int] = None,
               model_parallel_submesh: Optional[HardwareMesh] = None,
               params_on_devices: bool = True, backend: Optional[str] = None,
               ici_mesh_shape: Optional[HardwareMesh] = None,
               dcn_mesh_shape: Optional[HardwareMesh] = None,
               logical_axis_rules: Optional[LogicalAxisRules] = None,
               world_size: Optional[int] = None, local_rank: Optional[int] = None):
    super().__init__(num_partitions=num_partitions,
                     model_parallel_submesh=model_parallel_submesh,
                     params_on_devices=params_on_devices, backend=backend,
                     ici_mesh_shape=ici_mesh_shape, dcn_mesh_shape=dcn_mesh_shape,
                     world_size=world_size, local_rank=local_rank)
    if logical_axis_rules is None:
      logical_axis_rules = standard_logical_axis_rules()
    if ici_mesh_shape is not None and dcn_mesh_shape is not None:
      # Split the batch over the replica axis too (t5x/partitioning.py:1077-1086).
      logical_axis_rules = [(k, ("replica", "data") if k == "batch" else v)
                            for k, v in logical_axis_rules]
      self._data_axis = ("replica", "data")
    self._logical_axis_rules = tuple(logical_axis_rules)

  @property
  def logical_axis_rules(self):
    return self._logical_axis_rules

  @property
  def partitions_parameters_over_data(self) -> bool:
    """True when the rules place a parameter axis on the 'data' mesh axis
    (`parameter_partitioning_dims=2`: 'embed' -> 'data', t5x/partitioning.py:584-604). The
    trainer enacts that as optimizer sharding by ownership over the data axis: each replica
    holds the fp32 master, the optimizer slots and the update of its share of the parameters."""
    for logical, mesh_axis in self._logical_axis_rules:
      axes = mesh_axis if isinstance(mesh_axis, (tuple, list)) else (mesh_axis,)
      if logical == "embed" and "data" in axes:
        return True
    return False

  use_shardy_partitioner = False

  def partition(self, fn, in_axis_resources, out_axis_resources, static_argnums=(),
                donate_argnums=()):
    return PjittedFnWithContext(fn, self.mesh, self._logical_axis_rules, in_axis_resources,
                                out_axis_resources, static_argnums, donate_argnums)

  def get_logical_axes(self, train_state):
    return train_state.as_logical_axes()

  def get_mesh_axes(self, train_state):
    """PartitionSpec for every leaf of the train state (same tree as `state_dict()`)."""
    logical_axes = self.get_logical_axes(train_state)

    def to_mesh(names):
      if names is None:
        return None
      return logical_to_mesh_axes(tuple(names), self._logical_axis_rules)

    sd = logical_axes.state_dict()
    flat = tree_utils.flatten_dict(sd, is_leaf=lambda x: not isinstance(x, Mapping))
    out = {k: (to_mesh(v) if isinstance(v, (tuple, list)) else None) for k, v in flat.items()}
    return logical_axes.restore_state_axes(tree_utils.unflatten_dict(out)) if hasattr(
        logical_axes, "restore_state_axes") else _AxesState(tree_utils.unflatten_dict(out))


class _AxesState:
  """A train-state-shaped container of PartitionSpecs (result of `get_mesh_axes`)."""

  def __init__(self, state_dict):
    self._sd = state_dict

  def state_dict(self):
    return self._sd

  @property
  def params(self):
    return self._sd["target"]

  @property
  def step(self):
    return self._sd["state"].get("step")

  @property
  def param_states(self):
    return self._sd["state"].get("param_states")

  @property
  def flax_mutables(self):
    return self._sd.get("flax_mutables", {})


def host_local_array_to_global_array(arr, mesh=None, pspec=None):
  """Arrays are always rank-local here (t5x/partitioning.py:1154-1162)."""
  return arr


def global_array_to_host_local_array(arr, mesh=None, pspec=None):
  return arr
