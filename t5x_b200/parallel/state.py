"""Process-level parallel state: one process per GPU, a `data x model` (x `expert`) mesh.

The reference derives every collective from pjit shardings (t5x/partitioning.py); here
the mesh is explicit. `model` is the fastest-varying axis so that tensor-parallel peers
are NVLink neighbours on one node (the role of t5x/partitioning.py:272-291).
"""
from __future__ import annotations

import dataclasses
import os
from typing import Optional

import torch
import torch.distributed as dist


@dataclasses.dataclass
class ParallelState:
  world_size: int = 1
  rank: int = 0
  data_size: int = 1
  model_size: int = 1
  expert_size: int = 1
  data_rank: int = 0
  model_rank: int = 0
  expert_rank: int = 0
  model_group: Optional[object] = None
  data_group: Optional[object] = None
  expert_group: Optional[object] = None
  device: torch.device = torch.device("cpu")

  @property
  def tp(self) -> int:
    return self.model_size

  @property
  def is_distributed(self) -> bool:
    return self.world_size > 1


_STATE = ParallelState()


def get() -> ParallelState:
  return _STATE


def reset() -> None:
  global _STATE, _CONTROL_GROUP
  _STATE = ParallelState()
  _CONTROL_GROUP = None


def init_distributed(backend: Optional[str] = None, timeout_s: float = 600.0) -> None:
  """Joins the torchrun rendezvous (RANK/WORLD_SIZE/MASTER_* from the environment)."""
  if dist.is_initialized() or int(os.environ.get("WORLD_SIZE", "1")) <= 1:
    return
  import datetime
  os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
  if backend is None:
    backend = "nccl" if torch.cuda.is_available() else "gloo"
  if backend == "nccl":
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
  dist.init_process_group(backend=backend, timeout=datetime.timedelta(seconds=timeout_s))


# ----------------------------------------------------------------------------
# Host-side control plane
# ----------------------------------------------------------------------------
class HostSyncError(RuntimeError):
  """A host-level barrier or agreement between ranks did not complete in time: some rank
  crashed, hung or never reached the named point."""


_CONTROL_GROUP = None


def control_group():
  """A gloo group over all ranks for host-level synchronisation (checkpoint phases, stop and
  preemption flags: the role of the coordination service behind
  jax.experimental.multihost_utils). It involves no GPU work, so a rank that died cannot park
  the others inside a device collective: its absence shows up as a timeout error on the host.
  Created on first use; with a gloo default group that group itself serves."""
  global _CONTROL_GROUP
  if not dist.is_initialized() or dist.get_world_size() <= 1:
    return None
  if _CONTROL_GROUP is None:
    if dist.get_backend() == "gloo":
      _CONTROL_GROUP = dist.group.WORLD
    else:
      _CONTROL_GROUP = dist.new_group(backend="gloo")
  return _CONTROL_GROUP


def host_sync_timeout_s() -> float:
  return float(os.environ.get("T5X_B200_HOST_SYNC_TIMEOUT_S", "1800"))


def host_barrier(name: str, timeout_s: Optional[float] = None) -> None:
  """Barrier over all ranks on the host. If a rank does not arrive within `timeout_s`
  (default `T5X_B200_HOST_SYNC_TIMEOUT_S`, 30 minutes) every waiting rank raises
  `HostSyncError` naming the barrier instead of waiting forever."""
  group = control_group()
  if group is None:
    return
  import datetime
  t = host_sync_timeout_s() if timeout_s is None else float(timeout_s)
  try:
    dist.monitored_barrier(group=group, timeout=datetime.timedelta(seconds=t))
  except RuntimeError as e:
    raise HostSyncError(f"host barrier '{name}' did not complete within {t:.0f} s on rank "
                        f"{dist.get_rank()}: {e}") from e


def host_any(flag: bool) -> bool:
  """True on every rank if `flag` is true on any rank (one small gloo all-reduce)."""
  group = control_group()
  if group is None:
    return bool(flag)
  t = torch.tensor([1 if flag else 0], dtype=torch.int32)
  dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
  return bool(int(t[0]))


def setup_mesh(model_size: int = 1, expert_size: int = 1,
               device: Optional[torch.device] = None) -> ParallelState:
  """Builds the mesh groups. world = data x expert x model, model fastest.

  The `expert` axis is carved out of the data axis (t5x/contrib/moe/partitioning.py:59-118):
  data-parallel batch sharding uses both `expert` and `data`.
  """
  global _STATE
  world = dist.get_world_size() if dist.is_initialized() else 1
  rank = dist.get_rank() if dist.is_initialized() else 0
  if world % (model_size * expert_size) != 0:
    raise ValueError(f"world size {world} is not divisible by model={model_size} x "
                     f"expert={expert_size}")
  data_size = world // (model_size * expert_size)
  if device is None:
    device = (torch.device("cuda", torch.cuda.current_device())
              if torch.cuda.is_available() else torch.device("cpu"))
  st = ParallelState(world_size=world, rank=rank, data_size=data_size, model_size=model_size,
                     expert_size=expert_size, device=device)
  st.model_rank = rank % model_size
  st.expert_rank = (rank // model_size) % expert_size
  st.data_rank = rank // (model_size * expert_size)
  if world > 1:
    # model groups: consecutive ranks
    for start in range(0, world, model_size):
      ranks = list(range(start, start + model_size))
      g = dist.new_group(ranks) if model_size > 1 else None
      if rank in ranks:
        st.model_group = g
    # expert groups: same data index and model index
    for d in range(data_size):
      for m in range(model_size):
        ranks = [d * expert_size * model_size + e * model_size + m for e in range(expert_size)]
        g = dist.new_group(ranks) if expert_size > 1 else None
        if rank in ranks:
          st.expert_group = g
    # data groups (gradient reduction for non-expert params): same model index, all data+expert
    for m in range(model_size):
      ranks = [r for r in range(world) if r % model_size == m]
      g = dist.new_group(ranks) if len(ranks) > 1 else None
      if rank in ranks:
        st.data_group = g
  _STATE = st
  return st
