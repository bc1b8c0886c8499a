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
  global _STATE
  _STATE = ParallelState()


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
