"""Tensor-parallel region boundaries as autograd functions.

These are the collectives that GSPMD inserts for the reference's `heads/mlp/vocab ->
'model'` rules (t5x/partitioning.py:564-573): an all-reduce after every row-parallel
projection and, in backward, after every column-parallel one. This module is the NCCL
form (the comparator); the fused GEMM+collective kernels replace the pair
(projection, collective) where they apply.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from t5x_b200.parallel import state as pstate


def _all_reduce(x: torch.Tensor, group) -> torch.Tensor:
  if group is None:
    return x
  x = x.contiguous()
  dist.all_reduce(x, group=group)
  return x


class _CopyToModel(torch.autograd.Function):
  """Identity forward; all-reduce of the gradient over the model axis backward."""

  @staticmethod
  def forward(ctx, x):
    return x

  @staticmethod
  def backward(ctx, g):
    return _all_reduce(g, pstate.get().model_group)


class _ReduceFromModel(torch.autograd.Function):
  """All-reduce over the model axis forward; identity backward."""

  @staticmethod
  def forward(ctx, x):
    return _all_reduce(x, pstate.get().model_group)

  @staticmethod
  def backward(ctx, g):
    return g


def copy_to_model_parallel(x: torch.Tensor) -> torch.Tensor:
  if pstate.get().model_size == 1:
    return x
  return _CopyToModel.apply(x)


def reduce_from_model_parallel(x: torch.Tensor) -> torch.Tensor:
  if pstate.get().model_size == 1:
    return x
  return _ReduceFromModel.apply(x)


def all_reduce_model(x: torch.Tensor, op=dist.ReduceOp.SUM) -> torch.Tensor:
  """Plain (non-differentiable) all-reduce over the model axis."""
  st = pstate.get()
  if st.model_size == 1:
    return x
  x = x.contiguous()
  dist.all_reduce(x, op=op, group=st.model_group)
  return x


def shard_range(global_size: int, parts: int, index: int):
  """[start, end) of shard `index` when `global_size` is split evenly over `parts`."""
  if global_size % parts != 0:
    raise ValueError(f"size {global_size} is not divisible by {parts} partitions")
  per = global_size // parts
  return index * per, (index + 1) * per
