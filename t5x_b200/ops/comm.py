"""Python entry points of the NVLink peer-memory kernels in `csrc/comm.cu`.

`SymmetricBuffer` is a device buffer that every rank of a process group has mapped: rank d's
copy is visible here as `peer_ptrs[d]`. Allocation and handle exchange go through
`torch.distributed._symmetric_memory`; the data path (reduce, broadcast, barrier, and the
optimizer kernels fused with them) is this package's own kernels using plain loads and stores
on the peer mappings.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from t5x_b200.ops import native

c_void_p, c_int, c_ll, c_float = native.c_void_p, native.c_int, native.c_ll, native.c_float
c_uint, c_ull = ctypes.c_uint, ctypes.c_ulonglong
_PP = ctypes.POINTER(c_void_p)

native.register_signature("t5x_comm_barrier", [_PP, c_int, c_int, c_int, c_uint, c_ull, c_void_p])
native.register_signature("t5x_peer_reduce_f32", [c_void_p, _PP, c_int, c_ll, c_void_p])
native.register_signature("t5x_peer_push_bf16", [_PP, c_void_p, c_int, c_int, c_ll, c_void_p])
native.register_signature("t5x_dist_adafactor_stats",
                          [c_void_p, _PP, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                           c_float, c_void_p])
native.register_signature("t5x_dist_adafactor_apply",
                          [c_void_p, c_void_p, c_void_p, _PP, c_int, c_void_p, c_int, c_int, c_int,
                           c_ll, c_float, c_float, c_float, c_float, c_float, c_float, c_int,
                           c_void_p])

native.register_signature("t5x_dist_adafactor_stats_mc",
                          [c_void_p, _PP, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                           c_float, c_void_p])
native.register_signature("t5x_dist_adafactor_apply_mc",
                          [c_void_p, c_void_p, c_void_p, _PP, c_int, c_void_p, c_void_p, c_int,
                           c_int, c_int, c_ll, c_float, c_float, c_float, c_float, c_float,
                           c_float, c_int, c_void_p])
native.register_signature("t5x_comm_set_max_ctas", [c_int])

MAX_PEERS = 16
# Polls (64 ns apart at least) a barrier waits before it gives up: about two seconds.
DEFAULT_SPIN_LIMIT = 1 << 24


def nvls_requested() -> bool:
  """In-switch reduction / multicast for the sharded-optimizer exchange (`T5X_B200_NVLS=1`)."""
  return os.environ.get("T5X_B200_NVLS", "0") == "1"


def _ptr_array(ptrs: Sequence[int]):
  return (c_void_p * len(ptrs))(*[c_void_p(int(p)) for p in ptrs])


class SymmetricBuffer:
  """`numel` elements of `dtype` on every rank of `group`, mapped into every rank."""

  def __init__(self, numel: int, dtype: torch.dtype, group=None, device=None):
    import torch.distributed._symmetric_memory as symm_mem
    # By default memory stays unbound from the switch's multicast object (plain peer loads and
    # stores only): a rank that dies then cannot disturb its peers' GPUs. `T5X_B200_NVLS=1`
    # (set before the first buffer of the process is created) binds the buffers, and
    # `multicast_ptr` is then the address on which `multimem` instructions reach all copies.
    if not nvls_requested():
      os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    group = group if group is not None else dist.group.WORLD
    device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    self.group = group
    self.rank = dist.get_rank(group)
    self.world = dist.get_world_size(group)
    if self.world > MAX_PEERS:
      raise ValueError(f"at most {MAX_PEERS} ranks per symmetric buffer, got {self.world}")
    self.tensor = symm_mem.empty(int(numel), dtype=dtype, device=device)
    self.handle = symm_mem.rendezvous(self.tensor, group)
    self.peer_ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
    self.pad_ptrs: List[int] = [int(p) for p in self.handle.signal_pad_ptrs]
    self.itemsize = self.tensor.element_size()
    self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0) \
        if nvls_requested() else 0
    self._epochs = {}

  def mc_ptr_at(self, offset_elems: int) -> int:
    """Multicast address of element `offset_elems` (0 when the buffer is not bound)."""
    return self.multicast_ptr + offset_elems * self.itemsize if self.multicast_ptr else 0

  def ptrs_at(self, offset_elems: int):
    """ctypes array of every rank's address of element `offset_elems`."""
    return _ptr_array([p + offset_elems * self.itemsize for p in self.peer_ptrs])

  def barrier(self, channel: int = 0, spin_limit: int = DEFAULT_SPIN_LIMIT) -> None:
    """Stream-ordered barrier over the group through the signal pads. Work enqueued before it
    on every rank's stream is complete, and its writes visible, once it returns on the
    stream. A rank that never arrives makes the wait give up after `spin_limit` polls with
    status 'peer flag timeout' (read by `native.check_status()`)."""
    barrier(self.pad_ptrs, self.rank, self.world, channel, self._next_epoch(channel), spin_limit)

  def _next_epoch(self, channel: int) -> int:
    e = self._epochs.get(channel, 0) + 1
    self._epochs[channel] = e
    return e & 0xFFFFFFFF or 1


def barrier(pad_ptrs: Sequence[int], rank: int, world: int, channel: int, epoch: int,
            spin_limit: int = DEFAULT_SPIN_LIMIT) -> None:
  native._check(native.lib().t5x_comm_barrier(_ptr_array(pad_ptrs), rank, world, channel,
                                              epoch, spin_limit, native.stream_ptr()),
                "comm_barrier")


def peer_reduce_f32_(dst: torch.Tensor, src_ptrs, n: int) -> None:
  """dst[:n] = sum over ranks of the fp32 arrays at `src_ptrs` (ctypes pointer array)."""
  native._check(native.lib().t5x_peer_reduce_f32(dst.data_ptr(), src_ptrs, len(src_ptrs), n,
                                                 native.stream_ptr()), "peer_reduce_f32")


def peer_copy_bf16_(dst_ptr: int, src_ptr: int, n: int) -> None:
  """Copies n bf16 elements between raw addresses (either may be another rank's memory as
  mapped here; plain loads and stores)."""
  native._check(native.lib().t5x_peer_push_bf16(_ptr_array([dst_ptr]), c_void_p(int(src_ptr)), 1,
                                                -1, n, native.stream_ptr()), "peer_copy_bf16")


def peer_push_bf16_(dst_ptrs, src: torch.Tensor, n: int, skip_rank: int = -1) -> None:
  """Stores src[:n] (bf16) to every rank's array at `dst_ptrs` except `skip_rank`."""
  native._check(native.lib().t5x_peer_push_bf16(dst_ptrs, src.data_ptr(), len(dst_ptrs),
                                                skip_rank, n, native.stream_ptr()),
                "peer_push_bf16")


def dist_adafactor_stats_(p, grad_ptrs, g_out, scratch, batch, rows, cols, eps1,
                          grad_mc: int = 0) -> None:
  """`grad_mc`: multicast address of the gradient (0: the owner loads every rank's copy)."""
  native._check(native.lib().t5x_dist_adafactor_stats_mc(
      p.data_ptr(), grad_ptrs, len(grad_ptrs), grad_mc, g_out.data_ptr(), scratch.data_ptr(),
      batch, rows, cols, eps1, native.stream_ptr()), "dist_adafactor_stats")


def dist_adafactor_apply_(p, g, m, bf16_ptrs, scratch, batch, rows, cols, n_global, *, lr, eps2,
                          clip_threshold, weight_decay, beta1, max_param_scale, flags,
                          bf16_mc: int = 0) -> None:
  """`bf16_mc`: multicast address of the working copies (0: one store per rank)."""
  native._check(native.lib().t5x_dist_adafactor_apply_mc(
      p.data_ptr(), g.data_ptr(), native.ptr(m), bf16_ptrs, len(bf16_ptrs), bf16_mc,
      scratch.data_ptr(), batch, rows, cols, n_global, lr, eps2, clip_threshold, weight_decay,
      beta1, max_param_scale, flags, native.stream_ptr()), "dist_adafactor_apply")


def set_max_ctas(max_ctas: int) -> None:
  """Caps the grid of the NVLink-fused optimizer kernels (0: two CTAs per SM), so that they
  leave room for the GEMMs they overlap with."""
  native.lib().t5x_comm_set_max_ctas(int(max_ctas))
