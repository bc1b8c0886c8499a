"""Expert-parallel dispatch / combine fused with the NVLink transfers (kernels in csrc/moe.cu).

`MoeExchange` owns two symmetric buffers per expert-parallel group, both laid out
`[E_local, EP, capacity, d]`: `inbox`, which peers write into (token rows on the way to the
experts, or gradients on the way back), and `outbox`, which peers read from (expert outputs,
or gradients of the expert inputs). Phases are separated by the bounded signal-pad barrier.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from t5x_b200.ops import comm, native
from t5x_b200.parallel import state as pstate

c_void_p, c_int = native.c_void_p, native.c_int
_PP = comm._PP
native.register_signature("t5x_moe_scatter", [c_void_p, c_void_p, c_void_p, _PP] + [c_int] * 7 +
                          [c_void_p])
native.register_signature("t5x_moe_gather", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                             _PP] + [c_int] * 7 + [c_void_p])


def enabled(tokens: torch.Tensor) -> bool:
  """The scatter / gather kernels serve any expert-parallel size, one rank included (the
  "peers" are then this GPU's own buffers and no barrier is needed)."""
  return (tokens.is_cuda and tokens.dtype == torch.bfloat16 and
          tokens.shape[-1] % 8 == 0 and os.environ.get("T5X_B200_MOE_FUSED", "1") != "0")


class MoeExchange:
  """Symmetric inbox / outbox of one expert-parallel group (grown on demand, collectively)."""

  def __init__(self, group):
    self.group = group
    self.inbox: Optional[comm.SymmetricBuffer] = None
    self.outbox: Optional[comm.SymmetricBuffer] = None
    self.numel = 0

  def ensure(self, numel: int, device) -> None:
    if numel <= self.numel:
      return
    # every rank computes the same sizes from the same shapes, so this is collective
    self.numel = int(numel * 1.25)
    self.inbox = comm.SymmetricBuffer(self.numel, torch.bfloat16, self.group, device)
    self.outbox = comm.SymmetricBuffer(self.numel, torch.bfloat16, self.group, device)

  def barrier(self, channel: int) -> None:
    self.inbox.barrier(channel)


_EXCHANGES = {}


def exchange_for(group) -> Optional[MoeExchange]:
  if group is None:  # one expert-parallel rank: no shared buffers
    return None
  key = id(group)
  if key not in _EXCHANGES:
    _EXCHANGES[key] = MoeExchange(group)
  return _EXCHANGES[key]


def _scatter(rows, scale, flat_slot, ptrs, capacity, e_local):
  """`ptrs`: ctypes array of every expert-parallel rank's buffer address."""
  st = pstate.get()
  t, d = rows.shape
  native._check(native.lib().t5x_moe_scatter(
      rows.data_ptr(), native.ptr(scale), flat_slot.data_ptr(), ptrs, t,
      flat_slot.shape[1], capacity, e_local, st.expert_size, st.expert_rank, d,
      native.stream_ptr()), "moe_scatter")


def _gather(out, dw, dout, w, flat_slot, ptrs, capacity, e_local, t, d):
  st = pstate.get()
  native._check(native.lib().t5x_moe_gather(
      native.ptr(out), native.ptr(dw), native.ptr(dout), native.ptr(w), flat_slot.data_ptr(),
      ptrs, t, flat_slot.shape[1], capacity, e_local, st.expert_size, st.expert_rank,
      d, native.stream_ptr()), "moe_gather")


def _push(ex: Optional[MoeExchange], rows, scale, flat_slot, capacity, e_local, ep,
          d) -> torch.Tensor:
  """rows -> owners' inboxes; returns this rank's received [E_local, EP * C, d] (a copy)."""
  n = e_local * ep * capacity * d
  if ep == 1:
    # one rank: the "inbox" is a fresh local buffer that is returned as it is
    buf = torch.zeros(n, dtype=torch.bfloat16, device=rows.device)
    _scatter(rows.contiguous(), scale, flat_slot, comm._ptr_array([buf.data_ptr()]), capacity,
             e_local)
    return buf.view(e_local, capacity, d)
  ex.ensure(n, rows.device)
  ex.inbox.tensor[:n].zero_()       # unused slots must read as zero rows
  ex.barrier(0)                     # everyone has cleared before anyone writes
  _scatter(rows.contiguous(), scale, flat_slot, ex.inbox.ptrs_at(0), capacity, e_local)
  ex.barrier(1)                     # all rows have landed
  return ex.inbox.tensor[:n].view(e_local, ep * capacity, d).clone()


def _pull(ex: MoeExchange, local, out, dw, dout, w, flat_slot, capacity, e_local, ep, t, d):
  """Publishes `local` [E_local, EP * C, d] in the outbox and reads this rank's rows back."""
  n = e_local * ep * capacity * d
  if ep == 1:
    local = local.contiguous()
    _gather(out, dw, dout, w, flat_slot, comm._ptr_array([local.data_ptr()]), capacity, e_local,
            t, d)
    return
  ex.ensure(n, local.device)
  ex.outbox.tensor[:n].copy_(local.reshape(-1))
  ex.barrier(2)                     # every outbox is published
  _gather(out, dw, dout, w, flat_slot, ex.outbox.ptrs_at(0), capacity, e_local, t, d)
  ex.barrier(3)                     # nobody still reads an outbox that is about to change


class FusedDispatch(torch.autograd.Function):
  """tokens [T, d] -> expert inputs [E_local, EP * C, d] on the owning ranks."""

  @staticmethod
  def forward(ctx, tokens, flat_slot, num_experts, capacity):
    st = pstate.get()
    ep, el = st.expert_size, num_experts // st.expert_size
    fs = flat_slot.to(torch.int32).contiguous()
    ex = exchange_for(st.expert_group)
    ctx.save_for_backward(fs)
    ctx.meta = (tokens.shape[0], tokens.shape[1], capacity, el, ep)
    return _push(ex, tokens, None, fs, capacity, el, ep, tokens.shape[1])

  @staticmethod
  def backward(ctx, grad_out):
    (fs,) = ctx.saved_tensors
    t, d, capacity, el, ep = ctx.meta
    ex = exchange_for(pstate.get().expert_group)
    g = torch.empty(t, d, dtype=torch.bfloat16, device=grad_out.device)
    _pull(ex, grad_out.contiguous(), g, None, None, None, fs, capacity, el, ep, t, d)
    return g, None, None, None


class FusedCombine(torch.autograd.Function):
  """expert outputs [E_local, EP * C, d] + gates [T, k] -> tokens [T, d]."""

  @staticmethod
  def forward(ctx, expert_out, flat_slot, gate, num_experts, capacity):
    st = pstate.get()
    ep, el = st.expert_size, num_experts // st.expert_size
    fs = flat_slot.to(torch.int32).contiguous()
    t, d = flat_slot.shape[0], expert_out.shape[-1]
    w = gate.float().contiguous()
    ex = exchange_for(st.expert_group)
    out = torch.empty(t, d, dtype=torch.bfloat16, device=expert_out.device)
    _pull(ex, expert_out, out, None, None, w, fs, capacity, el, ep, t, d)
    ctx.save_for_backward(fs, w, expert_out)
    ctx.meta = (t, d, capacity, el, ep, gate.dtype)
    return out

  @staticmethod
  def backward(ctx, grad_out):
    fs, w, expert_out = ctx.saved_tensors
    t, d, capacity, el, ep, gate_dtype = ctx.meta
    ex = exchange_for(pstate.get().expert_group)
    grad_out = grad_out.contiguous()
    # gate gradients: dot(dout[t], expert row) - the rows are read from the owners again
    dw = torch.zeros(t, fs.shape[1], dtype=torch.float32, device=grad_out.device)
    _pull(ex, expert_out, None, dw, grad_out, None, fs, capacity, el, ep, t, d)
    # gradient of the expert outputs: gate-scaled dout rows pushed to the owners
    d_expert = _push(ex, grad_out, w, fs, capacity, el, ep, d)
    return d_expert, None, dw.to(gate_dtype), None, None
