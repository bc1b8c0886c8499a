"""Tensor parallelism with the collectives inside the GEMM kernels.

The reference shards `heads`, `mlp` and `vocab` over the 'model' mesh axis and lets the
compiler place an all-reduce after every row-parallel projection
(t5x/partitioning.py:564-573). Here the residual stream is instead kept row-sharded
(each model rank holds `M / T` consecutive rows of the `[batch * length, d_model]`
activations, "sequence parallel"), which turns every all-reduce into a reduce-scatter after
the row-parallel projection and an all-gather before the next column-parallel one, and both
run inside the tensor-core kernels:

  all_gather_linears      the column-parallel projections (q/k/v, wi_0/wi_1, logits): the
                          kernel pulls the other ranks' row blocks over NVLink into a local
                          buffer while its tensor cores work on the blocks already there
                          (`t5x_gemm_allgather_bf16`); the gathered rows are kept for the
                          weight gradient.
  linear_reduce_scatter   the row-parallel projections (attention out, wo): the epilogue of
                          the GEMM stores each row of the partial product into the inbox of the
                          rank that owns the row (`t5x_gemm_reducescatter_bf16`); the owner adds
                          its `T` inbox slots in fp32.

Backward of one is the other. Buffers that peers read or write live in one symmetric-memory
arena per model group. The kernels order their accesses themselves, through epoch-numbered
signal words that every rank maps (`csrc/gemm_common.cuh`): an all-gather GEMM announces that
its rank's rows are in place and waits for a peer's announcement before it reads from it; a
reduce-scatter GEMM announces that all its stores have been performed and the kernel that sums
the inbox slots waits for every peer's announcement. No barrier kernel runs between them.
Two rules on the host keep reuse of memory safe:

  * the inbox is double-buffered: call n writes the buffer call n - 2 used, and a rank can only
    get to call n after its sum of call n - 1 has seen every peer finish GEMM n - 1, which
    those peers ran after their sum of call n - 2;
  * an arena block that peers may still be reading is not handed out again until this rank has
    enqueued a slot sum (whose wait proves that every peer is past the GEMMs issued before it),
    or a real barrier.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from t5x_b200.ops import comm
from t5x_b200.parallel import state as pstate

_ALIGN = 1024


class _Block:
  """A byte range of the arena. Blocks go back to the free list only at points that every
  rank reaches in the same order: an explicit `release()` (end of the autograd function that
  owns the block) or the arena's `end_step()`. Object lifetime plays no part: a block that is
  merely dropped stays allocated until the end of the step, so ranks whose garbage collectors
  run at different times still hand out identical offsets."""

  def __init__(self, arena, offset: int, size: int):
    self.arena, self.offset, self.size = arena, offset, size
    self.generation = arena.generation

  def tensor(self, shape, dtype=torch.bfloat16) -> torch.Tensor:
    n = 1
    for s in shape:
      n *= int(s)
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    assert nbytes <= self.size
    # `.data`: a tensor of its own for autograd's version counting (kernels and other views
    # write the arena all the time)
    return self.arena.buf.tensor[self.offset:self.offset + nbytes].view(dtype).view(*shape).data

  def peer_ptrs(self, extra_bytes: int = 0) -> List[int]:
    return [p + self.offset + extra_bytes for p in self.arena.buf.peer_ptrs]

  def release(self) -> None:
    """Gives the bytes back. They become allocatable again once peers can no longer be
    reading them (see `SymmetricArena.peers_are_past`)."""
    ar, self.arena = self.arena, None
    if ar is not None and self.generation == ar.generation:
      ar.quarantine.append((self.offset, self.size))


class _Inbox:
  """The reduce-scatter inbox as [T, M / T, N] bf16 on every rank."""

  def __init__(self, arena, buf):
    self.arena, self.buf = arena, buf

  def tensor(self, shape, dtype=torch.bfloat16) -> torch.Tensor:
    n = 1
    for s in shape:
      n *= int(s)
    return self.buf.tensor[:n * 2].view(dtype).view(*shape).data

  def peer_ptrs(self, extra_bytes: int = 0) -> List[int]:
    return [p + extra_bytes for p in self.buf.peer_ptrs]


class SymmetricArena:
  """One symmetric allocation per model group with a first-fit allocator. Every rank runs the
  same program, so every rank hands out the same offsets and a peer's copy of a block is at
  the same offset of the peer's mapping."""

  def __init__(self, nbytes: int, group):
    self.buf = comm.SymmetricBuffer(int(nbytes), torch.uint8, group)
    self.rank, self.world = self.buf.rank, self.buf.world
    self.nbytes = int(nbytes)
    self.free = [(0, self.nbytes)]
    self.quarantine = []  # released blocks that peers may still be reading
    self.generation = 0   # bumped by end_step(); blocks of older generations are void
    self.allocations = 0  # blocks handed out so far (cross-checked over ranks in debug runs)
    dev = self.buf.tensor.device
    # arrival counters of the all-gather GEMM (zero between calls) and its exit counter
    self.flags = torch.zeros(1 << 16, dtype=torch.int32, device=dev)
    self.exit_count = torch.zeros(1, dtype=torch.int32, device=dev)
    # epoch-numbered signal words, one array per rank, mapped by all ranks
    self.sig = comm.SymmetricBuffer(64, torch.int32, group, dev)
    self.sig.tensor.zero_()
    torch.cuda.synchronize(dev)
    dist.barrier(group=group)  # every rank's words are zero before anyone raises one
    self.epoch = 0
    # The inboxes of the reduce-scatter kernels are buffers of their own (peers write them,
    # only this rank reads them), used alternately.
    self._inboxes = [None, None]
    self._inbox_turn = 0
    self._group = group

  def alloc(self, nbytes: int) -> _Block:
    size = -(-int(nbytes) // _ALIGN) * _ALIGN
    for i, (off, sz) in enumerate(self.free):
      if sz >= size:
        if sz == size:
          del self.free[i]
        else:
          self.free[i] = (off + size, sz - size)
        self.allocations += 1
        return _Block(self, off, size)
    if self.quarantine:
      # out of proven-free bytes: a real barrier proves the quarantined ones free
      self.barrier()
      return self.alloc(nbytes)
    raise RuntimeError(
        f"tensor-parallel arena exhausted ({size} bytes wanted); raise T5X_B200_TP_ARENA_GB")

  def _free(self, offset: int, size: int) -> None:
    self.free.append((offset, size))
    self.free.sort()
    merged = []
    for off, sz in self.free:
      if merged and merged[-1][0] + merged[-1][1] == off:
        merged[-1] = (merged[-1][0], merged[-1][1] + sz)
      else:
        merged.append((off, sz))
    self.free = merged

  def next_epoch(self) -> int:
    """The epoch number of the next tensor-parallel GEMM (every rank counts the same calls)."""
    self.epoch = (self.epoch + 1) & 0xFFFFFFFF
    return self.epoch

  def sig_local_ptr(self, kind: int) -> int:
    return self.sig.tensor.data_ptr() + kind * 16 * 4

  def peers_are_past(self) -> None:
    """Called when a kernel has been enqueued whose wait proves that every peer has finished
    the tensor-parallel GEMMs issued so far: released blocks may be handed out again to work
    enqueued from here on."""
    for off, size in self.quarantine:
      self._free(off, size)
    self.quarantine = []

  def end_step(self) -> None:
    """Called by the trainer between steps, when no activation of the step is alive any more:
    after a barrier every block still allocated (dropped without `release()`, or kept by an
    exception path) is voided and the whole arena is free again. With
    `T5X_B200_TP_ARENA_CHECK=1` the ranks also compare how many blocks they have handed out; a
    difference means their programs diverged and peers would read each other's bytes at the
    wrong offsets."""
    self.barrier()
    self.generation += 1
    self.free = [(0, self.nbytes)]
    self.quarantine = []
    if os.environ.get("T5X_B200_TP_ARENA_CHECK", "0") == "1" and dist.is_initialized():
      mine = torch.tensor([self.allocations], dtype=torch.int64, device=self.buf.tensor.device)
      every = [torch.zeros_like(mine) for _ in range(self.world)]
      dist.all_gather(every, mine, group=self._group)
      counts = [int(t) for t in every]
      if len(set(counts)) != 1:
        raise RuntimeError(f"tensor-parallel arena: ranks handed out {counts} blocks; their "
                           "allocation sequences differ")

  def next_inbox(self, nbytes: int) -> "_Inbox":
    """The inbox for the next reduce-scatter (the two buffers take turns). Growing them is a
    collective allocation behind a barrier."""
    if self._inboxes[0] is None or self._inboxes[0].tensor.numel() < nbytes:
      self.barrier()  # nobody is still writing the buffers being replaced
      self._inboxes = [comm.SymmetricBuffer(int(nbytes), torch.uint8, self._group),
                       comm.SymmetricBuffer(int(nbytes), torch.uint8, self._group)]
    self._inbox_turn ^= 1
    return _Inbox(self, self._inboxes[self._inbox_turn])

  def barrier(self) -> None:
    """A real barrier kernel over the group (step boundaries, buffer growth, arena pressure)."""
    self.buf.barrier(channel=0)
    self.peers_are_past()

  def settle(self) -> None:
    """Barrier if released blocks are still waiting for proof that peers are done with them."""
    if self.quarantine:
      self.barrier()


_ARENA: Optional[SymmetricArena] = None


def arena() -> SymmetricArena:
  global _ARENA
  if _ARENA is None:
    st = pstate.get()
    gb = float(os.environ.get("T5X_B200_TP_ARENA_GB", "12"))
    _ARENA = SymmetricArena(int(gb * (1 << 30)), st.model_group)
  return _ARENA


def end_step() -> None:
  """Between forward passes that no trainer step follows (evaluation, scoring, the encoder pass
  of a decode): gives all bytes of the arena back, at a point every rank reaches in the same
  order. A training loop does this once per step (`Trainer._after_step`)."""
  if _ARENA is not None:
    _ARENA.end_step()


def enabled() -> bool:
  """Fused tensor-parallel kernels run on GPUs when the model axis has more than one rank
  (`T5X_B200_TP_FUSED=0` keeps the all-reduce form of `t5x_b200.parallel.tp`)."""
  st = pstate.get()
  return (st.model_size > 1 and st.device.type == "cuda" and dist.is_initialized() and
          os.environ.get("T5X_B200_TP_FUSED", "1") != "0")


# ---- kernel wrappers ----------------------------------------------------------------------
def _native():
  from t5x_b200.ops import native
  if not getattr(_native, "_registered", False):
    vp, ci, ll = native.c_void_p, native.c_int, native.c_ll
    pp = ctypes.POINTER(vp)
    cu = ctypes.c_uint
    native.register_signature(
        "t5x_gemm_allgather_bf16",
        [vp, pp, ci, ci, ci, vp, vp, vp, vp, ci, ci, ci, ll, ll, ci, ci, vp, vp, ll, vp, pp, cu,
         vp, vp])
    native.register_signature("t5x_gemm_allgather_flag_words", [ci, ci])
    native.register_signature("t5x_slot_sum_bf16", [vp, ci, ll, vp, vp, vp])
    native.register_signature("t5x_slot_sum_wait_bf16", [vp, ci, ll, vp, vp, vp, ci, ci, cu, vp])
    native.register_signature(
        "t5x_gemm_reducescatter_bf16",
        [vp, vp, pp, ci, ci, ci, ci, ci, ci, ll, ll, ll, ci, ci, vp, ll, vp, pp, cu, vp, vp])
    _native._registered = True
  return native


def _ptr_array(ptrs: Sequence[int]):
  from t5x_b200.ops import comm
  return comm._ptr_array(ptrs)


def _b_layout(b: torch.Tensor):
  """(mn_major, ld) of b as the [K, N] operand of the kernel."""
  if b.stride(-2) == 1:
    return 0, b.stride(-1)
  if b.stride(-1) == 1:
    return 1, b.stride(-2)
  raise ValueError(f"b with strides {b.stride()} is neither row- nor column-major")


def gemm_allgather(block: _Block, M: int, K: int, b: torch.Tensor, *,
                   b2: Optional[torch.Tensor] = None, save_h: Optional[torch.Tensor] = None
                   ) -> torch.Tensor:
  """C [M, N] = A @ b (or gelu(A @ b) * (A @ b2)), where A [M, K] is `block` of the arena on
  every rank and only this rank's row block of it is filled on entry; the rest arrives from
  the peers inside the kernel. On return (in stream order) `block` holds all of A."""
  native = _native()
  ar = block.arena
  N = b.shape[1]
  b_mn, ldb = _b_layout(b)
  out = torch.empty((M, N), dtype=torch.bfloat16, device=b.device)
  h0 = h1 = ldh = 0
  if b2 is not None:
    assert b2.stride() == b.stride() and b2.shape == b.shape
    if save_h is not None:
      h0 = save_h.data_ptr()
      h1 = h0 + N * 2
      ldh = save_h.stride(0)
  a = block.tensor((M, K))
  if native.lib().t5x_gemm_allgather_flag_words(ar.world, M // ar.world) > ar.flags.numel():
    raise RuntimeError(f"gemm_allgather: {M} rows need more arrival counters than the arena has")
  native._check(native.lib().t5x_gemm_allgather_bf16(
      a.data_ptr(), _ptr_array(block.peer_ptrs()), ar.world, ar.rank, M // ar.world,
      ar.flags.data_ptr(), b.data_ptr(), native.ptr(b2), out.data_ptr(), M, N, K, ldb,
      out.stride(0), b_mn, 1 if b2 is not None else 0, h0, h1, ldh, ar.sig.tensor.data_ptr(),
      _ptr_array(ar.sig.peer_ptrs), ar.next_epoch(), ar.exit_count.data_ptr(),
      native.stream_ptr()), "gemm_allgather")
  return out


def gemm_reducescatter(a: torch.Tensor, b: torch.Tensor, inbox: _Inbox, *,
                       residual: Optional[torch.Tensor] = None) -> int:
  """Stores the bf16 partial product a [M, K] @ b [K, N] (+ residual [M, N]) of this rank
  into slot `rank` of the owners' inboxes (`inbox`: [T, M / T, N] bf16 on every rank).
  Returns the epoch whose "scattered" signals the sum over the slots has to wait for."""
  native = _native()
  ar = inbox.arena
  M, K = a.shape
  N = b.shape[1]
  a_mn, lda, _ = native._mat_layout(a, M, K)
  b_mn, ldb = _b_layout(b)
  rows = M // ar.world
  slot = ar.rank * rows * N * 2
  r_ptr = ldr = 0
  if residual is not None:
    assert residual.dtype == torch.bfloat16 and residual.stride(1) == 1
    r_ptr, ldr = residual.data_ptr(), residual.stride(0)
  epoch = ar.next_epoch()
  native._check(native.lib().t5x_gemm_reducescatter_bf16(
      a.data_ptr(), b.data_ptr(), _ptr_array(inbox.peer_ptrs(slot)), ar.world, ar.rank, rows, M,
      N, K, lda, ldb, N, a_mn, b_mn, r_ptr, ldr, ar.sig.tensor.data_ptr(),
      _ptr_array(ar.sig.peer_ptrs), epoch, ar.exit_count.data_ptr(), native.stream_ptr()),
      "gemm_reducescatter")
  return epoch


# ---- building blocks ----------------------------------------------------------------------
def rows_buffer(m: int, k: int):
  """(block, dst): an arena block for a gathered [m * T, k] bf16 matrix and the view of this
  rank's rows of it. A producer that writes its [m, k] result into `dst` saves the copy that
  `all_gather_linears(..., block=None)` would make."""
  ar = arena()
  blk = ar.alloc(m * ar.world * k * 2)  # only bytes no peer can still be reading
  return blk, blk.tensor((m * ar.world, k))[ar.rank * m:(ar.rank + 1) * m]


def _gather_block(rows: torch.Tensor, blk: Optional[_Block] = None) -> _Block:
  """An arena block shaped [M, K] whose block of this rank holds `rows` ([M / T, K]). `blk`:
  the block `rows` already lives in (see `rows_buffer`). The all-gather GEMM that consumes
  the block tells the peers that the rows are there."""
  m, k = rows.shape
  if blk is None:
    blk, dst = rows_buffer(m, k)
    dst.copy_(rows)
  return blk


def _reduce_scatter(a: torch.Tensor, b: torch.Tensor, residual: Optional[torch.Tensor] = None,
                    add_rows: Optional[torch.Tensor] = None) -> torch.Tensor:
  """bf16 [M / T, N]: this rank's rows of the sum over ranks of (a @ b + residual), plus
  `add_rows` ([M / T, N], this rank's rows of a replicated-sum term such as the residual
  stream). The sum over the inbox slots is taken in fp32."""
  native = _native()
  ar = arena()
  M, N = a.shape[0], b.shape[1]
  m = M // ar.world
  inbox = ar.next_inbox(M * N * 2)
  epoch = gemm_reducescatter(a, b, inbox, residual=residual)
  out = torch.empty((m, N), dtype=torch.bfloat16, device=a.device)
  if add_rows is not None:
    assert add_rows.dtype == torch.bfloat16 and add_rows.is_contiguous()
  # the sum waits (inside the kernel) until every peer's rows have landed
  native._check(native.lib().t5x_slot_sum_wait_bf16(
      inbox.tensor((ar.world, m, N)).data_ptr(), ar.world, m * N, native.ptr(add_rows),
      out.data_ptr(), ar.sig_local_ptr(1), ar.world, ar.rank, epoch, native.stream_ptr()),
      "slot_sum_wait_bf16")
  ar.peers_are_past()
  return out


def _weight2d(w: torch.Tensor, k: int) -> torch.Tensor:
  from t5x_b200.ops import functional as F
  return F.compute_weight(w, torch.bfloat16).reshape(k, -1)


def _column_blocks(ts: Sequence[torch.Tensor]) -> Optional[torch.Tensor]:
  """If the 2-D tensors `ts` ([rows, n_i], unit inner stride) are consecutive column blocks of
  one row-major matrix, that matrix [rows, sum n_i]; else None. Used to run the projections of
  q, k and v (whose bf16 weights are kept side by side in one buffer) as one GEMM, and to use
  their gradients, which the attention backward writes side by side, without a copy."""
  t0 = ts[0]
  if t0.dim() != 2 or t0.stride(1) != 1:
    return None
  ld, total = t0.stride(0), 0
  for t in ts:
    if (t.dim() != 2 or t.stride() != (ld, 1) or t.shape[0] != t0.shape[0] or
        t.dtype != t0.dtype or t.data_ptr() != t0.data_ptr() + total * t0.element_size()):
      return None
    total += t.shape[1]
  if total > ld:
    return None
  return torch.as_strided(t0, (t0.shape[0], total), (ld, 1))


def fuse_weight_columns(params: Sequence[torch.Tensor]) -> bool:
  """Puts the bf16 working copies (`p.bf16`) of 2-D parameters with equal row counts side by
  side in one buffer, as strided views, so that `_column_blocks` finds them. The optimizer
  kernels write working copies through their row stride, so the views stay current. Returns
  False (and changes nothing) when a copy is missing or managed elsewhere (optimizer sharding
  keeps the working copies in a buffer of its own)."""
  bfs = [getattr(p, "bf16", None) for p in params]
  if any(b is None or b.dim() != 2 for b in bfs) or \
      any(getattr(p, "zero", None) is not None for p in params):
    return False
  if _column_blocks(bfs) is not None:
    return True
  with torch.no_grad():
    k = bfs[0].shape[0]
    widths = [b.shape[1] for b in bfs]
    fused = torch.empty((k, sum(widths)), dtype=bfs[0].dtype, device=bfs[0].device)
    col = 0
    for p, b, n in zip(params, bfs, widths):
      view = fused[:, col:col + n]
      view.copy_(b)
      p.bf16 = view
      col += n
  return True


class _AllGatherLinearsFn(torch.autograd.Function):
  """(h_sp [M/T, K]; W_0.. [K, N_i]) -> y_i [M, N_i] = allgather(h_sp) @ W_i. With `gated`,
  the single output is gelu(A @ W_0) * (A @ W_1)."""

  @staticmethod
  def forward(ctx, h_sp, gated, blk, *weights):
    from t5x_b200.ops import native
    ar = arena()
    m, k = h_sp.shape
    M = m * ar.world
    blk = _gather_block(h_sp, blk)
    ws = [_weight2d(w, k) for w in weights]
    ctx.h = None
    if gated:
      ctx.h = torch.empty((M, 2 * ws[0].shape[1]), dtype=torch.bfloat16, device=h_sp.device)
      outs = [gemm_allgather(blk, M, k, ws[0], b2=ws[1], save_h=ctx.h)]
    else:
      fused = _column_blocks(ws) if len(ws) > 1 else None
      if fused is not None:
        # q | k | v side by side: one GEMM with three times the work to hide the gather behind
        out = gemm_allgather(blk, M, k, fused)
        outs = list(torch.split(out, [w.shape[1] for w in ws], dim=1))
      else:
        outs = [gemm_allgather(blk, M, k, ws[0])]
        a_full = blk.tensor((M, k))
        outs += [native.gemm(a_full, w) for w in ws[1:]]
    ctx.blk, ctx.weights, ctx.gated, ctx.shape = blk, weights, gated, (M, k)
    if not any(ctx.needs_input_grad):
      # no backward will come for this block: give the bytes back here (the next user of
      # them waits at the arena's barrier for the peers that still read them)
      blk.release()
      ctx.blk = ctx.h = None
    return tuple(outs)

  @staticmethod
  def backward(ctx, *douts):
    from t5x_b200.ops import functional as F, native
    M, k = ctx.shape
    blk, weights = ctx.blk, ctx.weights
    a_full = blk.tensor((M, k))
    ws = [_weight2d(w, k) for w in weights]
    if ctx.gated:
      dff = ws[0].shape[1]
      dh = ctx.h
      native.gated_gelu_bwd_(douts[0].reshape(M, dff).contiguous(), dh)
      dys = [dh[:, :dff], dh[:, dff:]]
    else:
      dys = []
      for d in douts:
        if d is not None:
          d = d.reshape(M, -1)
          d = d if d.stride(1) == 1 else d.contiguous()
        dys.append(d)
    dws = []
    for i, (w, dy) in enumerate(zip(weights, dys)):
      need = ctx.needs_input_grad[3 + i] and dy is not None
      dws.append(F._accumulate_wgrad(w, a_full.t(), dy) if need else None)
    blk.release()
    ctx.blk = ctx.h = None
    dh_sp = None
    if ctx.needs_input_grad[0]:
      live = [(dy, w) for dy, w in zip(dys, ws) if dy is not None]
      fused_w = _column_blocks([w for _, w in live]) if len(live) > 1 else None
      if fused_w is not None:
        # dx = [dq | dk | dv] @ [Wq | Wk | Wv]^T as one reduce-scatter GEMM
        dy_all = _column_blocks([dy for dy, _ in live])
        if dy_all is None:
          dy_all = torch.cat([dy for dy, _ in live], dim=1)
        live = [(dy_all, fused_w)]
      partial = None
      for dy, w in live[:-1]:
        if partial is None:
          partial = native.gemm(dy, w.t())
        else:
          native.gemm(dy, w.t(), out=partial, accumulate=True)
      dy, w = live[-1]
      dh_sp = _reduce_scatter(dy, w.t(), residual=partial)
    return (dh_sp, None, None) + tuple(dws)


class _LinearReduceScatterFn(torch.autograd.Function):
  """(a [M, K_local]; W [K_local, N]; residual_sp [M/T, N]) -> this rank's rows of
  sum_ranks(a @ W) + residual_sp."""

  @staticmethod
  def forward(ctx, a, weight, residual_sp):
    k = a.shape[-1]
    a2 = a.reshape(-1, k)
    w2 = _weight2d(weight, k)
    y = _reduce_scatter(a2, w2, add_rows=None if residual_sp is None else residual_sp.contiguous())
    ctx.save_for_backward(a, weight)
    ctx.has_res = residual_sp is not None
    return y

  @staticmethod
  def backward(ctx, dy_sp):
    from t5x_b200.ops import functional as F
    a, weight = ctx.saved_tensors
    k = a.shape[-1]
    a2 = a.reshape(-1, k)
    w2 = _weight2d(weight, k)
    M, N = a2.shape[0], w2.shape[1]
    blk = _gather_block(dy_sp.contiguous())
    da = gemm_allgather(blk, M, N, w2.t()).view(a.shape)
    dw = None
    if ctx.needs_input_grad[1]:
      dw = F._accumulate_wgrad(weight, a2.t(), blk.tensor((M, N)))
    blk.release()
    return da, dw, (dy_sp if ctx.has_res else None)


def all_gather_linears(h_sp: torch.Tensor, weights: Sequence[torch.Tensor],
                       block: Optional[_Block] = None) -> List[torch.Tensor]:
  """Column-parallel projections of row-sharded activations: [allgather(h_sp) @ W for W].
  `block`: the `rows_buffer` block whose `dst` view `h_sp` is."""
  return list(_AllGatherLinearsFn.apply(h_sp.contiguous(), False, block, *weights))


def all_gather_gated_gelu(h_sp: torch.Tensor, wi_0: torch.Tensor, wi_1: torch.Tensor,
                          block: Optional[_Block] = None) -> torch.Tensor:
  """gelu(A @ wi_0) * (A @ wi_1) with A = allgather(h_sp)."""
  return _AllGatherLinearsFn.apply(h_sp.contiguous(), True, block, wi_0, wi_1)[0]


def linear_reduce_scatter(a: torch.Tensor, weight: torch.Tensor,
                          residual_sp: Optional[torch.Tensor] = None) -> torch.Tensor:
  """Row-parallel projection: this rank's rows of sum_ranks(a @ W) (+ residual_sp)."""
  return _LinearReduceScatterFn.apply(a, weight, residual_sp)


# ---- entering and leaving the row-sharded region (NCCL; once per layer stack) --------------
class _ScatterRowsFn(torch.autograd.Function):
  """Replicated [M, d] -> this rank's rows. Backward all-gathers the row gradients."""

  @staticmethod
  def forward(ctx, x):
    st = pstate.get()
    m = x.shape[0] // st.model_size
    return x[st.model_rank * m:(st.model_rank + 1) * m].contiguous()

  @staticmethod
  def backward(ctx, g):
    st = pstate.get()
    out = torch.empty((g.shape[0] * st.model_size,) + tuple(g.shape[1:]), dtype=g.dtype,
                      device=g.device)
    dist.all_gather_into_tensor(out, g.contiguous(), group=st.model_group)
    return out


class _GatherRowsFn(torch.autograd.Function):
  """Row-sharded [M/T, d] -> replicated [M, d]. With `partial_grads` the consumers are
  model-sharded and leave partial sums as gradients, which backward reduce-scatters;
  otherwise the gradient arrives already summed and backward keeps this rank's rows."""

  @staticmethod
  def forward(ctx, x_sp, partial_grads):
    st = pstate.get()
    ctx.partial_grads = partial_grads
    out = torch.empty((x_sp.shape[0] * st.model_size,) + tuple(x_sp.shape[1:]), dtype=x_sp.dtype,
                      device=x_sp.device)
    dist.all_gather_into_tensor(out, x_sp.contiguous(), group=st.model_group)
    return out

  @staticmethod
  def backward(ctx, g):
    st = pstate.get()
    m = g.shape[0] // st.model_size
    if not ctx.partial_grads:
      return g[st.model_rank * m:(st.model_rank + 1) * m].contiguous(), None
    out = torch.empty((m,) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
    dist.reduce_scatter_tensor(out, g.contiguous(), group=st.model_group)
    return out, None


def scatter_rows(x: torch.Tensor) -> torch.Tensor:
  return _ScatterRowsFn.apply(x)


def gather_rows(x_sp: torch.Tensor, partial_grads: bool) -> torch.Tensor:
  return _GatherRowsFn.apply(x_sp, partial_grads)


def usable(x: torch.Tensor, rows: int) -> bool:
  """The fused path covers bf16 CUDA activations whose rows divide evenly over the ranks."""
  st = pstate.get()
  return (enabled() and x.is_cuda and x.dtype == torch.bfloat16 and rows % st.model_size == 0)
