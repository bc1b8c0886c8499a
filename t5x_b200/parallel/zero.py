"""Optimizer sharding over the data axis by parameter ownership.

With D data-parallel replicas, every parameter has one owner rank. All ranks hold the bf16
working weights and accumulate full fp32 gradients locally; at the end of a step the owner of
a parameter

  1. pulls the D gradient copies over NVLink and sums them inside the optimizer's first pass
     (`t5x_dist_adafactor_stats`), so the reduce-scatter is never a separate collective,
  2. runs the rest of the update on its own fp32 master copy and optimizer slots, and
  3. stores the new bf16 weights straight into every replica's working copy from the update
     kernel (`t5x_dist_adafactor_apply`), so there is no separate all-gather either.

Two stream-ordered barriers bracket the update: one after backward (all gradient copies are
complete) and one after the update (all pushes have landed, and nobody is still reading this
rank's gradients). fp32 master weights and optimizer slots of parameters a rank does not own go
stale during training; `sync_replicas()` refreshes them from the owners and is called whenever
the state leaves the training loop (end of `Trainer.train`, checkpointing, evaluation of
weight metrics).

This is the reference's "2-D parameter partitioning" (optimizer state sharded over the data
axis, t5x/partitioning.py:615-676) restated for one process per GPU with peer memory.
"""
from __future__ import annotations

import logging
import os
import re
from typing import Dict, List, Mapping, Optional

import numpy as np
import torch
import torch.distributed as dist

from t5x_b200.parallel import state as pstate

_ALIGN = 128  # elements; keeps every parameter's offset 256-byte aligned in both buffers
_LAYER_RE = re.compile(r"(.*\.)?layers_\d+")  # the transformer layers of a stack


class ZeroInfo:
  """Per-parameter record: where it lives in the symmetric buffers and who updates it.

  `offset` locates the fp32 gradient (every rank holds a full copy). `w_offset` locates the
  bf16 working weights: for a replicated parameter the same place on every rank; for a
  `streamed` one (weights sharded over the data axis) the place in the OWNER's buffer, the only
  copy that persists between uses."""
  __slots__ = ("ctx", "offset", "numel", "owner", "w_offset", "streamed")

  def __init__(self, ctx, offset: int, numel: int, owner: int, w_offset: Optional[int] = None,
               streamed: bool = False):
    self.ctx, self.offset, self.numel, self.owner = ctx, offset, numel, owner
    self.w_offset = offset if w_offset is None else w_offset
    self.streamed = streamed

  @property
  def mine(self) -> bool:
    return self.owner == self.ctx.rank

  def grad_ptrs(self):
    return self.ctx.grads.ptrs_at(self.offset)

  def bf16_ptrs(self):
    """Where the owner's update kernel stores the new bf16 weights: every replica's working
    copy, or the owner's own shard only when the weights are sharded."""
    if self.streamed:
      from t5x_b200.ops import comm
      return comm._ptr_array([self.owner_weight_ptr()])
    return self.ctx.weights.ptrs_at(self.w_offset)

  def owner_weight_ptr(self) -> int:
    w = self.ctx.weights
    return w.peer_ptrs[self.owner] + self.w_offset * w.itemsize

  def push_skip_rank(self) -> int:
    """`skip_rank` for a separate push of the owner's `p.bf16`: its own replica when weights
    are replicated; none when they are sharded (`p.bf16` is then a transient gather slot and
    the single destination is the owner's shard)."""
    return -1 if self.streamed else self.ctx.rank

  def grad_mc(self) -> int:
    """Multicast address of this parameter's gradient over all replicas (0 without NVLS)."""
    return self.ctx.grads.mc_ptr_at(self.offset) if self.ctx.nvls else 0

  def bf16_mc(self) -> int:
    if self.streamed:
      return 0
    return self.ctx.weights.mc_ptr_at(self.w_offset) if self.ctx.nvls else 0


# Parameters below this size stay replicated: their gradients are all-reduced (coalesced into
# one small collective) and every rank applies the same update to its own fp32 copy.
MIN_OWNED_NUMEL = 1 << 14


def owned_by_one_rank(p) -> bool:
  """Whether parameter `p` gets a single owner rank under optimizer sharding. Only the large
  matrices do: the forward pass reads those through their bf16 working copies, which the
  owner refreshes on every rank. Norm scales, relative-position tables and other small fp32
  parameters are read by the forward pass in fp32 on every rank, so every rank keeps and
  updates its own copy of them."""
  return (isinstance(p, torch.Tensor) and p.is_cuda and p.dtype == torch.float32 and
          p.dim() >= 2 and p.numel() >= MIN_OWNED_NUMEL)


def assign_owners(sizes: Mapping[str, int], world: int) -> Dict[str, int]:
  """Largest-first greedy balancing of parameter sizes over ranks; deterministic."""
  load = [0] * world
  owners = {}
  for name in sorted(sizes, key=lambda k: (-sizes[k], k)):
    r = min(range(world), key=lambda i: (load[i], i))
    owners[name] = r
    load[r] += sizes[name]
  return owners


def plan_buffers(names, sizes: Mapping[str, int], owners: Mapping[str, int], streamed,
                 world: int):
  """Element offsets of every owned parameter in the two symmetric buffers.

  Gradients: a full fp32 copy on every rank, the same layout everywhere. Weights (bf16): the
  replicated parameters first, at the same place on every rank, then each rank's own
  `streamed` parameters (the only persistent copy of those); the buffer is as large as the
  fullest rank needs. Returns (grad offsets, grad elements, weight offsets, weight elements);
  a streamed parameter's weight offset is the one in its OWNER's buffer. Every offset is a
  multiple of `_ALIGN` elements."""
  pad = lambda n: -(-n // _ALIGN) * _ALIGN
  g_off, cursor = {}, 0
  for k in names:
    g_off[k] = cursor
    cursor += pad(sizes[k])
  grad_total = max(cursor, _ALIGN)
  w_off, cursor = {}, 0
  for k in names:
    if k not in streamed:
      w_off[k] = cursor
      cursor += pad(sizes[k])
  own = [cursor] * world
  for k in names:
    if k in streamed:
      w_off[k] = own[owners[k]]
      own[owners[k]] += pad(sizes[k])
  return g_off, grad_total, w_off, max(max(own), _ALIGN)


class ZeroContext:
  """Symmetric gradient / weight buffers for a flat {name: fp32 parameter} mapping."""

  def __init__(self, params_flat: Mapping[str, torch.Tensor], group=None,
               module: Optional[torch.nn.Module] = None, shard_weights: bool = False):
    from t5x_b200.ops import comm
    st = pstate.get()
    self.group = group if group is not None else (st.data_group or dist.group.WORLD)
    self.rank = dist.get_rank(self.group)
    self.world = dist.get_world_size(self.group)
    names = [k for k, p in params_flat.items() if owned_by_one_rank(p)]
    sizes = {k: int(params_flat[k].numel()) for k in names}
    padded = {k: -(-sizes[k] // _ALIGN) * _ALIGN for k in names}
    self.owners = assign_owners(sizes, self.world)
    device = params_flat[names[0]].device
    # Weights sharded over the data axis: the parameters of the transformer layers keep their
    # bf16 working copy on the owner only; everything else (embedding, output projection)
    # stays replicated. `layer_names[j]` lists the streamed parameters of the j-th layer in
    # execution order.
    self.layer_names: List[List[str]] = []
    self._layer_modules: List[torch.nn.Module] = []
    if shard_weights and module is not None:
      by_id = {id(params_flat[k]): k for k in names}
      for mod_name, mod in module.named_modules():
        if _LAYER_RE.fullmatch(mod_name):
          ks = [by_id[id(q)] for q in mod.parameters(recurse=True) if id(q) in by_id]
          if ks:
            self.layer_names.append(ks)
            self._layer_modules.append(mod)
    streamed = {k: j for j, ks in enumerate(self.layer_names) for k in ks}
    self.shard_weights = bool(streamed)
    g_off, self.total, w_off, self.weights_total = plan_buffers(
        names, sizes, self.owners, set(streamed), self.world)
    self.infos: Dict[str, ZeroInfo] = {}
    for k in names:
      self.infos[k] = ZeroInfo(self, g_off[k], sizes[k], self.owners[k], w_off[k], k in streamed)
    self.grads = comm.SymmetricBuffer(self.total, torch.float32, self.group, device)
    self.weights = comm.SymmetricBuffer(self.weights_total, torch.bfloat16, self.group, device)
    # two gather slots, each as large as the largest layer: layer j is gathered into slot j % 2
    self._slots: List[torch.Tensor] = []
    self._slot_off: Dict[str, int] = {}
    if self.shard_weights:
      most = 0
      for ks in self.layer_names:
        cursor = 0
        for k in ks:
          self._slot_off[k] = cursor
          cursor += padded[k]
        most = max(most, cursor)
      self._slots = [torch.empty(most, dtype=torch.bfloat16, device=device) for _ in range(2)]
    for k in names:
      p, info = params_flat[k], self.infos[k]
      g = self.grads.tensor[info.offset:info.offset + info.numel].view(p.shape)
      old = getattr(p, "bf16", None)
      src = old if old is not None else p.detach()
      if info.streamed:
        if info.mine:  # the persistent copy
          self.weights.tensor[info.w_offset:info.w_offset + info.numel].view(p.shape).copy_(src)
        so = self._slot_off[k]
        w = self._slots[streamed[k] % 2][so:so + info.numel].view(p.shape)
      else:
        w = self.weights.tensor[info.w_offset:info.w_offset + info.numel].view(p.shape)
        w.copy_(src)
      g.zero_()
      p.bf16, p.main_grad, p.grad_ready, p.zero = w, g, False, info
    self.params = {k: params_flat[k] for k in names}
    if self.shard_weights:
      self._attach_weight_streaming()
    self._masters_released = False
    if os.environ.get("T5X_B200_ZERO_SHARD_MASTERS", "1") != "0":
      self.release_replica_masters()
    torch.cuda.synchronize(device)
    dist.barrier(group=self.group)
    owned = sum(sizes[k] for k in names if self.owners[k] == self.rank)
    # in-switch gradient sum / multicast weight push (T5X_B200_NVLS=1 and a fabric that has it)
    self.nvls = bool(self.grads.multicast_ptr and self.weights.multicast_ptr)
    logging.info("optimizer sharding: rank %d/%d owns %.1f M of %.1f M parameters%s%s", self.rank,
                 self.world, owned / 1e6, sum(sizes.values()) / 1e6,
                 ", exchange through NVSwitch multimem" if self.nvls else "",
                 (f", bf16 weights of {len(self.layer_names)} layers sharded "
                  f"({self.weights_total / 1e6:.1f} M resident + 2 slots of "
                  f"{self._slots[0].numel() / 1e6:.1f} M)") if self.shard_weights else "")

  # -- weights sharded over the data axis -----------------------------------------------------
  # The forward and backward pass of layer j read its weights from gather slot j % 2. Before
  # the layer runs (module pre-hooks), a side stream copies each of its parameters from the
  # owner's shard (peer loads over NVLink, or a local copy on the owner) into the slot, and the
  # layer after it (before it, in the backward pass) is requested at once into the other slot,
  # so that the copy runs under the current layer's kernels. A gather first waits for
  # everything enqueued on the compute stream so far: that covers the previous user of the
  # slot and, at the start of a step, the barrier after the owners' updates. Slots are
  # invalidated whenever the owners have written new weights.
  def _attach_weight_streaming(self) -> None:
    self._gather_stream = torch.cuda.Stream(device=self.grads.tensor.device)
    self._slot_holds: List[Optional[int]] = [None, None]
    self._slot_ready: List[Optional[torch.cuda.Event]] = [None, None]
    n = len(self._layer_modules)
    self._stream_hooks = []
    for j, mod in enumerate(self._layer_modules):
      self._stream_hooks.append(mod.register_forward_pre_hook(
          lambda m, args, j=j: self._layer_begins(j, j + 1 if j + 1 < n else None)))
      self._stream_hooks.append(mod.register_full_backward_pre_hook(
          lambda m, gout, j=j: self._layer_begins(j, j - 1 if j > 0 else None)))

  def detach_weight_streaming(self) -> None:
    """Removes the gather hooks and gives every streamed parameter a full private bf16 copy
    again (taken from the owners), so that the module keeps working without this context."""
    if not self.shard_weights:
      return
    for h in self._stream_hooks:
      h.remove()
    self._stream_hooks = []
    from t5x_b200.ops import comm
    torch.cuda.current_stream().wait_stream(self._gather_stream)
    for ks in self.layer_names:
      for k in ks:
        p, info = self.params[k], self.infos[k]
        full = torch.empty(p.shape, dtype=torch.bfloat16, device=p.device)
        comm.peer_copy_bf16_(full.data_ptr(), info.owner_weight_ptr(), info.numel)
        p.bf16 = full
    self.shard_weights = False
    torch.cuda.synchronize()
    dist.barrier(group=self.group)  # nobody frees its shard while a peer still copies from it

  def _gather(self, j: int) -> None:
    from t5x_b200.ops import comm
    slot = j % 2
    if self._slot_holds[slot] == j:
      return
    main = torch.cuda.current_stream()
    fence = torch.cuda.Event()
    fence.record(main)
    with torch.cuda.stream(self._gather_stream):
      self._gather_stream.wait_event(fence)
      buf = self._slots[slot]
      for k in self.layer_names[j]:
        info = self.infos[k]
        dst = buf.data_ptr() + self._slot_off[k] * buf.element_size()
        comm.peer_copy_bf16_(dst, info.owner_weight_ptr(), info.numel)
      ready = torch.cuda.Event()
      ready.record(self._gather_stream)
    self._slot_holds[slot] = j
    self._slot_ready[slot] = ready

  def _layer_begins(self, j: int, then: Optional[int]) -> None:
    self._gather(j)
    torch.cuda.current_stream().wait_event(self._slot_ready[j % 2])
    if then is not None:
      self._gather(then)

  def weights_changed(self) -> None:
    """The owners have stored new weights: what the gather slots hold is stale."""
    if self.shard_weights:
      self._slot_holds = [None, None]

  # -- overlap with backward ----------------------------------------------------------------
  # During the last microbatch of a step, the parameters of a transformer layer are final as
  # soon as that layer's backward has been issued. A backward hook on every `layers_N` module
  # then lets a side stream wait for the main stream (CUDA event), meet the other ranks at a
  # barrier, and run the owner's fused reduce + update + weight push for that layer while the
  # main stream continues with the backward pass of the layers below.
  def attach_overlap(self, module: torch.nn.Module, optimizer_def, state_of) -> None:
    """`state_of(name)` returns the optimizer slots of parameter `name` ('/'-joined)."""
    import re
    self._opt_def = optimizer_def
    self._state_of = state_of
    self._side = torch.cuda.Stream(device=self.grads.tensor.device)
    if os.environ.get("T5X_B200_COMM_MAX_CTAS"):
      from t5x_b200.ops import comm
      comm.set_max_ctas(int(os.environ["T5X_B200_COMM_MAX_CTAS"]))
    self._overlap = None          # (step, hyper_params) while the last microbatch runs
    self.done_this_step = set()
    self._buckets = {}
    by_id = {id(p): k for k, p in self.params.items()}
    taken = set()
    stacks = set()
    for mod_name, mod in module.named_modules():
      if not re.fullmatch(r"(.*\.)?layers_\d+", mod_name):
        continue
      names = [by_id[id(p)] for p in mod.parameters(recurse=True) if id(p) in by_id]
      if not names:
        continue
      self._buckets[mod_name] = names
      taken.update(names)
      stacks.add(mod_name.rpartition(".")[0])
      mod.register_full_backward_hook(
          lambda m, gin, gout, bucket=mod_name: self._bucket_ready(bucket))
    # What a layer stack owns besides its layers (final norm, output projection, position
    # biases) is final once the gradient with respect to the stack's input exists. A stack
    # whose inputs need no gradient (token ids) fires its hook early, with no input gradient:
    # `_bucket_ready` ignores that call. Parameters shared between stacks wait for the end.
    uses = {}
    for stack in stacks:
      if stack:
        for p in module.get_submodule(stack).parameters(recurse=True):
          uses[id(p)] = uses.get(id(p), 0) + 1
    for stack in sorted(s for s in stacks if s):
      mod = module.get_submodule(stack)
      names = [by_id[id(p)] for p in mod.parameters(recurse=True)
               if id(p) in by_id and by_id[id(p)] not in taken and uses[id(p)] == 1]
      if not names:
        continue
      self._buckets[stack] = names
      mod.register_full_backward_hook(
          lambda m, gin, gout, bucket=stack: self._bucket_ready(
              bucket, has_input_grad=any(g is not None for g in gin)))

  def begin_overlap(self, step: int, hyper_params) -> None:
    if getattr(self, "_release_after_sync", False):
      self._release_after_sync = False
      self.release_replica_masters()  # full copies were only needed outside the loop
    if getattr(self, "_side", None) is not None:
      self._overlap = (int(step), hyper_params)
      self.done_this_step = set()

  def end_overlap(self) -> None:
    if getattr(self, "_side", None) is not None:
      self._overlap = None
      torch.cuda.current_stream().wait_stream(self._side)

  def _bucket_ready(self, bucket: str, has_input_grad: bool = True) -> None:
    if self._overlap is None or not has_input_grad:
      return
    step, hp = self._overlap
    names = self._final_names(bucket)
    if not names:
      return
    main = torch.cuda.current_stream()
    ev = torch.cuda.Event()
    ev.record(main)
    with torch.cuda.stream(self._side):
      self._side.wait_event(ev)
      self.grads.barrier(channel=2)   # every rank has issued this layer's backward
      saved = self._opt_def.hyper_params
      self._opt_def.hyper_params = hp
      try:
        with torch.no_grad():
          for k in names:
            p = self.params[k]
            if p.zero.mine:
              self._opt_def.apply_param_gradient(step, hp, p, self._state_of(k), p.main_grad, k)
      finally:
        self._opt_def.hyper_params = saved
    self.done_this_step.update(names)

  def _final_names(self, bucket: str) -> List[str]:
    """Parameters of `bucket` whose gradient is final once the bucket's backward has been
    issued: the whole gradient went through the native accumulate path, and no reduction
    over another mesh axis is still owed. Norm scales applied to row-sharded activations
    (`sp_partial_grad`) hold only this model rank's rows until the model-axis sum that runs
    after the backward pass; updating them here would let the model ranks apply different
    updates to a replicated parameter, so they take the ordinary path after that sum."""
    partial_pending = pstate.get().model_size > 1
    out = []
    for k in self._buckets[bucket]:
      p = self.params[k]
      if not getattr(p, "grad_ready", False) or p.grad is not None:
        continue
      if partial_pending and getattr(p, "sp_partial_grad", False):
        continue
      out.append(k)
    return out

  # -- step protocol -------------------------------------------------------------------------
  def gradients_complete(self) -> None:
    """Barrier after the last backward pass: every rank's gradient copy is final."""
    if getattr(self, "_release_after_sync", False):
      self._release_after_sync = False
      self.release_replica_masters()
    self.end_overlap()
    self.grads.barrier(channel=0)

  def update_complete(self) -> None:
    """Barrier after the update: all weight pushes have landed and no rank still reads
    another's gradients."""
    self.grads.barrier(channel=1)
    self.weights_changed()

  # -- fp32 masters live on their owner only ------------------------------------------------
  # Forward and backward read the bf16 working copies and write the gradient buffers; the fp32
  # master of a parameter is touched only by the optimizer, i.e. by its owner. Every other rank
  # therefore keeps no storage for it during training: its `.data` is a one-element tensor
  # expanded to the parameter's shape (all shape queries keep working, 4 bytes are held). For
  # T5.1.1-XXL on 8 GPUs that returns 7/8 of 44.5 GB per rank. `sync_replicas` brings full
  # copies back for checkpointing / returning the state, and the next step drops them again.
  def release_replica_masters(self) -> None:
    if self._masters_released:
      return
    for k, p in self.params.items():
      if self.owners[k] != self.rank:
        p.data = torch.zeros((), dtype=p.dtype, device=p.device).expand(p.shape)
    self._masters_released = True

  def _materialize_replica_masters(self) -> None:
    if not self._masters_released:
      return
    for k, p in self.params.items():
      if self.owners[k] != self.rank:
        p.data = torch.empty(p.shape, dtype=p.dtype, device=p.device)
    self._masters_released = False

  def sync_replicas(self, optimizer_state=None) -> None:
    """Refreshes fp32 master weights (and optimizer slots) on non-owners from the owners."""
    ranks = dist.get_process_group_ranks(self.group)
    was_released = self._masters_released
    self._materialize_replica_masters()
    self._release_after_sync = was_released
    for k, p in self.params.items():
      dist.broadcast(p.data, src=ranks[self.owners[k]], group=self.group)
    if optimizer_state is not None:
      for k, leaves in state_leaves_by_param(self.params.keys(), optimizer_state).items():
        for v in leaves:
          if v.is_cuda:
            dist.broadcast(v, src=ranks[self.owners[k]], group=self.group)


def state_leaves_by_param(param_names, optimizer_state) -> Dict[str, List[torch.Tensor]]:
  """The tensors of an optimizer-state tree that belong to each parameter. Two layouts occur:
  Adafactor keeps a dict of slots under the parameter's path ('<param>/v_row'), optax-style
  states keep a copy of the parameter tree under each moment ('1/0/mu/<param>'). A leaf belongs
  to the parameter whose name is the head or the tail of its path; counters and other leaves
  that match no parameter are left out (they are identical on every rank)."""
  from t5x_b200.utils import tree as tree_utils
  # keyed in the caller's order: every rank walks the result to issue collectives, and the
  # iteration order of a set of strings differs from process to process
  out: Dict[str, List[torch.Tensor]] = {k: [] for k in param_names}
  names = set(out)
  for path, v in tree_utils.flatten_dict(optimizer_state).items():
    if not isinstance(v, torch.Tensor):
      continue
    parts = path.split("/")
    for i in range(len(parts), 0, -1):
      head = "/".join(parts[:i])
      if head in names:
        out[head].append(v)
        break
    else:
      for i in range(1, len(parts)):
        tail = "/".join(parts[i:])
        if tail in names:
          out[tail].append(v)
          break
  return out


class LocalUpdateOverlap:
  """The single-replica form of the overlap above: no gradients to exchange, but the
  optimizer update of a transformer layer (memory-bound) can still run on a side stream as
  soon as that layer's backward has been issued in the last microbatch, under the GEMMs
  (compute-bound) of the layers below."""

  def __init__(self, params_flat: Mapping[str, torch.Tensor], module: torch.nn.Module,
               optimizer_def, state_of):
    import re
    self.params = {k: p for k, p in params_flat.items()
                   if isinstance(p, torch.Tensor) and p.is_cuda and p.dtype == torch.float32}
    self._opt_def, self._state_of = optimizer_def, state_of
    device = next(iter(self.params.values())).device
    self._side = torch.cuda.Stream(device=device)
    self._overlap = None
    self.done_this_step = set()
    self._buckets = {}
    by_id = {id(p): k for k, p in self.params.items()}
    for mod_name, mod in module.named_modules():
      if not re.fullmatch(r"(.*\.)?layers_\d+", mod_name):
        continue
      names = [by_id[id(p)] for p in mod.parameters(recurse=True) if id(p) in by_id]
      if names:
        self._buckets[mod_name] = names
        mod.register_full_backward_hook(
            lambda m, gin, gout, bucket=mod_name: self._bucket_ready(bucket))

  def begin_overlap(self, step: int, hyper_params) -> None:
    self._overlap = (int(step), hyper_params)
    self.done_this_step = set()

  def end_overlap(self) -> None:
    self._overlap = None
    torch.cuda.current_stream().wait_stream(self._side)

  def _bucket_ready(self, bucket: str) -> None:
    if self._overlap is None:
      return
    step, hp = self._overlap
    names = [k for k in self._buckets[bucket]
             if getattr(self.params[k], "grad_ready", False) and self.params[k].grad is None
             and getattr(self.params[k], "main_grad", None) is not None]
    if not names:
      return
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream())
    with torch.cuda.stream(self._side):
      self._side.wait_event(ev)
      saved = self._opt_def.hyper_params
      self._opt_def.hyper_params = hp
      try:
        with torch.no_grad():
          for k in names:
            p = self.params[k]
            self._opt_def.apply_param_gradient(step, hp, p, self._state_of(k), p.main_grad, k)
      finally:
        self._opt_def.hyper_params = saved
    self.done_this_step.update(names)


_ACTIVE: Optional[ZeroContext] = None
_LOCAL: Optional[LocalUpdateOverlap] = None


def enable_local_overlap(params_flat, module, optimizer_def, state_of) -> LocalUpdateOverlap:
  global _LOCAL
  _LOCAL = LocalUpdateOverlap(params_flat, module, optimizer_def, state_of)
  return _LOCAL


def disable_local_overlap() -> None:
  global _LOCAL
  _LOCAL = None


def overlap_controller():
  """Whoever runs optimizer updates under the last backward pass: the sharded-optimizer
  context, the single-replica overlap, or None."""
  if _ACTIVE is not None and getattr(_ACTIVE, "_side", None) is not None:
    return _ACTIVE
  return _LOCAL


def done_this_step():
  """Names of the parameters already updated during the current step's backward pass."""
  ctl = overlap_controller()
  return ctl.done_this_step if ctl is not None else ()


def active() -> Optional[ZeroContext]:
  return _ACTIVE


def enable(params_flat: Mapping[str, torch.Tensor], group=None,
           module: Optional[torch.nn.Module] = None,
           shard_weights: bool = False) -> Optional[ZeroContext]:
  """Shards the optimizer over the data axis if it has more than one replica on GPUs. With
  `shard_weights` (and the model's `module`, whose `layers_N` sub-modules delimit the units of
  gathering) the bf16 working weights of the transformer layers are sharded as well."""
  global _ACTIVE
  st = pstate.get()
  if not dist.is_initialized() or st.data_size <= 1 or st.device.type != "cuda":
    return None
  _ACTIVE = ZeroContext(params_flat, group, module=module, shard_weights=shard_weights)
  return _ACTIVE


def disable() -> None:
  global _ACTIVE, _LOCAL
  if _ACTIVE is not None and getattr(_ACTIVE, "shard_weights", False):
    _ACTIVE.detach_weight_streaming()
  _ACTIVE = None
  _LOCAL = None
