"""Mixture-of-experts feed-forward layer: tokens-choose top-k router with fixed expert capacity,
expert-parallel dispatch / combine, gated-GELU experts.

The reference takes these layers from Flaxformer; its own code fixes only their contract: the
per-layer metrics `auxiliary_loss, router_z_loss, fraction_tokens_left_behind, expert_usage,
router_confidence` (t5x/contrib/moe/models.py:40-46), the `expert` logical axis and the
`.*expert.*` parameter-name convention (t5x/contrib/moe/trainer.py:39-99,
t5x/contrib/moe/partitioning.py:365-424).

Parameter tree of the layer (it replaces `mlp` of a Transformer block):
  router/router_weights/w/kernel      [embed, num_experts]            fp32, replicated
  expert/wi_0/kernel, expert/wi_1/kernel  [experts, embed, mlp]       sharded over `expert`
  expert/wo/kernel                        [experts, mlp, embed]

Data path with EP expert-parallel ranks (each holds E / EP experts). Every rank routes its own
T tokens into a fixed-capacity buffer `[E, C, d]`:

  dispatch  : token rows are written to slot (expert, position) of the owner rank's receive
              buffer `[E_local, EP, C, d]`;
  experts   : one batched GEMM pair over `[E_local, EP * C, d]`;
  combine   : each rank reads its tokens' expert outputs back and sums them with the gates.

On GPUs dispatch is a push over NVLink peer memory and combine a pull (`ops/moe.py`), so the
all-to-alls never exist as separate collectives; elsewhere (`gloo`, one process) the same slot
arithmetic runs with `all_to_all_single`.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
from torch import nn

from t5x_b200.models.t5 import layers as t5_layers
from t5x_b200.ops import functional as F
from t5x_b200.ops import reference as ref
from t5x_b200.parallel import state as pstate

MOE_METRICS = ("auxiliary_loss", "router_z_loss", "fraction_tokens_left_behind", "expert_usage",
               "router_confidence")

# Per-forward collection of the layers' metrics (the role of flax `sow('intermediates', ...)`).
_COLLECTED: List[Dict[str, torch.Tensor]] = []


def reset_collected_metrics() -> None:
  _COLLECTED.clear()


def collected_metrics() -> List[Dict[str, torch.Tensor]]:
  return list(_COLLECTED)


# ----------------------------------------------------------------------------
# Router
# ----------------------------------------------------------------------------
def expert_capacity(num_tokens: int, num_experts: int, capacity_factor: float,
                    num_selected_experts: int = 1, min_capacity: int = 4) -> int:
  """Slots per expert for a group of `num_tokens` tokens."""
  cap = int(math.ceil(capacity_factor * num_tokens * num_selected_experts / num_experts))
  return max(cap, min_capacity)


def load_balancing_loss(router_probs: torch.Tensor, expert_index: torch.Tensor) -> torch.Tensor:
  """Switch-Transformer auxiliary loss: E^2 * mean_e(fraction routed to e * mean prob of e).
  router_probs [T, E] fp32; expert_index [T, k]."""
  e = router_probs.shape[-1]
  mask = torch.zeros_like(router_probs).scatter_(1, expert_index, 1.0)
  tokens_per_expert = mask.mean(0)
  prob_per_expert = router_probs.mean(0)
  return (tokens_per_expert * prob_per_expert).mean() * float(e * e)


def router_z_loss(router_logits: torch.Tensor) -> torch.Tensor:
  """mean_t logsumexp(logits_t)^2 (ST-MoE)."""
  return torch.logsumexp(router_logits.float(), dim=-1).pow(2).mean()


class RouterWeights(nn.Module):
  def __init__(self, emb_dim: int, num_experts: int, device=None):
    super().__init__()
    self.w = t5_layers.DenseGeneral(emb_dim, num_experts, ("embed", "unmodeled"),
                                    kernel_init=t5_layers.normal_init(2e-2), dtype="float32",
                                    device=device)


class _FusedRouterFn(torch.autograd.Function):
  """The whole tokens-choose router as native kernels (csrc/router.cu): fp32 logits, softmax,
  top-k, capacity positions in token order (first choices before second choices), the two
  losses and the usage metrics in three launches; backward in two. Differentiable outputs:
  the gates (zero where a choice lost its slot), the load-balancing loss and the z-loss."""

  @staticmethod
  def forward(ctx, tokens, w, k, capacity):
    from t5x_b200.ops import native
    wc = w.detach().float().contiguous()
    fwd = native.moe_router_fwd(tokens, wc, k, capacity)
    ctx.save_for_backward(tokens, wc)
    ctx.fwd, ctx.cfg, ctx.w_dtype = fwd, (k, capacity), w.dtype
    m = fwd["metrics"]
    index, flat_slot = fwd["index"], fwd["flat_slot"]
    ctx.mark_non_differentiable(index, flat_slot, m)
    return fwd["gate"], m[0].clone(), m[1].clone(), index, flat_slot, m

  @staticmethod
  def backward(ctx, dgate, daux, dz, _di, _ds, _dm):
    from t5x_b200.ops import native
    tokens, wc = ctx.saved_tensors
    k, capacity = ctx.cfg
    zero = torch.zeros((), dtype=torch.float32, device=tokens.device)
    coef = torch.stack([zero if daux is None else daux.float().reshape(()),
                        zero if dz is None else dz.float().reshape(())])
    if dgate is None:
      dgate = torch.zeros_like(ctx.fwd["gate"])
    dx, dw = native.moe_router_bwd(tokens, wc, k, capacity, ctx.fwd, dgate, coef,
                                   need_dx=ctx.needs_input_grad[0])
    ctx.fwd = None
    return dx, dw.to(ctx.w_dtype), None, None


def fused_router_usable(tokens: torch.Tensor, num_experts: int, k: int) -> bool:
  import os
  from t5x_b200.ops import native
  if os.environ.get("T5X_B200_MOE_FUSED_ROUTER", "1") == "0":
    return False
  return (tokens.is_cuda and tokens.dtype == torch.bfloat16 and tokens.dim() == 2 and
          num_experts <= native.ROUTER_MAX_EXPERTS and k <= native.ROUTER_MAX_CHOICES and
          (num_experts * tokens.shape[1] + 9 * tokens.shape[1]) * 4 <= 190 * 1024)


class TokensChooseRouter(nn.Module):
  """Every token picks its top-k experts; an expert keeps the first `capacity` tokens that
  picked it (all first choices are placed before any second choice)."""

  def __init__(self, emb_dim: int, num_experts: int, num_selected_experts: int = 1,
               jitter_noise: float = 0.0, device=None):
    super().__init__()
    self.num_experts = num_experts
    self.k = num_selected_experts
    self.jitter_noise = jitter_noise
    self.router_weights = RouterWeights(emb_dim, num_experts, device=device)

  def forward(self, tokens: torch.Tensor, capacity: int, enable_dropout: bool = False):
    """tokens [T, d] -> dict(expert_index [T,k], slot [T,k] (−1 = dropped), gate [T,k],
    plus the two losses and the three usage metrics)."""
    jitter = enable_dropout and self.jitter_noise > 0
    if not jitter and fused_router_usable(tokens, self.num_experts, self.k):
      gate, aux, z, index, flat_slot, m = _FusedRouterFn.apply(
          tokens.contiguous(), self.router_weights.w.kernel, self.k, capacity)
      metrics = {"auxiliary_loss": aux, "router_z_loss": z,
                 "fraction_tokens_left_behind": m[2], "expert_usage": m[3],
                 "router_confidence": m[4]}
      return {"expert_index": index, "flat_slot": flat_slot, "gate": gate}, metrics
    x = tokens.float()
    if jitter:
      x = x * torch.empty_like(x).uniform_(1.0 - self.jitter_noise, 1.0 + self.jitter_noise)
    logits = x @ self.router_weights.w.kernel.float()
    probs = torch.softmax(logits, dim=-1)
    gate, index = torch.topk(probs, self.k, dim=-1)              # [T, k]
    t, e = probs.shape
    # position of every (token, choice) inside its expert: choice-major priority
    # (running count per expert along the contiguous axis of an [E, k*T] int32 matrix: the
    # scan over the outer axis of a [k*T, E] int64 one-hot is ~40x slower on the GPU)
    flat = index.t().reshape(-1)                                   # [k*T], choice-major
    hits = (flat[None, :] == torch.arange(e, device=flat.device)[:, None]).to(torch.int32)
    position = torch.cumsum(hits, dim=1).gather(0, flat[None, :]).squeeze(0).long() - 1
    position = position.view(self.k, t).t()                        # [T, k]
    kept = position < capacity
    slot = torch.where(kept, position, torch.full_like(position, -1))
    z = router_z_loss(logits)
    aux = load_balancing_loss(probs, index)
    dispatched_somewhere = kept.any(dim=1).float().sum()
    metrics = {
        "auxiliary_loss": aux,
        "router_z_loss": z,
        "fraction_tokens_left_behind": 1.0 - dispatched_somewhere / float(t),
        "expert_usage": kept.float().sum() / float(e * capacity),
        "router_confidence": (gate * kept.float()).sum() / dispatched_somewhere.clamp(min=1.0),
    }
    return {"expert_index": index, "slot": slot, "gate": gate * kept.to(gate.dtype),
            "flat_slot": _flat_slots(index, slot, capacity)}, metrics


class ExpertsChooseRouter(nn.Module):
  """Every expert picks its `capacity` highest-probability tokens ("experts choose" routing of
  the Flaxformer MoE layers the reference builds on). Experts are always full, so there is no
  load-balancing loss; a token may be processed by several experts or by none. The routing is
  reported in the same form as `TokensChooseRouter` with one "choice" column per expert:
  flat_slot[t, e] is the row of (expert e, position) in the dispatch buffer, or -1 when expert
  e did not pick token t, and gate[t, e] the router probability of the picks."""

  def __init__(self, emb_dim: int, num_experts: int, jitter_noise: float = 0.0, device=None):
    super().__init__()
    self.num_experts = num_experts
    self.jitter_noise = jitter_noise
    self.router_weights = RouterWeights(emb_dim, num_experts, device=device)

  def forward(self, tokens: torch.Tensor, capacity: int, enable_dropout: bool = False):
    x = tokens.float()
    if enable_dropout and self.jitter_noise > 0:
      x = x * torch.empty_like(x).uniform_(1.0 - self.jitter_noise, 1.0 + self.jitter_noise)
    logits = x @ self.router_weights.w.kernel.float()
    probs = torch.softmax(logits, dim=-1)                            # [T, E]
    t, e = probs.shape
    picks = min(capacity, t)
    top_p, top_tok = torch.topk(probs.t(), picks, dim=1)             # [E, picks]
    rows = (torch.arange(e, device=probs.device)[:, None] * capacity +
            torch.arange(picks, device=probs.device)[None, :])       # slot row of (e, position)
    cols = torch.arange(e, device=probs.device)[:, None].expand(e, picks)
    flat_slot = torch.full((t, e), -1, dtype=torch.long, device=probs.device)
    flat_slot[top_tok, cols] = rows
    gate = torch.zeros_like(probs)
    gate[top_tok, cols] = top_p
    chosen = flat_slot >= 0
    dispatched_somewhere = chosen.any(dim=1).float().sum()
    metrics = {
        "auxiliary_loss": torch.zeros((), dtype=torch.float32, device=probs.device),
        "router_z_loss": router_z_loss(logits),
        "fraction_tokens_left_behind": 1.0 - dispatched_somewhere / float(t),
        "expert_usage": torch.as_tensor(float(picks) / float(capacity), device=probs.device),
        "router_confidence": gate.sum() / dispatched_somewhere.clamp(min=1.0),
    }
    index = torch.arange(e, device=probs.device)[None, :].expand(t, e)
    return {"expert_index": index, "flat_slot": flat_slot, "gate": gate}, metrics


# ----------------------------------------------------------------------------
# Dispatch / combine
# ----------------------------------------------------------------------------
def _flat_slots(expert_index, slot, capacity):
  """Row index into the [E * C] dispatch buffer per (token, choice); -1 = dropped."""
  return torch.where(slot >= 0, expert_index * capacity + slot, torch.full_like(slot, -1))


class _Dispatch(torch.autograd.Function):
  """tokens [T, d] -> expert inputs [E_local, EP * C, d] on the owning ranks."""

  @staticmethod
  def forward(ctx, tokens, flat_slot, num_experts, capacity):
    st = pstate.get()
    ep = st.expert_size
    t, d = tokens.shape
    k = flat_slot.shape[1]
    buf = tokens.new_zeros(num_experts * capacity, d)
    valid = flat_slot >= 0
    rows = flat_slot[valid]
    src = torch.arange(t, device=tokens.device)[:, None].expand(t, k)[valid]
    buf[rows] = tokens[src]
    ctx.save_for_backward(flat_slot)
    ctx.shape = (t, d, num_experts, capacity)
    return _exchange(buf.view(num_experts, capacity, d), ep, st.expert_group)

  @staticmethod
  def backward(ctx, grad_out):
    (flat_slot,) = ctx.saved_tensors
    t, d, e, c = ctx.shape
    st = pstate.get()
    g = _exchange_back(grad_out.contiguous(), st.expert_size, st.expert_group, e, c)
    g = g.reshape(e * c, d)
    valid = flat_slot >= 0
    contrib = torch.where(valid[..., None], g[flat_slot.clamp(min=0)], torch.zeros(
        (), dtype=g.dtype, device=g.device))
    return contrib.sum(1), None, None, None


def _exchange(buf: torch.Tensor, ep: int, group) -> torch.Tensor:
  """[E, C, d] on every rank -> [E_local, EP * C, d]: expert e's rows go to rank e // E_local,
  which lays the sources side by side."""
  e, c, d = buf.shape
  if ep == 1:
    return buf
  el = e // ep
  send = buf.view(ep, el, c, d).contiguous()
  recv = torch.empty_like(send)
  dist.all_to_all_single(recv, send, group=group)       # recv[s] = rows sent by rank s
  return recv.permute(1, 0, 2, 3).reshape(el, ep * c, d)


def _exchange_back(x: torch.Tensor, ep: int, group, e: int, c: int) -> torch.Tensor:
  """Inverse of `_exchange`: [E_local, EP * C, d] -> [E, C, d]."""
  if ep == 1:
    return x.view(e, c, -1)
  el, _, d = x.shape
  send = x.view(el, ep, c, d).permute(1, 0, 2, 3).contiguous()
  recv = torch.empty_like(send)
  dist.all_to_all_single(recv, send, group=group)       # recv[r] = my tokens' rows from owner r
  return recv.view(e, c, d)


class _Combine(torch.autograd.Function):
  """expert outputs [E_local, EP * C, d] + gates -> tokens [T, d]."""

  @staticmethod
  def forward(ctx, expert_out, flat_slot, gate, num_experts, capacity):
    st = pstate.get()
    mine = _exchange_back(expert_out.contiguous(), st.expert_size, st.expert_group, num_experts,
                          capacity)
    d = mine.shape[-1]
    mine = mine.reshape(num_experts * capacity, d)
    valid = flat_slot >= 0
    rows = mine[flat_slot.clamp(min=0)]                              # [T, k, d]
    w = (gate * valid.to(gate.dtype)).to(rows.dtype)
    ctx.save_for_backward(flat_slot, gate, rows)
    ctx.shape = (num_experts, capacity, d)
    return (rows * w[..., None]).sum(1)

  @staticmethod
  def backward(ctx, grad_out):
    flat_slot, gate, rows = ctx.saved_tensors
    e, c, d = ctx.shape
    st = pstate.get()
    valid = flat_slot >= 0
    vf = valid.to(grad_out.dtype)
    d_gate = ((rows.float() * grad_out.float()[:, None, :]).sum(-1) * valid.float()).to(gate.dtype)
    buf = grad_out.new_zeros(e * c, d)
    contrib = grad_out[:, None, :] * (gate.to(grad_out.dtype) * vf)[..., None]   # [T, k, d]
    buf[flat_slot[valid]] = contrib[valid]
    d_expert = _exchange(buf.view(e, c, d), st.expert_size, st.expert_group)
    return d_expert, None, d_gate, None, None


# ----------------------------------------------------------------------------
# The layer
# ----------------------------------------------------------------------------
class Experts(nn.Module):
  """E_local gated-GELU (or single-activation) MLPs with stacked kernels."""

  def __init__(self, num_experts: int, emb_dim: int, mlp_dim: int, activations: Sequence[str],
               dtype, device=None):
    super().__init__()
    st = pstate.get()
    if num_experts % st.expert_size:
      raise ValueError(f"{num_experts} experts are not divisible by expert={st.expert_size}")
    self.local = num_experts // st.expert_size
    self.activations = tuple(activations)
    self.dtype = t5_layers.canonical_dtype(dtype)
    init_in = t5_layers.variance_scaling(1.0, "fan_in", "truncated_normal", in_axis=-2, out_axis=-1)

    def mk(shape, axes):
      # Every expert-parallel rank draws the global [experts, ...] tensor with the same seed
      # and keeps its own slice, so the initial values do not depend on the mesh.
      def init_local(t, shape=shape):
        full = torch.empty((num_experts,) + tuple(shape[1:]), dtype=t.dtype, device=t.device)
        init_in(full)
        lo = st.expert_rank * self.local
        with torch.no_grad():
          t.copy_(full[lo:lo + self.local])

      p = t5_layers.param_with_axes(shape, init_local, axes, shard_dim=None, device=device)
      p.global_shape = (num_experts,) + tuple(shape[1:])
      p.expert_sharded = st.expert_size > 1
      p.expert_shard_dim = 0
      return p

    class _K(nn.Module):
      def __init__(self, p):
        super().__init__()
        self.kernel = p

    names = ["wi"] if len(self.activations) == 1 else [f"wi_{i}" for i in
                                                       range(len(self.activations))]
    for n in names:
      setattr(self, n, _K(mk((self.local, emb_dim, mlp_dim), ("expert", "embed", "expert_mlp"))))
    self.wo = _K(mk((self.local, mlp_dim, emb_dim), ("expert", "expert_mlp", "embed")))
    self._wi_names = names

  def forward(self, x: torch.Tensor) -> torch.Tensor:
    """x [E_local, N, d] -> [E_local, N, d]."""
    hs = []
    for n, act in zip(self._wi_names, self.activations):
      w = getattr(self, n).kernel
      hs.append(ref.ACTIVATIONS[act](F.batched_linear(x, w, self.dtype)))
    h = hs[0]
    for other in hs[1:]:
      h = h * other
    return F.batched_linear(h, self.wo.kernel, self.dtype)


class MoeLayer(nn.Module):
  """Drop-in replacement of `MlpBlock` (call signature included)."""

  def __init__(self, emb_dim: int, mlp_dim: int, num_experts: int,
               activations: Sequence[str] = ("gelu", "linear"), num_selected_experts: int = 1,
               capacity_factor: float = 1.25, eval_capacity_factor: Optional[float] = None,
               min_expert_capacity: int = 4, dropout_rate: float = 0.0, jitter_noise: float = 0.0,
               dtype=torch.float32, device=None, router_type: str = "tokens_choose"):
    super().__init__()
    self.num_experts = num_experts
    self.k = num_selected_experts
    self.router_type = router_type
    self.capacity_factor = capacity_factor
    self.eval_capacity_factor = eval_capacity_factor or capacity_factor
    self.min_expert_capacity = min_expert_capacity
    self.dropout_rate = dropout_rate
    self.dtype = t5_layers.canonical_dtype(dtype)
    if router_type == "tokens_choose":
      self.router = TokensChooseRouter(emb_dim, num_experts, num_selected_experts, jitter_noise,
                                       device=device)
    elif router_type == "experts_choose":
      self.router = ExpertsChooseRouter(emb_dim, num_experts, jitter_noise, device=device)
    else:
      raise ValueError(f"router_type must be 'tokens_choose' or 'experts_choose', got "
                       f"{router_type!r}")
    self.expert = Experts(num_experts, emb_dim, mlp_dim, activations, dtype, device=device)

  def forward(self, inputs: torch.Tensor, residual: Optional[torch.Tensor] = None,
              enable_dropout: bool = False) -> torch.Tensor:
    b, l, d = inputs.shape
    tokens = inputs.reshape(b * l, d).to(self.dtype)
    cf = self.capacity_factor if enable_dropout or torch.is_grad_enabled() \
        else self.eval_capacity_factor
    cap = expert_capacity(b * l, self.num_experts, cf, self.k, self.min_expert_capacity)
    route, metrics = self.router(tokens, cap, enable_dropout)
    _COLLECTED.append(metrics)
    flat_slot = route["flat_slot"]
    from t5x_b200.ops import moe as moe_ops
    if moe_ops.enabled(tokens):
      # NVLink path: rows are pushed into / pulled from the owners' buffers by the kernels
      x = moe_ops.FusedDispatch.apply(tokens, flat_slot, self.num_experts, cap)
      y = self.expert(x)
      out = moe_ops.FusedCombine.apply(y, flat_slot, route["gate"], self.num_experts, cap)
    else:
      flat_slot = flat_slot.long()
      x = _Dispatch.apply(tokens, flat_slot, self.num_experts, cap)
      y = self.expert(x)
      out = _Combine.apply(y, flat_slot, route["gate"].to(self.dtype), self.num_experts, cap)
    out = out.view(b, l, d).to(inputs.dtype)
    out = ref.dropout(out, self.dropout_rate, enable_dropout, broadcast_dims=(-2,)) \
        if self.dropout_rate > 0 else out
    return out if residual is None else out + residual
