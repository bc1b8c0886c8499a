"""Vocabulary-parallel logits + z-loss cross-entropy.

The logits projection is column-parallel over the `model` axis (`vocab -> model` in the
reference's rules, t5x/partitioning.py:564-573): each rank produces the logits of its vocab
slice, reduces them to per-token (max, sum-exp, target logit, sum, argmax) and only those few
floats per token cross the NVLink; the full [tokens, vocab] matrix never exists on one GPU.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from t5x_b200.ops import functional as F
from t5x_b200.ops import native
from t5x_b200.ops import reference as ref
from t5x_b200.parallel import state as pstate


def _local_logits(h2, w, scale):
  if h2.is_cuda and h2.dtype == torch.bfloat16:
    return native.gemm(h2, w, out_dtype=torch.float32, alpha=scale)
  return (h2.float() @ w.float()) * scale


def _local_stats(logits, targets, vocab_start):
  """-> stats [T,4] = (max, sumexp, target_logit, sum_logits), arg_val [T], arg_idx [T]."""
  if logits.is_cuda:
    return native.ce_stats(logits, targets, vocab_start)
  v = logits.shape[1]
  m = logits.max(dim=1).values
  s = torch.exp(logits - m[:, None]).sum(dim=1)
  t = targets - vocab_start
  own = (t >= 0) & (t < v)
  tl = torch.where(own, logits.gather(1, t.clamp(0, v - 1)[:, None]).squeeze(1),
                   torch.zeros_like(m))
  av, ai = logits.max(dim=1)
  return torch.stack([m, s, tl, logits.sum(dim=1)], dim=1), av, (ai + vocab_start).int()


def _local_grad(logits, targets, lse, row_scale, z_loss, conf, low, vocab_start, out_dtype):
  if logits.is_cuda:
    return native.ce_grad(logits, targets, lse, row_scale, z_loss, conf, low, vocab_start)
  v = logits.shape[1]
  p = torch.exp(logits - lse[:, None])
  t = targets - vocab_start
  soft = torch.full_like(logits, low)
  own = (t >= 0) & (t < v)
  rows = torch.nonzero(own).squeeze(1)
  soft[rows, t[rows]] = conf
  return (row_scale[:, None] * ((1 + 2 * z_loss * lse)[:, None] * p - soft)).to(out_dtype)


class _VocabParallelCE(torch.autograd.Function):

  @staticmethod
  def forward(ctx, hidden, weight, targets, z_loss, label_smoothing, logits_scale):
    st = pstate.get()
    k = hidden.shape[-1]
    h2 = hidden.reshape(-1, k)
    cdt = torch.bfloat16 if (hidden.is_cuda and hidden.dtype == torch.bfloat16) else torch.float32
    w = F.compute_weight(weight, cdt)
    v_local = w.shape[1]
    vocab = v_local * st.model_size
    vocab_start = st.model_rank * v_local
    logits = _local_logits(h2, w, logits_scale)
    t2 = targets.reshape(-1).long()
    stats, av, ai = _local_stats(logits, t2, vocab_start)
    packed = torch.cat([stats, av[:, None], ai[:, None].float()], dim=1).contiguous()
    parts = [torch.empty_like(packed) for _ in range(st.model_size)]
    dist.all_gather(parts, packed, group=st.model_group)
    allp = torch.stack(parts, dim=0)  # [tp, T, 6]
    m_all, s_all = allp[..., 0], allp[..., 1]
    M = m_all.max(dim=0).values
    S = (s_all * torch.exp(m_all - M[None])).sum(dim=0)
    lse = M + torch.log(S)
    tl = allp[..., 2].sum(dim=0)
    tot = allp[..., 3].sum(dim=0)
    best = allp[..., 4].argmax(dim=0)  # first rank holding the max => lowest vocab index on ties
    pred = allp[..., 5].gather(0, best[None]).squeeze(0).long()
    conf, low, norm_const = ref.label_smoothing_constants(vocab, label_smoothing)
    soft_dot = conf * tl + low * (tot - tl) if label_smoothing > 0 else tl
    z = z_loss * lse * lse
    loss = lse - soft_dot + z - norm_const
    correct = pred == t2
    ctx.save_for_backward(hidden, weight, t2, lse, logits)
    ctx.cfg = (z_loss, conf, low, logits_scale, vocab_start, cdt)
    ctx.mark_non_differentiable(correct)
    return loss.view(targets.shape), z.view(targets.shape), correct.view(targets.shape)

  @staticmethod
  def backward(ctx, dloss, dz, _dc):
    hidden, weight, t2, lse, logits = ctx.saved_tensors
    z_loss, conf, low, logits_scale, vocab_start, cdt = ctx.cfg
    st = pstate.get()
    k = hidden.shape[-1]
    h2 = hidden.reshape(-1, k)
    w = F.compute_weight(weight, cdt)
    row_scale = (dloss.reshape(-1).float() * logits_scale).contiguous()
    dlogits = _local_grad(logits, t2, lse, row_scale, z_loss, conf, low, vocab_start, cdt)
    dh = dw = None
    if ctx.needs_input_grad[0]:
      if dlogits.is_cuda and cdt == torch.bfloat16:
        dh = native.gemm(dlogits, w.t())
      else:
        dh = (dlogits.float() @ w.float().t()).to(hidden.dtype)
      dh = dh.contiguous()
      dist.all_reduce(dh, group=st.model_group)
      dh = dh.view(hidden.shape)
    if ctx.needs_input_grad[1]:
      if dlogits.is_cuda and cdt == torch.bfloat16:
        dw = F._accumulate_wgrad(weight, h2.t(), dlogits)
      else:
        dw = (h2.float().t() @ dlogits.float()).to(weight.dtype)
    return dh, dw, None, None, None, None


def logits_cross_entropy(hidden, weight, targets, *, z_loss: float = 0.0,
                         label_smoothing: float = 0.0, logits_scale: float = 1.0):
  """Per-token (loss, z_loss, correct) with `weight` [emb, vocab/model] sharded over the model
  axis. Same contract as `ops.functional.logits_cross_entropy`."""
  return _VocabParallelCE.apply(hidden, weight, targets, z_loss, label_smoothing, logits_scale)
