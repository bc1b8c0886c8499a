"""Loss functions (API of t5x/losses.py): z-loss cross-entropy and loss normalisation."""
from __future__ import annotations

import enum
import math
from typing import Mapping, Optional, Tuple, Union

import numpy as np
import torch

from t5x_b200.ops import reference as ref


class _CrossEntropyWithLogits(torch.autograd.Function):
  """CE with z-loss and the reference's hand-written gradient (t5x/losses.py:62-124):
  d logits = g * ((1 + 2 z log_z) softmax - targets); the z-loss output carries no gradient."""

  @staticmethod
  def forward(ctx, logits, targets, z_loss):
    logits = logits.float()
    max_logit = logits.max(dim=-1, keepdim=True).values
    shifted = logits - max_logit
    exp_shifted = torch.exp(shifted)
    sum_exp = exp_shifted.sum(dim=-1, keepdim=True)
    log_softmax = shifted - torch.log(sum_exp)
    loss = -(targets * log_softmax).sum(dim=-1)
    log_z = (torch.log(sum_exp) + max_logit).squeeze(-1)
    total_z_loss = z_loss * log_z * log_z
    loss = loss + total_z_loss
    ctx.save_for_backward(targets, exp_shifted, sum_exp, log_z)
    ctx.z_loss = z_loss
    ctx.mark_non_differentiable(total_z_loss)
    return loss, total_z_loss

  @staticmethod
  def backward(ctx, g, _gz):
    targets, exp_shifted, sum_exp, log_z = ctx.saved_tensors
    deriv = (1 + 2 * ctx.z_loss * log_z)[..., None] * exp_shifted / sum_exp - targets
    g_logits = g[..., None] * deriv
    g_targets = -g[..., None] * (torch.log(exp_shifted / sum_exp))
    return g_logits, (g_targets if ctx.needs_input_grad[1] else None), None


def cross_entropy_with_logits(logits: torch.Tensor, targets: torch.Tensor,
                              z_loss: float) -> Tuple[torch.Tensor, torch.Tensor]:
  """logits, soft targets [..., classes] -> (loss incl. z-loss, z-loss), both [...]."""
  return _CrossEntropyWithLogits.apply(logits, targets, float(z_loss))


def compute_weighted_cross_entropy(
    logits: torch.Tensor, targets: torch.Tensor, weights: Optional[torch.Tensor] = None,
    label_smoothing: float = 0.0, z_loss: float = 0.0,
    loss_normalizing_factor: Optional[float] = None):
  """Sum (not mean) of weighted token losses; returns (loss, z_loss, weight_sum)
  (t5x/losses.py:132-193)."""
  if logits.dim() != targets.dim() + 1:
    raise ValueError(f"Incorrect shapes. Got shape {tuple(logits.shape)} logits and "
                     f"{tuple(targets.shape)} targets")
  vocab_size = logits.shape[-1]
  confidence = 1.0 - label_smoothing
  low_confidence = (1.0 - confidence) if vocab_size == 1 else (1.0 - confidence) / (vocab_size - 1)
  normalizing_constant = -(confidence * math.log(confidence) +
                           (vocab_size - 1) * low_confidence * math.log(low_confidence + 1e-20))
  soft_targets = torch.full(logits.shape, low_confidence, dtype=torch.float32,
                            device=logits.device)
  soft_targets.scatter_(-1, targets[..., None].long(), confidence)
  total_loss, total_z_loss = cross_entropy_with_logits(logits, soft_targets, z_loss)
  total_loss = total_loss - normalizing_constant
  return weight_and_normalize(total_loss, total_z_loss, targets, weights,
                              loss_normalizing_factor)


def weight_and_normalize(token_loss, token_z_loss, targets, weights, loss_normalizing_factor):
  """The weighting / normalising tail of `compute_weighted_cross_entropy`."""
  weight_sum = float(np.prod(targets.shape))
  if weights is not None:
    token_loss = token_loss * weights
    token_z_loss = token_z_loss * weights
    weight_sum = weights.sum()
  if loss_normalizing_factor is not None:
    token_loss = token_loss / loss_normalizing_factor
    token_z_loss = token_z_loss / loss_normalizing_factor
  return token_loss.sum(), token_z_loss.sum(), weight_sum


@enum.unique
class SpecialLossNormalizingFactor(enum.Enum):
  """Normalising factors computed from the batch (t5x/losses.py:196-217)."""
  NUM_REAL_TARGET_TOKENS = 1
  NUM_TOTAL_TARGET_TOKENS = 2
  AVERAGE_PER_SEQUENCE = 3


def convert_special_loss_normalizing_factor_to_enum(x: str) -> SpecialLossNormalizingFactor:
  try:
    return SpecialLossNormalizingFactor[x.upper()]
  except KeyError:
    raise ValueError(f'Could not convert string "{x}" to SpecialLossNormalizingFactor')


def _sum_weights_per_segment(positions, segment_ids, weights):
  """For packed rows: per-token total weight of the token's own segment
  (t5x/losses.py:246-275). Inputs [batch, length]."""
  out = torch.zeros_like(weights, dtype=torch.float32)
  b, l = weights.shape
  # segment ids are small positive ints (0 = padding); accumulate per (row, segment).
  seg = segment_ids.long()
  nseg = int(seg.max().item()) + 1 if seg.numel() else 1
  totals = torch.zeros((b, nseg), dtype=torch.float32, device=weights.device)
  totals.scatter_add_(1, seg, weights.float())
  out = totals.gather(1, seg)
  return torch.where(seg != 0, out, torch.zeros_like(out))


def get_loss_normalizing_factor_and_weights(
    loss_normalizing_factor: Optional[Union[float, int, str, SpecialLossNormalizingFactor]],
    batch: Mapping[str, torch.Tensor]):
  """Resolves a special factor into (float-like factor, per-token weights)
  (t5x/losses.py:278-356)."""
  loss_weights = batch.get("decoder_loss_weights", None)
  if loss_normalizing_factor is None or not isinstance(
      loss_normalizing_factor, (str, SpecialLossNormalizingFactor)):
    return loss_normalizing_factor, loss_weights
  if isinstance(loss_normalizing_factor, str):
    loss_normalizing_factor = convert_special_loss_normalizing_factor_to_enum(
        loss_normalizing_factor)
  if loss_weights is None:
    loss_weights = (batch["decoder_target_tokens"] > 0).float()
  if loss_normalizing_factor == SpecialLossNormalizingFactor.NUM_REAL_TARGET_TOKENS:
    output = loss_weights.sum()
  elif loss_normalizing_factor == SpecialLossNormalizingFactor.NUM_TOTAL_TARGET_TOKENS:
    output = float(np.prod(batch["decoder_target_tokens"].shape))
  elif loss_normalizing_factor == SpecialLossNormalizingFactor.AVERAGE_PER_SEQUENCE:
    if "decoder_segment_ids" in batch:
      norm_vec = _sum_weights_per_segment(batch["decoder_positions"],
                                          batch["decoder_segment_ids"], loss_weights)
    else:
      norm_vec = loss_weights.sum(dim=-1, keepdim=True)
    loss_weights = torch.nan_to_num(loss_weights / norm_vec, nan=0.0, posinf=0.0, neginf=0.0)
    output = loss_weights.sum()
  else:
    raise ValueError(f"Unsupported value of loss_normalizing_factor: {loss_normalizing_factor}")
  return _sum_over_data_replicas(output), loss_weights


def _sum_over_data_replicas(factor):
  """A factor derived from the batch counts the GLOBAL batch: the reference evaluates it
  inside the partitioned step over all replicas' examples (t5x/losses.py:278-356 under
  t5x/trainer.py:745-852), and gradients are summed over replicas afterwards. Each rank sees
  only its shard here, so the per-shard counts are added over the data (and expert) axis."""
  import torch.distributed as dist
  from t5x_b200.parallel import state as pstate
  st = pstate.get()
  if st.data_size * st.expert_size <= 1 or st.data_group is None or not dist.is_initialized():
    return factor
  t = torch.as_tensor(factor, dtype=torch.float32, device=st.device).detach().clone().reshape(1)
  dist.all_reduce(t, group=st.data_group)
  return t[0]
