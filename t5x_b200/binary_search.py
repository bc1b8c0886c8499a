"""Top-k / top-p masking (API of t5x/binary_search.py).

The reference finds the per-row cutoff with a 32-step bitwise binary search over the float
total order, because XLA lacks a cheap partial sort. On CUDA the cutoff comes from a four-pass
radix select inside one kernel (csrc/beam.cu); on the CPU from a sort / top-k. The bit-search
helpers are kept with the same contracts for callers that use them directly.
"""
from __future__ import annotations

from typing import Callable

import torch


def int32_bsearch(batch_shape, predicate: Callable[[torch.Tensor], torch.Tensor],
                  device=None) -> torch.Tensor:
  """Largest int32 per batch element for which `predicate` is False. The predicate must be
  monotone: False for every value up to a per-element threshold, True above it. Always True
  gives the smallest int32, always False the largest (t5x/binary_search.py:28-71)."""
  # Decide the sign first, then the remaining 31 bits from the top: a bit stays set while the
  # candidate that has it is still on the False side.
  zero = torch.zeros(batch_shape, dtype=torch.int64, device=device)
  negative = predicate(zero.to(torch.int32)).bool()
  current = torch.where(negative, torch.full_like(zero, -(2 ** 31)), zero)
  for bit in range(30, -1, -1):
    cand = current + (1 << bit)
    above = predicate(cand.to(torch.int32)).bool()
    current = torch.where(above, current, cand)
  return current.to(torch.int32)


def _monotonic_int32_to_float32(x: torch.Tensor) -> torch.Tensor:
  x = x.to(torch.int32)
  flipped = torch.where(x < 0, x ^ 0x7FFFFFFF, x)
  return flipped.view(torch.float32)


def _monotonic_float32_to_int32(x: torch.Tensor) -> torch.Tensor:
  i = x.to(torch.float32).contiguous().view(torch.int32)
  return torch.where(i < 0, i ^ 0x7FFFFFFF, i)


def float32_bsearch(batch_shape, predicate: Callable[[torch.Tensor], torch.Tensor],
                    device=None) -> torch.Tensor:
  """Largest float32, in the total order of bit patterns, per batch element for which the
  monotone `predicate` (False up to a threshold, True above it) is False
  (t5x/binary_search.py:121-164)."""
  res = int32_bsearch(batch_shape, lambda i: predicate(_monotonic_int32_to_float32(i)),
                      device=device)
  return _monotonic_int32_to_float32(res)


def topk_mask(x: torch.Tensor, k: int, replace_val) -> torch.Tensor:
  """Keeps the k largest entries of each row; the rest become `replace_val`. Entries equal
  to the k-th value are all kept (t5x/binary_search.py:167-227)."""
  k = min(int(k), x.shape[-1])
  if x.is_cuda and x.dtype == torch.float32 and k >= 1:
    from t5x_b200.ops import native
    return native.topk_topp_mask(x, k, None, float(replace_val))
  kth = torch.topk(x, k, dim=-1).values[..., -1:]
  return torch.where(x >= kth, x, torch.full_like(x, replace_val))


def topp_mask(logits: torch.Tensor, p, replace_val) -> torch.Tensor:
  """Nucleus mask: keeps the smallest set of top logits whose probability mass reaches `p`
  (entries tied with the cutoff are kept) (t5x/binary_search.py:230-299)."""
  if logits.is_cuda and logits.dtype == torch.float32:
    from t5x_b200.ops import native
    p_arg = p if not isinstance(p, torch.Tensor) else (
        p.reshape(-1).expand(logits.reshape(-1, logits.shape[-1]).shape[0]) if p.dim() > 0
        else float(p))
    return native.topk_topp_mask(logits, 0, p_arg, float(replace_val))
  probs = torch.softmax(logits.float(), dim=-1)
  sorted_probs, order = torch.sort(probs, dim=-1, descending=True)
  cum = torch.cumsum(sorted_probs, dim=-1)
  p_t = torch.as_tensor(p, dtype=torch.float32, device=logits.device)
  if p_t.dim() > 0:
    p_t = p_t.reshape(-1, *([1] * (logits.dim() - 1)))
  # index of the first position where the cumulative mass reaches p
  reached = (cum >= p_t).float()
  first = reached.argmax(dim=-1, keepdim=True)
  none_reached = reached.sum(dim=-1, keepdim=True) == 0
  first = torch.where(none_reached, torch.full_like(first, logits.shape[-1] - 1), first)
  cutoff_prob = torch.gather(sorted_probs, -1, first)
  return torch.where(probs >= cutoff_prob, logits, torch.full_like(logits, replace_val))
