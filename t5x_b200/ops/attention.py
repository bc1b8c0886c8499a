"""Flash attention with in-kernel T5 relative-position bias (CUDA path of `functional.attention`)."""
from __future__ import annotations

import torch


def flash_supported(q, k, v, explicit_bias, extra_mask) -> bool:
  """True when the sm_100a flash kernels cover this call."""
  return False


def flash_attention(q, k, v, **kwargs):
  raise NotImplementedError
