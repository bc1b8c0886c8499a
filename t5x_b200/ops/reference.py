"""Plain PyTorch statements of every op: the numerical oracle and the CPU path.

Each function restates the math of the corresponding reference op in fp32 (citations
give the file in the reference project whose behaviour is matched). The CUDA kernels in
``csrc/`` are tested against these.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

NEG_MASK = -1e10  # additive mask value (t5x/examples/t5/layers.py:306-318)


def rmsnorm(x: torch.Tensor, scale: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
  """T5 "LayerNorm": no mean subtraction, no bias, fp32 statistics (layers.py:683-702)."""
  xf = x.float()
  ms = (xf * xf).mean(dim=-1, keepdim=True)
  return (xf * torch.rsqrt(ms + eps) * scale.float()).to(x.dtype)


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
  return F.gelu(x, approximate="tanh")


ACTIVATIONS = {
    "relu": F.relu,
    "gelu": gelu_tanh,  # flax.linen.gelu defaults to the tanh approximation
    "linear": lambda x: x,
    "silu": F.silu,
    "swish": F.silu,
    "tanh": torch.tanh,
    "sigmoid": torch.sigmoid,
}


def relative_position_bucket(relative_position: torch.Tensor, bidirectional: bool = True,
                             num_buckets: int = 32, max_distance: int = 128) -> torch.Tensor:
  """T5 relative-position bucket of `k_pos - q_pos` (layers.py:581-625)."""
  ret = torch.zeros_like(relative_position)
  n = -relative_position
  if bidirectional:
    num_buckets //= 2
    ret = ret + (n < 0).to(n.dtype) * num_buckets
    n = n.abs()
  else:
    n = n.clamp(min=0)
  max_exact = num_buckets // 2
  is_small = n < max_exact
  eps = torch.finfo(torch.float32).eps
  val_if_large = max_exact + (
      torch.log(n.to(torch.float32) / max_exact + eps) / math.log(max_distance / max_exact) *
      (num_buckets - max_exact)).to(n.dtype)
  val_if_large = val_if_large.clamp(max=num_buckets - 1)
  return ret + torch.where(is_small, n, val_if_large)


def relative_position_bias(table: torch.Tensor, qlen: int, klen: int, bidirectional: bool,
                           num_buckets: int = 32, max_distance: int = 128,
                           q_offset: int = 0) -> torch.Tensor:
  """[heads, qlen, klen] bias from a [heads, num_buckets] table (layers.py:627-677)."""
  dev = table.device
  ctx = torch.arange(q_offset, q_offset + qlen, device=dev)[:, None]
  mem = torch.arange(klen, device=dev)[None, :]
  buckets = relative_position_bucket(mem - ctx, bidirectional, num_buckets, max_distance)
  return table[:, buckets]  # [H, q, k]


class PrefixLMMask:
  """Visibility of a prefix LM in factored form: key k is visible to query q when
  (k <= q, or both lie inside the prefix) and both are real tokens of the same packed segment
  (the semantics of make_decoder_mask with decoder_causal_attention,
  t5x/examples/t5/layers.py:842-924). `bool()` gives the dense [B, 1, L, L] mask, so the object
  can stand wherever a dense `extra_mask` is accepted; the flash kernels use the per-token
  vectors and never build the dense form."""

  def __init__(self, in_prefix: torch.Tensor, valid: torch.Tensor,
               segment_ids: Optional[torch.Tensor] = None):
    self.in_prefix, self.valid, self.segment_ids = in_prefix.bool(), valid.bool(), segment_ids

  def bool(self) -> torch.Tensor:
    b, l = self.valid.shape
    pos = torch.arange(l, device=self.valid.device)
    vis = (pos[None, :] <= pos[:, None])[None].expand(b, l, l)
    vis = vis | (self.in_prefix[:, :, None] & self.in_prefix[:, None, :])
    vis = vis & self.valid[:, :, None] & self.valid[:, None, :]
    if self.segment_ids is not None:
      vis = vis & (self.segment_ids[:, :, None] == self.segment_ids[:, None, :])
    return vis[:, None]

  def token_codes(self):
    """(query codes, key codes) int32 [B, L] for the kernels: the segment id (1 when unpacked)
    in the low 30 bits, bit 30 set inside the prefix; padding queries carry a segment id that no
    key has, so their rows see nothing."""
    seg = self.segment_ids.to(torch.int32) if self.segment_ids is not None else \
        torch.ones_like(self.valid, dtype=torch.int32)
    pre = self.in_prefix.to(torch.int32) << 30
    k_codes = seg | pre
    q_codes = torch.where(self.valid, seg, torch.full_like(seg, 0x3FFFFFFE)) | pre
    return q_codes.contiguous(), k_codes.contiguous()


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *,
              bias: Optional[torch.Tensor] = None, key_mask: Optional[torch.Tensor] = None,
              causal: bool = False, q_segment_ids: Optional[torch.Tensor] = None,
              kv_segment_ids: Optional[torch.Tensor] = None,
              extra_mask: Optional[torch.Tensor] = None,
              float32_logits: bool = True) -> torch.Tensor:
  """softmax(q k^T + bias + mask) v with no 1/sqrt(d) (T5 folds it into the init).

  q [B, Lq, H, D]; k, v [B, Lk, H, D]; bias [H or 1, Lq, Lk] (relative positions);
  key_mask [B, Lk] bool (True = attend). Masked logits get -1e10, so a fully masked
  row yields a uniform distribution, never NaN (layers.py:52-129).
  `extra_mask` [B, 1 or H, Lq, Lk] bool is and-ed in (prefix-LM blocks).
  """
  dt = torch.float32 if float32_logits else q.dtype
  logits = torch.einsum("bqhd,bkhd->bhqk", q.to(dt), k.to(dt))
  if bias is not None:
    logits = logits + bias.to(dt)[None]
  B, H, Lq, Lk = logits.shape
  mask = None

  def _and(m, new):
    return new if m is None else (m & new)

  if key_mask is not None:
    mask = _and(mask, key_mask[:, None, None, :].bool())
  if causal:
    qi = torch.arange(Lq, device=q.device)[:, None] + (Lk - Lq)
    ki = torch.arange(Lk, device=q.device)[None, :]
    mask = _and(mask, (ki <= qi)[None, None])
  if q_segment_ids is not None and kv_segment_ids is not None:
    mask = _and(mask, (q_segment_ids[:, None, :, None] == kv_segment_ids[:, None, None, :]))
  if extra_mask is not None:
    mask = _and(mask, extra_mask.bool())
  if mask is not None:
    # Additive, as in the reference (mask -> bias of 0 / -1e10 that is summed with the logits):
    # a masked logit equals -1e10 in fp32 and the softmax gradient still reaches q and k.
    logits = logits + torch.where(mask, 0.0, NEG_MASK).to(logits.dtype)
  probs = torch.softmax(logits.float(), dim=-1).to(v.dtype)
  return torch.einsum("bhqk,bkhd->bqhd", probs, v)


def cross_entropy_with_logits(logits: torch.Tensor, targets: torch.Tensor, z_loss: float):
  """Per-position (loss incl. z-loss, z-loss term) for soft `targets` (t5x/losses.py:62-95)."""
  logits = logits.float()
  lse = torch.logsumexp(logits, dim=-1)
  log_softmax = logits - lse[..., None]
  loss = -(targets * log_softmax).sum(-1)
  total_z = z_loss * lse * lse
  return loss + total_z, total_z


def label_smoothing_constants(vocab: int, label_smoothing: float):
  confidence = 1.0 - label_smoothing
  low_confidence = (1.0 - confidence) / (vocab - 1)
  normalizing_constant = -(confidence * math.log(confidence) +
                           (vocab - 1) * low_confidence * math.log(low_confidence + 1e-20))
  return confidence, low_confidence, normalizing_constant


def token_cross_entropy(logits: torch.Tensor, targets: torch.Tensor, z_loss: float = 0.0,
                        label_smoothing: float = 0.0):
  """Per-token (ce+z - normalizing const, z term, lse, argmax) for integer targets
  (t5x/losses.py:132-193 without the weighting/normalisation step)."""
  vocab = logits.shape[-1]
  confidence, low_confidence, norm_const = label_smoothing_constants(vocab, label_smoothing)
  lf = logits.float()
  lse = torch.logsumexp(lf, dim=-1)
  tl = lf.gather(-1, targets[..., None]).squeeze(-1)
  if label_smoothing > 0:
    soft_dot = confidence * tl + low_confidence * (lf.sum(-1) - tl)
  else:
    soft_dot = tl
  z = z_loss * lse * lse
  loss = lse - soft_dot + z - norm_const
  return loss, z, lse, lf.argmax(-1)


_DROPOUT_GENERATORS: dict = {}


def set_dropout_seed(seed: Optional[int]) -> None:
  """Seeds the generators used by `dropout` (one per device); None returns to global RNG.
  Also restarts the numbering of dropout sites used by the in-kernel masks."""
  _DROPOUT_GENERATORS.clear()
  _DROPOUT_SITE[0] = 0
  if seed is not None:
    _DROPOUT_GENERATORS["seed"] = int(seed)


_DROPOUT_SITE = [0]


def dropout_seed() -> Optional[int]:
  """The seed set by `set_dropout_seed`, or None."""
  return _DROPOUT_GENERATORS.get("seed")


def next_dropout_site() -> int:
  """A number that is different for every dropout call since the last `set_dropout_seed`:
  together with the seed it names the mask of that call (the in-kernel generator is keyed by
  (seed, site, element))."""
  _DROPOUT_SITE[0] += 1
  return _DROPOUT_SITE[0]


def dropout_site_state() -> int:
  return _DROPOUT_SITE[0]


def set_dropout_site_state(n: int) -> None:
  """Restores the site counter (recomputation of a checkpointed block must draw the masks of
  its first pass)."""
  _DROPOUT_SITE[0] = int(n)


def _dropout_generator(device) -> Optional[torch.Generator]:
  if "seed" not in _DROPOUT_GENERATORS:
    return None
  key = str(device)
  if key not in _DROPOUT_GENERATORS:
    g = torch.Generator(device=device)
    g.manual_seed(_DROPOUT_GENERATORS["seed"])
    _DROPOUT_GENERATORS[key] = g
  return _DROPOUT_GENERATORS[key]


def dropout(x: torch.Tensor, rate: float, training: bool, broadcast_dims=(),
            generator: Optional[torch.Generator] = None) -> torch.Tensor:
  """Dropout whose mask is shared along `broadcast_dims` (flax nn.Dropout semantics)."""
  if not training or rate == 0.0:
    return x
  if generator is None and dropout_seed() is not None:
    # one generator per call, keyed by (step seed, call number): a block that is recomputed in
    # the backward pass (rematerialisation) restores the call counter and so draws the masks
    # of its first pass again, as the in-kernel generator on the GPU does
    generator = torch.Generator(device=x.device)
    generator.manual_seed((dropout_seed() * 1000003 + next_dropout_site()) % (2 ** 63 - 1))
  shape = list(x.shape)
  for d in broadcast_dims:
    shape[d] = 1
  keep = 1.0 - rate
  mask = torch.rand(shape, device=x.device, generator=generator) < keep
  return torch.where(mask, x / keep, torch.zeros_like(x))
