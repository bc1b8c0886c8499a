"""Flash attention with in-kernel T5 relative-position bias (CUDA path of `functional.attention`).

The [heads, buckets] bias table is expanded on the host into a per-relative-offset table
`rel_bias[h, (k - q) + Lq - 1]` with the oracle's own bucket function (so bucket boundaries are
bit-identical); the kernels index it by `k - q`, build the masks from per-token metadata and
never materialise [b, h, q, k] scores. The gradient of the expanded table comes back from the
backward kernel and autograd folds it into the bucket table.
"""
from __future__ import annotations

from typing import Optional

import torch

from t5x_b200.ops import native
from t5x_b200.ops import reference as ref

c_void_p, c_int, c_ll = native.c_void_p, native.c_int, native.c_ll
native.register_signature("t5x_attention_fwd", [c_void_p] * 5 + [c_int] * 4 + [c_ll] * 12 +
                          [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                           c_void_p])
native.register_signature("t5x_attention_bwd", [c_void_p] * 10 + [c_int] * 5 + [c_ll] * 18 +
                          [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                           c_int, c_void_p])

native.register_signature("t5x_attention_fwd_stream", [c_void_p] * 5 + [c_int] * 5 + [c_ll] * 12 +
                          [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                           c_void_p])

# The short-range forward kernel keeps the scores of a whole key range in TMEM.
CLASSIC_MAX_LK = 512
CLASSIC_MAX_LQ = 512
# The backward kernel keeps bias-gradient bins for the whole query range in shared memory.
BWD_MAX_LQ = 4096


def forward_kernel(Lq: int, Lk: int, D: int, prefix_lm: bool = False) -> str:
  """'classic' (head_dim 64, up to 512 x 512 keys, scores of the whole key range in TMEM: the
  faster of the two on the shapes it covers) or 'stream' (any length, head_dim 64 or 128,
  prefix-LM masks). `T5X_B200_ATTN_FWD=stream` forces the streaming kernel everywhere."""
  import os
  classic_ok = D == 64 and Lq <= CLASSIC_MAX_LQ and Lk <= CLASSIC_MAX_LK and not prefix_lm
  want = os.environ.get("T5X_B200_ATTN_FWD", "classic")
  return "classic" if (classic_ok and want == "classic") else "stream"


def _strides_ok(t: torch.Tensor) -> bool:
  return (t.dim() == 4 and t.stride(3) == 1 and t.stride(0) % 8 == 0 and t.stride(1) % 8 == 0 and
          t.stride(2) % 8 == 0 and t.data_ptr() % 16 == 0)


def flash_supported(q, k, v, explicit_bias, extra_mask) -> bool:
  """True when the sm_100a flash kernels cover this call."""
  prefix_lm = isinstance(extra_mask, ref.PrefixLMMask)
  if prefix_lm and q.shape[1] != k.shape[1]:
    return False
  return (explicit_bias is None and (extra_mask is None or prefix_lm) and
          q.shape[-1] in (64, 128) and q.shape[1] <= BWD_MAX_LQ and q.dtype == torch.bfloat16 and
          k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16)


def _sbh(t):
  return t.stride(0), t.stride(1), t.stride(2)


def _packed_qkv(q, k, v) -> bool:
  """True when q, k, v [B, L, H, D] are the three column blocks of one [B * L, 3 * H * D]
  projection output (a fused q/k/v GEMM): their gradients are then written as the column
  blocks of one buffer too, so that the projection's backward is a single GEMM over it."""
  if q.shape != k.shape or q.shape != v.shape:
    return False
  b, l, h, d = q.shape
  row = 3 * h * d
  want = (l * row, row, d, 1)
  step = h * d * q.element_size()
  return (q.stride() == want and k.stride() == want and v.stride() == want and
          k.data_ptr() == q.data_ptr() + step and v.data_ptr() == q.data_ptr() + 2 * step)


class _FlashAttentionFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, q, k, v, rel_bias, key_mask, q_seg, kv_seg, causal, causal_off, rel_off):
    q = q if _strides_ok(q) else q.contiguous()
    k = k if _strides_ok(k) else k.contiguous()
    v = v if _strides_ok(v) else v.contiguous()
    B, Lq, H, D = q.shape
    Lk = k.shape[1]
    o = torch.empty((B, Lq, H, D), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((B, H, Lq), dtype=torch.float32, device=q.device)
    nrel = rel_bias.shape[1] if rel_bias is not None else 0
    tail = (*_sbh(q), *_sbh(k), *_sbh(v), *_sbh(o), native.ptr(rel_bias), nrel, rel_off,
            native.ptr(key_mask), native.ptr(q_seg), native.ptr(kv_seg), int(causal), causal_off,
            native.stream_ptr())
    if forward_kernel(Lq, Lk, D, int(causal) == 2) == "classic":
      rc = native.lib().t5x_attention_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                          lse.data_ptr(), B, H, Lq, Lk, *tail)
    else:
      rc = native.lib().t5x_attention_fwd_stream(q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                                 o.data_ptr(), lse.data_ptr(), B, H, Lq, Lk, D,
                                                 *tail)
    native._check(rc, "attention_fwd")
    ctx.save_for_backward(q, k, v, o, lse, rel_bias, key_mask, q_seg, kv_seg)
    ctx.cfg = (causal, causal_off, rel_off)
    return o

  @staticmethod
  def backward(ctx, do):
    q, k, v, o, lse, rel_bias, key_mask, q_seg, kv_seg = ctx.saved_tensors
    causal, causal_off, rel_off = ctx.cfg
    B, Lq, H, D = q.shape
    Lk = k.shape[1]
    do = do if _strides_ok(do) else do.contiguous()
    dq32 = torch.zeros((B, Lq, H, D), dtype=torch.float32, device=q.device)
    packed = _packed_qkv(q, k, v)
    if packed:
      dqkv = torch.empty((B, Lq, 3, H, D), dtype=torch.bfloat16, device=q.device)
      dq, dk, dv = dqkv[:, :, 0], dqkv[:, :, 1], dqkv[:, :, 2]
    else:
      dk = torch.empty((B, Lk, H, D), dtype=torch.bfloat16, device=q.device)
      dv = torch.empty((B, Lk, H, D), dtype=torch.bfloat16, device=q.device)
    delta = torch.empty((B, H, Lq), dtype=torch.float32, device=q.device)
    d_rel = torch.zeros_like(rel_bias) if rel_bias is not None else None
    nrel = rel_bias.shape[1] if rel_bias is not None else 0
    rc = native.lib().t5x_attention_bwd(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
        delta.data_ptr(), dq32.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, H, Lq, Lk, D,
        *_sbh(q),
        *_sbh(k), *_sbh(v), *_sbh(o), *_sbh(do), *_sbh(dk), native.ptr(rel_bias),
        native.ptr(d_rel), nrel, rel_off, native.ptr(key_mask), native.ptr(q_seg),
        native.ptr(kv_seg), int(causal), causal_off, native.stream_ptr())
    native._check(rc, "attention_bwd")
    if packed:
      dq.copy_(dq32)
    else:
      dq = dq32.to(torch.bfloat16)
    return dq, dk, dv, d_rel, None, None, None, None, None, None


_BUCKET_CACHE: dict = {}


def _rel_buckets(Lq, Lk, q_offset, bidirectional, num_buckets, max_distance, device):
  """Bucket index for every relative offset of an [Lq, Lk] attention: entry t stands for
  (k - q_pos) = t - (Lq - 1) - q_offset. Cached: it depends on the shapes only."""
  key = (Lq, Lk, q_offset, bool(bidirectional), num_buckets, max_distance, str(device))
  b = _BUCKET_CACHE.get(key)
  if b is None:
    rel = torch.arange(Lq + Lk - 1, device=device) - (Lq - 1) - q_offset
    b = ref.relative_position_bucket(rel, bidirectional, num_buckets, max_distance)
    if len(_BUCKET_CACHE) > 256:
      _BUCKET_CACHE.clear()
    _BUCKET_CACHE[key] = b
  return b


def flash_attention(q, k, v, *, bias_table: Optional[torch.Tensor] = None,
                    bidirectional: bool = True, num_buckets: int = 32, max_distance: int = 128,
                    key_mask: Optional[torch.Tensor] = None, causal: bool = False,
                    q_segment_ids=None, kv_segment_ids=None, q_offset: int = 0,
                    prefix_lm: Optional["ref.PrefixLMMask"] = None) -> torch.Tensor:
  """q [B,Lq,H,D], k/v [B,Lk,H,D] bf16 -> [B,Lq,H,D], D = 64 or 128. `prefix_lm`: prefix-LM visibility in factored form; it replaces `causal`,
  `key_mask` and the segment ids (which it contains)."""
  B, Lq, H, D = q.shape
  Lk = k.shape[1]
  rel_bias = None
  if bias_table is not None:
    rel_bias = bias_table.float()[:, _rel_buckets(Lq, Lk, q_offset, bidirectional, num_buckets,
                                                  max_distance, q.device)].contiguous()
  km = key_mask.to(torch.uint8).contiguous() if key_mask is not None else None
  qs = q_segment_ids.to(torch.int32).contiguous() if q_segment_ids is not None else None
  ks = kv_segment_ids.to(torch.int32).contiguous() if kv_segment_ids is not None else None
  if qs is None or ks is None:
    qs = ks = None
  mode = int(bool(causal))
  if prefix_lm is not None:
    qs, ks = prefix_lm.token_codes()
    valid = prefix_lm.valid.to(torch.uint8)
    km = valid.contiguous() if km is None else (km & valid).contiguous()
    mode = 2
  return _FlashAttentionFn.apply(q, k, v, rel_bias, km, qs, ks, mode,
                                 (Lk - Lq) if mode else 0, Lq - 1)
