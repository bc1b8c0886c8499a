"""Differentiable ops of the T5 block.

On CUDA with bf16 activations every function here runs the hand-written sm_100a
kernels (tcgen05 GEMMs with fused epilogues, fused RMSNorm, flash attention with
in-kernel relative-position bias, fused z-loss cross-entropy); anything else (CPU,
fp32 numerics tests) runs the PyTorch statements in :mod:`t5x_b200.ops.reference`.

Weights are fp32 master parameters. A parameter may carry two attributes managed by
the train state:
  * ``bf16``       a bf16 working copy refreshed by the optimizer kernel,
  * ``main_grad``  an fp32 accumulator; weight gradients are accumulated there directly
                   by the wgrad GEMM epilogue (``C +=``) instead of being returned.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from t5x_b200.ops import native
from t5x_b200.ops import reference as ref


def _native_ok(x: torch.Tensor) -> bool:
  return x.is_cuda and x.dtype == torch.bfloat16


def compute_weight(p: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
  """The copy of parameter `p` in the compute dtype (cached bf16 copy when attached)."""
  if dtype == torch.bfloat16:
    w = getattr(p, "bf16", None)
    if w is not None:
      return w
  return p if p.dtype == dtype else p.to(dtype)


def _accumulate_wgrad(weight: torch.Tensor, a_t: torch.Tensor, b: torch.Tensor):
  """dW = a_t @ b. With a main_grad buffer: accumulate in place and return None."""
  mg = getattr(weight, "main_grad", None)
  if mg is not None:
    first = not getattr(weight, "grad_ready", False)
    out = mg.view(a_t.shape[0], b.shape[1])
    splits = native.wgrad_splits(a_t.shape[0], b.shape[1], a_t.shape[1])
    if splits > 1 and out.is_contiguous():
      native.gemm_splitk_accumulate(a_t, b, out, splits, accumulate=not first)
    else:
      native.gemm(a_t, b, out=out, accumulate=not first)
    weight.grad_ready = True
    return None
  return native.gemm(a_t, b, out_dtype=torch.float32).view(weight.shape).to(weight.dtype)


class _LinearFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x, weight, residual):
    k = x.shape[-1]
    w2 = compute_weight(weight, torch.bfloat16).reshape(k, -1)
    x2 = x.reshape(-1, k)
    r2 = residual.reshape(-1, w2.shape[1]) if residual is not None else None
    y = native.gemm(x2, w2, residual=r2)
    ctx.save_for_backward(x, weight)
    ctx.has_res = residual is not None
    return y.view(*x.shape[:-1], w2.shape[1])

  @staticmethod
  def backward(ctx, dy):
    x, weight = ctx.saved_tensors
    k = x.shape[-1]
    w2 = compute_weight(weight, torch.bfloat16).reshape(k, -1)
    dy2 = dy.reshape(-1, w2.shape[1])
    if not dy2.is_contiguous():
      dy2 = dy2.contiguous()
    x2 = x.reshape(-1, k)
    dx = None
    if ctx.needs_input_grad[0]:
      dx = native.gemm(dy2, w2.t()).view(x.shape)
    dw = None
    if ctx.needs_input_grad[1]:
      dw = _accumulate_wgrad(weight, x2.t(), dy2)
    return dx, dw, (dy if ctx.has_res else None)


class _MultiLinearFn(torch.autograd.Function):
  """(x @ W_0, x @ W_1, ...) for projections that share their input (q/k/v, cross k/v). In
  backward the input gradient is built by accumulating GEMMs (dx = dy_0 W_0^T, then
  dx += dy_i W_i^T in the epilogue), not by separate GEMMs whose results autograd would add
  with elementwise kernels over the activations."""

  @staticmethod
  def forward(ctx, x, *weights):
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    outs = []
    for w in weights:
      w2 = compute_weight(w, torch.bfloat16).reshape(k, -1)
      outs.append(native.gemm(x2, w2).view(*x.shape[:-1], w2.shape[1]))
    ctx.save_for_backward(x, *weights)
    return tuple(outs)

  @staticmethod
  def backward(ctx, *dys):
    x, *weights = ctx.saved_tensors
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    dx = None
    dws = []
    for i, (w, dy) in enumerate(zip(weights, dys)):
      if dy is None:
        dws.append(None)
        continue
      w2 = compute_weight(w, torch.bfloat16).reshape(k, -1)
      dy2 = dy.reshape(-1, w2.shape[1])
      if not dy2.is_contiguous():
        dy2 = dy2.contiguous()
      if ctx.needs_input_grad[0]:
        if dx is None:
          dx = native.gemm(dy2, w2.t())
        else:
          native.gemm(dy2, w2.t(), out=dx, accumulate=True)
      dws.append(_accumulate_wgrad(w, x2.t(), dy2) if ctx.needs_input_grad[1 + i] else None)
    return (None if dx is None else dx.view(x.shape),) + tuple(dws)


def multi_linear(x: torch.Tensor, weights: Sequence[torch.Tensor],
                 dtype: Optional[torch.dtype] = None):
  """[x @ W for W in weights] with one fused backward for the shared input."""
  if _native_ok(x):
    return list(_MultiLinearFn.apply(x, *weights))
  return [linear(x, w, dtype=dtype) for w in weights]


def linear(x: torch.Tensor, weight: torch.Tensor, residual: Optional[torch.Tensor] = None,
           dtype: Optional[torch.dtype] = None) -> torch.Tensor:
  """y = x @ W (+ residual). W is [in, out...] (T5X kernel layout); trailing kernel dims are
  flattened for the contraction and kept flat in the output."""
  if _native_ok(x):
    return _LinearFn.apply(x, weight, residual)
  dt = dtype or x.dtype
  w = compute_weight(weight, dt).reshape(x.shape[-1], -1)
  y = x.to(dt) @ w
  return y if residual is None else y + residual


class _BatchedLinearFn(torch.autograd.Function):
  """y[e] = x[e] @ w[e] for stacked expert kernels (one batched GEMM each way)."""

  @staticmethod
  def forward(ctx, x, weight):
    w = compute_weight(weight, torch.bfloat16)
    ctx.save_for_backward(x, weight)
    return native.gemm(x.contiguous(), w)

  @staticmethod
  def backward(ctx, dy):
    x, weight = ctx.saved_tensors
    w = compute_weight(weight, torch.bfloat16)
    dy = dy.contiguous()
    dx = dw = None
    if ctx.needs_input_grad[0]:
      dx = native.gemm(dy, w.transpose(1, 2))
    if ctx.needs_input_grad[1]:
      mg = getattr(weight, "main_grad", None)
      xt = x.contiguous().transpose(1, 2)
      if mg is not None:
        first = not getattr(weight, "grad_ready", False)
        native.gemm(xt, dy, out=mg, accumulate=not first)
        weight.grad_ready = True
      else:
        dw = native.gemm(xt, dy, out_dtype=torch.float32).to(weight.dtype)
    return dx, dw


def batched_linear(x: torch.Tensor, weight: torch.Tensor,
                   dtype: Optional[torch.dtype] = None) -> torch.Tensor:
  """x [E, N, in] @ weight [E, in, out] -> [E, N, out]."""
  if _native_ok(x):
    return _BatchedLinearFn.apply(x, weight)
  dt = dtype or x.dtype
  return torch.bmm(x.to(dt), compute_weight(weight, dt))


class _RmsNormFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x, scale, eps, out=None):
    xc = x.contiguous()
    y, rstd = native.rmsnorm_fwd(xc, scale.float(), eps, out=out)
    ctx.save_for_backward(xc, scale, rstd)
    return y

  @staticmethod
  def backward(ctx, dy):
    x, scale, rstd = ctx.saved_tensors
    mg = getattr(scale, "main_grad", None)
    if mg is not None:
      if not getattr(scale, "grad_ready", False):
        mg.zero_()
        scale.grad_ready = True
      dscale_buf, ret = mg, None
    else:
      dscale_buf = torch.zeros_like(scale, dtype=torch.float32)
      ret = dscale_buf
    dx = native.rmsnorm_bwd(dy.contiguous(), x, scale.float(), rstd, None, dscale_buf)
    return dx, ret, None, None


class _ResidualRmsNormFn(torch.autograd.Function):
  """x -> (x, rmsnorm(x)): the first output is the residual branch. Its gradient is added to
  the norm's input gradient inside the backward kernel instead of by a separate elementwise
  add over the activations."""

  @staticmethod
  def forward(ctx, x, scale, eps, out=None):
    xc = x.contiguous()
    y, rstd = native.rmsnorm_fwd(xc, scale.float(), eps, out=out)
    ctx.save_for_backward(xc, scale, rstd)
    return x.view_as(x), y

  @staticmethod
  def backward(ctx, dres, dy):
    x, scale, rstd = ctx.saved_tensors
    if dy is None:
      return dres, None, None, None
    mg = getattr(scale, "main_grad", None)
    if mg is not None:
      if not getattr(scale, "grad_ready", False):
        mg.zero_()
        scale.grad_ready = True
      dscale_buf, ret = mg, None
    else:
      dscale_buf = torch.zeros_like(scale, dtype=torch.float32)
      ret = dscale_buf
    if dres is not None:
      dres = dres.to(torch.bfloat16).contiguous()
    dx = native.rmsnorm_bwd(dy.contiguous(), x, scale.float(), rstd, dres, dscale_buf)
    return dx, ret, None, None


def residual_rmsnorm(x: torch.Tensor, scale: torch.Tensor, eps: float = 1e-6,
                     out: Optional[torch.Tensor] = None):
  """(x, rmsnorm(x)); use the first element as the residual input of the block the norm
  feeds, so that the two gradient paths into x meet inside the norm's backward kernel."""
  if _native_ok(x):
    return _ResidualRmsNormFn.apply(x, scale, eps, out)
  return x, ref.rmsnorm(x, scale, eps)


def rmsnorm(x: torch.Tensor, scale: torch.Tensor, eps: float = 1e-6,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
  """`out` (CUDA path only): a bf16 buffer of x's shape that receives the result."""
  if _native_ok(x):
    return _RmsNormFn.apply(x, scale, eps, out)
  return ref.rmsnorm(x, scale, eps)


class _GatedGeluMlpInFn(torch.autograd.Function):
  """g = gelu(x @ wi_0) * (x @ wi_1) with the activation fused in the GEMM epilogue."""

  @staticmethod
  def forward(ctx, x, wi_0, wi_1):
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    w0 = compute_weight(wi_0, torch.bfloat16)
    w1 = compute_weight(wi_1, torch.bfloat16)
    dff = w0.shape[1]
    h = torch.empty((x2.shape[0], 2 * dff), dtype=torch.bfloat16, device=x.device)
    g = native.gemm(x2, w0, b2=w1, save_h=h)
    ctx.save_for_backward(x, wi_0, wi_1, h)
    return g.view(*x.shape[:-1], dff)

  @staticmethod
  def backward(ctx, dg):
    x, wi_0, wi_1, h = ctx.saved_tensors
    k = x.shape[-1]
    dff = h.shape[1] // 2
    x2 = x.reshape(-1, k)
    # The saved pre-activations are overwritten with their gradients (one backward per forward).
    dh = h
    native.gated_gelu_bwd_(dg.reshape(-1, dff).contiguous(), dh)  # dh <- [dh0|dh1]
    w0 = compute_weight(wi_0, torch.bfloat16)
    w1 = compute_weight(wi_1, torch.bfloat16)
    dh0, dh1 = dh[:, :dff], dh[:, dff:]
    dx = None
    if ctx.needs_input_grad[0]:
      dx = native.gemm(dh0, w0.t())
      native.gemm(dh1, w1.t(), out=dx, accumulate=True)
      dx = dx.view(x.shape)
    d0 = _accumulate_wgrad(wi_0, x2.t(), dh0) if ctx.needs_input_grad[1] else None
    d1 = _accumulate_wgrad(wi_1, x2.t(), dh1) if ctx.needs_input_grad[2] else None
    return dx, d0, d1


def gated_gelu_mlp_in(x, wi_0, wi_1, dtype: Optional[torch.dtype] = None):
  if _native_ok(x):
    return _GatedGeluMlpInFn.apply(x, wi_0, wi_1)
  dt = dtype or x.dtype
  return ref.gelu_tanh(x.to(dt) @ compute_weight(wi_0, dt)) * (x.to(dt) @ compute_weight(wi_1, dt))


class _EmbeddingFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, ids, table):
    ctx.save_for_backward(ids, table)
    return native.embedding_fwd(ids, compute_weight(table, torch.bfloat16))

  @staticmethod
  def backward(ctx, dout):
    ids, table = ctx.saved_tensors
    mg = getattr(table, "main_grad", None)
    if mg is not None:
      if not getattr(table, "grad_ready", False):
        mg.zero_()
        table.grad_ready = True
      native.embedding_bwd_(ids, dout.contiguous(), mg)
      return None, None
    dt = torch.zeros(table.shape, dtype=torch.float32, device=table.device)
    native.embedding_bwd_(ids, dout.contiguous(), dt)
    return None, dt.to(table.dtype)


def embedding(ids: torch.Tensor, table: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
  if table.is_cuda and dtype == torch.bfloat16:
    return _EmbeddingFn.apply(ids, table)
  return compute_weight(table, dtype)[ids]


# ----------------------------------------------------------------------------
# Dropout
# ----------------------------------------------------------------------------
class _DropoutFn(torch.autograd.Function):
  """x * mask / keep with the mask drawn inside the kernel from (seed, site, key); backward
  runs the same kernel on the gradient."""

  @staticmethod
  def forward(ctx, x, rate, seed, site, group_rows, col_group, row_offset):
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
      x2 = x2.contiguous()
    ctx.cfg = (rate, seed, site, group_rows, col_group, row_offset)
    y = native.dropout_rows(x2, rate, seed, site, group_rows=group_rows, col_group=col_group,
                            row_offset=row_offset)
    return y.view(x.shape)

  @staticmethod
  def backward(ctx, dy):
    rate, seed, site, group_rows, col_group, row_offset = ctx.cfg
    d2 = dy.reshape(-1, dy.shape[-1])
    if d2.stride(-1) != 1:
      d2 = d2.contiguous()
    dx = native.dropout_rows(d2, rate, seed, site, group_rows=group_rows, col_group=col_group,
                             row_offset=row_offset)
    return dx.view(dy.shape), None, None, None, None, None, None


def _dropout_seed_and_site(sharded: bool):
  seed = ref.dropout_seed()
  if seed is None:  # no step seed: one from the host generator (no device synchronisation)
    seed = int(torch.empty((), dtype=torch.int64).random_().item())
  site = ref.next_dropout_site()
  if sharded:
    # activations whose columns are split over the model axis: every rank draws its own mask
    from t5x_b200.parallel import state as pstate
    site = (site & 0xFFFFFF) | ((pstate.get().model_rank & 0xFF) << 24)
  return seed, site


def dropout(x: torch.Tensor, rate: float, training: bool, broadcast_dims=(), *,
            seq_len: Optional[int] = None, row_offset: int = 0,
            sharded: bool = False) -> torch.Tensor:
  """Dropout whose mask is shared along `broadcast_dims` (`()` or `(-2,)`, the length axis of
  [batch, length, features]; t5x/examples/t5/network.py:76-78). On CUDA with bf16 the mask is
  drawn inside the kernel. For a 2-D block of rows of a row-sharded [batch * length, features]
  activation pass `seq_len` (the length) and `row_offset` (global index of the block's first
  row): the block then gets the mask the whole tensor would get. `sharded`: the feature axis is
  split over the model axis, so ranks draw independent masks."""
  if not training or rate == 0.0:
    return x
  bd = tuple(broadcast_dims)
  if _native_ok(x) and bd in ((), (-2,)):
    seed, site = _dropout_seed_and_site(sharded)
    if bd == (-2,):
      group_rows = int(seq_len if seq_len is not None else x.shape[-2])
    else:
      group_rows = 1
    return _DropoutFn.apply(x, float(rate), seed, site, group_rows, 1, int(row_offset))
  return ref.dropout(x, rate, training, broadcast_dims=broadcast_dims)


def attention_value_dropout(v: torch.Tensor, rate: float, training: bool) -> torch.Tensor:
  """Attention-weight dropout with the mask shared along the query axis
  (t5x/examples/t5/layers.py:115-126) restated on the values: with one keep decision per
  (batch, head, key), sum_k (w[q, k] m[k]) v[k] = sum_k w[q, k] (m[k] v[k]), so scaling the rows
  of v [batch, keys, heads, dim] gives the same result and the attention kernel needs no mask
  input. CUDA bf16 only (callers fall back to explicit weights elsewhere)."""
  if not training or rate == 0.0:
    return v
  seed, site = _dropout_seed_and_site(sharded=True)
  return _DropoutFn.apply(v, float(rate), seed, site, 1, int(v.shape[-1]), 0)


# ----------------------------------------------------------------------------
# Attention
# ----------------------------------------------------------------------------
def attention(q, k, v, *, bias_table: Optional[torch.Tensor] = None, bidirectional: bool = True,
              num_buckets: int = 32, max_distance: int = 128,
              key_mask: Optional[torch.Tensor] = None, causal: bool = False,
              q_segment_ids=None, kv_segment_ids=None, extra_mask=None,
              explicit_bias: Optional[torch.Tensor] = None, q_offset: int = 0,
              float32_logits: bool = False) -> torch.Tensor:
  """Multi-head attention without 1/sqrt(d) scaling. q [B,Lq,H,D], k/v [B,Lk,H,D].

  `bias_table` [H, num_buckets] is the T5 relative-position table; on the CUDA path the
  bias is evaluated inside the kernel and never materialised.
  """
  from t5x_b200.ops import attention as attn_ops
  if (_native_ok(q) and attn_ops.flash_supported(q, k, v, explicit_bias, extra_mask)):
    return attn_ops.flash_attention(q, k, v, bias_table=bias_table, bidirectional=bidirectional,
                                    num_buckets=num_buckets, max_distance=max_distance,
                                    key_mask=key_mask, causal=causal,
                                    q_segment_ids=q_segment_ids, kv_segment_ids=kv_segment_ids,
                                    q_offset=q_offset,
                                    prefix_lm=extra_mask)  # None or a ref.PrefixLMMask
  bias = explicit_bias
  if bias_table is not None:
    rb = ref.relative_position_bias(bias_table.float(), q.shape[1], k.shape[1], bidirectional,
                                    num_buckets, max_distance, q_offset=q_offset)
    bias = rb if bias is None else bias + rb
  if q.is_cuda and q.dtype == torch.bfloat16 and not float32_logits:
    return _library_attention(q, k, v, bias, key_mask, causal, q_segment_ids, kv_segment_ids,
                              extra_mask)
  return ref.attention(q, k, v, bias=bias, key_mask=key_mask, causal=causal,
                       q_segment_ids=q_segment_ids, kv_segment_ids=kv_segment_ids,
                       extra_mask=extra_mask,
                       float32_logits=float32_logits or q.dtype == torch.float32)


def _library_attention(q, k, v, bias, key_mask, causal, q_seg, kv_seg, extra_mask):
  """Library (torch SDPA) attention for shapes the flash kernels do not cover yet: bias and
  masks are folded into one additive [B or 1, H or 1, Lq, Lk] tensor."""
  b, lq, h, d = q.shape
  lk = k.shape[1]
  add = None
  if bias is not None:
    add = bias.to(q.dtype)
    add = add[None] if add.dim() == 3 else add
  mask = None
  if key_mask is not None:
    mask = key_mask[:, None, None, :].bool()
  if causal:
    cm = (torch.arange(lk, device=q.device)[None, :] <=
          torch.arange(lq, device=q.device)[:, None] + (lk - lq))[None, None]
    mask = cm if mask is None else mask & cm
  if q_seg is not None and kv_seg is not None:
    sm = q_seg[:, None, :, None] == kv_seg[:, None, None, :]
    mask = sm if mask is None else mask & sm
  if extra_mask is not None:
    mask = extra_mask.bool() if mask is None else mask & extra_mask.bool()
  if mask is not None:
    neg = torch.zeros(mask.shape, dtype=q.dtype, device=q.device).masked_fill_(~mask, -1e10)
    add = neg if add is None else add + neg
  if add is not None and lk % 8:
    pad = 8 - lk % 8  # the library kernels want the bias rows 16-byte aligned
    add = torch.nn.functional.pad(add.expand(-1, -1, lq, lk), (0, pad))[..., :lk]
  out = torch.nn.functional.scaled_dot_product_attention(
      q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=add, scale=1.0)
  return out.transpose(1, 2)


# ----------------------------------------------------------------------------
# Cross entropy with z-loss on top of the logits projection
# ----------------------------------------------------------------------------
class _LogitsCrossEntropyFn(torch.autograd.Function):
  """per-token (loss, z_loss, correct) = CE(hidden @ W) with the [tokens, vocab] logits never
  written to memory: the projection GEMM folds each accumulator tile into softmax partials in
  its epilogue (forward), and backward runs the projection again with an epilogue that turns
  each tile straight into bf16 dlogits for the two gradient GEMMs. The per-row log-sum-exp is
  all that is kept between the passes (`T5X_B200_FUSED_CE=0` restores materialised logits)."""

  @staticmethod
  def forward(ctx, hidden, weight, targets, z_loss, label_smoothing, logits_scale):
    k = hidden.shape[-1]
    h2 = hidden.reshape(-1, k)
    w = compute_weight(weight, torch.bfloat16)
    if w.shape[0] != k:  # tied embedding [V, d]: logits = h @ E^T
      w = w.t()
    vocab = w.shape[1]
    t2 = targets.reshape(-1)
    fused = _fused_ce_enabled()
    if fused:
      logits = None
      stats, _, arg_idx = native.gemm_ce_stats(h2, w, t2, alpha=logits_scale)
    else:
      logits = native.gemm(h2, w, out_dtype=torch.float32, alpha=logits_scale)
      stats, _, arg_idx = native.ce_stats(logits, t2)
    lse = stats[:, 0] + torch.log(stats[:, 1])
    conf, low, norm_const = ref.label_smoothing_constants(vocab, label_smoothing)
    tl = stats[:, 2]
    soft_dot = conf * tl + low * (stats[:, 3] - tl) if label_smoothing > 0 else tl
    z = z_loss * lse * lse
    loss = lse - soft_dot + z - norm_const
    correct = (arg_idx.long() == t2)
    if fused:
      ctx.save_for_backward(hidden, weight, t2, lse)
    else:
      ctx.save_for_backward(hidden, weight, t2, lse, logits)
    ctx.cfg = (z_loss, conf, low, logits_scale)
    ctx.mark_non_differentiable(correct)
    return loss.view(targets.shape), z.view(targets.shape), correct.view(targets.shape)

  @staticmethod
  def backward(ctx, dloss, dz, _dcorrect):
    saved = ctx.saved_tensors
    hidden, weight, t2, lse = saved[:4]
    logits = saved[4] if len(saved) > 4 else None
    z_loss, conf, low, logits_scale = ctx.cfg
    k = hidden.shape[-1]
    h2 = hidden.reshape(-1, k)
    w = compute_weight(weight, torch.bfloat16)
    tied = w.shape[0] != k
    if tied:
      w = w.t()
    # `loss` already contains the z term; a gradient arriving through the separate z output
    # (metrics only) is ignored, as in the reference's custom VJP (t5x/losses.py:98-124).
    row_scale = (dloss.reshape(-1).float() * logits_scale).contiguous()
    if logits is None:
      dlogits = native.gemm_ce_grad(h2, w, t2, lse.contiguous(), row_scale, z_loss, conf, low,
                                    alpha=logits_scale)
    else:
      dlogits = native.ce_grad(logits, t2, lse, row_scale, z_loss, conf, low)
    dh = native.gemm(dlogits, w.t()).view(hidden.shape) if ctx.needs_input_grad[0] else None
    dw = None
    if ctx.needs_input_grad[1]:
      if tied:
        mg = getattr(weight, "main_grad", None)
        if mg is not None:
          first = not getattr(weight, "grad_ready", False)
          native.gemm(dlogits.t(), h2, out=mg, accumulate=not first)
          weight.grad_ready = True
        else:
          dw = native.gemm(dlogits.t(), h2, out_dtype=torch.float32).to(weight.dtype)
      else:
        dw = _accumulate_wgrad(weight, h2.t(), dlogits)
    return dh, dw, None, None, None, None


def _fused_ce_enabled() -> bool:
  import os
  return os.environ.get("T5X_B200_FUSED_CE", "1") != "0"


def logits_cross_entropy(hidden, weight, targets, *, z_loss: float = 0.0,
                         label_smoothing: float = 0.0, logits_scale: float = 1.0,
                         dtype: Optional[torch.dtype] = None):
  """Per-token (loss, z_loss, correct) of softmax cross-entropy over `hidden @ weight`.

  The loss includes the z-loss term and subtracts the label-smoothing normalising
  constant, as `compute_weighted_cross_entropy` does before weighting (t5x/losses.py:132-193).
  """
  if _native_ok(hidden):
    return _LogitsCrossEntropyFn.apply(hidden, weight, targets, z_loss, label_smoothing,
                                       logits_scale)
  k = hidden.shape[-1]
  w = weight.float()
  if w.shape[0] != k:
    w = w.t()
  logits = (hidden.float() @ w) * logits_scale
  loss, z, _, am = ref.token_cross_entropy(logits, targets, z_loss, label_smoothing)
  return loss, z, (am == targets)
