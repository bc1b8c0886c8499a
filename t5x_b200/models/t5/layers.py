"""T5 layer library: attention, dense, gated MLP, embedding, relative position bias, RMSNorm.

Behavioural parity target: t5x/examples/t5/layers.py (parameter names, kernel layouts
`[in, out]`, fp32 master weights cast to the compute dtype, no biases, no 1/sqrt(d) on the
attention logits, additive -1e10 masks). The implementation is PyTorch modules over
:mod:`t5x_b200.ops.functional`, whose CUDA path is the hand-written sm_100a kernel set.
Every parameter carries `axes` (logical axis names) used by the partitioner, the
optimizer's factoring rules and the checkpoint writer.

Tensor parallelism is explicit: column-parallel q/k/v/wi hold `1/model` of their output
features, row-parallel out/wo hold `1/model` of their input features and are followed by a
reduction over the `model` axis.
"""
from __future__ import annotations

import math
from typing import Callable, Optional, Sequence, Tuple

import torch
from torch import nn

from t5x_b200.ops import functional as F
from t5x_b200.ops import reference as ref
from t5x_b200.parallel import state as pstate
from t5x_b200.parallel import tp

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16,
          torch.float32: torch.float32, torch.bfloat16: torch.bfloat16,
          torch.float16: torch.float16}


def canonical_dtype(d) -> torch.dtype:
  if isinstance(d, torch.dtype):
    return d
  name = getattr(d, "__name__", None) or str(d)
  name = name.replace("jnp.", "").replace("torch.", "")
  return DTYPES[name]


# ----------------------------------------------------------------------------
# Parameter helpers
# ----------------------------------------------------------------------------
def param_with_axes(shape: Sequence[int], init: Callable[[torch.Tensor], None],
                    axes: Tuple[str, ...], shard_dim: Optional[int] = None,
                    device=None) -> nn.Parameter:
  """fp32 parameter annotated with logical axis names. With `shard_dim` the parameter is the
  local 1/model slice along that dim of a global tensor of shape `global_shape`."""
  st = pstate.get()
  shape = list(shape)
  global_shape = tuple(shape)
  if shard_dim is not None and st.model_size > 1:
    if shape[shard_dim] % st.model_size:
      raise ValueError(f"dim {shard_dim} of {shape} is not divisible by model={st.model_size}")
    shape[shard_dim] //= st.model_size
  else:
    shard_dim = None
  p = nn.Parameter(torch.empty(shape, dtype=torch.float32, device=device))
  if p.device.type != "meta":
    if shard_dim is None:
      with torch.no_grad():
        init(p)
    else:
      # Initialise the global tensor's statistics, then keep the local slice, so that the
      # fan-in/fan-out used by the initialiser is that of the unsharded parameter.
      full = torch.empty(global_shape, dtype=torch.float32, device=p.device)
      init(full)
      lo, hi = tp.shard_range(global_shape[shard_dim], st.model_size, st.model_rank)
      with torch.no_grad():
        p.copy_(full.narrow(shard_dim, lo, hi - lo))
  p.axes = tuple(axes)
  p.global_shape = global_shape
  p.shard_dim = shard_dim
  p.init_fn = init
  return p


def reinitialize(module: nn.Module, seed: int) -> None:
  """Re-draws every parameter from its initialiser under `seed` (same draw on every rank
  for the global tensor; each rank keeps its own slice)."""
  st = pstate.get()
  gen_state = torch.random.get_rng_state()
  torch.manual_seed(int(seed))
  try:
    for _, p in module.named_parameters():
      init = getattr(p, "init_fn", None)
      if init is None or p.device.type == "meta":
        continue
      if getattr(p, "shard_dim", None) is None:
        with torch.no_grad():
          init(p)
      else:
        full = torch.empty(p.global_shape, dtype=torch.float32, device=p.device)
        init(full)
        lo, hi = tp.shard_range(p.global_shape[p.shard_dim], st.model_size, st.model_rank)
        with torch.no_grad():
          p.copy_(full.narrow(p.shard_dim, lo, hi - lo))
      bf = getattr(p, "bf16", None)
      if bf is not None:
        with torch.no_grad():
          bf.copy_(p)
  finally:
    torch.random.set_rng_state(gen_state)


def _fans(shape, in_axis=-2, out_axis=-1):
  receptive = 1
  for i, s in enumerate(shape):
    if i not in (in_axis % len(shape), out_axis % len(shape)):
      receptive *= s
  return shape[in_axis] * receptive, shape[out_axis] * receptive


def variance_scaling(scale: float, mode: str, distribution: str, in_axis=-2, out_axis=-1,
                     divide_by: float = 1.0):
  """jax.nn.initializers.variance_scaling (distribution parity; the bits differ)."""

  def init(t: torch.Tensor):
    fan_in, fan_out = _fans(tuple(t.shape), in_axis, out_axis)
    denom = {"fan_in": fan_in, "fan_out": fan_out, "fan_avg": (fan_in + fan_out) / 2}[mode]
    var = scale / max(1.0, denom)
    with torch.no_grad():
      if distribution == "normal":
        t.normal_(0.0, math.sqrt(var))
      elif distribution == "truncated_normal":
        std = math.sqrt(var) / 0.87962566103423978
        nn.init.trunc_normal_(t, 0.0, std, -2 * std, 2 * std)
      elif distribution == "uniform":
        lim = math.sqrt(3.0 * var)
        t.uniform_(-lim, lim)
      else:
        raise ValueError(distribution)
      if divide_by != 1.0:
        t.div_(divide_by)

  return init


def normal_init(stddev: float):
  def init(t):
    with torch.no_grad():
      t.normal_(0.0, stddev)
  return init


def ones_init(t):
  with torch.no_grad():
    t.fill_(1.0)


# ----------------------------------------------------------------------------
# Mask helpers (API parity with layers.py:708-924; the attention op itself takes
# per-token metadata and never needs these [b,1,q,k] tensors)
# ----------------------------------------------------------------------------
def make_attention_mask(query_input, key_input, pairwise_fn=torch.mul, dtype=torch.float32):
  mask = pairwise_fn(query_input[..., :, None], key_input[..., None, :])
  return mask[..., None, :, :].to(dtype)


def make_causal_mask(x, dtype=torch.float32):
  idxs = torch.arange(x.shape[-1], device=x.device).expand(x.shape)
  return make_attention_mask(idxs, idxs, torch.ge, dtype=dtype)


def combine_masks(*masks, dtype=torch.float32):
  masks = [m for m in masks if m is not None]
  if not masks:
    return None
  out = masks[0]
  for m in masks[1:]:
    out = torch.logical_and(out.bool(), m.bool())
  return out.to(dtype)


def combine_biases(*biases):
  biases = [b for b in biases if b is not None]
  if not biases:
    return None
  out = biases[0]
  for b in biases[1:]:
    out = out + b
  return out


def make_decoder_mask(decoder_target_tokens, dtype=torch.float32, decoder_causal_attention=None,
                      decoder_segment_ids=None):
  masks = []
  causal = make_causal_mask(decoder_target_tokens, dtype=dtype)
  if decoder_causal_attention is not None:
    inputs_mask = make_attention_mask(decoder_causal_attention, decoder_causal_attention,
                                      torch.logical_and, dtype=dtype)
    masks.append(torch.logical_or(causal.bool(), inputs_mask.bool()).to(dtype))
  else:
    masks.append(causal)
  masks.append(make_attention_mask(decoder_target_tokens > 0, decoder_target_tokens > 0,
                                   dtype=dtype))
  if decoder_segment_ids is not None:
    masks.append(make_attention_mask(decoder_segment_ids, decoder_segment_ids, torch.eq,
                                     dtype=dtype))
  return combine_masks(*masks, dtype=dtype)


def dot_product_attention(query, key, value, bias=None, dropout_rate=0.0, deterministic=True,
                          dtype=torch.float32, float32_logits=False):
  """[b, q, h, d] attention with a materialised additive bias (layers.py:52-129)."""
  if float32_logits:
    query, key = query.float(), key.float()
  w = torch.einsum("bqhd,bkhd->bhqk", query, key)
  if bias is not None:
    w = w + bias.to(w.dtype)
  w = torch.softmax(w, dim=-1).to(dtype)
  if not deterministic and dropout_rate > 0.0:
    w = ref.dropout(w, dropout_rate, True, broadcast_dims=(-2,))
  return torch.einsum("bhqk,bkhd->bqhd", w, value.to(dtype))


# ----------------------------------------------------------------------------
# Modules
# ----------------------------------------------------------------------------
class DenseGeneral(nn.Module):
  """Bias-free projection y = x @ kernel, kernel [in, out] fp32 (layers.py:364-414)."""

  def __init__(self, in_features: int, out_features: int, kernel_axes: Tuple[str, str],
               kernel_init=None, dtype=torch.float32, shard_dim: Optional[int] = None,
               device=None):
    super().__init__()
    self.dtype = canonical_dtype(dtype)
    init = kernel_init or variance_scaling(1.0, "fan_in", "truncated_normal")
    self.kernel = param_with_axes((in_features, out_features), init, kernel_axes,
                                  shard_dim=shard_dim, device=device)

  def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    return F.linear(x.to(self.dtype), self.kernel, residual=residual, dtype=self.dtype)


class LayerNorm(nn.Module):
  """T5 RMS norm: scale only, fp32 statistics, eps 1e-6 (layers.py:683-702)."""

  def __init__(self, features: int, epsilon: float = 1e-6, dtype=torch.float32, device=None):
    super().__init__()
    self.epsilon = epsilon
    self.dtype = canonical_dtype(dtype)
    self.scale = param_with_axes((features,), ones_init, ("embed",), device=device)

  def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
              with_residual: bool = False):
    """`with_residual`: returns (x, norm(x)); pass the first element on as the residual."""
    if with_residual:
      return F.residual_rmsnorm(x.to(self.dtype), self.scale, self.epsilon, out=out)
    return F.rmsnorm(x.to(self.dtype), self.scale, self.epsilon, out=out)


class Embed(nn.Module):
  """Token embedding [vocab, features]; `attend` gives tied logits (layers.py:490-557).
  Under tensor parallelism the vocabulary is sharded: each rank looks up the ids it owns
  and the partial results are summed over the model axis."""

  def __init__(self, num_embeddings: int, features: int, dtype=torch.float32,
               embedding_init=None, one_hot: bool = False, device=None):
    super().__init__()
    self.num_embeddings = num_embeddings
    self.features = features
    self.dtype = canonical_dtype(dtype)
    self.embedding = param_with_axes((num_embeddings, features),
                                     embedding_init or normal_init(1.0), ("vocab", "embed"),
                                     shard_dim=0, device=device)

  def forward(self, ids: torch.Tensor) -> torch.Tensor:
    st = pstate.get()
    if self.embedding.shard_dim is None:
      return F.embedding(ids.long(), self.embedding, self.dtype)
    lo, hi = tp.shard_range(self.num_embeddings, st.model_size, st.model_rank)
    local = ids.long() - lo
    own = (local >= 0) & (local < hi - lo)
    out = F.embedding(torch.where(own, local, torch.zeros_like(local)), self.embedding,
                      self.dtype)
    out = out * own[..., None].to(out.dtype)
    return tp.reduce_from_model_parallel(out)

  def attend(self, query: torch.Tensor) -> torch.Tensor:
    w = F.compute_weight(self.embedding, torch.float32)
    return query.float() @ w.t()


class RelativePositionBiases(nn.Module):
  """[heads, num_buckets] table of learned biases per relative-position bucket
  (layers.py:560-677). Heads are sharded over the model axis."""

  def __init__(self, num_buckets: int, max_distance: int, num_heads: int, dtype=torch.float32,
               embedding_init=None, device=None):
    super().__init__()
    self.num_buckets = num_buckets
    self.max_distance = max_distance
    self.num_heads = num_heads
    self.dtype = canonical_dtype(dtype)
    self.rel_embedding = param_with_axes(
        (num_heads, num_buckets),
        embedding_init or variance_scaling(1.0, "fan_avg", "uniform", in_axis=-1, out_axis=-2),
        ("heads", "relpos_buckets"), shard_dim=0, device=device)

  @staticmethod
  def _relative_position_bucket(relative_position, bidirectional=True, num_buckets=32,
                                max_distance=128):
    return ref.relative_position_bucket(relative_position, bidirectional, num_buckets,
                                        max_distance)

  def forward(self, qlen: int, klen: int, bidirectional: bool = True,
              q_offset: int = 0) -> torch.Tensor:
    """Materialised [1, heads, qlen, klen] bias (API parity / CPU path)."""
    b = ref.relative_position_bias(self.rel_embedding.to(self.dtype), qlen, klen, bidirectional,
                                   self.num_buckets, self.max_distance, q_offset=q_offset)
    return b[None]


def sp_output_dropout(y_sp: torch.Tensor, rate: float, seq_len: int) -> torch.Tensor:
  """Dropout (mask shared along the sequence) of this rank's rows of a row-sharded
  [batch * seq_len, emb] activation: the rows' global indices select the mask, so the ranks
  together apply exactly the mask one rank holding all rows would."""
  st = pstate.get()
  return F.dropout(y_sp, rate, True, broadcast_dims=(-2,), seq_len=seq_len,
                   row_offset=st.model_rank * y_sp.shape[0])


class MultiHeadDotProductAttention(nn.Module):
  """Multi-head attention with q/k/v/out projections (layers.py:132-346).

  The relative-position table and the padding/causal/segment structure are passed as
  per-token metadata so the CUDA flash kernel can build bias and masks on the fly.
  """

  def __init__(self, emb_dim: int, num_heads: int, head_dim: int, dtype=torch.float32,
               dropout_rate: float = 0.0, float32_logits: bool = False,
               scale_attn_logits: bool = False, device=None):
    super().__init__()
    st = pstate.get()
    if num_heads % st.model_size:
      raise ValueError(f"{num_heads} heads are not divisible by model={st.model_size}")
    self.num_heads = num_heads
    self.local_heads = num_heads // st.model_size
    self.head_dim = head_dim
    self.dtype = canonical_dtype(dtype)
    self.dropout_rate = dropout_rate
    self.float32_logits = float32_logits
    self.scale_attn_logits = scale_attn_logits
    inner = num_heads * head_dim
    depth_scaling = 1.0 if scale_attn_logits else math.sqrt(head_dim)
    kv_init = variance_scaling(1.0, "fan_in", "normal")
    q_init = variance_scaling(1.0, "fan_in", "normal", divide_by=depth_scaling)
    self.query = DenseGeneral(emb_dim, inner, ("embed", "joined_kv"), q_init, dtype, 1, device)
    self.key = DenseGeneral(emb_dim, inner, ("embed", "joined_kv"), kv_init, dtype, 1, device)
    self.value = DenseGeneral(emb_dim, inner, ("embed", "joined_kv"), kv_init, dtype, 1, device)
    self.out = DenseGeneral(inner, emb_dim, ("joined_kv", "embed"), kv_init, dtype, 0, device)

  # -- cache helpers ----------------------------------------------------------------------
  def init_cache(self, batch: int, max_len: int, device) -> dict:
    shape = (batch, max_len, self.local_heads, self.head_dim)
    return {"cached_key": torch.zeros(shape, dtype=self.dtype, device=device),
            "cached_value": torch.zeros(shape, dtype=self.dtype, device=device),
            "cache_index": torch.zeros((), dtype=torch.int32, device=device)}

  def project_kv(self, inputs_kv: torch.Tensor):
    b, lk, _ = inputs_kv.shape
    kv_in = tp.copy_to_model_parallel(inputs_kv).to(self.dtype)
    k, v = F.multi_linear(kv_in, [self.key.kernel, self.value.kernel], dtype=self.dtype)
    return (k.view(b, lk, self.local_heads, self.head_dim),
            v.view(b, lk, self.local_heads, self.head_dim))

  def forward(self, inputs_q: torch.Tensor, inputs_kv: Optional[torch.Tensor], *,
              bias_table: Optional[torch.Tensor] = None, bidirectional: bool = True,
              num_buckets: int = 32, max_distance: int = 128,
              key_mask: Optional[torch.Tensor] = None, causal: bool = False,
              q_segment_ids=None, kv_segment_ids=None, extra_mask=None, explicit_bias=None,
              cache: Optional[dict] = None, decode: bool = False, prefill: bool = False,
              prefill_lengths: Optional[torch.Tensor] = None,
              precomputed_kv: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
              residual: Optional[torch.Tensor] = None, enable_dropout: bool = False,
              beams_per_kv: int = 1) -> torch.Tensor:
    b, lq, _ = inputs_q.shape
    q_in = tp.copy_to_model_parallel(inputs_q)
    if (precomputed_kv is None and inputs_kv is inputs_q and not self.scale_attn_logits):
      # self-attention: the three projections share their input, and one backward builds its
      # gradient by accumulating GEMMs
      q, k, v = F.multi_linear(q_in.to(self.dtype),
                               [self.query.kernel, self.key.kernel, self.value.kernel],
                               dtype=self.dtype)
      q = q.view(b, lq, self.local_heads, self.head_dim)
      k = k.view(b, lq, self.local_heads, self.head_dim)
      v = v.view(b, lq, self.local_heads, self.head_dim)
    else:
      if self.scale_attn_logits:
        q_in = q_in / math.sqrt(self.head_dim)
      q = self.query(q_in).view(b, lq, self.local_heads, self.head_dim)
      if precomputed_kv is not None:
        k, v = precomputed_kv
      else:
        k, v = self.project_kv(inputs_kv)
    q_offset = 0
    if cache is not None and prefill:
      # Fill the cache with the prompt's keys/values in one pass.
      lk = k.shape[1]
      cache["cached_key"][:, :lk] = k
      cache["cached_value"][:, :lk] = v
      if prefill_lengths is not None:
        cache["cache_index"] = prefill_lengths.to(torch.int32)
      else:
        cache["cache_index"] = torch.full((), lk, dtype=torch.int32, device=q.device)
    elif cache is not None and decode:
      idx = cache["cache_index"]
      max_len = cache["cached_key"].shape[1]
      pos = torch.arange(max_len, device=q.device)
      if idx.dim() == 0:
        i = int(idx)
        cache["cached_key"][:, i] = k[:, 0]
        cache["cached_value"][:, i] = v[:, 0]
        key_mask = (pos <= i)[None].expand(b, max_len)
        q_offset = i
        cache["cache_index"] = idx + 1
        k, v = cache["cached_key"], cache["cached_value"]
        if bias_table is not None:
          explicit_bias = ref.relative_position_bias(
              F.compute_weight(bias_table, torch.float32), 1, max_len, bidirectional,
              num_buckets, max_distance, q_offset=i)
          bias_table = None
      else:
        # Per-example cache positions (prefix-LM prefill paths).
        rows = torch.arange(b, device=q.device)
        il = idx.long()
        # A row already at the end of its buffer keeps stepping until the whole batch is done;
        # its write is dropped (the one-hot update of the reference is all-zero there).
        inb = (il < max_len)[:, None, None]
        ic = il.clamp(max=max_len - 1)
        cache["cached_key"][rows, ic] = torch.where(inb, k[:, 0], cache["cached_key"][rows, ic])
        cache["cached_value"][rows, ic] = torch.where(inb, v[:, 0],
                                                      cache["cached_value"][rows, ic])
        key_mask = pos[None, :] <= il[:, None]
        cache["cache_index"] = idx + 1
        k, v = cache["cached_key"], cache["cached_value"]
        if bias_table is not None:
          rel = pos[None, :] - il[:, None]  # [b, max_len]
          buckets = ref.relative_position_bucket(rel, bidirectional, num_buckets, max_distance)
          tab = F.compute_weight(bias_table, torch.float32)
          eb = tab[:, buckets].permute(1, 0, 2)[:, :, None, :]  # [b, h, 1, k]
          extra = eb
          explicit_bias = None
          bias_table = None
          x = self._attend(q, k, v, None, bidirectional, num_buckets, max_distance, key_mask,
                           False, None, None, extra_mask, None, 0, enable_dropout,
                           per_example_bias=extra)
          return self._project_out(x, b, lq, residual)
      causal = False
    x = self._attend(q, k, v, bias_table, bidirectional, num_buckets, max_distance, key_mask,
                     causal, q_segment_ids, kv_segment_ids, extra_mask, explicit_bias, q_offset,
                     enable_dropout, beams_per_kv=beams_per_kv)
    return self._project_out(x, b, lq, residual)

  def forward_sp(self, h_sp: torch.Tensor, x_sp: torch.Tensor, batch: int, lq: int, *,
                 kv_full: Optional[torch.Tensor] = None, h_block=None, bias_table=None,
                 bidirectional: bool = True, num_buckets: int = 32, max_distance: int = 128,
                 key_mask=None, causal: bool = False, q_segment_ids=None,
                 kv_segment_ids=None, dropout_rate: float = 0.0) -> torch.Tensor:
    """Row-sharded ("sequence parallel") form under tensor parallelism: `h_sp` / `x_sp` are
    this rank's rows of the normed input and of the residual stream ([batch * lq / T, emb]).
    The q/k/v projections gather the rows inside their GEMM kernel and the output projection
    scatters its partial sums from its epilogue (see `t5x_b200.parallel.tp_fused`); returns
    this rank's rows of the new residual stream. `kv_full` (cross-attention) is the replicated
    [batch, lk, emb] encoder output."""
    from t5x_b200.parallel import tp_fused
    if self.scale_attn_logits:
      h_sp, h_block = h_sp / math.sqrt(self.head_dim), None
    hd = (self.local_heads, self.head_dim)
    if kv_full is None:
      tp_fused.fuse_weight_columns([self.query.kernel, self.key.kernel, self.value.kernel])
      q, k, v = tp_fused.all_gather_linears(
          h_sp, [self.query.kernel, self.key.kernel, self.value.kernel], block=h_block)
      lk = lq
    else:
      (q,) = tp_fused.all_gather_linears(h_sp, [self.query.kernel], block=h_block)
      lk = kv_full.shape[1]
      k, v = self.key(kv_full), self.value(kv_full)
    q = q.view(batch, lq, *hd)
    k = k.view(batch, lk, *hd)
    v = v.view(batch, lk, *hd)
    x = self._attend(q, k, v, bias_table, bidirectional, num_buckets, max_distance, key_mask,
                     causal, q_segment_ids, kv_segment_ids, None, None, 0, dropout_rate > 0.0)
    x = x.reshape(batch * lq, self.local_heads * self.head_dim)
    if dropout_rate > 0.0:
      return x_sp + sp_output_dropout(tp_fused.linear_reduce_scatter(x, self.out.kernel, None),
                                      dropout_rate, lq)
    return tp_fused.linear_reduce_scatter(x, self.out.kernel, x_sp)

  def _project_out(self, x, b, lq, residual):
    x = x.reshape(b, lq, self.local_heads * self.head_dim)
    st = pstate.get()
    if st.model_size == 1:
      return self.out(x, residual=residual)
    y = tp.reduce_from_model_parallel(self.out(x))
    return y if residual is None else y + residual

  def _attend(self, q, k, v, bias_table, bidirectional, num_buckets, max_distance, key_mask,
              causal, q_seg, kv_seg, extra_mask, explicit_bias, q_offset, enable_dropout,
              per_example_bias=None, beams_per_kv: int = 1):
    if beams_per_kv > 1:
      # q rows are [batch*beams]; k/v are shared by the beams of one example.
      bb, lq, h, d = q.shape
      b0 = bb // beams_per_kv
      qg = q.view(b0, beams_per_kv * lq, h, d)
      out = F.attention(qg, k, v, key_mask=key_mask, float32_logits=self.float32_logits)
      return out.reshape(bb, lq, h, d)
    drop = enable_dropout and self.dropout_rate > 0.0
    if drop and per_example_bias is None and q.is_cuda and q.dtype == torch.bfloat16:
      from t5x_b200.ops import attention as attn_ops
      if attn_ops.flash_supported(q, k, v, explicit_bias, extra_mask):
        # the dropout mask of the attention weights is shared along the query axis, so it can
        # be applied to the rows of v instead and the flash kernel runs unchanged
        v = F.attention_value_dropout(v, self.dropout_rate, True)
        drop = False
    if per_example_bias is not None or drop:
      dt = torch.float32 if self.float32_logits else q.dtype
      logits = torch.einsum("bqhd,bkhd->bhqk", q.to(dt), k.to(dt))
      if per_example_bias is not None:
        logits = logits + per_example_bias.to(dt)
      if bias_table is not None:
        logits = logits + ref.relative_position_bias(
            F.compute_weight(bias_table, torch.float32), q.shape[1], k.shape[1], bidirectional,
            num_buckets, max_distance, q_offset=q_offset).to(dt)[None]
      if explicit_bias is not None:
        logits = logits + explicit_bias.to(dt)
      mask = None
      if key_mask is not None:
        mask = key_mask[:, None, None, :].bool()
      if causal:
        lq, lk = q.shape[1], k.shape[1]
        cm = (torch.arange(lk, device=q.device)[None, :] <=
              torch.arange(lq, device=q.device)[:, None] + (lk - lq))[None, None]
        mask = cm if mask is None else mask & cm
      if q_seg is not None and kv_seg is not None:
        sm = q_seg[:, None, :, None] == kv_seg[:, None, None, :]
        mask = sm if mask is None else mask & sm
      if extra_mask is not None:
        mask = extra_mask.bool() if mask is None else mask & extra_mask.bool()
      if mask is not None:
        logits = torch.where(mask, logits, torch.full_like(logits, ref.NEG_MASK))
      w = torch.softmax(logits.float(), dim=-1).to(v.dtype)
      if enable_dropout and self.dropout_rate > 0.0:
        w = ref.dropout(w, self.dropout_rate, True, broadcast_dims=(-2,))
      return torch.einsum("bhqk,bkhd->bqhd", w, v)
    return F.attention(q, k, v, bias_table=bias_table, bidirectional=bidirectional,
                       num_buckets=num_buckets, max_distance=max_distance, key_mask=key_mask,
                       causal=causal, q_segment_ids=q_seg, kv_segment_ids=kv_seg,
                       extra_mask=extra_mask, explicit_bias=explicit_bias, q_offset=q_offset,
                       float32_logits=self.float32_logits)


class MlpBlock(nn.Module):
  """wi (or wi_0, wi_1, ...) -> activations -> product -> dropout -> wo (layers.py:417-487)."""

  def __init__(self, emb_dim: int, intermediate_dim: int = 2048,
               activations: Sequence[str] = ("relu",), intermediate_dropout_rate: float = 0.1,
               dtype=torch.float32, kernel_init=None, device=None):
    super().__init__()
    self.activations = tuple(activations)
    self.dropout_rate = intermediate_dropout_rate
    self.dtype = canonical_dtype(dtype)
    init = kernel_init or variance_scaling(1.0, "fan_in", "truncated_normal")
    if len(self.activations) == 1:
      self.wi = DenseGeneral(emb_dim, intermediate_dim, ("embed", "mlp"), init, dtype, 1, device)
    else:
      for i in range(len(self.activations)):
        setattr(self, f"wi_{i}", DenseGeneral(emb_dim, intermediate_dim, ("embed", "mlp"), init,
                                              dtype, 1, device))
    self.wo = DenseGeneral(intermediate_dim, emb_dim, ("mlp", "embed"), init, dtype, 0, device)

  def forward_sp(self, h_sp: torch.Tensor, x_sp: torch.Tensor, h_block=None, *,
                 seq_len: Optional[int] = None, dropout_rate: float = 0.0) -> torch.Tensor:
    """Row-sharded form under tensor parallelism: wi gathers the rows inside its GEMM kernel,
    wo scatters its partial sums from its epilogue; returns this rank's rows of the new
    residual stream. `h_block`: the arena block `h_sp` was written into, if any. With
    `dropout_rate` > 0 (training) the intermediate and the block output are dropped out with
    masks shared along the `seq_len` positions of a sequence."""
    from t5x_b200.parallel import tp_fused
    if self.activations == ("gelu", "linear"):
      g = tp_fused.all_gather_gated_gelu(h_sp, self.wi_0.kernel, self.wi_1.kernel, block=h_block)
    elif len(self.activations) == 1:
      (g,) = tp_fused.all_gather_linears(h_sp, [self.wi.kernel], block=h_block)
      g = ref.ACTIVATIONS[self.activations[0]](g)
    else:
      hs = tp_fused.all_gather_linears(
          h_sp, [getattr(self, f"wi_{i}").kernel for i in range(len(self.activations))],
          block=h_block)
      g = None
      for act, h in zip(self.activations, hs):
        h = ref.ACTIVATIONS[act](h)
        g = h if g is None else g * h
    if dropout_rate > 0.0:
      g = F.dropout(g, self.dropout_rate, True, broadcast_dims=(-2,), seq_len=seq_len,
                    sharded=True)
      return x_sp + sp_output_dropout(tp_fused.linear_reduce_scatter(g, self.wo.kernel, None),
                                      dropout_rate, seq_len)
    return tp_fused.linear_reduce_scatter(g, self.wo.kernel, x_sp)

  def forward(self, inputs: torch.Tensor, residual: Optional[torch.Tensor] = None,
              enable_dropout: bool = False) -> torch.Tensor:
    x_in = tp.copy_to_model_parallel(inputs.to(self.dtype))
    if self.activations == ("gelu", "linear"):
      x = F.gated_gelu_mlp_in(x_in, self.wi_0.kernel, self.wi_1.kernel, dtype=self.dtype)
    elif len(self.activations) == 1:
      x = ref.ACTIVATIONS[self.activations[0]](self.wi(x_in))
    else:
      x = None
      for i, act in enumerate(self.activations):
        h = ref.ACTIVATIONS[act](getattr(self, f"wi_{i}")(x_in))
        x = h if x is None else x * h
    x = F.dropout(x, self.dropout_rate, enable_dropout, broadcast_dims=(-2,),
                  sharded=pstate.get().model_size > 1)
    st = pstate.get()
    if st.model_size == 1:
      return self.wo(x, residual=residual)
    y = tp.reduce_from_model_parallel(self.wo(x))
    return y if residual is None else y + residual
