"""T5 encoder-decoder network (parity target: t5x/examples/t5/network.py).

Parameter tree (names joined by '/', identical to the reference checkpoint layout):
  token_embedder/embedding
  encoder/relpos_bias/rel_embedding, encoder/layers_{i}/{pre_attention_layer_norm/scale,
    attention/{query,key,value,out}/kernel, pre_mlp_layer_norm/scale, mlp/{wi_0,wi_1|wi,wo}/kernel},
  encoder/encoder_norm/scale
  decoder/relpos_bias/rel_embedding, decoder/layers_{i}/{pre_self_attention_layer_norm,
    self_attention, pre_cross_attention_layer_norm, encoder_decoder_attention,
    pre_mlp_layer_norm, mlp}, decoder/decoder_norm/scale, decoder/logits_dense/kernel
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any, Optional, Sequence

import torch
from torch import nn

from t5x_b200.models.t5 import layers
from t5x_b200.ops import functional as F
from t5x_b200.ops import reference as ref
from t5x_b200.parallel import state as pstate
from t5x_b200.parallel import tp_fused
from t5x_b200.parallel import tp


@dataclasses.dataclass
class T5Config:
  """Hyper-parameters (field names as in t5x/examples/t5/network.py:25-44)."""
  vocab_size: int
  dtype: Any = "float32"
  emb_dim: int = 512
  num_heads: int = 8
  num_encoder_layers: int = 6
  num_decoder_layers: int = 6
  head_dim: int = 64
  mlp_dim: int = 2048
  mlp_activations: Sequence[str] = ("relu",)
  dropout_rate: float = 0.1
  logits_via_embedding: bool = False
  float32_attention_logits: bool = False
  # extensions
  scale_attn_logits: bool = False      # t5x/contrib/gpu/t5/layers.py:205-206
  relpos_num_buckets: int = 32
  relpos_max_distance: int = 128


def _dropout(x, rate, enable, broadcast=True, **kw):
  return F.dropout(x, rate, enable, broadcast_dims=(-2,) if broadcast else (), **kw)


class EncoderLayer(nn.Module):
  """pre-LN self-attention and pre-LN MLP, each with a residual (network.py:47-96)."""

  def __init__(self, config: T5Config, device=None):
    super().__init__()
    c = config
    self.config = c
    self.pre_attention_layer_norm = layers.LayerNorm(c.emb_dim, dtype=c.dtype, device=device)
    self.attention = layers.MultiHeadDotProductAttention(
        c.emb_dim, c.num_heads, c.head_dim, c.dtype, c.dropout_rate, c.float32_attention_logits,
        c.scale_attn_logits, device=device)
    self.pre_mlp_layer_norm = layers.LayerNorm(c.emb_dim, dtype=c.dtype, device=device)
    self.mlp = layers.MlpBlock(c.emb_dim, c.mlp_dim, c.mlp_activations, c.dropout_rate, c.dtype,
                               device=device)

  def forward(self, x, *, bias_table, key_mask, segment_ids=None, enable_dropout=False):
    c = self.config
    drop = enable_dropout and c.dropout_rate > 0
    x, h = self.pre_attention_layer_norm(x, with_residual=True)
    if drop:
      a = self.attention(h, h, bias_table=bias_table, bidirectional=True,
                         num_buckets=c.relpos_num_buckets, max_distance=c.relpos_max_distance,
                         key_mask=key_mask, q_segment_ids=segment_ids, kv_segment_ids=segment_ids,
                         enable_dropout=True)
      x = x + _dropout(a, c.dropout_rate, True)
    else:
      x = self.attention(h, h, bias_table=bias_table, bidirectional=True,
                         num_buckets=c.relpos_num_buckets, max_distance=c.relpos_max_distance,
                         key_mask=key_mask, q_segment_ids=segment_ids, kv_segment_ids=segment_ids,
                         residual=x)
    x, h = self.pre_mlp_layer_norm(x, with_residual=True)
    if drop:
      x = x + _dropout(self.mlp(h, enable_dropout=True), c.dropout_rate, True)
    else:
      x = self.mlp(h, residual=x)
    return x

  def forward_sp(self, x_sp, batch, length, *, bias_table, key_mask, segment_ids=None,
                 enable_dropout=False):
    """Row-sharded residual stream under fused tensor parallelism."""
    c = self.config
    rate = c.dropout_rate if enable_dropout else 0.0
    _mark_partial(self.pre_attention_layer_norm, self.pre_mlp_layer_norm)
    # each norm writes straight into this rank's rows of the buffer the next GEMM gathers
    blk, dst = tp_fused.rows_buffer(*x_sp.shape)
    x_sp, h = self.pre_attention_layer_norm(x_sp, out=dst, with_residual=True)
    x_sp = self.attention.forward_sp(
        h, x_sp, batch, length, h_block=blk, bias_table=bias_table, bidirectional=True,
        num_buckets=c.relpos_num_buckets, max_distance=c.relpos_max_distance, key_mask=key_mask,
        q_segment_ids=segment_ids, kv_segment_ids=segment_ids, dropout_rate=rate)
    blk, dst = tp_fused.rows_buffer(*x_sp.shape)
    x_sp, h = self.pre_mlp_layer_norm(x_sp, out=dst, with_residual=True)
    return self.mlp.forward_sp(h, x_sp, h_block=blk, seq_len=length, dropout_rate=rate)


def _sp_dropout_ok(x, c, enable_dropout) -> bool:
  """The row-sharded path handles dropout through the in-kernel masks (CUDA, bf16)."""
  return not (enable_dropout and c.dropout_rate > 0) or (x.is_cuda and x.dtype == torch.bfloat16)


def _mark_partial(*norms) -> None:
  """Norm scales applied to row-sharded activations get gradients that cover this rank's
  rows only; the trainer sums them over the model axis."""
  for n in norms:
    n.scale.sp_partial_grad = True


class DecoderLayer(nn.Module):
  """Causal self-attention (+relpos), cross-attention (no bias), MLP (network.py:99-179)."""

  def __init__(self, config: T5Config, device=None):
    super().__init__()
    c = config
    self.config = c
    mk_attn = lambda: layers.MultiHeadDotProductAttention(
        c.emb_dim, c.num_heads, c.head_dim, c.dtype, c.dropout_rate, c.float32_attention_logits,
        c.scale_attn_logits, device=device)
    self.pre_self_attention_layer_norm = layers.LayerNorm(c.emb_dim, dtype=c.dtype, device=device)
    self.self_attention = mk_attn()
    self.pre_cross_attention_layer_norm = layers.LayerNorm(c.emb_dim, dtype=c.dtype,
                                                           device=device)
    self.encoder_decoder_attention = mk_attn()
    self.pre_mlp_layer_norm = layers.LayerNorm(c.emb_dim, dtype=c.dtype, device=device)
    self.mlp = layers.MlpBlock(c.emb_dim, c.mlp_dim, c.mlp_activations, c.dropout_rate, c.dtype,
                               device=device)

  def forward(self, x, encoded, *, bias_table, decoder_key_mask, encoder_key_mask,
              decoder_segment_ids=None, encoder_segment_ids=None, enable_dropout=False,
              decode=False, cache: Optional[dict] = None, beams_per_kv: int = 1):
    c = self.config
    drop = enable_dropout and c.dropout_rate > 0
    rate = c.dropout_rate
    x, h = self.pre_self_attention_layer_norm(x, with_residual=True)
    self_kwargs = dict(bias_table=bias_table, bidirectional=False,
                       num_buckets=c.relpos_num_buckets, max_distance=c.relpos_max_distance)
    if decode:
      a = self.self_attention(h, h, cache=cache["self_attention"], decode=True, **self_kwargs)
      x = x + a
    elif drop:
      a = self.self_attention(h, h, key_mask=decoder_key_mask, causal=True,
                              q_segment_ids=decoder_segment_ids,
                              kv_segment_ids=decoder_segment_ids, enable_dropout=True,
                              **self_kwargs)
      x = x + _dropout(a, rate, True)
    else:
      x = self.self_attention(h, h, key_mask=decoder_key_mask, causal=True,
                              q_segment_ids=decoder_segment_ids,
                              kv_segment_ids=decoder_segment_ids, residual=x, **self_kwargs)
    x, h = self.pre_cross_attention_layer_norm(x, with_residual=True)
    if decode:
      cross = cache["encoder_decoder_attention"]
      if "cross_key" not in cross:
        k, v = self.encoder_decoder_attention.project_kv(encoded)
        cross["cross_key"], cross["cross_value"] = k, v
      x = self.encoder_decoder_attention(
          h, None, key_mask=encoder_key_mask,
          precomputed_kv=(cross["cross_key"], cross["cross_value"]), residual=x,
          beams_per_kv=beams_per_kv)
    elif drop:
      a = self.encoder_decoder_attention(h, encoded, key_mask=encoder_key_mask,
                                         q_segment_ids=decoder_segment_ids,
                                         kv_segment_ids=encoder_segment_ids, enable_dropout=True)
      x = x + _dropout(a, rate, True)
    else:
      x = self.encoder_decoder_attention(h, encoded, key_mask=encoder_key_mask,
                                         q_segment_ids=decoder_segment_ids,
                                         kv_segment_ids=encoder_segment_ids, residual=x)
    x, h = self.pre_mlp_layer_norm(x, with_residual=True)
    if drop:
      x = x + _dropout(self.mlp(h, enable_dropout=True), rate, True)
    else:
      x = self.mlp(h, residual=x)
    return x

  def forward_sp(self, x_sp, encoded, batch, length, *, bias_table, decoder_key_mask,
                 encoder_key_mask, decoder_segment_ids=None, encoder_segment_ids=None,
                 enable_dropout=False):
    """Row-sharded residual stream under fused tensor parallelism (training); `encoded` is the
    replicated encoder output."""
    c = self.config
    rate = c.dropout_rate if enable_dropout else 0.0
    _mark_partial(self.pre_self_attention_layer_norm, self.pre_cross_attention_layer_norm,
                  self.pre_mlp_layer_norm)
    blk, dst = tp_fused.rows_buffer(*x_sp.shape)
    x_sp, h = self.pre_self_attention_layer_norm(x_sp, out=dst, with_residual=True)
    x_sp = self.self_attention.forward_sp(
        h, x_sp, batch, length, h_block=blk, bias_table=bias_table, bidirectional=False,
        num_buckets=c.relpos_num_buckets, max_distance=c.relpos_max_distance,
        key_mask=decoder_key_mask, causal=True, q_segment_ids=decoder_segment_ids,
        kv_segment_ids=decoder_segment_ids, dropout_rate=rate)
    blk, dst = tp_fused.rows_buffer(*x_sp.shape)
    x_sp, h = self.pre_cross_attention_layer_norm(x_sp, out=dst, with_residual=True)
    x_sp = self.encoder_decoder_attention.forward_sp(
        h, x_sp, batch, length, kv_full=encoded, h_block=blk, key_mask=encoder_key_mask,
        q_segment_ids=decoder_segment_ids, kv_segment_ids=encoder_segment_ids,
        dropout_rate=rate)
    blk, dst = tp_fused.rows_buffer(*x_sp.shape)
    x_sp, h = self.pre_mlp_layer_norm(x_sp, out=dst, with_residual=True)
    return self.mlp.forward_sp(h, x_sp, h_block=blk, seq_len=length, dropout_rate=rate)


class Encoder(nn.Module):
  """Embedding (shared) -> dropout -> layers -> final norm -> dropout (network.py:182-219)."""

  def __init__(self, config: T5Config, shared_embedding: nn.Module, device=None):
    super().__init__()
    c = config
    self.config = c
    self._shared = [shared_embedding]  # not registered twice
    self.relpos_bias = layers.RelativePositionBiases(c.relpos_num_buckets, c.relpos_max_distance,
                                                     c.num_heads, c.dtype, device=device)
    for i in range(c.num_encoder_layers):
      setattr(self, f"layers_{i}", EncoderLayer(c, device=device))
    self.encoder_norm = layers.LayerNorm(c.emb_dim, dtype=c.dtype, device=device)

  def forward(self, encoder_input_tokens, encoder_segment_ids=None, enable_dropout=False):
    c = self.config
    key_mask = encoder_input_tokens > 0
    x = self._shared[0](encoder_input_tokens.long())
    b, l, d = x.shape
    if tp_fused.usable(x, b * l) and _sp_dropout_ok(x, c, enable_dropout):
      # row-sharded residual stream; collectives inside the GEMM kernels
      drop = enable_dropout and c.dropout_rate > 0
      x_sp = tp_fused.scatter_rows(x.reshape(b * l, d))
      if drop:
        x_sp = layers.sp_output_dropout(x_sp, c.dropout_rate, l)
      for i in range(c.num_encoder_layers):
        x_sp = getattr(self, f"layers_{i}").forward_sp(
            x_sp, b, l, bias_table=self.relpos_bias.rel_embedding, key_mask=key_mask,
            segment_ids=encoder_segment_ids, enable_dropout=drop)
      _mark_partial(self.encoder_norm)
      y_sp = self.encoder_norm(x_sp)
      if drop:  # the mask after the final norm is not shared along the sequence
        y_sp = F.dropout(y_sp, c.dropout_rate, True,
                         row_offset=pstate.get().model_rank * y_sp.shape[0])
      return tp_fused.gather_rows(y_sp, partial_grads=True).view(b, l, d)
    x = _dropout(x, c.dropout_rate, enable_dropout)
    for i in range(c.num_encoder_layers):
      x = getattr(self, f"layers_{i}")(x, bias_table=self.relpos_bias.rel_embedding,
                                       key_mask=key_mask, segment_ids=encoder_segment_ids,
                                       enable_dropout=enable_dropout)
    x = self.encoder_norm(x)
    return _dropout(x, c.dropout_rate, enable_dropout, broadcast=False)


class Decoder(nn.Module):
  """Decoder stack + final norm + logits (network.py:222-292)."""

  def __init__(self, config: T5Config, shared_embedding: nn.Module, device=None):
    super().__init__()
    c = config
    self.config = c
    self._shared = [shared_embedding]
    self.relpos_bias = layers.RelativePositionBiases(c.relpos_num_buckets, c.relpos_max_distance,
                                                     c.num_heads, c.dtype, device=device)
    for i in range(c.num_decoder_layers):
      setattr(self, f"layers_{i}", DecoderLayer(c, device=device))
    self.decoder_norm = layers.LayerNorm(c.emb_dim, dtype=c.dtype, device=device)
    if not c.logits_via_embedding:
      self.logits_dense = layers.DenseGeneral(c.emb_dim, c.vocab_size, ("embed", "vocab"),
                                              dtype="float32", shard_dim=1, device=device)

  def init_cache(self, batch: int, max_decode_length: int, device) -> dict:
    c = self.config
    cache = {}
    for i in range(c.num_decoder_layers):
      layer = getattr(self, f"layers_{i}")
      cache[f"layers_{i}"] = {
          "self_attention": layer.self_attention.init_cache(batch, max_decode_length, device),
          "encoder_decoder_attention": {},
      }
    return cache

  def hidden(self, encoded, decoder_input_tokens, *, encoder_key_mask, decoder_key_mask=None,
             decoder_segment_ids=None, encoder_segment_ids=None, enable_dropout=False,
             decode=False, cache=None, beams_per_kv: int = 1):
    """Final-norm hidden states [batch, len, emb] (what the logits projection consumes)."""
    c = self.config
    y = self._shared[0](decoder_input_tokens.long())
    b, l, d = y.shape
    if (tp_fused.usable(y, b * l) and not decode and cache is None and
        _sp_dropout_ok(y, c, enable_dropout)):
      drop = enable_dropout and c.dropout_rate > 0
      y_sp = tp_fused.scatter_rows(y.reshape(b * l, d))
      if drop:
        y_sp = layers.sp_output_dropout(y_sp, c.dropout_rate, l)
      for i in range(c.num_decoder_layers):
        y_sp = getattr(self, f"layers_{i}").forward_sp(
            y_sp, encoded, b, l, bias_table=self.relpos_bias.rel_embedding,
            decoder_key_mask=decoder_key_mask, encoder_key_mask=encoder_key_mask,
            decoder_segment_ids=decoder_segment_ids, encoder_segment_ids=encoder_segment_ids,
            enable_dropout=drop)
      _mark_partial(self.decoder_norm)
      y_sp = self.decoder_norm(y_sp)
      if drop:
        y_sp = layers.sp_output_dropout(y_sp, c.dropout_rate, l)
      # the vocabulary-parallel loss hands back a gradient already summed over the model axis
      return tp_fused.gather_rows(y_sp, partial_grads=False).view(b, l, d)
    y = _dropout(y, c.dropout_rate, enable_dropout)
    for i in range(c.num_decoder_layers):
      y = getattr(self, f"layers_{i}")(
          y, encoded, bias_table=self.relpos_bias.rel_embedding,
          decoder_key_mask=decoder_key_mask, encoder_key_mask=encoder_key_mask,
          decoder_segment_ids=decoder_segment_ids, encoder_segment_ids=encoder_segment_ids,
          enable_dropout=enable_dropout, decode=decode,
          cache=None if cache is None else cache[f"layers_{i}"], beams_per_kv=beams_per_kv)
    y = self.decoder_norm(y)
    return _dropout(y, c.dropout_rate, enable_dropout)

  def logits_weight_and_scale(self):
    """(weight, scale): logits = scale * hidden @ weight (weight [emb, vocab] or tied [vocab, emb])."""
    c = self.config
    if c.logits_via_embedding:
      return self._shared[0].embedding, 1.0 / math.sqrt(c.emb_dim)
    return self.logits_dense.kernel, 1.0

  def logits(self, hidden: torch.Tensor) -> torch.Tensor:
    """float32 logits (network.py:279-291). Under tensor parallelism the local vocab slices
    are gathered so callers always see the full vocabulary."""
    w, scale = self.logits_weight_and_scale()
    wf = F.compute_weight(w, torch.bfloat16 if hidden.dtype == torch.bfloat16 else torch.float32)
    if w.shape[0] != hidden.shape[-1]:
      wf = wf.t()
    if hidden.is_cuda and hidden.dtype == torch.bfloat16:
      from t5x_b200.ops import native
      out = native.gemm(hidden.reshape(-1, hidden.shape[-1]), wf, out_dtype=torch.float32,
                        alpha=scale).view(*hidden.shape[:-1], wf.shape[1])
    else:
      out = (hidden.float() @ wf.float()) * scale
    st = pstate.get()
    if st.model_size > 1 and getattr(w, "shard_dim", None) is not None:
      import torch.distributed as dist
      parts = [torch.empty_like(out) for _ in range(st.model_size)]
      dist.all_gather(parts, out.contiguous(), group=st.model_group)
      out = torch.cat(parts, dim=-1)
    return out

  def forward(self, encoded, decoder_input_tokens, **kwargs):
    return self.logits(self.hidden(encoded, decoder_input_tokens, **kwargs))


class Transformer(nn.Module):
  """Encoder-decoder with a shared token embedding (network.py:295-461)."""

  def __init__(self, config: T5Config, device=None):
    super().__init__()
    self.config = config
    c = config
    self.token_embedder = layers.Embed(c.vocab_size, c.emb_dim, c.dtype, device=device)
    self.encoder = Encoder(c, self.token_embedder, device=device)
    self.decoder = Decoder(c, self.token_embedder, device=device)

  scan_layers = False

  def encode(self, encoder_input_tokens, encoder_segment_ids=None, enable_dropout=True):
    return self.encoder(encoder_input_tokens, encoder_segment_ids, enable_dropout)

  def decode_hidden(self, encoded, encoder_input_tokens, decoder_input_tokens,
                    decoder_target_tokens, encoder_segment_ids=None, decoder_segment_ids=None,
                    decoder_positions=None, enable_dropout=True, decode=False,
                    max_decode_length=None, cache=None, beams_per_kv: int = 1):
    encoder_key_mask = encoder_input_tokens > 0
    decoder_key_mask = None if decode else (decoder_target_tokens > 0)
    return self.decoder.hidden(
        encoded, decoder_input_tokens, encoder_key_mask=encoder_key_mask,
        decoder_key_mask=decoder_key_mask, decoder_segment_ids=decoder_segment_ids,
        encoder_segment_ids=encoder_segment_ids, enable_dropout=enable_dropout, decode=decode,
        cache=cache, beams_per_kv=beams_per_kv)

  def decode(self, encoded, encoder_input_tokens, decoder_input_tokens, decoder_target_tokens,
             **kwargs):
    return self.decoder.logits(
        self.decode_hidden(encoded, encoder_input_tokens, decoder_input_tokens,
                           decoder_target_tokens, **kwargs))

  def forward(self, encoder_input_tokens, decoder_input_tokens, decoder_target_tokens,
              encoder_segment_ids=None, decoder_segment_ids=None, encoder_positions=None,
              decoder_positions=None, *, enable_dropout: bool = True, decode: bool = False,
              return_hidden: bool = False):
    encoded = self.encode(encoder_input_tokens, encoder_segment_ids, enable_dropout)
    hidden = self.decode_hidden(encoded, encoder_input_tokens, decoder_input_tokens,
                                decoder_target_tokens, encoder_segment_ids=encoder_segment_ids,
                                decoder_segment_ids=decoder_segment_ids,
                                enable_dropout=enable_dropout, decode=decode)
    if return_hidden:
      return hidden
    return self.decoder.logits(hidden)

  def init_cache(self, batch: int, max_decode_length: int, device=None):
    device = device or next(self.parameters()).device
    return self.decoder.init_cache(batch, max_decode_length, device)
