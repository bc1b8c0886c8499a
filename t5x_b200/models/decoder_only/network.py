"""Decoder-only Transformer (language model / prefix LM): one stack of self-attention + MLP
blocks with a relative-position bias shared by all layers
(t5x/examples/decoder_only/network.py:28-270).

Parameter tree: `decoder/{token_embedder, relpos_bias, layers_N/{pre_self_attention_layer_norm,
self_attention/{query,key,value,out}, pre_mlp_layer_norm, mlp/{wi[_0,_1],wo}}, decoder_norm,
logits_dense}`.

The padding / causal / packing structure is handed to the attention op as per-token metadata
(key-valid bits, a causal flag, segment ids); only the prefix-LM case, whose visible set is
"causal OR both-in-prefix", builds an explicit mask.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any, Optional, Sequence

import torch
from torch import nn

from t5x_b200.models.t5 import layers
from t5x_b200.models.t5.network import _dropout
from t5x_b200.ops import functional as F
from t5x_b200.ops import reference as ref
from t5x_b200.parallel import state as pstate


@dataclasses.dataclass
class TransformerConfig:
  """Hyper-parameters (t5x/examples/decoder_only/network.py:28-46)."""
  vocab_size: int
  dtype: Any = "float32"
  emb_dim: int = 512
  num_heads: int = 8
  num_layers: int = 6
  head_dim: int = 64
  mlp_dim: int = 2048
  mlp_activations: Sequence[str] = ("relu",)
  dropout_rate: float = 0.1
  logits_via_embedding: bool = False
  relpos_num_buckets: int = 32
  relpos_max_distance: int = 128
  float32_attention_logits: bool = False
  scale_attn_logits: bool = False


class DecoderLayer(nn.Module):
  """pre-LN -> causal self-attention -> dropout -> +res -> pre-LN -> MLP -> dropout -> +res."""

  def __init__(self, config: TransformerConfig, device=None):
    super().__init__()
    c = config
    self.config = c
    self.pre_self_attention_layer_norm = layers.LayerNorm(c.emb_dim, dtype=c.dtype, device=device)
    self.self_attention = layers.MultiHeadDotProductAttention(
        c.emb_dim, c.num_heads, c.head_dim, c.dtype, c.dropout_rate, c.float32_attention_logits,
        c.scale_attn_logits, device=device)
    self.pre_mlp_layer_norm = layers.LayerNorm(c.emb_dim, dtype=c.dtype, device=device)
    self.mlp = layers.MlpBlock(c.emb_dim, c.mlp_dim, c.mlp_activations, c.dropout_rate, c.dtype,
                               device=device)

  def forward(self, x, *, bias_table, key_mask=None, causal=True, segment_ids=None,
              extra_mask=None, enable_dropout=False, decode=False, prefill=False,
              prefill_lengths=None, cache: Optional[dict] = None):
    c = self.config
    drop = enable_dropout and c.dropout_rate > 0
    h = self.pre_self_attention_layer_norm(x)
    kw = dict(bias_table=bias_table, bidirectional=False, num_buckets=c.relpos_num_buckets,
              max_distance=c.relpos_max_distance)
    if decode and not prefill:
      x = x + self.self_attention(h, h, cache=cache, decode=True, **kw)
    else:
      kw.update(key_mask=key_mask, causal=causal, q_segment_ids=segment_ids,
                kv_segment_ids=segment_ids, extra_mask=extra_mask)
      if prefill:
        kw.update(cache=cache, prefill=True, prefill_lengths=prefill_lengths)
      if drop:
        a = self.self_attention(h, h, enable_dropout=True, **kw)
        x = x + _dropout(a, c.dropout_rate, True)
      else:
        x = self.self_attention(h, h, residual=x, **kw)
    h = self.pre_mlp_layer_norm(x)
    if drop:
      return x + _dropout(self.mlp(h, enable_dropout=True), c.dropout_rate, True)
    return self.mlp(h, residual=x)


class Decoder(nn.Module):
  """Token embedding -> layers -> final norm -> logits (network.py:104-257)."""

  def __init__(self, config: TransformerConfig, device=None):
    super().__init__()
    c = config
    self.config = c
    self.token_embedder = layers.Embed(c.vocab_size, c.emb_dim, c.dtype, device=device)
    self.relpos_bias = layers.RelativePositionBiases(
        c.relpos_num_buckets, c.relpos_max_distance, c.num_heads, c.dtype, device=device)
    for i in range(c.num_layers):
      setattr(self, f"layers_{i}", DecoderLayer(c, device=device))
    self.decoder_norm = layers.LayerNorm(c.emb_dim, dtype=c.dtype, device=device)
    if not c.logits_via_embedding:
      self.logits_dense = layers.DenseGeneral(c.emb_dim, c.vocab_size, ("embed", "vocab"),
                                              dtype="float32", shard_dim=1, device=device)

  def init_cache(self, batch: int, max_decode_length: int, device=None) -> dict:
    device = device or self.token_embedder.embedding.device
    return {f"layers_{i}": getattr(self, f"layers_{i}").self_attention.init_cache(
        batch, max_decode_length, device) for i in range(self.config.num_layers)}

  @staticmethod
  def _prefix_lm_mask(decoder_target_tokens, decoder_causal_attention, decoder_segment_ids):
    """Prefix-LM visibility: causal, or both positions inside the prefix; restricted to
    non-padding positions of the same packed segment (the semantics of
    layers.make_decoder_mask, t5x/examples/t5/layers.py:842-924), in factored form."""
    return ref.PrefixLMMask(decoder_causal_attention > 0, decoder_target_tokens > 0,
                            decoder_segment_ids)

  def hidden(self, decoder_input_tokens, decoder_target_tokens, decoder_segment_ids=None,
             decoder_positions=None, decoder_causal_attention=None, *, enable_dropout=True,
             decode=False, max_decode_length=None, prefill=False, prefill_lengths=None,
             cache: Optional[dict] = None):
    c = self.config
    assert decoder_input_tokens.dim() == 2
    key_mask = extra_mask = None
    causal = True
    if not decode or prefill:
      if decoder_causal_attention is not None:
        extra_mask = self._prefix_lm_mask(decoder_target_tokens, decoder_causal_attention,
                                          decoder_segment_ids)
        causal = False
      else:
        key_mask = decoder_target_tokens > 0
    y = self.token_embedder(decoder_input_tokens.long())
    y = _dropout(y, c.dropout_rate, enable_dropout)
    for i in range(c.num_layers):
      y = getattr(self, f"layers_{i}")(
          y, bias_table=self.relpos_bias.rel_embedding, key_mask=key_mask, causal=causal,
          segment_ids=None if extra_mask is not None else decoder_segment_ids,
          extra_mask=extra_mask, enable_dropout=enable_dropout, decode=decode, prefill=prefill,
          prefill_lengths=prefill_lengths,
          cache=None if cache is None else cache[f"layers_{i}"])
    y = self.decoder_norm(y)
    return _dropout(y, c.dropout_rate, enable_dropout)

  def logits_weight_and_scale(self):
    c = self.config
    if c.logits_via_embedding:
      return self.token_embedder.embedding, 1.0 / math.sqrt(c.emb_dim)
    return self.logits_dense.kernel, 1.0

  def logits(self, hidden: torch.Tensor) -> torch.Tensor:
    """float32 logits over the full vocabulary (local slices are gathered under TP)."""
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

  def forward(self, decoder_input_tokens, decoder_target_tokens, decoder_segment_ids=None,
              decoder_positions=None, decoder_causal_attention=None, *, return_hidden=False,
              **kwargs):
    h = self.hidden(decoder_input_tokens, decoder_target_tokens, decoder_segment_ids,
                    decoder_positions, decoder_causal_attention, **kwargs)
    return h if return_hidden else self.logits(h)


class DecoderWrapper(nn.Module):
  """Outer `decoder/` name scope (network.py:260-270)."""

  scan_layers = False

  def __init__(self, config: TransformerConfig, device=None):
    super().__init__()
    self.config = config
    self.decoder = Decoder(config, device=device)

  def init_cache(self, batch: int, max_decode_length: int, device=None):
    return self.decoder.init_cache(batch, max_decode_length, device)

  def forward(self, *args, **kwargs):
    return self.decoder(*args, **kwargs)
