"""Scalable T5 (t5x/examples/scalable_t5/network.py): T5.1.1 with a relative-position bias per
layer, optional rematerialisation, and a "scanned" checkpoint layout in which the parameters of
all layers are stacked along a `layers` axis.

The reference scans over layers to keep XLA compile time flat; nothing is traced here, so the
layers always run as ordinary modules (`layers_0 ... layers_{N-1}`), each with kernels the GEMM
consumes directly. Training dynamics are the same either way: the reference's factor rules
treat the `layers` axis as a batch dimension, i.e. every layer is updated independently. What
remains of `scan_layers` is the checkpoint layout, provided by `stack_layers` /
`unstack_layers` (usable as checkpoint state-transformation functions):

  unscanned:  encoder/layers_3/attention/query/kernel          [embed, heads * kv]
  scanned:    encoder/encoder/attention/query/kernel           [embed, layers, heads, kv]

`remat_policy`: 'none' keeps activations; 'full' re-runs each layer in backward
(`torch.utils.checkpoint`); 'minimal' (keep matmul outputs, recompute the rest) is what the fused
ops already do, since they never store element-wise intermediates, so it equals 'none'.
"""
from __future__ import annotations

import dataclasses
import re
from typing import Any, Mapping, Optional, Sequence

import torch
import torch.utils.checkpoint
from torch import nn

from t5x_b200.models.t5 import layers
from t5x_b200.models.t5 import network as t5_network
from t5x_b200.models.t5.network import _dropout


@dataclasses.dataclass
class T5Config(t5_network.T5Config):
  """t5x/examples/scalable_t5/network.py:31-53."""
  remat_policy: str = "none"   # 'none' | 'minimal' | 'full'
  scan_layers: bool = True
  param_scan_axis: int = 1


def _maybe_remat(fn, policy: str, training: bool):
  if policy == "full" and training and torch.is_grad_enabled():
    from t5x_b200.ops import reference as ref

    def rematerialised(*a, **kw):
      # The recomputation in backward must draw the dropout masks of the first pass: every
      # dropout call is numbered, so the block remembers the number it started at and the
      # second pass counts from there again (and leaves the counter where it found it).
      first_site = ref.dropout_site_state()
      passes = [0]

      def block(*ba, **bkw):
        passes[0] += 1
        if passes[0] == 1:
          return fn(*ba, **bkw)
        resume = ref.dropout_site_state()
        ref.set_dropout_site_state(first_site)
        try:
          return fn(*ba, **bkw)
        finally:
          ref.set_dropout_site_state(resume)

      return torch.utils.checkpoint.checkpoint(block, *a, use_reentrant=False, **kw)

    return rematerialised
  if policy not in (None, "none", "minimal", "full"):
    raise ValueError(f"unknown remat_policy {policy!r}")
  return fn


class EncoderLayer(t5_network.EncoderLayer):
  """Encoder layer that owns its relative-position bias."""

  def __init__(self, config: T5Config, device=None):
    super().__init__(config, device=device)
    c = config
    self.relpos_bias = layers.RelativePositionBiases(c.relpos_num_buckets, c.relpos_max_distance,
                                                     c.num_heads, c.dtype, device=device)

  def forward(self, x, *, key_mask, segment_ids=None, enable_dropout=False, bias_table=None):
    return super().forward(x, bias_table=self.relpos_bias.rel_embedding, key_mask=key_mask,
                           segment_ids=segment_ids, enable_dropout=enable_dropout)


class DecoderLayer(t5_network.DecoderLayer):
  """Decoder layer that owns its relative-position bias."""

  def __init__(self, config: T5Config, device=None):
    super().__init__(config, device=device)
    c = config
    self.relpos_bias = layers.RelativePositionBiases(c.relpos_num_buckets, c.relpos_max_distance,
                                                     c.num_heads, c.dtype, device=device)

  def forward(self, x, encoded, *, bias_table=None, **kwargs):
    return super().forward(x, encoded, bias_table=self.relpos_bias.rel_embedding, **kwargs)


class Encoder(nn.Module):

  def __init__(self, config: T5Config, shared_embedding: nn.Module, device=None):
    super().__init__()
    c = config
    self.config = c
    self._shared = [shared_embedding]
    for i in range(c.num_encoder_layers):
      setattr(self, f"layers_{i}", EncoderLayer(c, device=device))
    self.encoder_norm = layers.LayerNorm(c.emb_dim, dtype=c.dtype, device=device)

  def forward(self, encoder_input_tokens, encoder_segment_ids=None, enable_dropout=False):
    c = self.config
    key_mask = encoder_input_tokens > 0
    x = self._shared[0](encoder_input_tokens.long())
    x = _dropout(x, c.dropout_rate, enable_dropout)
    for i in range(c.num_encoder_layers):
      layer = getattr(self, f"layers_{i}")
      run = _maybe_remat(
          lambda x_, layer=layer: layer(x_, key_mask=key_mask, segment_ids=encoder_segment_ids,
                                        enable_dropout=enable_dropout),
          c.remat_policy, x.requires_grad or enable_dropout)
      x = run(x)
    x = self.encoder_norm(x)
    return _dropout(x, c.dropout_rate, enable_dropout, broadcast=False)


class Decoder(t5_network.Decoder):

  def __init__(self, config: T5Config, shared_embedding: nn.Module, device=None):
    nn.Module.__init__(self)
    c = config
    self.config = c
    self._shared = [shared_embedding]
    for i in range(c.num_decoder_layers):
      setattr(self, f"layers_{i}", DecoderLayer(c, device=device))
    self.decoder_norm = layers.LayerNorm(c.emb_dim, dtype=c.dtype, device=device)
    if not c.logits_via_embedding:
      self.logits_dense = layers.DenseGeneral(c.emb_dim, c.vocab_size, ("embed", "vocab"),
                                              dtype="float32", shard_dim=1, device=device)

  def hidden(self, encoded, decoder_input_tokens, *, encoder_key_mask, decoder_key_mask=None,
             decoder_segment_ids=None, encoder_segment_ids=None, enable_dropout=False,
             decode=False, cache=None, beams_per_kv: int = 1):
    c = self.config
    y = self._shared[0](decoder_input_tokens.long())
    y = _dropout(y, c.dropout_rate, enable_dropout)
    for i in range(c.num_decoder_layers):
      layer = getattr(self, f"layers_{i}")
      layer_cache = None if cache is None else cache[f"layers_{i}"]

      def body(y_, layer=layer, layer_cache=layer_cache):
        return layer(y_, encoded, decoder_key_mask=decoder_key_mask,
                     encoder_key_mask=encoder_key_mask, decoder_segment_ids=decoder_segment_ids,
                     encoder_segment_ids=encoder_segment_ids, enable_dropout=enable_dropout,
                     decode=decode, cache=layer_cache, beams_per_kv=beams_per_kv)

      run = body if decode else _maybe_remat(body, c.remat_policy,
                                             y.requires_grad or enable_dropout)
      y = run(y)
    y = self.decoder_norm(y)
    return _dropout(y, c.dropout_rate, enable_dropout)


class Transformer(t5_network.Transformer):
  """Encoder-decoder with per-layer position biases (network.py:388-520)."""

  def __init__(self, config: T5Config, device=None):
    nn.Module.__init__(self)
    self.config = config
    c = config
    self.token_embedder = layers.Embed(c.vocab_size, c.emb_dim, c.dtype, device=device)
    self.encoder = Encoder(c, self.token_embedder, device=device)
    self.decoder = Decoder(c, self.token_embedder, device=device)

  # The run-time layout is always per layer; `cache_offset` logic keyed on this flag in the
  # model wrappers therefore sees False.
  scan_layers = False


# ----------------------------------------------------------------------------
# Scanned <-> per-layer checkpoint layout
# ----------------------------------------------------------------------------
_LAYER_RE = re.compile(r"^layers_(\d+)$")
_ATTN_KERNELS = {"query": "in", "key": "in", "value": "in", "out": "out"}


def _reshape_attn(name_path, value, heads: int, kv: int, to_3d: bool):
  """[embed, heads*kv] <-> [embed, heads, kv] (and [heads*kv, embed] <-> [heads, kv, embed])."""
  if isinstance(name_path, str):
    name_path = tuple(name_path.split("/"))
  if len(name_path) < 3 or name_path[-1] != "kernel" or name_path[-2] not in _ATTN_KERNELS:
    return value
  if not any(part.endswith("attention") for part in name_path):
    return value
  kind = _ATTN_KERNELS[name_path[-2]]
  if to_3d:
    return value.reshape(value.shape[0], heads, kv) if kind == "in" else \
        value.reshape(heads, kv, value.shape[-1])
  return value.reshape(value.shape[0], heads * kv) if kind == "in" else \
      value.reshape(heads * kv, value.shape[-1])


def stack_layers(params: Mapping[str, Any], num_heads: int, head_dim: int, scan_axis: int = 1):
  """Per-layer parameter tree -> the scanned layout of the reference: `encoder/layers_i/...`
  become `encoder/encoder/...` with a new `layers` axis at `scan_axis` (a norm scale [embed]
  becomes [embed, layers] for axis 1), attention kernels become 3-D. Works on numpy arrays or
  tensors (anything with reshape and stackable by torch/numpy)."""
  import numpy as np

  def stack(values, ndim):
    axis = min(scan_axis, ndim)
    if isinstance(values[0], torch.Tensor):
      return torch.stack(values, dim=axis)
    return np.stack([np.asarray(v) for v in values], axis=axis)

  out = {}
  for side in params:
    sub = params[side]
    if side not in ("encoder", "decoder") or not isinstance(sub, Mapping):
      out[side] = sub
      continue
    layer_ids = sorted(int(_LAYER_RE.match(k).group(1)) for k in sub if _LAYER_RE.match(k))
    new = {k: v for k, v in sub.items() if not _LAYER_RE.match(k)}
    if layer_ids:
      from t5x_b200.utils import tree as tree_utils
      flats = [tree_utils.flatten_dict(sub[f"layers_{i}"]) for i in layer_ids]
      stacked = {}
      for path in flats[0]:
        vals = [_reshape_attn(path, f[path], num_heads, head_dim, True) for f in flats]
        stacked[path] = stack(vals, vals[0].ndim)
      new[side] = tree_utils.unflatten_dict(stacked)
    out[side] = new
  return out


def unstack_layers(params: Mapping[str, Any], num_heads: int, head_dim: int, scan_axis: int = 1):
  """Inverse of `stack_layers`."""
  from t5x_b200.utils import tree as tree_utils
  out = {}
  for side in params:
    sub = params[side]
    if side not in ("encoder", "decoder") or not isinstance(sub, Mapping) or side not in sub:
      out[side] = sub
      continue
    new = {k: v for k, v in sub.items() if k != side}
    flat = tree_utils.flatten_dict(sub[side])
    n_layers = None
    per_layer = {}
    for path, v in flat.items():
      axis = min(scan_axis, v.ndim - 1)
      n_layers = v.shape[axis]
      for i in range(n_layers):
        piece = v.select(axis, i) if isinstance(v, torch.Tensor) else v.take(i, axis=axis)
        per_layer.setdefault(i, {})[path] = _reshape_attn(path, piece, num_heads, head_dim, False)
    for i, fl in per_layer.items():
      new[f"layers_{i}"] = tree_utils.unflatten_dict(fl)
    out[side] = new
  return out
