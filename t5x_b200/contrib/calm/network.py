"""T5 network with the hooks early-exit decoding needs.

The reference's CALM wrappers drive an external architecture through
`decode(start_idx, end_idx, return_prelogits, only_propagate_state, decoder_embedded_input)`
and `compute_logits` (t5x/contrib/calm/models.py:539-856). This module provides that
architecture on top of the T5 stack of `t5x_b200.models.t5.network`:

  * training can return the logits after every decoder layer (`return_all_logits`), each
    taken through the shared final norm and output projection;
  * a decode step can run any contiguous range of decoder layers on top of a given hidden
    state, or only write that state's keys / values into the caches of skipped layers, so
    that later tokens that do reach those layers can attend to this position;
  * an optional two-class "meta" head on the hidden state scores whether to exit.
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch

from t5x_b200.models.t5 import layers
from t5x_b200.models.t5 import network


@dataclasses.dataclass
class CalmT5Config(network.T5Config):
  return_all_logits: bool = False
  meta_cls: bool = False


class Transformer(network.Transformer):
  """Encoder-decoder whose decoder can be run layer range by layer range."""

  def __init__(self, config: CalmT5Config, device=None):
    super().__init__(config, device=device)
    if config.meta_cls:
      self.decoder.meta_cls = layers.DenseGeneral(config.emb_dim, 2, ("embed", "meta"),
                                                  dtype=config.dtype, device=device)

  # -- heads -------------------------------------------------------------------------------
  def compute_logits(self, hidden: torch.Tensor, logit_mask=None, enable_dropout: bool = False):
    """Final norm + output projection of a pre-norm hidden state [batch, len, emb]; with the
    meta head, (logits, meta_logits)."""
    dec = self.decoder
    normed = dec.decoder_norm(hidden)
    logits = dec.logits(normed)
    if logit_mask is not None:
      logits = logits * logit_mask
    if self.config.meta_cls:
      return logits, dec.meta_cls(normed).float()
    return logits

  # -- decoder -----------------------------------------------------------------------------
  def _embed(self, decoder_input_tokens):
    return self.decoder._shared[0](decoder_input_tokens.long())

  def _layer(self, i: int):
    return getattr(self.decoder, f"layers_{i}")

  def decode(self, encoded, encoder_input_tokens, decoder_input_tokens, decoder_target_tokens,
             encoder_segment_ids=None, decoder_segment_ids=None, decoder_positions=None,
             enable_dropout: bool = False, decode: bool = False, max_decode_length=None,
             cache=None, start_idx: int = 0, end_idx: Optional[int] = None,
             decoder_embedded_input: Optional[torch.Tensor] = None,
             return_prelogits: bool = False, only_propagate_state: bool = False,
             beams_per_kv: int = 1, **_):
    """Decoder layers [start_idx, end_idx).

    Training (`decode=False`): all layers; returns final logits, or the stacked per-layer
    logits [layers, batch, len, vocab] (and meta logits) under `return_all_logits`.
    Decoding: starts from `decoder_embedded_input` (the hidden state after layer
    `start_idx - 1`) when `start_idx > 0`; returns the pre-norm hidden state
    (`return_prelogits`) or the logits. `only_propagate_state` writes the hidden state's
    keys / values into the self-attention caches of the layers in range without running them."""
    c = self.config
    dec = self.decoder
    n = c.num_decoder_layers
    end_idx = n if end_idx is None else end_idx
    encoder_key_mask = encoder_input_tokens > 0
    y = decoder_embedded_input if start_idx > 0 else self._embed(decoder_input_tokens)
    if not decode:
      decoder_key_mask = decoder_target_tokens > 0
      outs = []
      for i in range(n):
        y = self._layer(i)(y, encoded, bias_table=dec.relpos_bias.rel_embedding,
                           decoder_key_mask=decoder_key_mask, encoder_key_mask=encoder_key_mask,
                           decoder_segment_ids=decoder_segment_ids,
                           encoder_segment_ids=encoder_segment_ids,
                           enable_dropout=enable_dropout)
        if c.return_all_logits:
          outs.append(self.compute_logits(y))
      if not c.return_all_logits:
        return self.compute_logits(y)
      if c.meta_cls:
        return torch.stack([o[0] for o in outs]), torch.stack([o[1] for o in outs])
      return torch.stack(outs)
    for i in range(start_idx, end_idx):
      layer = self._layer(i)
      if only_propagate_state:
        _write_state(layer, y, cache[f"layers_{i}"]["self_attention"])
      else:
        y = layer(y, encoded, bias_table=dec.relpos_bias.rel_embedding, decoder_key_mask=None,
                  encoder_key_mask=encoder_key_mask, decode=True, cache=cache[f"layers_{i}"],
                  beams_per_kv=beams_per_kv)
    if return_prelogits or only_propagate_state:
      return y
    return self.compute_logits(y)

  def forward(self, encoder_input_tokens, decoder_input_tokens, decoder_target_tokens,
              encoder_segment_ids=None, decoder_segment_ids=None, encoder_positions=None,
              decoder_positions=None, *, enable_dropout: bool = True, decode: bool = False,
              return_hidden: bool = False, **kwargs):
    if return_hidden:
      return super().forward(encoder_input_tokens, decoder_input_tokens, decoder_target_tokens,
                             encoder_segment_ids, decoder_segment_ids, encoder_positions,
                             decoder_positions, enable_dropout=enable_dropout, decode=decode,
                             return_hidden=True)
    encoded = self.encode(encoder_input_tokens, encoder_segment_ids, enable_dropout)
    return self.decode(encoded, encoder_input_tokens, decoder_input_tokens,
                       decoder_target_tokens, encoder_segment_ids=encoder_segment_ids,
                       decoder_segment_ids=decoder_segment_ids, enable_dropout=enable_dropout,
                       decode=decode, **kwargs)


def _write_state(layer, hidden: torch.Tensor, cache: dict) -> None:
  """Stores the keys / values that `layer`'s self-attention would compute for `hidden`
  ([rows, 1, emb]) at the cache's current position and advances the position."""
  attn = layer.self_attention
  h = layer.pre_self_attention_layer_norm(hidden)
  k, v = attn.project_kv(h)
  idx = cache["cache_index"]
  max_len = cache["cached_key"].shape[1]
  if idx.dim() == 0:
    i = int(idx)
    if i < max_len:
      cache["cached_key"][:, i] = k[:, 0]
      cache["cached_value"][:, i] = v[:, 0]
  else:
    rows = torch.arange(k.shape[0], device=k.device)
    il = idx.long()
    inb = (il < max_len)[:, None, None]
    ic = il.clamp(max=max_len - 1)
    cache["cached_key"][rows, ic] = torch.where(inb, k[:, 0], cache["cached_key"][rows, ic])
    cache["cached_value"][rows, ic] = torch.where(inb, v[:, 0], cache["cached_value"][rows, ic])
  cache["cache_index"] = idx + 1
