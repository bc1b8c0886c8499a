"""Temperature sampling that records, per generated token, how many decoder layers ran and
how confident the model was when it stopped (role of t5x/contrib/calm/decoding.py:70-683).

`tokens_to_logits(state)` returns `(logits, cache, confidence, layers_used)` here, the last
two per row ([batch * num_decodes]) or scalars. The sampling itself (prompts, top-k / top-p,
EOS handling, per-example start positions) is the shared loop of `t5x_b200.decoding`; this
wrapper adds the two records and orders them like the returned sequences.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple, Union

import torch

from t5x_b200 import decoding

DecodingState = decoding.DecodingState
SamplingLoopState = decoding.SamplingLoopState


def temperature_sample(inputs: torch.Tensor, cache, tokens_to_logits: Callable, eos_id: int,
                       decode_rng=None, num_decodes: int = 1,
                       temperature: Union[float, torch.Tensor] = 1.0, topk: int = 1,
                       topp: float = 0.0, cache_offset: int = 0,
                       initial_index: Optional[torch.Tensor] = None,
                       max_decode_steps: Optional[Union[int, torch.Tensor]] = None,
                       max_decode_steps_hard_limit: Optional[int] = None,
                       rescale_log_probs: bool = True,
                       state_callback_fn: Optional[Callable] = None,
                       logit_callback_fn: Optional[Callable] = None
                       ) -> Tuple[torch.Tensor, Tuple[torch.Tensor, torch.Tensor, torch.Tensor]]:
  """Returns `(decodes, (log_probs, exits, confidences))`: decodes [batch, num_decodes, len]
  sorted ascending by log-probability, log_probs [batch, num_decodes], and for every position
  the number of decoder layers used (`exits`, int32) and the confidence at the exit
  (`confidences`, float32), both [batch, num_decodes, len] in the same order."""
  device = inputs.device
  batch_size, seq_len = inputs.shape
  rows = batch_size * num_decodes
  exits = torch.zeros((rows, seq_len), dtype=torch.int32, device=device)
  confidences = torch.zeros((rows, seq_len), dtype=torch.float32, device=device)

  def recording(state: DecodingState):
    logits, new_cache, conf, layer = tokens_to_logits(state)
    idx = state.cur_index
    if not isinstance(idx, torch.Tensor):
      idx = torch.full((rows,), int(idx), dtype=torch.int64, device=device)
    idx = idx.long().clamp(max=seq_len - 1)[:, None]
    conf_t = torch.as_tensor(conf, dtype=torch.float32, device=device).reshape(-1)
    layer_t = torch.as_tensor(layer, dtype=torch.int32, device=device).reshape(-1)
    confidences.scatter_(1, idx, conf_t.expand(rows)[:, None])
    exits.scatter_(1, idx, layer_t.expand(rows)[:, None])
    return logits, new_cache

  gen = decoding._make_generator(decode_rng, device)
  if (max_decode_steps_hard_limit is not None and max_decode_steps_hard_limit > 0 and
      max_decode_steps is not None):
    if isinstance(max_decode_steps, torch.Tensor):
      max_decode_steps = torch.clamp(max_decode_steps, max=max_decode_steps_hard_limit)
    else:
      max_decode_steps = min(max_decode_steps, max_decode_steps_hard_limit)
  if num_decodes > 1:
    expanded_inputs = decoding.flat_batch_beam_expand(inputs, num_decodes)
    expanded_cache = decoding.cache_map(
        lambda x: decoding.flat_batch_beam_expand(x, num_decodes, cache_offset).contiguous(),
        cache, apply_to_index=initial_index is not None)
    if initial_index is not None:
      initial_index = decoding.flat_batch_beam_expand(initial_index, num_decodes)
  else:
    expanded_inputs, expanded_cache = inputs, cache
  decodes, log_prob = decoding._temperature_sample_single_trial(
      expanded_inputs, expanded_cache, recording, eos_id, gen, num_decodes, temperature, topk,
      topp, initial_index=initial_index, max_decode_steps=max_decode_steps,
      rescale_log_probs=rescale_log_probs, state_callback_fn=state_callback_fn,
      logit_callback_fn=logit_callback_fn)
  unflat = lambda x: decoding.unflatten_beam_dim(x, batch_size, num_decodes)
  decodes, log_prob = unflat(decodes), unflat(log_prob)
  exits_b, conf_b = unflat(exits), unflat(confidences)
  order = torch.argsort(log_prob, dim=-1, stable=True)
  pick = lambda x: torch.gather(x, 1, order[:, :, None].expand_as(x))
  return pick(decodes), (torch.gather(log_prob, 1, order), pick(exits_b), pick(conf_b))
