"""Fast decoding routines: beam search and temperature sampling (API of t5x/decoding.py).

Semantics follow the reference: sequences carry a dummy BOS at position 0, live log-probs
start as [0, -1e7, ...], each step keeps 2*beam candidates of beam*vocab (lowest flat index
wins ties), finished beams are ranked by log-prob / ((5+len)/6)^alpha, forced prompt
decoding, and results come back sorted ascending so index -1 is the best.

The loops are host-driven PyTorch: every tensor op runs on the device, and the only
device->host read per step is the termination flag (optionally every k-th step).
The KV cache is a nested dict of tensors whose leading dim is batch*beam; leaves named
`cache_index`, `cached_bias`, `position_embedder_index`, `cross_key`, `cross_value` are not
expanded or gathered per beam (cross-attention K/V are shared by the beams of an example).
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Mapping, Optional, Tuple, Union

import numpy as np
import torch

from t5x_b200 import binary_search

PyTree = Any

# Constants
NEG_INF = -1.0e7          # effective negative infinity
NEG_INF_VALUE = NEG_INF
MIN_TEMPERATURE = 1e-4    # below this, sampling is greedy

_CACHE_SKIP = ("cache_index", "cached_bias", "position_embedder_index", "cross_key",
               "cross_value")


@dataclasses.dataclass
class DecodingState:
  """What `tokens_to_logits` receives (t5x/decoding.py:42-66)."""
  cur_index: Any        # scalar or [batch] int: index of cur_token in `sequences`
  sequences: torch.Tensor  # [batch*beam, length]
  cur_token: torch.Tensor  # [batch*beam, 1]
  cache: PyTree


@dataclasses.dataclass
class SamplingLoopState:
  """State visible to temperature-sampling callbacks (t5x/decoding.py:75-99)."""
  step: int
  cur_index: torch.Tensor
  sequences: torch.Tensor
  cache: PyTree
  cur_token: torch.Tensor
  ended: torch.Tensor
  rng: Optional[torch.Generator]
  log_prob: torch.Tensor

  def replace(self, **kw):
    return dataclasses.replace(self, **kw)


# ----------------------------------------------------------------------------
# Beam-dimension helpers
# ----------------------------------------------------------------------------
def brevity_penalty(alpha: float, length) -> Any:
  """((5 + length) / 6) ** alpha (t5x/decoding.py:723-733)."""
  if isinstance(length, torch.Tensor):
    return torch.pow((5.0 + length.float()) / 6.0, alpha)
  return ((5.0 + float(length)) / 6.0) ** alpha


def cache_map(fn, cache, apply_to_index: bool = False):
  """Maps `fn` over cache tensors, skipping per-example / shared leaves
  (t5x/decoding.py:739-770)."""
  def rec(node):
    if isinstance(node, Mapping):
      out = {}
      for k, v in node.items():
        if isinstance(v, Mapping):
          out[k] = rec(v)
        elif k in _CACHE_SKIP and not (apply_to_index and k == "cache_index" and
                                       isinstance(v, torch.Tensor) and v.dim() > 0):
          out[k] = v
        else:
          out[k] = fn(v)
      return out
    return fn(node)
  return rec(cache)


def add_beam_dim(x: torch.Tensor, beam_size: int, offset: int = 0) -> torch.Tensor:
  x = x.unsqueeze(offset + 1)
  shape = list(x.shape)
  shape[offset + 1] = beam_size
  return x.expand(shape)


def flatten_beam_dim(x: torch.Tensor, offset: int = 0) -> torch.Tensor:
  shape = list(x.shape)
  new = shape[:offset] + [shape[offset] * shape[offset + 1]] + shape[offset + 2:]
  return x.reshape(new)


def unflatten_beam_dim(x: torch.Tensor, batch_size: int, beam_size: int,
                       offset: int = 0) -> torch.Tensor:
  shape = list(x.shape)
  assert shape[offset] == batch_size * beam_size
  return x.reshape(shape[:offset] + [batch_size, beam_size] + shape[offset + 1:])


def flat_batch_beam_expand(x: torch.Tensor, beam_size: int, offset: int = 0) -> torch.Tensor:
  return flatten_beam_dim(add_beam_dim(x, beam_size, offset), offset)


def gather_beams(nested, beam_indices: torch.Tensor, batch_size: int, old_beam_size: int,
                 new_beam_size: int, one_hot: bool = True):
  """Selects beams [batch, new_beam] out of [batch, old_beam, ...] tensors
  (t5x/decoding.py:873-915; a plain gather here, no one-hot contraction is needed)."""
  def g(x):
    idx = beam_indices.view(batch_size, new_beam_size, *([1] * (x.dim() - 2)))
    idx = idx.expand(batch_size, new_beam_size, *x.shape[2:])
    return torch.gather(x, 1, idx)
  if isinstance(nested, (list, tuple)):
    return type(nested)(g(x) for x in nested)
  return g(nested)


def cache_gather_beams(nested, beam_indices, batch_size, old_beam_size, new_beam_size,
                       one_hot: bool = True, offset: int = 0):
  """Gathers beams in every cache leaf whose dims are [..offset.., batch, beam, ...]
  (t5x/decoding.py:808-870)."""
  def g(x):
    bi = beam_indices
    if offset:
      moved = x.movedim(tuple(range(offset, offset + 2)), (0, 1))
      out = gather_beams(moved, bi, batch_size, old_beam_size, new_beam_size)
      return out.movedim((0, 1), tuple(range(offset, offset + 2)))
    return gather_beams(x, bi, batch_size, old_beam_size, new_beam_size)
  return cache_map(g, nested)


def top_k_two_stage(x: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
  """Top-k along the last dim, descending, lowest index first among ties
  (t5x/decoding.py:918-966)."""
  # Small inputs (the 2k / 3k candidate sets, where -1e7 ties are common) and CPU runs use a
  # stable sort, which is exact; the large beam*vocab selection on the GPU uses torch.topk
  # without any device->host read.
  if x.shape[-1] <= 4096 or not x.is_cuda:
    order = torch.argsort(x, dim=-1, descending=True, stable=True)[..., :k]
    return torch.gather(x, -1, order), order
  return torch.topk(x, k, dim=-1, largest=True, sorted=True)


def gather_topk_beams(nested, score_or_log_prob, batch_size, new_beam_size,
                      one_hot: bool = True):
  """Keeps the best `new_beam_size` beams, returned in ascending order
  (t5x/decoding.py:969-996)."""
  _, topk = top_k_two_stage(score_or_log_prob, new_beam_size)
  topk = torch.flip(topk, dims=[1])
  return gather_beams(nested, topk, batch_size, score_or_log_prob.shape[1], new_beam_size)


def _shift_rows(x: torch.Tensor, shifts: torch.Tensor) -> torch.Tensor:
  """Row r shifted right by shifts[r] (left if negative), zero filled."""
  b, l = x.shape
  src = torch.arange(l, device=x.device)[None, :] - shifts[:, None]
  valid = (src >= 0) & (src < l)
  out = torch.gather(x, 1, src.clamp(0, l - 1))
  return torch.where(valid, out, torch.zeros_like(out))


def _right_align_prompts(prompts: torch.Tensor) -> torch.Tensor:
  l = prompts.shape[1]
  idx = torch.arange(l, device=prompts.device)
  prompt_max_index = ((prompts != 0) * idx[None, :]).argmax(dim=1)
  return _shift_rows(prompts, l - prompt_max_index - 1)


def _left_align_prompts(prompts: torch.Tensor) -> torch.Tensor:
  l = prompts.shape[1]
  idx = torch.arange(l, device=prompts.device)
  nonpad = (prompts != 0) * (idx[None, :] + 1)
  m = torch.where(nonpad != 0, nonpad, torch.full_like(nonpad, l + 1))
  return _shift_rows(prompts, -m.argmin(dim=1))


def _pick_last_prompt_token(prompts: torch.Tensor) -> torch.Tensor:
  lengths = (prompts != 0).sum(dim=1)
  return prompts[torch.arange(prompts.shape[0], device=prompts.device), lengths]


# ----------------------------------------------------------------------------
# Beam search
# ----------------------------------------------------------------------------
@dataclasses.dataclass
class BeamState:
  cur_index: int
  live_logprobs: torch.Tensor
  finished_scores: torch.Tensor
  live_seqs: torch.Tensor
  finished_seqs: torch.Tensor
  finished_flags: torch.Tensor
  cache: PyTree
  initial_index: Optional[torch.Tensor]


def beam_init(batch_size, beam_size, max_decode_len, cache, offset=0, live_seqs=None,
              initial_index=None, device=None) -> BeamState:
  live_logprobs0 = torch.tensor([0.0] + [NEG_INF] * (beam_size - 1), dtype=torch.float32,
                                device=device).repeat(batch_size, 1)
  finished_scores0 = torch.full((batch_size, beam_size), NEG_INF, dtype=torch.float32,
                                device=device)
  live_seqs0 = live_seqs if live_seqs is not None else torch.zeros(
      (batch_size, beam_size, max_decode_len), dtype=torch.int64, device=device)
  finished_seqs0 = torch.zeros((batch_size, beam_size, max_decode_len), dtype=torch.int64,
                               device=device)
  finished_flags0 = torch.zeros((batch_size, beam_size), dtype=torch.bool, device=device)
  beam_cache0 = cache_map(lambda x: add_beam_dim(x, beam_size, offset).contiguous(), cache,
                          apply_to_index=live_seqs is not None)
  return BeamState(0, live_logprobs0, finished_scores0, live_seqs0, finished_seqs0,
                   finished_flags0, beam_cache0, initial_index)


def beam_search(inputs: torch.Tensor, cache: PyTree, tokens_to_logits: Callable, eos_id: int,
                num_decodes: int = 4, alpha: float = 0.6, max_decode_len: Optional[int] = None,
                max_decode_step: int = -1, min_log_prob: float = NEG_INF, decode_rng=None,
                cache_offset: int = 0, initial_index: Optional[torch.Tensor] = None,
                termination_check_period: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
  """Beam search (t5x/decoding.py:1131-1569).

  Returns ([batch, beam, max_decode_len] sequences, [batch, beam] scores), ascending.
  `termination_check_period` > 1 reads the early-termination flag from the device only every
  k-th step (extra steps after termination cannot change the finished set).
  """
  del decode_rng
  beam_size = num_decodes
  batch_size = inputs.shape[0]
  device = inputs.device
  inputs = inputs.long()
  if max_decode_len is None:
    max_decode_len = inputs.shape[1]
  max_decode_len += 1  # dummy BOS

  right_aligned_input = None
  live_seqs = None
  if initial_index is not None:
    right_aligned_input = _right_align_prompts(inputs)
    length = inputs.shape[1]
    last = right_aligned_input[:, -1:]
    inputs = torch.nn.functional.pad(last, (0, length - 1))
    live_seqs = torch.nn.functional.pad(last, (0, max_decode_len - 1))
    live_seqs = live_seqs[:, None, :].expand(batch_size, num_decodes, -1).contiguous()
  else:
    initial_index = torch.zeros((batch_size,), dtype=torch.int64, device=device)
  initial_index = initial_index.long()
  min_initial_index = int(initial_index.min()) if batch_size else 0

  state = beam_init(batch_size, beam_size, max_decode_len, cache, cache_offset,
                    live_seqs=live_seqs, initial_index=initial_index, device=device)
  min_brevity_penalty = brevity_penalty(alpha, max_decode_len)
  # `inputs` padded so that position cur_index+1 is always readable.
  padded_inputs = torch.nn.functional.pad(inputs, (0, max(0, max_decode_len + 1 - inputs.shape[1])))

  def device_terminated(st: BeamState) -> torch.Tensor:
    best_live = st.live_logprobs[:, -1:] / min_brevity_penalty
    worst_finished = st.finished_scores.min(dim=1, keepdim=True).values
    worst_finished = torch.where(st.finished_flags, worst_finished,
                                 torch.full_like(worst_finished, NEG_INF))
    search_terminated = (worst_finished > best_live).all()
    raw_min = min_log_prob / min_brevity_penalty
    none_pass = (best_live < raw_min).all() & (st.cur_index > 0)
    return search_terminated | none_pass

  step_count = 0
  while True:
    if not (state.cur_index + min_initial_index < max_decode_len - 1):
      break
    if max_decode_step > 0 and state.cur_index >= max_decode_step:
      break
    if step_count % max(1, termination_check_period) == 0 and bool(device_terminated(state)):
      break
    step_count += 1
    ci = state.cur_index
    flat_ids = flatten_beam_dim(state.live_seqs[:, :, ci:ci + 1])
    flat_cache = cache_map(lambda x: flatten_beam_dim(x, cache_offset), state.cache)
    dstate = DecodingState(cur_index=ci, sequences=flatten_beam_dim(state.live_seqs),
                           cur_token=flat_ids, cache=flat_cache)
    flat_logits, new_flat_cache = tokens_to_logits(dstate)
    logits = unflatten_beam_dim(flat_logits.float(), batch_size, beam_size)
    new_cache = cache_map(lambda x: unflatten_beam_dim(x, batch_size, beam_size, cache_offset),
                          new_flat_cache)
    candidate_log_probs = torch.log_softmax(logits, dim=-1)
    log_probs = candidate_log_probs + state.live_logprobs[:, :, None]
    vocab_size = log_probs.shape[-1]
    beams_to_keep = 2 * beam_size
    flat_log_probs = log_probs.reshape(batch_size, beam_size * vocab_size)
    topk_log_probs, topk_indices = top_k_two_stage(flat_log_probs, beams_to_keep)
    topk_ids = topk_indices % vocab_size

    next_input_token = padded_inputs[:, ci + 1][:, None]
    out_of_prompt = next_input_token == 0
    inside_prompt_log_probs = torch.cat([
        torch.zeros((batch_size, 1), dtype=topk_log_probs.dtype, device=device),
        torch.full((batch_size, beams_to_keep - 1), NEG_INF, dtype=topk_log_probs.dtype,
                   device=device)], dim=1)
    topk_log_probs = torch.where(out_of_prompt, topk_log_probs, inside_prompt_log_probs)
    topk_ids = torch.where(out_of_prompt, topk_ids, next_input_token.expand_as(topk_ids))

    topk_beam_indices = topk_indices // vocab_size
    topk_seq = gather_beams(state.live_seqs, topk_beam_indices, batch_size, beam_size,
                            beams_to_keep)
    topk_seq = topk_seq.clone()
    topk_seq[:, :, ci + 1] = topk_ids

    newly_finished = topk_seq[:, :, ci + 1] == eos_id
    new_log_probs = topk_log_probs + newly_finished.float() * NEG_INF
    _, new_topk_indices = top_k_two_stage(new_log_probs, beam_size)
    new_topk_indices = torch.flip(new_topk_indices, dims=[1])
    top_alive_seq, top_alive_log_probs = gather_beams([topk_seq, new_log_probs], new_topk_indices,
                                                      batch_size, 2 * beam_size, beam_size)
    top_alive_indices = gather_beams(topk_beam_indices, new_topk_indices, batch_size,
                                     2 * beam_size, beam_size)
    top_alive_cache = cache_gather_beams(new_cache, top_alive_indices, batch_size, beam_size,
                                         beam_size, True, cache_offset)

    lengths = initial_index[:, None].expand(batch_size, beams_to_keep) + (ci + 1)
    new_scores = topk_log_probs / brevity_penalty(alpha, lengths)
    new_scores = new_scores + (~newly_finished).float() * NEG_INF
    finished_seqs = torch.cat([state.finished_seqs, topk_seq], dim=1)
    finished_scores = torch.cat([state.finished_scores, new_scores], dim=1)
    finished_flags = torch.cat([state.finished_flags, newly_finished], dim=1)
    top_finished_seq, top_finished_scores, top_finished_flags = gather_topk_beams(
        [finished_seqs, finished_scores, finished_flags], finished_scores, batch_size, beam_size)
    state = BeamState(ci + 1, top_alive_log_probs, top_finished_scores, top_alive_seq,
                      top_finished_seq, top_finished_flags, top_alive_cache, initial_index)

  any_finished = state.finished_flags.any(dim=1)
  finished_seqs = torch.where(any_finished[:, None, None], state.finished_seqs, state.live_seqs)
  finished_scores = torch.where(any_finished[:, None], state.finished_scores,
                                state.live_logprobs)
  if right_aligned_input is not None:
    finished_seqs = finished_seqs[:, :, 1:]
    rai = right_aligned_input[:, None, :].expand(batch_size, finished_seqs.shape[1], -1)
    finished_seqs = torch.cat([rai, finished_seqs], dim=-1)
    flat = finished_seqs.reshape(-1, finished_seqs.shape[-1])
    flat = _left_align_prompts(flat)
    finished_seqs = flat.reshape(finished_seqs.shape)[:, :, :max_decode_len - 1]
  else:
    finished_seqs = finished_seqs[:, :, 1:]
  return finished_seqs, finished_scores


# ----------------------------------------------------------------------------
# Temperature sampling
# ----------------------------------------------------------------------------
def _make_generator(decode_rng, device) -> Optional[torch.Generator]:
  if decode_rng is None:
    decode_rng = 0
  if isinstance(decode_rng, torch.Generator):
    return decode_rng
  g = torch.Generator(device=device)
  g.manual_seed(int(decode_rng))
  return g


def temperature_sample(inputs: torch.Tensor, cache: PyTree, tokens_to_logits: Callable,
                       eos_id: int, decode_rng=None, num_decodes: int = 1,
                       temperature: Union[float, torch.Tensor] = 1.0, topk: int = 1,
                       topp: float = 0.0, cache_offset: int = 0,
                       initial_index: Optional[torch.Tensor] = None,
                       max_decode_steps: Optional[Union[int, torch.Tensor]] = None,
                       max_decode_steps_hard_limit: Optional[int] = None,
                       rescale_log_probs: bool = True,
                       state_callback_fn: Optional[Callable] = None,
                       logit_callback_fn: Optional[Callable] = None):
  """Temperature sampling with top-k / top-p (t5x/decoding.py:115-409).

  Returns ([batch, num_decodes, len] sequences sorted ascending by log-prob, log-probs).
  """
  device = inputs.device
  gen = _make_generator(decode_rng, device)
  if (max_decode_steps_hard_limit is not None and max_decode_steps_hard_limit > 0 and
      max_decode_steps is not None):
    if isinstance(max_decode_steps, torch.Tensor):
      max_decode_steps = torch.clamp(max_decode_steps, max=max_decode_steps_hard_limit)
    else:
      max_decode_steps = min(max_decode_steps, max_decode_steps_hard_limit)
  if num_decodes > 1:
    expanded_inputs = flat_batch_beam_expand(inputs, num_decodes)
    expanded_cache = cache_map(
        lambda x: flat_batch_beam_expand(x, num_decodes, cache_offset).contiguous(), cache,
        apply_to_index=initial_index is not None)
    if initial_index is not None:
      initial_index = flat_batch_beam_expand(initial_index, num_decodes)
  else:
    expanded_inputs, expanded_cache = inputs, cache
  decodes, log_prob = _temperature_sample_single_trial(
      expanded_inputs, expanded_cache, tokens_to_logits, eos_id, gen, num_decodes, temperature,
      topk, topp, initial_index=initial_index, max_decode_steps=max_decode_steps,
      rescale_log_probs=rescale_log_probs, state_callback_fn=state_callback_fn,
      logit_callback_fn=logit_callback_fn)
  batch_size = inputs.shape[0]
  decodes = unflatten_beam_dim(decodes, batch_size, num_decodes)
  log_prob = unflatten_beam_dim(log_prob, batch_size, num_decodes)
  idxs = torch.argsort(log_prob, dim=-1, stable=True)
  return (torch.gather(decodes, 1, idxs[:, :, None].expand_as(decodes)),
          torch.gather(log_prob, 1, idxs))


def _temperature_sample_single_trial(inputs, cache, tokens_to_logits, eos_id, gen, num_decodes=1,
                                     temperature=1.0, topk=20, topp=0.0, initial_index=None,
                                     max_decode_steps=None, rescale_log_probs=True,
                                     state_callback_fn=None, logit_callback_fn=None):
  if topp and topk:
    raise ValueError("At most one of `topp` or `topk` may be non-zero.")
  device = inputs.device
  inputs = inputs.long()
  batch_size, seq_len = inputs.shape
  max_decode_len: Any = seq_len
  if max_decode_steps is not None:
    if not isinstance(max_decode_steps, torch.Tensor) and max_decode_steps > inputs.shape[1]:
      raise ValueError("Cannot decode more steps than the sequence length.")
    max_decode_len = (inputs != 0).sum(dim=1) + max_decode_steps
    max_decode_len = torch.clamp(max_decode_len, max=inputs.shape[1])
  extra = 2
  sequences = torch.cat([inputs, torch.zeros((batch_size, extra), dtype=inputs.dtype,
                                             device=device)], dim=1)
  temperature_t = torch.as_tensor(temperature, dtype=torch.float32, device=device)
  if initial_index is None:
    i0 = torch.zeros((batch_size,), dtype=torch.int64, device=device)
    token0 = torch.zeros((batch_size, 1), dtype=torch.int64, device=device)
  else:
    i0 = initial_index.long()
    token0 = torch.gather(sequences, 1, i0[:, None])
  state = SamplingLoopState(0, i0, sequences, cache, token0,
                            torch.zeros((batch_size, 1), dtype=torch.bool, device=device), gen,
                            torch.zeros((batch_size,), dtype=torch.float32, device=device))
  initial_eos_count = (sequences == eos_id).sum(dim=-1, keepdim=True)
  mdl = (max_decode_len if isinstance(max_decode_len, torch.Tensor)
         else torch.full((batch_size,), max_decode_len, dtype=torch.int64, device=device))
  scalar_index = initial_index is None

  # On CUDA one kernel per step does the scaling, the top-k / top-p cut-off (radix select),
  # the draw (Gumbel noise from a counter-based generator keyed by this call's nonce and the
  # step) and the log-probability; the tensor-op statements below are the CPU path.
  native_nonce = None
  if device.type == "cuda":
    from t5x_b200.ops import native as _native
    if gen is not None:
      native_nonce = int(torch.randint(0, 2 ** 62, (1,), generator=gen, device=gen.device).item())
    else:
      native_nonce = int(torch.empty((), dtype=torch.int64).random_().item())

  def native_sample(logits, temp, step):
    return _native.sample_tokens(logits.contiguous(), temperature=temp, topk=topk or 0,
                                 topp=topp or 0.0, rescale_log_probs=rescale_log_probs,
                                 seed=native_nonce, stream_id=step)

  def nonzero_temp(logits, temp):
    scaled = logits / torch.clamp(temp, min=MIN_TEMPERATURE)
    if topk:
      scaled = binary_search.topk_mask(scaled, topk, NEG_INF)
    if topp:
      scaled = binary_search.topp_mask(scaled, topp, NEG_INF)
    probs = torch.softmax(scaled, dim=-1)
    nt = torch.multinomial(probs, 1, generator=gen).squeeze(-1)
    lp = torch.log_softmax(scaled if rescale_log_probs else logits, dim=-1)
    return nt, torch.gather(lp, 1, nt[:, None]).squeeze(-1)

  def zero_temp(logits):
    nt = logits.argmax(dim=-1)
    if rescale_log_probs:
      return nt, torch.zeros_like(nt, dtype=torch.float32)
    lp = torch.log_softmax(logits, dim=-1)
    return nt, torch.gather(lp, 1, nt[:, None]).squeeze(-1)

  while not bool(state.ended.all()):
    if state_callback_fn is not None:
      state = state_callback_fn(state)
    cur_index = state.cur_index
    dstate = DecodingState(cur_index=int(cur_index[0]) if scalar_index else cur_index,
                           sequences=state.sequences[:, :-extra], cur_token=state.cur_token,
                           cache=state.cache)
    logits, new_cache = tokens_to_logits(dstate)
    logits = logits.float()
    if logit_callback_fn is not None:
      logits = logit_callback_fn(logits, state)
    if native_nonce is not None and logits.dim() == 2:
      temp = (temperature_t.repeat_interleave(num_decodes) if temperature_t.dim() == 1
              else float(temperature_t))
      next_token, next_log_prob = native_sample(logits, temp, int(state.step))
    elif temperature_t.dim() == 1:
      temp_rows = temperature_t.repeat_interleave(num_decodes)[:, None]
      nt_a, lp_a = nonzero_temp(logits, temp_rows)
      nt_b, lp_b = zero_temp(logits)
      hot = temp_rows.squeeze(-1) > MIN_TEMPERATURE
      next_token = torch.where(hot, nt_a, nt_b)
      next_log_prob = torch.where(hot, lp_a, lp_b)
    elif float(temperature_t) > MIN_TEMPERATURE:
      next_token, next_log_prob = nonzero_temp(logits, temperature_t)
    else:
      next_token, next_log_prob = zero_temp(logits)
    i = torch.minimum(cur_index, mdl)
    next_input_token = torch.gather(state.sequences, 1, (i + 1)[:, None]).squeeze(1)
    out_of_prompt = next_input_token == 0
    next_token = torch.where(out_of_prompt, next_token, next_input_token)
    not_ended = (~state.ended).squeeze(-1)
    next_log_prob = state.log_prob + next_log_prob * out_of_prompt.float() * not_ended.float()
    next_token = next_token[:, None]
    next_token_or_endpad = next_token * (~state.ended).long()
    new_sequences = state.sequences.scatter(1, (i + 1)[:, None], next_token_or_endpad)
    cur_eos_count = (new_sequences == eos_id).sum(dim=-1, keepdim=True)
    ended = state.ended | (cur_eos_count > initial_eos_count) | (i >= mdl - 1)[:, None]
    state = SamplingLoopState(state.step + 1, i + 1, new_sequences, new_cache,
                              next_token_or_endpad, ended, gen, next_log_prob)
  if state_callback_fn is not None:
    state = state_callback_fn(state)
  return state.sequences[:, 1:-1], state.log_prob
