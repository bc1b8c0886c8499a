"""Log-probabilities reported by the samplers, cache mapping, the two-stage top-k and the prompt
alignment helpers (further cases of t5x/decoding_test.py)."""
import math

import pytest
import torch

from t5x_b200 import decoding


def _fixed(logits_rows):
  """tokens_to_logits that returns the same logits at every step (one row per example)."""
  table = torch.tensor(logits_rows, dtype=torch.float32)

  def fn(state):
    return table.clone(), state.cache
  return fn


def test_greedy_log_prob_is_the_sum_of_token_log_probs_until_eos():
  # token 3 (p = 0.6) twice, then the model is switched to emit EOS
  probs = [1e-9, 0.1, 0.3, 0.6]
  steps = {"n": 0}

  def fn(state):
    steps["n"] += 1
    row = [1e-9, 0.97, 0.01, 0.02] if steps["n"] > 2 else probs
    return torch.log(torch.tensor([row])), state.cache

  seqs, lp = decoding.temperature_sample(torch.zeros(1, 6, dtype=torch.long), {}, fn, eos_id=1,
                                         decode_rng=0, temperature=0.0, topk=0,
                                         rescale_log_probs=False)
  assert seqs[0, 0].tolist() == [3, 3, 1, 0, 0, 0]
  assert float(lp[0, 0]) == pytest.approx(2 * math.log(0.6) + math.log(0.97), rel=1e-4)


def test_sampled_log_prob_matches_the_sampled_tokens():
  torch.manual_seed(0)
  logits = torch.randn(3, 7)
  logits[:, 0] = -1e9  # never PAD
  logits[:, 1] = -1e9  # never EOS: every sequence runs to the end
  seqs, lp = decoding.temperature_sample(torch.zeros(3, 5, dtype=torch.long), {},
                                         _fixed(logits.tolist()), eos_id=1, decode_rng=3,
                                         temperature=1.0, topk=0)
  logp = torch.log_softmax(logits, -1)
  for b in range(3):
    want = sum(float(logp[b, t]) for t in seqs[b, 0].tolist())
    assert float(lp[b, 0]) == pytest.approx(want, rel=1e-4)


def test_temperature_rescales_the_reported_log_probs_only_when_asked():
  logits = [[-1e9, -1e9, 2.0, 1.0, 0.0]]
  common = dict(eos_id=1, decode_rng=0, topk=0)
  # temperature 0.5 sharpens the distribution the tokens are drawn from ...
  _, lp_scaled = decoding.temperature_sample(torch.zeros(1, 1, dtype=torch.long), {},
                                             _fixed(logits), temperature=1e-4,
                                             rescale_log_probs=True, **common)
  _, lp_raw = decoding.temperature_sample(torch.zeros(1, 1, dtype=torch.long), {},
                                          _fixed(logits), temperature=1e-4,
                                          rescale_log_probs=False, **common)
  # ... at temperature -> 0 the sharpened distribution gives log p = 0 for the arg-max token,
  # the raw one its untempered log-probability
  assert float(lp_scaled[0, 0]) == pytest.approx(0.0, abs=1e-3)
  raw = float(torch.log_softmax(torch.tensor(logits[0]), -1)[2])
  assert float(lp_raw[0, 0]) == pytest.approx(raw, rel=1e-4)


def test_topp_log_probs_are_renormalised_over_the_nucleus():
  probs = [1e-9, 1e-9, 0.5, 0.3, 0.2]
  logits = [[math.log(p) for p in probs]]
  seen = set()
  for seed in range(12):
    seqs, lp = decoding.temperature_sample(torch.zeros(1, 1, dtype=torch.long), {},
                                           _fixed(logits), eos_id=1, decode_rng=seed,
                                           temperature=1.0, topk=0, topp=0.7)
    tok = int(seqs[0, 0, 0])
    seen.add(tok)
    assert tok in (2, 3)                       # the nucleus of mass 0.7: {0.5, 0.3}
    assert float(lp[0, 0]) == pytest.approx(math.log(probs[tok] / 0.8), rel=1e-3)
  assert seen == {2, 3}


def test_num_decodes_with_initial_index_keeps_each_prompt():
  vocab = 8
  logits = torch.zeros(2, vocab)
  logits[:, :2] = -1e9

  def fn(state):
    return logits.repeat_interleave(3, dim=0), state.cache

  prompts = torch.tensor([[0, 5, 6, 0, 0, 0, 0], [0, 7, 0, 0, 0, 0, 0]])
  seqs, lp = decoding.temperature_sample(prompts, {}, fn, eos_id=1, decode_rng=1, num_decodes=3,
                                         temperature=1.0, topk=0,
                                         initial_index=torch.tensor([2, 1]))
  assert seqs.shape == (2, 3, 7) and lp.shape == (2, 3)
  assert (seqs[0, :, :2] == torch.tensor([5, 6])).all() and (seqs[1, :, 0] == 7).all()
  assert (seqs[:, :, 2:] >= 0).all()
  assert (lp[:, 1:] >= lp[:, :-1]).all()      # ascending
  # different samples per decode
  assert len({tuple(r) for r in seqs[0].tolist()}) > 1


def test_cache_map_skips_bookkeeping_leaves():
  cache = {"decoder": {"layers_0": {"self_attention": {
      "cached_key": torch.zeros(2, 4, 3), "cached_value": torch.zeros(2, 4, 3),
      "cache_index": torch.tensor(0)}},
      "relpos_bias": {"cached_bias": torch.zeros(1, 2, 1, 4)},
      "position_embedder": {"position_embedder_index": torch.tensor(-1)}}}
  out = decoding.cache_map(lambda x: x + 1, cache)
  attn = out["decoder"]["layers_0"]["self_attention"]
  assert float(attn["cached_key"].sum()) == 24.0 and float(attn["cached_value"].sum()) == 24.0
  assert int(attn["cache_index"]) == 0                         # scalar index: untouched
  assert float(out["decoder"]["relpos_bias"]["cached_bias"].sum()) == 0.0
  assert int(out["decoder"]["position_embedder"]["position_embedder_index"]) == -1
  # a per-example index is mapped when asked for (prefilled prompts of different lengths)
  cache["decoder"]["layers_0"]["self_attention"]["cache_index"] = torch.tensor([3, 1])
  out = decoding.cache_map(lambda x: x + 1, cache, apply_to_index=True)
  assert out["decoder"]["layers_0"]["self_attention"]["cache_index"].tolist() == [4, 2]
  out = decoding.cache_map(lambda x: x + 1, cache, apply_to_index=False)
  assert out["decoder"]["layers_0"]["self_attention"]["cache_index"].tolist() == [3, 1]


def test_beam_dim_helpers_and_cache_gather():
  x = torch.arange(6).view(2, 3)
  assert decoding.add_beam_dim(x, 2).shape == (2, 2, 3)
  flat = decoding.flat_batch_beam_expand(x, 2)
  assert flat.tolist() == [[0, 1, 2], [0, 1, 2], [3, 4, 5], [3, 4, 5]]
  assert decoding.unflatten_beam_dim(flat, 2, 2).shape == (2, 2, 3)
  with_offset = decoding.add_beam_dim(torch.zeros(5, 2, 3), 4, offset=1)   # [layers, batch, ...]
  assert with_offset.shape == (5, 2, 4, 3)
  beams = torch.arange(2 * 3 * 4).view(2, 3, 4)
  picked = decoding.gather_beams(beams, torch.tensor([[2, 0], [1, 1]]), 2, 3, 2)
  assert picked[0].tolist() == [beams[0, 2].tolist(), beams[0, 0].tolist()]
  assert picked[1].tolist() == [beams[1, 1].tolist(), beams[1, 1].tolist()]
  cache = {"k": beams.float(), "cache_index": torch.tensor(5)}
  out = decoding.cache_gather_beams(cache, torch.tensor([[2, 0], [1, 1]]), 2, 3, 2)
  assert out["k"].tolist() == picked.float().tolist() and int(out["cache_index"]) == 5


def test_top_k_two_stage_orders_ties_by_index():
  x = torch.tensor([[1.0, 5.0, 5.0, 3.0, -1e7, -1e7], [0.0, 0.0, 0.0, 0.0, 0.0, 2.0]])
  vals, idx = decoding.top_k_two_stage(x, 3)
  assert vals.tolist() == [[5.0, 5.0, 3.0], [2.0, 0.0, 0.0]]
  assert idx.tolist() == [[1, 2, 3], [5, 0, 1]]
  torch.manual_seed(0)
  big = torch.randn(4, 9000)
  v2, i2 = decoding.top_k_two_stage(big, 7)
  want_v, want_i = torch.topk(big, 7, dim=-1)
  assert v2.tolist() == want_v.tolist() and i2.tolist() == want_i.tolist()


def test_prompt_alignment_helpers():
  prompts = torch.tensor([[0, 5, 6, 0, 0], [0, 7, 0, 0, 0], [0, 0, 0, 0, 0]])
  right = decoding._right_align_prompts(prompts)
  assert right.tolist() == [[0, 0, 0, 5, 6], [0, 0, 0, 0, 7], [0, 0, 0, 0, 0]]
  assert decoding._left_align_prompts(right).tolist() == [[5, 6, 0, 0, 0], [7, 0, 0, 0, 0],
                                                          [0, 0, 0, 0, 0]]
  assert decoding._pick_last_prompt_token(prompts).tolist() == [6, 7, 0]
  assert decoding.brevity_penalty(0.6, 7) == pytest.approx((12 / 6) ** 0.6)
  torch.testing.assert_close(decoding.brevity_penalty(1.0, torch.tensor([1, 7])),
                             torch.tensor([1.0, 2.0]))
