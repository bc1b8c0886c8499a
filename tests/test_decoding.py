"""Decoding algorithms on toy models: temperature sampling with prompts, top-k / top-p masks
against a sort oracle, beam search against exhaustive enumeration
(cases and expected values after t5x/decoding_test.py and t5x/binary_search_test.py)."""
import itertools

import numpy as np
import pytest
import torch

from t5x_b200 import binary_search, decoding

EOS_ID = 1
NEG_INF = decoding.NEG_INF


def _fixed_logits(rows):
  table = torch.tensor(rows, dtype=torch.float32)

  def fn(state):
    return table.clone(), state.cache
  return fn


ALWAYS_2_AND_3 = [[-1e7, -1e7, 0, -1e7], [-1e7, -1e7, -1e7, 0]]


def test_sample_without_prompt():
  seqs, _ = decoding._temperature_sample_single_trial(
      torch.zeros(2, 3, dtype=torch.long), {}, _fixed_logits(ALWAYS_2_AND_3), EOS_ID, None, topk=0)
  assert seqs.tolist() == [[2, 2, 2], [3, 3, 3]]


def test_sample_keeps_prompt_then_samples():
  inputs = torch.tensor([[0, 5, 6, 7, 0], [0, 8, 9, 0, 0]])
  seqs, _ = decoding._temperature_sample_single_trial(
      inputs, {}, _fixed_logits(ALWAYS_2_AND_3), EOS_ID, None, topk=0)
  assert seqs.tolist() == [[5, 6, 7, 2, 2], [8, 9, 3, 3, 3]]


def test_sample_from_uneven_initial_index():
  inputs = torch.tensor([[0, 5, 7, 1, 0, 0], [0, 6, 1, 0, 0, 0]])
  seqs, _ = decoding._temperature_sample_single_trial(
      inputs, {}, _fixed_logits(ALWAYS_2_AND_3), EOS_ID, None, topk=0,
      initial_index=torch.tensor([3, 2]))
  assert seqs.tolist() == [[5, 7, 1, 2, 2, 2], [6, 1, 3, 3, 3, 3]]


def test_zero_temperature_is_argmax():
  logits = [[1700.47, 1700.48, 1700.51, 1700.45], [3.2, 4.8, -5.3, 5.6]]
  seqs, _ = decoding._temperature_sample_single_trial(
      torch.zeros(2, 3, dtype=torch.long), {}, _fixed_logits(logits), EOS_ID, None, topk=4,
      temperature=0.0)
  assert seqs.tolist() == [[2, 2, 2], [3, 3, 3]]


def test_prompt_ending_with_eos_does_not_stop_decoding():
  inputs = torch.tensor([[0, 5, 6, 1, 0], [0, 8, 1, 0, 0]])
  seqs, _ = decoding._temperature_sample_single_trial(
      inputs, {}, _fixed_logits(ALWAYS_2_AND_3), EOS_ID, None, topk=1)
  assert seqs.tolist() == [[5, 6, 1, 2, 2], [8, 1, 3, 3, 3]]


def test_sampling_stops_at_eos_and_pads():
  # token 1 (EOS) is certain: decoding ends after one step, the rest stays 0
  logits = [[-1e7, 0, -1e7, -1e7]] * 2
  seqs, lp = decoding._temperature_sample_single_trial(
      torch.zeros(2, 4, dtype=torch.long), {}, _fixed_logits(logits), EOS_ID, None, topk=0)
  assert seqs.tolist() == [[1, 0, 0, 0], [1, 0, 0, 0]]
  np.testing.assert_allclose(lp.numpy(), 0.0, atol=1e-4)


def test_num_decodes_sorted_by_log_prob():
  torch.manual_seed(0)
  probs = torch.tensor([[0.05, 0.05, 0.6, 0.3]])

  def fn(state):
    rows = state.cur_token.shape[0]
    return torch.log(probs).expand(rows, 4).clone(), state.cache

  seqs, lp = decoding.temperature_sample(torch.zeros(1, 3, dtype=torch.long), {}, fn, EOS_ID,
                                         decode_rng=0, num_decodes=6, topk=0)
  assert seqs.shape == (1, 6, 3) and lp.shape == (1, 6)
  assert torch.all(lp[0, 1:] >= lp[0, :-1])  # ascending: best last


def test_max_decode_steps_counts_from_prompt_end():
  inputs = torch.tensor([[0, 5, 6, 0, 0, 0], [0, 8, 0, 0, 0, 0]])
  seqs, _ = decoding._temperature_sample_single_trial(
      inputs, {}, _fixed_logits(ALWAYS_2_AND_3), EOS_ID, None, topk=0, max_decode_steps=2)
  assert seqs.tolist() == [[5, 6, 2, 2, 0, 0], [8, 3, 3, 0, 0, 0]]


# ---- masks ----------------------------------------------------------------------------------
@pytest.mark.parametrize("k", [1, 3, 7])
def test_topk_mask_matches_sort(k):
  torch.manual_seed(k)
  x = torch.randn(5, 40)
  masked = binary_search.topk_mask(x, k, -1e9)
  kth = torch.sort(x, dim=-1, descending=True).values[:, k - 1:k]
  expect = torch.where(x >= kth, x, torch.full_like(x, -1e9))
  torch.testing.assert_close(masked, expect)


@pytest.mark.parametrize("p", [0.1, 0.5, 0.9])
def test_topp_mask_keeps_smallest_nucleus(p):
  torch.manual_seed(3)
  logits = torch.randn(4, 30) * 2
  masked = binary_search.topp_mask(logits, p, -1e9)
  probs = torch.softmax(logits, -1)
  for r in range(4):
    order = torch.argsort(probs[r], descending=True)
    csum = torch.cumsum(probs[r][order], 0)
    n_keep = int((csum < p).sum()) + 1
    keep = set(order[:n_keep].tolist())
    got = set(torch.nonzero(masked[r] > -1e8).flatten().tolist())
    assert got == keep


def test_float_bsearch_finds_threshold():
  target = torch.tensor([-3.5, 0.0, 12.25])
  found = binary_search.float32_bsearch((3,), lambda x: x > target)
  torch.testing.assert_close(found, target)


# ---- beam search ----------------------------------------------------------------------------
def test_beam_helpers():
  x = torch.arange(6).view(2, 3)
  assert decoding.add_beam_dim(x, 2).shape == (2, 2, 3)
  assert decoding.flat_batch_beam_expand(x, 2).tolist() == [[0, 1, 2], [0, 1, 2], [3, 4, 5],
                                                            [3, 4, 5]]
  v, i = decoding.top_k_two_stage(torch.tensor([[1.0, 9.0, 3.0, 7.0, 5.0, 8.0]]), 3)
  assert v.tolist() == [[9.0, 8.0, 7.0]] and i.tolist() == [[1, 5, 3]]
  assert decoding.brevity_penalty(0.6, 7) == pytest.approx(2.0 ** 0.6)


def _markov_logits(trans, start):
  """First-order Markov 'model': logits of the next token depend on the current token only."""
  trans = torch.tensor(trans, dtype=torch.float32)
  start = torch.tensor(start, dtype=torch.float32)

  def fn(state):
    tok = state.cur_token[:, 0]
    first = (state.cache["step"][:, 0] == 0)
    logits = torch.where(first[:, None], start[None], trans[tok])
    return logits, {"step": state.cache["step"] + 1}
  return fn


def _brute_force(trans, start, length, eos, alpha, n_best):
  """All finished hypotheses (ending in EOS within `length`) with length-normalised scores."""
  trans = torch.log_softmax(torch.tensor(trans, dtype=torch.float32), -1)
  start = torch.log_softmax(torch.tensor(start, dtype=torch.float32), -1)
  vocab = trans.shape[0]
  out = []
  for n in range(1, length + 1):
    for body in itertools.product([t for t in range(1, vocab) if t != eos], repeat=n - 1):
      seq = list(body) + [eos]
      lp = float(start[seq[0]])
      for a, b in zip(seq[:-1], seq[1:]):
        lp += float(trans[a, b])
      out.append((lp / decoding.brevity_penalty(alpha, n), seq))
  out.sort(key=lambda t: -t[0])
  return out[:n_best]


@pytest.mark.parametrize("alpha", [0.0, 0.6])
def test_beam_search_finds_the_exhaustive_optimum(alpha):
  torch.manual_seed(5)
  vocab, eos, length, beams = 5, 4, 5, 8
  trans = (torch.randn(vocab, vocab) * 1.5).tolist()
  start = (torch.randn(vocab) * 1.5).tolist()
  for row in trans:
    row[0] = -1e9  # never emit PAD
  start[0] = -1e9
  seqs, scores = decoding.beam_search(
      torch.zeros(2, length, dtype=torch.long), {"step": torch.zeros(2, 1)},
      _markov_logits(trans, start), eos_id=eos, num_decodes=beams, alpha=alpha)
  assert seqs.shape == (2, beams, length) and scores.shape == (2, beams)
  best_score, best_seq = _brute_force(trans, start, length, eos, alpha, 1)[0]
  got = seqs[0, -1].tolist()
  assert got[:len(best_seq)] == best_seq and all(t == 0 for t in got[len(best_seq):])
  assert float(scores[0, -1]) == pytest.approx(best_score, rel=1e-4)
  assert torch.all(scores[:, 1:] >= scores[:, :-1])  # ascending
  torch.testing.assert_close(seqs[0], seqs[1])       # batch rows are independent and equal


def test_beam_search_forces_prompt():
  vocab, eos = 5, 4
  trans = [[0.0] * vocab for _ in range(vocab)]
  start = [0.0, 0.0, 5.0, 0.0, 0.0]
  prompt = torch.tensor([[0, 3, 3, 0, 0, 0]])
  seqs, _ = decoding.beam_search(prompt, {"step": torch.zeros(1, 1)},
                                 _markov_logits(trans, start), eos_id=eos, num_decodes=2,
                                 alpha=0.0)
  assert seqs[0, -1, :2].tolist() == [3, 3]
