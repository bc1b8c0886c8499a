"""Further cases of beam search and temperature sampling on toy models: prefilled prompts with
per-example `initial_index`, step and probability limits, termination periods, length
penalties, per-example temperatures, the state / logit callbacks and the hard step limit
(the behaviours exercised by t5x/decoding_test.py beyond the basic ones)."""
import pytest
import torch

from t5x_b200 import decoding

NEG_INF = decoding.NEG_INF


def _markov(trans, start):
  """Next-token logits that depend on the previous token only (`start` after the BOS 0)."""
  trans = torch.tensor(trans, dtype=torch.float32)
  start = torch.tensor(start, dtype=torch.float32)

  def fn(state):
    tok = state.cur_token[:, 0]
    logits = torch.where((tok == 0)[:, None], start[None], trans[tok])
    return logits, state.cache
  return fn


def _random_chain(vocab, seed, eos=None, eos_boost=0.0):
  g = torch.Generator().manual_seed(seed)
  trans = torch.randn(vocab, vocab, generator=g) * 1.5
  start = torch.randn(vocab, generator=g) * 1.5
  trans[:, 0] = -1e9  # never emit PAD
  start[0] = -1e9
  if eos is not None:
    trans[:, eos] += eos_boost
  return trans.tolist(), start.tolist()


def test_beam_search_with_prefilled_prompts_matches_forced_prompts():
  """`initial_index` says how much of each row is an already-prefilled prompt: decoding starts
  from the last prompt token and the result is prompt + continuation, left-aligned. On a model
  whose logits depend on the previous token only, that equals forcing the same prompt."""
  vocab, eos, length, beams = 6, 5, 8, 3
  trans, start = _random_chain(vocab, 11)
  prompts = torch.tensor([[2, 3, 4, 0, 0, 0, 0, 0], [3, 0, 0, 0, 0, 0, 0, 0]])
  lengths = torch.tensor([3, 1])
  forced = torch.cat([torch.zeros(2, 1, dtype=torch.long), prompts[:, :-1]], dim=1)  # after BOS
  want_seqs, want_scores = decoding.beam_search(forced, {}, _markov(trans, start), eos_id=eos,
                                                num_decodes=beams, alpha=0.0)
  got_seqs, got_scores = decoding.beam_search(prompts, {}, _markov(trans, start), eos_id=eos,
                                              num_decodes=beams, alpha=0.0,
                                              initial_index=lengths)
  for b in range(2):
    n = int(lengths[b])
    assert got_seqs[b, -1, :n].tolist() == prompts[b, :n].tolist()
    # the continuation after the prompt is the one the forced-prompt search finds
    cont = got_seqs[b, -1, n:].tolist()
    ref = want_seqs[b, -1, n:].tolist()
    k = min(len(cont), len(ref)) - n
    assert cont[:k] == ref[:k]
  # log-probabilities of the best hypotheses agree (the forced prompt itself scores zero)
  torch.testing.assert_close(got_scores[:, -1], want_scores[:, -1], rtol=1e-4, atol=1e-4)


def test_max_decode_step_bounds_the_number_of_steps():
  vocab, eos = 5, 4
  trans, start = _random_chain(vocab, 3)
  for row in trans:
    row[eos] = -1e9  # never finishes by itself
  start[eos] = -1e9
  calls = []

  def counting(state):
    calls.append(int(state.cur_index))
    return _markov(trans, start)(state)

  seqs, _ = decoding.beam_search(torch.zeros(1, 10, dtype=torch.long), {}, counting, eos_id=eos,
                                 num_decodes=2, alpha=0.6, max_decode_step=4)
  assert calls == [0, 1, 2, 3]
  assert (seqs[0, -1, :4] > 0).all() and (seqs[0, -1, 4:] == 0).all()


def test_min_log_prob_stops_the_search_once_nothing_can_pass():
  """With a floor on the (length-normalised) log-probability the search ends as soon as the
  best live beam has fallen below it; without the floor it runs to the length limit."""
  vocab, eos = 4, 3
  uniform = [[0.0, 0.0, 0.0, -1e9] for _ in range(vocab)]  # three equally likely tokens, no EOS
  start = [-1e9, 0.0, 0.0, -1e9]
  steps = {"n": 0}

  def counting(state):
    steps["n"] += 1
    return _markov(uniform, start)(state)

  decoding.beam_search(torch.zeros(1, 12, dtype=torch.long), {}, counting, eos_id=eos,
                       num_decodes=2, alpha=0.0, min_log_prob=-3.0)
  with_floor = steps["n"]
  steps["n"] = 0
  decoding.beam_search(torch.zeros(1, 12, dtype=torch.long), {}, counting, eos_id=eos,
                       num_decodes=2, alpha=0.0)
  assert with_floor < steps["n"] == 12
  # log(1/2) then log(1/3) per step: below -3 after the third step
  assert with_floor == 4


@pytest.mark.parametrize("period", [1, 3, 8])
def test_termination_check_period_does_not_change_the_result(period):
  vocab, eos, beams = 6, 5, 4
  trans, start = _random_chain(vocab, 7, eos=eos, eos_boost=2.0)
  args = (torch.zeros(3, 10, dtype=torch.long), {}, _markov(trans, start))
  want = decoding.beam_search(*args, eos_id=eos, num_decodes=beams, alpha=0.6)
  got = decoding.beam_search(*args, eos_id=eos, num_decodes=beams, alpha=0.6,
                             termination_check_period=period)
  torch.testing.assert_close(got[0], want[0])
  torch.testing.assert_close(got[1], want[1])


def test_length_penalty_changes_which_hypothesis_wins():
  """alpha = 0 ranks by total log-probability (short wins), a large alpha by per-token
  quality (long wins): a chain where stopping at once costs log 0.4 and each further token
  only log 0.9."""
  import math
  eos = 2
  p = lambda x: math.log(x)
  start = [-1e9, p(0.6), p(0.4), -1e9]          # token 1 (continue) or EOS at once
  trans = [[-1e9] * 4,
           [-1e9, p(0.9), p(0.1), -1e9],       # after 1: mostly continue
           [-1e9] * 4, [-1e9] * 4]
  args = (torch.zeros(1, 6, dtype=torch.long), {}, _markov(trans, start))
  short, _ = decoding.beam_search(*args, eos_id=eos, num_decodes=2, alpha=0.0)
  long_, _ = decoding.beam_search(*args, eos_id=eos, num_decodes=2, alpha=3.0)
  assert short[0, -1].tolist() == [2, 0, 0, 0, 0, 0]
  assert long_[0, -1].tolist()[:2] == [1, 1] and 2 in long_[0, -1].tolist()


def test_beam_search_scores_are_length_normalised_log_probabilities():
  vocab, eos = 5, 4
  trans, start = _random_chain(vocab, 21, eos=eos, eos_boost=1.0)
  seqs, scores = decoding.beam_search(torch.zeros(1, 6, dtype=torch.long), {},
                                      _markov(trans, start), eos_id=eos, num_decodes=3, alpha=0.6)
  lt = torch.log_softmax(torch.tensor(trans), -1)
  ls = torch.log_softmax(torch.tensor(start), -1)
  for j in range(3):
    seq = [t for t in seqs[0, j].tolist() if t != 0]
    if not seq or seq[-1] != eos:
      continue
    lp = float(ls[seq[0]]) + sum(float(lt[a, b]) for a, b in zip(seq[:-1], seq[1:]))
    assert float(scores[0, j]) == pytest.approx(lp / decoding.brevity_penalty(0.6, len(seq)),
                                                rel=1e-4)


# ---- temperature sampling ----------------------------------------------------------------
def test_per_example_temperature():
  """Row 0 at temperature 0 is greedy; row 1 at a high temperature visits other tokens."""
  logits = torch.tensor([[-1e9, -1e9, 3.0, 2.5, 2.0, 1.5]] * 2)

  def fn(state):
    return logits.clone(), state.cache

  seqs, _ = decoding.temperature_sample(
      torch.zeros(2, 64, dtype=torch.long), {}, fn, eos_id=1, decode_rng=5,
      temperature=torch.tensor([0.0, 5.0]), topk=0)
  assert set(seqs[0, 0].tolist()) == {2}
  assert len(set(seqs[1, 0].tolist())) > 2


def test_logit_callback_can_forbid_tokens_and_state_callback_sees_every_step():
  logits = torch.tensor([[-1e9, -1e9, 5.0, 4.0, 3.0]])
  seen = []

  def fn(state):
    return logits.clone(), state.cache

  def forbid_two(lg, state):
    lg = lg.clone()
    lg[:, 2] = -1e9
    return lg

  def record(state):
    seen.append(int(state.cur_index.max()) if isinstance(state.cur_index, torch.Tensor)
                else int(state.cur_index))
    return state

  seqs, _ = decoding.temperature_sample(
      torch.zeros(1, 5, dtype=torch.long), {}, fn, eos_id=1, decode_rng=0, temperature=0.0,
      topk=0, logit_callback_fn=forbid_two, state_callback_fn=record)
  assert seqs[0, 0].tolist() == [3, 3, 3, 3, 3]
  assert len(seen) >= 5 and seen == sorted(seen)


def test_max_decode_steps_per_example_and_hard_limit():
  inputs = torch.tensor([[0, 5, 6, 0, 0, 0, 0, 0], [0, 7, 0, 0, 0, 0, 0, 0]])
  fn = lambda state: (torch.tensor([[-1e9, -1e9, 0.0, -1e9]] * 2), state.cache)
  seqs, _ = decoding.temperature_sample(inputs, {}, fn, eos_id=1, decode_rng=0, topk=1,
                                        max_decode_steps=torch.tensor([2, 4]))
  assert seqs[0, 0].tolist() == [5, 6, 2, 2, 0, 0, 0, 0]
  assert seqs[1, 0].tolist() == [7, 2, 2, 2, 2, 0, 0, 0]
  seqs, _ = decoding.temperature_sample(inputs, {}, fn, eos_id=1, decode_rng=0, topk=1,
                                        max_decode_steps=torch.tensor([6, 6]),
                                        max_decode_steps_hard_limit=3)
  assert seqs[0, 0].tolist() == [5, 6, 2, 2, 2, 0, 0, 0]
  assert seqs[1, 0].tolist() == [7, 2, 2, 2, 0, 0, 0, 0]


def test_rescale_log_probs_switch():
  """With top-k the sampled token's log-probability is taken from the truncated distribution
  when `rescale_log_probs` is set, from the full one otherwise."""
  import math
  logits = torch.log(torch.tensor([[1e-9, 1e-9, 0.5, 0.3, 0.2]]))
  fn = lambda state: (logits.clone(), state.cache)
  common = dict(eos_id=1, decode_rng=0, temperature=1.0, topk=1)
  _, lp_rescaled = decoding.temperature_sample(torch.zeros(1, 3, dtype=torch.long), {}, fn,
                                               rescale_log_probs=True, **common)
  _, lp_raw = decoding.temperature_sample(torch.zeros(1, 3, dtype=torch.long), {}, fn,
                                          rescale_log_probs=False, **common)
  assert float(lp_rescaled[0, 0]) == pytest.approx(0.0, abs=1e-4)
  assert float(lp_raw[0, 0]) == pytest.approx(3 * math.log(0.5), rel=1e-3)
