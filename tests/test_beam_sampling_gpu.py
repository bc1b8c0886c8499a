"""Native beam-search step, sampling and top-k / top-p mask kernels (csrc/beam.cu) against the
tensor-op statements of the same algorithms in fp32."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


class _State:
  """Search state of `GraphBeamDecoder` without a model: lets the native step and the
  tensor-op step run on identical inputs."""

  def __init__(self, b, k, L, eos, alpha, dev):
    from t5x_b200 import decoding, decoding_fast
    d = object.__new__(decoding_fast.GraphBeamDecoder)
    d.b, d.k, d.L, d.eos, d.alpha, d.dev = b, k, L, eos, alpha, dev
    d.rows = b * k
    i64 = dict(dtype=torch.int64, device=dev)
    d.cur = torch.zeros(1, dtype=torch.int32, device=dev)
    d.live_seqs = torch.zeros(b, k, L, **i64)
    d.fin_seqs = torch.zeros(b, k, L, **i64)
    d.live_lp = torch.zeros(b, k, device=dev)
    d.fin_scores = torch.zeros(b, k, device=dev)
    d.fin_flags = torch.zeros(b, k, dtype=torch.bool, device=dev)
    d.anc = torch.zeros(b, k, L, dtype=torch.int32, device=dev)
    d.terminated = torch.zeros(1, dtype=torch.bool, device=dev)
    d.positions = torch.arange(L, device=dev)
    d.min_brevity = float(decoding.brevity_penalty(alpha, L))
    d._beam_scratch = None
    d._reset()
    self.d = d

  def snapshot(self):
    d = self.d
    return {n: getattr(d, n).clone() for n in ("cur", "live_seqs", "fin_seqs", "live_lp",
                                                "fin_scores", "fin_flags", "anc", "terminated")}


@pytest.mark.parametrize("beams,vocab", [(1, 37), (2, 300), (4, 5000), (8, 32128), (4, 9001)])
def test_native_beam_step_matches_tensor_ops(beams, vocab):
  dev = torch.device("cuda")
  b, L, eos = 5, 12, 1
  native_s, tensor_s = _State(b, beams, L, eos, 0.6, dev), _State(b, beams, L, eos, 0.6, dev)
  g = torch.Generator(device="cuda").manual_seed(vocab + beams)
  for step in range(L - 1):
    logits = torch.randn(b * beams, vocab, device=dev, generator=g) * 3.0
    logits[::3, eos] += 6.0  # make the end-of-sequence token win sometimes
    native_s.d._beam_step(logits.clone())
    tensor_s.d._beam_step_tensor_ops(logits.clone())
    a, r = native_s.snapshot(), tensor_s.snapshot()
    assert int(a["cur"]) == int(r["cur"]) == step + 1
    torch.testing.assert_close(a["live_lp"], r["live_lp"], rtol=1e-5, atol=2e-4)
    assert torch.equal(a["fin_flags"], r["fin_flags"])
    # slots without a finished hypothesis hold placeholders near -1e7 (which placeholder
    # survives a tie is not part of the contract)
    assert bool((a["fin_scores"][~a["fin_flags"]] < -9.9e6).all())
    # sequences and ancestry of every live beam, and of every finished slot that is real
    assert torch.equal(a["live_seqs"], r["live_seqs"]), step
    assert torch.equal(a["anc"][:, :, :step + 1], r["anc"][:, :, :step + 1])
    real = a["fin_flags"]
    assert torch.equal(a["fin_seqs"][real], r["fin_seqs"][real])
    torch.testing.assert_close(a["fin_scores"][real], r["fin_scores"][real], rtol=1e-5, atol=2e-4)
    assert bool(a["terminated"]) == bool(r["terminated"])
  from t5x_b200.ops import native
  native.check_status()


def test_native_beam_step_breaks_ties_by_lowest_index():
  """All logits equal: the candidates must be tokens 0, 1, 2, ... of beam 0 first."""
  dev = torch.device("cuda")
  st = _State(2, 4, 6, eos=1, alpha=0.6, dev=dev)
  st.d._beam_step(torch.zeros(8, 50, device=dev))
  s = st.snapshot()
  # best 2k = tokens 0..7 of beam 0; token 1 is EOS, so the live beams (ascending) are
  # tokens 4, 3, 2, 0 and the finished slot holds token 1
  assert s["live_seqs"][0, :, 1].tolist() == [4, 3, 2, 0]
  assert s["fin_flags"][0].tolist() == [False, False, False, True]
  assert int(s["fin_seqs"][0, 3, 1]) == 1


def _reference_masks(x, topk, topp):
  neg = -1e7
  if topk:
    kth = torch.topk(x, topk, dim=-1).values[..., -1:]
    return torch.where(x >= kth, x, torch.full_like(x, neg))
  probs = torch.softmax(x.double(), dim=-1)
  sp, _ = torch.sort(probs, dim=-1, descending=True)
  cum = torch.cumsum(sp, dim=-1)
  first = (cum >= topp).float().argmax(dim=-1, keepdim=True)
  cutoff = torch.gather(sp, -1, first)
  return torch.where(probs >= cutoff, x, torch.full_like(x, neg))


@pytest.mark.parametrize("vocab", [64, 1000, 32128])
def test_topk_and_topp_masks_match_sorting(vocab):
  from t5x_b200 import binary_search
  torch.manual_seed(vocab)
  x = (torch.randn(33, vocab, device="cuda") * 2.5).contiguous()
  x[:, 5] = x[:, 9]  # ties at the cut-off are kept on both sides
  for k in (1, 3, 20, min(vocab, 250)):
    got = binary_search.topk_mask(x, k, -1e7)
    assert torch.equal(got, _reference_masks(x, k, 0.0)), k
  for p in (0.1, 0.5, 0.9, 0.999):
    got = binary_search.topp_mask(x, p, -1e7)
    want = _reference_masks(x, 0, p)
    # summation order differs (fp32 mass histogram vs fp64 cumsum): allow the cut-off to move
    # by entries that carry almost no mass
    differ = (got != want)
    mass = torch.softmax(x.double(), -1)
    assert float((mass * differ).sum(-1).max()) < 2e-4, p


def test_sampling_distribution_and_log_probs():
  from t5x_b200.ops import native
  torch.manual_seed(0)
  vocab, rows = 48, 60000
  base = torch.randn(vocab, device="cuda") * 1.5
  logits = base[None].expand(rows, vocab).contiguous()
  temperature, topk = 0.7, 12
  tok, lp = native.sample_tokens(logits, temperature=temperature, topk=topk, topp=0.0,
                                 rescale_log_probs=True, seed=1234, stream_id=3)
  scaled = base / temperature
  kth = torch.topk(scaled, topk).values[-1]
  masked = torch.where(scaled >= kth, scaled, torch.full_like(scaled, -1e7))
  want = torch.softmax(masked.double(), -1)
  freq = torch.bincount(tok, minlength=vocab).double() / rows
  assert float((freq - want).abs().max()) < 6e-3
  assert int((freq > 0).sum()) == topk
  torch.testing.assert_close(lp, torch.log(want)[tok].float(), rtol=1e-4, atol=1e-4)
  # a second draw with the same key repeats, another stream differs
  tok2, _ = native.sample_tokens(logits, temperature=temperature, topk=topk, topp=0.0,
                                 rescale_log_probs=True, seed=1234, stream_id=3)
  tok3, _ = native.sample_tokens(logits, temperature=temperature, topk=topk, topp=0.0,
                                 rescale_log_probs=True, seed=1234, stream_id=4)
  assert torch.equal(tok, tok2) and not torch.equal(tok, tok3)


def test_sampling_top_p_per_row_temperature_and_greedy():
  from t5x_b200.ops import native
  torch.manual_seed(1)
  vocab, rows = 1000, 4096
  logits = (torch.randn(rows, vocab, device="cuda") * 2.0).contiguous()
  temps = torch.ones(rows, device="cuda")
  temps[::2] = 0.0  # greedy rows
  tok, lp = native.sample_tokens(logits, temperature=temps, topk=0, topp=0.3,
                                 rescale_log_probs=False, seed=7, stream_id=0)
  assert torch.equal(tok[::2], logits[::2].argmax(-1))
  full_lp = torch.log_softmax(logits, -1)
  torch.testing.assert_close(lp, full_lp.gather(1, tok[:, None]).squeeze(1), rtol=1e-4, atol=1e-4)
  # sampled rows stay inside the nucleus
  probs = torch.softmax(logits[1::2].double(), -1)
  sp, order = torch.sort(probs, -1, descending=True)
  inside = (torch.cumsum(sp, -1) - sp) < 0.3 + 1e-6
  allowed = torch.zeros_like(probs, dtype=torch.bool).scatter_(1, order, inside)
  assert bool(allowed.gather(1, tok[1::2, None]).all())


def test_temperature_sample_runs_on_the_native_kernel():
  """`decoding.temperature_sample` on CUDA: greedy sampling reproduces the arg-max decode, and
  top-k sampling only emits tokens of the top-k set."""
  from t5x_b200 import decoding
  from t5x_b200.ops import native
  torch.manual_seed(3)
  vocab, b, L = 90, 6, 7
  table = torch.randn(vocab, vocab, device="cuda") * 2

  def tokens_to_logits(state):
    return table[state.cur_token.squeeze(-1)], state.cache

  inputs = torch.zeros(b, L, dtype=torch.long, device="cuda")
  n0 = native.launch_count()
  seqs, _ = decoding.temperature_sample(inputs, {}, tokens_to_logits, eos_id=1, decode_rng=0,
                                        temperature=0.0, topk=0)
  assert native.launch_count() > n0
  cur = torch.zeros(b, dtype=torch.long, device="cuda")
  for t in range(L):
    nxt = table[cur].argmax(-1)
    live = seqs[:, 0, t] != 0
    assert torch.equal(seqs[:, 0, t][live], nxt[live])
    cur = nxt
  seqs, _ = decoding.temperature_sample(inputs, {}, tokens_to_logits, eos_id=1, decode_rng=1,
                                        temperature=1.0, topk=3, num_decodes=4)
  prev = torch.zeros(b, 4, dtype=torch.long, device="cuda")
  for t in range(L):
    top3 = torch.topk(table[prev], 3, dim=-1).indices
    tok = seqs[:, :, t]
    ok = (top3 == tok[..., None]).any(-1) | (tok == 0)
    assert bool(ok.all())
    prev = tok
