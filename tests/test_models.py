"""The encoder-decoder model API on the CPU: helpers, initial variables, loss and metrics
against a hand-computed cross-entropy, sequence scores, cached decoding against a full forward
pass per step, sampling seeds, prompts (the behaviours of t5x/models_test.py)."""
import functools

import pytest
import torch

from t5x_b200 import adafactor, decoding, models
from t5x_b200.data import vocabularies
from t5x_b200.models import base
from t5x_b200.models.t5 import network
from t5x_b200.utils import tree


def _model(decode_fn=decoding.beam_search, seed=3, z_loss=0.0, label_smoothing=0.0):
  cfg = network.T5Config(vocab_size=64, dtype="float32", emb_dim=32, num_heads=2,
                         num_encoder_layers=2, num_decoder_layers=2, head_dim=16, mlp_dim=64,
                         mlp_activations=("gelu", "linear"), dropout_rate=0.0)
  torch.manual_seed(seed)
  module = network.Transformer(cfg)
  with torch.no_grad():  # sharper output distributions than the initialisation gives
    module.token_embedder.embedding.mul_(6.0)
  vocab = vocabularies.PassThroughVocabulary(64)
  return models.EncoderDecoderModel(module, vocab, vocab, adafactor.Adafactor(),
                                    decode_fn=decode_fn, z_loss=z_loss,
                                    label_smoothing=label_smoothing)


def _batch(b=3, le=7, ld=6, seed=0):
  g = torch.Generator().manual_seed(seed)
  enc = torch.randint(2, 64, (b, le), generator=g)
  enc[0, 5:] = 0
  tgt = torch.randint(2, 64, (b, ld), generator=g)
  tgt[1, 4:] = 0
  dec_in = torch.cat([torch.zeros(b, 1, dtype=torch.long), tgt[:, :-1]], 1)
  return {"encoder_input_tokens": enc, "decoder_input_tokens": dec_in,
          "decoder_target_tokens": tgt, "decoder_loss_weights": (tgt > 0).float()}


def test_remove_prefix():
  seq = torch.tensor([[1, 2, 3, 4, 5, 0], [6, 7, 8, 9, 0, 0]])
  out = base.remove_prefix(seq, torch.tensor([2, 1]))
  assert out.tolist() == [[3, 4, 5, 0, 0, 0], [7, 8, 9, 0, 0, 0]]
  assert base.remove_prefix(seq, torch.tensor([0, 0])).tolist() == seq.tolist()
  three = torch.stack([seq, seq + 10], dim=1)   # [batch, decodes, len]
  out = base.remove_prefix(three, torch.tensor([2, 1]))
  assert out[0].tolist() == [[3, 4, 5, 0, 0, 0], [13, 14, 15, 10, 0, 0]]
  assert out[1].tolist() == [[7, 8, 9, 0, 0, 0], [17, 18, 19, 10, 10, 0]]


def test_count_packed_examples():
  seg = torch.tensor([[1, 1, 2, 2, 3, 0], [1, 1, 1, 1, 1, 1], [0, 0, 0, 0, 0, 0]])
  assert int(base.count_packed_examples(seg)) == 4


def test_initial_variables_carry_shapes_and_axis_names():
  model = _model()
  variables = model.get_initial_variables(0, {"encoder_input_tokens": (2, 8)})
  flat = tree.flatten_dict(variables["params"])
  axes = tree.flatten_dict(variables["params_axes"], is_leaf=lambda x: not isinstance(x, dict))
  assert set(flat) == set(axes)
  assert tuple(flat["token_embedder/embedding"].shape) == (64, 32)
  assert tuple(axes["token_embedder/embedding"]) == ("vocab", "embed")
  assert tuple(flat["encoder/layers_0/attention/query/kernel"].shape) == (32, 32)
  assert tuple(axes["encoder/layers_0/attention/query/kernel"]) == ("embed", "joined_kv")
  assert tuple(axes["decoder/layers_1/mlp/wo/kernel"]) == ("mlp", "embed")
  # a seed decides the values
  a = flat["decoder/layers_0/mlp/wi_0/kernel"].detach().clone()
  b = tree.flatten_dict(model.get_initial_variables(0, None)["params"])[
      "decoder/layers_0/mlp/wi_0/kernel"]
  torch.testing.assert_close(a, b)


@pytest.mark.parametrize("z_loss,smoothing", [(0.0, 0.0), (1e-3, 0.0), (0.0, 0.1)])
def test_loss_fn_matches_a_hand_computed_cross_entropy(z_loss, smoothing):
  model = _model(z_loss=z_loss, label_smoothing=smoothing)
  batch = _batch()
  loss, metrics = model.loss_fn(None, batch, None)
  logits = model._compute_logits(None, batch).double()
  logp = torch.log_softmax(logits, -1)
  tgt, w = batch["decoder_target_tokens"], batch["decoder_loss_weights"].double()
  v = logits.shape[-1]
  conf, low = 1.0 - smoothing, smoothing / (v - 1)
  soft = torch.full_like(logp, low).scatter_(-1, tgt[..., None], conf)
  ce = -(soft * logp).sum(-1)
  if smoothing:
    import math
    ce = ce + (conf * math.log(conf) + (v - 1) * low * math.log(low + 1e-20))
  z = z_loss * torch.logsumexp(logits, -1) ** 2
  want = ((ce + z) * w).sum()
  assert float(loss.detach()) == pytest.approx(float(want), rel=1e-4)
  assert {"accuracy", "loss", "loss_per_nonpadding_target_token", "timing/seqs_per_second",
          "non_padding_fraction/loss_weights"} <= set(metrics)
  acc = (logits.argmax(-1) == tgt).double().mul(w).sum() / w.sum()
  assert float(metrics["accuracy"].compute()) == pytest.approx(100.0 * float(acc), rel=1e-5)
  if z_loss:
    assert float(metrics["z_loss"].compute_value().value) == pytest.approx(float((z * w).sum()),
                                                                          rel=1e-3)


def test_score_batch_is_the_sum_of_target_log_probabilities():
  model = _model()
  batch = _batch()
  scores, inter = model.score_batch(None, batch, return_intermediates=True)
  logp = torch.log_softmax(model._compute_logits(None, batch).double(), -1)
  tok = logp.gather(-1, batch["decoder_target_tokens"][..., None])[..., 0]
  want = (tok * batch["decoder_loss_weights"].double()).sum(-1)
  torch.testing.assert_close(scores.double(), want, rtol=1e-4, atol=1e-4)
  assert scores.shape == (3,) and (scores < 0).all()
  torch.testing.assert_close(inter["decoder"]["token_scores"][0].double().sum(-1), want,
                             rtol=1e-4, atol=1e-4)
  assert inter["decoder"]["target_tokens"][0] is not None
  torch.testing.assert_close(model.score_batch(None, batch), scores)


def test_cached_greedy_decode_equals_a_full_forward_pass_per_step():
  """Decoding with the key / value cache must pick, at every position, the arg-max of a full
  teacher-forced forward pass over what has been decoded so far."""
  model = _model(decode_fn=functools.partial(decoding.temperature_sample, temperature=0.0))
  batch = _batch(ld=8)
  decoded, aux = model.predict_batch_with_aux(None, batch, num_decodes=1, rng=0)
  enc = batch["encoder_input_tokens"]
  b, ld = decoded.shape
  seq = torch.zeros(b, ld, dtype=torch.long)
  done = torch.zeros(b, dtype=torch.bool)
  for t in range(ld):
    dec_in = torch.cat([torch.zeros(b, 1, dtype=torch.long), seq[:, :-1]], 1)
    logits = model._compute_logits(None, {
        "encoder_input_tokens": enc, "decoder_input_tokens": dec_in,
        "decoder_target_tokens": torch.ones_like(seq)})   # targets only mark valid positions
    nxt = logits[:, t].argmax(-1)
    seq[:, t] = torch.where(done, torch.zeros_like(nxt), nxt)
    done |= nxt == 1
  assert decoded.tolist() == seq.tolist()
  assert aux["scores"].shape == (b,)


def test_beam_search_returns_all_decodes_in_ascending_score_order():
  model = _model()
  batch = _batch()
  decodes, aux = model.predict_batch_with_aux(None, batch, return_all_decodes=True, num_decodes=3)
  assert decodes.shape == (3, 3, 6) and aux["scores"].shape == (3, 3)
  assert (aux["scores"][:, 1:] >= aux["scores"][:, :-1]).all()
  best, best_aux = model.predict_batch_with_aux(None, batch, num_decodes=3)
  assert best.tolist() == decodes[:, -1].tolist()
  torch.testing.assert_close(best_aux["scores"], aux["scores"][:, -1])
  assert model.predict_batch(None, batch).shape == (3, 6)


def test_sampling_is_decided_by_the_seed():
  sample = functools.partial(decoding.temperature_sample, temperature=1.0, topk=0)
  model = _model(decode_fn=sample)
  batch = _batch(b=4, ld=10)
  a, _ = model.predict_batch_with_aux(None, batch, rng=7)
  b, _ = model.predict_batch_with_aux(None, batch, rng=7)
  c, _ = model.predict_batch_with_aux(None, batch, rng=8)
  assert a.tolist() == b.tolist()
  assert a.tolist() != c.tolist()
  many, aux = model.predict_batch_with_aux(None, batch, rng=7, num_decodes=3,
                                           return_all_decodes=True)
  assert many.shape == (4, 3, 10) and aux["scores"].shape == (4, 3)


def test_prompt_with_targets_keeps_the_prompt_and_continues_it():
  model = _model()
  batch = _batch(ld=8)
  prompt = torch.zeros(3, 8, dtype=torch.long)
  prompt[0, 1:4] = torch.tensor([9, 10, 11])     # BOS + three prompt tokens
  prompt[1, 1:2] = torch.tensor([20])
  batch = {**batch, "decoder_input_tokens": prompt}
  out, _ = model.predict_batch_with_aux(None, batch, num_decodes=1, prompt_with_targets=True)
  assert out[0, :3].tolist() == [9, 10, 11] and out[1, :1].tolist() == [20]
  free, _ = model.predict_batch_with_aux(None, batch, num_decodes=1, prompt_with_targets=False)
  # row 2 has no prompt: both calls decode it the same way
  assert out[2].tolist() == free[2].tolist()
