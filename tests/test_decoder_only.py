"""Decoder-only network and `DecoderOnlyModel` (cases modelled on t5x/models_test.py and
t5x/examples/decoder_only/network_test.py): loss, scoring, prefix-LM masks, prefilled
generation against teacher forcing."""
import numpy as np
import pytest
import torch

from t5x_b200 import adafactor
from t5x_b200 import decoding
from t5x_b200 import models
from t5x_b200.data import feature_converters, vocabularies
from t5x_b200.models.decoder_only import network


def _model(bidir=False, **kw):
  torch.manual_seed(0)
  cfg = network.TransformerConfig(vocab_size=32, emb_dim=16, num_heads=2, head_dim=8, mlp_dim=32,
                                  num_layers=2, dropout_rate=0.0,
                                  mlp_activations=("gelu", "linear"), **kw)
  module = network.DecoderWrapper(cfg)
  return models.DecoderOnlyModel(module, vocabularies.PassThroughVocabulary(32),
                                 adafactor.Adafactor(), inputs_bidirectional_attention=bidir)


def _batch():
  # inputs [9,4,6,1] + targets [3,9,1] as laid out by the decoder feature converter
  tgt = torch.tensor([[9, 4, 6, 1, 3, 9, 1, 0, 0], [5, 7, 1, 8, 2, 1, 0, 0, 0]])
  inp = torch.cat([torch.zeros(2, 1, dtype=torch.long), tgt[:, :-1]], 1)
  inp[1, 6:] = 0
  ca = torch.tensor([[1, 1, 1, 1, 1, 0, 0, 0, 0], [1, 1, 1, 1, 0, 0, 0, 0, 0]])
  w = torch.tensor([[0, 0, 0, 0, 1, 1, 1, 0, 0], [0, 0, 0, 1, 1, 1, 0, 0, 0]]).float()
  return {"decoder_input_tokens": inp, "decoder_target_tokens": tgt,
          "decoder_causal_attention": ca, "decoder_loss_weights": w}


def test_param_tree_names():
  m = _model()
  v = m.get_initial_variables(0, {"decoder_input_tokens": (2, 9)})
  dec = v["params"]["decoder"]
  assert set(dec) == {"token_embedder", "relpos_bias", "layers_0", "layers_1", "decoder_norm",
                      "logits_dense"}
  assert set(dec["layers_0"]) == {"pre_self_attention_layer_norm", "self_attention",
                                  "pre_mlp_layer_norm", "mlp"}
  assert v["params_axes"]["decoder"]["logits_dense"]["kernel"] == ("embed", "vocab")


def test_loss_and_score_agree():
  m = _model()
  b = _batch()
  loss, metrics = m.loss_fn(None, b, None)
  scores = m.score_batch(None, b)
  assert scores.shape == (2,)
  np.testing.assert_allclose(float(loss), float(-scores.sum()), rtol=1e-4)
  assert "accuracy" in metrics


def test_causal_masking_ignores_future():
  m = _model()
  b = _batch()
  logits = m._compute_logits(None, b)
  b2 = dict(b)
  it = b["decoder_input_tokens"].clone()
  tt = b["decoder_target_tokens"].clone()
  it[:, 5], tt[:, 4] = 11, 11  # change a later position
  b2["decoder_input_tokens"], b2["decoder_target_tokens"] = it, tt
  logits2 = m._compute_logits(None, b2)
  torch.testing.assert_close(logits[:, :4], logits2[:, :4])
  assert not torch.allclose(logits[:, 5], logits2[:, 5])


def test_prefix_lm_sees_whole_prefix():
  m = _model(bidir=True)
  b = _batch()
  logits = m._compute_logits(None, b)
  b2 = dict(b)
  it = b["decoder_input_tokens"].clone()
  it[0, 3] = 12  # inside the prefix of row 0: position 0 may look at it
  b2["decoder_input_tokens"] = it
  logits2 = m._compute_logits(None, b2)
  assert not torch.allclose(logits[0, 0], logits2[0, 0])
  with pytest.raises(ValueError):
    m._compute_logits(None, {k: v for k, v in b.items() if k != "decoder_causal_attention"})


@pytest.mark.parametrize("bidir", [False, True])
def test_prefilled_greedy_decode_matches_teacher_forcing(bidir):
  m = _model(bidir=bidir)
  m._decode_fn = lambda **kw: decoding.temperature_sample(topk=1, **kw)
  b = _batch()
  out, aux = m.predict_batch_with_aux(None, b)
  assert out.shape == (2, 9) and aux["scores"].shape == (2,)
  # replay: feed prompt + generated tokens with teacher forcing, argmax must reproduce them
  for row in range(2):
    n_prompt = int((b["decoder_input_tokens"][row] * b["decoder_causal_attention"][row])[1:]
                   .ne(0).sum())
    gen = out[row].tolist()
    seq_in = (b["decoder_input_tokens"][row] * b["decoder_causal_attention"][row]).clone()
    k = 0
    while n_prompt + 1 + k < 9 and k < len(gen) and gen[k] != 0:
      seq_in[n_prompt + 1 + k] = gen[k]
      k += 1
    tgt = torch.cat([seq_in[1:], torch.zeros(1, dtype=torch.long)])
    fb = {"decoder_input_tokens": seq_in[None], "decoder_target_tokens": tgt[None].clamp(min=0),
          "decoder_causal_attention": b["decoder_causal_attention"][row][None]}
    fb["decoder_target_tokens"] = torch.where(torch.arange(9)[None] <= n_prompt + k,
                                              torch.ones_like(fb["decoder_target_tokens"]),
                                              torch.zeros_like(fb["decoder_target_tokens"]))
    logits = m._compute_logits(None, fb)
    pred = logits[0].argmax(-1)
    for j in range(k):
      assert int(pred[n_prompt + j]) == gen[j], (row, j, pred.tolist(), gen)


def test_feature_converter_default():
  assert _model().FEATURE_CONVERTER_CLS is feature_converters.DecoderFeatureConverter
