"""CALM: anytime loss, exit-classifier losses, confidence measures, early-exit decoding
(behaviour of t5x/contrib/calm/models.py and decoding.py)."""
import numpy as np
import pytest
import torch

from t5x_b200 import adafactor, decoding, losses
from t5x_b200.contrib.calm import decoding as calm_decoding
from t5x_b200.contrib.calm import models as calm_models
from t5x_b200.contrib.calm import network as calm_network
from t5x_b200.data import vocabularies


def _model(layers=4, meta=False, **kw):
  cfg = calm_network.CalmT5Config(vocab_size=48, emb_dim=16, num_heads=2, head_dim=8, mlp_dim=32,
                                  num_encoder_layers=2, num_decoder_layers=layers,
                                  dropout_rate=0.0, dtype="float32", return_all_logits=True,
                                  meta_cls=meta)
  torch.manual_seed(0)
  module = calm_network.Transformer(cfg)
  v = vocabularies.PassThroughVocabulary(48)
  return calm_models.EncoderDecoderModel(module, v, v, adafactor.Adafactor(),
                                         decoder_layers=layers, **kw), module


def _batch(b=3, le=6, ld=5):
  g = torch.Generator().manual_seed(1)
  enc = torch.randint(2, 48, (b, le), generator=g)
  tgt = torch.randint(2, 48, (b, ld), generator=g)
  tgt[0, -2:] = 0
  dec_in = torch.cat([torch.zeros(b, 1, dtype=torch.long), tgt[:, :-1]], 1)
  return {"encoder_input_tokens": enc, "decoder_input_tokens": dec_in,
          "decoder_target_tokens": tgt, "decoder_loss_weights": (tgt > 0).float()}


@pytest.mark.parametrize("agg,expect", [(1, [1, 2, 3, 4]), (0, [1, 1, 1, 1]), (-1, [1, 2, 4, 8]),
                                        (2, [1, 3, 5, 7])])
def test_anytime_loss_is_the_weighted_average_of_layer_losses(agg, expect):
  model, module = _model(aggregation_weights=agg)
  batch = _batch()
  loss, metrics = model.loss_fn(None, batch, None)
  all_logits = module(batch["encoder_input_tokens"], batch["decoder_input_tokens"],
                      batch["decoder_target_tokens"], enable_dropout=False)
  assert all_logits.shape[0] == 4
  per_layer = [losses.compute_weighted_cross_entropy(
      lg, targets=batch["decoder_target_tokens"], weights=batch["decoder_loss_weights"])[0]
      for lg in all_logits]
  w = np.asarray(expect, np.float64)
  want = sum(float(l) * wi for l, wi in zip(per_layer, w)) / w.sum()
  assert float(loss) == pytest.approx(want, rel=1e-5)
  for i in range(3):
    assert f"accuracy_per_layer/layer_{i}" in metrics and f"loss_per_layer/layer_{i}" in metrics
  assert "accuracy" in metrics and "loss" in metrics
  loss.backward()
  assert module.decoder.layers_0.mlp.wo.kernel.grad is not None


def test_meta_classifier_losses():
  batch = _batch()
  for geom in (False, True):
    model, module = _model(meta=True, train_meta_cls=True, geomlike_loss=geom)
    loss, metrics = model.loss_fn(None, batch, None)
    assert torch.isfinite(loss)
    loss.backward()
    g = module.decoder.meta_cls.kernel.grad
    assert g is not None and float(g.abs().sum()) > 0
    assert "meta_accuracy/layer_0" in metrics
    assert ("meta_accuracy/multiclass" in metrics) == geom
    assert ("meta_loss/layer_0" in metrics) == (not geom)


def test_confidence_measures():
  model, _ = _model()
  logits = torch.tensor([[[2.0, 0.0, 0.0], [0.0, 0.0, 0.0]]])
  p = torch.softmax(logits, -1)
  model.conf_method = "softmax_max"
  assert torch.allclose(model.get_pred_confidence(logits=logits), p.max(-1).values)
  model.conf_method = "softmax_diff"
  srt = p.sort(-1, descending=True).values
  assert torch.allclose(model.get_pred_confidence(logits=logits), srt[..., 0] - srt[..., 1])
  model.conf_method = "state"
  a = torch.tensor([[1.0, 0.0]]); b = torch.tensor([[1.0, 1.0]])
  assert float(model.get_pred_confidence(prev_state=a, new_state=b)) == pytest.approx(2 ** -0.5)
  model.conf_method = "meta"
  assert float(model.get_pred_confidence(meta_score=torch.tensor(0.3))) == pytest.approx(0.3)
  model.conf_method = "nope"
  with pytest.raises(NotImplementedError):
    model.get_pred_confidence(logits=logits)


def test_never_confident_equals_full_decoding():
  """With a threshold no confidence reaches, every token uses all layers and the output equals
  ordinary greedy decoding."""
  batch = _batch()
  model, _ = _model(apply_early_inference=True, conf_threshold=2.0)
  dec, aux = model.predict_batch_with_aux(None, batch)
  plain, _ = _model(apply_early_inference=False)[0].predict_batch_with_aux(None, batch)
  assert torch.equal(dec, plain)
  live = dec != 0
  assert bool((aux["exits"][live] == 4).all())
  assert aux["confidences"].shape == dec.shape


def test_always_confident_exits_at_the_first_exit_and_fills_skipped_caches():
  batch = _batch()
  model, module = _model(apply_early_inference=True, conf_threshold=0.0, first_exit=1,
                         exit_interval=2)
  dec, aux = model.predict_batch_with_aux(None, batch)
  live = dec != 0
  assert bool((aux["exits"][live] == 2).all())      # first_exit + 1 layers
  # a single early-exit step leaves every layer's cache at the same position
  enc = module.encode(batch["encoder_input_tokens"], enable_dropout=False)
  cache = module.init_cache(3, 6, device=enc.device)
  state = decoding.DecodingState(cur_index=0, sequences=torch.zeros(3, 5, dtype=torch.long),
                                 cur_token=torch.zeros(3, 1, dtype=torch.long), cache=cache)
  logits, cache, conf, layer = model._compute_logits_from_slice_early_exit(
      state, None, enc, batch["encoder_input_tokens"], 5, 0.0)
  assert layer == 2 and logits.shape == (3, 48) and conf.shape == (3,)
  idx = [int(cache[f"layers_{i}"]["self_attention"]["cache_index"]) for i in range(4)]
  assert idx == [1, 1, 1, 1]
  # skipped layers hold the keys of the propagated state, not zeros
  assert float(cache["layers_3"]["self_attention"]["cached_key"][:, 0].abs().sum()) > 0


def test_min_exit_and_oracle():
  batch = _batch()
  model, _ = _model(apply_early_inference=True, conf_threshold=0.0, min_exit=3)
  _, aux = model.predict_batch_with_aux(None, batch)
  assert int(aux["exits"].max()) == 3
  model, _ = _model(apply_early_inference=True, oracle_tok_consistency=True)
  dec, aux = model.predict_batch_with_aux(None, batch)
  plain, _ = _model(apply_early_inference=False)[0].predict_batch_with_aux(None, batch)
  assert dec.shape == plain.shape and int(aux["exits"].max()) <= 4


def test_sampling_records_follow_the_sort_order():
  vocab = 6

  def tokens_to_logits(state):
    rows = state.cur_token.shape[0]
    logits = torch.full((rows, vocab), -5.0)
    logits[:, 2] = 1.0
    logits[0, 3] = 3.0          # row 0 splits its mass over two tokens: lower log-prob
    conf = torch.arange(rows, dtype=torch.float32) + 10 * float(state.cur_index)
    return logits, state.cache, conf, 3
  inputs = torch.zeros((1, 4), dtype=torch.long)
  dec, (lp, exits, confs) = calm_decoding.temperature_sample(
      inputs, {}, tokens_to_logits, eos_id=1, num_decodes=2, temperature=0.0,
      rescale_log_probs=False)
  assert dec.shape == (1, 2, 4) and exits.shape == (1, 2, 4) and confs.shape == (1, 2, 4)
  assert bool((exits == 3).all())
  # ascending by log-prob: original row 1 (confidences 1, 11, 21, ...) comes last
  assert bool(lp[0, 0] < lp[0, 1])
  assert dec[0, 0].tolist() == [3, 3, 3, 3] and dec[0, 1].tolist() == [2, 2, 2, 2]
  assert confs[0, 0].tolist() == [0.0, 10.0, 20.0, 30.0]
  assert confs[0, 1].tolist() == [1.0, 11.0, 21.0, 31.0]


def test_gin_config_builds_the_model():
  import os
  import t5x_b200
  from t5x_b200 import gin
  pkg = os.path.dirname(t5x_b200.__file__)
  gin.clear_config(clear_constants=True)
  gin.add_config_file_search_path(pkg)
  gin.add_config_file_search_path(os.path.dirname(pkg))
  try:
    gin.parse_config_files_and_bindings(
        ["t5x/contrib/calm/configs/t5_1_1_small_calm.gin"],
        ["DROPOUT_RATE = 0.0", "VOCABULARY = @seqio.PassThroughVocabulary()",
         "seqio.PassThroughVocabulary.size = 32128",
         "calm_network.CalmT5Config.emb_dim = 64", "calm_network.CalmT5Config.mlp_dim = 64",
         "calm_network.CalmT5Config.num_heads = 2", "calm_network.CalmT5Config.head_dim = 32",
         "calm_network.CalmT5Config.num_encoder_layers = 1", "NUM_DECODER_LAYERS = 2",
         "calm_network.CalmT5Config.vocab_size = 256",
         "calm_network.CalmT5Config.dtype = 'float32'"])
    from t5x_b200.gin import config as gin_config
    model = gin_config._materialize(gin.query_parameter("%MODEL"))
    assert isinstance(model, calm_models.EncoderDecoderModel)
    assert model.apply_early_inference and model.decoder_layers == 2
    assert model.module.config.return_all_logits
  finally:
    gin.clear_config(clear_constants=True)
