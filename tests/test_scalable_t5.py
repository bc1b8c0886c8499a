"""scalable_t5: per-layer position biases, rematerialisation that reproduces gradients (and
dropout masks), and the scanned <-> per-layer checkpoint layout
(t5x/examples/scalable_t5/network_test.py, layers_test.py)."""
import numpy as np
import pytest
import torch

from t5x_b200 import adafactor, models
from t5x_b200.data import vocabularies
from t5x_b200.models import base
from t5x_b200.models.scalable_t5 import network as scalable
from t5x_b200.models.t5 import network as plain
from t5x_b200.utils import tree


def _config(**kw):
  args = dict(vocab_size=64, dtype="float32", emb_dim=32, num_heads=2, num_encoder_layers=2,
              num_decoder_layers=3, head_dim=16, mlp_dim=64, mlp_activations=("gelu", "linear"),
              dropout_rate=0.0)
  args.update(kw)
  return scalable.T5Config(**args)


def _batch(seed=0, b=3, le=9, ld=7):
  g = torch.Generator().manual_seed(seed)
  enc = torch.randint(2, 64, (b, le), generator=g)
  enc[0, 6:] = 0
  tgt = torch.randint(2, 64, (b, ld), generator=g)
  tgt[1, 5:] = 0
  dec_in = torch.cat([torch.zeros(b, 1, dtype=torch.long), tgt[:, :-1]], 1)
  return {"encoder_input_tokens": enc, "decoder_input_tokens": dec_in,
          "decoder_target_tokens": tgt, "decoder_loss_weights": (tgt > 0).float()}


def _model(cfg, seed=1):
  torch.manual_seed(seed)
  module = scalable.Transformer(cfg)
  vocab = vocabularies.PassThroughVocabulary(64)
  return models.EncoderDecoderModel(module, vocab, vocab, adafactor.Adafactor())


def test_every_layer_owns_a_position_bias():
  module = scalable.Transformer(_config())
  names = set(tree.flatten_dict(base.module_param_tree(module)))
  for i in range(2):
    assert f"encoder/layers_{i}/relpos_bias/rel_embedding" in names
  for i in range(3):
    assert f"decoder/layers_{i}/relpos_bias/rel_embedding" in names
  assert "encoder/relpos_bias/rel_embedding" not in names   # the plain T5 shares one per stack
  shared = set(tree.flatten_dict(base.module_param_tree(plain.Transformer(
      plain.T5Config(vocab_size=64, emb_dim=32, num_heads=2, num_encoder_layers=2,
                     num_decoder_layers=3, head_dim=16, mlp_dim=64)))))
  assert "encoder/relpos_bias/rel_embedding" in shared
  assert module.scan_layers is False          # run-time layout is per layer


def test_layers_use_their_own_bias():
  model = _model(_config())
  batch = _batch()
  before = model._compute_logits(None, batch).detach().clone()
  with torch.no_grad():
    model.module.encoder.layers_1.relpos_bias.rel_embedding.add_(1.5 * torch.randn(2, 32))
  after = model._compute_logits(None, batch)
  assert not torch.allclose(before, after)


@pytest.mark.parametrize("dropout", [0.0, 0.3])
def test_full_remat_reproduces_loss_and_gradients(dropout):
  batch = _batch()
  results = {}
  for policy in ("none", "full", "minimal"):
    model = _model(_config(remat_policy=policy, dropout_rate=dropout), seed=5)
    loss, _ = model.loss_fn(None, batch, 17 if dropout else None)
    loss.backward()
    grads = {n: p.grad.detach().clone() for n, p in model.module.named_parameters()
             if p.grad is not None}
    results[policy] = (float(loss.detach()), grads)
  for policy in ("full", "minimal"):
    assert results[policy][0] == pytest.approx(results["none"][0], rel=1e-6)
    for n, g in results["none"][1].items():
      torch.testing.assert_close(results[policy][1][n], g, rtol=1e-5, atol=1e-6)
  with pytest.raises(ValueError, match="remat_policy"):
    model = _model(_config(remat_policy="sometimes"))
    model.loss_fn(None, batch, None)[0].backward()


def test_scanned_layout_round_trip_and_shapes():
  cfg = _config()
  module = scalable.Transformer(cfg)
  params = tree.tree_map(lambda p: p.detach().clone(), base.module_param_tree(module))
  stacked = scalable.stack_layers(params, cfg.num_heads, cfg.head_dim, scan_axis=1)
  flat = tree.flatten_dict(stacked)
  assert not any("layers_" in k for k in flat)
  # kernels gain the layers axis at position 1, attention kernels are [embed, layers, heads, kv]
  assert tuple(flat["encoder/encoder/attention/query/kernel"].shape) == (32, 2, 2, 16)
  assert tuple(flat["encoder/encoder/attention/out/kernel"].shape) == (2, 2, 16, 32)
  assert tuple(flat["decoder/decoder/mlp/wi_0/kernel"].shape) == (32, 3, 64)
  assert tuple(flat["decoder/decoder/pre_mlp_layer_norm/scale"].shape) == (32, 3)   # [embed, layers]
  assert tuple(flat["decoder/decoder/relpos_bias/rel_embedding"].shape) == (2, 3, 32)
  assert tuple(flat["token_embedder/embedding"].shape) == (64, 32)
  assert "decoder/decoder_norm/scale" in flat
  # layer i of the stack is layer i of the tree
  q1 = tree.flatten_dict(params)["encoder/layers_1/attention/query/kernel"]
  torch.testing.assert_close(flat["encoder/encoder/attention/query/kernel"][:, 1].reshape(32, 32), q1)
  back = scalable.unstack_layers(stacked, cfg.num_heads, cfg.head_dim, scan_axis=1)
  flat_back, flat_orig = tree.flatten_dict(back), tree.flatten_dict(params)
  assert set(flat_back) == set(flat_orig)
  for k, v in flat_orig.items():
    torch.testing.assert_close(flat_back[k], v)
  # scan axis 0 and numpy arrays (what a checkpoint reader hands over)
  as_np = tree.tree_map(lambda t: t.numpy(), params)
  stacked0 = scalable.stack_layers(as_np, cfg.num_heads, cfg.head_dim, scan_axis=0)
  flat0 = tree.flatten_dict(stacked0)
  assert flat0["encoder/encoder/attention/query/kernel"].shape == (2, 32, 2, 16)
  back0 = tree.flatten_dict(scalable.unstack_layers(stacked0, cfg.num_heads, cfg.head_dim, 0))
  for k, v in flat_orig.items():
    np.testing.assert_allclose(np.asarray(back0[k]), v.numpy())


def test_decoding_with_per_layer_biases_matches_teacher_forcing():
  import functools
  from t5x_b200 import decoding
  cfg = _config()
  torch.manual_seed(2)
  module = scalable.Transformer(cfg)
  with torch.no_grad():
    module.token_embedder.embedding.mul_(5.0)
  vocab = vocabularies.PassThroughVocabulary(64)
  model = models.EncoderDecoderModel(
      module, vocab, vocab, adafactor.Adafactor(),
      decode_fn=functools.partial(decoding.temperature_sample, temperature=0.0))
  batch = _batch(ld=6)
  decoded, _ = model.predict_batch_with_aux(None, batch, rng=0)
  b, ld = decoded.shape
  seq = torch.zeros(b, ld, dtype=torch.long)
  done = torch.zeros(b, dtype=torch.bool)
  for t in range(ld):
    dec_in = torch.cat([torch.zeros(b, 1, dtype=torch.long), seq[:, :-1]], 1)
    logits = model._compute_logits(None, {**batch, "decoder_input_tokens": dec_in,
                                          "decoder_target_tokens": torch.ones_like(seq)})
    nxt = logits[:, t].argmax(-1)
    seq[:, t] = torch.where(done, torch.zeros_like(nxt), nxt)
    done |= nxt == 1
  assert decoded.tolist() == seq.tolist()
