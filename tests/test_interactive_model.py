"""InteractiveModel on CPU (cases modelled on t5x/interactive_model_test.py)."""
import numpy as np
import torch

from t5x_b200 import adafactor, interactive_model as im, models, partitioning
from t5x_b200.data import vocabularies
from t5x_b200.models.t5 import network


def _interactive(tmp_path, ckpt=""):
  cfg = network.T5Config(vocab_size=384, emb_dim=16, num_heads=2, head_dim=8, mlp_dim=32,
                         num_encoder_layers=1, num_decoder_layers=1, dropout_rate=0.0,
                         mlp_activations=("gelu", "linear"))
  torch.manual_seed(0)
  module = network.Transformer(cfg)
  v = vocabularies.ByteVocabulary()
  model = models.EncoderDecoderModel(module, v, v, adafactor.Adafactor(learning_rate=0.05))
  part = partitioning.PjitPartitioner(num_partitions=1, world_size=1, local_rank=0)
  return im.InteractiveModel(
      batch_size=2, task_feature_lengths={"inputs": 16, "targets": 8},
      output_dir=str(tmp_path), partitioner=part, model=model, dtype="float32",
      restore_mode="specific", checkpoint_path=ckpt,
      input_shapes={"encoder_input_tokens": (2, 16), "decoder_input_tokens": (2, 8)})


EXAMPLES = [{"input": "hello", "target": "world"}, {"input": "abc", "target": "de"},
            {"input": "x", "target": "y"}]


def test_batches_from_text():
  v = vocabularies.ByteVocabulary()
  from t5x_b200.data import feature_converters as fc
  batches = im.get_batches_from_seqio("t", {"inputs": 16, "targets": 8}, 2, EXAMPLES,
                                      fc.EncDecFeatureConverter(pack=False), (v, v), fill=True)
  assert len(batches) == 2
  b = batches[0]
  assert b["encoder_input_tokens"].shape == (2, 16) and b["decoder_target_tokens"].shape == (2, 8)
  assert b["decoder_input_tokens"][0, 0] == 0
  assert v.decode([int(t) for t in b["encoder_input_tokens"][0] if t > 1]) == "hello"


def test_train_predict_score_evaluate(tmp_path):
  m = _interactive(tmp_path)
  s0 = m.score(EXAMPLES)
  assert len(s0) == 3 and all(np.isfinite(s0))
  for _ in range(3):
    m.train_step(EXAMPLES[:2])
  assert m.step == 3
  assert "loss" in m.train_summary
  s1 = m.score(EXAMPLES[:2])
  assert sum(s1) > sum(s0[:2])  # training on these examples raised their likelihood
  preds, aux = m.predict_with_aux(EXAMPLES)
  assert len(preds) == 3 and all(isinstance(p, str) for p in preds) and len(aux["scores"]) == 3

  def accuracy(targets, predictions):
    return {"acc": float(np.mean([t == p for t, p in zip(targets, predictions)]))}

  def mean_score(targets, scores):
    return {"mean_score": float(np.mean(scores))}

  res = m.evaluate(EXAMPLES, [accuracy, mean_score])
  assert set(res) == {"acc", "mean_score"}
  m.save_checkpoint()
  m2 = _interactive(tmp_path / "second", ckpt=str(tmp_path / "checkpoint_3"))
  assert m2.step == 3
  np.testing.assert_allclose(m2.score(EXAMPLES[:2]), s1, rtol=1e-5)
  cfg = im.get_gin_config_from_interactive_model(
      m2, im.T5XScriptType.FINETUNING, "my_task", "", "", train_steps=5)
  assert "TRAIN_STEPS = 8" in cfg and "finetune.gin" in cfg
