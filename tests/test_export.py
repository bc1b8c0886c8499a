"""Export of an inference bundle and loading it back (role of t5x/export_lib.py)."""
import json
import os

import numpy as np
import torch

from t5x_b200 import adafactor, checkpoints, export_lib, models, partitioning, utils
from t5x_b200 import train_state as ts
from t5x_b200.data import vocabularies
from t5x_b200.models.t5 import network


def _model(seed):
  cfg = network.T5Config(vocab_size=384, emb_dim=16, num_heads=2, head_dim=8, mlp_dim=32,
                         num_encoder_layers=1, num_decoder_layers=1, dropout_rate=0.0,
                         mlp_activations=("gelu", "linear"))
  torch.manual_seed(seed)
  v = vocabularies.ByteVocabulary()
  return models.EncoderDecoderModel(network.Transformer(cfg), v, v, adafactor.Adafactor())


def test_export_and_load(tmp_path):
  part = partitioning.PjitPartitioner(num_partitions=1, world_size=1, local_rank=0)
  model = _model(0)
  state = ts.FlaxOptimTrainState.create(model.optimizer_def,
                                        model.get_initial_variables(None, None))
  ckpt_dir = str(tmp_path / "ckpt")
  checkpoints.Checkpointer(state, part, ckpt_dir).save(state)
  bundle = export_lib.save(
      model=model, inference_mode="predict",
      restore_checkpoint_cfg=utils.RestoreCheckpointConfig(path=ckpt_dir, mode="latest"),
      partitioner=part, task_feature_lengths={"inputs": 16, "targets": 8}, batch_size=2,
      output_dir=str(tmp_path / "export"), model_name="tiny", version=1,
      export_dtype="float32")
  assert os.path.exists(os.path.join(bundle, "signature.json"))
  assert os.path.exists(os.path.join(bundle, "warmup.jsonl"))
  sig = json.load(open(os.path.join(bundle, "signature.json")))
  assert sig["inference_mode"] == "predict" and sig["batch_size"] == 2
  # a freshly built model object + the bundle reproduces the original predictions
  served = export_lib.load(bundle, _model(1), partitioner=part)
  got = served(["hello", "abc", "xyz"])
  direct = export_lib.ExportableModule(
      model, state.params,
      export_lib.create_preprocessor({"inputs": type("F", (), {"vocabulary": model.input_vocabulary,
                                                               "add_eos": True})()},
                                     {"inputs": 16, "targets": 8}),
      export_lib.create_inference_function(model=model, inference_mode="predict"),
      export_lib.create_postprocessor(model.output_vocabulary), {"inputs": 16, "targets": 8},
      batch_size=2)(["hello", "abc", "xyz"])
  assert got["outputs"] == direct["outputs"] and len(got["outputs"]) == 3
  np.testing.assert_allclose(got["scores"], direct["scores"], rtol=1e-5)
