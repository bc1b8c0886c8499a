"""Mesh-TensorFlow T5 checkpoint import: translation rules, placeholder slots, shared relative
position bias, and a tensor-bundle round trip (cases modelled on
t5x/checkpoint_importer_test.py)."""
import numpy as np
import pytest
import torch

from t5x_b200 import adafactor, checkpoint_importer as ci, models, train_state as ts
from t5x_b200.data import vocabularies
from t5x_b200.io import tf_bundle
from t5x_b200.models.t5 import network
from t5x_b200.utils import tree as tree_utils


def test_translation_rules():
  tr = ci.t5_importer
  flat = {
      "global_step": np.asarray(7, np.int64),
      "shared/embedding": 1, "shared/embedding_slot_vc": 2,
      "encoder/block_000/layer_000/SelfAttention/relative_attention_bias": 3,
      "encoder/block_001/layer_000/SelfAttention/q": 4,
      "decoder/block_002/layer_001/EncDecAttention/o_slot_vr": 5,
      "decoder/block_002/layer_000/SelfAttention/k": 6,
      "encoder/block_000/layer_001/DenseReluDense/wi_0/kernel": 7,
      "decoder/block_001/layer_002/DenseReluDense/wo/kernel_slot_v": 8,
      "encoder/block_003/layer_001/rms_norm/scale": 9,
      "decoder/block_003/layer_001/layer_norm/scale": 10,
      "encoder/rms_norm/scale": 11, "decoder/final_layer_norm/scale_slot_v": 12,
      "decoder/logits/kernel": 13,
      "transformer/block_000/layer_001/rms_norm/scale": 14,
  }
  out = tr.apply(flat)
  assert out["state/step"] == 7
  assert out["target/token_embedder/embedding"] == 1
  assert out["state/param_states/token_embedder/embedding/v_col"] == 2
  assert out["target/encoder/layers_0/relpos_bias/rel_embedding"] == 3
  assert out["target/encoder/layers_1/attention/query/kernel"] == 4
  assert out["state/param_states/decoder/layers_2/encoder_decoder_attention/out/kernel/v_row"] == 5
  assert out["target/decoder/layers_2/self_attention/key/kernel"] == 6
  assert out["target/encoder/layers_0/mlp/wi_0/kernel"] == 7
  assert out["state/param_states/decoder/layers_1/mlp/wo/kernel/v"] == 8
  assert out["target/encoder/layers_3/pre_mlp_layer_norm/scale"] == 9
  assert out["target/decoder/layers_3/pre_cross_attention_layer_norm/scale"] == 10
  assert out["target/encoder/encoder_norm/scale"] == 11
  assert out["state/param_states/decoder/decoder_norm/scale/v"] == 12
  assert out["target/decoder/logits_dense/kernel"] == 13
  assert out["target/decoder/layers_0/pre_mlp_layer_norm/scale"] == 14
  with pytest.raises(ValueError, match="Unmapped"):
    tr.apply({"something/else": 1})


def test_placeholders_and_shared_relpos():
  data = {"target/a/kernel": 1, "state/param_states/a/kernel/v_row": 2,
          "state/param_states/a/kernel/v_col": 3, "target/b/scale": 4,
          "state/param_states/b/scale/v": 5}
  out = ci._add_missing_param_states(dict(data))
  assert out["state/param_states/a/kernel/v"].shape == (1,)
  assert out["state/param_states/b/scale/v_row"].shape == (1,)
  assert out["state/param_states/a/kernel/m"].shape == (1,)
  shared = ci._maybe_correct_relpos_bias({"target/encoder/layers_0/relpos_bias/rel_embedding": 1})
  assert list(shared) == ["target/encoder/relpos_bias/rel_embedding"]
  per_layer = {"target/encoder/layers_0/relpos_bias/rel_embedding": 1,
               "target/encoder/layers_1/relpos_bias/rel_embedding": 2}
  assert ci._maybe_correct_relpos_bias(per_layer) == per_layer


def test_bundle_round_trip(tmp_path):
  tensors = {"a/b": np.arange(12, dtype=np.float32).reshape(3, 4),
             "global_step": np.asarray(5, np.int64), "c": np.ones((2, 2, 2), np.int32)}
  prefix = str(tmp_path / "model.ckpt-5")
  tf_bundle.write_bundle(prefix, tensors)
  r = tf_bundle.BundleReader(prefix)
  assert r.get_variable_to_shape_map() == {"a/b": (3, 4), "global_step": (), "c": (2, 2, 2)}
  for k, v in tensors.items():
    np.testing.assert_array_equal(r.get_tensor(k), v)


def _tf_names(flat_params):
  """Inverse of the importer for the dense T5.1.1 layout (test fixture only)."""
  names = {}
  for key, v in flat_params.items():
    parts = key.split("/")
    if key == "token_embedder/embedding":
      names["shared/embedding"] = v
    elif parts[1] == "relpos_bias":
      names[f"{parts[0]}/block_000/layer_000/SelfAttention/relative_attention_bias"] = v
    elif parts[1].endswith("_norm"):
      names[f"{parts[0]}/rms_norm/scale"] = v
    elif parts[1] == "logits_dense":
      names["decoder/logits/kernel"] = v
    else:
      tower, block, sub = parts[0], int(parts[1].split("_")[1]), parts[2]
      order = {"encoder": ["attention", "mlp"],
               "decoder": ["self_attention", "encoder_decoder_attention", "mlp"]}[tower]
      if sub.endswith("layer_norm"):
        norms = {"encoder": ["pre_attention_layer_norm", "pre_mlp_layer_norm"],
                 "decoder": ["pre_self_attention_layer_norm", "pre_cross_attention_layer_norm",
                             "pre_mlp_layer_norm"]}[tower]
        names[f"{tower}/block_{block:03d}/layer_{norms.index(sub):03d}/rms_norm/scale"] = v
      elif sub == "mlp":
        names[f"{tower}/block_{block:03d}/layer_{order.index(sub):03d}/DenseReluDense/"
              f"{parts[3]}/kernel"] = v
      else:
        kind = "EncDecAttention" if sub == "encoder_decoder_attention" else "SelfAttention"
        letter = {"query": "q", "key": "k", "value": "v", "out": "o"}[parts[3]]
        names[f"{tower}/block_{block:03d}/layer_{order.index(sub):03d}/{kind}/{letter}"] = v
  return names


def test_restore_model_from_tf_checkpoint(tmp_path):
  cfg = network.T5Config(vocab_size=64, emb_dim=16, num_heads=2, head_dim=8, mlp_dim=32,
                         num_encoder_layers=2, num_decoder_layers=2, dropout_rate=0.0,
                         mlp_activations=("gelu", "linear"))
  torch.manual_seed(0)
  src = network.Transformer(cfg)
  flat = {k: v.detach().numpy() for k, v in tree_utils.flatten_dict(
      models.module_param_tree(src)).items()}
  torch.manual_seed(1)
  dst = network.Transformer(cfg)
  v = vocabularies.PassThroughVocabulary(64)
  model = models.EncoderDecoderModel(dst, v, v, adafactor.Adafactor())
  state = ts.FlaxOptimTrainState.create(model.optimizer_def,
                                        model.get_initial_variables(None, None))
  # the checkpoint carries Adafactor slots next to every variable: `_slot_v` for unfactored
  # parameters, `_slot_vr` / `_slot_vc` for factored ones
  tensors = _tf_names(flat)
  slots = tree_utils.flatten_dict(state.param_states)
  by_param = {tf_name: key for key in flat
              for tf_name in _tf_names({key: flat[key]})}
  for tf_name, key in by_param.items():
    if tuple(slots[f"{key}/v"].shape) != (1,):
      tensors[tf_name + "_slot_v"] = np.full(slots[f"{key}/v"].shape, 0.5, np.float32)
    else:
      tensors[tf_name + "_slot_vr"] = np.full(slots[f"{key}/v_row"].shape, 0.25, np.float32)
      tensors[tf_name + "_slot_vc"] = np.full(slots[f"{key}/v_col"].shape, 0.75, np.float32)
  tensors["global_step"] = np.asarray(123, np.int64)
  prefix = str(tmp_path / "model.ckpt-123")
  tf_bundle.write_bundle(prefix, tensors)
  new_sd = ci.restore_from_t5_checkpoint(state.state_dict(), prefix, strict=True)
  restored = state.restore_state(new_sd)
  assert int(restored.step) == 123
  for k, want in flat.items():
    got = tree_utils.flatten_dict(restored.params)[k].detach().numpy()
    np.testing.assert_array_equal(got, want)


def test_convert_tf_checkpoint_script(tmp_path):
  """The conversion script writes a native checkpoint that restores the TF values."""
  from t5x_b200 import checkpoints, partitioning
  from t5x_b200.scripts import convert_tf_checkpoint as script
  cfg = network.T5Config(vocab_size=64, emb_dim=16, num_heads=2, head_dim=8, mlp_dim=32,
                         num_encoder_layers=2, num_decoder_layers=2, dropout_rate=0.0,
                         mlp_activations=("gelu", "linear"))
  torch.manual_seed(0)
  src = network.Transformer(cfg)
  flat = {k: v.detach().numpy() for k, v in tree_utils.flatten_dict(
      models.module_param_tree(src)).items()}
  v = vocabularies.PassThroughVocabulary(64)
  torch.manual_seed(1)
  model = models.EncoderDecoderModel(network.Transformer(cfg), v, v, adafactor.Adafactor())
  state = ts.FlaxOptimTrainState.create(model.optimizer_def,
                                        model.get_initial_variables(None, None))
  tensors = _tf_names(flat)
  slots = tree_utils.flatten_dict(state.param_states)
  for key in flat:
    for tf_name in _tf_names({key: flat[key]}):
      if tuple(slots[f"{key}/v"].shape) != (1,):
        tensors[tf_name + "_slot_v"] = np.full(slots[f"{key}/v"].shape, 0.5, np.float32)
      else:
        tensors[tf_name + "_slot_vr"] = np.full(slots[f"{key}/v_row"].shape, 0.25, np.float32)
        tensors[tf_name + "_slot_vc"] = np.full(slots[f"{key}/v_col"].shape, 0.75, np.float32)
  tensors["global_step"] = np.asarray(77, np.int64)
  prefix = str(tmp_path / "tf" / "model.ckpt-77")
  tf_bundle.write_bundle(prefix, tensors)
  out_dir = str(tmp_path / "native")
  script.convert_checkpoint(model, prefix, out_dir)
  ck = checkpoints.Checkpointer(state, partitioning.PjitPartitioner(1), out_dir)
  assert ck.all_steps() == [77]
  restored = ck.restore(step=77)
  for k, want in flat.items():
    got = tree_utils.flatten_dict(restored.params)[k].detach().numpy()
    np.testing.assert_array_equal(got, want)
