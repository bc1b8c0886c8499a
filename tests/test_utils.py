"""`t5x_b200.utils`: zero batches, model-info log, axis-name overrides, checkpoint-step
arithmetic, restore-config resolution, train-state initialisation from scratch / checkpoints,
the inference function, vocabulary rounding, learning-rate schedules and tree helpers
(the behaviours that t5x/utils_test.py pins down)."""
import os
import types

import numpy as np
import pytest
import torch

from t5x_b200 import adafactor, checkpoints, models, partitioning
from t5x_b200 import train_state as ts_lib
from t5x_b200.data import vocabularies
from t5x_b200.models.t5 import network
from t5x_b200.utils import core, data as data_utils, schedules, tree


def _model(seed=0):
  cfg = network.T5Config(vocab_size=128, dtype="float32", emb_dim=64, num_heads=2,
                         num_encoder_layers=1, num_decoder_layers=1, head_dim=32, mlp_dim=128,
                         mlp_activations=("gelu", "linear"), dropout_rate=0.0)
  module = network.Transformer(cfg)
  vocab = vocabularies.PassThroughVocabulary(128)
  opt = adafactor.Adafactor(decay_rate=0.8, step_offset=0,
                            logical_factor_rules=adafactor.standard_logical_factor_rules())
  return models.EncoderDecoderModel(module, vocab, vocab, opt)


# ---- zero batches ---------------------------------------------------------------------------
def test_get_zeros_batch_like_spec():
  spec = {"encoder_input_tokens": types.SimpleNamespace(shape=(4, 7), dtype=np.int32),
          "decoder_loss_weights": types.SimpleNamespace(shape=(4, 3), dtype=np.float32)}
  out = data_utils.get_zeros_batch_like_spec(spec)
  assert set(out) == set(spec)
  assert out["encoder_input_tokens"].shape == (4, 7) and out["encoder_input_tokens"].dtype == np.int32
  assert out["decoder_loss_weights"].dtype == np.float32 and not out["decoder_loss_weights"].any()


def test_get_zeros_batch_like_dataset_overrides_the_batch_dimension():
  ds = types.SimpleNamespace(element_spec={
      "inputs": types.SimpleNamespace(shape=(None, 5), dtype=np.int32),
      "targets": types.SimpleNamespace(shape=(None, 2), dtype=np.int32)})
  out = data_utils.get_zeros_batch_like_dataset(ds, batch_size=6)
  assert out["inputs"].shape == (6, 5) and out["targets"].shape == (6, 2)


# ---- model info -----------------------------------------------------------------------------
def test_log_model_info_lists_every_variable_and_the_total(tmp_path):
  model = _model()
  state = ts_lib.FlaxOptimTrainState.create(model.optimizer_def,
                                            model.get_initial_variables(0, None))
  part = partitioning.PjitPartitioner(num_partitions=1)
  log_file = str(tmp_path / "model-info.txt")
  core.log_model_info(log_file, state, part)
  lines = open(log_file).read().splitlines()
  flat = tree.flatten_dict(state.params)
  named = [l for l in lines if l.startswith("Variable ") and "param_states/" not in l]
  assert len(named) == len(flat)
  total = sum(int(np.prod(p.shape)) for p in flat.values())
  assert f"Total number of parameters: {total}" in lines
  emb = next(l for l in named if "token_embedder/embedding" in l)
  assert "vocab=128" in emb and "embed=64" in emb and f"size {128 * 64}" in emb
  # optimizer slots follow, one line each
  assert any(l.startswith("Variable param_states/") and "v_row" in l for l in lines)


# ---- axis-name overrides ----------------------------------------------------------------------
def test_override_params_axes_names():
  variables = {
      "params": {"logits_dense": torch.zeros(2, 4),
                 "mlp": {"wo": {"kernel": torch.zeros(4, 6), "bias": torch.zeros(6),
                                "embedding": torch.zeros(2, 3, 5)}}},
      "params_axes": {"logits_dense": ("vocab", "embed"),
                      "mlp": {"wo": {"kernel": ("embed", "mlp"), "bias": ("mlp",),
                                     "embedding": ("a", "b", "c")}}}}
  out = data_utils.override_params_axes_names(
      variables, [("mlp/wo/kernel", ("embed_2", "mlp_2")), (".*/embedding", ("x", "y", "z")),
                  ("mlp/wo/kern", ("never", "matches"))])  # full match only
  assert out["params_axes"]["mlp"]["wo"]["kernel"] == ("embed_2", "mlp_2")
  assert out["params_axes"]["mlp"]["wo"]["embedding"] == ("x", "y", "z")
  assert out["params_axes"]["mlp"]["wo"]["bias"] == ("mlp",)
  assert out["params_axes"]["logits_dense"] == ("vocab", "embed")
  with pytest.raises(ValueError, match="does not match param rank"):
    data_utils.override_params_axes_names(variables, [("mlp/wo/bias", ("a", "b"))])
  with pytest.raises(ValueError, match="params_axes"):
    data_utils.override_params_axes_names({"params": {}}, [])


# ---- checkpoint-step arithmetic -----------------------------------------------------------------
def test_find_next_and_first_checkpoint_step():
  nxt = data_utils.find_next_checkpoint_step
  assert nxt(0, 100, 0, None) == (100, None, 0)
  assert nxt(100, 100, 0, None) == (200, None, 0)
  assert nxt(150, 100, 0, [120, 160, 500]) == (200, 160, 1)
  assert nxt(160, 100, 1, [120, 160, 500]) == (200, 500, 2)
  assert nxt(700, None, 2, [120, 160, 500]) == (None, None, 3)
  first = data_utils.find_first_checkpoint_step
  assert first(0, None) == (None, 0)
  assert first(130, [500, 120, 160]) == (160, 1)
  assert first(160, [120, 160, 500]) == (160, 1)
  assert first(900, [120, 160, 500]) == (None, 3)


def test_round_vocab_size_and_flatten_lists():
  assert core.round_vocab_size_to_multiple(types.SimpleNamespace(vocab_size=32100)) == 32128
  assert core.round_vocab_size_to_multiple(types.SimpleNamespace(vocab_size=256), 128) == 256
  assert core.round_vocab_size_to_multiple(types.SimpleNamespace(vocab_size=5), 16) == 16
  assert core.flatten_lists([[1, 2], [], [3]]) == [1, 2, 3]


# ---- restore configs and train-state initialisation ----------------------------------------------
def _initializer(model, part):
  return core.TrainStateInitializer(
      optimizer_def=model.optimizer_def, init_fn=model.get_initial_variables,
      input_shapes={"encoder_input_tokens": (2, 8), "decoder_input_tokens": (2, 8)},
      partitioner=part)


def _save(state, part, directory, step, bump):
  """Writes `checkpoint_<step>` with every weight shifted by `bump`."""
  with torch.no_grad():
    for p in tree.flatten_dict(state.params).values():
      p.add_(bump)
  ck = checkpoints.Checkpointer(state, part, str(directory))
  ck.save(state.replace_step(step))


def test_restore_config_validation_and_resolution(tmp_path):
  with pytest.raises(ValueError, match="mode"):
    core.RestoreCheckpointConfig(path="x", mode="newest")
  with pytest.raises(ValueError, match="dtype"):
    core.RestoreCheckpointConfig(path="x", dtype="int8")
  with pytest.raises(ValueError, match="dtype"):
    core.SaveCheckpointConfig(dtype="float16")
  model, part = _model(), partitioning.PjitPartitioner(num_partitions=1)
  state = ts_lib.FlaxOptimTrainState.create(model.optimizer_def,
                                            model.get_initial_variables(0, None))
  empty, full = tmp_path / "empty", tmp_path / "full"
  empty.mkdir()
  _save(state, part, full, 3, 0.0)
  _save(state, part, full, 9, 0.0)
  get = core.get_first_valid_restore_config_and_paths
  # 'specific' is taken at its word; 'latest' / 'all' skip directories without checkpoints
  cfg, paths = get([core.RestoreCheckpointConfig(path=str(full / "checkpoint_3"), mode="specific")])
  assert paths == [str(full / "checkpoint_3")]
  cfgs = [core.RestoreCheckpointConfig(path=str(empty), mode="latest"),
          core.RestoreCheckpointConfig(path=str(full), mode="latest")]
  cfg, paths = get(cfgs)
  assert cfg is cfgs[1] and paths == [str(full / "checkpoint_9")]
  cfg, paths = get([core.RestoreCheckpointConfig(path=str(full), mode="all")])
  assert paths == [str(full / "checkpoint_3"), str(full / "checkpoint_9")]
  assert get([core.RestoreCheckpointConfig(path=str(empty), mode="all")]) == (None, [])
  with pytest.raises(ValueError, match="valid directories"):
    get([core.RestoreCheckpointConfig(path=str(tmp_path / "missing"), mode="latest")])


def test_train_state_initializer_from_scratch_and_from_checkpoints(tmp_path):
  model, part = _model(), partitioning.PjitPartitioner(num_partitions=1)
  init = _initializer(model, part)
  scratch = init.from_scratch(init_rng=11)
  assert int(scratch.step) == 0
  key = "encoder/layers_0/mlp/wo/kernel"
  base = tree.flatten_dict(scratch.params)[key].detach().clone()
  again = tree.flatten_dict(init.from_scratch(init_rng=11).params)[key]
  torch.testing.assert_close(again, base)  # the seed decides the values
  other = tree.flatten_dict(init.from_scratch(init_rng=12).params)[key].detach().clone()
  assert not torch.allclose(other, base)

  ckpt_dir = tmp_path / "ckpts"
  state = init.from_scratch(init_rng=11)
  _save(state, part, ckpt_dir, 5, 1.0)   # weights = base + 1
  _save(state, part, ckpt_dir, 8, 1.0)   # weights = base + 2
  latest = core.RestoreCheckpointConfig(path=str(ckpt_dir), mode="latest")
  restored = init.from_checkpoint([latest], init_rng=0)
  assert int(restored.step) == 8
  torch.testing.assert_close(tree.flatten_dict(restored.params)[key], base + 2.0)
  # 'all' yields every checkpoint in step order, each with its path
  got = [(int(s.step), os.path.basename(p)) for s, p in init.from_checkpoints(
      [core.RestoreCheckpointConfig(path=str(ckpt_dir), mode="all")])]
  assert got == [(5, "checkpoint_5"), (8, "checkpoint_8")]
  with pytest.raises(ValueError, match="at most 1 checkpoint"):
    init.from_checkpoint([core.RestoreCheckpointConfig(path=str(ckpt_dir), mode="all")])
  # nothing to restore: scratch
  empty = tmp_path / "empty"
  empty.mkdir()
  fresh = init.from_checkpoint_or_scratch(
      [core.RestoreCheckpointConfig(path=str(empty), mode="latest")], init_rng=11)
  assert int(fresh.step) == 0
  torch.testing.assert_close(tree.flatten_dict(fresh.params)[key], base)
  assert init.from_checkpoint([core.RestoreCheckpointConfig(path=str(empty), mode="latest")]) is None


def test_fallback_state_rules():
  cfg = core.RestoreCheckpointConfig(path="x", fallback_to_scratch=True)
  with pytest.raises(ValueError, match="state_transformation_fns"):
    core.get_fallback_state(cfg, lambda rng: {}, 0)
  cfg = core.RestoreCheckpointConfig(path="x", fallback_to_scratch=True,
                                     assignment_map=[("a", "b")])
  with pytest.raises(ValueError, match="init_rng"):
    core.get_fallback_state(cfg, lambda rng: {}, None)
  assert core.get_fallback_state(cfg, lambda rng: {"seed": rng}, 4) == {"seed": 4}
  assert core.get_fallback_state(core.RestoreCheckpointConfig(path="x"), lambda rng: 1 / 0, 0) is None
  assert core.get_fallback_state(None, lambda rng: 1 / 0, 0) is None


# ---- inference function ------------------------------------------------------------------------
@pytest.mark.parametrize("n_examples", [1, 4, 7])
def test_get_infer_fn_pads_batches_and_keeps_dataset_order(n_examples):
  calls = []

  def step(params, batch, rng):
    calls.append(tuple(batch["x"].shape))
    x = batch["x"].float()
    return x.sum(dim=1) * params["scale"], {"rows": x[:, 0]}

  infer_fn = data_utils.get_infer_fn(step, batch_size=4, train_state_axes=None, partitioner=None)
  ds = [(i, {"x": np.full((3,), i + 1, np.int32)}) for i in range(n_examples)]
  state = types.SimpleNamespace(params={"scale": 2.0})
  result, aux = infer_fn(ds, state)
  assert [i for i, _ in result] == list(range(n_examples))
  assert [float(o) for _, o in result] == [6.0 * (i + 1) for i in range(n_examples)]
  assert aux["rows"] == [float(i + 1) for i in range(n_examples)]
  assert all(shape == (4, 3) for shape in calls)          # every call sees a full batch
  assert len(calls) == -(-n_examples // 4)
  assert infer_fn([], state) == []


# ---- learning-rate schedules ----------------------------------------------------------------------
def test_learning_rate_schedules():
  mk = schedules.create_learning_rate_scheduler
  fn = mk("constant * linear_warmup * rsqrt_decay", base_learning_rate=0.01, warmup_steps=100)
  assert fn(0) == 1e-8  # never below `min_learning_rate`
  assert fn(50) == pytest.approx(0.01 * 0.5 / 10.0)
  assert fn(100) == pytest.approx(0.01 / 10.0)
  assert fn(400) == pytest.approx(0.01 / 20.0)
  fn = mk("constant * rsqrt_normalized_decay", base_learning_rate=1.0, warmup_steps=16)
  assert fn(4) == pytest.approx(1.0) and fn(64) == pytest.approx(0.5)
  fn = mk("constant * decay_every", base_learning_rate=1.0, decay_factor=0.5, steps_per_decay=10)
  assert [fn(s) for s in (0, 9, 10, 25)] == [1.0, 1.0, 0.5, 0.25]
  fn = mk("constant * cosine_decay", base_learning_rate=2.0, warmup_steps=0, steps_per_cycle=100)
  assert fn(0) == pytest.approx(2.0) and fn(50) == pytest.approx(1.0) and fn(99) < 1e-3
  assert fn(100) == pytest.approx(2.0)  # the cycle starts again
  fn = mk("constant", base_learning_rate=0.3, step_offset=1000)
  assert fn(5) == 0.3
  fn = mk("constant * linear_warmup", base_learning_rate=1.0, warmup_steps=10, step_offset=100)
  assert fn(100) == 1e-8 and fn(105) == pytest.approx(0.5) and fn(50) == 1e-8
  assert mk("constant * linear_warmup", min_learning_rate=0.0)(0) == 0.0
  with pytest.raises(ValueError, match="Unknown factor"):
    mk("constant * exponential")


# ---- tree helpers ------------------------------------------------------------------------------
def test_tree_helpers():
  t = {"a": {"b": 1, "c": {"d": 2}}, "e": 3, "empty": {}}
  flat = tree.flatten_dict(t)
  assert flat == {"a/b": 1, "a/c/d": 2, "e": 3}
  assert tree.flatten_dict(t, keep_empty_nodes=True)["empty"] == {}
  assert tree.unflatten_dict(flat) == {"a": {"b": 1, "c": {"d": 2}}, "e": 3}
  assert tree.tree_map(lambda x, y: x + y, {"a": 1, "b": {"c": 2}}, {"a": 10, "b": {"c": 20}}) == \
      {"a": 11, "b": {"c": 22}}
  assert list(tree.tree_leaves({"a": 1, "b": {"c": 2, "d": (3, 4)}},
                               is_leaf=lambda x: not isinstance(x, dict))) == [1, 2, (3, 4)]
  assert core.flatten_dict_string_keys({"x": {"y": 5}}) == {"x/y": 5}


def test_orbax_tree_checkpoints_restore_through_the_initializer_and_the_manager(tmp_path):
  """A checkpoint directory in Orbax's PyTree layout (`checkpoint_<step>/state/<array dirs>`)
  restores through the same user-level calls as a native one: latest / specific modes of the
  initializer, and the checkpoint manager built for a training run."""
  model, part = _model(), partitioning.PjitPartitioner(num_partitions=1)
  init = _initializer(model, part)
  key = "encoder/layers_0/mlp/wo/kernel"
  state = init.from_scratch(init_rng=11)
  base = tree.flatten_dict(state.params)[key].detach().clone()
  ckpt_dir = tmp_path / "orbax_ckpts"
  for step in (3, 6):
    with torch.no_grad():
      for p in tree.flatten_dict(state.params).values():
        p.add_(1.0)
    checkpoints.save_state_as_orbax_tree(state.replace_step(step), str(ckpt_dir))
  assert sorted(os.listdir(ckpt_dir)) == ["checkpoint_3", "checkpoint_6"]
  assert not (ckpt_dir / "checkpoint_6" / "checkpoint").exists()   # no native index file

  with torch.no_grad():
    for p in tree.flatten_dict(state.params).values():
      p.zero_()
  latest = init.from_checkpoint([core.RestoreCheckpointConfig(path=str(ckpt_dir), mode="latest")])
  assert int(latest.step) == 6
  torch.testing.assert_close(tree.flatten_dict(latest.params)[key], base + 2.0)
  specific = init.from_checkpoint([core.RestoreCheckpointConfig(
      path=str(ckpt_dir / "checkpoint_3"), mode="specific")])
  assert int(specific.step) == 3
  torch.testing.assert_close(tree.flatten_dict(specific.params)[key], base + 1.0)

  restore_cfg = core.RestoreCheckpointConfig(path=str(ckpt_dir), mode="latest")
  save_cfg = core.SaveCheckpointConfig(period=2, keep=1)
  model_dir = tmp_path / "run"
  restored, manager = core.create_checkpoint_manager_and_restore(
      init, part, restore_cfg, str(ckpt_dir / "checkpoint_6"), 0, save_checkpoint_cfg=save_cfg,
      model_dir=str(model_dir))
  assert int(restored.step) == 6
  torch.testing.assert_close(tree.flatten_dict(restored.params)[key], base + 2.0)
  # the run then saves in the native format, which restores as well
  manager.save(restored.replace_step(8))
  manager.wait_until_finished()
  assert (model_dir / "checkpoint_8" / "checkpoint").exists()
  again = init.from_checkpoint([core.RestoreCheckpointConfig(path=str(model_dir), mode="latest")])
  assert int(again.step) == 8
  manager.close()
