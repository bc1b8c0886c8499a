"""Buildable configs (`t5x_b200.fdl`), their command-line flags, and a training run configured
through them."""
import copy
import functools
import glob
import json
import os

import pytest

from t5x_b200 import config_utils, fdl
from t5x_b200 import train as train_lib


class Layer:
  def __init__(self, width: int, activation: str = "relu"):
    self.width, self.activation = width, activation


def make_model(encoder: Layer, decoder: Layer, name: str = "m", **extras):
  return {"encoder": encoder, "decoder": decoder, "name": name, **extras}


def test_build_nests_and_shares():
  shared = fdl.Config(Layer, 8)
  cfg = fdl.Config(make_model, encoder=shared, decoder=shared, name="x")
  built = fdl.build(cfg)
  assert built["encoder"] is built["decoder"] and built["encoder"].width == 8
  assert built["name"] == "x" and built["encoder"].activation == "relu"
  other = fdl.build(cfg)
  assert other["encoder"] is not built["encoder"]  # a new build makes new objects


def test_attributes_follow_the_signature():
  cfg = fdl.Config(Layer, width=4)
  assert cfg.width == 4 and cfg.activation == "relu"  # unset arguments read as their defaults
  cfg.activation = "gelu"
  assert fdl.build(cfg).activation == "gelu"
  del cfg.activation
  assert fdl.build(cfg).activation == "relu"
  with pytest.raises(AttributeError, match="no parameter 'depth'"):
    cfg.depth = 3
  with pytest.raises(TypeError):
    fdl.Config(Layer, 1, 2, 3)
  open_ended = fdl.Config(make_model, fdl.Config(Layer, 1), fdl.Config(Layer, 2))
  open_ended.anything = 5  # **extras accepts any name
  assert fdl.build(open_ended)["anything"] == 5
  with pytest.raises(AttributeError, match="no value has been set"):
    _ = fdl.Config(Layer).width


def test_partial_and_arg_factory():
  part = fdl.Partial(make_model, encoder=fdl.Config(Layer, 2), name="p")
  fn = fdl.build(part)
  assert isinstance(fn, functools.partial)
  a, b = fn(decoder=Layer(3)), fn(decoder=Layer(4))
  assert a["encoder"] is b["encoder"]  # a Config inside a Partial is built once
  fresh = fdl.Partial(make_model, encoder=fdl.ArgFactory(Layer, 2), decoder=fdl.Config(Layer, 3))
  fn = fdl.build(fresh)
  a, b = fn(), fn(name="second")
  assert a["encoder"] is not b["encoder"] and a["decoder"] is b["decoder"]
  assert b["name"] == "second"
  with pytest.raises(ValueError, match="ArgFactory inside Config"):
    fdl.build(fdl.Config(make_model, encoder=fdl.ArgFactory(Layer, 2), decoder=None))


def test_cast_copy_equality_and_printing():
  cfg = fdl.Config(make_model, encoder=fdl.Config(Layer, 2), decoder=fdl.Config(Layer, 3))
  part = fdl.cast(fdl.Partial, cfg)
  assert isinstance(part, fdl.Partial) and fdl.get_callable(part) is make_model
  assert callable(fdl.build(part))
  dup = copy.deepcopy(cfg)
  assert dup == cfg and dup.encoder is not cfg.encoder
  dup.encoder.width = 9
  assert dup != cfg and cfg.encoder.width == 2
  tweaked = fdl.copy_with(cfg, name="other")
  assert tweaked.name == "other" and cfg.name == "m"
  text = str(cfg)
  assert "Config[make_model(" in text and "width=2" in text


def test_paths_select_and_json():
  cfg = fdl.Config(make_model, encoder=fdl.Config(Layer, 2), decoder=fdl.Config(Layer, 3),
                   sizes=[1, 2, 3], table={"a": 1})
  fdl.set_by_path(cfg, "encoder.width", 16)
  fdl.set_by_path(cfg, "sizes[1]", 20)
  fdl.set_by_path(cfg, "table['a']", 7)
  assert cfg.encoder.width == 16 and cfg.sizes == [1, 20, 3] and cfg.table == {"a": 7}
  assert [n.width for n in fdl.select(cfg, Layer)] == [16, 3]
  again = fdl.load_json(fdl.dump_json(cfg))
  assert again == cfg and fdl.build(again)["encoder"].width == 16
  with pytest.raises(fdl.UnserializableValueError):
    fdl.dump_json(fdl.Config(make_model, encoder=lambda: 1, decoder=None))


def _flags(*argv):
  return train_lib.build_flag_parser("").parse_args(list(argv))


def test_flag_rules():
  spec = "t5x_b200.fiddle_configs.examples.synthetic:tiny_pretrain"
  assert not config_utils.using_fdl(_flags())
  assert config_utils.using_fdl(_flags(f"--fdl_config={spec}"))
  with pytest.raises(ValueError, match="exactly one of"):
    config_utils.config_with_fiddle(train_lib.train, _flags(f"--fdl_config={spec}",
                                                            "--gin_file=x.gin"))
  with pytest.raises(ValueError, match="exactly one of"):
    config_utils.config_with_fiddle(train_lib.train, _flags(f"--fdl_config={spec}",
                                                            "--fdl_config_file=x.json"))
  from t5x_b200 import eval as eval_lib
  with pytest.raises(ValueError, match="Expected the flags to configure function"):
    config_utils.config_with_fiddle(eval_lib.evaluate, _flags(f"--fdl_config={spec}"))
  cfg = config_utils.config_with_fiddle(
      train_lib.train, _flags(f"--fdl_config={spec}(train_steps=7)", "--fdl_set=eval_steps=1",
                              "--fdl_set=model.z_loss=0.5"))
  assert isinstance(cfg, fdl.Partial) and cfg.total_steps == 7 and cfg.eval_steps == 1
  assert cfg.model.z_loss == 0.5


def test_training_run_from_buildable_config(tmp_path):
  model_dir = str(tmp_path / "run")
  train_lib.main([
      "--fdl_config=t5x_b200.fiddle_configs.examples.synthetic:tiny_pretrain",
      f"--fdl_set=model_dir='{model_dir}'", "--fdl_set=total_steps=2",
      "--fdl_set=eval_period=2", "--fdl_set=checkpoint_cfg.save.period=2"])
  assert os.path.isdir(os.path.join(model_dir, "checkpoint_2"))
  text = open(os.path.join(model_dir, "fiddle_config.txt")).read()
  assert "Partial[train(" in text and "total_steps=2" in text
  saved = json.load(open(os.path.join(model_dir, "fiddle_config.json")))
  assert saved["__fdl__"] == "Partial" and saved["fn"].endswith(":train")
  # the written JSON configures the same run again
  flags = _flags(f"--fdl_config_file={os.path.join(model_dir, 'fiddle_config.json')}",
                 "--fdl_set=total_steps=3")
  again = config_utils.config_with_fiddle(train_lib.train, flags)
  assert again.total_steps == 3 and again.model.module.config.emb_dim == 8
  assert glob.glob(os.path.join(model_dir, "train", "events.*"))
