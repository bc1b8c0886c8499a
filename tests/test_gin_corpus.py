"""Every shipped gin file parses, and the model files bind the published dimensions."""
import glob
import os

import pytest

import t5x_b200
from t5x_b200 import gin

PKG = os.path.dirname(t5x_b200.__file__)
MODEL_FILES = sorted(
    glob.glob(os.path.join(PKG, "examples", "t5", "*", "*.gin")) +
    glob.glob(os.path.join(PKG, "examples", "decoder_only", "models", "*.gin")))
RUN_FILES = sorted(glob.glob(os.path.join(PKG, "configs", "runs", "*.gin")))


@pytest.fixture(autouse=True)
def _fresh():
  gin.clear_config(clear_constants=True)
  gin.add_config_file_search_path(PKG)
  gin.add_config_file_search_path(os.path.dirname(PKG))
  yield
  gin.clear_config(clear_constants=True)


@pytest.mark.parametrize("path", MODEL_FILES, ids=lambda p: os.path.relpath(p, PKG))
def test_model_file_parses(path):
  gin.parse_config_files_and_bindings([path], ["DROPOUT_RATE = 0.1"])
  cfg = "network.TransformerConfig" if "decoder_only" in path else "network.T5Config"
  emb = gin.query_parameter(f"{cfg}.emb_dim")
  heads = gin.query_parameter(f"{cfg}.num_heads")
  assert emb > 0 and heads > 0 and gin.query_parameter(f"{cfg}.vocab_size") % 128 == 0


def test_published_xxl_dimensions():
  gin.parse_config_files_and_bindings(["t5x/examples/t5/t5_1_1/xxl.gin"], ["DROPOUT_RATE = 0.0"])
  q = lambda n: gin.query_parameter(f"network.T5Config.{n}")
  assert (q("emb_dim"), q("num_heads"), q("head_dim"), q("mlp_dim"), q("num_encoder_layers"),
          q("num_decoder_layers"), q("vocab_size")) == (4096, 64, 64, 10240, 24, 24, 32128)
  assert tuple(q("mlp_activations")) == ("gelu", "linear")


@pytest.mark.parametrize("path", RUN_FILES, ids=os.path.basename)
def test_run_file_parses(path):
  from t5x_b200 import eval as eval_lib, infer, precompile, train
  main = {"pretrain.gin": train, "finetune.gin": train, "precompile.gin": precompile,
          "eval.gin": eval_lib, "infer.gin": infer, "infer_from_tfexample_file.gin": infer,
          "partitioner_defaults.gin": train}.get(os.path.basename(path), train)
  gin.set_main_module(main)
  files = ["t5x/examples/t5/t5_1_1/tiny.gin", path]
  gin.parse_config_files_and_bindings(files, ["DROPOUT_RATE = 0.0"], finalize_config=False)
  assert gin.query_parameter("partitioning.PjitPartitioner.num_partitions") == 1


def _main_module_for(path):
  from t5x_b200 import eval as eval_lib, infer, precompile, train
  base = os.path.basename(path)
  if "eval" in base and "train_eval" not in base:
    return eval_lib
  if "infer" in base:
    return infer
  if "precompile" in base:
    return precompile
  return train


# Every other shipped file: the GPU-contrib tree, scalable_t5 / uMT5, the example runs and the
# MoE run files. Model files need DROPOUT_RATE; run files and examples parse on top of the
# model they include (or of a tiny model when they are pure run files).
_COVERED = set(MODEL_FILES) | set(RUN_FILES)
OTHER_FILES = sorted(p for p in glob.glob(os.path.join(PKG, "**", "*.gin"), recursive=True)
                     if p not in _COVERED)


@pytest.mark.parametrize("path", OTHER_FILES, ids=lambda p: os.path.relpath(p, PKG))
def test_every_other_gin_file_parses(path):
  rel = os.path.relpath(path, PKG)
  gin.set_main_module(_main_module_for(path))
  text = open(path).read()
  files = [path]
  pure_run = ("/runs/" in rel.replace(os.sep, "/") and "umt5" not in rel)
  fragment = any(s in rel for s in ("umt5/architectures", "umt5/optimizer", "umt5/vocab",
                                    "umt5/runs", "adamw_opt", "local_tiny", "encdec_common"))
  if fragment:
    # fragments are meant to be included next to a model: check them in such a composition
    model = ("t5x/examples/scalable_t5/mt5/small.gin" if "scalable_t5" in rel
             else "t5x/examples/t5/t5_1_1/tiny.gin")
    run = "t5x/configs/runs/pretrain.gin" if "finetuning_common" not in rel else None
    files = [model] + ([run] if run and "umt5/runs" not in rel else []) + [path]
    if "umt5/architectures" in rel:
      files.append("t5x/examples/scalable_t5/umt5/vocab.gin")
  elif pure_run:
    model = ("t5x/contrib/moe/configs/models/switch_base.gin" if "contrib/moe" in rel
             else "t5x/examples/t5/t5_1_1/tiny.gin")
    files = [model, path]
  gin.parse_config_files_and_bindings(files, ["DROPOUT_RATE = 0.0"], finalize_config=False)
  assert "include" in text or "=" in text


def test_optax_names_bind_gradient_transformations():
  from t5x_b200 import optimizers
  gin.parse_config_files_and_bindings(
      ["t5x/examples/t5/t5_1_1/tiny.gin", "t5x/contrib/gpu/t5/t5_1_1/adamw_opt.gin"],
      ["DROPOUT_RATE = 0.0"], finalize_config=False)
  from t5x_b200.gin import config as gin_config
  opt = gin_config._materialize(gin.query_parameter("%OPTIMIZER"))
  assert isinstance(opt, optimizers.OptaxWrapper)
  assert gin.query_parameter("network.T5Config.scale_attn_logits") is True
