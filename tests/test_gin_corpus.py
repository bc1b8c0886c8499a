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
