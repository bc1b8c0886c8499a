"""End-to-end runs of the gin-configured entry points on CPU: train (with checkpoints and
resume), eval, infer and precompile — the flows of t5x/train.py, eval.py, infer.py."""
import json
import os

import pytest

from t5x_b200 import checkpoints
from t5x_b200 import eval as eval_lib
from t5x_b200 import gin
from t5x_b200 import infer as infer_lib
from t5x_b200 import main as main_lib
from t5x_b200 import train as train_lib

TASK = "synthetic_span_corruption"
MODEL = ["--gin_file=t5x/examples/t5/t5_1_1/tiny.gin"]
VOCAB = ["--gin.VOCABULARY=@seqio.PassThroughVocabulary()",
         "--gin.seqio.PassThroughVocabulary.size=32128", "--gin.DROPOUT_RATE=0.0"]


@pytest.fixture(autouse=True)
def _fresh_gin():
  gin.clear_config(clear_constants=True)
  yield
  gin.clear_config(clear_constants=True)


def _train_args(model_dir, steps, extra=()):
  return (MODEL + ["--gin_file=t5x/configs/runs/pretrain.gin",
                   "--gin_file=t5x/examples/t5/local_tiny.gin"] + VOCAB + [
      f'--gin.MODEL_DIR="{model_dir}"', f'--gin.MIXTURE_OR_TASK_NAME="{TASK}"',
      "--gin.USE_CACHED_TASKS=False", f"--gin.TRAIN_STEPS={steps}",
      "--gin.utils.CheckpointConfig.save=@utils.SaveCheckpointConfig()",
      "--gin.utils.SaveCheckpointConfig.period=2",
      "--gin.train_script.train.eval_period=2"] + list(extra))


def test_train_saves_and_resumes(tmp_path):
  model_dir = str(tmp_path / "run")
  train_lib.main(_train_args(model_dir, 4))
  assert checkpoints.all_steps(model_dir) == [0, 2, 4]
  assert os.path.exists(os.path.join(model_dir, "config.gin"))
  assert os.path.exists(os.path.join(model_dir, "model-info.txt"))
  gin.clear_config(clear_constants=True)
  # a second launch with a larger budget resumes at step 4
  train_lib.main(_train_args(model_dir, 6))
  assert checkpoints.all_steps(model_dir) == [0, 2, 4, 6]


def test_train_already_done_only_evaluates(tmp_path):
  model_dir = str(tmp_path / "run")
  train_lib.main(_train_args(model_dir, 2))
  gin.clear_config(clear_constants=True)
  train_lib.main(_train_args(model_dir, 2))
  assert checkpoints.all_steps(model_dir) == [0, 2]


def test_eval_and_infer_from_checkpoint(tmp_path):
  model_dir = str(tmp_path / "run")
  train_lib.main(_train_args(model_dir, 2))
  gin.clear_config(clear_constants=True)
  out = str(tmp_path / "eval")
  eval_lib.main(MODEL + ["--gin_file=t5x/configs/runs/eval.gin"] + VOCAB + [
      f'--gin.CHECKPOINT_PATH="{model_dir}"', f'--gin.EVAL_OUTPUT_DIR="{out}"',
      f'--gin.MIXTURE_OR_TASK_NAME="{TASK}"', "--gin.utils.RestoreCheckpointConfig.mode='all'",
      "--gin.utils.DatasetConfig.batch_size=4", "--gin.seqio.Evaluator.num_examples=8",
      "--gin.TASK_FEATURE_LENGTHS={'inputs': 8, 'targets': 8}"])
  done = open(os.path.join(out, f"eval.{TASK}.ckpt")).read().split()
  assert [os.path.basename(p) for p in done] == ["checkpoint_0", "checkpoint_2"]
  gin.clear_config(clear_constants=True)
  out = str(tmp_path / "infer")
  infer_lib.main(MODEL + ["--gin_file=t5x/configs/runs/infer.gin"] + VOCAB + [
      f'--gin.CHECKPOINT_PATH="{model_dir}/checkpoint_2"', f'--gin.INFER_OUTPUT_DIR="{out}"',
      f'--gin.MIXTURE_OR_TASK_NAME="{TASK}"', "--gin.utils.DatasetConfig.batch_size=4",
      "--gin.infer_script.infer.checkpoint_period=1",
      "--gin.TASK_FEATURE_LENGTHS={'inputs': 8, 'targets': 8}",
      "--gin.utils.DatasetConfig.split='validation'"])
  name = f"{TASK}-predict.jsonl-00000-of-00001"
  assert os.path.exists(os.path.join(out, name + ".COMPLETED"))
  rows = [json.loads(l) for l in open(os.path.join(out, name))]
  assert rows and all("prediction" in r for r in rows)


def test_main_dispatch_dry_run_and_precompile(tmp_path):
  model_dir = str(tmp_path / "pc")
  main_lib.main(["--run_mode=train", "--dry_run"] + _train_args(model_dir, 2))
  assert not os.path.exists(model_dir)
  gin.clear_config(clear_constants=True)
  main_lib.main(["--run_mode=precompile"] + MODEL + [
      "--gin_file=t5x/configs/runs/precompile.gin"] + VOCAB + [
      f'--gin.MODEL_DIR="{model_dir}"', f'--gin.MIXTURE_OR_TASK_NAME="{TASK}"',
      "--gin.USE_CACHED_TASKS=False", "--gin.BATCH_SIZE=8",
      "--gin.TASK_FEATURE_LENGTHS={'inputs': 8, 'targets': 8}",
      "--gin.network.T5Config.vocab_size=32128"])
  assert "gemm fwd" in open(os.path.join(model_dir, "launch_plan.txt")).read()


def test_moe_pretrain_from_gin(tmp_path):
  """Switch-style model through the MoE run config: MoE partitioner, MoE trainer, expert
  metrics in the training summary."""
  model_dir = str(tmp_path / "moe")
  tiny = ["--gin.moe_network.MoeT5Config.emb_dim=8", "--gin.moe_network.MoeT5Config.mlp_dim=16",
          "--gin.moe_network.MoeT5Config.num_heads=2", "--gin.moe_network.MoeT5Config.head_dim=4",
          "--gin.moe_network.MoeT5Config.num_encoder_layers=2",
          "--gin.moe_network.MoeT5Config.num_decoder_layers=2", "--gin.NUM_EXPERTS=4",
          "--gin.NUM_EXPERT_PARTITIONS=1"]
  train_lib.main(["--gin_file=t5x/contrib/moe/configs/models/switch_base.gin",
                  "--gin_file=t5x/contrib/moe/configs/runs/pretrain.gin"] + VOCAB + tiny + [
      f'--gin.MODEL_DIR="{model_dir}"', f'--gin.MIXTURE_OR_TASK_NAME="{TASK}"',
      "--gin.USE_CACHED_TASKS=False", "--gin.TRAIN_STEPS=2", "--gin.BATCH_SIZE=8",
      "--gin.TASK_FEATURE_LENGTHS={'inputs': 8, 'targets': 8}",
      "--gin.train_script.train.eval_period=2", "--gin.train_script.train.eval_steps=1",
      "--gin.utils.SaveCheckpointConfig.period=2", "--gin.train_script.train.random_seed=0"])
  assert checkpoints.all_steps(model_dir) == [0, 2]
  info = open(os.path.join(model_dir, "model-info.txt")).read()
  assert "mlp/expert/wi_0/kernel" in info and "router_weights" in info
