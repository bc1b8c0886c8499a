"""Example runs as buildables (t5x/fiddle_configs/examples/t5_1_1.py; gin forms under
t5x/examples/t5/t5_1_1/examples/). `model_dir` is left for `--fdl_set=model_dir=...`.

    python -m t5x_b200.train --fdl_config=t5x_b200.fiddle_configs.examples.t5_1_1:small_c4_pretrain \\
        --fdl_set=model_dir=/tmp/run
"""
from __future__ import annotations

from t5x_b200 import eval as eval_lib
from t5x_b200 import fdl
from t5x_b200.data import evaluation
from t5x_b200.fiddle_configs.configs import common, finetune, pretrain
from t5x_b200.fiddle_configs.models import t5_1_1

PRETRAINED_SMALL = "gs://t5-data/pretrained_models/t5x/t5_1_1_small/checkpoint_1000000"


def small_wmt_finetune() -> fdl.Buildable:
  model = t5_1_1.model(config=t5_1_1.small_config(dropout_rate=0.0),
                       loss_normalizing_factor=233472)
  return finetune.train(
      mixture_or_task_name="wmt_t2t_ende_v003", model_dir=None, model=model,
      task_feature_lengths={"inputs": 256, "targets": 256},
      train_steps=1_020_000,  # 1,000,000 pre-training steps + 20,000 of fine-tuning
      initial_checkpoint_path=PRETRAINED_SMALL, use_cached_tasks=False)


def small_wmt_eval() -> fdl.Buildable:
  model = t5_1_1.model(config=t5_1_1.small_config(dropout_rate=0.0))
  return fdl.Config(
      eval_lib.evaluate, model=model, partitioner=common.partitioner(),
      dataset_cfg=common.dataset_config("test", "wmt_t2t_ende_v003", None, 32, False, None,
                                        shuffle=False, seed=42, pack=False),
      inference_evaluator_cls=fdl.Partial(evaluation.Evaluator, num_examples=None,
                                          use_memory_cache=True),
      restore_checkpoint_cfg=common.checkpoint_config(PRETRAINED_SMALL, "specific").restore,
      output_dir=None)


def small_c4_pretrain() -> fdl.Buildable:
  model = t5_1_1.model(config=t5_1_1.small_config(dropout_rate=0.0))
  return pretrain.train(
      mixture_or_task_name="c4_v220_span_corruption", model_dir=None, model=model,
      task_feature_lengths={"inputs": 512, "targets": 114}, train_steps=10000, batch_size=256,
      use_cached_tasks=False)
