"""A run that needs no files: a tiny T5.1.1 on the synthetic span-corruption task with a
pass-through vocabulary (the buildable counterpart of t5x/examples/t5/local_tiny.gin).

    python -m t5x_b200.train \
        --fdl_config=t5x_b200.fiddle_configs.examples.synthetic:tiny_pretrain \
        --fdl_set=model_dir=/tmp/tiny --fdl_set=total_steps=5
"""
from __future__ import annotations

from t5x_b200 import fdl
from t5x_b200.data import vocabularies
from t5x_b200.fiddle_configs.configs import pretrain
from t5x_b200.fiddle_configs.models import t5_1_1


def tiny_pretrain(train_steps: int = 3, batch_size: int = 8) -> fdl.Buildable:
  config = t5_1_1.small_config(dropout_rate=0.0)
  config.emb_dim, config.mlp_dim, config.num_heads, config.head_dim = 8, 16, 4, 3
  config.num_encoder_layers = config.num_decoder_layers = 2
  vocab = fdl.Config(vocabularies.PassThroughVocabulary, size=32128)
  run = pretrain.train(
      model=t5_1_1.model(config=config, vocab=vocab), model_dir=None, train_steps=train_steps,
      mixture_or_task_name="synthetic_span_corruption",
      task_feature_lengths={"inputs": 8, "targets": 8}, eval_steps=2, eval_period=train_steps,
      random_seed=42, batch_size=batch_size, use_cached_tasks=False)
  run.train_dataset_cfg.shuffle = False
  run.train_dataset_cfg.seed = 42
  run.checkpoint_cfg.save.period = train_steps
  return run
