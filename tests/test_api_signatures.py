"""The public call surface that run configs bind by name: functions, classes and their
parameter names and defaults (what a `.gin` file or a launcher written for the reference
expects to find)."""
import inspect

import pytest

import t5x_b200
from t5x_b200 import (adafactor, checkpoints, decoding, eval as eval_lib, infer, models,
                      optimizers, partitioning, precompile, state_utils, train, trainer)
from t5x_b200.contrib.moe import partitioning as moe_partitioning
from t5x_b200.contrib.moe import trainer as moe_trainer
from t5x_b200.models.decoder_only import network as decoder_only_network
from t5x_b200.models.scalable_t5 import network as scalable_network
from t5x_b200.models.t5 import network
from t5x_b200.utils import core, data as data_utils, schedules


def _params(fn):
  return inspect.signature(fn).parameters


def _has(fn, *names):
  p = _params(fn)
  missing = [n for n in names if n not in p]
  assert not missing, f"{getattr(fn, '__qualname__', fn)} lacks parameters {missing}"
  return p


def test_run_functions():
  p = _has(train.train, "model", "train_dataset_cfg", "train_eval_dataset_cfg",
           "infer_eval_dataset_cfg", "checkpoint_cfg", "partitioner", "trainer_cls", "model_dir",
           "total_steps", "eval_steps", "eval_period", "relative_steps", "stats_period",
           "random_seed", "use_hardware_rng", "summarize_config_fn", "inference_evaluator_cls",
           "get_dataset_fn", "concurrent_metrics", "actions", "train_eval_get_dataset_fn",
           "run_eval_before_training", "train_state_initializer_cls", "use_orbax",
           "verify_matching_vocabs_fn", "gc_period")
  assert all(v.kind is inspect.Parameter.KEYWORD_ONLY for v in p.values())
  assert p["concurrent_metrics"].default is True and p["gc_period"].default == 0
  _has(eval_lib.evaluate, "model", "dataset_cfg", "restore_checkpoint_cfg", "partitioner",
       "output_dir", "inference_evaluator_cls", "training_evaluator_cls", "summarize_config_fn",
       "train_state_initializer_cls", "train_eval_get_dataset_fn", "fallback_init_rng", "use_orbax")
  p = _has(infer.infer, "mode", "model", "dataset_cfg", "restore_checkpoint_cfg", "partitioner",
           "output_dir", "checkpoint_period", "shard_id", "num_shards", "merge_chunked_results",
           "write_fn", "checkpoint_ds_iter", "train_state_initializer_cls", "fallback_init_rng",
           "merge_fn", "summarize_config_fn", "verify_matching_vocabs_fn",
           "output_vocab_feature_name", "file_extension", "keep_aux_as_numpy", "use_orbax")
  assert p["shard_id"].default == 0 and p["num_shards"].default == 1
  assert p["file_extension"].default == "jsonl"
  _has(precompile.precompile, "model", "train_dataset_cfg", "partitioner", "model_dir",
       "random_seed", "get_dataset_fn", "verify_matching_vocabs_fn")
  _has(eval_lib.InferenceEvaluator.__init__, "infer_eval_dataset_cfg", "inference_evaluator_cls",
       "model", "partitioner", "log_dir", "verify_matching_vocabs_fn")


def test_config_dataclasses_and_utils():
  p = _has(core.DatasetConfig, "mixture_or_task_name", "task_feature_lengths", "split",
           "batch_size", "shuffle", "seed", "use_cached", "pack", "use_custom_packing_ops",
           "module", "use_memory_cache", "trim_output_features", "runtime_preprocessors",
           "num_prefetch_threads", "num_workers")
  assert p["use_cached"].default is False and p["use_memory_cache"].default is True
  p = _has(core.SaveCheckpointConfig, "dtype", "period", "checkpoint_steps", "keep",
           "keep_dataset_checkpoints", "save_dataset", "checkpointer_cls",
           "state_transformation_fns", "checkpoint_manager_cls")
  assert p["dtype"].default == "float32"
  p = _has(core.RestoreCheckpointConfig, "path", "mode", "assignment_map", "strict",
           "fallback_to_scratch", "dtype", "restore_dataset", "checkpointer_cls",
           "state_transformation_fns", "checkpoint_manager_cls")
  assert p["mode"].default == "latest" and p["strict"].default is True
  _has(core.CheckpointConfig, "save", "restore")
  p = _has(schedules.create_learning_rate_scheduler, "factors", "base_learning_rate",
           "warmup_steps", "decay_factor", "steps_per_decay", "steps_per_cycle", "step_offset",
           "min_learning_rate")
  assert p["factors"].default == "constant * linear_warmup * rsqrt_decay"
  assert p["base_learning_rate"].default == 0.5 and p["min_learning_rate"].default == 1e-8
  _has(core.TrainStateInitializer.__init__, "optimizer_def", "init_fn", "input_shapes",
       "partitioner", "input_types")
  for name in ("from_scratch", "from_checkpoints", "from_checkpoint", "from_checkpoint_or_scratch"):
    assert callable(getattr(core.TrainStateInitializer, name))
  _has(data_utils.get_infer_fn, "infer_step", "batch_size", "train_state_axes", "partitioner",
       "keep_aux_as_numpy")
  for name in ("get_dataset", "get_training_eval_datasets", "verify_matching_vocabs",
               "get_vocabulary", "override_params_axes_names"):
    assert callable(getattr(data_utils, name))


def test_partitioning_surface():
  p = _has(partitioning.PjitPartitioner.__init__, "num_partitions", "model_parallel_submesh",
           "params_on_devices", "backend", "ici_mesh_shape", "dcn_mesh_shape", "logical_axis_rules")
  for name in ("mesh", "data_partition_spec", "data_mesh_size", "data_shards", "data_shard_id",
               "get_data_layout", "get_local_chunk_info", "params_on_devices",
               "move_params_to_devices", "get_logical_axes", "get_mesh_axes", "partition",
               "compile", "logical_axis_rules"):
    assert hasattr(partitioning.PjitPartitioner, name), name
  _has(partitioning.PjitPartitioner.partition, "fn", "in_axis_resources", "out_axis_resources",
       "static_argnums", "donate_argnums")
  p = _has(partitioning.standard_logical_axis_rules, "activation_partitioning_dims",
           "parameter_partitioning_dims", "additional_rules")
  assert p["activation_partitioning_dims"].default == 1
  assert {"batch_size", "shard_id", "num_shards", "is_first_host_in_replica_set"} <= \
      set(_params(partitioning.DataLayout))
  for name in ("get_mesh", "get_cpu_mesh", "get_gpu_mesh", "default_mesh", "LocalChunkInfo",
               "AxisNames", "with_sharding_constraint"):
    assert hasattr(partitioning, name), name
  p = _has(moe_partitioning.MoePjitPartitioner.__init__, "num_expert_partitions",
           "num_partitions", "model_parallel_submesh", "params_on_devices", "logical_axis_rules",
           "state_filter_fn")
  assert _params(moe_partitioning.standard_logical_axis_rules)[
      "activation_partitioning_dims"].default == 2
  _has(moe_trainer.MoeTrainer.__init__, "num_expert_partitions", "sharded_match_fn",
       "weight_metrics_computer")


def test_trainer_and_actions():
  _has(trainer.Trainer.__init__, "model", "train_state", "partitioner", "eval_names",
       "summary_dir", "train_state_axes", "rng", "learning_rate_fn", "num_microbatches",
       "weight_metrics_computer")
  _has(trainer.Trainer.train, "batch_iter", "num_steps", "start_step")
  for name in ("compile_train", "eval", "compile_eval", "train_state", "close",
               "train_metrics_manager" if False else "close"):
    assert hasattr(trainer.Trainer, name), name
  p = _has(trainer.EarlyStoppingAction.__init__, "metric", "mode", "patience", "atol", "rtol")
  assert p["patience"].default == 3 and p["atol"].default == 0.0
  assert _params(trainer.TerminateOnNanAction.__init__)["metric"].default == "loss"
  assert {m.name for m in trainer.ActionMode} == {"TRAIN", "TRAIN_EVAL", "INFER_EVAL"}


def test_models_and_networks():
  p = _has(models.EncoderDecoderModel.__init__, "module", "input_vocabulary", "output_vocabulary",
           "optimizer_def", "decode_fn", "feature_converter_cls", "label_smoothing", "z_loss",
           "loss_normalizing_factor", "default_decoder_params")
  assert p["decode_fn"].default is decoding.beam_search
  p = _has(models.EncoderDecoderModel.predict_batch_with_aux, "params", "batch", "rng",
           "decoder_params", "return_all_decodes", "num_decodes", "prompt_with_targets")
  assert p["prompt_with_targets"].default is False
  _has(models.EncoderDecoderModel.score_batch, "params", "batch", "return_intermediates")
  _has(models.EncoderDecoderModel.get_initial_variables, "rng", "input_shapes", "input_types")
  p = _has(models.DecoderOnlyModel.__init__, "module", "vocabulary", "optimizer_def", "decode_fn",
           "inputs_bidirectional_attention", "feature_converter_cls", "label_smoothing", "z_loss",
           "loss_normalizing_factor")
  assert p["decode_fn"].default is decoding.temperature_sample
  p = _has(models.DecoderOnlyModel.predict_batch_with_aux, "params", "batch", "rng",
           "return_all_decodes", "num_decodes", "decoder_params")
  assert p["num_decodes"].default == 1
  p = _has(network.T5Config, "vocab_size", "dtype", "emb_dim", "num_heads", "num_encoder_layers",
           "num_decoder_layers", "head_dim", "mlp_dim", "mlp_activations", "dropout_rate",
           "logits_via_embedding", "float32_attention_logits")
  assert p["emb_dim"].default == 512 and p["mlp_activations"].default == ("relu",)
  assert p["dropout_rate"].default == 0.1 and p["logits_via_embedding"].default is False
  p = _has(scalable_network.T5Config, "remat_policy", "scan_layers", "param_scan_axis")
  assert p["remat_policy"].default == "none" and p["scan_layers"].default is True
  _has(decoder_only_network.TransformerConfig, "vocab_size", "dtype", "emb_dim", "num_heads",
       "num_layers", "head_dim", "mlp_dim", "mlp_activations", "dropout_rate",
       "logits_via_embedding")
  assert hasattr(decoder_only_network, "DecoderWrapper")


def test_decoding_optimizers_and_checkpoints():
  p = _has(decoding.beam_search, "inputs", "cache", "tokens_to_logits", "eos_id", "num_decodes",
           "alpha", "max_decode_len", "max_decode_step", "min_log_prob", "decode_rng",
           "cache_offset", "initial_index")
  assert p["num_decodes"].default == 4 and p["alpha"].default == 0.6
  p = _has(decoding.temperature_sample, "inputs", "cache", "tokens_to_logits", "eos_id",
           "decode_rng", "num_decodes", "temperature", "topk", "topp", "cache_offset",
           "initial_index", "max_decode_steps", "max_decode_steps_hard_limit",
           "rescale_log_probs", "state_callback_fn", "logit_callback_fn")
  assert p["topk"].default == 1 and p["topp"].default == 0.0
  assert {"cur_index", "sequences", "cur_token", "cache"} <= set(_params(decoding.DecodingState))
  p = _has(adafactor.Adafactor.__init__, "learning_rate", "factored",
           "multiply_by_parameter_scale", "beta1", "decay_rate", "step_offset",
           "clipping_threshold", "weight_decay_rate", "min_dim_size_to_factor", "epsilon1",
           "epsilon2", "dtype_momentum", "factor_map", "logical_factor_rules",
           "weight_decay_rate_lr_exponent", "global_norm_clip_threshold", "max_parameter_scale",
           "skip_nan_updates")
  assert p["decay_rate"].default == 0.8 and p["min_dim_size_to_factor"].default == 128
  assert p["epsilon1"].default == 1e-30 and p["epsilon2"].default == 1e-3
  for name in ("standard_logical_factor_rules", "HParamMap", "FactorDim"):
    assert hasattr(adafactor, name)
  for name in ("create", "init_state", "apply_gradient", "update_hyper_params", "state_dict",
               "restore_state"):
    assert hasattr(optimizers.OptimizerDef, name), name
  for name in ("Optimizer", "OptimizerState", "wrap_optax_optimizer", "MultiOptimizer", "chain"):
    assert hasattr(optimizers, name), name
  p = _has(checkpoints.Checkpointer.__init__, "train_state", "partitioner", "checkpoints_dir",
           "dataset_iterator", "keep", "save_dtype", "restore_dtype", "keep_dataset_checkpoints")
  _has(checkpoints.Checkpointer.save, "train_state", "state_transformation_fns")
  _has(checkpoints.Checkpointer.restore, "step", "path", "state_transformation_fns",
       "fallback_state")
  p = _has(checkpoints.SaveBestCheckpointer.__init__, "metric_name_to_monitor", "metric_mode",
           "keep_checkpoints_without_metrics", "force_keep_period")
  assert p["metric_name_to_monitor"].default == "train/accuracy" and p["metric_mode"].default == "max"
  p = _has(checkpoints.load_t5x_checkpoint, "path", "step", "state_transformation_fns", "remap",
           "restore_dtype", "lazy_parameters")
  assert p["remap"].default is True and p["lazy_parameters"].default is False
  for name in ("find_checkpoint", "get_checkpoint_dir", "all_steps", "latest_step",
               "OrbaxCheckpointManagerInterface"):
    assert hasattr(checkpoints, name), name
  p = _has(state_utils.apply_assignment_map, "ckpt_optimizer_state", "optimizer_state",
           "assignment_map", "require_all_rules_match", "is_resuming")
  assert p["require_all_rules_match"].default is True
  assert p["is_resuming"].kind is inspect.Parameter.KEYWORD_ONLY
  for name in ("intersect_state", "merge_state", "flatten_state_dict", "get_name_tree",
               "tensorstore_leaf"):
    assert hasattr(state_utils, name), name
  assert t5x_b200.__name__ == "t5x_b200"
