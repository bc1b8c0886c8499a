"""Run-level utilities (the public names of t5x/utils.py).

The names are resolved on first access: the low-level helpers `utils.tree`, `utils.schedules`
and `utils.metric_writers` are imported by modules (`partitioning`, `checkpoints`) that
`utils.core` itself depends on, so this package must be importable before they are."""
import importlib

_CORE = (
    "CheckpointConfig", "DatasetConfig", "RestoreCheckpointConfig", "SaveCheckpointConfig",
    "TrainStateInitializer", "broadcast_one_to_all", "create_checkpoint_manager",
    "create_checkpoint_manager_and_restore", "flatten_dict_string_keys", "flatten_lists",
    "get_fallback_state", "get_first_valid_restore_config_and_paths", "get_local_data",
    "log_model_info", "multihost_assert_equal", "restore", "round_vocab_size_to_multiple",
    "set_hardware_rng_ops", "sync_global_devices")
_DATA = (
    "ShardedDatasetIterator", "find_first_checkpoint_step", "find_next_checkpoint_step",
    "get_dataset", "get_dataset_inner", "get_infer_fn", "get_training_eval_datasets",
    "get_vocabulary", "get_zeros_batch_like_dataset", "get_zeros_batch_like_spec",
    "import_module", "override_params_axes_names", "prepare_train_iter",
    "verify_matching_vocabs")
_SCHEDULES = ("create_learning_rate_scheduler",)
_WHERE = {**{n: "core" for n in _CORE}, **{n: "data" for n in _DATA},
          **{n: "schedules" for n in _SCHEDULES}}
__all__ = sorted(_WHERE)


def __getattr__(name):
  where = _WHERE.get(name)
  if where is None:
    if name in ("core", "data", "schedules", "tree", "metric_writers"):
      return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
  value = getattr(importlib.import_module(f"{__name__}.{where}"), name)
  globals()[name] = value
  return value


def __dir__():
  return sorted(set(globals()) | set(_WHERE))
