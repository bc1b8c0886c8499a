r"""Training entry point (API of t5x/train.py).

  python -m t5x_b200.train --gin_file=t5x/configs/runs/pretrain.gin --gin.MODEL_DIR=\"/tmp/m\" ...
  torchrun --nproc-per-node 8 -m t5x_b200.train --gin_file=... --multiprocess_gpu

One process per GPU. `train()` is configured by gin; flags mirror the reference's
(`--gin_file`, `--gin_bindings` / `--gin.X=Y`, `--gin_search_paths`, `--multiprocess_gpu`,
`--coordinator_address`, `--process_count`, `--process_index`, `--initialization_timeout`).
"""
from __future__ import annotations

import gc
import logging
import math
import os
import signal
import sys
import time
from typing import Callable, Mapping, Optional, Sequence, Tuple, Type

import numpy as np
import torch

from t5x_b200 import checkpoints
from t5x_b200 import gin
from t5x_b200 import gin_utils
from t5x_b200 import models
from t5x_b200 import partitioning
from t5x_b200 import train_state as train_state_lib
from t5x_b200 import trainer as trainer_lib
from t5x_b200 import utils
from t5x_b200.data import seqio_api as seqio
from t5x_b200.parallel import state as pstate

_DEFAULT_GIN_SEARCH_PATHS = [os.path.dirname(os.path.abspath(__file__)),
                             os.path.dirname(os.path.dirname(os.path.abspath(__file__)))]
PyTree = object
P = partitioning.PartitionSpec


def run_actions(mode: trainer_lib.ActionMode, actions, train_state, metrics_by_task) -> bool:
  """Runs the actions registered for `mode`; the stop decision of rank 0 wins on every rank
  (t5x/train.py:64-93)."""
  stop = False
  for action in (actions or {}).get(mode, []):
    stop |= bool(action.run(train_state, metrics_by_task=metrics_by_task))
  return bool(utils.broadcast_one_to_all(stop))


def train(*, model: models.BaseModel, train_dataset_cfg: utils.DatasetConfig,
          train_eval_dataset_cfg: Optional[utils.DatasetConfig],
          infer_eval_dataset_cfg: Optional[utils.DatasetConfig],
          checkpoint_cfg: utils.CheckpointConfig, partitioner: partitioning.BasePartitioner,
          trainer_cls, model_dir: str, total_steps: int, eval_steps: int, eval_period: int,
          relative_steps: Optional[int] = None, stats_period: Optional[int] = None,
          random_seed: Optional[int], use_hardware_rng: bool = False,
          summarize_config_fn: Callable = gin_utils.summarize_gin_config,
          inference_evaluator_cls=seqio.Evaluator, get_dataset_fn=utils.get_dataset,
          concurrent_metrics: bool = True,
          actions: Optional[Mapping[str, Sequence[trainer_lib.BaseAction]]] = None,
          train_eval_get_dataset_fn=utils.get_training_eval_datasets,
          run_eval_before_training: bool = False,
          train_state_initializer_cls: Type[utils.TrainStateInitializer] = utils.TrainStateInitializer,
          use_orbax: bool = True, verify_matching_vocabs_fn=utils.verify_matching_vocabs,
          gc_period: int = 0) -> Tuple[int, train_state_lib.TrainState]:
  """Trains `model`, with periodic checkpoints, teacher-forced and inference evaluation
  (t5x/train.py:96-812). Returns (last step, train state)."""
  logging.info("Process ID: %d", pstate.get().rank)
  os.makedirs(model_dir, exist_ok=True)
  if actions is None:
    actions = {}
  actions = {(trainer_lib.ActionMode[k] if isinstance(k, str) else k): v
             for k, v in actions.items()}
  if random_seed is None:
    random_seed = int(utils.broadcast_one_to_all(np.int32(time.time() % 2 ** 31)))
    logging.info("Using time-based random seed %d", random_seed)
  init_rng, trainer_rng = int(random_seed), int(random_seed) + 1
  if use_hardware_rng:
    utils.set_hardware_rng_ops()

  # ---- data ------------------------------------------------------------------------------
  if train_dataset_cfg.seed is not None and not (
      checkpoint_cfg.save and checkpoint_cfg.save.save_dataset):
    logging.warning("Providing a random seed for the train dataset with "
                    "`checkpoint_train_ds=False` is dangerous since each preemption of the "
                    "training job will cause the dataset to be reset to the start.")
  data_layout = partitioner.get_data_layout(train_dataset_cfg.batch_size)
  if verify_matching_vocabs_fn is not None:
    verify_matching_vocabs_fn(train_dataset_cfg, model)
  train_ds = get_dataset_fn(train_dataset_cfg, data_layout.shard_id, data_layout.num_shards,
                            model.FEATURE_CONVERTER_CLS, num_epochs=None)
  train_iter = utils.prepare_train_iter(train_ds, partitioner=partitioner,
                                        checkpoint_cfg=checkpoint_cfg, data_layout=data_layout)
  input_shapes = {k: (train_dataset_cfg.batch_size, *v.shape[1:])
                  for k, v in train_iter.element_spec.items()}
  input_types = {k: v.dtype for k, v in train_iter.element_spec.items()}

  train_eval_datasets = {}
  if train_eval_dataset_cfg:
    if verify_matching_vocabs_fn is not None:
      verify_matching_vocabs_fn(train_eval_dataset_cfg, model)
    train_eval_datasets = train_eval_get_dataset_fn(
        train_eval_dataset_cfg, data_layout.shard_id, data_layout.num_shards, eval_steps,
        model.FEATURE_CONVERTER_CLS)
    if not train_eval_datasets:
      logging.warning("No train_eval datasets loaded from config `train_eval_dataset_cfg`")

  # ---- state -----------------------------------------------------------------------------
  # Auto-resume: the run directory's latest checkpoint takes precedence over any configured
  # initial checkpoint; its restore transformations are told the run is resuming so that
  # assignment maps are not applied twice.
  checkpoint_period = checkpoint_cfg.save.period if checkpoint_cfg.save else None
  checkpoint_steps = (list(checkpoint_cfg.save.checkpoint_steps)
                      if checkpoint_cfg.save and checkpoint_cfg.save.checkpoint_steps else [])
  valid_restore_cfg = None
  restore_paths: Sequence[str] = []
  if checkpoint_cfg.restore:
    import dataclasses
    import functools
    fns = [functools.partial(fn, is_resuming=True)
           for fn in checkpoint_cfg.restore.state_transformation_fns]
    resume_cfg = dataclasses.replace(checkpoint_cfg.restore, path=model_dir, mode="latest",
                                     assignment_map=None, state_transformation_fns=tuple(fns))
    restore_cfgs = [resume_cfg, checkpoint_cfg.restore]
  else:
    restore_cfgs = [utils.RestoreCheckpointConfig(path=model_dir, mode="latest")]
  valid_restore_cfg, restore_paths = utils.get_first_valid_restore_config_and_paths(restore_cfgs)
  if len(restore_paths) > 1:
    raise ValueError("Multiple restore paths not permitted in training.")

  initializer = train_state_initializer_cls(
      optimizer_def=model.optimizer_def, init_fn=model.get_initial_variables,
      input_shapes=input_shapes, input_types=input_types, partitioner=partitioner)
  train_state_axes = initializer.train_state_axes
  init_tick = time.time()
  train_state, checkpoint_manager = utils.create_checkpoint_manager_and_restore(
      initializer, partitioner, valid_restore_cfg, restore_paths[0] if restore_paths else None,
      init_rng, save_checkpoint_cfg=checkpoint_cfg.save, model_dir=model_dir,
      ds_iter=train_iter if (checkpoint_cfg.save and checkpoint_cfg.save.save_dataset) else None,
      use_orbax=use_orbax)
  first_batch_ready = train_iter.peek_async() if hasattr(train_iter, "peek_async") else None
  if train_state is None:
    train_state = initializer.from_scratch(init_rng)
  init_seconds = time.time() - init_tick
  utils.log_model_info(os.path.join(model_dir, "model-info.txt"), train_state, partitioner)

  host_step = int(utils.get_local_data(train_state.step))
  if relative_steps:
    total_steps = host_step + relative_steps
  if eval_period or checkpoint_period or gc_period:
    steps_per_epoch = int(min(eval_period or math.inf, checkpoint_period or math.inf,
                              gc_period or math.inf))
  else:
    steps_per_epoch = total_steps
  stats_period = stats_period or steps_per_epoch
  if (eval_period and eval_period % steps_per_epoch or
      checkpoint_period and checkpoint_period % steps_per_epoch or
      gc_period and gc_period % steps_per_epoch):
    raise ValueError(f"Checkpoint period ({checkpoint_period}), eval period ({eval_period}), "
                     f"and GC period ({gc_period}) must all be multiples of each other.")
  if host_step > total_steps:
    raise ValueError(f"Restored step ({host_step}) exceeds total steps ({total_steps}).")

  # ---- trainer ---------------------------------------------------------------------------
  trainer = trainer_cls(model=model, train_state=train_state, partitioner=partitioner,
                        train_state_axes=train_state_axes,
                        eval_names=list(train_eval_datasets.keys()), summary_dir=model_dir,
                        rng=trainer_rng)
  del train_state
  train_metrics = trainer.train_metrics_manager
  summarize_config_fn(model_dir, train_metrics.summary_writer, host_step)
  train_metrics.write_scalar("timing/init_or_restore_seconds", init_seconds, host_step)

  evaluator = None
  if infer_eval_dataset_cfg is not None:
    from t5x_b200 import eval as eval_lib
    evaluator = eval_lib.InferenceEvaluator(
        infer_eval_dataset_cfg=infer_eval_dataset_cfg,
        inference_evaluator_cls=inference_evaluator_cls, model=model, partitioner=partitioner,
        log_dir=os.path.join(model_dir, "inference_eval"),
        verify_matching_vocabs_fn=verify_matching_vocabs_fn)
    if not evaluator.eval_tasks:
      evaluator = None

  def _run_training_eval(first_run: bool = False):
    if not train_eval_datasets:
      return False
    tick = time.time()
    summaries = trainer.eval({task: iter(ds) for task, ds in train_eval_datasets.items()})
    trainer.train_metrics_manager.write_scalar("timing/evaluate_seconds", time.time() - tick,
                                               int(trainer.train_state.step))
    return run_actions(trainer_lib.ActionMode.TRAIN_EVAL, actions, trainer.train_state, summaries)

  def _run_inference_eval():
    if evaluator is None:
      return False
    tick = time.time()
    all_metrics = evaluator.evaluate(trainer.train_state, train_state_axes)
    trainer.train_metrics_manager.write_scalar("timing/evaluate_seconds", time.time() - tick,
                                               int(trainer.train_state.step))
    return run_actions(trainer_lib.ActionMode.INFER_EVAL, actions, trainer.train_state,
                       all_metrics.result() if hasattr(all_metrics, "result") else all_metrics)

  def _save(force=True):
    tick = time.time()
    if hasattr(trainer, "sync_replicas"):
      trainer.sync_replicas()
    fns = checkpoint_cfg.save.state_transformation_fns if checkpoint_cfg.save else ()
    checkpoint_manager.save(trainer.train_state, fns, force=force)
    checkpoint_manager.wait_until_finished()
    trainer.train_metrics_manager.write_scalar("timing/checkpoint_seconds", time.time() - tick,
                                               int(trainer.train_state.step))

  # Emergency checkpoint on SIGTERM (preemption).
  def _on_sigterm(signum, frame):
    # only a flag: the trainer raises PreemptionError at the next step boundary, on all ranks
    logging.warning("SIGTERM received: stopping at the next step boundary.")
    trainer.request_preemption()
  old_handler = None
  if threading_is_main():
    old_handler = signal.signal(signal.SIGTERM, _on_sigterm)

  # ---- step-0 / resume checkpoint, optional evaluation before training -------------------
  if checkpoint_cfg.save and checkpoint_period and host_step not in checkpoint_manager.all_steps():
    logging.info("Saving checkpoint before the training loop starts.")
    _save(force=True)
  if run_eval_before_training:
    _run_training_eval(first_run=True)
    _run_inference_eval()

  if host_step == total_steps:
    logging.info("Model has already been trained for %d steps; running evaluation only.",
                 total_steps)
    _run_training_eval()
    _run_inference_eval()
    checkpoint_manager.close()
    trainer.close()
    utils.sync_global_devices("complete")
    return host_step, trainer.train_state

  # ---- main loop -------------------------------------------------------------------------
  dummy_batch = utils.get_zeros_batch_like_spec(
      {k: _Spec(input_shapes[k], input_types[k]) for k in input_shapes})
  trainer.compile_train(dummy_batch)
  if first_batch_ready is not None:
    tick = time.time()
    first_batch_ready.result()
    train_metrics.write_scalar("timing/train_iter_warmup", time.time() - tick, host_step)

  first_epoch = host_step // steps_per_epoch
  num_epochs = -(-total_steps // steps_per_epoch)
  next_ckpt_step, ckpt_idx = utils.find_first_checkpoint_step(host_step + 1, checkpoint_steps)
  logging.info("Starting training loop over steps %d-%d.", host_step, total_steps)
  if gc_period:
    gc.disable()
  stop_training = False
  try:
    for epoch in range(first_epoch, num_epochs):
      final_epoch = epoch == num_epochs - 1
      epoch_end_step = min(total_steps, (epoch + 1) * steps_per_epoch)
      try:
        while host_step < epoch_end_step:
          if trainer.stop_training:
            stop_training = True
            break
          inner = min(epoch_end_step - host_step, stats_period)
          if next_ckpt_step is not None and host_step < next_ckpt_step < host_step + inner:
            inner = next_ckpt_step - host_step
          summary = trainer.train(train_iter, inner, start_step=host_step)
          host_step += inner
          if not concurrent_metrics or actions.get(trainer_lib.ActionMode.TRAIN):
            trainer.stop_training |= run_actions(trainer_lib.ActionMode.TRAIN, actions,
                                                 trainer.train_state, {"train": summary.result()})
          if next_ckpt_step is not None and host_step == next_ckpt_step:
            if checkpoint_cfg.save and not (checkpoint_period and
                                            host_step % checkpoint_period == 0):
              _save(force=True)
            _, next_ckpt_step, ckpt_idx = utils.find_next_checkpoint_step(
                host_step, None, ckpt_idx, checkpoint_steps)
      except trainer_lib.PreemptionError as e:
        logging.info("Saving emergency checkpoint.")
        _save(force=True)
        logging.info("Saving emergency checkpoint done.")
        raise e
      if stop_training:
        break
      if gc_period and (final_epoch or host_step % gc_period == 0):
        gc.collect()
      is_ckpt_epoch = checkpoint_period and (final_epoch or host_step % checkpoint_period == 0)
      is_eval_epoch = eval_period and (final_epoch or host_step % eval_period == 0)
      if checkpoint_cfg.save and is_ckpt_epoch:
        _save(force=True)
      if is_eval_epoch:
        stop_training |= _run_training_eval()
        stop_training |= _run_inference_eval()
        if stop_training:
          break
  finally:
    if gc_period:
      gc.enable()
    if hasattr(trainer, "sync_replicas"):
      trainer.sync_replicas()
    if old_handler is not None:
      signal.signal(signal.SIGTERM, old_handler)
    trainer.train_metrics_manager.flush()
    checkpoint_manager.close()
    trainer.close()
    if evaluator is not None:
      evaluator.close()
  utils.sync_global_devices("complete")
  logging.info("Finished.")
  return host_step, trainer.train_state


class _Spec:
  def __init__(self, shape, dtype):
    self.shape, self.dtype = tuple(shape), dtype


def threading_is_main() -> bool:
  import threading
  return threading.current_thread() is threading.main_thread()


# ----------------------------------------------------------------------------
# CLI
# ----------------------------------------------------------------------------
def build_flag_parser(description: str = ""):
  import argparse
  ap = argparse.ArgumentParser(description=description, allow_abbrev=False)
  ap.add_argument("--gin_file", action="append", default=[],
                  help="Path to gin configuration file; repeatable, later files override.")
  ap.add_argument("--gin_bindings", action="append", default=[],
                  help="Individual gin bindings.")
  ap.add_argument("--gin_search_paths", action="append", default=[],
                  help="Comma-separated list of gin config path prefixes to be prepended.")
  ap.add_argument("--tfds_data_dir", default=None)
  ap.add_argument("--dry_run", action="store_true")
  ap.add_argument("--multiprocess_gpu", action="store_true",
                  help="Join a multi-process run: one process per GPU (torchrun / SLURM).")
  ap.add_argument("--coordinator_address", default=None, help="IP:port of rank 0's rendezvous.")
  ap.add_argument("--process_count", type=int, default=None)
  ap.add_argument("--process_index", type=int, default=None)
  ap.add_argument("--initialization_timeout", type=int, default=None)
  ap.add_argument("--seqio_additional_cache_dirs", action="append", default=[])
  from t5x_b200 import config_utils
  config_utils.add_flags(ap)
  ap.add_argument("--profile_steps", default=None, metavar="FIRST:LAST",
                  help="Record train steps FIRST..LAST-1 with torch.profiler into "
                       "<model_dir>/profile/ (trace + kernels by device time).")
  return ap


def init_distributed_from_flags(flags) -> None:
  """Joins the process group (the role of jax.distributed.initialize, t5x/train.py:912-938)."""
  if flags.coordinator_address:
    host, _, port = flags.coordinator_address.partition(":")
    os.environ.setdefault("MASTER_ADDR", host)
    if port:
      os.environ.setdefault("MASTER_PORT", port)
  if flags.process_count is not None:
    os.environ.setdefault("WORLD_SIZE", str(flags.process_count))
  if flags.process_index is not None:
    os.environ.setdefault("RANK", str(flags.process_index))
    os.environ.setdefault("LOCAL_RANK", str(flags.process_index))
  if flags.multiprocess_gpu or int(os.environ.get("WORLD_SIZE", "1")) > 1:
    pstate.init_distributed(timeout_s=float(flags.initialization_timeout or 600))


def parse_gin_from_flags(flags, default_search_paths=()) -> None:
  paths = []
  for p in flags.gin_search_paths:
    paths.extend(p.split(","))
  gin_utils.parse_gin_flags(paths + list(default_search_paths), flags.gin_file,
                            flags.gin_bindings)


def main(argv: Optional[Sequence[str]] = None) -> None:
  logging.basicConfig(level=logging.INFO)
  argv = gin_utils.rewrite_gin_args(list(sys.argv[1:] if argv is None else argv))
  flags = build_flag_parser(__doc__).parse_args(argv)
  if flags.profile_steps:
    from t5x_b200.utils import profiling
    profiling.parse_step_range(flags.profile_steps)  # fail on a malformed range before training
    os.environ["T5X_B200_PROFILE_STEPS"] = flags.profile_steps
  init_distributed_from_flags(flags)
  from t5x_b200 import config_utils
  if config_utils.using_fdl(flags):
    config_utils.run_with_fiddle(train, flags)
    return
  gin.set_main_module(sys.modules[__name__])
  parse_gin_from_flags(flags, _DEFAULT_GIN_SEARCH_PATHS)
  train_using_gin = gin.get_configurable(train)
  if flags.dry_run:
    logging.info("Dry run: configuration parsed; not training.")
    return
  train_using_gin()


if __name__ == "__main__":
  main()
