r"""Batch inference entry point (API of t5x/infer.py).

  python -m t5x_b200.infer --gin_file=t5x/configs/runs/infer.gin --gin.CHECKPOINT_PATH=... \
      --gin.INFER_OUTPUT_DIR=...

Inference runs in chunks of `checkpoint_period` batches. Each chunk's results are written by a
background thread to `<output_dir>/tmp-<task>-<shard>/<name>-chunkNNNNN` followed by a
`.COMPLETED` marker and the input position, so that a restarted job resumes at the first
unfinished chunk. When every chunk is done the chunks are merged into one JSONL file.
"""
from __future__ import annotations

import concurrent.futures
import functools
import glob
import hashlib
import json
import logging
import os
import re
import shutil
import sys
import time
from typing import Any, Callable, Mapping, Optional, Sequence, Tuple, Type

import numpy as np

from t5x_b200 import gin
from t5x_b200 import gin_utils
from t5x_b200 import models
from t5x_b200 import partitioning
from t5x_b200 import utils
from t5x_b200.data import seqio_api as seqio
from t5x_b200.parallel import state as pstate

Inferences = Tuple[Sequence[Any], Mapping[str, Any]]
_Inferences = Inferences


class FailFastThreadPoolExecutor(concurrent.futures.ThreadPoolExecutor):
  """A pool whose `submit` and `shutdown` re-raise the first exception of an earlier task, so a
  failed write stops the job at the next chunk instead of at the end (t5x/infer.py:66-98)."""

  def __init__(self, *args, **kwargs):
    super().__init__(*args, **kwargs)
    self._incomplete = []

  def check_for_exceptions(self, wait: bool = False):
    still = []
    for fut in self._incomplete:
      try:
        exc = fut.exception(timeout=None if wait else 0)
      except concurrent.futures.TimeoutError:
        still.append(fut)
        continue
      if exc is not None:
        raise exc
    self._incomplete = still

  def submit(self, *args, **kwargs) -> concurrent.futures.Future:
    self.check_for_exceptions(wait=False)
    fut = super().submit(*args, **kwargs)
    self._incomplete.append(fut)
    return fut

  def shutdown(self, *args, wait: bool = False, **kwargs):
    self.check_for_exceptions(wait=wait)
    super().shutdown(*args, wait=wait, **kwargs)


def create_task_from_tfexample_file(paths: Sequence[str], file_type: str, inputs_key: str,
                                    targets_key: Optional[str],
                                    features: Mapping[str, seqio.Feature],
                                    task_id: Optional[str] = None) -> str:
  """Registers an ad-hoc task named `infer_<id>` with one split `infer` over text files
  (t5x/infer.py:101-170). `file_type` 'jsonl' reads one JSON object per line and 'text' one
  input per line; TFRecord protos need TensorFlow, which this stack does not depend on."""
  files = sorted(f for p in paths for f in glob.glob(p))
  if not files:
    raise ValueError(f"Missing or invalid paths: {paths}")
  if file_type not in ("jsonl", "text"):
    raise ValueError(f"Unsupported file_type {file_type!r}: expected 'jsonl' or 'text'")
  if task_id is None:
    task_id = hashlib.md5(":".join(list(paths) + [inputs_key, targets_key or ""]).encode()
                          ).hexdigest()[:10]

  def source(split, shard_info=None, seed=None, **_):
    idx = 0
    for fname in files:
      with open(fname) as f:
        for line in f:
          line = line.rstrip("\n")
          if not line:
            continue
          take = shard_info is None or idx % shard_info.num_shards == shard_info.index
          idx += 1
          if not take:
            continue
          rec = json.loads(line) if file_type == "jsonl" else {inputs_key: line}
          ex = {"inputs_pretokenized": rec[inputs_key]}
          ids = features["inputs"].vocabulary.encode(rec[inputs_key])
          if features["inputs"].add_eos:
            ids = list(ids) + [features["inputs"].vocabulary.eos_id]
          ex["inputs"] = np.asarray(ids, np.int32)
          if targets_key:
            ex["targets_pretokenized"] = rec[targets_key]
            tids = features["targets"].vocabulary.encode(rec[targets_key])
            if features["targets"].add_eos:
              tids = list(tids) + [features["targets"].vocabulary.eos_id]
            ex["targets"] = np.asarray(tids, np.int32)
          yield ex

  name = f"infer_{task_id}"
  if name not in seqio.TaskRegistry:
    seqio.TaskRegistry.add(name, source=source, output_features=features, splits=("infer",))
  return name


def merge_chunks_to_file(output_dir: str, output_fname: str, tmp_dir: str,
                         step: Optional[int]) -> None:
  """Concatenates `<output_fname>-chunkNNNNN` files into `<output_dir>/<output_fname>`."""
  del step
  chunk_paths = sorted(glob.glob(os.path.join(tmp_dir, f"{output_fname}-chunk?????")))
  if not chunk_paths:
    raise FileNotFoundError("No chunk results found! One possible explanation is that your "
                            "input did not contain any examples")
  expected = int(chunk_paths[-1][-5:]) + 1
  assert expected == len(chunk_paths), (
      f"Expecting {expected} chunk paths, found {len(chunk_paths)}")
  with open(os.path.join(output_dir, output_fname), "wb") as merged:
    for p in chunk_paths:
      with open(p, "rb") as f:
        shutil.copyfileobj(f, merged)


class _NumpyEncoder(json.JSONEncoder):
  def default(self, o):
    if isinstance(o, np.ndarray):
      return o.tolist()
    if isinstance(o, np.generic):
      return o.item()
    if isinstance(o, bytes):
      return o.decode("utf-8")
    return super().default(o)


def _json_compat(value):
  if isinstance(value, bytes):
    return value.decode("utf-8")
  if isinstance(value, np.generic):
    return float(value)
  if isinstance(value, np.ndarray):
    return value.tolist()
  return value


def _map_leaves(fn, tree):
  if isinstance(tree, Mapping):
    return {k: _map_leaves(fn, v) for k, v in tree.items()}
  return fn(tree)


def write_inferences_to_file(path: str, inferences: Inferences, task_ds, mode: str,
                             vocabulary=None, json_encoder_cls: Type[json.JSONEncoder] = _NumpyEncoder,
                             include_all_inputs: bool = False,
                             input_fields_to_include: Optional[Sequence[str]] = None,
                             output_ids: bool = False) -> None:
  """One JSON line per example: its pretokenized inputs plus `prediction` (decoded text) or
  `score`, and `aux` values (t5x/infer.py:209-325)."""
  all_predictions, all_aux = inferences
  if mode in ("predict", "predict_with_aux") and vocabulary is None:
    raise ValueError("The `vocabulary` parameter is required in `predict` and "
                     "`predict_with_aux` modes")
  if include_all_inputs and input_fields_to_include is not None:
    raise ValueError("include_all_inputs and input_fields_to_include should not be set "
                     "simultaneously.")
  with open(path, "w") as f:
    for i, inp in enumerate(task_ds):
      prediction = all_predictions[i]
      aux = _map_leaves(lambda v, i=i: v[i], all_aux)
      if include_all_inputs:
        inputs = inp
      elif input_fields_to_include is not None:
        inputs = {k: v for k, v in inp.items()
                  if k in input_fields_to_include or (
                      k.endswith("_pretokenized") and
                      k[:-len("_pretokenized")] in input_fields_to_include)}
      else:
        inputs = {k: v for k, v in inp.items() if k.endswith("_pretokenized")}
      out = {"inputs": {k: _json_compat(v) for k, v in inputs.items()}}
      if mode in ("predict", "predict_with_aux"):
        ids = [int(t) for t in np.asarray(prediction).reshape(-1)]
        out["prediction"] = vocabulary.decode(ids)
        if output_ids:
          out["prediction_tokens"] = ids[:ids.index(0)] if 0 in ids else ids
        if mode == "predict_with_aux":
          out["aux"] = _map_leaves(_json_compat, aux)
      elif mode == "score":
        out["score"] = _json_compat(np.asarray(prediction))
        if aux:
          out["aux"] = _map_leaves(_json_compat, aux)
      else:
        raise ValueError(f"Invalid mode: {mode}")
      f.write(json.dumps(out, cls=json_encoder_cls) + "\n")


def _extract_tokens_and_aux_values(outputs) -> Inferences:
  aux = {}
  if isinstance(outputs, tuple):
    indices_and_tokens, aux = outputs
  else:
    indices_and_tokens = outputs
  return [t for _, t in indices_and_tokens], aux


def update_measurement_series(series_name: str, step: int, value: float):
  """Hook for external experiment trackers; a no-op here."""


def infer(*, mode: str, model: models.BaseTransformerModel, dataset_cfg: utils.DatasetConfig,
          restore_checkpoint_cfg: utils.RestoreCheckpointConfig,
          partitioner: partitioning.BasePartitioner, output_dir: str, checkpoint_period: int,
          shard_id: int = 0, num_shards: int = 1, merge_chunked_results: bool = True,
          write_fn: Callable = write_inferences_to_file, checkpoint_ds_iter: bool = True,
          train_state_initializer_cls=utils.TrainStateInitializer,
          fallback_init_rng: Optional[int] = None, merge_fn: Callable = merge_chunks_to_file,
          summarize_config_fn: Callable = gin_utils.summarize_gin_config,
          verify_matching_vocabs_fn: Optional[Callable] = utils.verify_matching_vocabs,
          output_vocab_feature_name: str = "targets", file_extension: str = "jsonl",
          keep_aux_as_numpy: bool = False, use_orbax: bool = True):
  """Runs `mode` ('predict', 'score' or 'predict_with_aux') over a task or mixture and writes
  JSONL results (t5x/infer.py:365-738)."""
  is_rank0 = pstate.get().rank == 0
  os.makedirs(output_dir, exist_ok=True)
  if shard_id == 0:
    summarize_config_fn(model_dir=output_dir, summary_writer=None, step=0)
  if mode not in ("predict", "score", "predict_with_aux"):
    raise ValueError("`mode` must be one of 'predict', 'score' or 'predict_with_aux'. "
                     f"Got '{mode}'")
  output_dir = re.sub(r"(?<!gs:)([\/]{2,})", "/", output_dir)
  if verify_matching_vocabs_fn is not None:
    verify_matching_vocabs_fn(dataset_cfg, model)
  batch_size = dataset_cfg.batch_size
  if dataset_cfg.module:
    utils.import_module(dataset_cfg.module)
  shard_info = seqio.ShardInfo(index=shard_id, num_shards=num_shards)
  task_or_mixture = seqio.get_mixture_or_task(dataset_cfg.mixture_or_task_name)
  converter = model.FEATURE_CONVERTER_CLS(pack=False)

  def _get_dataset(provider):
    return provider.get_dataset(sequence_length=dataset_cfg.task_feature_lengths,
                                split=dataset_cfg.split, shuffle=False, num_epochs=1,
                                shard_info=shard_info, use_cached=dataset_cfg.use_cached,
                                seed=dataset_cfg.seed)

  logging.info("Inferring with checkpoints every %d batches of %d examples.",
               checkpoint_period, batch_size)
  lengths = converter.get_model_feature_lengths(dataset_cfg.task_feature_lengths)
  input_shapes = {k: (batch_size, v) for k, v in lengths.items()}
  initializer = train_state_initializer_cls(optimizer_def=None,
                                            init_fn=model.get_initial_variables,
                                            input_shapes=input_shapes, partitioner=partitioner)
  if shard_id == 0:
    utils.log_model_info(os.path.join(output_dir, "model-info.txt"),
                         initializer.global_train_state_shape, partitioner)
  restore_checkpoint_cfg.strict = False
  train_state, manager = utils.create_checkpoint_manager_and_restore(
      initializer, partitioner, restore_checkpoint_cfg, restore_checkpoint_cfg.path,
      fallback_init_rng, use_orbax=use_orbax)
  if train_state is None:
    raise ValueError("TrainState was not found or could not be restored.")
  infer_step = {"predict": model.predict_batch, "predict_with_aux": model.predict_batch_with_aux,
                "score": model.score_batch}[mode]
  infer_fn = functools.partial(
      utils.get_infer_fn(infer_step=infer_step, batch_size=batch_size,
                         train_state_axes=initializer.train_state_axes, partitioner=partitioner,
                         keep_aux_as_numpy=keep_aux_as_numpy), train_state=train_state)

  def infer_task(task):
    tmp_dir = os.path.join(output_dir, f"tmp-{task.name}-{shard_id:05}-of-{num_shards:05}")
    if is_rank0:
      os.makedirs(tmp_dir, exist_ok=True)
    utils.sync_global_devices(f"{task.name}:tmp_dir")
    output_fname = f"{task.name}-{mode}.{file_extension}-{shard_id:05}-of-{num_shards:05}"
    if os.path.exists(os.path.join(output_dir, f"{output_fname}.COMPLETED")):
      logging.info("File %s exists. Skipping inference for shard %d/%d of task '%s'",
                   output_fname, shard_id, num_shards, task.name)
      return
    pool = FailFastThreadPoolExecutor(max_workers=1)
    examples = list(_get_dataset(task))
    chunk_examples = checkpoint_period * batch_size
    num_chunks = -(-len(examples) // chunk_examples) if examples else 0
    # The input position is the index of the first chunk not yet written.
    pos_path = os.path.join(tmp_dir, "input.ckpt")
    first_chunk = 0
    if checkpoint_ds_iter and os.path.exists(pos_path):
      with open(pos_path) as f:
        first_chunk = int(json.load(f)["next_chunk"])
      logging.info("Restoring input iterator from %s (chunk %d)", pos_path, first_chunk)
    vocabulary = task.output_features[output_vocab_feature_name].vocabulary

    def write_chunk(chunk, chunk_path, inferences, task_examples):
      tick = time.time()
      write_fn(chunk_path, inferences, task_examples, mode, vocabulary)
      with open(chunk_path + ".COMPLETED", "w") as f:
        f.write("")
      dt = max(time.time() - tick, 1e-9)
      update_measurement_series("writing_total_sec", chunk, dt)
      update_measurement_series("writing_examples_per_sec", chunk, len(inferences[0]) / dt)
      if checkpoint_ds_iter:
        tmp = pos_path + f".{chunk}.tmp"
        with open(tmp, "w") as f:
          json.dump({"next_chunk": chunk + 1}, f)
        os.replace(tmp, pos_path)

    for chunk in range(first_chunk, num_chunks):
      tick = time.time()
      chunk_path = os.path.join(tmp_dir, f"{output_fname}-chunk{chunk:05}")
      if os.path.exists(chunk_path + ".COMPLETED") and not checkpoint_ds_iter:
        assert os.path.exists(chunk_path)
        logging.info("Skipping chunk %s. Chunk file already exists.", chunk)
        continue
      task_examples = examples[chunk * chunk_examples:(chunk + 1) * chunk_examples]
      model_ds = seqio.Dataset.from_examples(task_examples).convert(
          converter, dataset_cfg.task_feature_lengths)
      result = infer_fn(model_ds.enumerate(), rng=chunk)
      inferences = _extract_tokens_and_aux_values(result)
      if is_rank0:
        dt = max(time.time() - tick, 1e-9)
        logging.info("chunk %d completed in %02f seconds (%02f examples/sec).", chunk, dt,
                     len(inferences[0]) / dt)
        update_measurement_series("inference_total_sec", chunk, dt)
        update_measurement_series("inference_examples_per_sec", chunk, len(inferences[0]) / dt)
        pool.submit(write_chunk, chunk, chunk_path, inferences, task_examples)
      utils.sync_global_devices(f"{task.name}:checkpoint_chunk{chunk:05}")
    pool.shutdown(wait=True)
    if is_rank0 and merge_chunked_results:
      merge_fn(output_dir, output_fname, tmp_dir, int(utils.get_local_data(train_state.step)))
      shutil.rmtree(tmp_dir)
    if is_rank0:
      with open(os.path.join(output_dir, f"{output_fname}.COMPLETED"), "w") as f:
        f.write("")
    utils.sync_global_devices(f"{task.name}:complete")

  subtasks = (task_or_mixture.tasks if isinstance(task_or_mixture, seqio.Mixture)
              else [task_or_mixture])
  for task in subtasks:
    logging.info("Starting inference for task '%s'", task.name)
    infer_task(task)
  manager.close()
  logging.info("DONE")


def main(argv: Optional[Sequence[str]] = None) -> None:
  from t5x_b200 import train as train_lib
  logging.basicConfig(level=logging.INFO)
  argv = gin_utils.rewrite_gin_args(list(sys.argv[1:] if argv is None else argv))
  ap = train_lib.build_flag_parser(__doc__)
  ap.add_argument("--shard_id", type=int, default=None,
                  help="Index of this job among independent inference jobs over one dataset.")
  flags = ap.parse_args(argv)
  train_lib.init_distributed_from_flags(flags)
  from t5x_b200 import config_utils
  if config_utils.using_fdl(flags):
    if flags.shard_id is not None:
      flags.fdl_set = list(flags.fdl_set) + [f"shard_id={flags.shard_id}"]
    config_utils.run_with_fiddle(infer, flags)
    return
  gin.set_main_module(sys.modules[__name__])
  train_lib.parse_gin_from_flags(flags, train_lib._DEFAULT_GIN_SEARCH_PATHS)
  fn = gin.get_configurable(infer)
  if flags.shard_id is not None:
    fn(shard_id=flags.shard_id)
  else:
    fn()


if __name__ == "__main__":
  main()
