"""Model export for serving (role of t5x/export_lib.py).

The reference converts the model to a TensorFlow SavedModel (jax2tf) for TPU/TF serving. The
equivalent here is a self-describing inference bundle that a B200 serving process loads with
`load()`:

  <output_dir>/<model_name>/<version>/
      checkpoint_<step>/   inference-only T5X-format checkpoint (parameters in `dtype`)
      config.gin           the operative configuration that rebuilds the model object
      signature.json       inference mode, feature lengths, batch size, decoding options
      warmup.jsonl         example requests (`write_warmup_examples`)

`ExportableModule` is the serving-side callable: text in, text (or scores) out, through the
same tokenisation, feature conversion and CUDA-graph decoder the batch entry points use.
"""
from __future__ import annotations

import dataclasses
import json
import logging
import os
import time
from typing import Any, Callable, List, Mapping, Optional, Sequence

import numpy as np
import torch

from t5x_b200 import checkpoints
from t5x_b200 import gin
from t5x_b200 import gin_utils
from t5x_b200 import models
from t5x_b200 import partitioning
from t5x_b200 import train_state as train_state_lib
from t5x_b200 import utils
from t5x_b200.parallel import state as pstate


def create_preprocessor(output_features: Mapping[str, Any],
                        task_feature_lengths: Mapping[str, int],
                        tokenized_inputs: bool = False) -> Callable:
  """text (or token lists) -> {"inputs": int32 [len]} examples."""
  vocab = output_features["inputs"].vocabulary
  add_eos = getattr(output_features["inputs"], "add_eos", True)
  limit = task_feature_lengths["inputs"]

  def preprocess(texts: Sequence[Any]) -> List[dict]:
    out = []
    for t in texts:
      ids = list(t) if tokenized_inputs else list(vocab.encode(t))
      if add_eos:
        ids = ids[:limit - 1] + [vocab.eos_id]
      out.append({"inputs": np.asarray(ids[:limit], np.int32),
                  "targets": np.zeros((0,), np.int32)})
    return out

  return preprocess


def create_preprocessor_from_task(model=None, task_feature_lengths: Mapping[str, int] = None,
                                  task_name: str = None, serialized_examples: bool = True,
                                  run_precache: bool = False, **_) -> Callable:
  """Serving preprocessor that takes whole examples of a registered task instead of bare
  input strings (role of t5x/export_lib.py `create_preprocessor_from_task`): each request is
  a feature dictionary (a JSON string of one when `serialized_examples`) whose text features
  are tokenised with the task's vocabularies and trimmed to `task_feature_lengths`."""
  from t5x_b200.data import tasks as tasks_lib
  features = tasks_lib.get_mixture_or_task(task_name).output_features

  def preprocess(items: Sequence[Any]) -> List[dict]:
    out = []
    for item in items:
      if serialized_examples and isinstance(item, (str, bytes)):
        item = json.loads(item)
      ex = {}
      for name, feat in features.items():
        value = item.get(name, [] if name != "inputs" else "")
        ids = list(feat.vocabulary.encode(value)) if isinstance(value, str) else list(value)
        limit = (task_feature_lengths or {}).get(name)
        if getattr(feat, "add_eos", True) and name == "inputs":
          ids = (ids[:limit - 1] if limit else ids) + [feat.vocabulary.eos_id]
        ex[name] = np.asarray(ids[:limit] if limit else ids, np.int32)
      ex.setdefault("targets", np.zeros((0,), np.int32))
      out.append(ex)
    return out

  return preprocess


def create_postprocessor(vocab, inference_mode: str = "predict", tokenized_outputs: bool = False,
                         output_feature_names: Optional[Sequence[str]] = None) -> Callable:
  def postprocess(values, aux=None):
    if inference_mode == "score":
      return {"scores": [float(v) for v in values]}
    if tokenized_outputs:
      texts = [[int(t) for t in row] for row in values]
    else:
      texts = [vocab.decode([int(t) for t in row]) for row in values]
    res = {"outputs": texts}
    if aux and "scores" in aux:
      res["scores"] = [float(s) for s in np.asarray(aux["scores"]).reshape(-1)]
    return res
  return postprocess


def create_inference_function(*, model: models.BaseTransformerModel, inference_mode: str,
                              train_state_initializer=None, partitioner=None,
                              decoder_params_spec=(), enable_xla: bool = True,
                              polymorphic_shapes_inputs=None, native_lowering: bool = True,
                              output_len: Optional[int] = None) -> Callable:
  """(params, batch) -> outputs for 'predict' or 'score'."""
  if inference_mode not in ("predict", "score"):
    raise ValueError("`inference_mode` must be a string in ('predict', 'score'). "
                     f"Got '{inference_mode}'")

  def fn(params, batch):
    with torch.no_grad():
      if inference_mode == "predict":
        out, aux = model.predict_batch_with_aux(params, batch)
        if output_len:
          out = out[:, :output_len]
        return out, aux
      return model.score_batch(params, batch), {}
  return fn


def create_batch_polymorphic_shapes(input_signature, preprocessor=None):
  """Shapes with a free batch dimension (serving batches of any size are padded by
  `ExportableModule`)."""
  return {k: ("b",) + tuple(v)[1:] for k, v in dict(input_signature).items()}


def write_warmup_examples(batch_size: int, output_dir: str, model_name: str,
                          input_texts: Sequence[str] = ("hello world",), **_) -> None:
  path = os.path.join(output_dir, "warmup.jsonl")
  with open(path, "w") as f:
    for i in range(max(1, batch_size)):
      f.write(json.dumps({"model": model_name, "inputs": input_texts[i % len(input_texts)]})
              + "\n")


class ExportableModule:
  """Serving callable: `module(["text", ...]) -> {"outputs": [...], "scores": [...]}`."""

  def __init__(self, model, params, preproc_fn: Callable, model_fn: Callable,
               postproc_fn: Callable, task_feature_lengths: Mapping[str, int],
               batch_size: Optional[int] = None, jit_compile: bool = True,
               use_batch_function: bool = False, **_):
    self._model, self._params = model, params
    self._pre, self._fn, self._post = preproc_fn, model_fn, postproc_fn
    self._lengths = dict(task_feature_lengths)
    self._batch_size = batch_size

  def __call__(self, texts: Sequence[Any]):
    from t5x_b200.data import dataset as dataset_lib
    n = len(texts)
    bs = self._batch_size or n
    examples = self._pre(texts)
    outs, scores = [], []
    dev = pstate.get().device
    for i in range(0, n, bs):
      chunk = examples[i:i + bs]
      chunk = chunk + [chunk[0]] * (bs - len(chunk))  # fixed batch shape
      ds = dataset_lib.Dataset.from_examples(chunk).convert(
          self._model.FEATURE_CONVERTER_CLS(pack=False), self._lengths)
      rows = list(ds)
      batch = {k: torch.from_numpy(np.stack([np.asarray(r[k]) for r in rows])).to(dev)
               for k in rows[0]}
      out, aux = self._fn(self._params, batch)
      res = self._post(out.cpu().numpy()[:min(bs, n - i)],
                       {k: v.cpu().numpy()[:min(bs, n - i)] for k, v in aux.items()})
      outs.extend(res.get("outputs", []))
      scores.extend(res.get("scores", []))
    result = {}
    if outs:
      result["outputs"] = outs
    if scores:
      result["scores"] = scores
    return result


def save(*, model: models.BaseTransformerModel, inference_mode: str,
         restore_checkpoint_cfg: utils.RestoreCheckpointConfig,
         exportable_module_cls=ExportableModule,
         create_preprocessor_fn: Callable = create_preprocessor,
         create_inference_function_fn: Callable = create_inference_function,
         create_postprocessor_fn: Callable = create_postprocessor,
         partitioner: Optional[partitioning.BasePartitioner] = None,
         create_polymorphic_shapes_fn: Callable = create_batch_polymorphic_shapes,
         write_warmup_example_fn: Callable = write_warmup_examples,
         output_features: Optional[Mapping[str, Any]] = None,
         task_feature_lengths: Mapping[str, int] = None, batch_size: Optional[int] = None,
         output_dir: str = None, model_name: str = "model", warmup_examples=None,
         tokenized_inputs: bool = False, tokenized_outputs: bool = False,
         export_dtype: str = "bfloat16", version: Optional[int] = None,
         mixture_or_task_name: Optional[str] = None, **_):
  """Restores the checkpoint and writes the inference bundle; returns its directory."""
  partitioner = partitioner or partitioning.PjitPartitioner(num_partitions=1)
  bs = batch_size or 1
  conv = model.FEATURE_CONVERTER_CLS(pack=False)
  lens = conv.get_model_feature_lengths(task_feature_lengths)
  input_shapes = {k: (bs, v) for k, v in lens.items()}
  init = utils.TrainStateInitializer(optimizer_def=None, init_fn=model.get_initial_variables,
                                     input_shapes=input_shapes, partitioner=partitioner)
  restore_checkpoint_cfg.strict = False
  cfg, paths = utils.get_first_valid_restore_config_and_paths([restore_checkpoint_cfg])
  state, manager = utils.create_checkpoint_manager_and_restore(
      init, partitioner, cfg, paths[0] if paths else None, None)
  if state is None:
    raise ValueError("TrainState was not found or could not be restored.")
  manager.close()
  version = int(time.time()) if version is None else version
  bundle = os.path.join(output_dir, model_name, str(version))
  os.makedirs(bundle, exist_ok=True)
  ck = checkpoints.Checkpointer(state, partitioner, bundle, save_dtype=np.dtype("float32")
                                if export_dtype == "float32" else export_dtype)
  ck.save(state)
  gin_utils.summarize_gin_config(bundle, None, 0)
  with open(os.path.join(bundle, "signature.json"), "w") as f:
    json.dump({"inference_mode": inference_mode, "task_feature_lengths": dict(task_feature_lengths),
               "batch_size": batch_size, "dtype": export_dtype,
               "step": int(utils.get_local_data(state.step)),
               "tokenized_inputs": tokenized_inputs, "tokenized_outputs": tokenized_outputs,
               "mixture_or_task_name": mixture_or_task_name,
               "polymorphic_shapes": create_polymorphic_shapes_fn(input_shapes)}, f, indent=1)
  write_warmup_example_fn(bs, bundle, model_name,
                          input_texts=warmup_examples or ("hello world",))
  logging.info("Exported inference bundle to %s", bundle)
  return bundle


def load(bundle_dir: str, model: models.BaseTransformerModel,
         output_features: Optional[Mapping[str, Any]] = None,
         partitioner: Optional[partitioning.BasePartitioner] = None) -> ExportableModule:
  """Rebuilds the serving callable of a bundle around `model` (constructed by the caller,
  e.g. by parsing the bundle's config.gin)."""
  from t5x_b200.data import tasks as tasks_lib
  sig = json.load(open(os.path.join(bundle_dir, "signature.json")))
  partitioner = partitioner or partitioning.PjitPartitioner(num_partitions=1)
  lengths = sig["task_feature_lengths"]
  bs = sig["batch_size"] or 1
  conv = model.FEATURE_CONVERTER_CLS(pack=False)
  input_shapes = {k: (bs, v) for k, v in conv.get_model_feature_lengths(lengths).items()}
  init = utils.TrainStateInitializer(optimizer_def=None, init_fn=model.get_initial_variables,
                                     input_shapes=input_shapes, partitioner=partitioner)
  cfg = utils.RestoreCheckpointConfig(path=bundle_dir, mode="latest", strict=False)
  cfg, paths = utils.get_first_valid_restore_config_and_paths([cfg])
  state, manager = utils.create_checkpoint_manager_and_restore(init, partitioner, cfg, paths[0],
                                                               None)
  manager.close()
  if output_features is None:
    output_features = {"inputs": tasks_lib.Feature(model.input_vocabulary),
                       "targets": tasks_lib.Feature(model.output_vocabulary)}
  if sig.get("mixture_or_task_name"):
    pre = create_preprocessor_from_task(model, lengths, sig["mixture_or_task_name"])
  else:
    pre = create_preprocessor(output_features, lengths, sig.get("tokenized_inputs", False))
  fn = create_inference_function(model=model, inference_mode=sig["inference_mode"])
  post = create_postprocessor(model.output_vocabulary, sig["inference_mode"],
                              sig.get("tokenized_outputs", False))
  return ExportableModule(model, state.params, pre, fn, post, lengths, batch_size=sig["batch_size"])
