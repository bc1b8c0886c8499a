"""Trainer and training-loop actions (API of t5x/trainer.py).

The train step is eager PyTorch on one CUDA stream per rank:
  lr = schedule(step); dropout seed = fold(base seed, step)
  for each microbatch: loss.backward()   (weight grads accumulate in fp32 `main_grad` buffers
                                          straight from the wgrad GEMM epilogues)
  gradient reduction over the data axis; optimizer kernels update the fp32 masters and the
  bf16 working copies in place.
Metrics stay on the device until a background thread formats them, so the host never waits
for the GPU inside the loop.
"""
from __future__ import annotations

import abc
import concurrent.futures
import enum
import logging
import os
import threading
import time
from typing import (Any, Callable, Dict, Iterator, Mapping, MutableMapping, Optional, Sequence,
                    Tuple)

import numpy as np
import torch
import torch.distributed as dist

from t5x_b200 import metrics as metrics_lib
from t5x_b200 import train_state as train_state_lib
from t5x_b200.parallel import state as pstate
from t5x_b200.utils import metric_writers
from t5x_b200.utils import tree as tree_utils

BatchType = Mapping[str, Any]
MetricMapType = Mapping[str, metrics_lib.Metric]
LearningRateCallable = Callable[[int], float]


class PreemptionError(Exception):
  """Training has been interrupted and needs an emergency checkpoint."""


def merge_metrics(a, b):
  return metrics_lib.merge_metrics(a, b)


def fold_in_seed(base_seed: int, step: int) -> int:
  """Deterministic per-step seed (the role of jax.random.fold_in in t5x/trainer.py:524)."""
  x = (int(base_seed) * 0x9E3779B97F4A7C15 + int(step) * 0xBF58476D1CE4E5B9 + 0x94D049BB133111EB)
  x &= (1 << 64) - 1
  x ^= x >> 31
  return x & ((1 << 62) - 1)


# ----------------------------------------------------------------------------
# Weight metrics
# ----------------------------------------------------------------------------
class WeightMetricsComputer:
  """Per-tensor RMS/max and global norms of weights, gradients and updates
  (t5x/trainer.py:151-232)."""

  _WEIGHT_METRICS = ["weight_rms", "weight_gradient_rms", "weight_update_rms", "weight_max"]

  @staticmethod
  def _rms(x):
    return torch.sqrt(torch.mean(x.float() ** 2))

  @staticmethod
  def holds(p) -> bool:
    """Whether this rank contributes parameter `p` to the metrics. With the optimizer sharded
    over the data axis, the reduced gradient, the fp32 weights and hence the update of a
    parameter exist on its owner only; replicated parameters are counted by data rank 0."""
    z = getattr(p, "zero", None)
    if z is not None:
      return z.mine
    from t5x_b200.parallel import zero
    return zero.active() is None or pstate.get().data_rank == 0

  def compute_metrics(self, gradients, old_params, new_train_state) -> MutableMapping[str, Any]:
    """`old_params` needs entries only for the parameters this rank `holds`."""
    flat_g = tree_utils.flatten_dict(gradients)
    flat_old = tree_utils.flatten_dict(old_params)
    flat_new = tree_utils.flatten_dict(new_train_state.params)
    names = list(flat_g)
    first = next(iter(flat_new.values()))
    # per parameter: sum g^2, sum w^2, sum (w - w_old)^2, max |w|
    stats = torch.zeros(len(names), 4, dtype=torch.float32, device=first.device)
    for i, k in enumerate(names):
      new = flat_new[k].detach()
      if not self.holds(flat_new[k]):
        continue
      upd = new.float() - flat_old[k].float()
      stats[i, 0] = (flat_g[k].float() ** 2).sum()
      stats[i, 1] = (new.float() ** 2).sum()
      stats[i, 2] = (upd ** 2).sum()
      stats[i, 3] = new.abs().max()
    from t5x_b200.parallel import zero
    if zero.active() is not None:
      st = pstate.get()
      sums, tops = stats[:, :3].contiguous(), stats[:, 3].contiguous()
      dist.all_reduce(sums, group=st.data_group)
      dist.all_reduce(tops, op=dist.ReduceOp.MAX, group=st.data_group)
      stats = torch.cat([sums, tops[:, None]], dim=1)
    out = {}
    for i, k in enumerate(names):
      n = float(max(flat_new[k].numel(), 1))
      avg = metrics_lib.AveragePerStep.from_model_output
      out[f"weight_rms/{k}"] = avg(torch.sqrt(stats[i, 1] / n))
      out[f"weight_gradient_rms/{k}"] = avg(torch.sqrt(stats[i, 0] / n))
      out[f"weight_update_rms/{k}"] = avg(torch.sqrt(stats[i, 2] / n))
      out[f"weight_max/{k}"] = avg(stats[i, 3])
    total = stats[:, :3].sum(dim=0)
    out["weight_gradient_norm"] = metrics_lib.AveragePerStep.from_model_output(torch.sqrt(total[0]))
    out["weight_norm"] = metrics_lib.AveragePerStep.from_model_output(torch.sqrt(total[1]))
    out["weight_update_norm"] = metrics_lib.AveragePerStep.from_model_output(torch.sqrt(total[2]))
    return out


# ----------------------------------------------------------------------------
# Metrics manager
# ----------------------------------------------------------------------------
class _AsyncTimer:
  """Wall-clock between two points at which given device work has completed
  (t5x/trainer.py:235-287): start/stop each record a CUDA event on the current stream and a
  worker thread waits on it, so the duration excludes host run-ahead."""

  def __init__(self):
    self._pool = concurrent.futures.ThreadPoolExecutor(max_workers=1,
                                                       thread_name_prefix="AsyncTimer")
    self._start_future = None

  def close(self):
    self._pool.shutdown(wait=True)

  @staticmethod
  def _marker():
    if torch.cuda.is_available():
      ev = torch.cuda.Event()
      ev.record()
      return ev
    return None

  def _stamp(self, marker):
    if marker is not None:
      marker.synchronize()
    return time.time()

  def start(self, block_on=()):
    self._start_future = self._pool.submit(self._stamp, self._marker())

  def stop(self, block_on=()) -> concurrent.futures.Future:
    if self._start_future is None:
      raise ValueError("The timer hasn't been started.")
    start_future = self._start_future
    marker = self._marker()

    def fn():
      start = start_future.result()
      return self._stamp(marker) - start

    return self._pool.submit(fn)


def _fetch(v):
  if isinstance(v, torch.Tensor):
    return v.detach().float().cpu().item() if v.numel() == 1 else v.detach().cpu()
  return v


def _fetch_metric(m: metrics_lib.Metric) -> metrics_lib.Metric:
  import dataclasses
  return m.replace(**{f.name: _fetch(getattr(m, f.name)) for f in dataclasses.fields(m)})


class MetricsManager:
  """Accumulated metrics -> TensorBoard + log, on rank 0 only (t5x/trainer.py:290-443)."""

  def __init__(self, name: str, summary_dir: Optional[str] = None):
    self._name = name
    if pstate.get().rank == 0:
      self._writer = self._create_writer(name, summary_dir)
    else:
      self._writer = metric_writers.MultiWriter([])
    self.summary_dir = os.path.join(summary_dir, name) if summary_dir else None
    self._writer_lock = threading.Lock()
    self._summary_pool = concurrent.futures.ThreadPoolExecutor(
        max_workers=1, thread_name_prefix="MetricsManager")
    self._pending = []
    self._duration_timer = _AsyncTimer()

  def _create_writer(self, name, summary_dir=None):
    return metric_writers.create_default_writer(summary_dir, collection=name, asynchronous=True)

  def close(self):
    try:
      self.flush()
      self._summary_pool.shutdown(wait=True)
    finally:
      try:
        self._duration_timer.close()
      finally:
        if self._writer:
          self._writer.close()
          self._writer = None

  @property
  def summary_writer(self):
    return self._writer

  def write_scalar(self, key: str, val, step: int):
    self.write_scalars(int(step), {key: val})

  def write_scalars(self, step: int, scalars: Mapping[str, Any]):
    with self._writer_lock:
      self._writer.write_scalars(int(step), scalars)

  def start_duration_timer(self, block_on=()):
    self._duration_timer.start(block_on=block_on)

  def write_metrics_summary(self, metrics: MetricMapType, step: int,
                            num_steps: int) -> concurrent.futures.Future:
    """Formats and writes the accumulated metrics on the background thread; the returned
    future resolves to {name: Scalar}."""
    step = int(step)
    duration_future = self._duration_timer.stop(block_on=metrics)

    def _summarize_and_write():
      fetched = {k: _fetch_metric(v) for k, v in metrics.items()}
      duration = duration_future.result()
      final = metrics_lib.set_time_metrics_duration(fetched, duration)
      final = metrics_lib.set_step_metrics_num_steps(final, num_steps)
      summary = {k: v.compute_value() for k, v in final.items()}
      with self._writer_lock:
        if self._writer is not None:
          self._writer.write_scalars(step, {k: v.value for k, v in summary.items()
                                           if isinstance(v, metric_writers.Scalar)})
      return summary

    fut = self._summary_pool.submit(_summarize_and_write)
    self._pending.append(fut)
    return fut

  def flush(self):
    for f in self._pending:
      f.result()
    self._pending = []
    if self._writer:
      self._writer.flush()


# ----------------------------------------------------------------------------
# Gradient buffers
# ----------------------------------------------------------------------------
def attach_compute_buffers(params, bf16_copy: bool = True, main_grad: bool = True) -> None:
  """Gives every fp32 CUDA parameter a bf16 working copy and an fp32 gradient accumulator
  (read by the ops in `t5x_b200.ops.functional`, written by the optimizer kernels)."""
  for p in tree_utils.flatten_dict(params).values():
    if not isinstance(p, torch.Tensor) or p.dtype != torch.float32:
      continue
    if bf16_copy and p.is_cuda and getattr(p, "bf16", None) is None:
      p.bf16 = p.detach().to(torch.bfloat16)
    if main_grad and getattr(p, "main_grad", None) is None:
      p.main_grad = torch.zeros_like(p, dtype=torch.float32, requires_grad=False)
    p.grad_ready = False


def _begin_step(params_flat) -> None:
  for p in params_flat.values():
    p.grad_ready = False
    p.grad = None


def _collect_grads(params_flat) -> Dict[str, torch.Tensor]:
  """After the last microbatch: every parameter's total gradient as an fp32 tensor."""
  grads = {}
  for k, p in params_flat.items():
    mg = getattr(p, "main_grad", None)
    if mg is None:
      grads[k] = (p.grad if p.grad is not None else torch.zeros_like(p)).float()
      continue
    if p.grad is not None:  # gradient that arrived through plain autograd
      if getattr(p, "grad_ready", False):
        mg.add_(p.grad)
      else:
        mg.copy_(p.grad)
        p.grad_ready = True
      p.grad = None
    if not getattr(p, "grad_ready", False):
      mg.zero_()
    grads[k] = mg
  return grads


def _fold_autograd_grads(params_flat) -> None:
  """Between microbatches: move `.grad` of autograd-path parameters into main_grad."""
  for p in params_flat.values():
    mg = getattr(p, "main_grad", None)
    if mg is None or p.grad is None:
      continue
    if getattr(p, "grad_ready", False):
      mg.add_(p.grad)
    else:
      mg.copy_(p.grad)
      p.grad_ready = True
    p.grad = None


def reduce_partial_gradients_over_model_axis(grads_flat, params_flat) -> None:
  """Replicated parameters applied to row-sharded activations (the norm scales of the fused
  tensor-parallel path, marked `sp_partial_grad`) hold the gradient of this rank's rows only:
  sums them over the model axis in one all-reduce."""
  st = pstate.get()
  if st.model_size <= 1 or st.model_group is None:
    return
  keys = [k for k, p in params_flat.items() if getattr(p, "sp_partial_grad", False)]
  if not keys:
    return
  flat = torch.cat([grads_flat[k].reshape(-1) for k in keys])
  dist.all_reduce(flat, group=st.model_group)
  off = 0
  for k in keys:
    n = grads_flat[k].numel()
    grads_flat[k].copy_(flat[off:off + n].view_as(grads_flat[k]))
    off += n


_COALESCE_MAX_NUMEL = 1 << 18  # gradients up to this size travel in one flattened all-reduce


def reduce_gradients_over_data_axis(grads_flat: Mapping[str, torch.Tensor], params_flat) -> None:
  """Sum of gradients over data-parallel replicas (losses are sums, not means, so the global
  gradient is the sum; t5x/trainer.py:815-828). Expert-sharded parameters are reduced over
  the pure data axis only."""
  st = pstate.get()
  if st.world_size == 1:
    return
  if st.data_size * st.expert_size > 1 and st.data_group is not None:
    small, small_numel = [], 0
    for k, g in grads_flat.items():
      if getattr(params_flat[k], "expert_sharded", False):
        continue
      if getattr(params_flat[k], "zero", None) is not None:
        continue  # summed by its owner inside the optimizer kernels
      if g.dtype == torch.float32 and g.numel() <= _COALESCE_MAX_NUMEL:
        small.append(g)
        small_numel += g.numel()
      else:
        dist.all_reduce(g, group=st.data_group)
    if small:
      # norm scales, bias tables and the like: one collective for all of them
      flat = torch.cat([g.reshape(-1) for g in small])
      dist.all_reduce(flat, group=st.data_group)
      off = 0
      for g in small:
        g.copy_(flat[off:off + g.numel()].view_as(g))
        off += g.numel()
  from t5x_b200.parallel import zero
  ctx = zero.active()
  if ctx is not None:
    ctx.gradients_complete()


# ----------------------------------------------------------------------------
# Step functions
# ----------------------------------------------------------------------------
def _slice_batch(batch, i: int, n: int):
  out = {}
  for k, v in batch.items():
    b = v.shape[0]
    if b % n:
      raise ValueError(f"Batch size {b} is not divisible by num_microbatches {n}")
    m = b // n
    out[k] = v[i * m:(i + 1) * m]
  return out


def accumulate_grads_microbatched(model, train_state, batch: BatchType, dropout_rng: int,
                                  num_microbatches: Optional[int],
                                  data_partition_spec=None, learning_rate=None):
  """Gradients (fp32, summed over microbatches) and merged metrics
  (t5x/trainer.py:704-852)."""
  params = train_state.params
  flat = tree_utils.flatten_dict(params)
  _begin_step(flat)
  n = num_microbatches if num_microbatches and num_microbatches > 1 else 1
  metrics = None
  from t5x_b200.parallel import zero
  ctx = zero.overlap_controller()
  for i in range(n):
    mb = batch if n == 1 else _slice_batch(batch, i, n)
    rng = None if dropout_rng is None else fold_in_seed(dropout_rng, i)
    loss, m = model.loss_fn(params, mb, rng)
    if ctx is not None and i == n - 1 and learning_rate is not None and \
        hasattr(train_state, "_optimizer"):
      # gradients become final layer by layer during this backward pass: let the owners
      # start their fused reduce + update while the pass is still running
      opt = train_state._optimizer
      ctx.begin_overlap(int(train_state.step), opt.optimizer_def.update_hyper_params(
          learning_rate=learning_rate))
    loss.backward()
    _fold_autograd_grads(flat)
    metrics = m if metrics is None else merge_metrics(metrics, m)
  if ctx is not None:
    ctx.end_overlap()  # updates issued under the last backward pass are ordered before what follows
  grads = _collect_grads(flat)
  reduce_partial_gradients_over_model_axis(grads, flat)
  reduce_gradients_over_data_axis(grads, flat)
  metrics = reduce_metrics_over_data_axis(metrics)
  return tree_utils.unflatten_dict(grads), metrics, None


_SUMMED_METRIC_FIELDS = ("total", "count", "numerator")


def reduce_metrics_over_data_axis(metrics: MetricMapType) -> MetricMapType:
  """Sums the per-example accumulators of model metrics over the data-parallel replicas, so
  that every rank reports the metrics of the global batch (one small all-reduce per step)."""
  st = pstate.get()
  if metrics is None or st.data_size * st.expert_size <= 1 or st.data_group is None \
      or not dist.is_initialized():
    return metrics
  slots = []
  for name in sorted(metrics):
    m = metrics[name]
    for f in _SUMMED_METRIC_FIELDS:
      v = getattr(m, f, None)
      if v is not None:
        slots.append((name, f, v))
  if not slots:
    return metrics
  vec = torch.stack([torch.as_tensor(v, device=st.device).double().reshape(()) for _, _, v in slots])
  dist.all_reduce(vec, group=st.data_group)
  out = dict(metrics)
  for i, (name, f, v) in enumerate(slots):
    dtype = v.dtype if isinstance(v, torch.Tensor) else torch.float32
    out[name] = out[name].replace(**{f: vec[i].to(dtype)})
  return out


def apply_grads(train_state, grad_accum, metrics: MetricMapType, learning_rate,
                weight_metrics_computer: Optional[WeightMetricsComputer],
                other_state_variables: Optional[Mapping[str, Any]] = None):
  """Optimizer update + learning-rate / weight metrics (t5x/trainer.py:855-896)."""
  old_params = None
  if weight_metrics_computer is not None:
    old_params = {k: v.detach().clone()
                  for k, v in tree_utils.flatten_dict(train_state.params).items()
                  if weight_metrics_computer.holds(v)}
  with torch.no_grad():
    new_train_state = train_state.apply_gradient(grad_accum, learning_rate=learning_rate,
                                                 **(other_state_variables or {}))
    from t5x_b200.parallel import zero
    ctx = zero.active()
    if ctx is not None:
      ctx.update_complete()
  metrics = dict(metrics)
  metrics["learning_rate"] = metrics_lib.AveragePerStep(total=torch.as_tensor(learning_rate))
  metrics["learning_rate/current"] = metrics_lib.LastValue(value=torch.as_tensor(learning_rate))
  if weight_metrics_computer is not None:
    metrics.update(weight_metrics_computer.compute_metrics(
        grad_accum, tree_utils.unflatten_dict(old_params), new_train_state))
  return new_train_state, metrics


def eval_step(model, train_state, batch: BatchType) -> MetricMapType:
  _, metrics = model.eval_fn(train_state.params, batch)
  return metrics


def train_with_lr(train_state, batch, learning_rate, dropout_rng, model, num_microbatches,
                  weight_metrics_computer=None, data_partition_spec=None):
  grad_accum, metrics, mutables = accumulate_grads_microbatched(
      model, train_state, batch, dropout_rng, num_microbatches, data_partition_spec,
      learning_rate=learning_rate)
  return apply_grads(train_state, grad_accum, metrics, learning_rate, weight_metrics_computer)


# ----------------------------------------------------------------------------
# Trainers
# ----------------------------------------------------------------------------
def _to_device_batch(batch, device):
  out = {}
  for k, v in batch.items():
    if isinstance(v, torch.Tensor):
      out[k] = v.to(device, non_blocking=True)
    else:
      a = np.asarray(v)
      if a.dtype.kind in "iu":
        t = torch.from_numpy(a.astype(np.int64, copy=False))
      else:
        t = torch.from_numpy(a)
      if device.type == "cuda":
        t = t.pin_memory()
      out[k] = t.to(device, non_blocking=True)
  return out


class BaseTrainer(abc.ABC):
  """Train/eval loops around abstract step functions (t5x/trainer.py:450-701)."""

  def __init__(self, model, train_state, partitioner, eval_names: Sequence[str],
               summary_dir: Optional[str], train_state_axes: Any, rng: Any):
    self._model = model
    self._train_state_axes = train_state_axes
    self._base_rng = int(rng) if rng is not None else 0
    self._partitioner = partitioner
    self._compiled_train_step = None
    self._compiled_eval_steps = {}
    self._compiled_eval_step_cache = {}
    self._train_state_mutex = threading.RLock()
    self._train_state = train_state
    self.stop_training = False
    self._summary_dir = summary_dir
    self.train_metrics_manager = MetricsManager("train", summary_dir=summary_dir)
    self.eval_metrics_managers = {
        n: MetricsManager(f"training_eval/{n}", summary_dir=summary_dir) for n in eval_names}
    self._device = pstate.get().device

  def __enter__(self):
    return self

  def __exit__(self, exc_type, exc_value, traceback):
    self.close()

  def close(self):
    self.train_metrics_manager.close()
    for mm in self.eval_metrics_managers.values():
      mm.close()

  def _get_step_rng(self, step: int) -> int:
    return fold_in_seed(self._base_rng, int(step))

  @property
  def train_state(self):
    with self._train_state_mutex:
      return self._train_state

  @train_state.setter
  def train_state(self, train_state):
    with self._train_state_mutex:
      self._train_state = train_state

  def train(self, batch_iter: Iterator[BatchType], num_steps: int,
            start_step: Optional[int] = None) -> concurrent.futures.Future:
    """Runs `num_steps` steps; returns a future of the written summary."""
    metrics = None
    if start_step is None:
      start_step = int(self.train_state.step)
    self.train_metrics_manager.start_duration_timer(block_on=self.train_state)
    last_log = time.time()
    profiler = self._step_profiler()
    for step_num in range(start_step, start_step + num_steps):
      self._check_preemption()
      if time.time() - last_log > 10.0:
        logging.info("Training: step %d", step_num)
        last_log = time.time()
      profiler.step_begin(step_num)
      if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(f"train_step_{step_num}")
      with self._train_state_mutex:
        batch = _to_device_batch(next(batch_iter), self._device)
        self.train_state, metrics_update = self._train_step(self.train_state, batch, step_num)
      if torch.cuda.is_available():
        torch.cuda.nvtx.range_pop()
      self._after_step()
      profiler.step_end(step_num)
      metrics = metrics_update if metrics is None else merge_metrics(metrics, metrics_update)
    profiler.finish()
    self._replicas_stale = True
    return self.train_metrics_manager.write_metrics_summary(metrics, start_step + num_steps,
                                                            num_steps)

  def _step_profiler(self):
    """The `--profile_steps a:b` capture (see `utils/profiling.py`); idle unless requested."""
    if getattr(self, "_profiler", None) is None:
      from t5x_b200.utils import profiling
      self._profiler = profiling.StepProfiler.from_environment(
          getattr(self, "_summary_dir", None), pstate.get().rank)
    return self._profiler

  def request_preemption(self) -> None:
    """Called from a signal handler: asks the loop to stop at the next step boundary. The
    handler must not raise by itself: an exception in the middle of a step would leave the
    parameters half updated (the optimizer kernels work in place)."""
    self._preemption_requested = True

  def _check_preemption(self) -> None:
    """Between steps: raises `PreemptionError` on every rank as soon as any rank has been asked
    to stop, so that all of them write the emergency checkpoint for the same step (the role of
    `multihost_utils.reached_preemption_sync_point`, t5x/train.py:660-666)."""
    if pstate.host_any(getattr(self, "_preemption_requested", False)):
      self._preemption_requested = False
      raise PreemptionError("stop requested (SIGTERM)")

  def _after_step(self) -> None:
    """Between steps: (1) look, without waiting for the GPU, at the device status words.
    Every cross-GPU wait in the kernels (barriers, the flags of the fused gather/scatter
    GEMMs) gives up after a bounded number of polls and records why; the kernels behind it
    would then run on incomplete gradients, weights or inbox rows, so the run stops with a
    `KernelStatusError` instead of training on them. (2) Return all bytes of the
    tensor-parallel arena, at a point every rank reaches in the same order."""
    if self._device.type != "cuda":
      return
    from t5x_b200.parallel import tp_fused
    if tp_fused._ARENA is not None:
      tp_fused._ARENA.end_step()
    if getattr(self, "_status_poller", None) is None:
      from t5x_b200.ops import native
      self._status_poller = native.StatusPoller()
    self._status_poller.poll()

  def check_kernel_status(self) -> None:
    """Blocking form of the status check, for points where the state leaves the loop."""
    if self._device.type == "cuda":
      if getattr(self, "_status_poller", None) is None:
        from t5x_b200.ops import native
        self._status_poller = native.StatusPoller()
      self._status_poller.check()

  def sync_replicas(self) -> None:
    """With the optimizer sharded over the data axis, brings every replica's fp32 master
    weights and optimizer slots up to date with their owners. Callers invoke it whenever the
    state leaves the training loop (checkpointing, returning the final state); forward passes
    do not need it because they read the bf16 working weights, which are always current."""
    from t5x_b200.parallel import zero
    self.check_kernel_status()  # a checkpoint must not be written from a step that gave up
    ctx = zero.active()
    if ctx is not None and getattr(self, "_replicas_stale", False):
      ctx.sync_replicas(getattr(self.train_state, "param_states", None))
    self._replicas_stale = False

  def compile_train(self, batch) -> None:
    """Warms up the train step's kernels and allocator pools (no-op on the CPU path): the
    analogue of ahead-of-time compilation in the reference (t5x/trainer.py:581-603)."""
    tick = time.time()
    self._compiled_train_step = self._train_step
    self.train_metrics_manager.write_scalar("timing/compilation_seconds", time.time() - tick,
                                            int(self.train_state.step))

  def eval(self, batch_iters: Mapping[str, Iterator[BatchType]]) -> Mapping[str, Any]:
    """Teacher-forced evaluation over whole iterators (t5x/trainer.py:605-649)."""
    eval_summaries = {}
    train_state = self.train_state
    for iter_name, batch_iter in batch_iters.items():
      logging.info("Evaluating: %s.", iter_name)
      metrics = None
      mm = self.eval_metrics_managers[iter_name]
      mm.start_duration_timer(block_on=train_state)
      num_steps = 0
      for batch in batch_iter:
        num_steps += 1
        with torch.no_grad():
          mu = self._eval_step(train_state, _to_device_batch(batch, self._device))
        if self._device.type == "cuda":
          from t5x_b200.parallel import tp_fused
          tp_fused.end_step()
        metrics = mu if metrics is None else merge_metrics(metrics, mu)
      _assert_equal_across_ranks(num_steps, "eval step mismatch across ranks")
      if metrics is None:
        continue
      eval_summaries[iter_name] = mm.write_metrics_summary(metrics, int(train_state.step),
                                                           num_steps)
    for mm in self.eval_metrics_managers.values():
      mm.flush()
    return {k: v.result() for k, v in eval_summaries.items()}

  def compile_eval(self, batches: Mapping[str, BatchType]) -> None:
    for name in batches:
      self._compiled_eval_steps[name] = self._eval_step

  @abc.abstractmethod
  def _train_step(self, train_state, batch, step_num):
    ...

  @abc.abstractmethod
  def _eval_step(self, train_state, batch):
    ...


def _assert_equal_across_ranks(value: int, msg: str) -> None:
  st = pstate.get()
  if st.world_size == 1 or not dist.is_initialized():
    return
  t = torch.tensor([value, -value], dtype=torch.int64, device=st.device)
  dist.all_reduce(t, op=dist.ReduceOp.MAX)
  if int(t[0]) != value or int(-t[1]) != value:
    raise AssertionError(f"{msg}: rank {st.rank} has {value}, range [{-int(t[1])}, {int(t[0])}]")


class Trainer(BaseTrainer):
  """The standard trainer (t5x/trainer.py:969-1051)."""

  def __init__(self, model, train_state, partitioner, eval_names: Sequence[str],
               summary_dir: Optional[str], train_state_axes: Any, rng: Any,
               learning_rate_fn: LearningRateCallable, num_microbatches: Optional[int],
               weight_metrics_computer: Optional[WeightMetricsComputer] = None):
    self._learning_rate_fn = learning_rate_fn
    self._num_microbatches = num_microbatches
    self._weight_metrics_computer = weight_metrics_computer
    super().__init__(model=model, train_state=train_state, partitioner=partitioner,
                     eval_names=eval_names, summary_dir=summary_dir,
                     train_state_axes=train_state_axes, rng=rng)
    if hasattr(train_state, "params"):
      # Sharding allocates the working weights and gradient accumulators itself (in memory
      # that all replicas map); only parameters it does not cover get private buffers.
      self._local_overlap_args = None
      self._maybe_shard_optimizer(train_state, weight_metrics_computer)
      attach_compute_buffers(train_state.params,
                             bf16_copy=self._device.type == "cuda", main_grad=True)
      if self._local_overlap_args is not None:
        from t5x_b200 import adafactor
        from t5x_b200.parallel import zero
        ts, opt_def = self._local_overlap_args
        slots = tree_utils.flatten_dict(ts.param_states, is_leaf=adafactor._is_state_leaf)
        zero.enable_local_overlap(tree_utils.flatten_dict(ts.params), self._model.module,
                                  opt_def, lambda name: slots[name])

  def _maybe_shard_optimizer(self, train_state, weight_metrics_computer) -> None:
    """Shards the optimizer over the data axis (see `t5x_b200.parallel.zero`) when there is
    more than one replica on GPUs (weight metrics are then gathered from the owners). A partitioner whose rules put a parameter axis on 'data', or
    `T5X_B200_ZERO_SHARD_WEIGHTS=1`, shards the bf16 working weights of the transformer layers
    too: each layer's weights are gathered from their owners just before the layer runs. Covered optimizers: Adafactor (with or without global-norm clipping) and
    the optax-style Adam / AdamW chains that the fused kernel handles
    (`OptaxWrapper.fused_plan`). The per-layer overlap with the backward pass is attached for
    Adafactor without clipping only: a clip factor needs every gradient first.
    `T5X_B200_OPTIMIZER_SHARDING=0` keeps the plain all-reduce."""
    from t5x_b200 import adafactor, optimizers
    from t5x_b200.parallel import zero
    zero.disable_local_overlap()  # a previous trainer's registration does not apply to this one
    st = pstate.get()
    opt_def = getattr(getattr(train_state, "_optimizer", None), "optimizer_def", None)
    is_adafactor = isinstance(opt_def, adafactor.Adafactor)
    is_fused_adam = isinstance(opt_def, optimizers.OptaxWrapper) and \
        opt_def.fused_plan is not None
    if self._device.type != "cuda" or not (is_adafactor or is_fused_adam):
      return
    # weight metrics compare the weights before and after the update: the updates then all run
    # after the backward pass (no overlap), and each rank reports the parameters it owns
    can_overlap = is_adafactor and not opt_def.hyper_params.global_norm_clip_threshold and \
        getattr(self._model, "module", None) is not None and weight_metrics_computer is None and \
        os.environ.get("T5X_B200_OVERLAP_GRAD_EXCHANGE", "1") != "0"
    if st.world_size == 1:
      if can_overlap:
        # one replica: nothing to exchange, but each layer's update can still run under the
        # backward pass of the layers below it (registered after the buffers are attached)
        self._local_overlap_args = (train_state, opt_def)
      return
    # A partitioner whose rules shard parameters over 'data' (parameter_partitioning_dims=2) asks
    # for this layout by itself; otherwise it is the default, which the environment can turn off.
    asked = bool(getattr(self._partitioner, "partitions_parameters_over_data", False))
    if st.data_size <= 1 or st.expert_size > 1:
      return
    if not asked and os.environ.get("T5X_B200_OPTIMIZER_SHARDING", "1") == "0":
      return
    # bf16 working weights sharded as well (the reference's parameter_partitioning_dims=2 shards
    # the parameters themselves): when the partitioner's rules ask for it or the environment
    # does; not combined with a model axis, whose fused kernels lay the weights out themselves
    shard_weights = (asked or os.environ.get("T5X_B200_ZERO_SHARD_WEIGHTS", "0") == "1") and \
        st.model_size == 1 and getattr(self._model, "module", None) is not None
    ctx = zero.enable(tree_utils.flatten_dict(train_state.params), st.data_group,
                      module=getattr(self._model, "module", None), shard_weights=shard_weights)
    if ctx is not None and can_overlap:
      slots = tree_utils.flatten_dict(train_state.param_states, is_leaf=adafactor._is_state_leaf)
      ctx.attach_overlap(self._model.module, opt_def, lambda name: slots[name])

  def _train_step(self, train_state, batch, step_num):
    step = int(step_num)
    lr = float(self._learning_rate_fn(step))
    return train_with_lr(train_state, batch, learning_rate=lr,
                         dropout_rng=self._get_step_rng(step), model=self._model,
                         num_microbatches=self._num_microbatches,
                         weight_metrics_computer=self._weight_metrics_computer)

  def _eval_step(self, train_state, batch):
    return eval_step(self._model, train_state, batch)


# ----------------------------------------------------------------------------
# Actions
# ----------------------------------------------------------------------------
class ActionMode(enum.Enum):
  TRAIN = 1
  TRAIN_EVAL = 2
  INFER_EVAL = 3


class BaseAction(abc.ABC):
  """Runs after a train / eval / infer-eval loop; returns True to stop training."""

  @abc.abstractmethod
  def run(self, train_state, metrics_by_task: Mapping[str, Mapping[str, Any]]) -> bool:
    raise NotImplementedError("Action must define its run method.")


ActionMapType = Mapping[ActionMode, Sequence[BaseAction]]


def _monitored_value(metrics_by_task, task: str, metric: str) -> Optional[float]:
  """The float behind metrics_by_task[task][metric], or None (with a warning naming what is
  missing) when the task, the metric or a scalar value is not there."""
  per_task = metrics_by_task.get(task)
  if per_task is None:
    logging.warning("action: no metrics for task %r (tasks present: %s)", task,
                    sorted(metrics_by_task))
    return None
  if metric not in per_task:
    logging.warning("action: task %r reports no metric %r", task, metric)
    return None
  m = per_task[metric]
  if isinstance(m, metric_writers.Scalar):
    return metric_writers.to_float(m)
  if isinstance(m, (float, int)):
    return float(m)
  logging.warning("action: metric %r of task %r is a %s, not a scalar", metric, task,
                  type(m).__name__)
  return None


class EarlyStoppingAction(BaseAction):
  """Asks to stop once the monitored metric has gone `patience` evaluations without getting
  better (the behaviour of t5x/trainer.py:1100-1228).

  A sliding window holds the last `patience` values. "Better" means lower for mode 'min' and
  higher for 'max', by more than `atol + rtol * |previous|`. Training stops when no value in
  the full window improved on the one before it."""

  def __init__(self, metric: Tuple[str, str], mode: str, patience: int = 3, atol: float = 0.0,
               rtol: float = 0.0):
    if mode not in ("min", "max"):
      raise ValueError(f"mode must be 'min' or 'max', got {mode!r}")
    if atol < 0 or rtol < 0:
      raise ValueError("atol and rtol must be >= 0")
    self._task, self._metric = metric
    self._sign = 1.0 if mode == "min" else -1.0  # compare sign * value, always minimising
    self._atol, self._rtol = atol, rtol
    self._patience = patience
    import collections
    self._window = collections.deque(maxlen=patience)

  def _stalled(self, now: float, before: float) -> bool:
    tolerance = self._atol + self._rtol * abs(before)
    return self._sign * now >= self._sign * before - tolerance

  def run(self, train_state, metrics_by_task) -> bool:
    value = _monitored_value(metrics_by_task, self._task, self._metric)
    if value is None:
      return False
    self._window.append(value)
    if len(self._window) < self._patience:
      return False
    values = list(self._window)
    if all(self._stalled(b, a) for a, b in zip(values, values[1:])):
      logging.warning("early stopping: %s of task %s did not improve over the last %d "
                      "evaluations (%s)", self._metric, self._task, self._patience, values)
      return True
    return False


class TerminateOnNanAction(BaseAction):
  """Asks to stop when the monitored metric is not finite (t5x/trainer.py:1231-1285)."""

  def __init__(self, task: str, metric: str = "loss"):
    self._task, self._metric = task, metric

  def run(self, train_state, metrics_by_task) -> bool:
    value = _monitored_value(metrics_by_task, self._task, self._metric)
    if value is None or np.isfinite(value):
      return False
    logging.warning("terminate on NaN: %s of task %s is %s", self._metric, self._task, value)
    return True
