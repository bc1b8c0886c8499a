"""Headline benchmark: T5.1.1-XXL training tokens/s (synthetic span corruption, bf16, Adafactor),
with the XL beam-decode tokens/s as a second record in the same JSON line.

  python bench.py --gpus N --steps K --warmup W            (N=1)
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
      --master-port P bench.py --gpus N --steps K --warmup W

One process per GPU, global batch 128, inputs 512 / targets 114. Rank 0 prints one JSON line:

  value / e2e    the train step on the default layout: data parallel over the N GPUs with the
                 optimizer sharded over the replicas (mesh data=N x model=1). `value` is
                 device-timed (CUDA events, max over ranks) over K steps with device-resident
                 batches; `e2e` repeats it through the public Trainer API with a pinned-host ->
                 device copy of every batch and a device -> host read of the step's metrics
                 inside the timed region.
  named_mesh     (N > 1) the same step on the mesh the named configuration prescribes,
                 data=1 x model=N: tensor parallel over heads / mlp / vocab with the all-gather
                 and reduce-scatter inside the GEMM kernels (3 warm-up + 5..8 timed steps).
  selfcheck      (N > 1) errors of the fused multi-GPU kernels against library collectives,
                 measured on this box right before the timed regions; the run fails if one
                 exceeds its tolerance.
  decode         T5.1.1-XL beam search (beam 4, batch 64, 512 encoder tokens, 128 steps).

`--impl reference` reports why the reference cannot run here; `--impl library` runs the same
train step as plain PyTorch (cuBLAS matmuls, library attention, NCCL all-reduce, none of this
repository's kernels): the same-box comparator.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

MODEL_SIZES = {
    # name: (emb_dim, num_heads, layers, head_dim, mlp_dim)
    "small": (512, 6, 8, 64, 1024),
    "base": (768, 12, 12, 64, 2048),
    "large": (1024, 16, 24, 64, 2816),
    "xl": (2048, 32, 24, 64, 5120),
    "xxl": (4096, 64, 24, 64, 10240),
}
# Derived from the reference's published A100 table: 1346 seq/s * 640 tokens / 512 GPUs.
BASELINE_TOKENS_PER_S_PER_GPU = 1346.0 * 640.0 / 512.0


def reference_arm(args) -> None:
  """The reference is JAX/Flax code; none of jax, jaxlib, flax, seqio, tensorflow is installed
  and there is no index to install them from, so its own code path cannot execute here."""
  why = ("reference installed with --no-deps under baseline/_ref but `import t5x` fails: "
         "jax/jaxlib/flax/seqio/tensorflow are not installed and cannot be (no network)")
  try:
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref"))
    import importlib
    importlib.import_module("jax")
    importlib.import_module("flax")
    why = "jax and flax import, but the reference arm is not wired: " + why
  except Exception as e:  # the expected outcome
    why = f"{why} ({type(e).__name__}: {e})"
  finally:
    sys.path.pop(0)
  if int(os.environ.get("RANK", "0")) == 0:
    print(json.dumps({"impl": "reference", "unavailable": why}))


class ClockSampler:
  """Samples nvidia-smi clocks / throttle reasons of this rank's GPU during the timed region."""

  FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
            "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
            "clocks_event_reasons.sw_power_cap")

  def __init__(self, gpu_index: int):
    self.gpu_index = gpu_index
    self.proc = None
    self.lines = []
    self.thread = None

  def start(self):
    try:
      self.proc = subprocess.Popen(
          ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}",
           "--format=csv,noheader,nounits", "-lms", "200"],
          stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
    except OSError:
      self.proc = None
      return
    def pump():
      for line in self.proc.stdout:
        self.lines.append(line.strip())
    self.thread = threading.Thread(target=pump, daemon=True)
    self.thread.start()

  def stop(self) -> dict:
    if self.proc is None:
      return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
    time.sleep(0.25)
    self.proc.terminate()  # the exact child this object started
    try:
      self.proc.wait(timeout=5)
    except subprocess.TimeoutExpired:
      self.proc.kill()
    sm, mx, reasons = [], [], set()
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    for line in self.lines:
      parts = [p.strip() for p in line.split(",")]
      if len(parts) < 7:
        continue
      try:
        sm.append(float(parts[0]))
        mx.append(float(parts[1]))
      except ValueError:
        continue
      for n, v in zip(names, parts[3:7]):
        if v.lower().startswith("active"):
          reasons.add(n)
    return {"sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
            "samples": len(sm)}


def default_microbatches(model: str, n_gpus: int) -> int:
  if model == "xxl":
    # 32 sequences per microbatch (7 % faster than 16 at one GPU, where it peaks at 170 GB;
    # `measure_train_or_halve` falls back to 16 if the allocator cannot fit it)
    return {1: 4, 2: 2}.get(n_gpus, 1)
  return 1


def _sync_all(world: int) -> None:
  import torch
  import torch.distributed as dist
  if world > 1:
    dist.barrier()
  torch.cuda.synchronize()


def _max_over_ranks(ms: float, world: int, dev) -> float:
  import torch
  import torch.distributed as dist
  t = torch.tensor([ms], dtype=torch.float64, device=dev)
  if world > 1:
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
  return float(t[0])


def measure_train_or_halve(args, parallelism: str, steps: int, warmup: int, e2e: bool) -> dict:
  """`measure_train`, repeated with microbatches of half the size if the default ones ran out
  of device memory (an explicit --microbatches is taken as given)."""
  import torch
  try:
    return measure_train(args, parallelism, steps, warmup, e2e)
  except torch.cuda.OutOfMemoryError:
    if args.microbatches:
      raise
    world = int(os.environ.get("WORLD_SIZE", "1"))
    first = (4 if args.model == "xxl" else 1) if parallelism == "tp" else \
        default_microbatches(args.model, world)
  _teardown()
  args.microbatches = 2 * first
  try:
    return measure_train(args, parallelism, steps, warmup, e2e)
  finally:
    args.microbatches = 0


def _teardown() -> None:
  """Drops everything a finished phase left on the device before the next phase builds its
  own model on another mesh."""
  import gc
  import torch
  from t5x_b200.parallel import tp_fused, zero
  zero.disable()
  tp_fused._ARENA = None
  gc.collect()
  torch.cuda.empty_cache()
  torch.cuda.reset_peak_memory_stats()


def measure_train(args, parallelism: str, steps: int, warmup: int, with_e2e: bool) -> dict:
  """Builds the model on the mesh of `parallelism` ("dp": data=N; "tp": model=N), runs
  `warmup` + `steps` train steps and returns the record of the timed ones."""
  import numpy as np
  import torch

  from t5x_b200 import adafactor, data, models, train_state as ts_lib, trainer as trainer_lib
  from t5x_b200.data import feature_converters as fc, vocabularies
  from t5x_b200.data.dataset import PrefetchIterator, ShardInfo
  from t5x_b200.models.t5 import network
  from t5x_b200.ops import native
  from t5x_b200.parallel import state as pstate
  from t5x_b200.utils import schedules

  world = int(os.environ.get("WORLD_SIZE", "1"))
  local_rank = int(os.environ.get("LOCAL_RANK", "0"))
  moe = args.model == "switch-base"
  if moe and (parallelism == "tp" or 8 % world):
    raise SystemExit("switch-base runs expert-parallel on 1, 2, 4 or 8 GPUs")
  st = pstate.setup_mesh(model_size=world if parallelism == "tp" else 1,
                         expert_size=world if moe else 1)
  data_shards = 1 if parallelism == "tp" else world
  if args.batch % data_shards:
    raise SystemExit(f"--batch {args.batch} is not divisible by {data_shards} data shards")
  dev, rank = st.device, st.rank

  emb, heads, layers, head_dim, mlp = MODEL_SIZES["base" if moe else args.model]
  common = dict(vocab_size=32128, dtype="bfloat16", emb_dim=emb, num_heads=heads,
                num_encoder_layers=layers, num_decoder_layers=layers, head_dim=head_dim,
                mlp_dim=mlp, mlp_activations=("gelu", "linear"), dropout_rate=0.0,
                logits_via_embedding=False)
  torch.manual_seed(1234)
  vocab = vocabularies.PassThroughVocabulary(32128)
  if moe:
    from t5x_b200.contrib.moe import adafactor_utils, models as moe_models, network as moe_network
    cfg = moe_network.MoeT5Config(num_experts=8, num_selected_experts=1,
                                  train_capacity_factor=1.25, sparse_layout="every_other",
                                  **common)
    module = moe_network.Transformer(cfg, device=dev)
    opt = adafactor.Adafactor(decay_rate=0.8, step_offset=0,
                              logical_factor_rules=adafactor_utils.logical_factor_rules())
    model = moe_models.MoeEncoderDecoderModel(module, vocab, vocab, opt, z_loss=1e-4,
                                              loss_normalizing_factor=None, aux_loss_factor=1e-2,
                                              router_z_loss_factor=1e-3)
  else:
    cfg = network.T5Config(**common)
    module = network.Transformer(cfg, device=dev)
    opt = adafactor.Adafactor(decay_rate=0.8, step_offset=0,
                              logical_factor_rules=adafactor.standard_logical_factor_rules())
    model = models.EncoderDecoderModel(module, vocab, vocab, opt, z_loss=1e-4,
                                       loss_normalizing_factor=None)
  state = ts_lib.FlaxOptimTrainState.create(opt, model.get_initial_variables(None, None))
  # tensor-parallel ranks all work on the same microbatch: 32 sequences at a time for XXL
  n_micro = args.microbatches or ((4 if args.model == "xxl" else 1) if parallelism == "tp"
                                  else default_microbatches(args.model, world))
  lr_fn = schedules.create_learning_rate_scheduler("constant * rsqrt_decay", 1.0, 10000)
  if moe:
    from t5x_b200.contrib.moe import trainer as moe_trainer
    trainer = moe_trainer.MoeTrainer(model, state, None, [], None, None, 0, lr_fn, n_micro,
                                     num_expert_partitions=world)
  else:
    trainer = trainer_lib.Trainer(model, state, None, [], None, None, 0, lr_fn, n_micro)
  n_params = sum(int(np.prod(getattr(p, "global_shape", p.shape))) for p in module.parameters())
  from t5x_b200.parallel import zero as zero_lib
  zctx = zero_lib.active()
  exchange = None
  if zctx is not None:
    exchange = ("NVSwitch multimem (in-switch gradient sum, multicast weight push)"
                if zctx.nvls else "peer loads / stores over NVLink")

  # Tensor-parallel ranks all consume the global batch; data-parallel ranks each take a shard.
  lengths = {"inputs": args.inputs_length, "targets": args.targets_length}
  ds = data.get_dataset("synthetic_span_corruption", lengths, fc.EncDecFeatureConverter(pack=False),
                        seed=0, batch_size=args.batch // data_shards, num_epochs=None,
                        shard_info=ShardInfo(st.rank % data_shards, data_shards))

  def pin(batch):
    return {k: torch.from_numpy(np.ascontiguousarray(v).astype(np.int64)).pin_memory()
            for k, v in batch.items()}

  host_iter = PrefetchIterator(iter(ds), depth=4, transform=pin)
  tokens_per_step = args.batch * (args.inputs_length + args.targets_length)

  # ---- device-timed region: batches already resident on the device -----------------------
  resident = []
  for _ in range(min(4, max(1, warmup + steps))):
    hb = next(host_iter)
    resident.append({k: v.to(dev, non_blocking=True) for k, v in hb.items()})
  torch.cuda.synchronize()

  def resident_iter():
    i = 0
    while True:
      yield resident[i % len(resident)]
      i += 1

  rit = resident_iter()
  step_no = 0
  for _ in range(warmup):
    trainer.train(rit, 1, start_step=step_no)
    step_no += 1
  native.check_status()
  _sync_all(world)
  sampler = ClockSampler(local_rank)
  sampler.start()
  launches0 = native.launch_count()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  futures = []
  for _ in range(steps):
    futures.append(trainer.train(rit, 1, start_step=step_no))
    step_no += 1
  e1.record()
  _sync_all(world)
  ms = e0.elapsed_time(e1)
  launches = native.launch_count() - launches0
  clocks = sampler.stop()
  native.check_status()
  last_loss = float(futures[-1].result()["loss"].value)
  ms_per_step = _max_over_ranks(ms, world, dev) / steps
  value = tokens_per_step / (ms_per_step / 1e3)

  # ---- end-to-end through the public API: H2D of inputs and D2H of metrics every step ----
  e2e = None
  if with_e2e:
    def e2e_iter():
      while True:
        yield next(host_iter)
    eit = e2e_iter()
    d2h_bytes = 0
    trainer.train(eit, 1, start_step=step_no).result()
    step_no += 1
    _sync_all(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
      s = trainer.train(eit, 1, start_step=step_no).result()   # waits for and reads the metrics
      step_no += 1
      d2h_bytes = 4 * len(s)
    e1.record()
    _sync_all(world)
    e_ms = _max_over_ranks(e0.elapsed_time(e1), world, dev) / steps
    h2d_bytes = sum(v.numel() * v.element_size() for v in resident[0].values())
    e2e = {"value": tokens_per_step / (e_ms / 1e3), "unit": "tokens/s",
           "ms_per_step": e_ms, "h2d_bytes_per_step": h2d_bytes,
           "d2h_bytes_per_step": d2h_bytes}
  trainer.close()
  peak_gb = torch.cuda.max_memory_allocated() / 2 ** 30
  # memory held on the device at the end of the run, symmetric (peer-mapped) buffers included,
  # which the caching allocator's statistics do not see
  free_b, total_b = torch.cuda.mem_get_info()
  device_used_gb = (total_b - free_b) / 2 ** 30
  weights_sharded = os.environ.get("T5X_B200_ZERO_SHARD_WEIGHTS", "0") == "1" and world > 1 and \
      parallelism != "tp" and not moe
  host_iter.close() if hasattr(host_iter, "close") else None
  del trainer, state, model, module, resident, futures
  _teardown()

  if moe:
    layout = f"expert{world} (tokens data-parallel over the same ranks)"
  elif parallelism == "tp":
    layout = f"data1 x model{world}" + (
        " (all-gather / reduce-scatter inside the GEMM kernels, row-sharded residual stream)"
        if world > 1 else "")
  else:
    layout = f"data{world} x model1" + (", optimizer sharded over data" if world > 1 else "") + (
        ", bf16 layer weights sharded over data" if weights_sharded else "")
  return {
      "metric": ("Switch-Base-8 train tokens/s" if moe else
                 f"T5.1.1-{args.model.upper()} train tokens/s"),
      "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps,
      "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
      "scaling": "strong",
      # the published figure is for XXL; other models have none
      "vs_baseline": (value / (BASELINE_TOKENS_PER_S_PER_GPU * world)
                      if args.model == "xxl" else None),
      "dtype": "bf16", "data": "synthetic span-corruption tokens, random-init weights",
      "impl": "ours",
      "config": {"model": "switch-base-8" if moe else f"t5.1.1-{args.model}", "params": n_params,
                 "global_batch": args.batch, "seq_len": args.inputs_length + args.targets_length,
                 "inputs_length": args.inputs_length, "targets_length": args.targets_length,
                 "parallelism": layout, "optimizer": "adafactor", "num_microbatches": n_micro,
                 "gradient_exchange": exchange,
                 "l2": "no explicit flush: every step streams the full weights, gradients and "
                       "activations (tens of GB), far larger than the 126 MB L2",
                 "baseline_note": "vs_baseline divides by the reference's published A100 figure "
                                  "scaled per GPU (1346 seq/s * 640 tok / 512 GPUs = 1682.5 tok/s/GPU)"},
      "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "final_loss": last_loss,
      "peak_memory_gb": peak_gb, "device_memory_used_gb": device_used_gb,
  }


class Watchdog:
  """Calls `on_deadline` from a daemon thread unless `finish()` comes within `seconds`."""

  def __init__(self, seconds: float, on_deadline):
    self._seconds, self._on_deadline = seconds, on_deadline
    self._done = threading.Event()

  def start(self) -> None:
    def run():
      if not self._done.wait(self._seconds):
        self._on_deadline()
    threading.Thread(target=run, daemon=True).start()

  def finish(self) -> None:
    self._done.set()


def run_selfcheck(world: int) -> dict:
  """Errors of the fused multi-GPU kernels against library collectives on this box; each
  family is checked on the mesh it serves. A family that exceeds the tolerance (or raises) is
  reported under "failed" next to the errors that were measured: the record says so, and the
  timed phases still run, so that one bad check does not leave a run without numbers."""
  from t5x_b200.parallel import selfcheck, state as pstate
  out, failed = {}, {}
  for name, mesh in (("dp", dict(model_size=1)), ("tp", dict(model_size=world)),
                     ("moe", dict(model_size=1, expert_size=world))):
    try:
      pstate.setup_mesh(**mesh)
      out.update(selfcheck.run([name]))
    except selfcheck.SelfCheckError as e:
      out.update(e.errors)
      failed[name] = str(e)
    except Exception as e:  # pylint: disable=broad-except
      failed[name] = f"{type(e).__name__}: {e}"
    _teardown()
  out["tolerance"] = 2e-2
  if failed:
    out["failed"] = failed
  return out


def main() -> None:
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=3)
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--impl", default="ours", choices=["ours", "reference", "library"])
  ap.add_argument("--model", default="xxl", choices=sorted(MODEL_SIZES) + ["switch-base"],
                  help="a T5.1.1 size, or switch-base: T5.1.1-Base with every other FFN replaced "
                       "by 8 top-1 experts, expert-parallel over all ranks")
  ap.add_argument("--batch", type=int, default=128)
  ap.add_argument("--inputs-length", type=int, default=512)
  ap.add_argument("--targets-length", type=int, default=114)
  ap.add_argument("--microbatches", type=int, default=0)
  ap.add_argument("--skip-e2e", action="store_true")
  ap.add_argument("--skip-extras", action="store_true",
                  help="only the headline train measurement: no self-check, named-mesh or decode "
                       "records")
  ap.add_argument("--mode", default="train", choices=["train", "decode"],
                  help="train: T5.1.1-XXL train step (default); decode: T5.1.1-XL beam decode")
  ap.add_argument("--parallelism", default="dp", choices=["dp", "tp"],
                  help="dp: data parallel with the optimizer sharded over replicas (gradient "
                       "reduction and weight broadcast fused into the Adafactor kernels over "
                       "NVLink peer memory); tp: tensor parallel over all GPUs")
  args = ap.parse_args()

  if args.impl == "reference":
    reference_arm(args)
    return
  if args.impl == "library":
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline"))
    import library_t5
    library_t5.run(args, ClockSampler, MODEL_SIZES, default_microbatches,
                   BASELINE_TOKENS_PER_S_PER_GPU)
    return
  if args.mode == "decode":
    import bench_decode
    bench_decode.run(args, ClockSampler)
    return

  import torch
  import torch.distributed as dist

  from t5x_b200.parallel import state as pstate

  # NCCL only carries barriers, the metrics all-reduce and (tensor-parallel runs) two gathers
  # per step here; the in-switch reduction buys nothing for those, and with it off a rank that
  # dies cannot raise NVLink faults on its peers' GPUs. An explicit setting wins.
  os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
  world = int(os.environ.get("WORLD_SIZE", "1"))
  if world != args.gpus:
    raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun "
                     f"--nproc-per-node {args.gpus}")
  torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
  pstate.init_distributed("nccl")
  rank = int(os.environ.get("RANK", "0"))
  extras = not args.skip_extras and args.model == "xxl"

  selfcheck = None
  if extras and world > 1:
    selfcheck = run_selfcheck(world)
  out = measure_train_or_halve(args, args.parallelism, args.steps, args.warmup, not args.skip_e2e)
  if selfcheck is not None:
    out["selfcheck"] = selfcheck
  # The records beyond the headline one. A phase that raises is reported under its key and ends
  # the extras on every rank (the ranks agree through the host control group), so that the
  # headline measurement above is printed whatever happens to them.
  keys = ("metric", "value", "unit", "ms_per_step", "steps", "warmup", "e2e", "clocks",
          "gpu_launches", "config", "peak_memory_gb")
  dec_steps = min(max(args.steps, 3), 5)

  def named_mesh_train():
    nm = measure_train_or_halve(args, "tp", min(max(args.steps, 5), 8), 3, not args.skip_e2e)
    rec = {k: nm[k] for k in ("value", "unit", "ms_per_step", "steps", "warmup", "e2e", "clocks",
                              "gpu_launches", "final_loss", "peak_memory_gb")}
    rec["parallelism"] = nm["config"]["parallelism"]
    rec["num_microbatches"] = nm["config"]["num_microbatches"]
    return rec

  def decode(model_parallel):
    import bench_decode
    dec = bench_decode.measure(world, dec_steps, 3, ClockSampler, model_parallel=model_parallel)
    return {k: dec[k] for k in keys}

  phases = []
  if extras and world > 1 and args.parallelism == "dp":
    phases.append(("named_mesh", named_mesh_train))
  if extras:
    phases.append(("decode", lambda: decode(1)))
    # the named decode mesh (a model axis of up to four GPUs, the rest splits the batch)
    named = os.environ.get("T5X_B200_BENCH_DECODE_NAMED_MESH", "1" if world > 1 else "0")
    if world > 1 and named == "1":
      phases.append(("decode_named_mesh", lambda: decode(min(4, world))))
  # A phase that neither returns nor raises (ranks stuck in a rendezvous, say) must not cost the
  # headline record: past the deadline every rank's watchdog ends its own process, rank 0 after
  # printing what has been measured so far. The headline above is complete by now.
  deadline_s = float(os.environ.get("T5X_B200_BENCH_EXTRAS_DEADLINE_S", "420"))
  current = ["(none)"]

  def on_deadline():
    if rank == 0:
      out.setdefault(current[0], {"failed": f"no result within {deadline_s:.0f} s; run ended "
                                            "by the bench's watchdog"})
      print(json.dumps(out), flush=True)
    os._exit(0)

  watchdog = Watchdog(deadline_s, on_deadline)
  if phases:
    watchdog.start()
  for name, phase in phases:
    failure = None
    current[0] = name
    try:
      out[name] = phase()
    except Exception as e:  # pylint: disable=broad-except
      failure = f"{type(e).__name__}: {e}"[:500]
      out[name] = {"failed": failure}
    try:
      _teardown()
      stop = pstate.host_any(failure is not None)
    except Exception:  # pylint: disable=broad-except
      stop = True
    if stop:
      if failure is None:
        out[name + "_note"] = "a later phase was skipped: this phase failed on another rank"
      break
  watchdog.finish()
  if rank == 0:
    print(json.dumps(out), flush=True)
  if world > 1:
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
  main()
