"""`bench.py --mode decode`: T5.1.1-XL beam-search decode throughput.

Workload: random-init XL (d_model 2048, 24+24 layers, 32 heads, d_ff 5120), batch 64 examples
of 512 uniform random encoder tokens, beam 4, 128 decode steps with a key/value cache, length
penalty alpha 0.6. With N GPUs the batch is split over ranks (the 3B bf16 weights fit on every
GPU, so replicas need no communication); the whole-job value is batch * 128 tokens per decode
divided by the slowest rank's time.

One timed "step" is one full decode of the batch (encoder pass + 128 decoder steps + beam
bookkeeping) through `EncoderDecoderModel.predict_batch_with_aux`.
"""
from __future__ import annotations

import json
import os

BATCH, ENC_LEN, DEC_LEN, BEAMS, ALPHA = 64, 512, 128, 4, 0.6


def run(args, ClockSampler) -> None:
  """`bench.py --mode decode`: prints the decode measurement as the JSON line."""
  import torch.distributed as dist
  out = measure(args.gpus, args.steps, args.warmup, ClockSampler)
  if int(os.environ.get("RANK", "0")) == 0:
    print(json.dumps(out))
  if dist.is_initialized():
    dist.barrier()
    dist.destroy_process_group()


def measure(gpus: int, steps: int, warmup: int, ClockSampler, model_parallel: int = 0) -> dict:
  """Builds the XL model, times `steps` decodes of the batch (device-timed and end to end) and
  returns the result record (the same on every rank)."""
  import torch
  import torch.distributed as dist

  from t5x_b200 import adafactor, models, trainer as trainer_lib
  from t5x_b200.data import vocabularies
  from t5x_b200.models import base
  from t5x_b200.models.t5 import network
  from t5x_b200.ops import native
  from t5x_b200.parallel import state as pstate

  os.environ.setdefault("NCCL_NVLS_ENABLE", "0")  # NCCL only synchronises ranks here
  world = int(os.environ.get("WORLD_SIZE", "1"))
  if world != gpus:
    raise SystemExit(f"--gpus {gpus} but WORLD_SIZE={world}")
  local_rank = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local_rank)
  pstate.init_distributed("nccl")
  # Default mesh: the batch split over all GPUs with replicated weights (the XL weights fit one
  # GPU many times over, and a decode step of a few dozen rows is bound by latency, which the
  # all-reduce sites of a model axis add to). `model_parallel` (or
  # T5X_B200_DECODE_MODEL_PARALLEL) puts that many GPUs on a model axis instead: weights, heads
  # and vocabulary sharded, all-reduce sites inside the captured step; the named decode
  # configuration is data2 x model4.
  tp = int(model_parallel or os.environ.get("T5X_B200_DECODE_MODEL_PARALLEL", 1))
  if world % tp:
    raise SystemExit(f"{world} ranks are not divisible by model axis {tp}")
  st = pstate.setup_mesh(model_size=tp)
  dev, rank = st.device, st.rank
  if BATCH % st.data_size:
    raise SystemExit(f"batch {BATCH} not divisible by {st.data_size} data ranks")
  per_rank = BATCH // st.data_size

  cfg = network.T5Config(vocab_size=32128, dtype="bfloat16", emb_dim=2048, num_heads=32,
                         num_encoder_layers=24, num_decoder_layers=24, head_dim=64, mlp_dim=5120,
                         mlp_activations=("gelu", "linear"), dropout_rate=0.0,
                         logits_via_embedding=False)
  torch.manual_seed(1234)
  module = network.Transformer(cfg, device=dev)
  vocab = vocabularies.PassThroughVocabulary(32128)
  model = models.EncoderDecoderModel(module, vocab, vocab, adafactor.Adafactor())
  trainer_lib.attach_compute_buffers(base.module_param_tree(module), bf16_copy=True,
                                     main_grad=False)
  n_params = sum(int(torch.Size(getattr(p, "global_shape", p.shape)).numel())
                 for p in module.parameters())
  # the graph decoder checks the (device-side) termination flag every `period` steps; a period
  # longer than the decode length makes every decode run all 128 steps
  os.environ["T5X_B200_DECODE_CHECK_PERIOD"] = str(DEC_LEN + 1)

  g = torch.Generator().manual_seed(100 + st.data_rank)  # model ranks share their batch
  host_inputs = [torch.randint(3, 32000, (per_rank, ENC_LEN), generator=g).pin_memory()
                 for _ in range(4)]
  dec_in = torch.zeros(per_rank, DEC_LEN, dtype=torch.long, device=dev)
  params = {"alpha": ALPHA}

  def decode(enc_dev):
    return model.predict_batch_with_aux(None, {"encoder_input_tokens": enc_dev,
                                               "decoder_input_tokens": dec_in},
                                        num_decodes=BEAMS, decoder_params=dict(params))

  def sync_all():
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize()

  resident = [h.to(dev) for h in host_inputs]
  for i in range(warmup):
    decode(resident[i % 4])
  native.check_status()
  sync_all()
  sampler = ClockSampler(local_rank)
  sampler.start()
  launches0 = native.launch_count()
  gd0 = next(iter(model.__dict__.get("_graph_decoders", {}).values()), None)
  replays0 = gd0.replays if gd0 is not None else 0
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  for i in range(steps):
    out, aux = decode(resident[i % 4])
  e1.record()
  sync_all()
  ms = e0.elapsed_time(e1)
  gd = next(iter(model.__dict__.get("_graph_decoders", {}).values()), None)
  graph_replays = (gd.replays - replays0) if gd is not None else 0
  # kernels launched directly plus those replayed from the captured decode step
  launches = (native.launch_count() - launches0 +
              graph_replays * (gd.kernels_per_step if gd is not None else 0))
  clocks = sampler.stop()
  native.check_status()
  t = torch.tensor([ms], dtype=torch.float64, device=dev)
  if world > 1:
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
  ms_per_decode = float(t[0]) / steps
  tokens = BATCH * DEC_LEN
  value = tokens / (ms_per_decode / 1e3)

  # end to end: encoder tokens from pinned host memory, decoded tokens and scores read back
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  sync_all()
  e0.record()
  d2h = 0
  for i in range(steps):
    enc_dev = host_inputs[i % 4].to(dev, non_blocking=True)
    out, aux = decode(enc_dev)
    out_h, sc_h = out.cpu(), aux["scores"].cpu()
    d2h = out_h.numel() * out_h.element_size() + sc_h.numel() * sc_h.element_size()
  e1.record()
  sync_all()
  t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
  if world > 1:
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
  e_ms = float(t[0]) / steps
  h2d = host_inputs[0].numel() * host_inputs[0].element_size()
  peak_gb = torch.cuda.max_memory_allocated() / 2 ** 30
  del model, module
  return {
      "metric": "T5.1.1-XL beam-decode tokens/s", "value": value, "unit": "tokens/s",
      "n_gpus": world, "steps": steps, "warmup": warmup,
      "ms_per_step": ms_per_decode, "higher_is_better": True, "scaling": "strong",
      "vs_baseline": None, "dtype": "bf16",
      "data": "uniform random encoder tokens, random-init weights", "impl": "ours",
      "config": {"model": "t5.1.1-xl", "params": n_params, "global_batch": BATCH,
                 "seq_len": ENC_LEN, "decode_steps": DEC_LEN, "beam": BEAMS, "alpha": ALPHA,
                 "parallelism": f"data{st.data_size} x model{tp}" +
                                (" (replicated weights, batch split)" if tp == 1 else
                                 " (weights sharded over the model axis, batch split over data)"),
                 "step": "one timed step = one full decode of the batch (encoder pass, 128 "
                         "decoder steps with KV cache, beam bookkeeping); tokens = batch x 128",
                 "l2": "no explicit flush: each decoder step streams 3.3 GB of decoder "
                       "weights plus the key/value caches, far larger than the 126 MB L2"},
      "clocks": clocks,
      "e2e": {"value": tokens / (e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e_ms,
              "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
      "gpu_launches": launches, "graph_replays_in_timed_region": graph_replays,
      "peak_memory_gb": peak_gb,
  }
