"""Child process of the multi-GPU tests: one rank per GPU, launched by torchrun.

  torchrun --nproc-per-node N tests/multi_gpu_worker.py <case> <out_dir>

Each case writes `<out_dir>/rank<r>.json` with what the parent test asserts on.
"""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from t5x_b200.parallel import state as pstate  # noqa: E402


def _setup():
  local = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local)
  pstate.init_distributed("nccl", timeout_s=120)
  return pstate.setup_mesh(model_size=1)


def case_collectives(out):
  """peer_reduce / peer_push / barrier against torch.distributed results."""
  from t5x_b200.ops import comm, native
  st = _setup()
  n = 1_000_003
  buf = comm.SymmetricBuffer(n, torch.float32)
  g = torch.Generator(device="cuda").manual_seed(100 + st.rank)
  buf.tensor.copy_(torch.randn(n, device="cuda", generator=g))
  expect = buf.tensor.clone()
  dist.all_reduce(expect)
  buf.barrier(0)
  dst = torch.empty(n, device="cuda")
  comm.peer_reduce_f32_(dst, buf.ptrs_at(0), n)
  buf.barrier(1)
  err_reduce = float((dst - expect).abs().max())
  # push: rank r broadcasts its slice [r*k, (r+1)*k) of a bf16 buffer to everyone
  k = 4099
  wb = comm.SymmetricBuffer(k * st.world_size, torch.bfloat16)
  wb.tensor.zero_()
  src = torch.full((k,), float(st.rank + 1), device="cuda", dtype=torch.bfloat16)
  wb.barrier(0)
  comm.peer_push_bf16_(wb.ptrs_at(st.rank * k), src, k)
  wb.barrier(1)
  native.check_status()
  got = wb.tensor.float().view(st.world_size, k)
  ok_push = all(bool((got[r] == r + 1).all()) for r in range(st.world_size))
  json.dump({"err_reduce": err_reduce, "ok_push": ok_push}, out)


def _tiny_trainer(n_micro=2):
  from t5x_b200 import adafactor, models, train_state as ts_lib, trainer as trainer_lib
  from t5x_b200.data import vocabularies
  from t5x_b200.models.t5 import network
  from t5x_b200.utils import schedules
  st = pstate.get()
  cfg = network.T5Config(vocab_size=512, dtype="bfloat16", emb_dim=128, num_heads=2,
                         num_encoder_layers=2, num_decoder_layers=2, head_dim=64, mlp_dim=256,
                         mlp_activations=("gelu", "linear"), dropout_rate=0.0)
  torch.manual_seed(7)
  module = network.Transformer(cfg, device=st.device)
  vocab = vocabularies.PassThroughVocabulary(512)
  kind = os.environ.get("T5X_TEST_OPTIMIZER", "adafactor")
  if kind == "adamw_clip":
    from t5x_b200 import optimizers
    opt = optimizers.chain([optimizers.clip_by_global_norm(1.0),
                            optimizers._adamw(1e-3, weight_decay=0.01)])
  else:
    opt = adafactor.Adafactor(decay_rate=0.8, step_offset=0,
                              global_norm_clip_threshold=1.0 if kind == "adafactor_clip" else None,
                              logical_factor_rules=adafactor.standard_logical_factor_rules())
  model = models.EncoderDecoderModel(module, vocab, vocab, opt, z_loss=1e-4)
  state = ts_lib.FlaxOptimTrainState.create(opt, model.get_initial_variables(None, None))
  lr_fn = schedules.create_learning_rate_scheduler("constant",
                                                   1e-3 if kind == "adamw_clip" else 0.01, 0)
  wmc = trainer_lib.WeightMetricsComputer() if os.environ.get("T5X_TEST_WEIGHT_METRICS") else None
  return trainer_lib.Trainer(model, state, None, [], None, None, 0, lr_fn, n_micro,
                             weight_metrics_computer=wmc), module


def _batches(rank, world, steps, per_rank=8):
  g = torch.Generator().manual_seed(3)
  out = []
  for _ in range(steps):
    enc = torch.randint(1, 512, (per_rank * world, 128), generator=g)
    dec = torch.randint(1, 512, (per_rank * world, 128), generator=g)
    sl = slice(rank * per_rank, (rank + 1) * per_rank)
    dec_in = torch.cat([torch.zeros(per_rank * world, 1, dtype=torch.long), dec[:, :-1]], 1)
    out.append({"encoder_input_tokens": enc[sl], "decoder_input_tokens": dec_in[sl],
                "decoder_target_tokens": dec[sl],
                "decoder_loss_weights": torch.ones(per_rank, 128)})
  return out


def case_train(out):
  """Three train steps of a small model; the parent compares the sharded-optimizer run with
  the all-reduce run (T5X_B200_OPTIMIZER_SHARDING=0)."""
  from t5x_b200.ops import native
  from t5x_b200.parallel import zero
  st = _setup()
  trainer, module = _tiny_trainer()
  batches = _batches(st.rank, st.world_size, 3)
  summary = trainer.train(iter(batches), 3, start_step=0).result()
  trainer.sync_replicas()
  native.check_status()
  torch.cuda.synchronize()
  ctx = zero.active()
  weights_sharded = bool(getattr(ctx, "shard_weights", False))
  weight_elems = (int(getattr(ctx, "weights_total", 0)), int(getattr(ctx, "total", 0)))
  overlapped = len(getattr(ctx, "done_this_step", ()))
  if weights_sharded:
    zero.disable()  # every rank gets full bf16 copies back from the owners
  flat = torch.cat([p.detach().float().reshape(-1) for p in module.parameters()])
  bf = torch.cat([p.bf16.float().reshape(-1) for p in module.parameters()])
  from t5x_b200.utils import tree as tree_utils
  slots = [v.double().abs().sum() for v in
           tree_utils.flatten_dict(trainer.train_state.param_states).values()
           if isinstance(v, torch.Tensor) and v.is_cuda and v.numel() > 1]
  weight_metrics = {k: float(v.value) for k, v in summary.items()
                    if k in ("weight_norm", "weight_update_norm", "weight_gradient_norm") or
                    k.startswith(("weight_update_rms/encoder/layers_1/mlp/wo",
                                  "weight_max/decoder/layers_0/self_attention/query"))}
  json.dump({"loss": float(summary["loss"].value), "sharded": ctx is not None,
             "weight_metrics": weight_metrics,
             "slot_abs": float(torch.stack(slots).sum()),
             "nvls": bool(getattr(ctx, "nvls", False)),
             "overlapped": overlapped, "weights_sharded": weights_sharded,
             "weight_elems": weight_elems,
             "param_sum": float(flat.double().sum()), "param_abs": float(flat.double().abs().sum()),
             "bf16_abs": float(bf.double().abs().sum()),
             "first": flat[:8].tolist()}, out)
  trainer.close()


def case_moe(out):
  """Loss and gradients of an expert-parallel MoE model; the parent compares the NVLink-fused
  dispatch/combine with the all_to_all path (T5X_B200_MOE_FUSED=0)."""
  from t5x_b200 import adafactor, trainer as trainer_lib
  from t5x_b200.contrib.moe import adafactor_utils, models as moe_models, network as moe_network
  from t5x_b200.data import vocabularies
  from t5x_b200.models import base
  from t5x_b200.ops import native
  local = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local)
  pstate.init_distributed("nccl", timeout_s=120)
  st = pstate.setup_mesh(model_size=1, expert_size=int(os.environ["WORLD_SIZE"]))
  cfg = moe_network.MoeT5Config(vocab_size=512, dtype="bfloat16", emb_dim=128, num_heads=2,
                                head_dim=64, mlp_dim=256, num_encoder_layers=2,
                                num_decoder_layers=2, dropout_rate=0.0,
                                mlp_activations=("gelu", "linear"), num_experts=4,
                                num_selected_experts=2, train_capacity_factor=2.0)
  torch.manual_seed(11)
  module = moe_network.Transformer(cfg, device=st.device)
  vocab = vocabularies.PassThroughVocabulary(512)
  opt = adafactor.Adafactor(logical_factor_rules=adafactor_utils.logical_factor_rules())
  model = moe_models.MoeEncoderDecoderModel(module, vocab, vocab, opt, aux_loss_factor=0.01,
                                            router_z_loss_factor=0.001)
  trainer_lib.attach_compute_buffers(base.module_param_tree(module), bf16_copy=True,
                                     main_grad=True)
  batch = {k: v.to(st.device) for k, v in _batches(st.rank, st.world_size, 1)[0].items()}
  loss, _ = model.loss_fn(None, batch, None)
  loss.backward()
  native.check_status()
  torch.cuda.synchronize()
  wi = module.encoder.layers_1.mlp.expert.wi_0.kernel
  wo = module.decoder.layers_1.mlp.expert.wo.kernel
  router = module.encoder.layers_1.mlp.router.router_weights.w.kernel
  dense = module.encoder.layers_0.mlp.wi_0.kernel
  g = lambda p: (p.main_grad if getattr(p, "grad_ready", False) else p.grad).float()
  json.dump({"loss": float(loss), "wi": float(g(wi).abs().sum()), "wo": float(g(wo).abs().sum()),
             "router": float(g(router).abs().sum()), "dense": float(g(dense).abs().sum()),
             "wi_first": g(wi).reshape(-1)[:6].tolist()}, out)


def _setup_tp():
  local = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local)
  pstate.init_distributed("nccl", timeout_s=120)
  return pstate.setup_mesh(model_size=int(os.environ["WORLD_SIZE"]))


def case_tp_ops(out):
  """all-gather -> GEMM and GEMM -> reduce-scatter (forward and backward) against fp32
  PyTorch on the gathered operands."""
  from t5x_b200.ops import native
  from t5x_b200.parallel import tp_fused
  st = _setup_tp()
  T, r = st.model_size, st.model_rank
  res = {}
  for name, (m, k, n) in {"even": (512, 256, 384), "ragged": (228, 192, 320)}.items():
    g = torch.Generator(device="cuda").manual_seed(50)
    h_all = torch.randn(T * m, k, device="cuda", generator=g).to(torch.bfloat16)
    ws = [(torch.randn(k, n, device="cuda", generator=g) * 0.05) for _ in range(3)]
    wo = torch.randn(T * n, k, device="cuda", generator=g) * 0.05     # row-parallel [T*n, k]
    dy_all = torch.randn(T * m, k, device="cuda", generator=g).to(torch.bfloat16)
    res_sp = torch.randn(T * m, k, device="cuda", generator=g).to(torch.bfloat16)
    sl = slice(r * m, (r + 1) * m)
    # --- fused: y = RS( gated(AG(h) @ w0, @ w1) ... ) chain: q = AG(h)@w2 ; z = RS(q @ wo_r) + res
    h_sp = h_all[sl].clone().requires_grad_(True)
    wp = [torch.nn.Parameter(w.clone()) for w in ws]
    wo_r = torch.nn.Parameter(wo[r * n:(r + 1) * n].clone())
    q0, q1, q2 = tp_fused.all_gather_linears(h_sp, wp)
    gg = tp_fused.all_gather_gated_gelu(h_sp, wp[0], wp[1])
    mix = (q0 + q1 * 0.5 + q2 * 0.25 + gg).to(torch.bfloat16)
    z = tp_fused.linear_reduce_scatter(mix, wo_r, res_sp[sl])
    z.backward(dy_all[sl])
    native.check_status()
    for w in wp:  # the same weights on every rank here: total gradient = sum of the ranks'
      dist.all_reduce(w.grad)
    # --- reference (fp32, whole problem on every rank)
    hf = h_all.float().requires_grad_(True)
    wf = [w.to(torch.bfloat16).float().requires_grad_(True) for w in ws]
    wof = wo.to(torch.bfloat16).float().requires_grad_(True)
    gelu = lambda t: 0.5 * t * (1 + torch.tanh(0.7978845608028654 * (t + 0.044715 * t ** 3)))
    # every rank has the same column-parallel weights here, so the sum over ranks of the
    # row-parallel products is mix @ sum_r wo_r
    mixf = hf @ wf[0] + 0.5 * (hf @ wf[1]) + 0.25 * (hf @ wf[2]) + gelu(hf @ wf[0]) * (hf @ wf[1])
    zf = sum(mixf @ wof[i * n:(i + 1) * n] for i in range(T)) + res_sp.float()
    zf.backward(dy_all.float())
    scale = float(zf.abs().max())
    res[name] = {
        "z": float((z.float() - zf[sl]).abs().max()) / scale,
        "dh": float((h_sp.grad.float() - hf.grad[sl]).abs().max()) / float(hf.grad.abs().max()),
        "dw0": float((wp[0].grad.float() - wf[0].grad).abs().max()) / float(wf[0].grad.abs().max()),
        "dw2": float((wp[2].grad.float() - wf[2].grad).abs().max()) / float(wf[2].grad.abs().max()),
        "dwo": float((wo_r.grad.float() - wof.grad[r * n:(r + 1) * n]).abs().max()) /
               float(wof.grad.abs().max()),
    }
  torch.cuda.synchronize()
  json.dump(res, out)


def case_tp_train(out):
  """Three train steps of a small tensor-parallel model; the parent compares the fused
  kernels with the all-reduce form (T5X_B200_TP_FUSED=0)."""
  from t5x_b200.ops import native
  from t5x_b200.parallel import tp_fused
  st = _setup_tp()
  trainer, module = _tiny_trainer()
  batches = _batches(0, 1, 3)   # model ranks all see the same batch
  summary = trainer.train(iter(batches), 3, start_step=0).result()
  native.check_status()
  torch.cuda.synchronize()
  flat = torch.cat([p.detach().float().reshape(-1) for p in module.parameters()])
  json.dump({"loss": float(summary["loss"].value), "fused": tp_fused.enabled(),
             "param_abs": float(flat.double().abs().sum()),
             "first": flat[:8].tolist(),
             "norm": module.encoder.layers_1.pre_mlp_layer_norm.scale.detach().float()[:6].tolist()},
            out)
  trainer.close()


def case_tp_decode(out):
  """Beam search through the graph decoder with the model axis spanning all ranks of the run
  (one rank: the plain single-GPU decoder); the parent compares the two runs."""
  from t5x_b200 import adafactor, decoding_fast, models, trainer as trainer_lib
  from t5x_b200.data import vocabularies
  from t5x_b200.models import base
  from t5x_b200.models.t5 import network
  from t5x_b200.ops import native
  st = _setup_tp()
  cfg = network.T5Config(vocab_size=512, dtype="bfloat16", emb_dim=256, num_heads=4,
                         num_encoder_layers=2, num_decoder_layers=2, head_dim=64, mlp_dim=512,
                         mlp_activations=("gelu", "linear"), dropout_rate=0.0,
                         logits_via_embedding=False)
  torch.manual_seed(21)
  module = network.Transformer(cfg, device=st.device)
  with torch.no_grad():
    # sharper next-token distributions than a random initialisation gives: near-ties between
    # candidates would otherwise let bf16 rounding differences reorder the beams
    module.decoder.logits_dense.kernel.mul_(8.0)
  vocab = vocabularies.PassThroughVocabulary(512)
  model = models.EncoderDecoderModel(module, vocab, vocab, adafactor.Adafactor())
  trainer_lib.attach_compute_buffers(base.module_param_tree(module), bf16_copy=True,
                                     main_grad=False)
  g = torch.Generator().manual_seed(5)
  enc = torch.randint(2, 512, (8, 128), generator=g).to(st.device)
  enc[1, 90:] = 0
  dec = decoding_fast.GraphBeamDecoder(module, 8, 4, 12, eos_id=1, alpha=0.6, use_graph=True)
  for _ in range(2):  # the second call replays the captured step
    seqs, scores = dec.decode(enc)
  native.check_status()
  torch.cuda.synchronize()
  json.dump({"tp": dec.tp, "seqs": seqs[:, -1].tolist(), "scores": scores[:, -1].tolist(),
             "kernels_per_step": dec.kernels_per_step}, out)


def case_selfcheck(out):
  """The data-axis checks that the benchmark runs on its own mesh before it reports a number."""
  from t5x_b200.parallel import selfcheck
  _setup()
  json.dump(selfcheck.run(["dp"]), out)


CASES = {"selfcheck": case_selfcheck, "tp_decode": case_tp_decode, "collectives": case_collectives, "train": case_train, "moe": case_moe,
         "tp_ops": case_tp_ops, "tp_train": case_tp_train}

if __name__ == "__main__":
  case, out_dir = sys.argv[1], sys.argv[2]
  rank = int(os.environ.get("RANK", "0"))
  with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
    CASES[case](f)
  if dist.is_initialized():
    dist.barrier()
    dist.destroy_process_group()
