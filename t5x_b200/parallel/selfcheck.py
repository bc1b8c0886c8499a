"""Quick numerical checks of the multi-GPU kernels against library collectives.

A benchmark run on N GPUs calls these before its timed region (a second or two in total) and
reports the errors next to its numbers, so that a throughput figure always comes with evidence
that the fused paths computed the right thing on that box:

  tp_gemms()       all-gather -> GEMM and GEMM -> reduce-scatter (`parallel/tp_fused.py`) against
                   fp32 products of operands gathered / reduced with NCCL;
  dp_exchange()    the NVLink gradient sum (`t5x_peer_reduce_f32`) against `all_reduce`, and one
                   Adafactor step of a small model with the optimizer sharded over the data
                   axis against the same step with plain all-reduce;
  moe_exchange()   NVLink dispatch / combine (`ops/moe.py`) against `all_to_all_single`.

Each returns {name: relative error}; `run` collects them and raises if one exceeds `tol`.
They need the mesh axis they exercise to have more than one rank.
"""
from __future__ import annotations

import os
from typing import Dict

import torch
import torch.distributed as dist

from t5x_b200.parallel import state as pstate


def _rel(a: torch.Tensor, b: torch.Tensor) -> float:
  return float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp(min=1e-20))


def tp_gemms() -> Dict[str, float]:
  from t5x_b200.parallel import tp_fused
  st = pstate.get()
  T, r, dev = st.model_size, st.model_rank, st.device
  m, K, N = 256, 1024, 768
  M = m * T
  g = torch.Generator(device=dev).manual_seed(11)               # same on every rank
  gr = torch.Generator(device=dev).manual_seed(100 + r)         # differs by rank
  w = (torch.randn(K, N, device=dev, generator=g) * 0.05).bfloat16()
  rows = (torch.randn(m, K, device=dev, generator=gr)).bfloat16()
  blk = tp_fused._gather_block(rows)
  got = tp_fused.gemm_allgather(blk, M, K, w)
  blk.release()
  full = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
  dist.all_gather_into_tensor(full, rows, group=st.model_group)
  out = {"allgather_gemm": _rel(got, full.float() @ w.float())}
  # reduce-scatter: every rank holds a different [M, K] factor of the sum over ranks
  a = (torch.randn(M, K, device=dev, generator=gr)).bfloat16()
  wr = (torch.randn(K, N, device=dev, generator=gr) * 0.05).bfloat16()
  got = tp_fused._reduce_scatter(a, wr)
  ref = a.float() @ wr.float()
  dist.all_reduce(ref, group=st.model_group)
  out["gemm_reducescatter"] = _rel(got, ref[r * m:(r + 1) * m])
  tp_fused.arena().settle()
  return out


def _tiny_step(sharded: bool):
  """The parameter change after two Adafactor steps of a 2+2-layer model on this rank's shard
  of a fixed batch."""
  from t5x_b200 import adafactor, models, train_state as ts_lib, trainer as trainer_lib
  from t5x_b200.data import vocabularies
  from t5x_b200.models.t5 import network
  from t5x_b200.parallel import zero
  st = pstate.get()
  prev = os.environ.get("T5X_B200_OPTIMIZER_SHARDING")
  os.environ["T5X_B200_OPTIMIZER_SHARDING"] = "1" if sharded else "0"
  try:
    cfg = network.T5Config(vocab_size=512, dtype="bfloat16", emb_dim=128, num_heads=2,
                           num_encoder_layers=2, num_decoder_layers=2, head_dim=64, mlp_dim=256,
                           mlp_activations=("gelu", "linear"), dropout_rate=0.0)
    torch.manual_seed(7)
    module = network.Transformer(cfg, device=st.device)
    vocab = vocabularies.PassThroughVocabulary(512)
    opt = adafactor.Adafactor(decay_rate=0.8, step_offset=0,
                              logical_factor_rules=adafactor.standard_logical_factor_rules())
    model = models.EncoderDecoderModel(module, vocab, vocab, opt, z_loss=1e-4)
    state = ts_lib.FlaxOptimTrainState.create(opt, model.get_initial_variables(None, None))
    # taken before the trainer exists: with the optimizer sharded, a rank holds no fp32 master
    # of the parameters it does not own until `sync_replicas` brings them back
    before = torch.cat([p.detach().float().reshape(-1) for p in module.parameters()])
    trainer = trainer_lib.Trainer(model, state, None, [], None, None, 0, lambda s: 0.01, 2)
    per = 4
    g = torch.Generator().manual_seed(3)
    n = per * st.data_size
    enc = torch.randint(1, 512, (n, 64), generator=g)
    dec = torch.randint(1, 512, (n, 64), generator=g)
    dec_in = torch.cat([torch.zeros(n, 1, dtype=torch.long), dec[:, :-1]], 1)
    sl = slice(st.data_rank * per, (st.data_rank + 1) * per)
    batch = {"encoder_input_tokens": enc[sl], "decoder_input_tokens": dec_in[sl],
             "decoder_target_tokens": dec[sl], "decoder_loss_weights": torch.ones(per, 64)}
    with torch.enable_grad():
      trainer.train(iter([batch, batch]), 2, start_step=0).result()
    trainer.sync_replicas()
    after = torch.cat([p.detach().float().reshape(-1) for p in module.parameters()])
    trainer.close()
    return after - before
  finally:
    zero.disable()
    if prev is None:
      os.environ.pop("T5X_B200_OPTIMIZER_SHARDING", None)
    else:
      os.environ["T5X_B200_OPTIMIZER_SHARDING"] = prev


def dp_exchange() -> Dict[str, float]:
  from t5x_b200.ops import comm
  st = pstate.get()
  n = 1_000_003
  buf = comm.SymmetricBuffer(n, torch.float32, st.data_group, st.device)
  g = torch.Generator(device=st.device).manual_seed(200 + st.rank)
  buf.tensor.copy_(torch.randn(n, device=st.device, generator=g))
  want = buf.tensor.clone()
  dist.all_reduce(want, group=st.data_group)
  buf.barrier(0)
  got = torch.empty(n, device=st.device)
  comm.peer_reduce_f32_(got, buf.ptrs_at(0), n)
  buf.barrier(1)
  out = {"peer_reduce": _rel(got, want)}
  # the updates of two steps are compared, not the weights: an error in the exchange would
  # hide behind the weights' magnitude
  a, b = _tiny_step(True), _tiny_step(False)
  out["sharded_adafactor_vs_allreduce"] = float((a - b).norm() / b.norm())
  return out


def moe_exchange() -> Dict[str, float]:
  from t5x_b200.contrib.moe import layers
  from t5x_b200.ops import moe as moe_ops
  st = pstate.get()
  dev, ep = st.device, st.expert_size
  t, d, e, k = 512, 256, 2 * ep, 2
  cap = layers.expert_capacity(t, e, 1.5, k)
  g = torch.Generator(device=dev).manual_seed(300 + st.rank)
  tokens = torch.randn(t, d, device=dev, generator=g).bfloat16()
  index = torch.stack([torch.randperm(e, device=dev, generator=g)[:k] for _ in range(t)])
  flat = index.t().reshape(-1)
  hits = (flat[None, :] == torch.arange(e, device=dev)[:, None]).to(torch.int32)
  pos = (torch.cumsum(hits, 1).gather(0, flat[None, :]).squeeze(0).long() - 1).view(k, t).t()
  flat_slot = torch.where(pos < cap, index * cap + pos, torch.full_like(pos, -1))
  gate = torch.rand(t, k, device=dev, generator=g)
  x_f = moe_ops.FusedDispatch.apply(tokens, flat_slot, e, cap)
  x_r = layers._Dispatch.apply(tokens, flat_slot, e, cap)
  y = (x_r.float() * 1.5 + 0.25).bfloat16()   # stand-in for the experts
  o_f = moe_ops.FusedCombine.apply(y, flat_slot, gate, e, cap)
  o_r = layers._Combine.apply(y, flat_slot, gate.bfloat16(), e, cap)
  return {"moe_dispatch": _rel(x_f, x_r), "moe_combine": _rel(o_f, o_r)}


class SelfCheckError(RuntimeError):
  """A check exceeded its tolerance; `errors` holds every measured error of the call."""

  def __init__(self, message: str, errors: Dict[str, float]):
    super().__init__(message)
    self.errors = errors


def run(which, tol: float = 2e-2) -> Dict[str, float]:
  """Runs the named checks (`tp`, `dp`, `moe`) on the current mesh; all ranks must call it.
  Returns the largest error over ranks per check and raises `SelfCheckError` if any exceeds
  `tol`."""
  from t5x_b200.ops import native
  fns = {"tp": tp_gemms, "dp": dp_exchange, "moe": moe_exchange}
  out: Dict[str, float] = {}
  with torch.no_grad():
    for name in which:
      out.update(fns[name]())
  native.check_status()
  keys = sorted(out)
  vec = torch.tensor([out[k] for k in keys], dtype=torch.float64, device=pstate.get().device)
  if dist.is_initialized():
    dist.all_reduce(vec, op=dist.ReduceOp.MAX)
  out = {k: float(v) for k, v in zip(keys, vec)}
  bad = {k: v for k, v in out.items() if not v <= tol}
  if bad:
    raise SelfCheckError(f"multi-GPU self-check failed (tolerance {tol}): {bad}", out)
  return out
