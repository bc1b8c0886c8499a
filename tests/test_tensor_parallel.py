"""Tensor-parallel (model axis) paths on CPU ranks over gloo: a 2-way sharded T5 must produce
the same loss, gradients and Adafactor update as the unsharded model."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
  s = socket.socket()
  s.bind(("127.0.0.1", 0))
  p = s.getsockname()[1]
  s.close()
  return p


def _build(seed=0):
  from t5x_b200 import adafactor, models
  from t5x_b200.data import vocabularies
  from t5x_b200.models.t5 import network
  cfg = network.T5Config(vocab_size=512, dtype="float32", emb_dim=256, num_heads=4,
                         num_encoder_layers=1, num_decoder_layers=1, head_dim=32, mlp_dim=512,
                         mlp_activations=("gelu", "linear"), dropout_rate=0.0)
  module = network.Transformer(cfg)
  vocab = vocabularies.PassThroughVocabulary(512)
  opt = adafactor.Adafactor(decay_rate=0.8, step_offset=0,
                            logical_factor_rules=adafactor.standard_logical_factor_rules())
  model = models.EncoderDecoderModel(module, vocab, vocab, opt, z_loss=1e-4)
  model.get_initial_variables(seed, None)
  return model


def _batch():
  g = torch.Generator().manual_seed(3)
  enc = torch.randint(3, 500, (4, 24), generator=g)
  enc[:, 20:] = 0
  tgt = torch.randint(3, 500, (4, 12), generator=g)
  tgt[:, 10:] = 0
  dec_in = torch.cat([torch.zeros(4, 1, dtype=torch.long), tgt[:, :-1]], 1)
  return {"encoder_input_tokens": enc, "decoder_target_tokens": tgt,
          "decoder_input_tokens": dec_in, "decoder_loss_weights": (tgt > 0).float()}


def _step(model):
  from t5x_b200 import train_state as ts_lib, trainer as trainer_lib
  from t5x_b200.models import base
  state = ts_lib.FlaxOptimTrainState.create(
      model.optimizer_def, {"params": base.module_param_tree(model.module),
                            "params_axes": base.module_param_axes(model.module)})
  tr = trainer_lib.Trainer(model, state, None, [], None, None, 0, lambda s: 0.01, 1)
  new_state, metrics = tr._train_step(state, _batch(), 0)
  tr.close()
  return new_state, metrics


def _gather_full(p, group):
  if getattr(p, "shard_dim", None) is None:
    return p.detach().clone()
  parts = [torch.empty_like(p) for _ in range(dist.get_world_size(group))]
  dist.all_gather(parts, p.detach().contiguous(), group=group)
  return torch.cat(parts, dim=p.shard_dim)


def _worker(rank, world, port, out_path):
  sys.path.insert(0, ROOT)
  os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                    WORLD_SIZE=str(world))
  dist.init_process_group("gloo", rank=rank, world_size=world)
  from t5x_b200.parallel import state as pstate
  st = pstate.setup_mesh(model_size=world, device=torch.device("cpu"))
  model = _build()
  new_state, metrics = _step(model)
  loss = float(metrics["loss"].total)
  full = {n: _gather_full(p, st.model_group) for n, p in model.module.named_parameters()}
  if rank == 0:
    torch.save({"loss": loss, "params": full}, out_path)
  dist.barrier()
  dist.destroy_process_group()


def test_two_way_tensor_parallel_matches_single(tmp_path):
  out = str(tmp_path / "tp.pt")
  mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
  got = torch.load(out)
  model = _build()
  _, metrics = _step(model)
  assert abs(float(metrics["loss"].total) - got["loss"]) / abs(got["loss"]) < 1e-4
  for n, p in model.module.named_parameters():
    a, b = got["params"][n], p.detach()
    assert a.shape == b.shape, n
    assert torch.allclose(a, b, rtol=2e-3, atol=2e-5), (n, (a - b).abs().max().item())


def test_symmetric_arena_allocator_is_deterministic_and_coalesces():
  """The first-fit allocator of the fused tensor-parallel path: every rank runs the same
  sequence, so offsets must depend on the sequence only; released blocks wait in quarantine
  until peers are known to be done with them; freed neighbours merge again."""
  from t5x_b200.parallel import tp_fused
  ar = object.__new__(tp_fused.SymmetricArena)
  ar.nbytes, ar.free, ar.generation, ar.allocations = 1 << 20, [(0, 1 << 20)], 0, 0
  ar.quarantine, ar.world = [], 1
  barriers = []
  ar.barrier = lambda: (barriers.append(1), ar.peers_are_past())
  a = ar.alloc(1000)          # rounded up to the 1024-byte granule
  b = ar.alloc(5000)
  c = ar.alloc(1024)
  assert (a.offset, a.size) == (0, 1024)
  assert (b.offset, b.size) == (1024, 5120)
  assert c.offset == 6144
  b.release()
  d = ar.alloc(2048)          # b's bytes may still be read by peers: not handed out yet
  assert d.offset == 7168
  ar.peers_are_past()         # e.g. a slot sum that waited for every peer has been enqueued
  e = ar.alloc(2048)          # first fit: the hole left by b
  assert e.offset == 1024
  for blk in (a, c, d, e):
    blk.release()
  b.release()                 # releasing twice is a no-op
  ar.peers_are_past()
  assert ar.free == [(0, 1 << 20)]
  f = ar.alloc(1 << 20)
  with pytest.raises(RuntimeError, match="arena exhausted"):
    ar.alloc(1)
  f.release()
  assert not barriers
  g = ar.alloc(4096)          # only quarantined bytes are left: a real barrier proves them free
  assert barriers == [1] and g.offset == 0
  del g                       # dropping a block frees nothing: object lifetime differs by rank
  assert ar.free == [(4096, (1 << 20) - 4096)]
  ar.end_step()               # the step boundary voids whatever is still allocated
  assert ar.free == [(0, 1 << 20)] and ar.allocations == 7
  h = ar.alloc(4096)
  ar.end_step()
  h.release()                 # a block of an earlier step is void: nothing is freed twice
  ar.peers_are_past()
  assert ar.free == [(0, 1 << 20)]


def test_owner_assignment_balances_and_is_deterministic():
  from t5x_b200.parallel import zero
  sizes = {"a": 100, "b": 90, "c": 50, "d": 40, "e": 10, "f": 10}
  owners = zero.assign_owners(sizes, 2)
  assert owners == zero.assign_owners(dict(reversed(list(sizes.items()))), 2)
  load = [sum(sizes[k] for k, r in owners.items() if r == rank) for rank in range(2)]
  assert sorted(load) == [150, 150]
  assert set(zero.assign_owners(sizes, 8).values()) <= set(range(8))
  assert zero.assign_owners({}, 4) == {}


def _partial_grad_worker(rank, world, port, out_path):
  sys.path.insert(0, ROOT)
  os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                    WORLD_SIZE=str(world))
  dist.init_process_group("gloo", rank=rank, world_size=world)
  from t5x_b200 import trainer as trainer_lib
  from t5x_b200.parallel import state as pstate
  pstate.setup_mesh(model_size=world, device=torch.device("cpu"))
  # two "norm scales" that saw this rank's rows only, one ordinary replicated parameter
  params = {"n1": torch.nn.Parameter(torch.zeros(4)), "n2": torch.nn.Parameter(torch.zeros(3)),
            "w": torch.nn.Parameter(torch.zeros(2))}
  params["n1"].sp_partial_grad = True
  params["n2"].sp_partial_grad = True
  grads = {"n1": torch.full((4,), float(rank + 1)), "n2": torch.arange(3.0) * (rank + 1),
           "w": torch.full((2,), 5.0)}
  trainer_lib.reduce_partial_gradients_over_model_axis(grads, params)
  torch.save({k: v.clone() for k, v in grads.items()}, f"{out_path}.{rank}")
  dist.destroy_process_group()


def test_partial_gradients_of_row_sharded_norms_are_summed_over_the_model_axis(tmp_path):
  out = str(tmp_path / "g")
  mp.spawn(_partial_grad_worker, args=(2, _free_port(), out), nprocs=2, join=True)
  for rank in range(2):
    g = torch.load(f"{out}.{rank}")
    assert g["n1"].tolist() == [3.0] * 4              # 1 + 2
    assert g["n2"].tolist() == [0.0, 3.0, 6.0]
    assert g["w"].tolist() == [5.0, 5.0]              # untouched
