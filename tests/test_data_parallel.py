"""Data-parallel (data axis) paths on CPU ranks over gloo.

  * a batch-derived loss normalising factor counts the global batch, so two replicas with half
    the batch each reproduce the single-process loss and update;
  * the sharded optimizer's overlapped update leaves out parameters whose gradient still owes
    a sum over the model axis.
"""
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


def _build(loss_normalizing_factor, seed=0):
  from t5x_b200 import adafactor, models
  from t5x_b200.data import vocabularies
  from t5x_b200.models.t5 import network
  cfg = network.T5Config(vocab_size=256, dtype="float32", emb_dim=128, num_heads=2,
                         num_encoder_layers=1, num_decoder_layers=1, head_dim=32, mlp_dim=256,
                         mlp_activations=("gelu", "linear"), dropout_rate=0.0)
  module = network.Transformer(cfg)
  vocab = vocabularies.PassThroughVocabulary(256)
  opt = adafactor.Adafactor(decay_rate=0.8, step_offset=0,
                            logical_factor_rules=adafactor.standard_logical_factor_rules())
  model = models.EncoderDecoderModel(module, vocab, vocab, opt, z_loss=1e-4,
                                     loss_normalizing_factor=loss_normalizing_factor)
  model.get_initial_variables(seed, None)
  return model


def _batch():
  """Four examples with different numbers of real target tokens, so that a per-shard count
  differs from the global one."""
  g = torch.Generator().manual_seed(5)
  enc = torch.randint(3, 250, (4, 16), generator=g)
  tgt = torch.randint(3, 250, (4, 10), generator=g)
  for row, n in enumerate((10, 3, 7, 5)):
    tgt[row, n:] = 0
  dec_in = torch.cat([torch.zeros(4, 1, dtype=torch.long), tgt[:, :-1]], 1)
  return {"encoder_input_tokens": enc, "decoder_target_tokens": tgt,
          "decoder_input_tokens": dec_in, "decoder_loss_weights": (tgt > 0).float()}


def _step(model, batch):
  from t5x_b200 import train_state as ts_lib, trainer as trainer_lib
  from t5x_b200.models import base
  state = ts_lib.FlaxOptimTrainState.create(
      model.optimizer_def, {"params": base.module_param_tree(model.module),
                            "params_axes": base.module_param_axes(model.module)})
  tr = trainer_lib.Trainer(model, state, None, [], None, None, 0, lambda s: 0.01, 1)
  _, metrics = tr._train_step(state, batch, 0)
  tr.close()
  return metrics


def _dp_worker(rank, world, port, factor, out_path):
  sys.path.insert(0, ROOT)
  os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                    WORLD_SIZE=str(world))
  dist.init_process_group("gloo", rank=rank, world_size=world)
  from t5x_b200.parallel import state as pstate
  pstate.setup_mesh(model_size=1, device=torch.device("cpu"))
  model = _build(factor)
  full = _batch()
  n = full["encoder_input_tokens"].shape[0] // world
  shard = {k: v[rank * n:(rank + 1) * n] for k, v in full.items()}
  metrics = _step(model, shard)
  if rank == 0:
    torch.save({"loss": float(metrics["loss"].total),
                "params": {k: p.detach().clone() for k, p in model.module.named_parameters()}},
               out_path)
  dist.barrier()
  dist.destroy_process_group()


@pytest.mark.parametrize("factor", ["NUM_REAL_TARGET_TOKENS", "NUM_TOTAL_TARGET_TOKENS",
                                    "AVERAGE_PER_SEQUENCE"])
def test_special_loss_normalizing_factor_counts_the_global_batch(tmp_path, factor):
  out = str(tmp_path / "dp.pt")
  mp.spawn(_dp_worker, args=(2, _free_port(), factor, out), nprocs=2, join=True)
  got = torch.load(out)
  model = _build(factor)
  metrics = _step(model, _batch())
  want = float(metrics["loss"].total)
  assert abs(got["loss"] - want) / abs(want) < 1e-5, (got["loss"], want)
  for n, p in model.module.named_parameters():
    a, b = got["params"][n], p.detach()
    assert torch.allclose(a, b, rtol=2e-4, atol=2e-6), (n, (a - b).abs().max().item())


def test_overlapped_update_skips_parameters_that_owe_a_model_axis_sum():
  """On a data x model mesh the norm scales of the row-sharded residual stream hold partial
  gradients until the model-axis all-reduce after backward; the per-layer update that runs
  under the backward pass must leave them to the ordinary path."""
  from t5x_b200.parallel import state as pstate, zero

  def param(ready=True, partial=False):
    p = torch.nn.Parameter(torch.zeros(4))
    p.grad_ready = ready
    if partial:
      p.sp_partial_grad = True
    return p

  ctx = object.__new__(zero.ZeroContext)
  ctx.params = {"w": param(), "scale": param(partial=True), "late": param(ready=False)}
  ctx._buckets = {"layers_0": ["w", "scale", "late"]}
  st = pstate.get()
  st.model_size = 1
  assert ctx._final_names("layers_0") == ["w", "scale"]
  st.model_size = 2
  assert ctx._final_names("layers_0") == ["w"]


def test_optimizer_slots_are_matched_to_their_parameters():
  """`sync_replicas` broadcasts each slot from its parameter's owner: both state layouts
  (slots under the parameter path; parameter tree under each moment) resolve, counters do not."""
  from t5x_b200.parallel import zero
  names = ["enc/mlp/kernel", "enc/norm/scale"]
  adafactor_like = {"enc": {"mlp": {"kernel": {"v_row": torch.ones(2), "v_col": torch.ones(3),
                                               "m": torch.zeros(1), "v": torch.zeros(1)}},
                            "norm": {"scale": {"v": torch.ones(4)}}}}
  got = zero.state_leaves_by_param(names, adafactor_like)
  assert [len(got[n]) for n in names] == [4, 1]
  # ranks walk the result to issue broadcasts: its order must be the caller's, not a set's
  many = [f"p{i}/kernel" for i in range(50)]
  assert list(zero.state_leaves_by_param(many, {})) == many
  tree = lambda: {"enc": {"mlp": {"kernel": torch.ones(2, 3)}, "norm": {"scale": torch.ones(4)}}}
  optax_like = {"0": {}, "1": {"0": {"count": torch.tensor(3), "mu": tree(), "nu": tree()},
                               "1": {}, "2": {"count": torch.tensor(3)}}}
  got = zero.state_leaves_by_param(names, optax_like)
  assert [len(got[n]) for n in names] == [2, 2]
  assert all(v.shape == (2, 3) for v in got["enc/mlp/kernel"])


def test_buffer_plan_for_sharded_weights():
  """Layout of the symmetric buffers: gradients replicated in full; weights replicated for the
  resident parameters and, for the streamed ones, packed per owner without overlap."""
  from t5x_b200.parallel import zero
  sizes = {"emb": 65536, "l0/q": 16384, "l0/wi": 32768 + 5, "l1/q": 16384, "l1/wi": 32768,
           "logits": 70000}
  names = list(sizes)
  world = 3
  owners = zero.assign_owners(sizes, world)
  assert sorted(set(owners.values())) == [0, 1, 2]
  streamed = {k for k in names if k.startswith("l")}
  g_off, g_total, w_off, w_total = zero.plan_buffers(names, sizes, owners, streamed, world)
  pad = lambda n: -(-n // 128) * 128
  assert g_total == sum(pad(n) for n in sizes.values())
  assert all(off % 128 == 0 for off in list(g_off.values()) + list(w_off.values()))
  # gradient ranges do not overlap
  spans = sorted((g_off[k], g_off[k] + sizes[k]) for k in names)
  assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))
  # resident weights sit first and at the same place for everyone; every owner's streamed
  # parameters follow without overlapping each other or the resident part
  resident_end = max(w_off[k] + pad(sizes[k]) for k in names if k not in streamed)
  for r in range(world):
    mine = sorted((w_off[k], w_off[k] + sizes[k]) for k in streamed if owners[k] == r)
    assert all(a[0] >= resident_end for a in mine)
    assert all(a[1] <= b[0] for a, b in zip(mine, mine[1:]))
    assert all(a[1] <= w_total for a in mine)
  assert w_total < g_total  # that is the point of sharding them
  # nothing streamed: both buffers have the same layout
  g2, t2, w2, wt2 = zero.plan_buffers(names, sizes, owners, set(), world)
  assert w2 == g2 and wt2 == t2


@pytest.mark.parametrize("world", [2, 4, 8])
def test_owner_plan_of_an_xxl_shaped_model(world):
  """The ownership plan on the parameter list of T5.1.1-XXL (shapes only, no storage): owners
  are balanced, every offset is aligned, nothing overlaps, and sharding the layer weights cuts
  the weight buffer to about the replicated part plus 1/world of the layers."""
  from t5x_b200.models.t5 import network
  from t5x_b200.parallel import zero
  cfg = network.T5Config(vocab_size=32128, dtype="bfloat16", emb_dim=4096, num_heads=64,
                         num_encoder_layers=24, num_decoder_layers=24, head_dim=64,
                         mlp_dim=10240, mlp_activations=("gelu", "linear"), dropout_rate=0.0)
  with torch.device("meta"):
    module = network.Transformer(cfg)
  sizes = {n: p.numel() for n, p in module.named_parameters()}
  names = list(sizes)
  total = sum(sizes.values())
  assert 11.0e9 < total < 11.6e9
  owners = zero.assign_owners(sizes, world)
  load = [sum(sizes[k] for k in names if owners[k] == r) for r in range(world)]
  assert max(load) - min(load) <= 0.02 * total / world
  streamed = {k for k in names if zero._LAYER_RE.search(k)}
  assert len(streamed) >= 48 * 6
  g_off, g_total, w_off, w_total = zero.plan_buffers(names, sizes, owners, streamed, world)
  assert all(o % zero._ALIGN == 0 for o in list(g_off.values()) + list(w_off.values()))
  assert total <= g_total <= total + zero._ALIGN * len(names)
  spans = sorted((g_off[k], g_off[k] + sizes[k]) for k in names)
  assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))
  resident = sum(sizes[k] for k in names if k not in streamed)
  layers = total - resident
  assert w_total <= resident + 1.05 * layers / world + zero._ALIGN * len(names)
  for r in range(world):
    mine = sorted((w_off[k], w_off[k] + sizes[k]) for k in streamed if owners[k] == r)
    assert all(a[1] <= b[0] for a, b in zip(mine, mine[1:])) and mine[-1][1] <= w_total
