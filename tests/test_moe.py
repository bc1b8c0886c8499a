"""Mixture-of-experts: router arithmetic, dispatch/combine against a dense oracle, model
wrapper metrics, partitioner, expert-parallel equivalence over gloo, sparse upcycling
(cases modelled on t5x/contrib/moe/*_test.py)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from t5x_b200 import adafactor
from t5x_b200.contrib.moe import adafactor_utils, layers, models, network
from t5x_b200.contrib.moe import partitioning as moe_partitioning
from t5x_b200.contrib.moe import training_utils
from t5x_b200.data import vocabularies


def test_router_capacity_and_priority():
  torch.manual_seed(0)
  r = layers.TokensChooseRouter(8, 4, num_selected_experts=2)
  tokens = torch.randn(12, 8)
  route, m = r(tokens, capacity=3)
  idx, slot, gate = route["expert_index"], route["slot"], route["gate"]
  assert idx.shape == slot.shape == gate.shape == (12, 2)
  for e in range(4):
    taken = sorted(int(s) for s in slot[idx == e] if s >= 0)
    assert taken == list(range(len(taken))) and len(taken) <= 3  # dense slots below capacity
  # first choices are placed before any second choice
  for e in range(4):
    first = slot[:, 0][(idx[:, 0] == e) & (slot[:, 0] >= 0)]
    second = slot[:, 1][(idx[:, 1] == e) & (slot[:, 1] >= 0)]
    if len(first) and len(second):
      assert int(first.max()) < int(second.min())
  assert torch.all(gate[slot < 0] == 0)
  assert set(m) == set(layers.MOE_METRICS)
  assert 0.0 <= float(m["fraction_tokens_left_behind"]) <= 1.0


def test_losses_closed_form():
  probs = torch.tensor([[0.7, 0.3], [0.6, 0.4], [0.2, 0.8], [0.9, 0.1]])
  idx = probs.argmax(-1, keepdim=True)
  # fractions (3/4, 1/4), mean probs (0.6, 0.4): 4 * mean(0.45, 0.1) = 1.1
  assert float(layers.load_balancing_loss(probs, idx)) == pytest.approx(1.1, rel=1e-6)
  logits = torch.log(probs)
  assert float(layers.router_z_loss(logits)) == pytest.approx(0.0, abs=1e-6)


def test_moe_layer_matches_dense_oracle_when_nothing_is_dropped():
  torch.manual_seed(1)
  layer = layers.MoeLayer(16, 32, num_experts=4, num_selected_experts=2, capacity_factor=8.0)
  x = torch.randn(2, 6, 16, requires_grad=True)
  layers.reset_collected_metrics()
  y = layer(x)
  # oracle: every token through its two experts, weighted by the router probabilities
  tokens = x.reshape(12, 16)
  probs = torch.softmax(tokens @ layer.router.router_weights.w.kernel, -1)
  gate, idx = torch.topk(probs, 2, -1)
  out = torch.zeros(12, 16)
  for t in range(12):
    for j in range(2):
      e = int(idx[t, j])
      h = torch.nn.functional.gelu(tokens[t] @ layer.expert.wi_0.kernel[e], approximate="tanh") * \
          (tokens[t] @ layer.expert.wi_1.kernel[e])
      out[t] += gate[t, j] * (h @ layer.expert.wo.kernel[e])
  torch.testing.assert_close(y.reshape(12, 16), out, rtol=1e-4, atol=1e-5)
  g1 = torch.autograd.grad(y.sum(), [x, layer.expert.wo.kernel], retain_graph=True)
  g2 = torch.autograd.grad(out.sum(), [x, layer.expert.wo.kernel])
  for a, b in zip(g1, g2):
    torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5)


def _moe_model(num_experts=4):
  cfg = network.MoeT5Config(vocab_size=64, emb_dim=16, num_heads=2, head_dim=8, mlp_dim=32,
                            num_encoder_layers=2, num_decoder_layers=2, dropout_rate=0.0,
                            mlp_activations=("gelu", "linear"), num_experts=num_experts)
  torch.manual_seed(3)
  m = network.Transformer(cfg)
  v = vocabularies.PassThroughVocabulary(64)
  opt = adafactor.Adafactor(logical_factor_rules=adafactor_utils.logical_factor_rules())
  return models.MoeEncoderDecoderModel(m, v, v, opt, aux_loss_factor=0.01,
                                       router_z_loss_factor=0.001)


def _batch(seed=0, b=4):
  g = torch.Generator().manual_seed(seed)
  x = torch.randint(1, 64, (b, 9), generator=g)
  y = torch.randint(1, 64, (b, 5), generator=g)
  return {"encoder_input_tokens": x, "decoder_input_tokens": y, "decoder_target_tokens": y,
          "decoder_loss_weights": torch.ones(b, 5)}


def test_model_adds_expert_losses_and_metrics():
  model = _moe_model()
  loss, metrics = model.loss_fn(None, _batch(), None)
  for name in ("auxiliary_loss", "router_z_loss", "fraction_tokens_left_behind", "expert_usage",
               "router_confidence"):
    assert f"experts/{name}" in metrics
  aux = float(metrics["experts/auxiliary_loss"].compute())
  rz = float(metrics["experts/router_z_loss"].compute())
  ce = float(metrics["cross_ent_loss"].compute())
  z = float(metrics["z_loss"].compute())
  assert float(loss) == pytest.approx(ce + z + aux + rz, rel=1e-5)
  names = [n for n, _ in model.module.named_parameters()]
  assert any("layers_1.mlp.expert.wi_0" in n for n in names)
  assert any("layers_0.mlp.wi_0" in n for n in names)  # dense layer kept


def test_training_utils():
  is_expert = training_utils.match_fn(r".*expert.*")
  assert is_expert("encoder/layers_1/mlp/expert/wi_0/kernel") and not is_expert("a/mlp/wi/kernel")
  tree = {"a": {"expert": {"w": torch.ones(2)}, "dense": {"w": torch.ones(2)}}}
  out = training_utils.scale_sharded_grads(tree, is_expert, 4.0)
  assert float(out["a"]["expert"]["w"][0]) == 4.0 and float(out["a"]["dense"]["w"][0]) == 1.0


def test_moe_partitioner_mesh_and_layout():
  p = moe_partitioning.MoePjitPartitioner(num_expert_partitions=4, num_partitions=1,
                                          world_size=8, local_rank=5)
  assert dict(p.mesh.shape) == {"data": 2, "expert": 4, "model": 1}
  lay = p.get_data_layout(16)
  assert lay.num_shards == 8 and 0 <= lay.shard_id < 8
  # expert axis shrinks to a divisor of the data axis
  p = moe_partitioning.MoePjitPartitioner(num_expert_partitions=3, num_partitions=1,
                                          world_size=8, local_rank=0)
  assert p.mesh.shape["expert"] == 2
  rules = dict(moe_partitioning.standard_logical_axis_rules())
  assert rules["batch"] == ("expert", "data") and rules["expert"] == "expert"
  assert moe_partitioning.compute_num_model_partitions(None, (1, 2, 1, 2)) == 4
  with pytest.raises(ValueError):
    moe_partitioning.compute_num_model_partitions(3, (1, 2, 1, 2))


# ---- expert parallelism over gloo ----------------------------------------------------------
def _ep_worker(rank, world, port, out):
  os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                    WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
  from t5x_b200.parallel import state as pstate
  pstate.init_distributed("gloo")
  pstate.setup_mesh(model_size=1, expert_size=world, device=torch.device("cpu"))
  model = _moe_model()
  full = _batch(seed=7, b=4)
  mine = {k: v[rank * 2:(rank + 1) * 2] for k, v in full.items()}
  loss, _ = model.loss_fn(None, mine, None)
  loss.backward()
  lt = loss.detach().clone()
  dist.all_reduce(lt)
  wi = model.module.encoder.layers_1.mlp.expert.wi_0.kernel
  dense = model.module.encoder.layers_0.mlp.wi_0.kernel.grad.clone()
  dist.all_reduce(dense)
  out[rank] = (float(lt), wi.grad.clone().numpy(), dense.numpy(), tuple(wi.shape))
  dist.barrier()
  dist.destroy_process_group()


def test_expert_parallel_matches_single_process(tmp_path):
  world = 2
  mgr = mp.Manager()
  out = mgr.dict()
  port = 29700 + os.getpid() % 200
  mp.spawn(_ep_worker, args=(world, port, out), nprocs=world, join=True)
  # single process, same global batch split in the same two groups
  model = _moe_model()
  full = _batch(seed=7, b=4)
  total = 0.0
  for r in range(world):
    loss, _ = model.loss_fn(None, {k: v[r * 2:(r + 1) * 2] for k, v in full.items()}, None)
    loss.backward()
    total += float(loss)
  wi_grad = model.module.encoder.layers_1.mlp.expert.wi_0.kernel.grad.numpy()
  dense_grad = model.module.encoder.layers_0.mlp.wi_0.kernel.grad.numpy()
  assert out[0][0] == pytest.approx(total, rel=1e-5)
  assert out[0][3] == (2, 16, 32)  # each rank holds half of the 4 experts
  ep_grad = np.concatenate([out[0][1], out[1][1]], axis=0)
  np.testing.assert_allclose(ep_grad, wi_grad, rtol=1e-4, atol=1e-6)
  np.testing.assert_allclose(out[0][2], dense_grad, rtol=1e-4, atol=1e-6)


def test_sparse_upcycling_broadcasts_dense_mlp(tmp_path):
  from t5x_b200 import checkpoints, partitioning, train_state as ts
  from t5x_b200 import models as base_models
  from t5x_b200.contrib.moe import checkpoints as moe_ckpt
  from t5x_b200.models.t5 import network as t5_network
  dense_cfg = t5_network.T5Config(vocab_size=64, emb_dim=16, num_heads=2, head_dim=8, mlp_dim=32,
                                  num_encoder_layers=2, num_decoder_layers=2, dropout_rate=0.0,
                                  mlp_activations=("gelu", "linear"))
  torch.manual_seed(11)
  dense = t5_network.Transformer(dense_cfg)
  v = vocabularies.PassThroughVocabulary(64)
  dmodel = base_models.EncoderDecoderModel(dense, v, v, adafactor.Adafactor())
  part = partitioning.PjitPartitioner(num_partitions=1, world_size=1, local_rank=0)
  dstate = ts.FlaxOptimTrainState.create(dmodel.optimizer_def,
                                         dmodel.get_initial_variables(None, None))
  checkpoints.Checkpointer(dstate, part, str(tmp_path)).save(dstate)

  sparse = _moe_model()
  sstate = ts.FlaxOptimTrainState.create(sparse.optimizer_def,
                                         sparse.get_initial_variables(None, None))
  moe_part = moe_partitioning.MoePjitPartitioner(num_expert_partitions=1, num_partitions=1,
                                                 world_size=1, local_rank=0)
  ck = moe_ckpt.UpcycleCheckpointer(sstate, moe_part, str(tmp_path), num_experts=4)
  from t5x_b200 import state_utils
  import functools
  # optimizer slots start from scratch (the tiny dense model is unfactored, the experts are
  # factored by rule); expert kernels map onto the dense MLP; routers have no dense source
  amap = [(r"state/param_states/.*", None), (r".*/router/.*", None),
          (r"(.*)/mlp/expert/(.*)", r"\1/mlp/\2")]
  fallback = {"target": {}, "state": {}}
  full_fallback = sstate.state_dict()
  restored = ck.restore(
      step=0, fallback_state=full_fallback,
      state_transformation_fns=[functools.partial(state_utils.apply_assignment_map,
                                                  assignment_map=amap)])
  e_w = restored.params["encoder"]["layers_1"]["mlp"]["expert"]["wi_0"]["kernel"]
  d_w = dense.encoder.layers_1.mlp.wi_0.kernel
  assert e_w.shape == (4, 16, 32)
  for e in range(4):
    torch.testing.assert_close(e_w[e].detach(), d_w.detach())
  torch.testing.assert_close(
      restored.params["encoder"]["layers_0"]["mlp"]["wi_0"]["kernel"].detach(),
      dense.encoder.layers_0.mlp.wi_0.kernel.detach())


def _moe_train_state(factored=True):
  from t5x_b200 import adafactor, train_state as ts_lib
  from t5x_b200.contrib.moe import adafactor_utils, models as moe_models, network as moe_network
  from t5x_b200.data import vocabularies
  cfg = moe_network.MoeT5Config(vocab_size=64, dtype="float32", emb_dim=128, num_heads=2,
                                head_dim=16, mlp_dim=256, num_encoder_layers=2,
                                num_decoder_layers=2, dropout_rate=0.0,
                                mlp_activations=("gelu", "linear"), num_experts=4,
                                num_selected_experts=1)
  module = moe_network.Transformer(cfg)
  v = vocabularies.PassThroughVocabulary(64)
  opt = adafactor.Adafactor(factored=factored,
                            logical_factor_rules=adafactor_utils.logical_factor_rules())
  model = moe_models.MoeEncoderDecoderModel(module, v, v, opt)
  return ts_lib.FlaxOptimTrainState.create(opt, model.get_initial_variables(None, None))


def test_moe_partitioner_marks_factored_expert_slots_and_lays_out_data():
  """The (data, expert, model) partitioner: factored Adafactor's v_row / v_col of expert
  kernels get the 'expert' axis (the reference's state filter), dense slots do not; data
  shards are numbered expert-major over the two data-like axes."""
  from t5x_b200.contrib.moe import partitioning as mp
  from t5x_b200.utils import tree
  state = _moe_train_state()
  part = mp.MoePjitPartitioner(num_expert_partitions=2, num_partitions=1, world_size=4,
                               local_rank=3)
  axes = tree.flatten_dict(part.get_mesh_axes(state).state_dict(),
                           is_leaf=lambda x: not isinstance(x, dict))
  expert_slot = "state/param_states/encoder/layers_1/mlp/expert/wi_0/kernel/"
  dense_slot = "state/param_states/encoder/layers_0/mlp/wi_0/kernel/"
  assert axes[expert_slot + "v_row"] == mp.PartitionSpec("expert",)
  assert axes[expert_slot + "v_col"] == mp.PartitionSpec("expert",)
  assert axes[dense_slot + "v_row"] is None
  assert axes["target/encoder/layers_1/mlp/expert/wi_0/kernel"][0] == "expert"
  # mesh data=2 x expert=2 x model=1: rank 3 is (data 1, expert 1) -> shard 1 + 1 * 2
  layout = part.get_data_layout(16)
  assert (layout.shard_id, layout.num_shards, layout.batch_size) == (3, 4, 16)
  assert layout.is_first_host_in_replica_set
  with pytest.raises(ValueError, match="entire data mesh size"):
    part.get_data_layout(6)
  # unfactored Adafactor: slots inherit the parameter's names, nothing to override
  assert mp._infer_state_filter_fn(_moe_train_state(factored=False)) is None


def test_experts_choose_router_fills_every_expert_with_its_best_tokens():
  from t5x_b200.contrib.moe import layers
  torch.manual_seed(0)
  t, d, e, cap = 40, 16, 4, 6
  router = layers.ExpertsChooseRouter(d, e)
  tokens = torch.randn(t, d)
  route, metrics = router(tokens, cap)
  probs = torch.softmax(tokens @ router.router_weights.w.kernel.float(), -1)
  fs, gate = route["flat_slot"], route["gate"]
  for ex in range(e):
    best = set(torch.topk(probs[:, ex], cap).indices.tolist())
    picked = set(torch.nonzero(fs[:, ex] >= 0).squeeze(1).tolist())
    assert picked == best
    # its capacity rows of the dispatch buffer are all used, each once
    assert sorted(fs[fs[:, ex] >= 0, ex].tolist()) == list(range(ex * cap, (ex + 1) * cap))
    assert torch.allclose(gate[list(best), ex], probs[list(best), ex])
  assert float(metrics["auxiliary_loss"]) == 0.0 and float(metrics["expert_usage"]) == 1.0
  left = 1.0 - (fs >= 0).any(1).float().mean()
  assert float(metrics["fraction_tokens_left_behind"]) == pytest.approx(float(left))
  # the whole layer runs and is differentiable with this router
  layer = layers.MoeLayer(d, 32, e, router_type="experts_choose", capacity_factor=1.0)
  x = torch.randn(2, 20, d, requires_grad=True)
  layer(x).sum().backward()
  assert x.grad is not None and layer.router.router_weights.w.kernel.grad is not None
