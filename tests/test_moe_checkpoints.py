"""The dense-to-sparse checkpointer (contracts of t5x/contrib/moe/checkpoints.py): plain round
trips of a sparse state, lazy and typed restores, and upcycling of weights and optimizer
slots from native and Orbax-layout dense checkpoints."""
import functools

import numpy as np
import pytest
import torch

from t5x_b200 import adafactor, checkpoints, partitioning, state_utils
from t5x_b200 import models as base_models
from t5x_b200 import train_state as ts
from t5x_b200.contrib.moe import adafactor_utils, checkpoints as moe_ckpt
from t5x_b200.contrib.moe import models as moe_models, network as moe_network
from t5x_b200.contrib.moe import partitioning as moe_partitioning
from t5x_b200.data import vocabularies
from t5x_b200.models.t5 import network as t5_network
from t5x_b200.utils import tree

COMMON = dict(vocab_size=64, dtype="float32", emb_dim=128, num_heads=2, head_dim=16, mlp_dim=256,
              num_encoder_layers=2, num_decoder_layers=2, dropout_rate=0.0,
              mlp_activations=("gelu", "linear"))


def _sparse_state(seed=0):
  torch.manual_seed(seed)
  module = moe_network.Transformer(moe_network.MoeT5Config(num_experts=4, num_selected_experts=1,
                                                           **COMMON))
  v = vocabularies.PassThroughVocabulary(64)
  opt = adafactor.Adafactor(logical_factor_rules=adafactor_utils.logical_factor_rules())
  model = moe_models.MoeEncoderDecoderModel(module, v, v, opt)
  return ts.FlaxOptimTrainState.create(opt, model.get_initial_variables(None, None))


def _dense_state(seed=1):
  torch.manual_seed(seed)
  module = t5_network.Transformer(t5_network.T5Config(**COMMON))
  v = vocabularies.PassThroughVocabulary(64)
  opt = adafactor.Adafactor(logical_factor_rules=adafactor.standard_logical_factor_rules())
  model = base_models.EncoderDecoderModel(module, v, v, opt)
  state = ts.FlaxOptimTrainState.create(opt, model.get_initial_variables(None, None))
  g = torch.Generator().manual_seed(3)
  for slot in tree.flatten_dict(state.param_states).values():
    slot.copy_(torch.rand(slot.shape, generator=g))
  return state.replace_step(11)


def _moe_part():
  return moe_partitioning.MoePjitPartitioner(num_expert_partitions=1, num_partitions=1,
                                             world_size=1, local_rank=0)


def _values(state):
  return {k: np.asarray(v.detach()) if isinstance(v, torch.Tensor) else np.asarray(v)
          for k, v in tree.flatten_dict(state.state_dict()).items()}


def test_sparse_state_round_trips_unchanged(tmp_path):
  state = _sparse_state(0).replace_step(4)
  want = _values(state)
  moe_ckpt.UpcycleCheckpointer(state, _moe_part(), str(tmp_path), num_experts=4).save(state)
  other = _sparse_state(5)
  restored = moe_ckpt.UpcycleCheckpointer(other, _moe_part(), str(tmp_path),
                                          num_experts=4).restore()
  got = _values(restored)
  assert got.keys() == want.keys() and int(restored.step) == 4
  for k in want:
    np.testing.assert_array_equal(got[k], want[k], err_msg=k)


# Expert arrays take the dense MLP's values; routers have no dense source and stay as initialised.
AMAP = [(r"(.*)/mlp/expert/(.*)", r"\1/mlp/\2"), (r".*/router/.*", None)]


def _upcycle(tmp_path, sparse, **kw):
  ck = moe_ckpt.UpcycleCheckpointer(sparse, _moe_part(), str(tmp_path), num_experts=4,
                                    **{k: v for k, v in kw.items() if k == "restore_dtype"})
  return ck.restore(
      fallback_state=sparse.state_dict(),
      state_transformation_fns=[functools.partial(state_utils.apply_assignment_map,
                                                  assignment_map=AMAP)],
      lazy_parameters=kw.get("lazy", False))


@pytest.mark.parametrize("layout", ["native", "orbax_tree"])
def test_upcycling_repeats_weights_and_optimizer_slots_over_experts(tmp_path, layout):
  dense = _dense_state()
  part = partitioning.PjitPartitioner(num_partitions=1, world_size=1, local_rank=0)
  if layout == "native":
    checkpoints.Checkpointer(dense, part, str(tmp_path)).save(dense)
  else:
    checkpoints.save_state_as_orbax_tree(dense, str(tmp_path))
  dvals = _values(dense)
  sparse = _sparse_state(0)
  router_before = sparse.params["encoder"]["layers_1"]["mlp"]["router"]["router_weights"]["w"][
      "kernel"].detach().clone()
  restored = _upcycle(tmp_path, sparse)
  assert int(restored.step) == 11
  rvals = _values(restored)
  # sparse layers: every expert is a copy of the dense MLP, weights and slots alike
  n_checked = 0
  for k, v in rvals.items():
    if "/mlp/expert/" not in k:
      continue
    src = dvals[k.replace("/mlp/expert/", "/mlp/")]
    if v.shape == src.shape == (1,):   # placeholder of an unused slot (factored: no full `v`)
      continue
    assert v.shape == (4,) + src.shape, k
    for e in range(4):
      np.testing.assert_array_equal(v[e], src, err_msg=k)
    n_checked += 1
  assert n_checked >= 2 * 3 * 2   # two sparse layers x three kernels x (weight + a slot)
  assert any(k.startswith("state/param_states/") and "/mlp/expert/" in k for k in rvals)
  # everything else is restored as is; routers keep their initial values
  for k in ("target/token_embedder/embedding", "target/encoder/layers_0/mlp/wi_0/kernel",
            "state/param_states/encoder/layers_0/attention/query/kernel/v_row"):
    np.testing.assert_array_equal(rvals[k], dvals[k], err_msg=k)
  torch.testing.assert_close(
      restored.params["encoder"]["layers_1"]["mlp"]["router"]["router_weights"]["w"]["kernel"],
      router_before)


def test_upcycling_with_restore_dtype(tmp_path):
  dense = _dense_state()
  part = partitioning.PjitPartitioner(num_partitions=1, world_size=1, local_rank=0)
  checkpoints.Checkpointer(dense, part, str(tmp_path)).save(dense)
  ck = moe_ckpt.UpcycleCheckpointer(_sparse_state(0), _moe_part(), str(tmp_path), num_experts=4,
                                    restore_dtype=np.dtype("float16"))
  leaf_name = "target/encoder/layers_1/mlp/expert/wo/kernel"
  sd = ck._train_state.state_dict()
  index = checkpoints.load_t5x_checkpoint(str(tmp_path), lazy_parameters=True)
  target = tree.flatten_dict(sd)[leaf_name]
  from t5x_b200.io import msgpack_io
  raw = msgpack_io.msgpack_restore(open(tmp_path / "checkpoint_11" / "checkpoint", "rb").read())
  ckpt_leaf = raw["optimizer"]["target"]["encoder"]["layers_1"]["mlp"]["wo"]["kernel"]
  lazy = ck._read_leaf(leaf_name, ckpt_leaf, target, None, str(tmp_path / "checkpoint_11"), 3, True)
  assert isinstance(lazy, checkpoints.LazyArray)
  assert lazy.shape == (4, 256, 128) and np.dtype(lazy.dtype) == np.float16
  arr = lazy.get()
  assert arr.dtype == np.float16 and arr.shape == (4, 256, 128)
  dense_w = np.asarray(dense.params["encoder"]["layers_1"]["mlp"]["wo"]["kernel"].detach())
  np.testing.assert_array_equal(arr[2], dense_w.astype(np.float16))
  # optimizer slots keep their stored type
  slot_name = "state/param_states/encoder/layers_1/mlp/expert/wo/kernel/v_row"
  slot_leaf = raw["optimizer"]["state"]["param_states"]["encoder"]["layers_1"]["mlp"]["wo"][
      "kernel"]["v_row"]
  slot = ck._read_leaf(slot_name, slot_leaf, tree.flatten_dict(sd)[slot_name], None,
                       str(tmp_path / "checkpoint_11"), 3, False)
  assert slot.dtype == np.float32 and slot.shape[0] == 4
  del index


def test_broadcast_rule():
  assert moe_ckpt._needs_broadcast((16, 32), (4, 16, 32), 4)
  assert not moe_ckpt._needs_broadcast((16, 32), (8, 16, 32), 4)     # not the expert count
  assert not moe_ckpt._needs_broadcast((4, 16, 32), (4, 16, 32), 4)  # already per expert
  assert not moe_ckpt._needs_broadcast((16, 32), (4, 16, 64), 4)     # trailing dims differ
  assert not moe_ckpt._needs_broadcast((32,), (4, 16, 32), 4)
