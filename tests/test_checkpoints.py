"""Native T5X checkpoint format: round trip, on-disk layout, retention, simulated multi-host
save under one topology / restore under another, assignment maps and fallback state."""
import json
import os

import numpy as np
import pytest
import torch

from t5x_b200 import adafactor, checkpoints, models, partitioning, state_utils
from t5x_b200 import train_state as ts_lib
from t5x_b200.data import vocabularies
from t5x_b200.io import msgpack_io
from t5x_b200.models import base
from t5x_b200.models.t5 import network
from t5x_b200.utils import tree


def make_state(seed=0, beta1=None):
  cfg = network.T5Config(vocab_size=256, dtype="float32", emb_dim=128, num_heads=2,
                         num_encoder_layers=1, num_decoder_layers=1, head_dim=32, mlp_dim=256,
                         mlp_activations=("gelu", "linear"), dropout_rate=0.0)
  module = network.Transformer(cfg)
  vocab = vocabularies.PassThroughVocabulary(256)
  opt = adafactor.Adafactor(decay_rate=0.8, step_offset=0, beta1=beta1,
                            logical_factor_rules=adafactor.standard_logical_factor_rules())
  model = models.EncoderDecoderModel(module, vocab, vocab, opt)
  variables = model.get_initial_variables(seed, None)
  return ts_lib.FlaxOptimTrainState.create(opt, variables)


def randomize_opt_state(state):
  flat = tree.flatten_dict(state.param_states)
  g = torch.Generator().manual_seed(5)
  for v in flat.values():
    v.copy_(torch.rand(v.shape, generator=g))
  return state.replace_step(7)


def flat_values(state):
  return {k: np.asarray(v.detach().cpu() if isinstance(v, torch.Tensor) else v)
          for k, v in tree.flatten_dict(state.state_dict()).items()}


def test_round_trip_and_layout(tmp_path):
  state = randomize_opt_state(make_state(0))
  part = partitioning.PjitPartitioner(num_partitions=1, world_size=1, local_rank=0)
  ck = checkpoints.Checkpointer(state, part, str(tmp_path), keep=2)
  ck.save(state)
  d = tmp_path / "checkpoint_7"
  assert (d / "checkpoint").exists()
  # every parameter with logical axes is a zarr array named by its dotted path
  zdir = d / "target.encoder.layers_0.mlp.wi_0.kernel"
  meta = json.loads((zdir / ".zarray").read_text())
  assert meta["shape"] == [128, 256] and meta["compressor"]["id"] == "gzip" and meta["dtype"] == "<f4"
  index = msgpack_io.msgpack_restore((d / "checkpoint").read_bytes())
  assert index["version"] == 3
  leaf = index["optimizer"]["target"]["encoder"]["layers_0"]["mlp"]["wi_0"]["kernel"]
  assert leaf["driver"] == "zarr" and leaf["kvstore"] == {
      "driver": "file", "path": "target.encoder.layers_0.mlp.wi_0.kernel"}
  # factored moments are inline arrays, the unfactored `v` of a norm scale is a zarr array
  ps = index["optimizer"]["state"]["param_states"]["encoder"]["layers_0"]["mlp"]["wi_0"]["kernel"]
  assert isinstance(ps["v_row"], np.ndarray) and ps["v_row"].shape == (128,)
  assert ps["v"].shape == (1,)
  norm_v = index["optimizer"]["state"]["param_states"]["encoder"]["encoder_norm"]["scale"]["v"]
  assert state_utils.tensorstore_leaf(None, norm_v)
  assert int(index["optimizer"]["state"]["step"]) == 7

  other = make_state(1)
  ck2 = checkpoints.Checkpointer(other, part, str(tmp_path))
  restored = ck2.restore()
  a, b = flat_values(state), flat_values(restored)
  assert a.keys() == b.keys()
  for k in a:
    np.testing.assert_array_equal(a[k], b[k], err_msg=k)
  assert int(restored.step) == 7
  # load without a model
  loaded = checkpoints.load_t5x_checkpoint(str(tmp_path))
  np.testing.assert_array_equal(loaded["target"]["token_embedder"]["embedding"],
                                a["target/token_embedder/embedding"])


def test_keep_and_pinned(tmp_path):
  from t5x_b200 import checkpoint_utils
  state = make_state(0)
  part = partitioning.PjitPartitioner(num_partitions=1, world_size=1, local_rank=0)
  ck = checkpoints.Checkpointer(state, part, str(tmp_path), keep=2)
  for step in (1, 2):
    ck.save(state.replace_step(step))
  checkpoint_utils.pin_checkpoint(str(tmp_path / "checkpoint_1"))
  for step in (3, 4):
    ck.save(state.replace_step(step))
  assert ck.all_steps() == [1, 3, 4]
  assert not any(".tmp-" in n for n in os.listdir(tmp_path))
  ck.save(state.replace_step(4))  # existing directory: skipped, not an error


def test_save_dtype_bfloat16_and_restore_dtype(tmp_path):
  state = make_state(0)
  part = partitioning.PjitPartitioner(num_partitions=1, world_size=1, local_rank=0)
  ck = checkpoints.Checkpointer(state, part, str(tmp_path), save_dtype="bfloat16")
  ck.save(state)
  meta = json.loads((tmp_path / "checkpoint_0" / "target.token_embedder.embedding" /
                     ".zarray").read_text())
  assert meta["dtype"] == "bfloat16"
  # optimizer state is never cast
  meta_v = json.loads((tmp_path / "checkpoint_0" /
                       "state.param_states.encoder.encoder_norm.scale.v" / ".zarray").read_text())
  assert meta_v["dtype"] == "<f4"
  restored = checkpoints.Checkpointer(make_state(1), part, str(tmp_path)).restore()
  want = state.params["token_embedder"]["embedding"].detach().bfloat16().float()
  torch.testing.assert_close(restored.params["token_embedder"]["embedding"].detach(), want)


class _FakeShardedState:
  """A train state as one simulated host of a `model`-sharded job sees it: column-parallel
  kernels hold only this host's slice."""


def _shard_state(full_state, model_size, model_rank):
  """Builds the per-rank view of `full_state` by slicing every parameter the way the layer
  library shards it, keeping global_shape/shard_dim annotations."""
  st = make_state(0)
  flat_full = tree.flatten_dict(full_state.state_dict())
  sd = st.state_dict()
  flat = tree.flatten_dict(sd)
  shard_dims = {"query": 1, "key": 1, "value": 1, "out": 0, "wi_0": 1, "wi_1": 1, "wo": 0,
                "embedding": 0, "logits_dense": 1, "rel_embedding": 0}
  new = {}
  for k, v in flat.items():
    parts = k.split("/")
    full = flat_full[k]
    dim = None
    if parts[0] == "target" or parts[-1] in ("v", "m"):
      for name, d in shard_dims.items():
        if name in parts and tuple(full.shape) != (1,):
          dim = d
    if dim is None or not isinstance(full, torch.Tensor) or full.dim() == 0:
      new[k] = full
      continue
    per = full.shape[dim] // model_size
    t = full.detach().narrow(dim, model_rank * per, per).clone()
    t.global_shape = tuple(full.shape)
    t.shard_dim = dim
    new[k] = t
  return new


class _DictState:
  """Minimal train-state protocol over a flat dict (for simulated hosts)."""

  def __init__(self, flat, axes_state):
    self._flat = flat
    self._axes_state = axes_state

  @property
  def step(self):
    return self._flat["state/step"]

  def state_dict(self):
    return tree.unflatten_dict(self._flat)

  def as_logical_axes(self):
    return self._axes_state

  def restore_state(self, sd):
    return _DictState(tree.flatten_dict(sd), self._axes_state)


@pytest.mark.parametrize("save_topology,restore_topology", [((2, 2), (1, 1)), ((1, 1), (4, 2)),
                                                            ((4, 2), (2, 1)), ((2, 1), (2, 2))])
def test_cross_topology_restore(tmp_path, save_topology, restore_topology):
  """Save with (hosts, model partitions) = A, restore with B; every simulated host calls the
  checkpointer in turn, as the reference's multi-host test does
  (t5x/contrib/moe/checkpoints_test.py:285-318)."""
  full = randomize_opt_state(make_state(0))
  want = flat_values(full)
  axes_state = full.as_logical_axes()

  def run_hosts(topology, fn):
    hosts, model = topology
    for rank in range(hosts):
      part = partitioning.PjitPartitioner(num_partitions=model, world_size=hosts, local_rank=rank)
      coords = part.mesh.coords()
      flat = _shard_state(full, model, coords["model"])
      fn(rank, part, _DictState(flat, axes_state), coords)

  saved_order = []

  def save(rank, part, st, coords):
    ck = checkpoints.Checkpointer(st, part, str(tmp_path))
    # ranks other than 0 write chunks only; emulate the rank-0-only index/rename
    import t5x_b200.checkpoints as C
    orig = C._rank
    C._rank = lambda: rank
    try:
      if rank != 0:
        os.makedirs(str(tmp_path), exist_ok=True)
      saved_order.append(rank)
      ck.save(st)
    finally:
      C._rank = orig

  # rank 0 must run last so that the directory rename happens after every host wrote.
  hosts = save_topology[0]
  import t5x_b200.checkpoints as C
  fixed_ts = 1234
  orig_b = C._broadcast_int_from_rank0
  C._broadcast_int_from_rank0 = lambda v: fixed_ts
  try:
    for rank in list(range(1, hosts)) + [0]:
      part = partitioning.PjitPartitioner(num_partitions=save_topology[1], world_size=hosts,
                                          local_rank=rank)
      coords = part.mesh.coords()
      save(rank, part, _DictState(_shard_state(full, save_topology[1], coords["model"]),
                                  axes_state), coords)
  finally:
    C._broadcast_int_from_rank0 = orig_b
  assert (tmp_path / "checkpoint_7" / "checkpoint").exists()

  def restore(rank, part, st, coords):
    ck = checkpoints.Checkpointer(st, part, str(tmp_path))
    got = tree.flatten_dict(ck.restore().state_dict())
    expect = _shard_state(full, restore_topology[1], coords["model"])
    for k, v in expect.items():
      if isinstance(v, torch.Tensor):
        g = got[k]
        if getattr(v, "shard_dim", None) is not None and tuple(np.shape(g)) == tuple(v.global_shape):
          per = v.global_shape[v.shard_dim] // restore_topology[1]
          g = np.take(np.asarray(g), range(coords["model"] * per, (coords["model"] + 1) * per),
                      axis=v.shard_dim)
        np.testing.assert_array_equal(np.asarray(g), v.detach().numpy(), err_msg=f"{k} rank {rank}")

  run_hosts(restore_topology, restore)


def test_assignment_map_and_fallback(tmp_path):
  state = randomize_opt_state(make_state(0))
  part = partitioning.PjitPartitioner(num_partitions=1, world_size=1, local_rank=0)
  checkpoints.Checkpointer(state, part, str(tmp_path)).save(state)
  target = make_state(1)
  before = {k: v.clone() for k, v in tree.flatten_dict(target.param_states).items()}
  # drop the checkpoint's optimizer state; it comes from the fallback (fresh) state instead
  amap = [(r"state/param_states.*", None)]
  import functools
  fn = functools.partial(state_utils.apply_assignment_map, assignment_map=amap)
  fallback = {"state": {"param_states": target.state_dict()["state"]["param_states"]}}
  restored = checkpoints.Checkpointer(target, part, str(tmp_path)).restore(
      state_transformation_fns=[fn], fallback_state=fallback)
  torch.testing.assert_close(restored.params["decoder"]["layers_0"]["mlp"]["wo"]["kernel"],
                             state.params["decoder"]["layers_0"]["mlp"]["wo"]["kernel"])
  for k, v in tree.flatten_dict(restored.param_states).items():
    torch.testing.assert_close(v, before[k])
  # without the fallback the missing optimizer state is an error
  with pytest.raises(ValueError):
    checkpoints.Checkpointer(make_state(2), part, str(tmp_path)).restore(
        state_transformation_fns=[fn])


def test_apply_assignment_map_semantics():
  ckpt = {"target": {"old_a": 1, "old_b": 2, "shared": 3}, "state": {"step": 9}}
  opt = {"target": {"new_a": 0, "new_a2": 0, "shared": 0, "dropped": 0, "absent": 0},
         "state": {"step": 0}}
  out = state_utils.apply_assignment_map(
      ckpt, opt, [(r"target/new_a(.*)", r"target/old_a"), (r"target/dropped", None)])
  # two new keys may take the same old key; matched old keys disappear; unmatched old keys stay;
  # unmapped new keys are copied when the checkpoint has them; None drops
  assert out["target"] == {"new_a": 1, "new_a2": 1, "old_b": 2, "shared": 3}
  assert out["state"]["step"] == 9
  with pytest.raises(ValueError, match="Unused patterns"):
    state_utils.apply_assignment_map(ckpt, opt, [(r"target/nothing", r"target/old_a")])
  with pytest.raises(ValueError, match="does not exist"):
    state_utils.apply_assignment_map(ckpt, opt, [(r"target/new_a", r"target/missing")])
  assert state_utils.apply_assignment_map(ckpt, opt, [("x", "y")], is_resuming=True) is ckpt
