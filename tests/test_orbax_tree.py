"""PyTree checkpoint directories (one zarr array per leaf): reading the sample the reference
ships, round trips of the writer, the metadata fallbacks, and restoring a train state."""
import json
import os

import numpy as np
import pytest

from t5x_b200 import checkpoint_utils, checkpoints, partitioning
from t5x_b200.io import orbax_tree

from test_checkpoints import flat_values, make_state, randomize_opt_state

# A PyTree checkpoint written by Orbax itself (the `tiny_orbax` sample of the reference's test
# data: aggregate file + one zstd chunk per array, zarr metadata files not shipped), base64.
_SAMPLE_FILES = {
    "checkpoint":
        "hKpfb3B0aW1pemVygqVzdGF0ZYKscGFyYW1fc3RhdGVzg6RiaWFz2TBQTEFDRUhPTERFUjovL19vcHRp"
        "bWl6ZXIuc3RhdGUucGFyYW1fc3RhdGVzLmJpYXOma2VybmVs2TJQTEFDRUhPTERFUjovL19vcHRpbWl6"
        "ZXIuc3RhdGUucGFyYW1fc3RhdGVzLmtlcm5lbKRzdGVw2TBQTEFDRUhPTERFUjovL19vcHRpbWl6ZXIu"
        "c3RhdGUucGFyYW1fc3RhdGVzLnN0ZXCkc3RlcNkjUExBQ0VIT0xERVI6Ly9fb3B0aW1pemVyLnN0YXRl"
        "LnN0ZXCmdGFyZ2V0gK1mbGF4X211dGFibGVzwLJmbGF4X211dGFibGVzX2F4ZXPAq3BhcmFtc19heGVz"
        "wA==",
    "_optimizer.state.param_states.bias/0":
        "KLUv/QAAVQAAIAAAgD8BACOOCA==",
    "_optimizer.state.param_states.kernel/0.0":
        "KLUv/QAAgQwAOOHmH8k/wz/yzF69RmzmP29GUy0bE+A/f4kfqZmk5T+OAVa64MPaP2r+91XkZ9U/AhZg"
        "hM1U7T+g5QS5IFqbP2b/lPLjkt0/6THuGYjl7j/fUuPYbsrlPyTLyUnT7Os/QAhyynmF6z+fekOQD23l"
        "P2xjXkoZOsk/oXFsS6QU7T+sEEEdgmfZP/HlajAr/OA/1FL3QcDB0D/wThzNe7TGP21W90anZ+Q/b3Xd"
        "v2ic4z/qvXuwxr/tPwjZYU1z6b4/CiOY/Oc01j/QRSpmgR3RP+qYIHvEK9Q/lD8kTUdtxz84yhFsUHLr"
        "PzDdTthumOA/X5xQi05I6z8k/H45GxfJP9AjLs1Zoqk/vLTqy+PL2j9j82XthbjjP6yHbw3kss0/GHL4"
        "UqCUwD8bUuRUE+vvP1fPtKyN3e4/uBVixhY+xT8LXewE6XDoP0YmLRmJTOo/nBnW6Eu03T9QXMFX0MzH"
        "P0BYgJosQek/zuf/lOM87j8mHnvOQ1DYP5zMsFggedU/ag+AL9nA6D9hypYAPNntPw==",
    "_optimizer.state.param_states.step/0":
        "KLUv/QAAIQAAAQAAAA==",
    "_optimizer.state.step/0":
        "KLUv/QAAIQAAAQAAAA==",
}


@pytest.fixture
def sample(tmp_path):
  import base64
  root = tmp_path / "tiny_orbax" / "1"
  for name, data in _SAMPLE_FILES.items():
    f = root / name
    f.parent.mkdir(parents=True, exist_ok=True)
    f.write_bytes(base64.b64decode(data))
  return str(root)


def test_reads_the_sample_tree(sample):
  assert orbax_tree.is_tree_dir(sample) and not orbax_tree.is_ocdbt(sample)
  assert orbax_tree.find_state_dir(sample) == sample
  tree = orbax_tree.load_tree(sample)
  assert set(tree) == {"_optimizer", "flax_mutables", "flax_mutables_axes", "params_axes"}
  assert tree["flax_mutables"] is None and tree["_optimizer"]["target"] == {}
  state = tree["_optimizer"]["state"]
  # The sample's zarr metadata files were not shipped: shapes come from the caller.
  assert state["step"].shape is None
  step = state["step"].read(expected_shape=(), expected_dtype=np.int32)
  assert step.shape == () and int(step) == 1
  bias = state["param_states"]["bias"].read(expected_shape=(5,), expected_dtype=np.float32)
  np.testing.assert_array_equal(bias, np.ones(5, np.float32))
  # 400 bytes for 50 elements: the stored type is float64 although the target asks for float32
  kernel = state["param_states"]["kernel"].read(expected_shape=(10, 5),
                                                expected_dtype=np.float32, dtype=np.float32)
  assert kernel.shape == (10, 5) and kernel.dtype == np.float32
  assert np.all((kernel >= 0) & (kernel <= 1)) and kernel.std() > 0.1
  with pytest.raises(ValueError, match="do not fill shape"):
    state["param_states"]["kernel"].read(expected_shape=(7, 3), expected_dtype=np.float32)
  with pytest.raises(ValueError, match="no zarr metadata"):
    state["param_states"]["kernel"].read()


def test_sample_is_detected_as_orbax(sample):
  types = checkpoint_utils.CheckpointTypes
  assert checkpoint_utils.detect_checkpoint_type(sample) == types.ORBAX
  assert checkpoint_utils.detect_checkpoint_type(os.path.join(sample, "checkpoint")) == types.ORBAX


def _tree():
  rng = np.random.default_rng(0)
  return {"state": {"step": np.int32(7),
                    "param_states": {"a": {"v_row": rng.random(4).astype(np.float32), "m": None}}},
          "target": {"layers": [rng.random((3, 2)).astype(np.float32),
                                rng.integers(0, 9, (2,)).astype(np.int64)],
                     "empty": {}}}


@pytest.mark.parametrize("compressor", [None, {"id": "gzip", "level": 1}, False])
def test_round_trip_with_every_source_of_structure(tmp_path, compressor):
  d = str(tmp_path)
  tree = _tree()
  orbax_tree.save_tree(d, tree, compressor)
  assert sorted(os.listdir(d)) == ["_METADATA", "checkpoint", "state.param_states.a.v_row",
                                   "state.step", "target.layers.0", "target.layers.1"]
  meta = json.loads(open(os.path.join(d, "target.layers.0", ".zarray")).read())
  want = "gzip" if isinstance(compressor, dict) else ("zstd" if compressor is None else None)
  assert (meta["compressor"] or {}).get("id") == want

  def check(loaded, lists=True):
    assert int(loaded["state"]["step"].read()) == 7
    assert loaded["state"]["step"].shape == () and loaded["state"]["step"].dtype == np.int32
    np.testing.assert_array_equal(loaded["state"]["param_states"]["a"]["v_row"].read(),
                                  tree["state"]["param_states"]["a"]["v_row"])
    layers = loaded["target"]["layers"]
    first, second = (layers[0], layers[1]) if lists else (layers["0"], layers["1"])
    np.testing.assert_array_equal(first.read(), tree["target"]["layers"][0])
    np.testing.assert_array_equal(first.read((slice(1, 3), slice(0, 1)), dtype=np.float64),
                                  tree["target"]["layers"][0][1:3, 0:1].astype(np.float64))
    assert second.read().dtype == np.int64

  # 1. the aggregate file of placeholders
  loaded = orbax_tree.load_tree(d)
  check(loaded)
  assert loaded["state"]["param_states"]["a"]["m"] is None
  # 2. the metadata file's key list
  os.remove(os.path.join(d, "checkpoint"))
  loaded = orbax_tree.load_tree(d)
  check(loaded)
  assert loaded["state"]["param_states"]["a"]["m"] is None and loaded["target"]["empty"] == {}
  # 3. the array directories alone (sequence indices stay string keys)
  os.remove(os.path.join(d, "_METADATA"))
  check(orbax_tree.load_tree(d), lists=False)


def test_metadata_without_key_metadata_and_missing_tree(tmp_path):
  d = str(tmp_path / "t")
  orbax_tree.save_tree(d, {"a": {"b": np.arange(3)}}, aggregate=False)
  meta = json.load(open(os.path.join(d, "_METADATA")))
  (key, entry), = meta["tree_metadata"].items()
  assert key == "('a', 'b')" and entry["key_metadata"] == [{"key": "a", "key_type": 2},
                                                            {"key": "b", "key_type": 2}]
  del entry["key_metadata"]
  json.dump(meta, open(os.path.join(d, "_METADATA"), "w"))
  np.testing.assert_array_equal(orbax_tree.load_tree(d)["a"]["b"].read(), np.arange(3))
  empty = tmp_path / "none"
  empty.mkdir()
  assert not orbax_tree.is_tree_dir(str(empty)) and orbax_tree.find_state_dir(str(empty)) is None
  with pytest.raises(ValueError, match="No PyTree checkpoint"):
    orbax_tree.load_tree(str(empty))


def test_ocdbt_directories_are_refused(tmp_path):
  d = tmp_path / "checkpoint_3" / "state"
  d.mkdir(parents=True)
  (d / "manifest.ocdbt").write_bytes(b"\x0c\xdb\x3a\x2a")
  assert orbax_tree.is_ocdbt(str(d)) and orbax_tree.is_tree_dir(str(d))
  assert orbax_tree.find_state_dir(str(tmp_path / "checkpoint_3")) == str(d)
  with pytest.raises(NotImplementedError, match="OCDBT"):
    orbax_tree.load_tree(str(d))
  state = make_state(0)
  part = partitioning.PjitPartitioner(num_partitions=1, world_size=1, local_rank=0)
  with pytest.raises(NotImplementedError, match="OCDBT"):
    checkpoints.Checkpointer(state, part, str(tmp_path)).restore(step=3)


def test_zarr_v3_arrays(tmp_path):
  import gzip
  d = tmp_path / "w"
  (d / "c" / "0").mkdir(parents=True)
  (d / "c" / "1").mkdir(parents=True)
  full = np.arange(12, dtype=np.float32).reshape(3, 4)
  meta = {"zarr_format": 3, "node_type": "array", "shape": [3, 4], "data_type": "float32",
          "chunk_grid": {"name": "regular", "configuration": {"chunk_shape": [2, 4]}},
          "chunk_key_encoding": {"name": "default", "configuration": {"separator": "/"}},
          "fill_value": 0.0,
          "codecs": [{"name": "bytes", "configuration": {"endian": "little"}},
                     {"name": "gzip", "configuration": {"level": 1}}]}
  (d / "zarr.json").write_text(json.dumps(meta))
  (d / "c" / "0" / "0").write_bytes(gzip.compress(full[0:2].tobytes()))
  pad = np.zeros((2, 4), np.float32)
  pad[0] = full[2]
  (d / "c" / "1" / "0").write_bytes(gzip.compress(pad.tobytes()))
  ref = orbax_tree.ArrayRef(str(d), "w")
  assert ref.shape == (3, 4) and ref.dtype == np.float32
  np.testing.assert_array_equal(ref.read(), full)
  np.testing.assert_array_equal(ref.read((slice(2, 3), slice(1, 3))), full[2:3, 1:3])
  with pytest.raises(ValueError, match="does not match expectation"):
    ref.read(expected_shape=(4, 3))
  meta["codecs"].insert(0, {"name": "transpose", "configuration": {"order": [1, 0]}})
  (d / "zarr.json").write_text(json.dumps(meta))
  with pytest.raises(NotImplementedError, match="transpose"):
    orbax_tree.ArrayRef(str(d), "w")


def test_train_state_restores_from_a_tree_directory(tmp_path):
  state = randomize_opt_state(make_state(0))
  ckpt_dir = checkpoints.save_state_as_orbax_tree(state, str(tmp_path))
  assert ckpt_dir == str(tmp_path / "checkpoint_7")
  assert (tmp_path / "checkpoint_7" / "state" / "_METADATA").exists()
  assert (tmp_path / "checkpoint_7" / "state" / "target.encoder.layers_0.mlp.wi_0.kernel"
          / ".zarray").exists()
  types = checkpoint_utils.CheckpointTypes
  assert checkpoint_utils.detect_checkpoint_type(ckpt_dir) == types.ORBAX
  part = partitioning.PjitPartitioner(num_partitions=1, world_size=1, local_rank=0)
  other = make_state(1)
  # through the manager surface the training loop uses, by latest step and by path
  mgr = checkpoints.OrbaxCheckpointManagerInterface(str(tmp_path), other, part)
  assert mgr.all_steps() == [7]
  for restored in (mgr.restore(), mgr.restore(path=ckpt_dir)):
    a, b = flat_values(state), flat_values(restored)
    assert a.keys() == b.keys()
    for k in a:
      np.testing.assert_array_equal(a[k], b[k], err_msg=k)
    assert int(restored.step) == 7
  mgr.close()
  # without a model
  loaded = checkpoints.load_t5x_checkpoint(str(tmp_path))
  np.testing.assert_array_equal(loaded["target"]["token_embedder"]["embedding"],
                                flat_values(state)["target/token_embedder/embedding"])
  loaded = checkpoints.load_t5x_checkpoint(ckpt_dir, restore_dtype="bfloat16")
  assert loaded["target"]["token_embedder"]["embedding"].dtype.name == "bfloat16"
  assert loaded["state"]["param_states"]["token_embedder"]["embedding"]["v_row"].dtype == np.float32
  # a shape mismatch is reported with the parameter's name
  bad = tmp_path / "checkpoint_7" / "state" / "target.encoder.layers_0.mlp.wi_0.kernel" / ".zarray"
  meta = json.loads(bad.read_text())
  meta["shape"] = [64, 256]
  bad.write_text(json.dumps(meta))
  with pytest.raises(ValueError, match="wi_0/kernel"):
    checkpoints.Checkpointer(other, part, str(tmp_path)).restore()
