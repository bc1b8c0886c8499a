"""Feature converters: what the models are fed for given task features, unpacked and packed
(the seqio converter contract worked through in t5x/models.py:1105-1148), and the remaining
checkpoint bookkeeping helpers."""
import os

import numpy as np
import pytest

from t5x_b200 import checkpoint_utils
from t5x_b200.data import feature_converters as fc
from t5x_b200.io import msgpack_io


def test_encoder_decoder_unpacked():
  conv = fc.EncDecFeatureConverter(pack=False)
  lengths = {"inputs": 6, "targets": 5}
  assert conv.get_model_feature_lengths(lengths) == {
      "encoder_input_tokens": 6, "decoder_target_tokens": 5, "decoder_input_tokens": 5,
      "decoder_loss_weights": 5}
  (a, b) = list(conv([{"inputs": [7, 8, 9, 1], "targets": [3, 4, 1]},
                      {"inputs": [5] * 9, "targets": [6] * 9}], lengths))
  assert a["encoder_input_tokens"].tolist() == [7, 8, 9, 1, 0, 0]
  assert a["decoder_target_tokens"].tolist() == [3, 4, 1, 0, 0]
  assert a["decoder_input_tokens"].tolist() == [0, 3, 4, 1, 0]
  assert a["decoder_loss_weights"].tolist() == [1, 1, 1, 0, 0]
  assert b["encoder_input_tokens"].tolist() == [5] * 6        # trimmed to the feature length
  assert b["decoder_target_tokens"].tolist() == [6] * 5


def test_encoder_decoder_packed():
  conv = fc.EncDecFeatureConverter(pack=True)
  lengths = {"inputs": 8, "targets": 6}
  assert set(conv.get_model_feature_lengths(lengths)) >= {
      "encoder_segment_ids", "decoder_segment_ids", "encoder_positions", "decoder_positions"}
  rows = list(conv([{"inputs": [7, 8, 1], "targets": [3, 1]},
                    {"inputs": [9, 9, 9, 1], "targets": [4, 5, 1]},
                    {"inputs": [2, 2, 2, 2, 1], "targets": [6, 1]}], lengths))
  assert len(rows) == 2                                         # the third does not fit the first row
  r = rows[0]
  assert r["encoder_input_tokens"].tolist() == [7, 8, 1, 9, 9, 9, 1, 0]
  assert r["encoder_segment_ids"].tolist() == [1, 1, 1, 2, 2, 2, 2, 0]
  assert r["encoder_positions"].tolist() == [0, 1, 2, 0, 1, 2, 3, 0]
  assert r["decoder_target_tokens"].tolist() == [3, 1, 4, 5, 1, 0]
  assert r["decoder_segment_ids"].tolist() == [1, 1, 2, 2, 2, 0]
  assert r["decoder_positions"].tolist() == [0, 1, 0, 1, 2, 0]
  # the shifted inputs restart at every packed example
  assert r["decoder_input_tokens"].tolist() == [0, 3, 0, 4, 5, 0]
  assert r["decoder_loss_weights"].tolist() == [1, 1, 1, 1, 1, 0]
  assert rows[1]["encoder_segment_ids"].tolist() == [1, 1, 1, 1, 1, 0, 0, 0]


def test_language_model_converter():
  conv = fc.LMFeatureConverter(pack=False)
  lengths = {"targets": 6}
  assert set(conv.get_model_feature_lengths(lengths)) == {
      "decoder_target_tokens", "decoder_input_tokens", "decoder_loss_weights"}
  (row,) = list(conv([{"targets": [3, 4, 5, 1]}], lengths))
  assert row["decoder_target_tokens"].tolist() == [3, 4, 5, 1, 0, 0]
  assert row["decoder_input_tokens"].tolist() == [0, 3, 4, 5, 1, 0]
  assert row["decoder_loss_weights"].tolist() == [1, 1, 1, 1, 0, 0]
  assert "decoder_causal_attention" not in row and "decoder_segment_ids" not in row
  packed = list(fc.LMFeatureConverter(pack=True)(
      [{"targets": [3, 4, 1]}, {"targets": [5, 1]}, {"targets": [6, 7, 8, 1]}], lengths))
  assert len(packed) == 2
  assert packed[0]["decoder_target_tokens"].tolist() == [3, 4, 1, 5, 1, 0]
  assert packed[0]["decoder_segment_ids"].tolist() == [1, 1, 1, 2, 2, 0]
  assert packed[0]["decoder_positions"].tolist() == [0, 1, 2, 0, 1, 0]
  assert packed[0]["decoder_input_tokens"].tolist() == [0, 3, 4, 0, 5, 0]


@pytest.mark.parametrize("loss_on_targets_only", [True, False])
def test_prefix_lm_converter(loss_on_targets_only):
  conv = fc.PrefixLMFeatureConverter(pack=False, loss_on_targets_only=loss_on_targets_only)
  lengths = {"inputs": 4, "targets": 4}
  assert conv.get_model_feature_lengths(lengths)["decoder_causal_attention"] == 8
  (row,) = list(conv([{"inputs": [9, 8, 7], "targets": [3, 4, 1]}], lengths))
  assert row["decoder_target_tokens"].tolist() == [9, 8, 7, 3, 4, 1, 0, 0]
  assert row["decoder_input_tokens"].tolist() == [0, 9, 8, 7, 3, 4, 1, 0]
  # the prefix plus the position that predicts the first target attend bidirectionally
  assert row["decoder_causal_attention"].tolist() == [1, 1, 1, 1, 0, 0, 0, 0]
  want = [0, 0, 0, 1, 1, 1, 0, 0] if loss_on_targets_only else [1, 1, 1, 1, 1, 1, 0, 0]
  assert row["decoder_loss_weights"].tolist() == want
  packed = list(fc.PrefixLMFeatureConverter(pack=True)(
      [{"inputs": [9, 8], "targets": [3, 1]}, {"inputs": [7], "targets": [4, 5, 1]}], lengths))
  (row,) = packed
  assert row["decoder_target_tokens"].tolist() == [9, 8, 3, 1, 7, 4, 5, 1]
  assert row["decoder_segment_ids"].tolist() == [1, 1, 1, 1, 2, 2, 2, 2]
  assert row["decoder_causal_attention"].tolist() == [1, 1, 1, 0, 1, 1, 0, 0]
  assert row["decoder_input_tokens"].tolist() == [0, 9, 8, 3, 0, 7, 4, 5]


# ---- checkpoint bookkeeping ---------------------------------------------------------------------
def test_unpin_and_dataset_checkpoint_removal(tmp_path):
  d = tmp_path / "checkpoint_5"
  d.mkdir()
  checkpoint_utils.unpin_checkpoint(str(d))                    # nothing to unpin: no error
  checkpoint_utils.pin_checkpoint(str(d), "keep me")
  assert open(checkpoint_utils.pinned_checkpoint_filepath(str(d))).read() == "keep me"
  assert not checkpoint_utils.is_pinned_checkpoint(str(tmp_path / "checkpoint_missing"))
  for name in ("train_ds-000-of-002", "train_ds-001-of-002", "other"):
    (d / name).write_text("x")
  checkpoint_utils.remove_dataset_checkpoint(str(d), "train_ds")     # pinned: kept
  assert sorted(os.listdir(d)).count("train_ds-000-of-002") == 1
  checkpoint_utils.unpin_checkpoint(str(d))
  checkpoint_utils.remove_dataset_checkpoint(str(d), "train_ds")
  assert sorted(f for f in os.listdir(d)) == ["other"]


def test_detect_checkpoint_type(tmp_path):
  types = checkpoint_utils.CheckpointTypes
  native = tmp_path / "native" / "checkpoint_3"
  native.mkdir(parents=True)
  spec = {"driver": "zarr", "kvstore": {"driver": "file", "path": "target.w"},
          "metadata": {"chunks": [2], "dtype": "<f4", "shape": [2]}}
  (native / "checkpoint").write_bytes(msgpack_io.msgpack_serialize(
      {"optimizer": {"target": {"w": spec}, "state": {"step": np.int32(3)}}, "version": 3}))
  assert checkpoint_utils.detect_checkpoint_type(str(native)) == types.T5X
  assert checkpoint_utils.detect_checkpoint_type(str(native / "checkpoint")) == types.T5X
  orbax = tmp_path / "orbax" / "7"
  (orbax / "state").mkdir(parents=True)
  (orbax / "_CHECKPOINT_METADATA").write_text("{}")
  assert checkpoint_utils.detect_checkpoint_type(str(orbax)) == types.ORBAX
  ocdbt = tmp_path / "ocdbt"
  ocdbt.mkdir()
  (ocdbt / "manifest.ocdbt").write_bytes(b"\x00")
  assert checkpoint_utils.detect_checkpoint_type(str(ocdbt)) == types.ORBAX
  tf = tmp_path / "tf"
  tf.mkdir()
  (tf / "model.ckpt-100.index").write_bytes(b"\x00")
  (tf / "checkpoint").write_text('model_checkpoint_path: "model.ckpt-100"\n')
  assert checkpoint_utils.detect_checkpoint_type(str(tf / "model.ckpt-100")) == types.T5X_TF
  # a mismatch with what the caller expected is only a warning
  assert checkpoint_utils.detect_checkpoint_type(str(native), expected=types.ORBAX) == types.T5X
