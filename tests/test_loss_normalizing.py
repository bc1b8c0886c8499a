"""Special loss-normalizing factors (contracts of t5x/losses.py:220-343): golden values for
padded and packed batches, with and without explicit loss weights."""
import numpy as np
import torch

from t5x_b200 import losses

F = losses.SpecialLossNormalizingFactor


def _resolve(factor, batch):
  batch = {k: torch.as_tensor(v) for k, v in batch.items()}
  lnf, w = losses.get_loss_normalizing_factor_and_weights(factor, batch)
  return float(lnf) if lnf is not None else None, None if w is None else np.asarray(w)


def test_constant_factor_passes_through():
  batch = {"decoder_target_tokens": [[1, 2, 0]]}
  lnf, w = _resolve(7.0, batch)
  assert lnf == 7.0
  assert w is None or np.array_equal(w, [[1.0, 1.0, 0.0]])
  lnf, w = _resolve(None, batch)
  assert lnf is None


def test_num_real_target_tokens():
  lnf, w = _resolve(F.NUM_REAL_TARGET_TOKENS,
                    {"decoder_target_tokens": [[1, 2, 3, 4, 0], [5, 6, 0, 0, 0]]})
  np.testing.assert_allclose(lnf, 6.0, rtol=1e-6)
  np.testing.assert_allclose(w, [[1, 1, 1, 1, 0], [1, 1, 0, 0, 0]])


def test_num_total_target_tokens():
  lnf, w = _resolve(F.NUM_TOTAL_TARGET_TOKENS,
                    {"decoder_target_tokens": [[1, 2, 3, 4, 0], [5, 6, 0, 0, 0]]})
  np.testing.assert_allclose(lnf, 10.0, rtol=1e-6)
  np.testing.assert_allclose(w, [[1, 1, 1, 1, 0], [1, 1, 0, 0, 0]])


def test_average_per_sequence():
  lnf, w = _resolve(F.AVERAGE_PER_SEQUENCE,
                    {"decoder_target_tokens": [[1, 2, 3, 4, 0], [5, 6, 0, 0, 0]]})
  np.testing.assert_allclose(lnf, 2.0, rtol=1e-6)
  np.testing.assert_allclose(w, [[0.25, 0.25, 0.25, 0.25, 0], [0.5, 0.5, 0, 0, 0]], rtol=1e-6)


def test_average_per_sequence_with_weights():
  lnf, w = _resolve(F.AVERAGE_PER_SEQUENCE, {
      "decoder_target_tokens": [[1, 2, 3, 4, 0], [5, 6, 0, 0, 0]],
      "decoder_loss_weights": [[0.5, 1.0, 0.25, 2.0, 0.0], [1.0, 1.0, 0.0, 0.0, 0.0]]})
  np.testing.assert_allclose(lnf, 2.0, rtol=1e-6)
  np.testing.assert_allclose(w, [[0.5 / 3.75, 1 / 3.75, 0.25 / 3.75, 2 / 3.75, 0],
                                 [0.5, 0.5, 0, 0, 0]], rtol=1e-6)


def test_sum_weights_per_segment():
  weights = torch.tensor([[0.5, 1.0, 0.25, 2.0, 1.5], [1.0, 2.0, 3.0, 4.0, 5.0]])
  positions = torch.tensor([[0, 1, 2, 0, 0], [0, 0, 1, 0, 0]])
  segment_ids = torch.tensor([[1, 1, 1, 2, 3], [1, 2, 2, 3, 0]])
  got = losses._sum_weights_per_segment(positions, segment_ids, weights)
  np.testing.assert_allclose(np.asarray(got), [[1.75, 1.75, 1.75, 2.0, 1.5],
                                               [1.0, 5.0, 5.0, 4.0, 0.0]], rtol=1e-6)


def test_average_per_sequence_with_weights_and_packing():
  lnf, w = _resolve(F.AVERAGE_PER_SEQUENCE, {
      "decoder_target_tokens": [[1, 2, 3, 4, 5], [5, 6, 7, 8, 0]],
      "decoder_loss_weights": [[0.5, 1.0, 0.25, 2.0, 1.5], [1.0, 2.0, 3.0, 4.0, 5.0]],
      "decoder_positions": [[0, 1, 2, 0, 0], [0, 0, 1, 0, 0]],
      "decoder_segment_ids": [[1, 1, 1, 2, 3], [1, 2, 2, 3, 0]]})
  np.testing.assert_allclose(lnf, 6.0, rtol=1e-6)
  np.testing.assert_allclose(w, [[0.5 / 1.75, 1 / 1.75, 0.25 / 1.75, 1.0, 1.0],
                                 [1.0, 2 / 5, 3 / 5, 1.0, 0.0]], rtol=1e-6)


def test_string_names_convert_to_the_enum():
  conv = losses.convert_special_loss_normalizing_factor_to_enum
  assert conv("NUM_REAL_TARGET_TOKENS") == F.NUM_REAL_TARGET_TOKENS
  assert conv("num_total_target_tokens") == F.NUM_TOTAL_TARGET_TOKENS
  assert conv("Average_Per_Sequence") == F.AVERAGE_PER_SEQUENCE
  try:
    conv("nonsense")
  except ValueError as e:
    assert "nonsense" in str(e)
  else:
    raise AssertionError("an unknown name must be rejected")
