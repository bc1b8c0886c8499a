"""Synthetic T5 span-corruption examples (seeded, no files needed).

Tokens are uniform in [3, 32000); about `noise_density` of them are masked in noise spans of
mean length `mean_noise_span_length`; each span is replaced in the inputs by a sentinel id
counting down from `first_sentinel`, and the targets are the sentinel + span concatenations.
EOS = 1 closes both sides, pad = 0. The span segmentation follows the published T5 recipe
(random partition of the noise / non-noise token counts into the same number of spans).
"""
from __future__ import annotations

from typing import Dict, Iterator

import numpy as np


def _random_segmentation(rng: np.random.Generator, num_items: int, num_segments: int):
  """Partition `num_items` into `num_segments` positive lengths, uniformly at random."""
  first = np.zeros(num_items - 1, dtype=np.int64)
  first[:num_segments - 1] = 1
  rng.shuffle(first)
  seg_id = np.concatenate([[0], np.cumsum(first)])
  return np.bincount(seg_id, minlength=num_segments)


def span_corruption_example(rng: np.random.Generator, inputs_length: int, targets_length: int,
                            noise_density: float = 0.15, mean_noise_span_length: float = 3.0,
                            vocab_low: int = 3, vocab_high: int = 32000,
                            first_sentinel: int = 32099, eos_id: int = 1) -> Dict[str, np.ndarray]:
  """One example whose corrupted input fills `inputs_length` (incl. EOS) as closely as possible."""
  # Pick the raw length so that inputs (non-noise + sentinels + EOS) fit inputs_length.
  raw = inputs_length
  for cand in range(inputs_length, int(inputs_length / (1 - noise_density)) + 8):
    n_noise = int(round(cand * noise_density))
    n_spans = max(1, int(round(n_noise / mean_noise_span_length)))
    if cand - n_noise + n_spans + 1 <= inputs_length and n_noise + n_spans + 1 <= targets_length:
      raw = cand
    else:
      break
  num_noise = max(1, min(raw - 1, int(round(raw * noise_density))))
  num_spans = max(1, int(round(num_noise / mean_noise_span_length)))
  num_nonnoise = raw - num_noise
  tokens = rng.integers(vocab_low, vocab_high, size=raw, dtype=np.int64)
  noise_lens = _random_segmentation(rng, num_noise, num_spans)
  nonnoise_lens = _random_segmentation(rng, num_nonnoise, num_spans)
  inputs, targets = [], []
  pos = 0
  for i in range(num_spans):
    sentinel = first_sentinel - i
    inputs.extend(tokens[pos:pos + nonnoise_lens[i]])
    pos += nonnoise_lens[i]
    inputs.append(sentinel)
    targets.append(sentinel)
    targets.extend(tokens[pos:pos + noise_lens[i]])
    pos += noise_lens[i]
  inputs.append(eos_id)
  targets.append(eos_id)
  return {"inputs": np.asarray(inputs[:inputs_length], dtype=np.int32),
          "targets": np.asarray(targets[:targets_length], dtype=np.int32)}


def span_corruption_stream(seed: int, inputs_length: int, targets_length: int,
                           shard_id: int = 0, num_shards: int = 1,
                           **kwargs) -> Iterator[Dict[str, np.ndarray]]:
  """Infinite deterministic stream; shard `shard_id` of `num_shards` takes every n-th example."""
  index = shard_id
  while True:
    rng = np.random.default_rng([seed, index])
    yield span_corruption_example(rng, inputs_length, targets_length, **kwargs)
    index += num_shards
