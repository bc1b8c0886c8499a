"""Example-level preprocessors for file-backed tasks (the `t5.data.preprocessors` /
`seqio.preprocessors` functions the reference's task definitions compose).

Everything here works on Python / numpy values one example at a time and is deterministic given
its seed; the T5 span-corruption recipe is the published one: i.i.d.-length noise spans covering
`noise_density` of the tokens with mean length `mean_noise_span_length`, each replaced in the
inputs by one sentinel counting down from the top of the vocabulary, targets = sentinel + span.
"""
from __future__ import annotations

import re
import string
from typing import Callable, Dict, Iterable, Iterator, Mapping, Sequence

import numpy as np


def rekey(example: Mapping, key_map: Mapping[str, str]) -> Dict:
  """{new_key: example[old_key]}; a falsy old key gives an empty string."""
  return {new: (example[old] if old else "") for new, old in key_map.items()}


def tokenize(example: Mapping, output_features: Mapping, copy_pretokenized: bool = True) -> Dict:
  out = dict(example)
  for k, feat in output_features.items():
    if k in example and isinstance(example[k], str):
      if copy_pretokenized:
        out[f"{k}_pretokenized"] = example[k]
      out[k] = np.asarray(feat.vocabulary.encode(example[k]), dtype=np.int32)
  return out


def append_eos_after_trim(example: Mapping, output_features: Mapping,
                          sequence_length: Mapping[str, int] = None) -> Dict:
  out = dict(example)
  for k, feat in output_features.items():
    if k not in out or not feat.add_eos:
      continue
    v = np.asarray(out[k])
    if sequence_length and k in sequence_length:
      v = v[:sequence_length[k] - 1]
    out[k] = np.concatenate([v, [feat.vocabulary.eos_id]]).astype(np.int32)
  return out


# ----------------------------------------------------------------------------
# Span corruption of real token streams
# ----------------------------------------------------------------------------
def random_spans_noise_mask(length: int, noise_density: float, mean_noise_span_length: float,
                            rng: np.random.Generator) -> np.ndarray:
  """Boolean mask over `length` tokens: alternating non-noise / noise spans, starting with
  non-noise, with the published T5 segment-length sampling."""
  orig = length
  length = max(length, 2)
  num_noise = int(round(length * noise_density))
  num_noise = min(max(num_noise, 1), length - 1)
  num_spans = max(int(round(num_noise / mean_noise_span_length)), 1)
  num_nonnoise = length - num_noise

  def segment(n_items, n_segments):
    first = np.zeros(n_items - 1, dtype=np.int64)
    first[:n_segments - 1] = 1
    rng.shuffle(first)
    seg = np.concatenate([[0], np.cumsum(first)])
    return np.bincount(seg, minlength=n_segments)

  noise = segment(num_noise, num_spans)
  nonnoise = segment(num_nonnoise, num_spans)
  lengths = np.stack([nonnoise, noise], axis=1).reshape(-1)
  starts = np.cumsum(lengths)[:-1]
  span_id = np.zeros(length, dtype=np.int64)
  span_id[starts] = 1
  span_id = np.cumsum(span_id)
  return (span_id % 2 == 1)[:orig]


def noise_span_to_unique_sentinel(tokens: np.ndarray, noise_mask: np.ndarray,
                                  vocab_size: int) -> np.ndarray:
  """Each run of noise tokens becomes one sentinel: vocab_size - 1, vocab_size - 2, ..."""
  prev = np.concatenate([[False], noise_mask[:-1]])
  first = noise_mask & ~prev
  subsequent = noise_mask & prev
  sentinel = vocab_size - np.cumsum(first)
  out = np.where(first, sentinel, tokens)
  return out[~subsequent]


def span_corruption_lengths(inputs_length: int, noise_density: float,
                            mean_noise_span_length: float):
  """(raw tokens to take, resulting targets length) such that corrupting that many tokens fills
  `inputs_length` inputs (sentinels and EOS included) as closely as possible."""
  def lengths(n):
    num_noise = int(round(n * noise_density))
    num_nonnoise = n - num_noise
    spans = int(round(num_noise / mean_noise_span_length))
    return num_nonnoise + spans + 1, num_noise + spans + 1

  n = inputs_length
  while lengths(n + 1)[0] <= inputs_length:
    n += 1
  return n, lengths(n)[1]


def span_corruption(token_stream: Iterable[np.ndarray], sequence_length: Mapping[str, int],
                    vocab_size: int, seed: int, noise_density: float = 0.15,
                    mean_noise_span_length: float = 3.0) -> Iterator[Dict[str, np.ndarray]]:
  """Concatenates the documents of `token_stream`, cuts the result into windows whose corrupted
  form fills sequence_length['inputs'], and corrupts each window (the `targets`-only pipeline
  of t5.data.preprocessors.span_corruption: select_random_chunk / reduce_concat_tokens /
  split_tokens / denoise, restated as one streaming pass)."""
  window, _ = span_corruption_lengths(sequence_length["inputs"], noise_density,
                                      mean_noise_span_length)
  buf = np.zeros(0, dtype=np.int64)
  index = 0
  for doc in token_stream:
    buf = np.concatenate([buf, np.asarray(doc, dtype=np.int64)])
    while len(buf) >= window:
      tokens, buf = buf[:window], buf[window:]
      rng = np.random.default_rng([seed, index])
      index += 1
      mask = random_spans_noise_mask(len(tokens), noise_density, mean_noise_span_length, rng)
      yield {"inputs": noise_span_to_unique_sentinel(tokens, mask, vocab_size).astype(np.int32),
             "targets": noise_span_to_unique_sentinel(tokens, ~mask, vocab_size).astype(np.int32)}


# ----------------------------------------------------------------------------
# Text-to-text formats and metrics of the fine-tuning tasks
# ----------------------------------------------------------------------------
def glue_text(example: Mapping, benchmark_name: str, label_names: Sequence[str],
              feature_names: Sequence[str]) -> Dict[str, str]:
  """'mnli hypothesis: ... premise: ...' -> label name (t5.data.glue_utils text format)."""
  parts = [benchmark_name]
  for f in feature_names:
    parts += [f"{f}:", str(example[f])]
  label = int(example.get("label", -1))
  return {"inputs": " ".join(parts),
          "targets": label_names[label] if 0 <= label < len(label_names) else "<unk>",
          "idx": example.get("idx", -1)}


def squad_text(example: Mapping, include_context: bool = True) -> Dict:
  """'question: ... context: ...' -> first answer; all answers kept for the metric."""
  def pad_punct(s):
    s = re.sub(r"'(.*?)'", r"\1", s)
    return re.sub(r"\s+", " ", s).strip()
  q, c = pad_punct(example["question"]), pad_punct(example["context"])
  answers = [pad_punct(a) for a in example["answers"]] or [""]
  inputs = f"question: {q} context: {c}" if include_context else f"squad trivia question: {q}"
  return {"inputs": inputs, "targets": answers[0], "answers": answers, "id": example.get("id")}


def string_label_to_class_id(string_label: str, label_classes: Sequence[str],
                             default: int = -1, **_) -> int:
  return list(label_classes).index(string_label) if string_label in label_classes else default


def accuracy(targets: Sequence, predictions: Sequence) -> Dict[str, float]:
  n = max(len(targets), 1)
  return {"accuracy": 100.0 * sum(int(t == p) for t, p in zip(targets, predictions)) / n}


def _normalize_answer(s: str) -> str:
  s = s.lower()
  s = "".join(ch for ch in s if ch not in set(string.punctuation))
  s = re.sub(r"\b(a|an|the)\b", " ", s)
  return " ".join(s.split())


def squad_metric(targets: Sequence[Sequence[str]], predictions: Sequence[str]) -> Dict[str, float]:
  """Exact match and token F1 against the best of each example's reference answers."""
  def f1(a, b):
    ta, tb = a.split(), b.split()
    common = sum(min(ta.count(w), tb.count(w)) for w in set(ta))
    if not common:
      return 0.0
    p, r = common / len(tb), common / len(ta)
    return 2 * p * r / (p + r)
  em = f1s = 0.0
  for refs, pred in zip(targets, predictions):
    refs = [refs] if isinstance(refs, str) else list(refs)
    p = _normalize_answer(pred)
    em += max(float(_normalize_answer(r) == p) for r in refs)
    f1s += max(f1(_normalize_answer(r), p) for r in refs)
  n = max(len(predictions), 1)
  return {"em": 100.0 * em / n, "f1": 100.0 * f1s / n}
