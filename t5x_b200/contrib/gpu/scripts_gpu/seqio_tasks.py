"""Tasks of the GPU launch scripts: The Pile span corruption, GLUE MNLI and SQuAD v1.1
(the registrations of t5x/contrib/gpu/scripts_gpu/seqio_tasks.py:53-85).

The reference reads these through TFDS builders; here each task reads plain files that the
user has placed in a directory (no network access, no TensorFlow):

  the_pile_span_corruption   $THE_PILE_DIR/{train,validation}/*.jsonl  ({"text": ...} per line,
                             The Pile's own format once decompressed) or *.txt (a document per
                             line); tokens are concatenated and span-corrupted on the fly.
  glue_mnli_v2               $GLUE_DIR/MNLI/{train,dev_matched}.tsv (the GLUE download) or
                             {train,validation}.jsonl with premise / hypothesis / label.
  squad_v010_allanswers      $SQUAD_DIR/{train,dev}-v1.1.json.

`register()` is called on import with directories from the environment; call it again with
explicit directories / vocabulary to override. A task whose files are missing is still
registered and raises a FileNotFoundError naming what it looked for when a dataset is built.
"""
from __future__ import annotations

import functools
import glob
import json
import os
from typing import Dict, Iterator, Mapping, Optional

from t5x_b200.data import preprocessors as prep
from t5x_b200.data import tasks as tasks_lib
from t5x_b200.data import vocabularies

DEFAULT_SPM = "vocabs/cc_all.32000.100extra/sentencepiece.model"
MNLI_LABELS = ("entailment", "neutral", "contradiction")


def default_vocabulary() -> vocabularies.Vocabulary:
  """The 32k SentencePiece model with 100 sentinel ids that the reference's GPU tasks use
  (`$T5X_B200_SPM_MODEL`, default `vocabs/cc_all.32000.100extra/sentencepiece.model`)."""
  return vocabularies.SentencePieceVocabulary(os.environ.get("T5X_B200_SPM_MODEL", DEFAULT_SPM))


def _shard(items, shard_info):
  return [x for i, x in enumerate(items) if i % shard_info.num_shards == shard_info.index]


def _need(paths, what):
  if not paths:
    raise FileNotFoundError(f"no data files found for {what}")
  return paths


# ---- The Pile ------------------------------------------------------------------------------
def _pile_documents(data_dir: str, split: str, shard_info) -> Iterator[str]:
  base = os.path.join(data_dir, split)
  files = sorted(glob.glob(os.path.join(base, "*.jsonl")) + glob.glob(os.path.join(base, "*.txt")))
  _need(files, f"the_pile_span_corruption ({base}/*.jsonl or *.txt; set THE_PILE_DIR)")
  # whole files per shard when there are enough of them, else lines round-robin
  by_file = len(files) >= shard_info.num_shards
  mine = _shard(files, shard_info) if by_file else files
  for path in mine:
    with open(path, encoding="utf-8") as f:
      for i, line in enumerate(f):
        if not by_file and i % shard_info.num_shards != shard_info.index:
          continue
        line = line.strip()
        if not line:
          continue
        yield json.loads(line)["text"] if path.endswith(".jsonl") else line


def _pile_source(data_dir, vocab, split, shard_info, seed, sequence_length=None, **_):
  sl = sequence_length or {"inputs": 512, "targets": 128}

  def token_docs():
    epoch = 0
    while True:
      n = 0
      for text in _pile_documents(data_dir, split, shard_info):
        n += 1
        yield vocab.encode(text)
      if split != "train" or n == 0:
        return
      epoch += 1

  feats = {"inputs": tasks_lib.Feature(vocab), "targets": tasks_lib.Feature(vocab)}
  for ex in prep.span_corruption(token_docs(), sl, vocab.vocab_size, seed):
    yield prep.append_eos_after_trim(ex, feats, sl)


# ---- GLUE MNLI ------------------------------------------------------------------------------
def _mnli_rows(data_dir: str, split: str) -> Iterator[Dict]:
  base = os.path.join(data_dir, "MNLI")
  jsonl = os.path.join(base, f"{split}.jsonl")
  tsv = os.path.join(base, {"train": "train.tsv", "validation": "dev_matched.tsv",
                            "validation_matched": "dev_matched.tsv",
                            "validation_mismatched": "dev_mismatched.tsv"}.get(split, split))
  if os.path.exists(jsonl):
    with open(jsonl, encoding="utf-8") as f:
      for i, line in enumerate(f):
        row = json.loads(line)
        label = row["label"]
        if isinstance(label, str):
          label = MNLI_LABELS.index(label) if label in MNLI_LABELS else -1
        yield {"premise": row["premise"], "hypothesis": row["hypothesis"], "label": label,
               "idx": row.get("idx", i)}
    return
  if not os.path.exists(tsv):
    raise FileNotFoundError(f"no data files found for glue_mnli_v2 ({jsonl} or {tsv}; set GLUE_DIR)")
  with open(tsv, encoding="utf-8") as f:
    header = f.readline().rstrip("\n").split("\t")
    col = {name: i for i, name in enumerate(header)}
    for i, line in enumerate(f):
      parts = line.rstrip("\n").split("\t")
      label = parts[col["gold_label"]] if "gold_label" in col else ""
      yield {"premise": parts[col["sentence1"]], "hypothesis": parts[col["sentence2"]],
             "label": MNLI_LABELS.index(label) if label in MNLI_LABELS else -1,
             "idx": int(parts[col["index"]]) if "index" in col else i}


def _text_to_features(text_ex: Mapping, vocab, sl) -> Dict:
  feats = {"inputs": tasks_lib.Feature(vocab), "targets": tasks_lib.Feature(vocab)}
  ex = prep.tokenize(text_ex, feats)
  return prep.append_eos_after_trim(ex, feats, sl)


def _mnli_source(data_dir, vocab, split, shard_info, seed, sequence_length=None, **_):
  for i, row in enumerate(_mnli_rows(data_dir, split)):
    if i % shard_info.num_shards != shard_info.index:
      continue
    text = prep.glue_text(row, "mnli", MNLI_LABELS, ("hypothesis", "premise"))
    yield _text_to_features(text, vocab, sequence_length)


# ---- SQuAD v1.1 -----------------------------------------------------------------------------
def _squad_rows(data_dir: str, split: str) -> Iterator[Dict]:
  name = {"train": "train-v1.1.json", "validation": "dev-v1.1.json"}.get(split, split)
  path = os.path.join(data_dir, name)
  if not os.path.exists(path):
    raise FileNotFoundError(f"no data files found for squad_v010_allanswers ({path}; set "
                            "SQUAD_DIR)")
  with open(path, encoding="utf-8") as f:
    data = json.load(f)["data"]
  for article in data:
    for para in article["paragraphs"]:
      for qa in para["qas"]:
        yield {"id": qa["id"], "question": qa["question"], "context": para["context"],
               "answers": [a["text"] for a in qa["answers"]]}


def _squad_source(data_dir, vocab, split, shard_info, seed, sequence_length=None, **_):
  for i, row in enumerate(_squad_rows(data_dir, split)):
    if i % shard_info.num_shards != shard_info.index:
      continue
    yield _text_to_features(prep.squad_text(row), vocab, sequence_length)


def _squad_postprocess(answer, example=None, is_target=False):
  if is_target and example is not None:
    return [a for a in example["answers"]]
  return answer


def _mnli_postprocess(string_label, example=None, is_target=False):
  return prep.string_label_to_class_id(string_label, MNLI_LABELS)


def register(vocabulary: Optional[vocabularies.Vocabulary] = None,
             data_dirs: Optional[Mapping[str, str]] = None) -> None:
  """(Re-)registers the three tasks. `data_dirs`: {'the_pile', 'glue', 'squad'} -> directory;
  defaults come from $THE_PILE_DIR, $GLUE_DIR, $SQUAD_DIR."""
  dirs = {"the_pile": os.environ.get("THE_PILE_DIR", "the_pile"),
          "glue": os.environ.get("GLUE_DIR", "glue"),
          "squad": os.environ.get("SQUAD_DIR", "squad")}
  dirs.update(data_dirs or {})

  class _LazyVocab:
    """Loads the SentencePiece model on first use, so that importing this module never needs
    the model file."""
    _v = vocabulary

    def __getattr__(self, name):
      if _LazyVocab._v is None:
        _LazyVocab._v = default_vocabulary()
      return getattr(_LazyVocab._v, name)

  vocab = vocabulary if vocabulary is not None else _LazyVocab()
  feats = {"inputs": tasks_lib.Feature(vocab, required=False), "targets": tasks_lib.Feature(vocab)}
  reg = tasks_lib.TaskRegistry
  for name in ("the_pile_span_corruption", "glue_mnli_v2", "squad_v010_allanswers"):
    reg.remove(name)
  reg.add("the_pile_span_corruption",
          functools.partial(_pile_source, dirs["the_pile"], vocab), feats, metric_fns=[],
          splits=("train", "validation"))
  reg.add("glue_mnli_v2", functools.partial(_mnli_source, dirs["glue"], vocab), feats,
          metric_fns=[prep.accuracy], postprocess_fn=_mnli_postprocess,
          splits=("train", "validation", "validation_matched", "validation_mismatched"))
  reg.add("squad_v010_allanswers", functools.partial(_squad_source, dirs["squad"], vocab), feats,
          metric_fns=[prep.squad_metric], postprocess_fn=_squad_postprocess,
          splits=("train", "validation"))


register()
