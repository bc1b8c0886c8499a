"""Helpers of the inference script: the fail-fast writer pool, ad-hoc tasks over text / JSONL
files, chunk merging and the JSONL writer in its three modes (t5x/infer.py:66-325)."""
import json
import os
import time

import numpy as np
import pytest

from t5x_b200 import infer
from t5x_b200.data import seqio_api as seqio
from t5x_b200.data import vocabularies


def test_fail_fast_pool_raises_an_earlier_failure_at_the_next_submit():
  pool = infer.FailFastThreadPoolExecutor(max_workers=1)

  def boom():
    raise RuntimeError("disk full")

  pool.submit(boom)
  time.sleep(0.05)
  with pytest.raises(RuntimeError, match="disk full"):
    pool.submit(lambda: 1)
  pool2 = infer.FailFastThreadPoolExecutor(max_workers=1)
  pool2.submit(boom)
  with pytest.raises(RuntimeError, match="disk full"):
    pool2.shutdown(wait=True)
  ok = infer.FailFastThreadPoolExecutor(max_workers=2)
  futs = [ok.submit(lambda i=i: i * i) for i in range(4)]
  ok.shutdown(wait=True)
  assert [f.result() for f in futs] == [0, 1, 4, 9]


def _features():
  vocab = vocabularies.ByteVocabulary()
  return {"inputs": seqio.Feature(vocab, add_eos=True), "targets": seqio.Feature(vocab, add_eos=True)}


def test_task_from_jsonl_and_text_files(tmp_path):
  jl = tmp_path / "data.jsonl"
  jl.write_text("\n".join(json.dumps({"q": f"question {i}", "a": f"answer {i}"})
                          for i in range(5)) + "\n\n")
  name = infer.create_task_from_tfexample_file([str(jl)], "jsonl", "q", "a", _features(),
                                               task_id="unit_jsonl")
  assert name == "infer_unit_jsonl"
  task = seqio.get_mixture_or_task(name)
  rows = list(task._source("infer"))
  assert [r["inputs_pretokenized"] for r in rows] == [f"question {i}" for i in range(5)]
  assert rows[2]["targets_pretokenized"] == "answer 2"
  vocab = _features()["inputs"].vocabulary
  assert rows[0]["inputs"][-1] == vocab.eos_id
  assert vocab.decode([int(t) for t in rows[0]["inputs"][:-1]]) == "question 0"
  # shards deal lines round-robin
  shard = list(task._source("infer", shard_info=seqio.ShardInfo(index=1, num_shards=2)))
  assert [r["inputs_pretokenized"] for r in shard] == ["question 1", "question 3"]
  txt = tmp_path / "plain.txt"
  txt.write_text("first line\nsecond line\n")
  name = infer.create_task_from_tfexample_file([str(txt)], "text", "inputs", None, _features(),
                                               task_id="unit_text")
  rows = list(seqio.get_mixture_or_task(name)._source("infer"))
  assert [r["inputs_pretokenized"] for r in rows] == ["first line", "second line"]
  assert "targets" not in rows[0]
  # a stable name derived from the arguments when no id is given
  a = infer.create_task_from_tfexample_file([str(txt)], "text", "inputs", None, _features())
  b = infer.create_task_from_tfexample_file([str(txt)], "text", "inputs", None, _features())
  assert a == b and a.startswith("infer_")
  with pytest.raises(ValueError, match="Missing or invalid paths"):
    infer.create_task_from_tfexample_file([str(tmp_path / "none*")], "text", "inputs", None,
                                          _features())
  with pytest.raises(ValueError, match="Unsupported file_type"):
    infer.create_task_from_tfexample_file([str(txt)], "tfrecord", "inputs", None, _features())


def test_merge_chunks(tmp_path):
  tmp = tmp_path / "tmp"
  tmp.mkdir()
  for i, text in enumerate(["a\n", "b\nc\n", "d\n"]):
    (tmp / f"out.jsonl-chunk{i:05d}").write_text(text)
  infer.merge_chunks_to_file(str(tmp_path), "out.jsonl", str(tmp), step=None)
  assert (tmp_path / "out.jsonl").read_text() == "a\nb\nc\nd\n"
  os.remove(tmp / "out.jsonl-chunk00001")
  with pytest.raises(AssertionError, match="Expecting 3 chunk paths, found 2"):
    infer.merge_chunks_to_file(str(tmp_path), "out.jsonl", str(tmp), step=None)
  with pytest.raises(FileNotFoundError, match="No chunk results"):
    infer.merge_chunks_to_file(str(tmp_path), "other.jsonl", str(tmp), step=None)


def test_write_inferences_in_every_mode(tmp_path):
  vocab = vocabularies.ByteVocabulary()
  ds = [{"inputs_pretokenized": "hello", "inputs": np.array([1, 2]), "targets_pretokenized": b"x"},
        {"inputs_pretokenized": "world", "inputs": np.array([3]), "targets_pretokenized": b"y"}]
  preds = [np.array(vocab.encode("hi") + [1, 0, 0]), np.array(vocab.encode("yo") + [1, 0, 0])]
  path = str(tmp_path / "p.jsonl")
  infer.write_inferences_to_file(path, (preds, {}), ds, "predict", vocabulary=vocab,
                                 output_ids=True)
  rows = [json.loads(l) for l in open(path)]
  assert [r["prediction"] for r in rows] == ["hi", "yo"]
  assert rows[0]["inputs"] == {"inputs_pretokenized": "hello", "targets_pretokenized": "x"}
  assert rows[0]["prediction_tokens"] == vocab.encode("hi") + [1]      # cut at the padding
  aux = {"scores": np.array([-1.5, -2.5]), "nested": {"n": np.array([[1, 2], [3, 4]])}}
  infer.write_inferences_to_file(path, (preds, aux), ds, "predict_with_aux", vocabulary=vocab,
                                 input_fields_to_include=["inputs"])
  rows = [json.loads(l) for l in open(path)]
  assert rows[1]["aux"] == {"scores": -2.5, "nested": {"n": [3, 4]}}
  assert set(rows[1]["inputs"]) == {"inputs", "inputs_pretokenized"}
  infer.write_inferences_to_file(path, ([np.float32(-3.25), np.float32(-0.5)], {}), ds, "score",
                                 include_all_inputs=True)
  rows = [json.loads(l) for l in open(path)]
  assert [r["score"] for r in rows] == [-3.25, -0.5] and "aux" not in rows[0]
  assert rows[0]["inputs"]["inputs"] == [1, 2]
  with pytest.raises(ValueError, match="vocabulary"):
    infer.write_inferences_to_file(path, (preds, {}), ds, "predict")
  with pytest.raises(ValueError, match="simultaneously"):
    infer.write_inferences_to_file(path, (preds, {}), ds, "score", include_all_inputs=True,
                                   input_fields_to_include=["inputs"])
  with pytest.raises(ValueError, match="Invalid mode"):
    infer.write_inferences_to_file(path, (preds, {}), ds, "rank", vocabulary=vocab)
