"""File-backed tasks of the GPU launch scripts (The Pile span corruption, GLUE MNLI, SQuAD) on
small files written by the test, with a byte vocabulary."""
import json
import os

import numpy as np
import pytest

from t5x_b200.data import preprocessors as prep
from t5x_b200.data import tasks as tasks_lib
from t5x_b200.data import vocabularies
from t5x_b200.data.dataset import ShardInfo


def test_span_corruption_of_a_token_stream_is_invertible_and_fills_the_inputs():
  vocab_size, sl = 1000, {"inputs": 64, "targets": 32}
  rng = np.random.default_rng(0)
  docs = [rng.integers(3, 900, size=n) for n in (50, 7, 300, 120)]
  window, tgt_len = prep.span_corruption_lengths(64, 0.15, 3.0)
  stream = np.concatenate(docs)
  examples = list(prep.span_corruption(iter(docs), sl, vocab_size, seed=3))
  assert len(examples) == len(stream) // window
  for n, ex in enumerate(examples):
    inp, tgt = ex["inputs"], ex["targets"]
    assert len(inp) + 1 <= 64 and len(tgt) + 1 <= max(tgt_len, 32) + 4
    # sentinels count down from the top of the vocabulary, the same ones on both sides
    s_in = [t for t in inp if t >= 900]
    s_tg = [t for t in tgt if t >= 900]
    assert s_in[0] == vocab_size - 1 and s_in == sorted(s_in, reverse=True)
    assert len(s_tg) in (len(s_in), len(s_in) + 1, len(s_in) - 1)
    # splicing the target spans back into the inputs restores the window
    spans, cur = {}, None
    for t in tgt:
      if t >= 900:
        cur = t
        spans[cur] = []
      else:
        spans[cur].append(t)
    rebuilt = []
    for t in inp:
      rebuilt.extend(spans.get(t, [])) if t >= 900 else rebuilt.append(t)
    # inputs may start or end with a non-noise span the targets mark with a trailing sentinel
    assert rebuilt == stream[n * window:(n + 1) * window].tolist()
    noise = sum(len(v) for v in spans.values())
    assert abs(noise / window - 0.15) < 0.03


@pytest.fixture
def contrib_tasks(tmp_path):
  pile = tmp_path / "pile" / "train"
  pile.mkdir(parents=True)
  with open(pile / "00.jsonl", "w") as f:
    for i in range(40):
      f.write(json.dumps({"text": f"document {i} " + "lorem ipsum dolor sit amet " * 12}) + "\n")
  mnli = tmp_path / "glue" / "MNLI"
  mnli.mkdir(parents=True)
  with open(mnli / "dev_matched.tsv", "w") as f:
    f.write("index\tpromptID\tsentence1\tsentence2\tgold_label\n")
    f.write("0\t1\tA man eats.\tSomebody eats.\tentailment\n")
    f.write("1\t2\tA man eats.\tNobody eats.\tcontradiction\n")
  squad = tmp_path / "squad"
  squad.mkdir()
  with open(squad / "dev-v1.1.json", "w") as f:
    json.dump({"data": [{"paragraphs": [{"context": "The tower is 'tall' and old.", "qas": [
        {"id": "q1", "question": "How is the tower?",
         "answers": [{"text": "tall"}, {"text": "tall and old"}]}]}]}]}, f)
  from t5x_b200.contrib.gpu.scripts_gpu import seqio_tasks
  seqio_tasks.register(vocabulary=vocabularies.ByteVocabulary(extra_ids=100),
                       data_dirs={"the_pile": str(tmp_path / "pile"),
                                  "glue": str(tmp_path / "glue"), "squad": str(squad)})
  yield seqio_tasks
  seqio_tasks.register()


def test_pile_mnli_and_squad_tasks_read_plain_files(contrib_tasks):
  vocab = vocabularies.ByteVocabulary(extra_ids=100)
  pile = tasks_lib.TaskRegistry.get("the_pile_span_corruption")
  sl = {"inputs": 128, "targets": 64}
  it = iter(pile.get_dataset(sl, split="train", seed=1, shard_info=ShardInfo(0, 2),
                             num_epochs=None))
  first = [next(it) for _ in range(3)]
  for ex in first:
    assert ex["inputs"][-1] == vocab.eos_id and len(ex["inputs"]) <= 128
    assert max(ex["inputs"]) >= vocab.vocab_size - 100  # sentinels from the top of the vocab
  mnli = tasks_lib.TaskRegistry.get("glue_mnli_v2")
  rows = list(mnli.get_dataset({"inputs": 256, "targets": 16}, split="validation"))
  assert vocab.decode(rows[0]["inputs"][:-1]) == \
      "mnli hypothesis: Somebody eats. premise: A man eats."
  assert vocab.decode(rows[1]["targets"][:-1]) == "contradiction"
  assert mnli.postprocess("contradiction") == 2 and mnli.postprocess("gibberish") == -1
  assert mnli.metric_fns[0]([0, 2], [0, 1]) == {"accuracy": 50.0}
  squad = tasks_lib.TaskRegistry.get("squad_v010_allanswers")
  ex = next(iter(squad.get_dataset({"inputs": 256, "targets": 32}, split="validation")))
  assert vocab.decode(ex["inputs"][:-1]) == \
      "question: How is the tower? context: The tower is tall and old."
  assert vocab.decode(ex["targets"][:-1]) == "tall"
  m = squad.metric_fns[0]([["tall", "tall and old"]], ["The tall"])
  assert m["em"] == 100.0 and m["f1"] == 100.0
  with pytest.raises(FileNotFoundError, match="THE_PILE_DIR"):
    next(iter(pile.get_dataset(sl, split="validation")))
