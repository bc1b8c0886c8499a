"""The checkpointable dataset abstraction: combinators, exact resume positions through every
combinator, peeking, saved / restored iterators and the prefetch thread."""
import numpy as np
import pytest

from t5x_b200.data import dataset as ds_lib
from t5x_b200.data import feature_converters as fc


def _numbers(n=10):
  return ds_lib.Dataset.from_examples([{"x": np.array([i]), "y": np.array(i * 10)} for i in range(n)])


def _xs(ds, start=0):
  return [int(np.asarray(e["x"]).reshape(-1)[0]) for e in ds._make(start)]


def test_basic_combinators():
  ds = _numbers()
  assert len(ds) == 10 and ds.cardinality() == 10
  assert _xs(ds.map(lambda e: {**e, "x": e["x"] + 100})) == list(range(100, 110))
  assert _xs(ds.take(3)) == [0, 1, 2] and len(ds.take(3)) == 3 and len(ds.take(99)) == 10
  assert _xs(ds.skip(7)) == [7, 8, 9] and len(ds.skip(7)) == 3
  assert _xs(ds.shard(3, 1)) == [1, 4, 7] and len(ds.shard(3, 1)) == 3 and len(ds.shard(3, 0)) == 4
  pairs = list(ds.enumerate()._make(0))
  assert [i for i, _ in pairs] == list(range(10)) and int(pairs[4][1]["y"]) == 40
  rep = ds.take(3).repeat()
  it = rep._make(0)
  assert [int(next(it)["x"][0]) for _ in range(8)] == [0, 1, 2, 0, 1, 2, 0, 1]
  with pytest.raises(TypeError, match="unknown"):
    len(rep)
  assert rep.repeat() is rep


def test_batches_and_specs():
  ds = _numbers()
  b = ds.batch(4)
  assert len(b) == 2
  rows = list(b._make(0))
  assert rows[0]["x"].shape == (4, 1) and rows[1]["y"].tolist() == [40, 50, 60, 70]
  padded = ds.padded_batch(4)
  assert len(padded) == 3 and list(padded._make(0))[-1]["x"].shape == (2, 1)
  spec = b.element_spec
  assert spec["x"].shape == (4, 1) and spec["y"].shape == (4,)
  text = ds_lib.Dataset.from_examples([{"t": "ab"}, {"t": "c"}]).batch(2)
  assert list(text._make(0))[0]["t"].tolist() == ["ab", "c"]
  gen = ds_lib.Dataset.from_generator_fn(lambda: ({"x": np.array([i])} for i in range(5)), 5)
  assert _xs(gen, start=2) == [2, 3, 4]


def test_every_combinator_resumes_at_an_exact_position():
  ds = _numbers(20)
  pipelines = {
      "map": ds.map(lambda e: e),
      "skip": ds.skip(3),
      "shard": ds.shard(2, 1),
      "take": ds.take(15),
      "batch": ds.batch(3),
      "shard+batch": ds.shard(2, 0).batch(2),
      "repeat": ds.take(4).repeat().take(11),
  }
  for name, p in pipelines.items():
    full = list(p._make(0))
    for start in (0, 1, 2, 5):
      resumed = list(p._make(start))
      assert len(resumed) == max(0, len(full) - start), name
      for a, b in zip(resumed, full[start:]):
        np.testing.assert_array_equal(a["x"], b["x"], err_msg=f"{name} from {start}")


def test_iterator_position_peek_save_and_restore(tmp_path):
  it = iter(_numbers().batch(2))
  assert next(it)["x"].reshape(-1).tolist() == [0, 1]
  assert it.peek()["x"].reshape(-1).tolist() == [2, 3]
  assert it.peek()["x"].reshape(-1).tolist() == [2, 3]          # peeking does not advance
  assert it.peek_async().result()["x"].reshape(-1).tolist() == [2, 3]
  assert it.get_state() == {"index": 1}
  assert next(it)["x"].reshape(-1).tolist() == [2, 3]
  path = str(tmp_path / "ckpt" / "train_ds-000-of-001")
  it.save(path)
  assert next(it)["x"].reshape(-1).tolist() == [4, 5]
  other = iter(_numbers().batch(2))
  other.restore(path)
  assert next(other)["x"].reshape(-1).tolist() == [4, 5]
  other.set_state({"index": 4})
  assert next(other)["x"].reshape(-1).tolist() == [8, 9]
  with pytest.raises(StopIteration):
    next(other)
  other.reset()
  assert next(other)["x"].reshape(-1).tolist() == [0, 1]
  assert it.element_spec["x"].shape == (2, 1)


def test_conversion_keeps_positions_and_packing_recounts_rows():
  examples = [{"inputs": [5, 6, 1], "targets": [7, 1]} for _ in range(6)]
  ds = ds_lib.Dataset.from_examples(examples)
  lengths = {"inputs": 8, "targets": 6}
  unpacked = ds.convert(fc.EncDecFeatureConverter(pack=False), lengths)
  assert len(unpacked) == 6 and len(list(unpacked._make(4))) == 2
  packed = ds.convert(fc.EncDecFeatureConverter(pack=True), lengths)
  rows = list(packed._make(0))
  assert len(rows) == 3                                   # two examples fit one row
  assert packed.cardinality() is None
  assert len(list(packed._make(1))) == 2                  # positions count packed rows
  assert rows[0]["encoder_segment_ids"].tolist() == [1, 1, 1, 2, 2, 2, 0, 0]


def test_prefetch_thread_keeps_order_and_surfaces_errors():
  out = list(ds_lib.PrefetchIterator(iter(range(20)), depth=3, transform=lambda v: v * 2))
  assert out == [2 * i for i in range(20)]

  def broken():
    yield 1
    raise ValueError("bad shard")

  it = ds_lib.PrefetchIterator(broken(), depth=2)
  assert next(it) == 1
  with pytest.raises(ValueError, match="bad shard"):
    next(it)
