"""Bitwise binary search and the top-k / top-p masks: the contracts of t5x/binary_search.py
(predicate False up to a threshold and True above it; the search returns the largest value
on the False side), on fixed cases and on generated ones."""
import math

import numpy as np
import pytest
import torch
from hypothesis import given, settings, strategies as st

from t5x_b200 import binary_search

INT32_MIN, INT32_MAX = -(2 ** 31), 2 ** 31 - 1


def test_int32_bsearch_recovers_thresholds_at_the_edges_of_the_range():
  a = torch.tensor([1, 43, 79, 2048, 0, 2047, -1, INT32_MIN, INT32_MIN + 1, INT32_MAX,
                    INT32_MAX - 1], dtype=torch.int32)
  got = binary_search.int32_bsearch(a.shape, lambda x: x > a)
  assert got.dtype == torch.int32
  torch.testing.assert_close(got, a, rtol=0, atol=0)


def test_int32_bsearch_constant_predicates():
  always_false = binary_search.int32_bsearch((1,), lambda x: torch.zeros_like(x, dtype=torch.bool))
  assert always_false.tolist() == [INT32_MAX]
  always_true = binary_search.int32_bsearch((1,), lambda x: torch.ones_like(x, dtype=torch.bool))
  assert always_true.tolist() == [INT32_MIN]


@settings(max_examples=50, deadline=None)
@given(st.lists(st.integers(INT32_MIN, INT32_MAX), min_size=1, max_size=6))
def test_int32_bsearch_any_threshold(values):
  a = torch.tensor(values, dtype=torch.int32).view(1, -1)
  calls = []

  def predicate(x):
    calls.append(1)
    assert x.shape == a.shape and x.dtype == torch.int32
    return x > a

  torch.testing.assert_close(binary_search.int32_bsearch(a.shape, predicate), a, rtol=0, atol=0)
  assert len(calls) == 32  # one probe per bit


def test_float32_bsearch_recovers_thresholds():
  tiny = float(np.finfo(np.float32).tiny)
  a = torch.tensor([1.0, -1.0, 0.0, 43.5, -79.25, 3.0e38, -3.0e38, tiny, -tiny, tiny / 4,
                    1e-30, -1e-30, math.pi], dtype=torch.float32)
  got = binary_search.float32_bsearch(a.shape, lambda x: x > a)
  assert got.dtype == torch.float32
  torch.testing.assert_close(got, a, rtol=0, atol=0)


def test_float32_order_mapping_is_monotone_and_invertible():
  g = torch.Generator().manual_seed(0)
  bits = torch.randint(INT32_MIN, INT32_MAX, (4096,), generator=g, dtype=torch.int64).to(torch.int32)
  x = bits.view(torch.float32)
  x = x[torch.isfinite(x)]
  i = binary_search._monotonic_float32_to_int32(x)
  back = binary_search._monotonic_int32_to_float32(i)
  assert torch.equal(back.view(torch.int32), x.view(torch.int32))
  order = torch.argsort(i.to(torch.int64))
  xs = x[order].double()
  assert bool((xs[1:] >= xs[:-1]).all())


@settings(max_examples=40, deadline=None)
@given(st.lists(st.floats(width=32, allow_nan=False, allow_infinity=False), min_size=1, max_size=5))
def test_float32_bsearch_any_finite_threshold(values):
  a = torch.tensor(values, dtype=torch.float32)
  got = binary_search.float32_bsearch(a.shape, lambda x: x > a)
  # -0.0 and +0.0 compare equal: the search lands on the larger bit pattern, +0.0
  torch.testing.assert_close(got, a, rtol=0, atol=0)
  zero = a == 0
  assert not bool(torch.signbit(got[zero]).any())


def test_topk_mask_fixed_cases():
  mask = -1e10
  x = torch.tensor([[1.4, 7.9, -4.3, 100, 71, 6, -1e4],
                    [8.3, 1.2, 1.3, 1.2, 1.2, 9.7, -100]])
  m = mask
  np.testing.assert_array_equal(
      binary_search.topk_mask(x, 1, mask).numpy(),
      np.asarray([[m, m, m, 100, m, m, m], [m, m, m, m, m, 9.7, m]], np.float32))
  np.testing.assert_array_equal(
      binary_search.topk_mask(x, 2, mask).numpy(),
      np.asarray([[m, m, m, 100, 71, m, m], [8.3, m, m, m, m, 9.7, m]], np.float32))
  np.testing.assert_array_equal(
      binary_search.topk_mask(x, 3, mask).numpy(),
      np.asarray([[m, 7.9, m, 100, 71, m, m], [8.3, m, 1.3, m, m, 9.7, m]], np.float32))
  # the 4th largest of the second row is tied three ways: all of the tie is kept
  np.testing.assert_array_equal(
      binary_search.topk_mask(x, 4, mask).numpy(),
      np.asarray([[m, 7.9, m, 100, 71, 6, m], [8.3, 1.2, 1.3, 1.2, 1.2, 9.7, m]], np.float32))
  np.testing.assert_array_equal(binary_search.topk_mask(x, 7, mask).numpy(), x.numpy())
  np.testing.assert_array_equal(binary_search.topk_mask(x, 100, mask).numpy(), x.numpy())


@settings(max_examples=40, deadline=None)
@given(st.integers(1, 12), st.integers(1, 12), st.integers(0, 2 ** 31 - 1))
def test_topk_mask_against_a_sort(n, k, seed):
  g = torch.Generator().manual_seed(seed)
  # few distinct values, so that ties at the cutoff are common
  x = torch.randint(-3, 4, (3, n), generator=g).float()
  got = binary_search.topk_mask(x, k, -1e10)
  for row, out in zip(x, got):
    kth = torch.sort(row, descending=True).values[min(k, n) - 1]
    want = torch.where(row >= kth, row, torch.full_like(row, -1e10))
    assert torch.equal(out, want)
    assert int((out > -1e9).sum()) >= min(k, n)


def test_topp_mask_fixed_cases():
  probs = torch.tensor([[0.0, 0.7, 0.04, 0.06, 0.2, 0.0],
                        [0.0, 0.2, 0.2, 0.2, 0.3, 0.1]])
  logits = torch.log(probs)
  m = -1e10

  def kept(p):
    out = binary_search.topp_mask(logits, p, m)
    # masking only: the survivors are bit-identical to the input
    assert torch.equal(out[out > -1e9], logits[out > -1e9])
    return (out > -1e9).int().tolist()

  assert kept(0.1) == [[0, 1, 0, 0, 0, 0], [0, 0, 0, 0, 1, 0]]
  assert kept(0.3) == [[0, 1, 0, 0, 0, 0], [0, 0, 0, 0, 1, 0]]
  assert kept(0.4) == [[0, 1, 0, 0, 0, 0], [0, 1, 1, 1, 1, 0]]   # the tie at 0.2 is kept whole
  assert kept(0.8) == [[0, 1, 0, 0, 1, 0], [0, 1, 1, 1, 1, 0]]
  assert kept(0.95) == [[0, 1, 0, 1, 1, 0], [0, 1, 1, 1, 1, 1]]
  # per-row thresholds
  out = binary_search.topp_mask(logits, torch.tensor([0.8, 0.1]), m)
  assert (out > -1e9).int().tolist() == [[0, 1, 0, 0, 1, 0], [0, 0, 0, 0, 1, 0]]


@settings(max_examples=40, deadline=None)
@given(st.integers(2, 16), st.floats(0.01, 0.99), st.integers(0, 2 ** 31 - 1))
def test_topp_mask_keeps_the_smallest_sufficient_set(n, p, seed):
  g = torch.Generator().manual_seed(seed)
  logits = torch.randn(2, n, generator=g) * 2
  out = binary_search.topp_mask(logits, p, -1e10)
  probs = torch.softmax(logits.double(), -1)
  for row_p, row_out in zip(probs, out):
    keep = row_out > -1e9
    mass = float(row_p[keep].sum())
    assert mass >= p - 1e-5
    # dropping the least likely survivor must fall below p: nothing superfluous is kept
    smallest = float(row_p[keep].min())
    assert mass - smallest < p + 1e-5
    # survivors are exactly the most likely entries
    assert float(row_p[keep].min()) >= float(row_p[~keep].max()) if bool((~keep).any()) else True
