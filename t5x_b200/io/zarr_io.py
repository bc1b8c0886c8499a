"""zarr v2 directory arrays, laid out as TensorStore's `zarr` driver writes them.

  <dir>/.zarray   JSON: zarr_format 2, shape, chunks, dtype ('<f4', 'bfloat16', ...),
                  compressor ({'id':'gzip','level':N} | {'id':'zstd',...} | null), fill_value,
                  order 'C', filters null, dimension_separator '.'
  <dir>/i.j.k     one file per chunk: the compressed C-order bytes of a FULL chunk (edge chunks
                  are padded with the fill value)

Writers emit gzip; readers also accept zstd (decoded through pyarrow's codec) and
uncompressed chunks. Region writes that cover whole chunks never read the old chunk, so ranks
that own disjoint chunk-aligned slices can write one array concurrently.
"""
from __future__ import annotations

import gzip
import io
import itertools
import json
import os
import zlib
from typing import Any, Dict, Optional, Sequence, Tuple

import numpy as np


def _np_dtype(name: str) -> np.dtype:
  if name in ("bfloat16", "<V2:bfloat16"):
    import ml_dtypes
    return np.dtype(ml_dtypes.bfloat16)
  return np.dtype(name)


def dtype_to_zarr(dtype: np.dtype) -> str:
  dtype = np.dtype(dtype)
  if dtype.name == "bfloat16":
    return "bfloat16"
  return dtype.str if dtype.itemsize > 1 else dtype.str.replace("<", "|").replace(">", "|")


def dtype_name(dtype) -> str:
  return np.dtype(dtype).name


class ZarrArray:
  """One zarr v2 array on the local filesystem."""

  def __init__(self, path: str, meta: Dict[str, Any]):
    self.path = path
    self.meta = meta
    self.shape = tuple(int(s) for s in meta["shape"])
    self.chunks = tuple(int(c) for c in meta["chunks"]) if self.shape else ()
    self.dtype = _np_dtype(meta["dtype"])
    self.compressor = meta.get("compressor")
    self.fill_value = meta.get("fill_value")
    self.sep = meta.get("dimension_separator", ".")
    if meta.get("order", "C") != "C":
      raise NotImplementedError("only C-order zarr arrays are supported")
    if meta.get("filters"):
      raise NotImplementedError("zarr filters are not supported")

  # -- creation / opening -----------------------------------------------------------------
  @classmethod
  def create(cls, path: str, shape: Sequence[int], chunks: Sequence[int], dtype,
             compressor: Optional[Dict[str, Any]] = None, exist_ok: bool = True) -> "ZarrArray":
    os.makedirs(path, exist_ok=True)
    comp = compressor if compressor is None else dict(compressor)
    if comp is not None and comp.get("id") == "gzip":
      comp.setdefault("level", 6)
    meta = {
        "chunks": [int(c) for c in chunks], "compressor": comp, "dtype": dtype_to_zarr(dtype),
        "fill_value": None, "filters": None, "order": "C", "shape": [int(s) for s in shape],
        "zarr_format": 2, "dimension_separator": ".",
    }
    zpath = os.path.join(path, ".zarray")
    if os.path.exists(zpath) and exist_ok:
      with open(zpath) as f:
        old = json.load(f)
      if old["shape"] != meta["shape"] or old["chunks"] != meta["chunks"] or \
          old["dtype"] != meta["dtype"]:
        raise ValueError(f"existing zarr array at {path} has different metadata")
      return cls(path, old)
    tmp = zpath + f".tmp{os.getpid()}"
    with open(tmp, "w") as f:
      json.dump(meta, f, indent=1)
    os.replace(tmp, zpath)
    return cls(path, meta)

  @classmethod
  def open(cls, path: str) -> "ZarrArray":
    zpath = os.path.join(path, ".zarray")
    if not os.path.exists(zpath):
      raise FileNotFoundError(f"no zarr array at {path}")
    with open(zpath) as f:
      return cls(path, json.load(f))

  # -- codec ------------------------------------------------------------------------------
  def _encode(self, raw: bytes) -> bytes:
    c = self.compressor
    if c is None:
      return raw
    if c["id"] == "gzip":
      buf = io.BytesIO()
      with gzip.GzipFile(fileobj=buf, mode="wb", compresslevel=int(c.get("level", 6)),
                         mtime=0) as g:
        g.write(raw)
      return buf.getvalue()
    if c["id"] == "zlib":
      return zlib.compress(raw, int(c.get("level", 6)))
    if c["id"] == "zstd":
      import pyarrow as pa
      return pa.Codec("zstd").compress(raw, asbytes=True)
    raise NotImplementedError(f"zarr compressor {c}")

  def _decode(self, data: bytes, nbytes: int) -> bytes:
    c = self.compressor
    if c is None:
      return data
    if c["id"] == "gzip":
      return gzip.decompress(data)
    if c["id"] == "zlib":
      return zlib.decompress(data)
    if c["id"] == "zstd":
      import pyarrow as pa
      return pa.Codec("zstd").decompress(data, decompressed_size=nbytes, asbytes=True)
    if c["id"] == "blosc":
      raise NotImplementedError("blosc-compressed zarr chunks are not supported")
    raise NotImplementedError(f"zarr compressor {c}")

  def _chunk_file(self, idx: Tuple[int, ...]) -> str:
    name = self.sep.join(str(i) for i in idx) if idx else "0"
    return os.path.join(self.path, *name.split("/"))

  def _read_chunk(self, idx) -> Optional[np.ndarray]:
    fn = self._chunk_file(idx)
    if not os.path.exists(fn):
      return None
    with open(fn, "rb") as f:
      data = f.read()
    n = int(np.prod(self.chunks)) if self.chunks else 1
    raw = self._decode(data, n * self.dtype.itemsize)
    return np.frombuffer(raw, dtype=self.dtype, count=n).reshape(self.chunks)

  def _write_chunk(self, idx, arr: np.ndarray) -> None:
    fn = self._chunk_file(idx)
    os.makedirs(os.path.dirname(fn), exist_ok=True)
    tmp = fn + f".tmp{os.getpid()}"
    with open(tmp, "wb") as f:
      f.write(self._encode(np.ascontiguousarray(arr).tobytes("C")))
    os.replace(tmp, fn)

  def _fill(self):
    fv = self.fill_value
    return np.zeros((), self.dtype) if fv is None else np.asarray(fv).astype(self.dtype)

  # -- region IO --------------------------------------------------------------------------
  @staticmethod
  def _norm(region, shape):
    if region is None:
      region = tuple(slice(None) for _ in shape)
    out = []
    for sl, n in zip(region, shape):
      start, stop, step = sl.indices(n)
      assert step == 1
      out.append((start, stop))
    return out

  def write(self, value: np.ndarray, region: Optional[Sequence[slice]] = None) -> None:
    """Writes `value` into `region` (default: everything)."""
    value = np.asarray(value)
    if value.dtype != self.dtype:
      value = value.astype(self.dtype)
    if not self.shape:
      self._write_chunk((), value.reshape(()))
      return
    bounds = self._norm(region, self.shape)
    assert tuple(b - a for a, b in bounds) == tuple(value.shape), (bounds, value.shape)
    ranges = [range(a // c, (b - 1) // c + 1) if b > a else range(0)
              for (a, b), c in zip(bounds, self.chunks)]
    for idx in itertools.product(*ranges):
      c_lo = [i * c for i, c in zip(idx, self.chunks)]
      c_hi = [min(lo + c, n) for lo, c, n in zip(c_lo, self.chunks, self.shape)]
      lo = [max(a, cl) for (a, _), cl in zip(bounds, c_lo)]
      hi = [min(b, ch) for (_, b), ch in zip(bounds, c_hi)]
      covers = all(l == cl and h == ch for l, h, cl, ch in zip(lo, hi, c_lo, c_hi))
      full = all(ch - cl == c for cl, ch, c in zip(c_lo, c_hi, self.chunks))
      src = value[tuple(slice(l - a, h - a) for l, h, (a, _) in zip(lo, hi, bounds))]
      if covers and full:
        self._write_chunk(idx, src)
        continue
      chunk = None if covers else self._read_chunk(idx)
      if chunk is None:
        chunk = np.empty(self.chunks, self.dtype)
        chunk[...] = self._fill()
      else:
        chunk = chunk.copy()
      chunk[tuple(slice(l - cl, h - cl) for l, h, cl in zip(lo, hi, c_lo))] = src
      self._write_chunk(idx, chunk)

  def read(self, region: Optional[Sequence[slice]] = None, dtype=None) -> np.ndarray:
    """Reads `region` (default: everything), optionally cast to `dtype`."""
    if not self.shape:
      c = self._read_chunk(())
      out = np.array(self._fill() if c is None else c.reshape(()))
      return out.astype(dtype) if dtype is not None else out
    bounds = self._norm(region, self.shape)
    out = np.empty(tuple(b - a for a, b in bounds), self.dtype)
    ranges = [range(a // c, (b - 1) // c + 1) if b > a else range(0)
              for (a, b), c in zip(bounds, self.chunks)]
    for idx in itertools.product(*ranges):
      c_lo = [i * c for i, c in zip(idx, self.chunks)]
      lo = [max(a, cl) for (a, _), cl in zip(bounds, c_lo)]
      hi = [min(b, cl + c, n) for (_, b), cl, c, n in zip(bounds, c_lo, self.chunks, self.shape)]
      chunk = self._read_chunk(idx)
      dst = tuple(slice(l - a, h - a) for l, h, (a, _) in zip(lo, hi, bounds))
      if chunk is None:
        out[dst] = self._fill()
      else:
        out[dst] = chunk[tuple(slice(l - cl, h - cl) for l, h, cl in zip(lo, hi, c_lo))]
    if dtype is not None and np.dtype(dtype) != out.dtype:
      out = out.astype(dtype)
    return out
