"""Flax-compatible msgpack (de)serialisation of nested dicts with array leaves.

Wire format: numpy arrays travel as msgpack ext type 1 whose payload is
`packb((shape, dtype_name, raw_bytes))`; complex Python scalars as ext type 2 `(real, imag)`;
numpy scalars as ext type 3 (same payload as an array). Arrays larger than 1 GiB are split into
`{'__msgpack_chunked_array__': True, 'shape': [...], 'chunks': {'0': ext, '1': ext, ...}}`.
bfloat16 uses the dtype name 'bfloat16' (ml_dtypes).
"""
from __future__ import annotations

from typing import Any

import msgpack
import numpy as np

try:
  import ml_dtypes  # noqa: F401  registers bfloat16 with numpy
except ImportError:  # pragma: no cover
  ml_dtypes = None

EXT_NDARRAY, EXT_NATIVE_COMPLEX, EXT_NPSCALAR = 1, 2, 3
MAX_CHUNK_SIZE = 2 ** 30


def _dtype_from_name(name: str) -> np.dtype:
  if name == "bfloat16":
    import ml_dtypes as mld
    return np.dtype(mld.bfloat16)
  return np.dtype(name)


def _to_numpy(x):
  try:
    import torch
    if isinstance(x, torch.Tensor):
      t = x.detach().cpu()
      if t.dtype == torch.bfloat16:
        import ml_dtypes as mld
        return t.view(torch.int16).numpy().view(mld.bfloat16)
      return t.numpy()
  except ImportError:  # pragma: no cover
    pass
  return x


def _ndarray_to_bytes(arr: np.ndarray) -> bytes:
  if arr.dtype.hasobject or arr.dtype.isalignedstruct:
    raise ValueError("Object and structured dtypes not supported for serialization of ndarrays.")
  tpl = (list(arr.shape), arr.dtype.name, np.ascontiguousarray(arr).tobytes("C"))
  return msgpack.packb(tpl, use_bin_type=True)


def _ndarray_from_bytes(data: bytes) -> np.ndarray:
  shape, dtype_name, buffer = msgpack.unpackb(data, raw=True)
  if isinstance(dtype_name, bytes):
    dtype_name = dtype_name.decode()
  return np.frombuffer(buffer, dtype=_dtype_from_name(dtype_name), count=-1,
                       offset=0).reshape(shape, order="C").copy()


def _ext_pack(x):
  x = _to_numpy(x)
  if isinstance(x, np.ndarray):
    return msgpack.ExtType(EXT_NDARRAY, _ndarray_to_bytes(x))
  if isinstance(x, np.generic):
    return msgpack.ExtType(EXT_NPSCALAR, _ndarray_to_bytes(np.asarray(x)))
  if isinstance(x, complex):
    return msgpack.ExtType(EXT_NATIVE_COMPLEX, msgpack.packb((x.real, x.imag)))
  raise TypeError(f"cannot serialise object of type {type(x)}")


def _ext_unpack(code, data):
  if code == EXT_NDARRAY:
    return _ndarray_from_bytes(data)
  if code == EXT_NATIVE_COMPLEX:
    re, im = msgpack.unpackb(data)
    return complex(re, im)
  if code == EXT_NPSCALAR:
    ar = _ndarray_from_bytes(data)
    return ar[()]
  return msgpack.ExtType(code, data)


def _chunk(arr: np.ndarray):
  flat = arr.reshape(-1)
  per = max(1, MAX_CHUNK_SIZE // max(1, arr.dtype.itemsize))
  chunks = {str(i): flat[s:s + per] for i, s in enumerate(range(0, flat.size, per))}
  return {"__msgpack_chunked_array__": True, "shape": list(arr.shape), "chunks": chunks}


def _prepare(tree):
  """Converts tensors to numpy and splits oversized arrays."""
  if isinstance(tree, dict):
    return {str(k): _prepare(v) for k, v in tree.items()}
  if isinstance(tree, (list, tuple)):
    return [_prepare(v) for v in tree]
  tree = _to_numpy(tree)
  if isinstance(tree, np.ndarray) and tree.size * tree.dtype.itemsize > MAX_CHUNK_SIZE:
    return _chunk(tree)
  return tree


def _unchunk(tree):
  if isinstance(tree, dict):
    if tree.get("__msgpack_chunked_array__"):
      parts = [tree["chunks"][str(i)] for i in range(len(tree["chunks"]))]
      return np.concatenate([np.asarray(p).reshape(-1) for p in parts]).reshape(tree["shape"])
    return {k: _unchunk(v) for k, v in tree.items()}
  if isinstance(tree, list):
    return [_unchunk(v) for v in tree]
  return tree


def msgpack_serialize(pytree: Any) -> bytes:
  return msgpack.packb(_prepare(pytree), default=_ext_pack, strict_types=True)


def msgpack_restore(encoded: bytes) -> Any:
  return _unchunk(msgpack.unpackb(encoded, ext_hook=_ext_unpack, raw=False,
                                  strict_map_key=False))
