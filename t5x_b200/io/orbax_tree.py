"""PyTree checkpoints in the directory layout Orbax's PyTreeCheckpointHandler writes when it is
not packing arrays into an OCDBT database (the reference restores such trees through
`ocp.PyTreeCheckpointHandler`, t5x/checkpoints.py:2097-2183, 2386-2510).

Layout of one tree directory:
  <dir>/checkpoint          optional msgpack "aggregate" file: the tree with small values inline
                            and every array written separately as the string
                            'PLACEHOLDER://<name>'
  <dir>/_METADATA           optional JSON: {"tree_metadata": {"('a', 'b')": {"key_metadata":
                            [{"key": "a", "key_type": 2}, ...], "value_metadata": {...}}}}
  <dir>/<name>/             one array per leaf, <name> = key path joined with '.'; zarr v2
                            (`.zarray` + chunk files '0.0') or zarr v3 (`zarr.json` + 'c/0/0')
  <dir>/_sharding           optional, ignored (sharding is decided by the restoring job)

T5X puts the train state's `state_dict()` ({'state': ..., 'target': ...}) into
`checkpoint_<step>/state/`. Chunks are usually zstd frames; they are decoded through pyarrow's
codec. OCDBT-packed directories (`manifest.ocdbt`) are recognised and refused.
"""
import ast
import gzip
import io
import json
import os
from typing import Any, Dict, Mapping, Optional, Sequence, Tuple

import numpy as np

from t5x_b200.io import msgpack_io
from t5x_b200.io import zarr_io

PLACEHOLDER_PREFIX = "PLACEHOLDER://"
AGGREGATE_FILE = "checkpoint"
METADATA_FILE = "_METADATA"
_KEY_TYPE_SEQUENCE = 1
_KEY_TYPE_DICT = 2


def is_ocdbt(directory: str) -> bool:
  """True when the arrays of `directory` are packed into an OCDBT database."""
  if os.path.exists(os.path.join(directory, "manifest.ocdbt")):
    return True
  try:
    return any(n.startswith("ocdbt.process_") for n in os.listdir(directory))
  except OSError:
    return False


def _is_placeholder(x) -> bool:
  return isinstance(x, str) and x.startswith(PLACEHOLDER_PREFIX)


def _has_placeholder(tree) -> bool:
  if isinstance(tree, Mapping):
    return any(_has_placeholder(v) for v in tree.values())
  if isinstance(tree, (list, tuple)):
    return any(_has_placeholder(v) for v in tree)
  return _is_placeholder(tree)


def _read_aggregate(directory: str):
  f = os.path.join(directory, AGGREGATE_FILE)
  if not os.path.isfile(f):
    return None
  try:
    with open(f, "rb") as fp:
      return msgpack_io.msgpack_restore(fp.read())
  except Exception:  # not msgpack: some other file that happens to be called `checkpoint`
    return None


def is_tree_dir(directory: str) -> bool:
  """True when `directory` holds a tree in this layout (packed or not)."""
  if not os.path.isdir(directory):
    return False
  if is_ocdbt(directory) or os.path.exists(os.path.join(directory, METADATA_FILE)):
    return True
  agg = _read_aggregate(directory)
  return agg is not None and _has_placeholder(agg)


def find_state_dir(checkpoint_dir: str) -> Optional[str]:
  """The tree directory of a checkpoint: `<checkpoint_dir>/state` (how the T5X manager nests
  it), else the directory itself, else None."""
  nested = os.path.join(checkpoint_dir, "state")
  if is_tree_dir(nested):
    return nested
  if is_tree_dir(checkpoint_dir):
    return checkpoint_dir
  return None


# ----------------------------------------------------------------------------
# Arrays
# ----------------------------------------------------------------------------
def _zstd_stream_decode(data: bytes) -> bytes:
  import pyarrow as pa
  return pa.CompressedInputStream(io.BytesIO(data), "zstd").read()


_V3_DTYPES = {"bool": "bool", "int8": "i1", "int16": "i2", "int32": "i4", "int64": "i8",
              "uint8": "u1", "uint16": "u2", "uint32": "u4", "uint64": "u8",
              "float16": "f2", "float32": "f4", "float64": "f8"}


class _Zarr3Array:
  """Reader for a zarr v3 array with a regular chunk grid and a bytes -> (zstd | gzip) codec
  chain; the sharding and transpose codecs are not handled."""

  def __init__(self, path: str, meta: Dict[str, Any]):
    self.path = path
    self.shape = tuple(int(s) for s in meta["shape"])
    grid = meta.get("chunk_grid", {})
    if grid.get("name", "regular") != "regular":
      raise NotImplementedError(f"zarr v3 chunk grid {grid.get('name')}")
    self.chunks = tuple(int(c) for c in grid.get("configuration", {}).get("chunk_shape",
                                                                         self.shape))
    name = meta["data_type"]
    if name == "bfloat16":
      self.dtype = zarr_io._np_dtype("bfloat16")
    else:
      self.dtype = np.dtype(_V3_DTYPES[name])
    enc = meta.get("chunk_key_encoding", {"name": "default"})
    self.sep = enc.get("configuration", {}).get("separator",
                                                "/" if enc.get("name") == "default" else ".")
    self.prefix = "c" if enc.get("name", "default") == "default" else ""
    self.fill_value = meta.get("fill_value", 0)
    self.codecs = meta.get("codecs", [{"name": "bytes"}])
    for c in self.codecs:
      if c["name"] not in ("bytes", "zstd", "gzip"):
        raise NotImplementedError(f"zarr v3 codec {c['name']}")

  def _chunk_file(self, idx: Tuple[int, ...]) -> str:
    parts = [str(i) for i in idx]
    if self.prefix:
      key = self.sep.join([self.prefix] + parts)
    else:
      key = self.sep.join(parts) if parts else "0"
    return os.path.join(self.path, *key.split("/"))

  def _read_chunk(self, idx) -> Optional[np.ndarray]:
    fn = self._chunk_file(idx)
    if not os.path.exists(fn):
      return None
    with open(fn, "rb") as f:
      data = f.read()
    dtype = self.dtype
    for c in reversed(self.codecs):
      if c["name"] == "zstd":
        data = _zstd_stream_decode(data)
      elif c["name"] == "gzip":
        data = gzip.decompress(data)
      elif c["name"] == "bytes":
        if c.get("configuration", {}).get("endian", "little") == "big":
          dtype = dtype.newbyteorder(">")
    n = int(np.prod(self.chunks)) if self.chunks else 1
    return np.frombuffer(data, dtype=dtype, count=n).reshape(self.chunks).astype(self.dtype)

  def read(self, region=None, dtype=None) -> np.ndarray:
    out = np.full(self.shape, self.fill_value or 0, dtype=self.dtype)
    if not self.shape:
      c = self._read_chunk(())
      if c is not None:
        out[...] = c.reshape(())
    else:
      grid = [range(-(-s // c)) for s, c in zip(self.shape, self.chunks)]
      for idx in np.ndindex(*[len(g) for g in grid]):
        c = self._read_chunk(idx)
        if c is None:
          continue
        sl = tuple(slice(i * cs, min((i + 1) * cs, s))
                   for i, cs, s in zip(idx, self.chunks, self.shape))
        out[sl] = c[tuple(slice(0, s.stop - s.start) for s in sl)]
    if region is not None:
      out = out[tuple(region)]
    return out.astype(dtype) if dtype is not None else out


class ArrayRef:
  """One array of a tree directory, read on demand."""

  def __init__(self, path: str, name: str):
    self.path = path
    self.name = name
    self._arr = None
    if os.path.exists(os.path.join(path, ".zarray")):
      self._arr = zarr_io.ZarrArray.open(path)
    elif os.path.exists(os.path.join(path, "zarr.json")):
      with open(os.path.join(path, "zarr.json")) as f:
        self._arr = _Zarr3Array(path, json.load(f))

  @property
  def shape(self) -> Optional[Tuple[int, ...]]:
    return None if self._arr is None else tuple(self._arr.shape)

  @property
  def dtype(self) -> Optional[np.dtype]:
    return None if self._arr is None else self._arr.dtype

  def _read_without_metadata(self, shape, dtype) -> np.ndarray:
    """An array directory stripped of its metadata file: one chunk named '0', '0.0', ...
    whose shape and type kind come from the restore target and whose item size follows from
    the decoded length."""
    if shape is None:
      raise ValueError(f"Array `{self.name}` at {self.path} has no zarr metadata; its shape "
                       "must come from the restore target.")
    shape = tuple(int(s) for s in shape)
    key = ".".join("0" for _ in shape) or "0"
    fn = os.path.join(self.path, key)
    if not os.path.exists(fn):
      fn = os.path.join(self.path, *key.split("."))
    with open(fn, "rb") as f:
      data = f.read()
    raw = _zstd_stream_decode(data) if data[:4] == b"\x28\xb5\x2f\xfd" else (
        gzip.decompress(data) if data[:2] == b"\x1f\x8b" else data)
    n = int(np.prod(shape)) if shape else 1
    if n == 0 or len(raw) % n:
      raise ValueError(f"Array `{self.name}`: {len(raw)} bytes do not fill shape {shape}.")
    kind = np.dtype(dtype).kind if dtype is not None else "f"
    item = len(raw) // n
    if dtype is not None and np.dtype(dtype).itemsize == item:
      stored = np.dtype(dtype)
    else:
      stored = np.dtype(f"{kind if kind in 'fiub' else 'f'}{item}")
    return np.frombuffer(raw, dtype=stored, count=n).reshape(shape)

  def read(self, region: Optional[Sequence[slice]] = None, dtype=None, expected_shape=None,
           expected_dtype=None) -> np.ndarray:
    if self._arr is not None:
      if expected_shape is not None and tuple(expected_shape) != tuple(self._arr.shape):
        raise ValueError(f"Shape of `{self.name}` in checkpoint {tuple(self._arr.shape)} does "
                         f"not match expectation {tuple(expected_shape)}.")
      return self._arr.read(region, dtype=dtype)
    out = self._read_without_metadata(expected_shape, expected_dtype)
    if region is not None:
      out = out[tuple(region)]
    return out.astype(dtype) if dtype is not None else out

  def __repr__(self):
    return f"ArrayRef({self.name!r}, shape={self.shape}, dtype={self.dtype})"


# ----------------------------------------------------------------------------
# Trees
# ----------------------------------------------------------------------------
def _set_path(tree: Dict, keys: Sequence[Any], value) -> None:
  node = tree
  for k in keys[:-1]:
    node = node.setdefault(k, {})
  node[keys[-1]] = value


def _lists_from_int_keys(tree):
  """Dict nodes whose keys are 0..n-1 sequence indices become lists."""
  if not isinstance(tree, dict):
    return tree
  out = {k: _lists_from_int_keys(v) for k, v in tree.items()}
  if out and all(isinstance(k, int) for k in out) and sorted(out) == list(range(len(out))):
    return [out[i] for i in range(len(out))]
  return out


def _keys_from_metadata(entry_key: str, entry: Mapping[str, Any]):
  km = entry.get("key_metadata")
  if km:
    return [int(k["key"]) if int(k.get("key_type", _KEY_TYPE_DICT)) == _KEY_TYPE_SEQUENCE
            else k["key"] for k in km]
  try:
    keys = ast.literal_eval(entry_key)
    return list(keys) if isinstance(keys, (tuple, list)) else [keys]
  except (ValueError, SyntaxError):
    return entry_key.split(".")


def load_tree(directory: str) -> Any:
  """The tree of `directory` with every separately stored array as an `ArrayRef` and inline
  values as they are. Sources, in this order: the aggregate file, the `_METADATA` key list,
  the array sub-directories themselves."""
  if is_ocdbt(directory):
    raise NotImplementedError(
        f"{directory} packs its arrays into an OCDBT database (manifest.ocdbt); only the "
        "one-directory-per-array layout can be read. Re-save the checkpoint with "
        "`use_ocdbt=False`, or convert it to the native T5X format, with the tool that wrote it.")
  agg = _read_aggregate(directory)
  if agg is not None and (_has_placeholder(agg) or not os.path.exists(
      os.path.join(directory, METADATA_FILE))):
    def resolve(node):
      if isinstance(node, Mapping):
        return {k: resolve(v) for k, v in node.items()}
      if isinstance(node, (list, tuple)):
        return [resolve(v) for v in node]
      if _is_placeholder(node):
        name = node[len(PLACEHOLDER_PREFIX):]
        return ArrayRef(os.path.join(directory, name), name)
      return node
    return resolve(agg)
  tree: Dict[Any, Any] = {}
  meta_file = os.path.join(directory, METADATA_FILE)
  if os.path.exists(meta_file):
    with open(meta_file) as f:
      meta = json.load(f)
    for entry_key, entry in meta.get("tree_metadata", {}).items():
      keys = _keys_from_metadata(entry_key, entry)
      vm = entry.get("value_metadata", {})
      name = ".".join(str(k) for k in keys)
      if vm.get("skip_deserialize") or vm.get("value_type") in ("None", "Dict", "List"):
        _set_path(tree, keys, {} if vm.get("value_type") == "Dict" else
                  ([] if vm.get("value_type") == "List" else None))
        continue
      _set_path(tree, keys, ArrayRef(os.path.join(directory, name), name))
    return _lists_from_int_keys(tree)
  for name in sorted(os.listdir(directory)):
    sub = os.path.join(directory, name)
    if os.path.isdir(sub) and (os.path.exists(os.path.join(sub, ".zarray")) or
                               os.path.exists(os.path.join(sub, "zarr.json"))):
      _set_path(tree, name.split("."), ArrayRef(sub, name))
  if not tree:
    raise ValueError(f"No PyTree checkpoint found in {directory}")
  return tree


def _flatten(tree, prefix=()):
  if isinstance(tree, Mapping) and tree:
    for k, v in tree.items():
      yield from _flatten(v, prefix + ((k, _KEY_TYPE_DICT),))
  elif isinstance(tree, (list, tuple)) and tree:
    for i, v in enumerate(tree):
      yield from _flatten(v, prefix + ((i, _KEY_TYPE_SEQUENCE),))
  else:
    yield prefix, tree


def save_tree(directory: str, tree: Any, compressor: Optional[Dict[str, Any]] = None,
              aggregate: bool = True) -> None:
  """Writes `tree` (nested dicts / lists of arrays and scalars) in this layout: every array
  and scalar leaf as a one-chunk zarr v2 array, `_METADATA`, and (with `aggregate`) the msgpack
  file of placeholders. `None` leaves and empty containers live in the metadata only."""
  compressor = {"id": "zstd", "level": 1} if compressor is None else (compressor or None)
  os.makedirs(directory, exist_ok=True)
  tree_metadata = {}
  placeholders: Dict[Any, Any] = {}
  for path, leaf in _flatten(tree):
    keys = [k for k, _ in path]
    entry = {"key_metadata": [{"key": str(k), "key_type": t} for k, t in path]}
    name = ".".join(str(k) for k in keys)
    if leaf is None or (isinstance(leaf, (Mapping, list, tuple)) and not leaf):
      vt = "None" if leaf is None else ("Dict" if isinstance(leaf, Mapping) else "List")
      entry["value_metadata"] = {"value_type": vt, "skip_deserialize": True}
      _set_path(placeholders, keys, leaf)
    else:
      arr = np.asarray(leaf)
      entry["value_metadata"] = {"value_type": "np.ndarray" if arr.shape else "scalar",
                                 "skip_deserialize": False}
      z = zarr_io.ZarrArray.create(os.path.join(directory, name), arr.shape,
                                   arr.shape, arr.dtype, compressor)
      z.write(arr)
      _set_path(placeholders, keys, PLACEHOLDER_PREFIX + name)
    tree_metadata[str(tuple(str(k) for k in keys))] = entry
  with open(os.path.join(directory, METADATA_FILE), "w") as f:
    json.dump({"tree_metadata": tree_metadata, "use_zarr3": False}, f)
  if aggregate:
    with open(os.path.join(directory, AGGREGATE_FILE), "wb") as f:
      f.write(msgpack_io.msgpack_serialize(_lists_from_int_keys(placeholders)))
