"""TensorFlow tensor-bundle checkpoints (`<prefix>.index` + `<prefix>.data-NNNNN-of-MMMMM`)
without TensorFlow.

The index file is a LevelDB-format table: prefix-compressed key/value blocks, an index block
that locates them, and a 48-byte footer. Its values are small protocol buffers
(`BundleHeaderProto` under the empty key, one `BundleEntryProto` per tensor: dtype, shape,
shard, byte offset, byte size). Tensor bytes are stored raw, little-endian, in the data shards.

The reader handles uncompressed tables, which is what TensorFlow writes for bundles; the
writer exists to produce test fixtures and small exports.
"""
from __future__ import annotations

import dataclasses
import os
import struct
from typing import Dict, Iterator, List, Mapping, Tuple

import numpy as np

_MAGIC = 0xDB4775248B80FB57
_FOOTER = 48
# tensorflow.DataType values
_DTYPES = {1: np.float32, 2: np.float64, 3: np.int32, 4: np.uint8, 5: np.int16, 6: np.int8,
           9: np.int64, 10: np.bool_, 17: np.uint16, 19: np.float16, 22: np.uint32,
           23: np.uint64}
_BFLOAT16 = 14


def _bf16_dtype():
  try:
    import ml_dtypes
    return np.dtype(ml_dtypes.bfloat16)
  except ImportError:  # raw 16-bit payload; callers reinterpret
    return np.dtype(np.uint16)


def _np_dtype(code: int) -> np.dtype:
  if code == _BFLOAT16:
    return _bf16_dtype()
  if code not in _DTYPES:
    raise ValueError(f"unsupported tensor dtype code {code}")
  return np.dtype(_DTYPES[code])


def _dtype_code(dtype: np.dtype) -> int:
  if dtype == _bf16_dtype() and dtype != np.dtype(np.uint16):
    return _BFLOAT16
  for code, t in _DTYPES.items():
    if np.dtype(t) == dtype:
      return code
  raise ValueError(f"unsupported dtype {dtype}")


# ---- varints and protobuf wire format -------------------------------------------------------
def _read_varint(buf: bytes, pos: int) -> Tuple[int, int]:
  result = shift = 0
  while True:
    b = buf[pos]
    pos += 1
    result |= (b & 0x7F) << shift
    if not b & 0x80:
      return result, pos
    shift += 7


def _write_varint(v: int) -> bytes:
  out = bytearray()
  while True:
    b = v & 0x7F
    v >>= 7
    if v:
      out.append(b | 0x80)
    else:
      out.append(b)
      return bytes(out)


def _fields(buf: bytes) -> Iterator[Tuple[int, int, object]]:
  """(field number, wire type, value) triples of a serialized message."""
  pos = 0
  while pos < len(buf):
    tag, pos = _read_varint(buf, pos)
    num, wt = tag >> 3, tag & 7
    if wt == 0:
      val, pos = _read_varint(buf, pos)
    elif wt == 1:
      val = buf[pos:pos + 8]
      pos += 8
    elif wt == 2:
      n, pos = _read_varint(buf, pos)
      val = buf[pos:pos + n]
      pos += n
    elif wt == 5:
      val = buf[pos:pos + 4]
      pos += 4
    else:
      raise ValueError(f"unsupported wire type {wt}")
    yield num, wt, val


def _signed(v: int) -> int:
  return v - (1 << 64) if v >= 1 << 63 else v


@dataclasses.dataclass
class BundleEntry:
  dtype: np.dtype
  shape: Tuple[int, ...]
  shard_id: int = 0
  offset: int = 0
  size: int = 0


def _parse_entry(buf: bytes) -> BundleEntry:
  dtype_code, shape, shard, offset, size = 0, [], 0, 0, 0
  for num, _, val in _fields(buf):
    if num == 1:
      dtype_code = val
    elif num == 2:  # TensorShapeProto { repeated Dim dim = 2 { int64 size = 1 } }
      for n2, _, dim in _fields(val):
        if n2 == 2:
          dsize = 0
          for n3, _, v3 in _fields(dim):
            if n3 == 1:
              dsize = _signed(v3)
          shape.append(dsize)
    elif num == 3:
      shard = val
    elif num == 4:
      offset = val
    elif num == 5:
      size = val
    elif num == 7 and val:
      raise ValueError("partitioned (sliced) variables are not supported")
  return BundleEntry(_np_dtype(dtype_code), tuple(shape), shard, offset, size)


def _parse_header(buf: bytes) -> int:
  shards = 1
  for num, _, val in _fields(buf):
    if num == 1:
      shards = val
  return shards


# ---- LevelDB table ---------------------------------------------------------------------------
def _block_handle(buf: bytes, pos: int) -> Tuple[int, int, int]:
  off, pos = _read_varint(buf, pos)
  size, pos = _read_varint(buf, pos)
  return off, size, pos


def _block_entries(data: bytes, off: int, size: int) -> Iterator[Tuple[bytes, bytes]]:
  block = data[off:off + size]
  kind = data[off + size]
  if kind != 0:
    raise ValueError("compressed index blocks are not supported (block type "
                     f"{kind}); re-save the checkpoint without table compression")
  num_restarts = struct.unpack("<I", block[-4:])[0]
  limit = len(block) - 4 - 4 * num_restarts
  pos, key = 0, b""
  while pos < limit:
    shared, pos = _read_varint(block, pos)
    non_shared, pos = _read_varint(block, pos)
    vlen, pos = _read_varint(block, pos)
    key = key[:shared] + block[pos:pos + non_shared]
    pos += non_shared
    yield key, block[pos:pos + vlen]
    pos += vlen


def read_table(path: str) -> Dict[bytes, bytes]:
  with open(path, "rb") as f:
    data = f.read()
  if len(data) < _FOOTER or struct.unpack("<Q", data[-8:])[0] != _MAGIC:
    raise ValueError(f"{path} is not a tensor-bundle index (bad table magic)")
  footer = data[-_FOOTER:]
  _, _, pos = _block_handle(footer, 0)           # metaindex
  ioff, isize, _ = _block_handle(footer, pos)    # index
  out = {}
  for _, handle in _block_entries(data, ioff, isize):
    boff, bsize, _ = _block_handle(handle, 0)
    for k, v in _block_entries(data, boff, bsize):
      out[k] = v
  return out


class BundleReader:
  """`entries` (name -> BundleEntry) and `get_tensor(name)` of a checkpoint prefix."""

  def __init__(self, prefix: str):
    if os.path.isdir(prefix):
      state = os.path.join(prefix, "checkpoint")
      if os.path.exists(state):
        for line in open(state):
          if line.startswith("model_checkpoint_path:"):
            prefix = os.path.join(prefix, line.split(":", 1)[1].strip().strip('"'))
            break
    if prefix.endswith(".index"):
      prefix = prefix[:-len(".index")]
    self.prefix = prefix
    table = read_table(prefix + ".index")
    self.num_shards = _parse_header(table.get(b"", b""))
    self.entries: Dict[str, BundleEntry] = {
        k.decode(): _parse_entry(v) for k, v in table.items() if k != b""}

  def _shard_path(self, shard: int) -> str:
    return f"{self.prefix}.data-{shard:05d}-of-{self.num_shards:05d}"

  def get_tensor(self, name: str) -> np.ndarray:
    e = self.entries[name]
    with open(self._shard_path(e.shard_id), "rb") as f:
      f.seek(e.offset)
      raw = f.read(e.size)
    return np.frombuffer(raw, dtype=e.dtype).reshape(e.shape).copy()

  def get_variable_to_shape_map(self) -> Dict[str, Tuple[int, ...]]:
    return {k: e.shape for k, e in self.entries.items()}


# ---- writer (one shard, one data block) ------------------------------------------------------
def _msg_field(num: int, wt: int, payload: bytes) -> bytes:
  return _write_varint((num << 3) | wt) + payload


def _encode_entry(e: BundleEntry) -> bytes:
  dims = b"".join(_msg_field(2, 2, (lambda d: _write_varint(len(d)) + d)(
      _msg_field(1, 0, _write_varint(int(s))))) for s in e.shape)
  out = _msg_field(1, 0, _write_varint(_dtype_code(e.dtype)))
  out += _msg_field(2, 2, _write_varint(len(dims)) + dims)
  if e.shard_id:
    out += _msg_field(3, 0, _write_varint(e.shard_id))
  if e.offset:
    out += _msg_field(4, 0, _write_varint(e.offset))
  out += _msg_field(5, 0, _write_varint(e.size))
  return out


def _block(items: List[Tuple[bytes, bytes]]) -> bytes:
  body = bytearray()
  for k, v in items:  # keys are stored whole (shared prefix length 0)
    body += _write_varint(0) + _write_varint(len(k)) + _write_varint(len(v)) + k + v
  body += struct.pack("<I", 0) + struct.pack("<I", 1)  # one restart at offset 0
  return bytes(body)


def write_bundle(prefix: str, tensors: Mapping[str, np.ndarray]) -> None:
  """Writes `tensors` as a single-shard tensor bundle at `prefix`."""
  os.makedirs(os.path.dirname(prefix) or ".", exist_ok=True)
  entries, offset = {}, 0
  with open(f"{prefix}.data-00000-of-00001", "wb") as f:
    for name in sorted(tensors):
      arr = np.asarray(tensors[name], order="C")  # keeps 0-d scalars 0-d
      raw = arr.tobytes()
      entries[name] = BundleEntry(arr.dtype, tuple(arr.shape), 0, offset, len(raw))
      f.write(raw)
      offset += len(raw)
  header = _msg_field(1, 0, _write_varint(1))
  items = [(b"", header)] + [(k.encode(), _encode_entry(entries[k])) for k in sorted(entries)]
  data_block = _block(items)
  trailer = b"\x00" + struct.pack("<I", 0)
  out = bytearray(data_block + trailer)
  meta_off = len(out)
  meta_block = _block([])
  out += meta_block + trailer
  index_off = len(out)
  handle = _write_varint(0) + _write_varint(len(data_block))
  index_block = _block([(items[-1][0] + b"\xff", handle)])
  out += index_block + trailer
  footer = (_write_varint(meta_off) + _write_varint(len(meta_block)) +
            _write_varint(index_off) + _write_varint(len(index_block)))
  footer += b"\x00" * (40 - len(footer)) + struct.pack("<Q", _MAGIC)
  out += footer
  with open(prefix + ".index", "wb") as f:
    f.write(bytes(out))
