"""Vocabularies (the seqio.Vocabulary contract: pad 0, eos 1, unk 2, extra ids at the top)."""
from __future__ import annotations

from typing import List, Optional, Sequence


class Vocabulary:
  """Abstract vocabulary with `extra_ids` sentinel tokens counting down from the top id."""

  def __init__(self, extra_ids: int = 0):
    self._extra_ids = extra_ids or 0

  pad_id = 0

  @property
  def eos_id(self) -> Optional[int]:
    return 1

  @property
  def unk_id(self) -> Optional[int]:
    return 2

  @property
  def extra_ids(self) -> int:
    return self._extra_ids

  @property
  def _base_vocab_size(self) -> int:
    raise NotImplementedError

  @property
  def vocab_size(self) -> int:
    return self._base_vocab_size + self._extra_ids

  def _encode(self, s: str) -> List[int]:
    raise NotImplementedError

  def _decode(self, ids: Sequence[int]) -> str:
    raise NotImplementedError

  def encode(self, s: str) -> List[int]:
    return self._encode(s)

  def decode(self, ids) -> str:
    ids = [int(i) for i in ids]
    if self.eos_id is not None and self.eos_id in ids:
      ids = ids[:ids.index(self.eos_id) + 1]
    ids = [i for i in ids if i != self.pad_id]
    clean = [self.unk_id if (i >= self._base_vocab_size and self.unk_id is not None) else i
             for i in ids]
    return self._decode(clean)

  def __eq__(self, other):
    return type(self) is type(other) and self.__dict__ == other.__dict__


class PassThroughVocabulary(Vocabulary):
  """Ids in, ids out (used for synthetic token data)."""

  def __init__(self, size: int, eos_id: Optional[int] = 1):
    super().__init__(0)
    self._size = size
    self._eos_id = eos_id

  @property
  def eos_id(self):
    return self._eos_id

  @property
  def unk_id(self):
    return None

  @property
  def _base_vocab_size(self):
    return self._size

  def _encode(self, s):
    return [int(x) for x in s.split()] if isinstance(s, str) else list(s)

  def _decode(self, ids):
    return " ".join(str(i) for i in ids)

  def decode(self, ids):
    return self._decode([int(i) for i in ids])


class ByteVocabulary(Vocabulary):
  """UTF-8 bytes offset by 3 special ids (pad, eos, unk), as used by ByT5."""

  def __init__(self, extra_ids: int = 0):
    super().__init__(extra_ids)
    self._num_special = 3

  @property
  def _base_vocab_size(self):
    return self._num_special + 256

  def _encode(self, s):
    return [b + self._num_special for b in s.encode("utf-8")]

  def _decode(self, ids):
    bs = bytes(i - self._num_special for i in ids
               if self._num_special <= i < self._num_special + 256)
    return bs.decode("utf-8", errors="ignore")


class SentencePieceVocabulary(Vocabulary):
  """SentencePiece model file + `extra_ids` sentinels (T5: 32000 + 100)."""

  def __init__(self, sentencepiece_model_file: str, extra_ids: int = 0, **_):
    super().__init__(extra_ids)
    self._file = sentencepiece_model_file
    self._sp = None

  def _load(self):
    if self._sp is None:
      import sentencepiece as spm
      self._sp = spm.SentencePieceProcessor()
      self._sp.Load(self._file)
    return self._sp

  @property
  def _base_vocab_size(self):
    return self._load().GetPieceSize()

  def _encode(self, s):
    return list(self._load().EncodeAsIds(s))

  def _decode(self, ids):
    return self._load().DecodeIds([int(i) for i in ids])

  def __eq__(self, other):
    return (isinstance(other, SentencePieceVocabulary) and self._file == other._file and
            self._extra_ids == other._extra_ids)
