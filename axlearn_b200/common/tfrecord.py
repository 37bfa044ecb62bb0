"""TFRecord files and ``tf.train.Example`` records without TensorFlow.

The reference writes inference outputs and reads most of its datasets as TFRecord files of
serialised ``tf.train.Example`` protos (axlearn/common/inference_output.py:57-119,
axlearn/common/input_tf_data.py:204-330).  Both formats are small and public, so they are
implemented here directly:

* a TFRecord file is a sequence of ``uint64 length | uint32 masked_crc32c(length) | bytes data |
  uint32 masked_crc32c(data)`` frames, little endian, with ``masked = rotr15(crc) + 0xa282ead8``;
* an ``Example`` is ``{1: Features}``, ``Features`` is ``{1: map<string, Feature>}`` and a
  ``Feature`` is one of ``bytes_list = 1``, ``float_list = 2`` (packed fixed32) or
  ``int64_list = 3`` (packed varint), each ``{1: repeated value}``.
"""

from __future__ import annotations

import struct
from typing import Any, BinaryIO, Iterator, Mapping, Sequence, Union

import numpy as np

_CRC_TABLE = None
_MASK_DELTA = 0xA282EAD8


def _crc_table() -> np.ndarray:
    global _CRC_TABLE  # pylint: disable=global-statement
    if _CRC_TABLE is None:
        poly = 0x82F63B78  # Castagnoli, reflected.
        table = np.zeros((8, 256), dtype=np.uint32)
        for i in range(256):
            c = i
            for _ in range(8):
                c = (c >> 1) ^ poly if c & 1 else c >> 1
            table[0, i] = c
        for i in range(256):
            c = int(table[0, i])
            for k in range(1, 8):
                c = int(table[0, c & 0xFF]) ^ (c >> 8)
                table[k, i] = c
        _CRC_TABLE = table
    return _CRC_TABLE


def crc32c(data: bytes) -> int:
    """CRC-32C (Castagnoli) of ``data``; slicing-by-8 over a NumPy view, byte loop for the tail."""
    t = _crc_table()
    crc = 0xFFFFFFFF
    n8 = len(data) // 8
    if n8:
        t0, t1, t2, t3, t4, t5, t6, t7 = (t[k].tolist() for k in range(8))
        words = struct.unpack(f"<{n8 * 2}I", data[: n8 * 8])
        for i in range(0, n8 * 2, 2):
            lo = words[i] ^ crc
            hi = words[i + 1]
            crc = (t7[lo & 0xFF] ^ t6[(lo >> 8) & 0xFF] ^ t5[(lo >> 16) & 0xFF] ^ t4[lo >> 24]
                   ^ t3[hi & 0xFF] ^ t2[(hi >> 8) & 0xFF] ^ t1[(hi >> 16) & 0xFF] ^ t0[hi >> 24])
    t0 = t[0]
    for b in data[n8 * 8:]:
        crc = int(t0[(crc ^ b) & 0xFF]) ^ (crc >> 8)
    return crc ^ 0xFFFFFFFF


def masked_crc32c(data: bytes) -> int:
    crc = crc32c(data)
    return (((crc >> 15) | (crc << 17)) + _MASK_DELTA) & 0xFFFFFFFF


# ------------------------------------------------------------------------------------------------
# Record framing.


class TFRecordWriter:
    """Appends framed records to a binary file."""

    def __init__(self, path_or_file: Union[str, BinaryIO]):
        self._own = isinstance(path_or_file, str)
        self._f = open(path_or_file, "wb") if self._own else path_or_file  # pylint: disable=consider-using-with

    def write(self, record: bytes) -> None:
        header = struct.pack("<Q", len(record))
        self._f.write(header + struct.pack("<I", masked_crc32c(header)) + record
                      + struct.pack("<I", masked_crc32c(record)))

    def flush(self) -> None:
        self._f.flush()

    def close(self) -> None:
        if self._own:
            self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


def read_tfrecords(path_or_file: Union[str, BinaryIO], *, check_crc: bool = True) -> Iterator[bytes]:
    """Yields the records of one file; raises ``ValueError`` on a truncated or corrupt frame."""
    own = isinstance(path_or_file, str)
    f = open(path_or_file, "rb") if own else path_or_file  # pylint: disable=consider-using-with
    try:
        while True:
            header = f.read(12)
            if not header:
                return
            if len(header) < 12:
                raise ValueError("truncated TFRecord header")
            (length,), (crc,) = struct.unpack("<Q", header[:8]), struct.unpack("<I", header[8:])
            if check_crc and masked_crc32c(header[:8]) != crc:
                raise ValueError("corrupt TFRecord length")
            body = f.read(length + 4)
            if len(body) < length + 4:
                raise ValueError("truncated TFRecord body")
            data = body[:length]
            if check_crc and masked_crc32c(data) != struct.unpack("<I", body[length:])[0]:
                raise ValueError("corrupt TFRecord data")
            yield data
    finally:
        if own:
            f.close()


# ------------------------------------------------------------------------------------------------
# Protobuf wire format (only what Example needs).


def _varint(n: int) -> bytes:
    if n < 0:
        n += 1 << 64
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        if n:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _read_varint(buf: bytes, pos: int) -> tuple[int, int]:
    shift = value = 0
    while True:
        b = buf[pos]
        pos += 1
        value |= (b & 0x7F) << shift
        if not b & 0x80:
            return value, pos
        shift += 7


def _len_field(number: int, payload: bytes) -> bytes:
    return _varint((number << 3) | 2) + _varint(len(payload)) + payload


def _fields(buf: bytes) -> Iterator[tuple[int, int, Any]]:
    pos = 0
    while pos < len(buf):
        key, pos = _read_varint(buf, pos)
        number, wire = key >> 3, key & 7
        if wire == 0:
            value, pos = _read_varint(buf, pos)
        elif wire == 1:
            value, pos = buf[pos:pos + 8], pos + 8
        elif wire == 2:
            n, pos = _read_varint(buf, pos)
            value, pos = buf[pos:pos + n], pos + n
        elif wire == 5:
            value, pos = buf[pos:pos + 4], pos + 4
        else:
            raise ValueError(f"unsupported wire type {wire}")
        yield number, wire, value


FeatureValue = Union[np.ndarray, Sequence[bytes], Sequence[str], Sequence[int], Sequence[float], bytes, str, int, float]


def _encode_feature(value: FeatureValue) -> bytes:
    if isinstance(value, (bytes, str)):
        value = [value]
    if isinstance(value, (list, tuple)) and value and isinstance(value[0], (bytes, str)):
        items = b"".join(_len_field(1, v.encode("utf-8") if isinstance(v, str) else v) for v in value)
        return _len_field(1, items)
    arr = np.asarray(value).reshape(-1)
    if arr.dtype.kind in "SUO":
        return _encode_feature([v if isinstance(v, (bytes, str)) else bytes(v) for v in arr.tolist()])
    if arr.dtype.kind == "f":
        packed = arr.astype("<f4").tobytes()
        return _len_field(2, _len_field(1, packed) if arr.size else b"")
    if arr.dtype.kind in "biu":
        packed = b"".join(_varint(int(v)) for v in arr.tolist())
        return _len_field(3, _len_field(1, packed) if arr.size else b"")
    raise NotImplementedError(f"no Example feature for dtype {arr.dtype}")


def encode_example(features: Mapping[str, FeatureValue]) -> bytes:
    """Serialises ``{name: values}``: floats -> float_list, ints / bools -> int64_list, bytes / str
    -> bytes_list; arrays are flattened (as the reference's sink does)."""
    entries = b""
    for name in sorted(features):                       # deterministic bytes
        entry = _len_field(1, name.encode("utf-8")) + _len_field(2, _encode_feature(features[name]))
        entries += _len_field(1, entry)
    return _len_field(1, entries)


def decode_example(record: bytes) -> dict[str, Union[np.ndarray, list[bytes]]]:
    """Inverse of ``encode_example``: float32 / int64 arrays, or a list of ``bytes``."""
    out: dict[str, Any] = {}
    for number, _, features in _fields(record):
        if number != 1:
            continue
        for fnum, _, entry in _fields(features):
            if fnum != 1:
                continue
            name, feature = None, b""
            for enum, _, v in _fields(entry):
                if enum == 1:
                    name = v.decode("utf-8")
                elif enum == 2:
                    feature = v
            value: Any = []
            for kind, _, payload in _fields(feature):
                if kind == 1:
                    value = [v for n, _, v in _fields(payload) if n == 1]
                elif kind == 2:
                    chunks = []
                    for n, wire, v in _fields(payload):
                        if n == 1:
                            chunks.append(np.frombuffer(v, dtype="<f4"))
                    value = np.concatenate(chunks) if chunks else np.zeros([0], np.float32)
                elif kind == 3:
                    ints = []
                    for n, wire, v in _fields(payload):
                        if n != 1:
                            continue
                        if wire == 0:
                            ints.append(v)
                        else:
                            pos = 0
                            while pos < len(v):
                                x, pos = _read_varint(v, pos)
                                ints.append(x)
                    value = np.array([x - (1 << 64) if x >= 1 << 63 else x for x in ints], dtype=np.int64)
            out[name] = value
    return out
