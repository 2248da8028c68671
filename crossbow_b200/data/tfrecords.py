"""TFRecord files of ``tf.train.Example`` messages -> record files of the decoding data set, without TensorFlow.

The reference converts the ImageNet TFRecords (``train-00000-of-01024`` ...) with a TensorFlow 1 script
(scripts/datasets/imagenet/parse-records.py:15-56 features, :100-183 output files).  Here the container format and the
three protobuf messages involved are read directly:

* a TFRecord file is a sequence of ``[length u64][masked crc32c of length u32][payload][masked crc32c of payload u32]``,
  all little-endian;
* an ``Example`` is ``{1: Features}``, ``Features`` is ``{1: map<string, Feature>}`` (a repeated entry message with key 1
  and value 2) and a ``Feature`` is one of ``{1: BytesList, 2: FloatList, 3: Int64List}``, each list being field 1 of its
  message, repeated or packed.

``convert_imagenet`` keeps what the reference's script keeps (the JPEG bytes as they are, the label moved from 1..1000 to
0..999, the bounding boxes, height and width) and rotates output files every ``max_records_per_file`` records under the
reference's names, ``crossbow-<subset>.records.<n>``.  ``write_tfrecord`` writes the same container, for tests and for
users who have images but no TFRecords.
"""
from __future__ import annotations

import glob
import os
import struct
from typing import Dict, Iterable, Iterator, List, Sequence, Tuple, Union

Value = Union[List[bytes], List[float], List[int]]

# ---- crc32c (Castagnoli), masked as TFRecord does ------------------------------------------------------------------------
_TABLE: List[int] = []


def _table() -> List[int]:
    if not _TABLE:
        for i in range(256):
            c = i
            for _ in range(8):
                c = (c >> 1) ^ 0x82F63B78 if c & 1 else c >> 1
            _TABLE.append(c)
    return _TABLE


def crc32c(data: bytes) -> int:
    t, c = _table(), 0xFFFFFFFF
    for b in data:
        c = t[(c ^ b) & 0xFF] ^ (c >> 8)
    return c ^ 0xFFFFFFFF


def masked_crc(data: bytes) -> int:
    c = crc32c(data)
    return ((((c >> 15) | (c << 17)) & 0xFFFFFFFF) + 0xA282EAD8) & 0xFFFFFFFF


# ---- container -------------------------------------------------------------------------------------------------------------
def read_tfrecord(path: str, verify: bool = False) -> Iterator[bytes]:
    """Payloads of one file.  ``verify`` checks both checksums (pure Python: slow on large payloads); the length checksum is
    always checked, so that a file of another kind is refused at its first record."""
    with open(path, "rb") as f:
        index = 0
        while True:
            head = f.read(12)
            if not head:
                return
            if len(head) < 12:
                raise ValueError(f"{path}: truncated header of record {index}")
            n, c = struct.unpack("<QI", head)
            if masked_crc(head[:8]) != c:
                raise ValueError(f"{path}: record {index} has a corrupt length field (not a TFRecord file?)")
            body = f.read(n + 4)
            if len(body) < n + 4:
                raise ValueError(f"{path}: truncated record {index}")
            if verify and masked_crc(body[:n]) != struct.unpack("<I", body[n:])[0]:
                raise ValueError(f"{path}: checksum mismatch in record {index}")
            yield body[:n]
            index += 1


def write_tfrecord(path: str, payloads: Iterable[bytes]) -> int:
    n = 0
    with open(path, "wb") as f:
        for p in payloads:
            head = struct.pack("<Q", len(p))
            f.write(head + struct.pack("<I", masked_crc(head)) + p + struct.pack("<I", masked_crc(p)))
            n += 1
    return n


# ---- protobuf wire format (the subset Example needs) ---------------------------------------------------------------------
def _varint(buf: bytes, i: int) -> Tuple[int, int]:
    shift = value = 0
    while True:
        if i >= len(buf):
            raise ValueError("truncated varint")
        b = buf[i]
        i += 1
        value |= (b & 0x7F) << shift
        if not b & 0x80:
            return value, i
        shift += 7
        if shift > 63:
            raise ValueError("varint longer than 64 bits")


def _fields(buf: bytes) -> Iterator[Tuple[int, int, Union[int, bytes]]]:
    """(field number, wire type, value) of every field of a message; length-delimited values as bytes."""
    i = 0
    while i < len(buf):
        key, i = _varint(buf, i)
        field, wire = key >> 3, key & 7
        if wire == 0:
            v, i = _varint(buf, i)
        elif wire == 1:
            if i + 8 > len(buf):
                raise ValueError("64-bit field runs past the end of its message")
            v, i = buf[i:i + 8], i + 8
        elif wire == 2:
            n, i = _varint(buf, i)
            if i + n > len(buf):
                raise ValueError("length-delimited field runs past the end of its message")
            v, i = buf[i:i + n], i + n
        elif wire == 5:
            if i + 4 > len(buf):
                raise ValueError("32-bit field runs past the end of its message")
            v, i = buf[i:i + 4], i + 4
        else:
            raise ValueError(f"unsupported wire type {wire}")
        yield field, wire, v


def _feature(buf: bytes) -> Value:
    for field, wire, v in _fields(buf):
        if wire != 2:
            continue
        if field == 1:                                   # BytesList
            return [x for f, w, x in _fields(v) if f == 1 and w == 2]
        if field == 2:                                   # FloatList: packed (wire 2) or one fixed32 per value (wire 5)
            out: List[float] = []
            for f, w, x in _fields(v):
                if f == 1 and w == 2:
                    out.extend(struct.unpack(f"<{len(x) // 4}f", x[:len(x) // 4 * 4]))
                elif f == 1 and w == 5:
                    out.append(struct.unpack("<f", x)[0])
            return out
        if field == 3:                                   # Int64List: packed varints or one varint per value
            ints: List[int] = []
            for f, w, x in _fields(v):
                if f == 1 and w == 2:
                    j = 0
                    while j < len(x):
                        n, j = _varint(x, j)
                        ints.append(n - (1 << 64) if n >= 1 << 63 else n)
                elif f == 1 and w == 0:
                    ints.append(x - (1 << 64) if x >= 1 << 63 else x)
            return ints
    return []


def parse_example(payload: bytes) -> Dict[str, Value]:
    """``tf.train.Example`` -> {feature name: list of bytes / floats / ints}."""
    out: Dict[str, Value] = {}
    for f1, w1, features in _fields(payload):
        if f1 != 1 or w1 != 2:
            continue
        for f2, w2, entry in _fields(features):
            if f2 != 1 or w2 != 2:
                continue
            key, value = None, b""
            for f3, w3, x in _fields(entry):
                if f3 == 1 and w3 == 2:
                    key = x.decode("utf-8")
                elif f3 == 2 and w3 == 2:
                    value = x
            if key is not None:
                out[key] = _feature(value)
    return out


# ---- writer of Example messages (tests, and users without TensorFlow) ----------------------------------------------------
def _put_varint(n: int) -> bytes:
    n &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        out.append(b | (0x80 if n else 0))
        if not n:
            return bytes(out)


def _ld(field: int, body: bytes) -> bytes:
    return _put_varint(field << 3 | 2) + _put_varint(len(body)) + body


def make_example(features: Dict[str, Value]) -> bytes:
    entries = b""
    for key, values in features.items():
        if values and isinstance(values[0], (bytes, bytearray)):
            feat = _ld(1, b"".join(_ld(1, bytes(v)) for v in values))
        elif values and isinstance(values[0], float):
            feat = _ld(2, _ld(1, struct.pack(f"<{len(values)}f", *values)))
        else:
            feat = _ld(3, _ld(1, b"".join(_put_varint(int(v)) for v in values)))
        entries += _ld(1, _ld(1, key.encode("utf-8")) + _ld(2, feat))
    return _ld(1, entries)


# ---- ImageNet ------------------------------------------------------------------------------------------------------------
def imagenet_record(example: Dict[str, Value]):
    """(jpeg bytes, label in 0..999, boxes [(xmin, ymin, xmax, ymax)], height, width) of one ImageNet example."""
    jpeg = example.get("image/encoded") or [b""]
    label = example.get("image/class/label") or [0]
    cols = [example.get(f"image/object/bbox/{k}") or [] for k in ("xmin", "ymin", "xmax", "ymax")]
    k = min(len(c) for c in cols)
    boxes = [tuple(float(c[i]) for c in cols) for i in range(k)]
    h = (example.get("image/height") or [0])[0]
    w = (example.get("image/width") or [0])[0]
    return bytes(jpeg[0]), int(label[0]) - 1, boxes, int(h), int(w)


def convert_imagenet(files: Sequence[str], directory: str, subset: str = "train", max_records_per_file: int = 2048,
                     verify: bool = False, limit: int = 0) -> List[str]:
    """Write ``crossbow-<subset>.records.<n>`` files (n from 1) under ``directory``; returns their paths.  ``files`` may hold
    glob patterns (``train-*-of-*``); they are read in sorted order, as the reference's script reads them."""
    from .records import RecordWriter
    paths: List[str] = []
    for f in files:
        paths.extend(sorted(glob.glob(f)) if any(ch in f for ch in "*?[") else [f])
    if not paths:
        raise ValueError("no TFRecord files given")
    os.makedirs(directory, exist_ok=True)
    out: List[str] = []
    writer, in_file, total = None, 0, 0
    for path in paths:
        for payload in read_tfrecord(path, verify):
            jpeg, label, boxes, h, w = imagenet_record(parse_example(payload))
            if not jpeg:
                raise ValueError(f"{path}: example {total} has no image/encoded feature")
            if writer is None:
                out.append(os.path.join(directory, f"crossbow-{subset}.records.{len(out) + 1}"))
                writer, in_file = RecordWriter(out[-1]), 0
            writer.append(jpeg, label, boxes, h, w)
            in_file, total = in_file + 1, total + 1
            if in_file == max_records_per_file:
                writer.close()
                writer = None
            if limit and total >= limit:
                break
        if limit and total >= limit:
            break
    if writer is not None:
        writer.close()
    return out
