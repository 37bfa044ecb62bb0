"""TFRecord / tf.train.Example codec and the inference output writers."""

import io
import json
import struct

import numpy as np
import pytest
import torch

from axlearn_b200.common import tfrecord
from axlearn_b200.common.inference_output import (
    InputOutputRecordWriter,
    JsonlExampleRecordSink,
    OutputRecordWriter,
    TfExampleRecordSink,
)


def test_crc32c_known_vectors():
    # RFC 3720 appendix B.4 vectors.
    assert tfrecord.crc32c(b"123456789") == 0xE3069283
    assert tfrecord.crc32c(bytes(32)) == 0x8A9136AA
    assert tfrecord.crc32c(bytes([0xFF] * 32)) == 0x62A8AB43
    assert tfrecord.crc32c(bytes(range(32))) == 0x46DD794E
    assert tfrecord.crc32c(b"") == 0


def test_record_framing_round_trip_and_corruption():
    buf = io.BytesIO()
    w = tfrecord.TFRecordWriter(buf)
    recs = [b"", b"a", b"hello world" * 100, bytes(range(256))]
    for r in recs:
        w.write(r)
    raw = buf.getvalue()
    # First frame: zero length, crc of the 8 length bytes, no data, crc of the empty string.
    assert raw[:8] == struct.pack("<Q", 0)
    assert struct.unpack("<I", raw[12:16])[0] == tfrecord.masked_crc32c(b"") == 0xA282EAD8
    assert list(tfrecord.read_tfrecords(io.BytesIO(raw))) == recs
    bad = bytearray(raw)
    bad[-6] ^= 1
    with pytest.raises(ValueError, match="corrupt"):
        list(tfrecord.read_tfrecords(io.BytesIO(bytes(bad))))
    with pytest.raises(ValueError, match="truncated"):
        list(tfrecord.read_tfrecords(io.BytesIO(raw[:-3])))


def test_example_bytes_are_the_protobuf_wire_format():
    # One int64 feature "a" = [1, 300]: hand-assembled bytes of Example{features{feature{"a": int64_list{1,300}}}}.
    int_list = bytes([0x0A, 0x03, 0x01, 0xAC, 0x02])          # field 1 packed: 1, 300
    feature = bytes([0x1A, len(int_list)]) + int_list           # field 3 (int64_list)
    entry = bytes([0x0A, 0x01]) + b"a" + bytes([0x12, len(feature)]) + feature
    features = bytes([0x0A, len(entry)]) + entry
    want = bytes([0x0A, len(features)]) + features
    assert tfrecord.encode_example({"a": np.array([1, 300])}) == want
    got = tfrecord.decode_example(want)
    assert got["a"].tolist() == [1, 300]


def test_example_round_trip_all_kinds():
    ex = {"f": np.array([[1.5, -2.25], [0.0, 3.0]], np.float32), "i": np.array([-1, 0, 2**40]),
          "b": np.array([True, False]), "s": [b"ab", "cd"], "one": "x", "empty": np.zeros([0], np.int64)}
    got = tfrecord.decode_example(tfrecord.encode_example(ex))
    assert got["f"].tolist() == [1.5, -2.25, 0.0, 3.0] and got["f"].dtype == np.float32
    assert got["i"].tolist() == [-1, 0, 2**40]
    assert got["b"].tolist() == [1, 0]
    assert got["s"] == [b"ab", b"cd"] and got["one"] == [b"x"]
    assert len(got["empty"]) == 0


def _batches():
    inp = {"input_ids": torch.arange(6).reshape(3, 2), "text": [b"a", b"b", b"c"]}
    out = {"logits": torch.tensor([[0.5, 1.0], [2.0, 3.0], [4.0, 5.0]], dtype=torch.bfloat16),
           "nested": {"score": torch.tensor([1.0, 2.0, 3.0])}}
    return inp, out


def test_output_record_writer_tfrecord(tmp_path):
    path = str(tmp_path / "out" / "records-{process_index:05d}-of-{process_count:05d}.tfrecord")
    w = OutputRecordWriter.default_config().set(
        name="w", sink=TfExampleRecordSink.default_config().set(output_path=path)).instantiate(parent=None)
    inp, out = _batches()
    w.write(input_batch=inp, output_batch=out)
    w.flush()
    recs = [tfrecord.decode_example(r) for r in tfrecord.read_tfrecords(str(tmp_path / "out" / "records-00000-of-00001.tfrecord"))]
    assert len(recs) == 3
    assert sorted(recs[0]) == ["logits", "nested/score"]          # outputs only
    assert recs[1]["logits"].tolist() == [2.0, 3.0] and recs[2]["nested/score"].tolist() == [3.0]


def test_input_output_record_writer_jsonl(tmp_path):
    path = str(tmp_path / "out.jsonl")
    w = InputOutputRecordWriter.default_config().set(
        name="w", sink=JsonlExampleRecordSink.default_config().set(output_path=path)).instantiate(parent=None)
    inp, out = _batches()
    w.write(input_batch=inp, output_batch=out)
    w.flush()
    lines = [json.loads(l) for l in open(path, encoding="utf-8")]
    assert len(lines) == 3
    assert lines[2] == {"input/input_ids": [4, 5], "input/text": "c", "output/logits": [4.0, 5.0],
                        "output/nested/score": 3.0}


def test_tfrecord_source_reads_files_written_by_the_sink(tmp_path):
    from axlearn_b200.common import input_pipeline as ip

    paths = []
    for f in range(2):
        p = str(tmp_path / f"d-{f}.tfrecord")
        with tfrecord.TFRecordWriter(p) as w:
            for i in range(3):
                w.write(tfrecord.encode_example({"text": f"doc {f}-{i}", "label": i, "ids": np.arange(i + 1)}))
        paths.append(p)
    src = ip.TFRecordSource(paths, {"text": "str", "label": "int", "ids": "array"}, check_crc=True)
    assert len(src) == 6
    row = src[4]
    assert row["text"] == "doc 1-1" and row["label"] == 1 and row["ids"].tolist() == [0, 1]
    rows = list(ip.read(src))
    assert [r["text"] for r in rows] == [f"doc {f}-{i}" for f in range(2) for i in range(3)]
    with open(paths[0], "ab") as f:
        f.write(b"\x01\x02\x03")
    with pytest.raises(ValueError, match="truncated"):
        ip.TFRecordSource(paths)
