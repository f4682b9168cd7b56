"""Checkpoint container format (src/io/safetensor.rs) without a GPU: exact header bytes, padding,
offsets, round trip and the error cases of the reader."""
import io
import json
import struct

import numpy as np
import pytest

from soklyn_b200.function import Precision
from soklyn_b200.safetensor import SafetensorFile, SafetensorWriter, SerdeError


def _sample():
    w = SafetensorWriter()
    w.pass_("layer1.w", [2, 3], np.arange(6, dtype=np.float32).tobytes(), Precision.FP32)
    w.pass_("layer1.b", [3], np.array([1, 2, 3], np.float16).tobytes(), Precision.FP16)
    w.pass_metadata("epoch", "7")
    return w


def test_header_is_sorted_pretty_json_padded_to_eight_bytes():
    buf = io.BytesIO()
    _sample().write(buf)
    raw = buf.getvalue()
    (n,) = struct.unpack("<Q", raw[:8])
    assert n % 8 == 0
    head = raw[8:8 + n].decode()
    expected = ('{\n  "__metadata__": {\n    "epoch": "7"\n  },\n'
                '  "layer1.b": {\n    "data_offsets": [\n      24,\n      30\n    ],\n    "dtype": "F16",\n    "shape": [\n      3\n    ]\n  },\n'
                '  "layer1.w": {\n    "data_offsets": [\n      0,\n      24\n    ],\n    "dtype": "F32",\n    "shape": [\n      2,\n      3\n    ]\n  }\n}')
    assert head.rstrip(" ") == expected and head[len(expected):] == " " * (n - len(expected))
    assert raw[8 + n:8 + n + 24] == np.arange(6, dtype=np.float32).tobytes()      # data in pass order, not key order
    assert len(raw) == 8 + n + 30


def test_round_trip_and_metadata():
    buf = io.BytesIO()
    _sample().write(buf)
    buf.seek(0)
    r = SafetensorWriter.read(buf)
    by = {d["name"]: d for d in r.descriptors}
    assert by["layer1.w"]["shape"] == [2, 3] and by["layer1.w"]["precision"] == Precision.FP32
    assert np.frombuffer(by["layer1.b"]["data"], np.float16).tolist() == [1, 2, 3]
    assert r.metadata == {"epoch": "7"}


def test_reader_rejects_unknown_dtype_and_bad_names():
    head = json.dumps({"layer1.w": {"dtype": "I64", "shape": [1], "data_offsets": [0, 8]}}).encode()
    buf = io.BytesIO(struct.pack("<Q", len(head)) + head + b"\0" * 8)
    with pytest.raises(SerdeError):
        SafetensorWriter.read(buf)
    f = SafetensorFile()
    f.writer.pass_("layerX.w", [1], b"\0\0\0\0", Precision.FP32)
    with pytest.raises(SerdeError):
        f.layer_arrays(Precision.FP32)
    f = SafetensorFile()
    f.writer.pass_("layer1.dv_w", [1], b"\0\0", Precision.FP16)          # moments must be F32
    with pytest.raises(SerdeError):
        f.layer_arrays(Precision.FP16)
    f = SafetensorFile()
    f.writer.pass_("other", [1], b"\0\0\0\0", Precision.FP32)            # non-layer keys are skipped
    assert f.layer_arrays(Precision.FP32) == {}
    with pytest.raises(SerdeError):
        f.into_blocks(None, True, 4)                                       # no layers found


def test_truncated_file():
    buf = io.BytesIO()
    _sample().write(buf)
    with pytest.raises(SerdeError):
        SafetensorWriter.read(io.BytesIO(buf.getvalue()[:-4]))
