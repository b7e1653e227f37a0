"""The qpk1 layer-stream reader against the reference's known-answer bytes and messages."""

import struct

import numpy as np
import pytest

from quantibbler_b200 import qpk1

# crates/quantibbler-qpk1/src/lib.rs:334-344 (the pinned version-1 stream, dout 3, din 5, r 7)
V1_HEX = ("51504b31" "01000000" "01000000" "03000000" "05000000" "07000000"
          "003c003800c0" "003400b80040003c0030" "2b7307" "55e6413503")
# crates/quantibbler-qpk1/src/lib.rs:372-382 (version 2, r 3, bias [1.0, -0.5, 2.0])
V2_HEX = ("51504b31" "02000000" "01000000" "03000000" "05000000" "03000000"
          "003c003800c0" "003400b80040003c0030" "003c00b80040" "7301" "e535")


def test_known_answer_streams():
    a = qpk1.parse(bytes.fromhex(V1_HEX))
    assert (a["version"], a["dout"], a["din"], a["r"], a["dtype"]) == (1, 3, 5, 7, "float16")
    assert a["s1"].tolist() == [1.0, 0.5, -2.0]
    assert a["s2"].tolist() == [0.25, -0.5, 2.0, 1.0, 0.125]
    assert a["bias"] is None
    assert a["ub_packed"].tolist() == [0x2b, 0x73, 0x07]
    assert a["vb_packed"].tolist() == [0x55, 0xe6, 0x41, 0x35, 0x03]
    b = qpk1.parse(bytes.fromhex(V2_HEX))
    assert (b["version"], b["r"]) == (2, 3) and len(bytes.fromhex(V2_HEX)) == 50
    assert b["bias"].tolist() == [1.0, -0.5, 2.0]
    assert b["ub_packed"].tolist() == [0x73, 0x01] and b["vb_packed"].tolist() == [0xe5, 0x35]


def test_float32_scales_and_half_corner_cases():
    dout, din, r = 2, 3, 2
    s = np.array([1.5, -3.25e-7], np.float32), np.array([0.0, 65504.0, 1e-30], np.float32)
    body = s[0].tobytes() + s[1].tobytes() + np.zeros(dout, np.float32).tobytes() + b"\x05" + b"\x2a"
    raw = struct.pack("<4sIIIII", b"QPK1", 2, 2, dout, din, r) + body
    got = qpk1.parse(raw)
    assert np.array_equal(got["s1"], s[0]) and np.array_equal(got["s2"], s[1])
    halves = np.array([6.1e-5, 5.96e-8, -0.0, 65504.0], np.float16)   # normal edge, subnormal, -0, max
    raw = (struct.pack("<4sIIIII", b"QPK1", 1, 1, 4, 1, 1) + halves.tobytes()
           + np.array([2.0], np.float16).tobytes() + b"\x0f" + b"\x01")
    got = qpk1.parse(raw)
    assert np.array_equal(got["s1"], halves.astype(np.float32))
    assert np.signbit(got["s1"][2])


@pytest.mark.parametrize("mutate,text", [
    (lambda b: b[:10], "stream is 10 bytes; shorter than the 24-byte header"),
    (lambda b: b"XPK1" + b[4:], "bad magic [88, 80, 75, 49]; expected [81, 80, 75, 49]"),
    (lambda b: b[:4] + struct.pack("<I", 3) + b[8:], "unsupported representation version 3"),
    (lambda b: b[:8] + struct.pack("<I", 9) + b[12:], "unknown dtype tag 9; expected 1 (float16) or 2 (float32)"),
    (lambda b: b[:12] + struct.pack("<I", 0) + b[16:], "dout, din and r must all be >= 1, got (0, 5, 3)"),
    (lambda b: b[:-1], "truncated stream: 49 bytes; header declares 50"),
    (lambda b: b + b"\x00", "trailing garbage: 51 bytes; one layer at this header is 50"),
])
def test_reader_is_fail_closed_with_the_reference_texts(mutate, text):
    with pytest.raises(ValueError) as err:
        qpk1.parse(mutate(bytes.fromhex(V2_HEX)))
    assert text in str(err.value)


@pytest.mark.gpu
def test_layer_from_stream_matches_explicit_construction(gpu_ctx):
    from quantibbler_b200.gpu import PackedLayer
    rng = np.random.default_rng(5)
    dout, din, r = 70, 130, 24
    ub = rng.random((dout, r)) < 0.5
    vb = rng.random((din, r)) < 0.5
    s1 = (rng.standard_normal(dout) * 0.1).astype(np.float16)
    s2 = (rng.standard_normal(din) * 0.1).astype(np.float16)
    bias = rng.standard_normal(dout).astype(np.float16)
    raw = (struct.pack("<4sIIIII", b"QPK1", 2, 1, dout, din, r) + s1.tobytes() + s2.tobytes()
           + bias.tobytes() + np.packbits(ub, axis=None, bitorder="little").tobytes()
           + np.packbits(vb, axis=None, bitorder="little").tobytes())
    x = rng.standard_normal(din).astype(np.float32)
    a = PackedLayer.from_qpk1(gpu_ctx, raw)
    b = PackedLayer.from_container(gpu_ctx, np.packbits(ub, axis=None, bitorder="little"),
                                   np.packbits(vb, axis=None, bitorder="little"), dout, din, r,
                                   s1.astype(np.float32), s2.astype(np.float32),
                                   bias.astype(np.float32))
    assert np.array_equal(a.apply(x), b.apply(x))
    # the loader's rank gate
    with pytest.raises(ValueError, match=r"r=7 exceeds min\(dout, din\)=3"):
        PackedLayer.from_qpk1(gpu_ctx, bytes.fromhex(V1_HEX))
