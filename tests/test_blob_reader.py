"""The single-file blob reader against blobs written by the reference's own writer.

tests/golden/parity-tiny.qpk and parity-tiny-bf16.qpk were produced by
``quantibbler.blob.write_blob_from_directory`` (src/quantibbler/blob.py) from the reference's
parity-tiny model directory, at both remainder dtypes.  The reader must give what the
directory reader gives, select the serving dtype the header declares, and refuse damaged
files with the texts of crates/quantibbler-qpk1/src/blob.rs and loader.rs.  No GPU needed.
"""

import json
import os
import struct

import numpy as np
import pytest

from conftest import GOLDEN
from oracle import decoder_np
from quantibbler_b200 import blob, model_dir
from quantibbler_b200.model_dir import ModelDirError

FP32 = os.path.join(GOLDEN, "parity-tiny.qpk")
BF16 = os.path.join(GOLDEN, "parity-tiny-bf16.qpk")
DIRECTORY = os.path.join(GOLDEN, "parity-tiny")


def test_blob_equals_the_directory_it_was_packed_from():
    a, b = model_dir.load(DIRECTORY), blob.load_any(FP32)
    assert blob.load_any(DIRECTORY).model_id == a.model_id      # a directory path still works
    assert [n for n, _ in a.layers] == [n for n, _ in b.layers]
    for (_, la), (_, lb) in zip(a.layers, b.layers):
        assert (la["dout"], la["din"], la["r"], la["version"]) == (
            lb["dout"], lb["din"], lb["r"], lb["version"])
        for k in ("s1", "s2", "ub_packed", "vb_packed"):
            assert np.array_equal(la[k], lb[k])
    assert np.array_equal(a.embedding, b.embedding) and np.array_equal(a.lm_head, b.lm_head)
    assert np.array_equal(a.norm_weights, b.norm_weights)
    assert (a.norm_slots, a.rms_norm_eps, a.rope_theta, a.eos_token_id) == (
        b.norm_slots, b.rms_norm_eps, b.rope_theta, b.eos_token_id)
    assert b.extras["source"] == "blob" and b.extras["created_by"] == "make_golden"
    assert json.loads(b.extras["tokenizer_json"])     # carried verbatim as a raw section
    cfg, _ = model_dir.decoder_inputs(b)
    assert cfg.serving == "float32"


def test_bf16_blob_selects_bfloat16_serving_and_stays_inside_the_budget():
    md = blob.load_any(BF16)
    assert md.remainder_dtype == "bf16"
    ref = model_dir.load(DIRECTORY)
    # every remainder value is the bfloat16 rounding of the directory's float32 value
    assert np.array_equal(md.embedding, decoder_np._bf16(ref.embedding))
    assert np.array_equal(md.norm_weights, decoder_np._bf16(ref.norm_weights))
    cfg, w = model_dir.decoder_inputs(md, max_seq=16)
    assert cfg.serving == "bfloat16"       # model/mod.rs:725-734
    with open(os.path.join(DIRECTORY, "goldens.json")) as f:
        g = json.load(f)
    s = decoder_np.Session(cfg, w)
    worst = max(float(np.abs(s.step(t)[1] - np.asarray(g["logits"][p], np.float32)).max())
                for p, t in enumerate(g["input_ids"]))
    assert worst <= 1e-2


def _blob_bytes():
    with open(FP32, "rb") as f:
        return bytearray(f.read())


def _load_bytes(tmp_path, data):
    p = tmp_path / "m.qpk"
    p.write_bytes(bytes(data))
    return blob.load_any(str(p))


def _table_start(data):
    return -(-(12 + struct.unpack("<I", data[8:12])[0]) // 4096) * 4096


def test_prefix_refusals(tmp_path):
    data = _blob_bytes()
    with pytest.raises(ModelDirError, match="is not a qpk1 blob: its first four bytes are not"):
        _load_bytes(tmp_path, b"QPK1" + bytes(data[4:]))
    bad = bytearray(data); bad[4:8] = struct.pack("<I", 2)
    with pytest.raises(ModelDirError, match="unsupported blob format version 2; this reader implements 1"):
        _load_bytes(tmp_path, bad)
    bad = bytearray(data); bad[8:12] = struct.pack("<I", (16 << 20) + 1)
    with pytest.raises(ModelDirError, match="above the 16777216-byte cap"):
        _load_bytes(tmp_path, bad)
    bad = bytearray(data); bad[12] = ord("[")
    with pytest.raises(ModelDirError, match="blob header is not valid JSON"):
        _load_bytes(tmp_path, bad)
    bad = bytearray(data); bad[12 + struct.unpack("<I", data[8:12])[0] + 5] = 1
    with pytest.raises(ModelDirError, match="non-zero header padding byte at offset"):
        _load_bytes(tmp_path, bad)
    with pytest.raises(ModelDirError, match="truncated section table"):
        _load_bytes(tmp_path, data[:_table_start(data) + 9])
    (tmp_path / "empty.qpk").write_bytes(b"")
    with pytest.raises(ModelDirError, match="is not a qpk1 blob"):
        blob.load_any(str(tmp_path / "empty.qpk"))
    with pytest.raises(ModelDirError, match="an empty file is not a qpk1 blob"):
        blob.load_blob(str(tmp_path / "empty.qpk"))


def _rewrite_header(data, change):
    """The same blob with an edited header JSON (same length class: the padding absorbs it)."""
    hl = struct.unpack("<I", data[8:12])[0]
    header = json.loads(bytes(data[12:12 + hl]))
    change(header)
    raw = json.dumps(header, sort_keys=True, separators=(",", ":")).encode()
    start = _table_start(data)
    assert 12 + len(raw) <= start
    return bytearray(b"QKPB" + struct.pack("<II", 1, len(raw)) + raw
                     + bytes(start - 12 - len(raw)) + bytes(data[start:]))


@pytest.mark.parametrize("change,text", [
    (lambda h: h.pop("n_heads"), 'blob header is missing the required field "n_heads"'),
    (lambda h: h.update(vocab_size="128"), 'header field "vocab_size" must be a non-negative integer'),
    (lambda h: h.update(remainder_dtype="fp16"), 'header field `remainder_dtype` is "fp16"; declared dtypes are fp32 and bf16'),
    (lambda h: h.update(remainder_dtype="bf16"), 'weight_tying declares @fp32 but the header declares remainder_dtype "bf16"'),
    (lambda h: h.update(head_dim=16), "n_kv_heads * head_dim = 32 != d_model 64 (GQA width mismatch)"),
    (lambda h: h.update(layers=h["layers"][1:]), "unknown section name"),
    (lambda h: h.update(layers=h["layers"][::-1]), "is out of canonical order"),
    (lambda h: h.update(norm_slots=["input", "post_attention"]), 'remainder section "norms" is 1792 bytes; expected exactly 1280 bytes'),
    (lambda h: h.update(created_by=3), "header field `created_by` must be a JSON string"),
])
def test_header_refusals(tmp_path, change, text):
    with pytest.raises(ModelDirError) as info:
        _load_bytes(tmp_path, _rewrite_header(_blob_bytes(), change))
    assert text in str(info.value) and "m.qpk: " in str(info.value)


def _sections(data):
    at = _table_start(data)
    count = struct.unpack("<I", data[at:at + 4])[0]
    at += 4
    out = []
    for _ in range(count):
        n = data[at]
        name = bytes(data[at + 1:at + 1 + n]).decode()
        tag_at = at + 1 + n
        out.append((name, tag_at))
        at = tag_at + 17
    return out


def test_section_table_refusals(tmp_path):
    data = _blob_bytes()
    secs = dict(_sections(data))
    name = "layers.0.inner.mlp.gate_proj"
    bad = bytearray(data); bad[secs[name]] = 9
    with pytest.raises(ModelDirError, match=f'section "{name}": unknown section dtype tag 9'):
        _load_bytes(tmp_path, bad)
    bad = bytearray(data); bad[secs[name]] = 2
    with pytest.raises(ModelDirError, match="is tagged fp32_le; a layer section must carry a qpk1 stream"):
        _load_bytes(tmp_path, bad)
    bad = bytearray(data); bad[secs[name]] ^= 1       # v1 <-> v2
    with pytest.raises(ModelDirError, match="but its stream header declares version"):
        _load_bytes(tmp_path, bad)
    bad = bytearray(data); bad[secs["embedding"]] = 3
    with pytest.raises(ModelDirError, match='remainder section "embedding" is tagged bf16_le but the '
                                            'header declares remainder_dtype "fp32"'):
        _load_bytes(tmp_path, bad)
    bad = bytearray(data); bad[secs["tokenizer.json"]] = 2
    with pytest.raises(ModelDirError, match='section "tokenizer.json" is tagged fp32_le; tokenizer '
                                            "sections are raw"):
        _load_bytes(tmp_path, bad)
    off_at = secs["norms"] + 1
    off = struct.unpack("<Q", data[off_at:off_at + 8])[0]
    bad = bytearray(data); bad[off_at:off_at + 8] = struct.pack("<Q", off + 8)
    with pytest.raises(ModelDirError, match=f'section "norms": offset {off + 8} is not 4096-aligned'):
        _load_bytes(tmp_path, bad)
    bad = bytearray(data); bad[off_at:off_at + 8] = struct.pack("<Q", 0)
    with pytest.raises(ModelDirError, match="aliases the metadata region"):
        _load_bytes(tmp_path, bad)
    with pytest.raises(ModelDirError, match="runs past the"):
        _load_bytes(tmp_path, data[:-10])
    with pytest.raises(ModelDirError, match="trailing bytes: 3 byte"):
        _load_bytes(tmp_path, bytes(data) + b"\0\0\0")
    tok_at = secs["tokenizer.json"] + 1
    tok_off = struct.unpack("<Q", data[tok_at:tok_at + 8])[0]
    bad = bytearray(data); bad[tok_off - 1] = 7       # the zero gap after the 1792-byte norms
    with pytest.raises(ModelDirError, match="non-zero inter-payload padding byte at offset"):
        _load_bytes(tmp_path, bad)
