"""Reader of the single-file qpk1 blob (``QKPB``), host only.

Mirrors ``Blob::parse`` / ``validate_payload`` of crates/quantibbler-qpk1/src/blob.rs:226-398
(metadata rules :482-538, header fields :540-590) and ``load_blob`` / ``build_from_blob`` of
crates/quantibbler-qpk1/src/loader.rs:372-560,649-700; the layout is the one
src/quantibbler/blob.py:99-157 writes:

    "QKPB" | u32 version (1) | u32 header_len | header JSON | zeros to the next 4096 boundary
    u32 section count | per section: u8 name_len, name, u8 tag, u64 offset, u64 length
    zeros to the next 4096 boundary | payloads at 4096-aligned offsets, canonical order

Fail-closed, with the reference's refusal texts prefixed by the file's path.  The result is
the same ``ModelDirectory`` the directory reader gives, marked as coming from a blob: a blob
is served at the dtype its header declares (crates/quantibbler-server/src/model/mod.rs:725-734),
so a ``bf16`` blob selects bfloat16 serving in ``model_dir.decoder_inputs``.
"""

from __future__ import annotations

import json
import os
import struct

import numpy as np

from . import qpk1
from .model_dir import (ModelDirectory, ModelDirError, _ITEMSIZE, _quote, _slot_width,
                        _validate_config)

BLOB_MAGIC = b"QKPB"
BLOB_VERSION = 1
PAGE_SIZE = 4096
MAX_HEADER_BYTES = 16 << 20          # blob.rs:42
CHAT_TEMPLATE_FILE = "chat_template.jinja"
TAG_NAMES = {0: "qpk1_v1", 1: "qpk1_v2", 2: "fp32_le", 3: "bf16_le", 4: "raw"}
_STREAM_VERSION = {0: 1, 1: 2}
_TAG_DTYPE = {2: "fp32", 3: "bf16"}


class _Reader:
    def __init__(self, data: bytes):
        self.data, self.at = data, 0

    def take(self, n: int, what: str) -> bytes:
        if self.at + n > len(self.data):
            raise ModelDirError(f"truncated {what}: needs {n} byte(s): failed to fill whole buffer")
        out = self.data[self.at:self.at + n]
        self.at += n
        return out


def _next_page(x: int) -> int:
    return -(-x // PAGE_SIZE) * PAGE_SIZE


def _header_fields(value) -> dict:
    """blob.rs:540-590: required fields and their JSON types."""
    if not isinstance(value, dict):
        raise ModelDirError("blob header JSON is not an object")

    def need(field, ok, what):
        if field not in value:
            raise ModelDirError(f"blob header is missing the required field {_quote(field)}")
        if not ok(value[field]):
            raise ModelDirError(f"header field {_quote(field)} must be {what}")
        return value[field]

    def is_uint(v):
        return isinstance(v, int) and not isinstance(v, bool) and v >= 0

    def is_number(v):
        return isinstance(v, (int, float)) and not isinstance(v, bool)

    def is_str_list(v):
        return isinstance(v, list) and all(isinstance(s, str) for s in v)

    h = {"model_id": need("model_id", lambda v: isinstance(v, str), "a JSON string")}
    for f in ("vocab_size", "d_model", "n_layers", "n_heads", "n_kv_heads", "head_dim"):
        h[f] = need(f, is_uint, "a non-negative integer")
    for f in ("eos_token_id", "bos_token_id"):
        h[f] = need(f, lambda v: is_uint(v) and v < 1 << 32, "an integer in u32 range")
    for f in ("rms_norm_eps", "rope_theta"):
        h[f] = float(need(f, is_number, "a JSON number"))
    for f in ("norm_slots", "layers"):
        h[f] = need(f, is_str_list, "a JSON array of strings")
    h["weight_tying"] = need("weight_tying", lambda v: v is None or isinstance(v, str),
                             "a JSON string or null")
    token = need("remainder_dtype", lambda v: isinstance(v, str), "a JSON string")
    if token not in _ITEMSIZE:
        raise ModelDirError(f"header field `remainder_dtype` is {_quote(token)}; declared dtypes "
                            "are fp32 and bf16")
    h["remainder_dtype"] = token
    if "created_by" in value and not isinstance(value["created_by"], str):
        raise ModelDirError("header field `created_by` must be a JSON string; found another type")
    h["created_by"] = value.get("created_by")
    return h


def _order_key(name: str, layers: list):
    if name in layers:
        return (0, f"{layers.index(name):08d}")
    fixed = {"embedding": (1, "0"), "lm_head": (1, "1"), "norms": (1, "2")}
    if name in fixed:
        return fixed[name]
    if name.startswith("tokenizer."):
        return (2, name)
    if name == CHAT_TEMPLATE_FILE:
        return (3, name)
    return (9, name)


def parse(data: bytes):
    """``(header, sections)`` of a blob held in memory, metadata and payload rules checked
    (blob.rs ``parse_bytes``).  A section is ``{"name", "tag", "offset", "length"}``."""
    data = bytes(data)
    r = _Reader(data)
    if len(data) < 4:
        raise ModelDirError("bad blob magic: the file is shorter than 4 bytes "
                            "(failed to fill whole buffer)")
    magic = r.take(4, "blob magic")
    if magic != BLOB_MAGIC:
        raise ModelDirError(f"bad blob magic {list(magic)}; expected QKPB {list(BLOB_MAGIC)}")
    version = struct.unpack("<I", r.take(4, "blob version"))[0]
    if version != BLOB_VERSION:
        raise ModelDirError(f"unsupported blob format version {version}; this reader implements "
                            f"{BLOB_VERSION}")
    header_len = struct.unpack("<I", r.take(4, "blob header length"))[0]
    if header_len > MAX_HEADER_BYTES:
        raise ModelDirError(f"blob header declares {header_len} bytes, above the "
                            f"{MAX_HEADER_BYTES}-byte cap")
    header_end = 12 + header_len
    raw = r.take(header_len, "blob header")
    try:
        text = raw.decode("utf-8")
    except UnicodeDecodeError as e:
        raise ModelDirError(f"blob header is not valid UTF-8: {e}") from None
    try:
        value = json.loads(text)
    except json.JSONDecodeError as e:
        raise ModelDirError(f"blob header is not valid JSON: {e}") from None
    header = _header_fields(value)

    table_start = _next_page(header_end)
    padding = r.take(table_start - header_end, "blob header padding")
    if any(padding):
        pos = next(i for i, b in enumerate(padding) if b)
        raise ModelDirError(f"non-zero header padding byte at offset {header_end + pos}; "
                            "padding must be 0x00")
    count = struct.unpack("<I", r.take(4, "section table count"))[0]
    sections = []
    for index in range(count):
        name_len = r.take(1, "section table name length")[0]
        name_raw = r.take(name_len, "section table name")
        try:
            name = name_raw.decode("utf-8")
        except UnicodeDecodeError as e:
            raise ModelDirError(f"section table entry {index} has a non-UTF-8 name: {e}") from None
        tag = r.take(1, "section table tag")[0]
        if tag not in TAG_NAMES:
            raise ModelDirError(f"section {_quote(name)}: unknown section dtype tag {tag}; the "
                                "vocabulary is 0 qpk1_v1, 1 qpk1_v2, 2 fp32_le, 3 bf16_le, 4 raw")
        offset, length = struct.unpack("<QQ", r.take(16, "section table offset"))
        sections.append({"name": name, "tag": tag, "offset": offset, "length": length})
    table_end = r.at

    # metadata rules (blob.rs:482-538)
    seen, previous = set(), None
    layers = header["layers"]
    for s in sections:
        name = s["name"]
        declared = (name in layers or name in ("embedding", "lm_head", "norms")
                    or name.startswith("tokenizer.") or name == CHAT_TEMPLATE_FILE)
        if not name or not declared:
            raise ModelDirError(f"unknown section name {_quote(name)}; expected a declared layer, "
                                "embedding, lm_head, norms, tokenizer.*, or the chat-template "
                                "sidecar")
        if name in seen:
            raise ModelDirError(f"duplicate section name {_quote(name)}")
        seen.add(name)
        if s["offset"] + s["length"] >= 1 << 64:
            raise ModelDirError(f"section {_quote(name)}: offset {s['offset']} + length "
                                f"{s['length']} overflows u64")
        if s["offset"] % PAGE_SIZE:
            raise ModelDirError(f"section {_quote(name)}: offset {s['offset']} is not "
                                f"{PAGE_SIZE}-aligned")
        if s["offset"] < table_end:
            raise ModelDirError(f"section {_quote(name)}: offset {s['offset']} aliases the "
                                f"metadata region (the section table ends at {table_end}); a "
                                "section cannot start inside the magic/header/table bytes")
        key = _order_key(name, layers)
        if previous is not None and previous >= key:
            raise ModelDirError(f"section {_quote(name)} is out of canonical order (after "
                                f"{_quote(previous[1])}); the order is layers, then "
                                "embedding/lm_head/norms, then tokenizer.*, then the "
                                "chat-template sidecar")
        previous = key

    # payload rules (blob.rs:343-398)
    file_len = len(data)
    for s in sections:
        end = s["offset"] + s["length"]
        if end > file_len:
            raise ModelDirError(f"section {_quote(s['name'])}: range [{s['offset']} , {end}) runs "
                                f"past the {file_len}-byte file")
    ordered = sorted(sections, key=lambda s: s["offset"])
    for a, b in zip(ordered, ordered[1:]):
        if a["offset"] + a["length"] > b["offset"]:
            raise ModelDirError(
                f"sections {_quote(a['name'])} and {_quote(b['name'])} overlap: [{a['offset']}, "
                f"{a['offset'] + a['length']}) intersects [{b['offset']}, "
                f"{b['offset'] + b['length']})")
    cursor = table_end
    for s in ordered:
        if s["offset"] > cursor:
            gap = data[cursor:s["offset"]]
            if any(gap):
                pos = next(i for i, b in enumerate(gap) if b)
                raise ModelDirError(f"non-zero inter-payload padding byte at offset {cursor + pos}; "
                                    "padding must be 0x00")
        cursor = max(cursor, s["offset"] + s["length"])
    if cursor < file_len:
        raise ModelDirError(f"trailing bytes: {file_len - cursor} byte(s) begin at offset "
                            f"{cursor}, after the last section's end")
    return header, sections


def _tying(header: dict):
    """(path, dtype token) of ``weight_tying`` or None for null (blob.rs:147-185)."""
    wt = header["weight_tying"]
    if wt is None:
        return None
    if not wt.startswith("lm_head=") or "@" not in wt:
        raise ModelDirError(f"unknown weight_tying {_quote(wt)}; documented forms: null or "
                            '"lm_head=<path>@<dtype>" with dtype fp32 or bf16')
    path, token = wt[len("lm_head="):].rsplit("@", 1)
    if not path:
        raise ModelDirError(f"weight_tying {_quote(wt)} names an empty path; the form is "
                            '"lm_head=<path>@<dtype>"')
    if token not in _ITEMSIZE:
        raise ModelDirError(f"weight_tying {_quote(wt)} declares an undeclared dtype token "
                            f"{_quote(token)}; declared dtypes are fp32 and bf16")
    return path, token


def _widen(raw: bytes, dtype: str) -> np.ndarray:
    if dtype == "bf16":
        return (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
    return np.frombuffer(raw, dtype="<f4").astype(np.float32)


def load_blob(path: str) -> ModelDirectory:
    """loader.rs:372-560: a blob file as a ``ModelDirectory``."""
    path = os.fspath(path)
    try:
        with open(path, "rb") as f:
            data = f.read()
    except OSError as e:
        raise ModelDirError(f"{path}: {e.strerror}") from None
    if not data:
        raise ModelDirError(f"{path}: an empty file is not a qpk1 blob")
    try:
        header, sections = parse(data)
        config = {k: header[k] for k in ("vocab_size", "d_model", "eos_token_id", "bos_token_id",
                                         "n_layers", "n_heads", "n_kv_heads", "head_dim",
                                         "rms_norm_eps", "rope_theta", "norm_slots")}
        if header["weight_tying"] is not None:
            config["weight_tying"] = header["weight_tying"]
    except ModelDirError as e:
        raise ModelDirError(f"{path}: {e}") from None
    _validate_config(config, path)
    dtype = header["remainder_dtype"]
    try:
        tying = _tying(header)
    except ModelDirError as e:
        raise ModelDirError(f"{path}: {e}") from None
    if tying is not None and tying[1] != dtype:
        raise ModelDirError(f"{path}: weight_tying declares @{tying[1]} but the header declares "
                            f'remainder_dtype "{dtype}"; a remainder set cannot hold two dtypes')
    by_name = {s["name"]: s for s in sections}

    def payload(s):
        return data[s["offset"]:s["offset"] + s["length"]]

    layers = []
    for name in header["layers"]:
        s = by_name.get(name)
        if s is None:
            raise ModelDirError(f"{path}: blob is missing the required layer section {_quote(name)}")
        if s["tag"] not in _STREAM_VERSION:
            raise ModelDirError(f"{path}: layer section {_quote(name)} is tagged "
                                f"{TAG_NAMES[s['tag']]}; a layer section must carry a qpk1 stream "
                                "(tag 0 qpk1_v1 or 1 qpk1_v2)")
        try:
            layer = qpk1.parse(np.frombuffer(payload(s), dtype=np.uint8))
        except ValueError as e:
            raise ModelDirError(f"{path}: section {_quote(name)}: {e}") from None
        if _STREAM_VERSION[s["tag"]] != layer["version"]:
            raise ModelDirError(f"{path}: layer section {_quote(name)} is tagged "
                                f"{TAG_NAMES[s['tag']]} but its stream header declares version "
                                f"{layer['version']}")
        if layer["r"] > min(layer["dout"], layer["din"]):
            raise ModelDirError(f"{path}: section {_quote(name)}: rank r={layer['r']} exceeds "
                                f"min(dout, din)={min(layer['dout'], layer['din'])}")
        layers.append((name, layer))

    def remainder(name, count):
        s = by_name.get(name)
        if s is None:
            raise ModelDirError(f"{path}: blob is missing the required section {_quote(name)}")
        if s["tag"] not in _TAG_DTYPE:
            raise ModelDirError(f"{path}: remainder section {_quote(name)} is tagged "
                                f"{TAG_NAMES[s['tag']]}; a remainder section must be fp32_le "
                                "(tag 2) or bf16_le (tag 3)")
        if _TAG_DTYPE[s["tag"]] != dtype:
            raise ModelDirError(f"{path}: remainder section {_quote(name)} is tagged "
                                f"{TAG_NAMES[s['tag']]} but the header declares remainder_dtype "
                                f'"{dtype}"')
        expected = count * _ITEMSIZE[dtype]
        if s["length"] != expected:
            raise ModelDirError(f"{path}: remainder section {_quote(name)} is {s['length']} bytes; "
                                f"expected exactly {expected} bytes (a {count}-element remainder "
                                f"declared @{dtype})")
        return _widen(payload(s), dtype)

    vocab, d = header["vocab_size"], header["d_model"]
    embedding = remainder("embedding", vocab * d).reshape(vocab, d)
    if "lm_head" in by_name:
        lm_head = remainder("lm_head", vocab * d).reshape(vocab, d)
    elif tying is None or tying[0] != "e1":
        raise ModelDirError(f'{path}: blob is missing the required section "lm_head" (the header '
                            "declares an untied head, so the head is not the embedding)")
    else:
        lm_head = None
    per_block = sum(_slot_width(s, d, header["head_dim"]) for s in header["norm_slots"])
    norm_weights = remainder("norms", per_block * header["n_layers"] + d)
    tok = by_name.get("tokenizer.json")
    if tok is None:
        raise ModelDirError(f'{path}: blob is missing the required section "tokenizer.json"')
    if tok["tag"] != 4:
        raise ModelDirError(f'{path}: section "tokenizer.json" is tagged {TAG_NAMES[tok["tag"]]}; '
                            "tokenizer sections are raw (tag 4)")
    return ModelDirectory(
        model_id=header["model_id"], layers=layers, eos_token_id=header["eos_token_id"],
        bos_token_id=header["bos_token_id"], vocab_size=vocab, d_model=d,
        n_layers=header["n_layers"], n_heads=header["n_heads"], n_kv_heads=header["n_kv_heads"],
        head_dim=header["head_dim"], rms_norm_eps=header["rms_norm_eps"],
        rope_theta=header["rope_theta"], norm_slots=list(header["norm_slots"]),
        remainder_dtype=dtype, embedding=embedding, lm_head=lm_head, norm_weights=norm_weights,
        extras={"source": "blob", "tokenizer_json": payload(tok),
                "created_by": header["created_by"]})


def load_any(path: str) -> ModelDirectory:
    """loader.rs:318-348 (``ModelDirectory::load``): a directory goes to the directory reader, a
    regular file must be a blob."""
    from . import model_dir
    path = os.fspath(path)
    if os.path.isdir(path):
        return model_dir.load(path)
    if not os.path.isfile(path):
        if not os.path.exists(path):
            raise ModelDirError(f"{path}: No such file or directory")
        raise ModelDirError(f"model path {path} is neither a directory nor a regular file")
    with open(path, "rb") as f:
        magic = f.read(4)
    if magic == BLOB_MAGIC:
        return load_blob(path)
    raise ModelDirError(f"model file {path} is not a qpk1 blob: its first four bytes are not "
                        f"{list(BLOB_MAGIC)}. A regular file is only ever read as a blob; the "
                        "legacy directory format is read from a directory path")
