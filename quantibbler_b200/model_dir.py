"""Reader of a qpk1 model directory (host only): manifest, config, layers, sidecars.

Mirrors ``load`` of crates/quantibbler-qpk1/src/loader.rs:172-312 (manifest.toml and
config.toml checks :855-1023, path containment :705-727, exact-size remainder files
:777-805, the declared norm inventory :111-170) and the per-block resolution of
crates/quantibbler-server/src/engine/mod.rs:510-580 (projections by their manifest names
``layers.<b>.inner.self_attn.q_proj`` ..., norm vectors by walking the inventory).  Every
layer stream goes through the library's qpk1 reader; a refusal is a ``ValueError`` whose
text starts with the offending file, as in the reference.

``load`` returns a ``ModelDirectory``; ``decoder_inputs`` turns it into the
``DecoderConfig`` and weight dictionary that ``quantibbler_b200.decoder.Decoder`` takes.
A directory is always served in float32 (crates/quantibbler-server/src/model/mod.rs:725-734:
bfloat16 serving is reachable only through single-file blobs, which ``blob.py`` reads into the
same ``ModelDirectory``).
"""

from __future__ import annotations

import math
import os
import stat
import tomllib
from dataclasses import dataclass, field

import numpy as np

from . import _lib, qpk1
from ._lib import check

MAX_LAYER_BYTES = 4 << 30      # loader.rs:51
MAX_SIDECAR_BYTES = 4 << 30    # loader.rs:55
MAX_DIM = 1 << 26              # loader.rs:59
MAX_LAYERS = 1 << 12           # loader.rs:63
NORM_SLOTS = ("input", "post_attention", "q_norm", "k_norm", "post_feedforward")
PROJECTIONS = {"q": "self_attn.q_proj", "k": "self_attn.k_proj", "v": "self_attn.v_proj",
               "o": "self_attn.o_proj", "gate": "mlp.gate_proj", "up": "mlp.up_proj",
               "down": "mlp.down_proj"}
_ITEMSIZE = {"fp32": 4, "bf16": 2}


class ModelDirError(ValueError):
    """A refused model directory; the text names the file that caused it."""


def _quote(s: str) -> str:
    return '"' + str(s).replace("\\", "\\\\").replace('"', '\\"') + '"'


def _slot_width(slot: str, d_model: int, head_dim: int) -> int:
    return head_dim if slot in ("q_norm", "k_norm") else d_model


def contained_join(base: str, rel: str) -> str:
    """loader.rs:705-727: a relative path that stays inside ``base``."""
    if rel == "":
        raise ModelDirError("path is empty")
    if rel.startswith("/"):
        raise ModelDirError("absolute paths are not allowed")
    depth = 0
    for comp in rel.split("/"):
        if comp == "..":
            raise ModelDirError("'..' components are not allowed")
        if comp not in ("", "."):
            depth += 1
    if depth == 0:
        raise ModelDirError("path names no file")
    return os.path.join(base, rel)


def _stat_regular_capped(path: str, cap: int, what: str) -> int:
    try:
        st = os.lstat(path)
    except OSError as e:
        raise ModelDirError(f"{path}: {e.strerror}") from None
    if not stat.S_ISREG(st.st_mode):
        raise ModelDirError(f"{path}: not a regular file (symlinks and specials are rejected); "
                            f"{what} must be a plain file inside the model directory")
    if st.st_size > cap:
        raise ModelDirError(f"{path}: {st.st_size} bytes exceeds the {what} cap of {cap} bytes")
    return st.st_size


def _read_toml(path: str) -> dict:
    try:
        with open(path, "rb") as f:
            return tomllib.load(f)
    except OSError as e:
        raise ModelDirError(f"{path}: {e.strerror}") from None
    except tomllib.TOMLDecodeError as e:
        raise ModelDirError(f"{path}: {e}") from None


def _read_remainder_exact(path: str, count: int, dtype: str) -> np.ndarray:
    """loader.rs:777-805: exactly ``count`` little-endian values at the declared dtype."""
    expected = count * _ITEMSIZE[dtype]
    size = _stat_regular_capped(path, MAX_SIDECAR_BYTES, "sidecar matrix")
    if size != expected:
        raise ModelDirError(f"{path}: {size} bytes; expected exactly {expected} bytes "
                            f"(a {count}-element remainder declared @{dtype})")
    raw = np.fromfile(path, dtype="<u2" if dtype == "bf16" else "<f4")
    if dtype == "bf16":
        return (raw.astype(np.uint32) << 16).view(np.float32)
    return raw.astype(np.float32)


def _require(table: dict, keys, path: str) -> None:
    for k in keys:
        if k not in table:
            raise ModelDirError(f"{path}: missing field `{k}`")


def _validate_config(c: dict, path: str) -> None:
    """loader.rs:880-1023, in the reference's order."""
    _require(c, ("vocab_size", "d_model", "eos_token_id", "bos_token_id", "n_layers", "n_heads",
                 "n_kv_heads", "head_dim", "rms_norm_eps", "rope_theta", "norm_slots"), path)
    if not 1 <= c["vocab_size"] <= MAX_DIM:
        raise ModelDirError(f"{path}: vocab_size {c['vocab_size']} outside 1..={MAX_DIM}")
    if not 1 <= c["d_model"] <= MAX_DIM:
        raise ModelDirError(f"{path}: d_model {c['d_model']} outside 1..={MAX_DIM}")
    for name in ("eos_token_id", "bos_token_id"):
        if c[name] >= c["vocab_size"]:
            raise ModelDirError(f"{path}: {name} {c[name]} >= vocab_size {c['vocab_size']}")
    if not 1 <= c["n_layers"] <= MAX_LAYERS:
        raise ModelDirError(f"{path}: n_layers {c['n_layers']} outside 1..={MAX_LAYERS}")
    if not 1 <= c["n_heads"] <= MAX_DIM:
        raise ModelDirError(f"{path}: n_heads {c['n_heads']} outside 1..={MAX_DIM}")
    if c["n_kv_heads"] == 0:
        raise ModelDirError(f"{path}: n_kv_heads must be at least 1 (got 0)")
    if c["head_dim"] == 0:
        raise ModelDirError(f"{path}: head_dim must be at least 1 (got 0)")
    kv_width = c["n_kv_heads"] * c["head_dim"]
    if kv_width != c["d_model"]:
        raise ModelDirError(f"{path}: n_kv_heads * head_dim = {kv_width} != d_model "
                            f"{c['d_model']} (GQA width mismatch)")
    if c["n_heads"] % c["n_kv_heads"]:
        raise ModelDirError(f"{path}: n_heads {c['n_heads']} is not a multiple of n_kv_heads "
                            f"{c['n_kv_heads']} (GQA group mismatch)")
    for name in ("rms_norm_eps", "rope_theta"):
        v = float(c[name])
        if not (v > 0.0 and math.isfinite(v)):
            raise ModelDirError(f"{path}: {name} must be finite and > 0 (got {v})")
    if not c["norm_slots"]:
        raise ModelDirError(f"{path}: norm_slots must declare at least one slot")
    for s in c["norm_slots"]:
        if s not in NORM_SLOTS:
            raise ModelDirError(f"{path}: unknown norm slot {_quote(s)}; known: input, "
                                "post_attention, q_norm, k_norm, post_feedforward")
    seen = set()
    for s in c["norm_slots"]:
        if s in seen:
            raise ModelDirError(f"{path}: duplicate norm slot {_quote(s)}")
        seen.add(s)
    wt = c.get("weight_tying")
    if wt is not None and _tying_dtype(wt) is None:
        raise ModelDirError(f"{path}: unknown weight_tying {_quote(wt)}; documented forms: unset "
                            'or "lm_head=<path>@<dtype>" with dtype fp32 or bf16 '
                            '(tied: "lm_head=e1@fp32")')


def _tying_dtype(wt: str):
    if not wt.startswith("lm_head=") or "@" not in wt:
        return None
    path, token = wt[len("lm_head="):].rsplit("@", 1)
    return token if path and token in _ITEMSIZE else None


@dataclass
class ModelDirectory:
    """loader.rs ``ModelDirectory``: what the files declare, nothing derived."""
    model_id: str
    layers: list                      # [(manifest name, parsed qpk1 layer dict)] in serving order
    eos_token_id: int
    bos_token_id: int
    vocab_size: int
    d_model: int
    n_layers: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    norm_slots: list
    remainder_dtype: str
    embedding: np.ndarray             # [vocab_size, d_model] float32
    lm_head: np.ndarray | None        # None when weight-tied
    norm_weights: np.ndarray          # n_layers * per-block inventory + d_model (final norm)
    extras: dict = field(default_factory=dict)


def load(model_dir: str) -> ModelDirectory:
    model_dir = os.fspath(model_dir)
    if not os.path.isdir(model_dir):
        raise ModelDirError(f"model dir {model_dir} does not exist or is not a directory")
    manifest_path = os.path.join(model_dir, "manifest.toml")
    manifest = _read_toml(manifest_path)
    _require(manifest, ("model_id", "layers", "layer_files"), manifest_path)
    if not manifest["layers"]:
        raise ModelDirError(f"{manifest_path}: manifest lists no layers; nothing to serve")
    for name in manifest["layers"]:
        if name not in manifest["layer_files"]:
            raise ModelDirError(f"{manifest_path}: layer {_quote(name)} has no entry in [layer_files]")
    config_path = os.path.join(model_dir, "config.toml")
    config = _read_toml(config_path)
    _validate_config(config, config_path)

    layers = []
    for name in manifest["layers"]:
        rel = manifest["layer_files"][name]
        try:
            layer_path = contained_join(model_dir, rel)
        except ModelDirError as why:
            raise ModelDirError(f"{manifest_path}: layer {_quote(name)} file path {_quote(rel)} "
                                f"rejected: {why}") from None
        _stat_regular_capped(layer_path, MAX_LAYER_BYTES, "layer file")
        try:
            layer = qpk1.parse(np.fromfile(layer_path, dtype=np.uint8))
        except ValueError as e:
            raise ModelDirError(f"{layer_path}: {e}") from None
        if layer["r"] > min(layer["dout"], layer["din"]):
            raise ModelDirError(f"{layer_path}: rank r={layer['r']} exceeds min(dout, din)="
                                f"{min(layer['dout'], layer['din'])}")
        layers.append((name, layer))

    sidecar = manifest.get("sidecar")
    if sidecar is None:
        raise ModelDirError(f"{manifest_path}: missing [sidecar] block "
                            "(embedding/lm_head/norms weights)")
    _require(sidecar, ("embedding", "lm_head", "norms"), manifest_path)
    dtype = sidecar.get("dtype", "fp32")
    if dtype not in _ITEMSIZE:
        raise ModelDirError(f"{manifest_path}: [sidecar] dtype = {_quote(dtype)} is not a declared "
                            "remainder dtype (fp32 or bf16); an absent key reads as fp32")
    wt = config.get("weight_tying")
    if wt is not None and _tying_dtype(wt) != dtype:
        raise ModelDirError(f"{config_path}: weight_tying declares @{_tying_dtype(wt)} but the "
                            f'manifest [sidecar] block declares dtype = "{dtype}"; a remainder '
                            "set cannot hold two dtypes")

    def sidecar_path(key):
        try:
            return contained_join(model_dir, sidecar[key])
        except ModelDirError as why:
            raise ModelDirError(f"{manifest_path}: [sidecar] {key} = {_quote(sidecar[key])} "
                                f"rejected: {why}") from None

    vocab, d = config["vocab_size"], config["d_model"]
    emb_path, head_path = sidecar_path("embedding"), sidecar_path("lm_head")
    embedding = _read_remainder_exact(emb_path, vocab * d, dtype).reshape(vocab, d)
    lm_head = None if head_path == emb_path else _read_remainder_exact(
        head_path, vocab * d, dtype).reshape(vocab, d)
    per_block = sum(_slot_width(s, d, config["head_dim"]) for s in config["norm_slots"])
    norm_weights = _read_remainder_exact(sidecar_path("norms"),
                                         per_block * config["n_layers"] + d, dtype)
    return ModelDirectory(
        model_id=manifest["model_id"], layers=layers, eos_token_id=config["eos_token_id"],
        bos_token_id=config["bos_token_id"], vocab_size=vocab, d_model=d,
        n_layers=config["n_layers"], n_heads=config["n_heads"], n_kv_heads=config["n_kv_heads"],
        head_dim=config["head_dim"], rms_norm_eps=float(config["rms_norm_eps"]),
        rope_theta=float(config["rope_theta"]), norm_slots=list(config["norm_slots"]),
        remainder_dtype=dtype, embedding=embedding, lm_head=lm_head, norm_weights=norm_weights)


class _Factors(dict):
    """One layer of a model directory as ``Decoder`` takes it: the container's two bit streams
    (``ub_packed``, ``vb_packed``), which the device separates into rows at upload, and, made
    on first use only (the tensor-parallel split and the CPU restatement read them), the row
    bitplanes of Ub and of Vb^T (engine/mod.rs:342-381, PackedLayer::from_layer)."""

    def __missing__(self, key):
        if key not in ("ub_rows", "vb_t_rows"):
            raise KeyError(key)
        dout, din, r = self["dout"], self["din"], self["r"]
        ub, vb = self["ub_packed"], self["vb_packed"]
        ub_rows = np.zeros((dout, (r + 7) // 8), np.uint8)
        vb_t_rows = np.zeros((r, (din + 7) // 8), np.uint8)
        check(_lib.lib().qk_container_to_rows(ub.ctypes.data, ub.size, dout, r,
                                              ub_rows.ctypes.data, ub_rows.size))
        check(_lib.lib().qk_container_to_rows_transposed(vb.ctypes.data, vb.size, din, r,
                                                         vb_t_rows.ctypes.data, vb_t_rows.size))
        self["ub_rows"], self["vb_t_rows"] = ub_rows, vb_t_rows
        return dict.__getitem__(self, key)


def _rows(layer: dict) -> dict:
    return _Factors(ub_packed=np.ascontiguousarray(layer["ub_packed"], dtype=np.uint8).ravel(),
                    vb_packed=np.ascontiguousarray(layer["vb_packed"], dtype=np.uint8).ravel(),
                    dout=layer["dout"], din=layer["din"], r=layer["r"], s1=layer["s1"],
                    s2=layer["s2"], bias=layer["bias"])


def decoder_inputs(md: ModelDirectory, **overrides):
    """``(DecoderConfig, weights)`` for ``Decoder``: the per-block resolution of
    engine/mod.rs:510-580 and the geometry checks of ``ModelWeights::new`` (:651-735)."""
    from .decoder import DecoderConfig
    index = {name: i for i, (name, _) in enumerate(md.layers)}
    d, hd = md.d_model, md.head_dim
    per_block = sum(_slot_width(s, d, hd) for s in md.norm_slots)
    if "post_feedforward" in md.norm_slots:
        raise ModelDirError("the post_feedforward norm slot is not served by this decoder")
    blocks = []
    for b in range(md.n_layers):
        lw = {}
        for short, suffix in PROJECTIONS.items():
            name = f"layers.{b}.inner.{suffix}"
            if name not in index:
                raise ModelDirError(f"block {b}: missing packed layer {_quote(name)}")
            lw[short] = _rows(md.layers[index[name]][1])
        at = b * per_block
        found = {}
        for slot in md.norm_slots:
            w = _slot_width(slot, d, hd)
            found[slot] = md.norm_weights[at:at + w].copy()
            at += w
        for need in ("input", "post_attention"):
            if need not in found:
                raise ModelDirError(f"block {b}: required norm slot {_quote(need)} not in the "
                                    f"declared inventory {md.norm_slots}")
        lw["input_norm"], lw["post_norm"] = found["input"], found["post_attention"]
        if "q_norm" in found and "k_norm" in found:   # applied only as a pair (:908-911)
            lw["q_norm"], lw["k_norm"] = found["q_norm"], found["k_norm"]
        want = {"q": (md.n_heads * hd, d), "k": (md.n_kv_heads * hd, d),
                "v": (md.n_kv_heads * hd, d), "o": (d, md.n_heads * hd)}
        for short, (dout, din) in want.items():
            if (lw[short]["dout"], lw[short]["din"]) != (dout, din):
                raise ModelDirError(f"block {b}: {short}_proj is {lw[short]['dout']}x"
                                    f"{lw[short]['din']}, the geometry wants {dout}x{din}")
        blocks.append(lw)
    d_ff = blocks[0]["gate"]["dout"]
    # model/mod.rs:725-734: a directory is always served in float32; a blob at the dtype its
    # header declares
    serving = ("bfloat16" if md.extras.get("source") == "blob" and md.remainder_dtype == "bf16"
               else "float32")
    settings = dict(serving=serving, kv_dtype="float32")
    settings.update(overrides)
    cfg = DecoderConfig(n_layers=md.n_layers, d_model=d, n_heads=md.n_heads,
                        n_kv_heads=md.n_kv_heads, head_dim=hd, d_ff=d_ff, vocab=md.vocab_size,
                        rms_eps=md.rms_norm_eps, rope_theta=md.rope_theta, **settings)
    weights = dict(layers=blocks, final_norm=md.norm_weights[md.n_layers * per_block:].copy(),
                   embedding=md.embedding,
                   lm_head=md.embedding if md.lm_head is None else md.lm_head, vocab_offset=0)
    return cfg, weights
