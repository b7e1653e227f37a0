"""The model-directory reader and, through it, the reference's model-level golden.

tests/golden/parity-tiny is the reference's own fixture (tests/fixtures/parity-tiny): a
two-block model directory with q/k norms, and goldens.json with the logits its quantised HF
original gives at eight teacher-forced positions.  The reference's test
(crates/quantibbler-server/tests/parity_tiny.rs) loads the directory, checks the norm
inventory and asks for max |delta logit| <= 1e-2; here the same is asked of the NumPy
restatement of the forward, which pins it (and the reader, the container repack and the
norm inventory walk) to the reference.  No GPU is needed.
"""

import json
import os
import shutil

import numpy as np
import pytest

from conftest import GOLDEN
from oracle import decoder_np
from quantibbler_b200 import model_dir
from quantibbler_b200.model_dir import ModelDirError

FIXTURE = os.path.join(GOLDEN, "parity-tiny")
BUDGET = 1e-2   # parity_tiny.rs:26


def goldens():
    with open(os.path.join(FIXTURE, "goldens.json")) as f:
        return json.load(f)


def test_directory_loads_with_the_declared_inventory_and_geometry():
    md = model_dir.load(FIXTURE)
    g = goldens()
    assert md.model_id == "parity-tiny"
    assert md.norm_slots == g["norm_slots"]          # parity_tiny.rs:44-56
    geo = g["geometry"]
    assert (md.n_layers, md.n_heads, md.n_kv_heads, md.head_dim) == (
        geo["n_layers"], geo["n_heads"], geo["n_kv_heads"], geo["head_dim"])
    assert (md.rms_norm_eps, md.rope_theta) == (geo["rms_norm_eps"], geo["rope_theta"])
    assert len(md.layers) == 7 * md.n_layers and md.remainder_dtype == "fp32"
    assert md.embedding.shape == (128, 64) and md.lm_head.shape == (128, 64)
    per_block = 2 * md.d_model + 2 * md.head_dim
    assert md.norm_weights.shape == (per_block * md.n_layers + md.d_model,)
    cfg, w = model_dir.decoder_inputs(md, max_seq=16)
    assert (cfg.d_ff, cfg.vocab, cfg.serving, cfg.kv_dtype) == (128, 128, "float32", "float32")
    blk = w["layers"][1]
    at = per_block
    assert np.array_equal(blk["input_norm"], md.norm_weights[at:at + 64])
    assert np.array_equal(blk["post_norm"], md.norm_weights[at + 64:at + 128])
    assert np.array_equal(blk["q_norm"], md.norm_weights[at + 128:at + 160])
    assert np.array_equal(blk["k_norm"], md.norm_weights[at + 160:at + 192])
    assert np.array_equal(w["final_norm"], md.norm_weights[-64:])
    # a layer carries the container's bit streams (what the device separates into rows at upload);
    # the row bitplanes are made on first use and are the repack of engine/mod.rs:258-289
    q = blk["q"]
    assert "ub_packed" in q and "vb_packed" in q and "ub_rows" not in q and "vb_t_rows" not in q
    assert q["ub_rows"].shape == (128, 1) and q["vb_t_rows"].shape == (8, 8)
    assert "ub_rows" in q and "vb_t_rows" in q
    import oracle
    assert np.array_equal(q["ub_rows"], oracle.container_to_rows(q["ub_packed"], q["dout"], q["r"]))
    assert np.array_equal(q["vb_t_rows"],
                          oracle.container_to_rows_transposed(q["vb_packed"], q["din"], q["r"]))
    with pytest.raises(KeyError):
        q["no_such_key"]
    # a tensor-parallel shard holds rows only: the streams describe the whole layer
    from quantibbler_b200 import tp
    part = tp.shard_column_parallel(blk["k"], 1, 2)
    assert "ub_packed" not in part and part["ub_rows"].shape[0] == blk["k"]["dout"] // 2


def test_forward_restatement_reproduces_the_reference_goldens():
    md = model_dir.load(FIXTURE)
    cfg, w = model_dir.decoder_inputs(md, max_seq=16)
    g = goldens()
    session = decoder_np.Session(cfg, w)
    worst = 0.0
    for pos, tok in enumerate(g["input_ids"]):     # one cache, teacher-forced tokens
        _, logits = session.step(tok)
        worst = max(worst, float(np.abs(logits - np.asarray(g["logits"][pos], np.float32)).max()))
    assert worst <= BUDGET
    assert worst <= 5e-4   # what float32 against the HF reference actually leaves


def test_prefix_invariance_of_the_restatement():
    # parity_tiny.rs:71-83: a fresh cache per prefix gives the same last row
    md = model_dir.load(FIXTURE)
    cfg, w = model_dir.decoder_inputs(md, max_seq=16)
    ids = goldens()["input_ids"][:4]
    whole = decoder_np.Session(cfg, w)
    rows = [whole.step(t)[1] for t in ids]
    fresh = decoder_np.Session(cfg, w)
    for t in ids[:3]:
        last = fresh.step(t)[1]
    assert np.array_equal(last, rows[2])


@pytest.fixture()
def broken(tmp_path):
    dst = tmp_path / "model"
    shutil.copytree(FIXTURE, dst)

    def edit(name, old, new):
        p = dst / name
        text = p.read_text()
        assert old in text
        p.write_text(text.replace(old, new, 1))
        return str(dst)
    return dst, edit


def test_refusals_name_the_file_and_the_reason(broken, tmp_path):
    dst, edit = broken
    with pytest.raises(ModelDirError, match="does not exist or is not a directory"):
        model_dir.load(str(tmp_path / "nowhere"))
    # a layer listed without a file (loader.rs:192-199)
    edit("manifest.toml", '"layers.0.inner.mlp.down_proj" = ', '"layers.9.unused" = ')
    with pytest.raises(ModelDirError, match=r'manifest.toml: layer "layers.0.inner.mlp.down_proj" '
                                            r"has no entry in \[layer_files\]"):
        model_dir.load(str(dst))


@pytest.mark.parametrize("old,new,text", [
    ('"layers/layers/0/inner/mlp/up_proj.qpk1"', '"../up_proj.qpk1"',
     "rejected: '..' components are not allowed"),
    ('"layers/layers/0/inner/mlp/up_proj.qpk1"', '"/etc/passwd"',
     "rejected: absolute paths are not allowed"),
    ('"layers/layers/0/inner/mlp/up_proj.qpk1"', '"norms.bin"', "norms.bin: "),
    ('embedding = "e1.f32.bin"', 'embedding = "norms.bin"',
     "norms.bin: 1792 bytes; expected exactly 32768 bytes (a 8192-element remainder declared @fp32)"),
    ('[sidecar]', '[sidecar]\ndtype = "fp16"', 'dtype = "fp16" is not a declared remainder dtype'),
    ('[sidecar]', '[sidecar]\ndtype = "bf16"',
     'weight_tying declares @fp32 but the manifest [sidecar] block declares dtype = "bf16"'),
])
def test_manifest_refusals(broken, old, new, text):
    dst, edit = broken
    edit("manifest.toml", old, new)
    with pytest.raises(ModelDirError) as info:
        model_dir.load(str(dst))
    assert text in str(info.value)


@pytest.mark.parametrize("old,new,text", [
    ("head_dim = 32", "head_dim = 16", "n_kv_heads * head_dim = 32 != d_model 64 (GQA width mismatch)"),
    ("n_heads = 4", "n_heads = 3", "n_heads 3 is not a multiple of n_kv_heads 2 (GQA group mismatch)"),
    ("eos_token_id = 0", "eos_token_id = 128", "eos_token_id 128 >= vocab_size 128"),
    ('"q_norm", "k_norm"]', '"q_norm", "banana"]', 'unknown norm slot "banana"; known: input, '
     "post_attention, q_norm, k_norm, post_feedforward"),
    ('"q_norm", "k_norm"]', '"q_norm", "q_norm"]', 'duplicate norm slot "q_norm"'),
    ('"q_norm", "k_norm"]', '"q_norm"]', "norms.bin: 1792 bytes; expected exactly 1536 bytes"),
    ("rope_theta = 10000.0", "rope_theta = 0.0", "rope_theta must be finite and > 0"),
    ('weight_tying = "lm_head=head.f32.bin@fp32"', 'weight_tying = "lm_head=head.f32.bin"',
     "unknown weight_tying"),
    ("n_layers = 2", "", "missing field `n_layers`"),
])
def test_config_refusals(broken, old, new, text):
    dst, edit = broken
    edit("config.toml", old, new)
    with pytest.raises(ModelDirError) as info:
        model_dir.load(str(dst))
    assert "config.toml" in str(info.value) or "norms.bin" in str(info.value)
    assert text in str(info.value)


def test_symlinked_and_truncated_layer_files_are_refused(broken):
    dst, _ = broken
    layer = dst / "layers/layers/0/inner/mlp/up_proj.qpk1"
    raw = layer.read_bytes()
    layer.write_bytes(raw[:-3])
    with pytest.raises(ModelDirError, match="up_proj.qpk1: "):
        model_dir.load(str(dst))
    layer.unlink()
    (dst / "real.qpk1").write_bytes(raw)
    os.symlink(dst / "real.qpk1", layer)
    with pytest.raises(ModelDirError, match="not a regular file"):
        model_dir.load(str(dst))


def test_missing_projection_and_missing_required_slot(broken):
    dst, edit = broken
    edit("manifest.toml", '  "layers.1.inner.self_attn.v_proj",\n', "")
    md = model_dir.load(str(dst))
    with pytest.raises(ModelDirError, match='block 1: missing packed layer '
                                            '"layers.1.inner.self_attn.v_proj"'):
        model_dir.decoder_inputs(md)


def test_generate_restatement_semantics():
    # engine/mod.rs:1427-1456 (push_token): EOS is not part of the completion, the first
    # token is kept even with max_tokens = 0, an empty prompt is refused
    md = model_dir.load(FIXTURE)
    cfg, w = model_dir.decoder_inputs(md, max_seq=64)
    full, finish = decoder_np.generate(cfg, w, [5, 17, 3], 8, eos_token_id=md.eos_token_id)
    assert finish == "length" and len(full) == 8
    cut, finish = decoder_np.generate(cfg, w, [5, 17, 3], 8, eos_token_id=full[3])
    assert finish == "stop" and cut == full[:3]
    assert decoder_np.generate(cfg, w, [5, 17, 3], 0) == (full[:1], "length")
    with pytest.raises(ValueError, match="prompt tokenized to zero tokens"):
        decoder_np.generate(cfg, w, [], 4)


def _patch_layer(dst, offset, value):
    layer = dst / "layers/layers/0/inner/self_attn/q_proj.qpk1"
    raw = bytearray(layer.read_bytes())
    raw[offset:offset + len(value)] = value
    layer.write_bytes(bytes(raw))


@pytest.mark.parametrize("variant,needle", [
    # the names and needles of the reference's corrupted-variant table
    # (crates/quantibbler-server/tests/common/mod.rs:497-526), rebuilt on the parity-tiny copy
    ("missing_manifest", "manifest.toml"),
    ("missing_layer_file", "q_proj.qpk1"),
    ("bad_magic", "q_proj.qpk1: bad magic"),
    ("wrong_version", "q_proj.qpk1: unsupported representation version 7"),
    ("unknown_dtype_tag", "q_proj.qpk1: unknown dtype tag 9"),
    ("rank_zero", "q_proj.qpk1: dout, din and r must all be >= 1"),
    ("trailing_bytes", "q_proj.qpk1: trailing garbage"),
    ("missing_sidecar_block", "missing [sidecar] block"),
    ("missing_norms_manifest", "missing field `norms`"),
    ("missing_norms_file", "norms.bin"),
    ("missing_geometry", "missing field `n_heads`"),
])
def test_reference_corrupted_variants(broken, variant, needle):
    dst, edit = broken
    q_proj = dst / "layers/layers/0/inner/self_attn/q_proj.qpk1"
    if variant == "missing_manifest":
        (dst / "manifest.toml").unlink()
    elif variant == "missing_layer_file":
        q_proj.unlink()
    elif variant == "bad_magic":
        _patch_layer(dst, 0, b"X")
    elif variant == "wrong_version":
        _patch_layer(dst, 4, (7).to_bytes(4, "little"))
    elif variant == "unknown_dtype_tag":
        _patch_layer(dst, 8, (9).to_bytes(4, "little"))     # magic, version, dtype tag, dout, din, r
    elif variant == "rank_zero":
        _patch_layer(dst, 20, (0).to_bytes(4, "little"))
    elif variant == "trailing_bytes":
        q_proj.write_bytes(q_proj.read_bytes() + b"\0")
    elif variant == "missing_sidecar_block":
        text = (dst / "manifest.toml").read_text()
        (dst / "manifest.toml").write_text(text[:text.index("[sidecar]")])
    elif variant == "missing_norms_manifest":
        edit("manifest.toml", 'norms = "norms.bin"\n', "")
    elif variant == "missing_norms_file":
        (dst / "norms.bin").unlink()
    elif variant == "missing_geometry":
        edit("config.toml", "n_heads = 4\n", "")
    with pytest.raises(ModelDirError) as info:
        model_dir.load(str(dst))
    assert needle in str(info.value)
