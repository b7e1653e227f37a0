#!/usr/bin/env python
"""Regenerate tests/golden/*.npz from the reference checkout.

Run in a container that has the reference mounted:

    python tests/golden/make_golden.py /path/to/reference
    python tests/golden/make_golden.py /path/to/reference joint_itq    # that family alone
    python tests/golden/make_golden.py /path/to/reference parity_tiny  # the model fixture alone

It does two things, and commits nothing by itself:

1. Re-emits the reference's own kernel fixtures
   (crates/quantibbler-kernels/tests/fixtures/*.json) as compact ``.npz`` archives,
   after checking that the reference's NumPy implementation still reproduces every
   recorded output.
2. Imports the reference's NumPy implementation (``src/quantibbler/kernels``) and runs
   it on extra seeded inputs (odd shapes, the three product dtypes, the factorized
   linear at a small and at the 4096x4096 rank-1024 shape, attention at shapes with
   ragged tiles) to produce further golden outputs.

3. Copies the reference's model-level fixture directory (``tests/fixtures/parity-tiny``).

The tests only read the ``.npz`` files and that directory; the reference checkout is not needed to run
them.
"""

from __future__ import annotations

import json
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def joint_itq_cases(rk, load):
    """The reference's four joint_itq fixtures plus seeded larger factors run through its
    NumPy implementation (kernels/__init__.py:420-512)."""
    NR = "numpy-reference"
    itq: dict[str, np.ndarray] = {}
    imeta: dict[str, dict] = {}
    n = 0
    for rec in load("joint_itq"):
        key = f"itq{n}"
        itq[key + "_u_hat"] = np.asarray(rec["inputs"]["u_hat"], dtype=np.float64)
        itq[key + "_v_hat"] = np.asarray(rec["inputs"]["v_hat"], dtype=np.float64)
        itq[key + "_u_t"] = np.asarray(rec["faces"][NR]["u_t"], dtype=np.int8)
        itq[key + "_v_t"] = np.asarray(rec["faces"][NR]["v_t"], dtype=np.int8)
        imeta[key] = {"scenario": rec["scenario"], "kwargs": rec["inputs"]["kwargs"],
                      "n_iter": rec["faces"][NR]["n_iter"],
                      "converged": rec["faces"][NR]["converged"]}
        n += 1
    # seeded: (dout, din, rank, kwargs); low-rank-plus-noise factors as a compressor sees them
    seeded = [
        (24, 17, 5, {"max_iter": 50, "tol": 1e-12, "seed": 7}),
        (40, 33, 8, {"max_iter": 3, "tol": 1e-12, "seed": 123456789}),
        (64, 48, 12, {"max_iter": 50, "tol": 1e-12, "seed": 0}),
        (96, 80, 16, {"max_iter": 20, "tol": 0.0, "seed": 2**63 + 11}),
        (1, 9, 2, {"max_iter": 50, "tol": 1e-12, "seed": 5}),
        (6, 0, 3, {"max_iter": 50, "tol": 1e-12, "seed": 5}),
        (30, 30, 6, {"max_iter": 0, "tol": 1e-12, "seed": 99}),
    ]
    for i, (dout, din, rank, kwargs) in enumerate(seeded):
        rng = np.random.default_rng(7300 + i)
        u_hat = rng.standard_normal((dout, rank))
        v_hat = rng.standard_normal((din, rank))
        u_t, v_t, n_iter, conv = rk.joint_itq(u_hat, v_hat, backend=NR, **kwargs)
        # a golden sign is only useful if it does not hang on the last bit of Z R
        key = f"itq{n}"
        itq[key + "_u_hat"], itq[key + "_v_hat"] = u_hat, v_hat
        itq[key + "_u_t"], itq[key + "_v_t"] = u_t, v_t
        imeta[key] = {"scenario": f"seeded_{dout}+{din}x{rank}", "kwargs": kwargs,
                      "n_iter": int(n_iter), "converged": bool(conv)}
        n += 1
    return itq, imeta


def copy_parity_tiny(ref_root: str) -> None:
    """The reference's model-level fixture (tests/fixtures/parity-tiny: a two-block model
    directory with q/k norms and the logits its quantised HF original gives for eight
    teacher-forced positions, budget 1e-2 in crates/quantibbler-server/tests/parity_tiny.rs)
    copied as data; the tokenizer is not part of the forward and stays behind."""
    import shutil
    src = os.path.join(ref_root, "tests", "fixtures", "parity-tiny")
    dst = os.path.join(HERE, "parity-tiny")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("tokenizer.json"))
    for root, _dirs, files in os.walk(dst):   # the checkout may be read-only
        os.chmod(root, 0o755)
        for f in files:
            os.chmod(os.path.join(root, f), 0o644)
    print("parity-tiny", sum(len(f) for _r, _d, f in os.walk(dst)), "files")
    # the same model as single-file blobs, written by the reference's own writer
    # (src/quantibbler/blob.py) at both remainder dtypes
    from pathlib import Path

    from quantibbler.blob import write_blob_from_directory
    for dtype, name in (("fp32", "parity-tiny.qpk"), ("bf16", "parity-tiny-bf16.qpk")):
        sha = write_blob_from_directory(Path(src), Path(HERE) / name, remainder_dtype=dtype,
                                        created_by="make_golden")
        print(name, sha[:16])


def main(ref_root: str, only: str | None = None) -> None:
    sys.path.insert(0, os.path.join(ref_root, "src"))
    import quantibbler.kernels as rk
    from quantibbler.kernels.attention_sage import attention_sage
    from quantibbler.kernels.attention_tiled import attention_tiled

    fx = os.path.join(ref_root, "crates", "quantibbler-kernels", "tests", "fixtures")

    def load(name):
        with open(os.path.join(fx, name + ".json")) as f:
            return json.load(f)

    def dump(name, arrays, m):
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **arrays)
        with open(os.path.join(HERE, name + ".json"), "w") as f:
            json.dump(m, f, indent=1, sort_keys=True)
        print(name, len(arrays), "arrays")

    if only == "parity_tiny":
        copy_parity_tiny(ref_root)   # needs only the import path set above
        return
    if only == "joint_itq":   # this family alone (the others take minutes of Python loops)
        dump("joint_itq", *joint_itq_cases(rk, load))
        return

    NR = "numpy-reference"
    out: dict[str, np.ndarray] = {}
    meta: dict[str, dict] = {}

    # ------------------------------------------------------------ bitplanes
    for i, rec in enumerate(load("pack_bits")):
        key = f"pack{i}"
        factor = np.asarray(rec["inputs"]["factor"], dtype=np.int8)
        n_bits = int(rec["dtypes"]["n_bits"])
        if factor.ndim == 1:  # degenerate (n, 0) shapes serialise as nested empties
            factor = factor.reshape(len(rec["inputs"]["factor"]), n_bits)
        packed = np.asarray(rec["faces"][NR]["packed"], dtype=np.uint8).reshape(
            factor.shape[0], (n_bits + 7) // 8)
        assert np.array_equal(rk.pack_bits(factor, backend=NR), packed), rec["scenario"]
        out[key + "_factor"] = factor
        out[key + "_packed"] = packed
        meta[key] = {"scenario": rec["scenario"], "n_bits": n_bits}
        if "expected_bytes" in rec["inputs"]:
            out[key + "_expected_bytes"] = np.asarray(rec["inputs"]["expected_bytes"], np.uint8)
    for i, rec in enumerate(load("sign_estimate")):
        key = f"sign{i}"
        for name, val in rec["inputs"].items():
            x = np.asarray(val, dtype=np.float64)
            out[f"{key}_{name}"] = x
            out[f"{key}_{name}_signs"] = rk.sign_estimate(x, backend=NR).reshape(x.shape)
        meta[key] = {"scenario": rec["scenario"], "inputs": list(rec["inputs"].keys())}
        got = rk.sign_estimate(np.asarray(rec["inputs"]["x"]), backend=NR)
        assert np.array_equal(got.ravel(), np.asarray(rec["faces"][NR]["signs"]).ravel())

    # ------------------------------------------------------------ products (reference fixtures)
    prod: dict[str, np.ndarray] = {}
    pmeta: dict[str, dict] = {}
    for i, rec in enumerate(load("packed_matvec")):
        key = f"refmv{i}"
        n_bits = int(rec["dtypes"]["n_bits"])
        vec = np.asarray(rec["inputs"]["vec"], dtype=np.float64)
        for variant, res in (("packed", "result"), ("packed_dirty", "result_dirty")):
            if variant not in rec["inputs"]:
                continue
            p = np.asarray(rec["inputs"][variant], dtype=np.uint8)
            want = np.asarray(rec["faces"][NR][res], dtype=np.float64)
            assert np.array_equal(rk.packed_matvec(p, n_bits, vec, backend=NR), want)
            prod[f"{key}_{variant}"] = p
            prod[f"{key}_{res}"] = want
        prod[key + "_vec"] = vec
        pmeta[key] = {"scenario": rec["scenario"], "n_bits": n_bits, "kind": "matvec",
                      "dtype": "float64"}
    for i, rec in enumerate(load("packed_matmul")):
        key = f"refmm{i}"
        n_bits = int(rec["dtypes"]["n_bits"])
        p = np.asarray(rec["inputs"]["packed"], dtype=np.uint8)
        mat = np.asarray(rec["inputs"]["mat"], dtype=np.float64)
        want = np.asarray(rec["faces"][NR]["result"], dtype=np.float64)
        assert np.array_equal(rk.packed_matmul(p, n_bits, mat, backend=NR), want)
        prod[key + "_packed"], prod[key + "_mat"], prod[key + "_result"] = p, mat, want
        pmeta[key] = {"scenario": rec["scenario"], "n_bits": n_bits, "kind": "matmul",
                      "dtype": "float64"}
    for i, rec in enumerate(load("dtype_parity")):
        key = f"refdt{i}"
        n_bits = int(rec["dtypes"]["n_bits"])
        dt = rec["dtypes"]["operand"]
        npdt = np.uint16 if dt == "bfloat16" else np.float32
        p = np.asarray(rec["inputs"]["packed"], dtype=np.uint8)
        matvec = "vec" in rec["inputs"]
        opnd = np.asarray(rec["inputs"]["vec" if matvec else "mat"], dtype=npdt)
        want = np.asarray(rec["faces"][NR]["result"], dtype=npdt)
        fn = rk.packed_matvec if matvec else rk.packed_matmul
        got = fn(p, n_bits, opnd, dtype=dt, backend=NR)
        assert np.array_equal(got, want), rec["scenario"]
        prod[key + "_packed"], prod[key + "_operand"], prod[key + "_result"] = p, opnd, want
        pmeta[key] = {"scenario": rec["scenario"], "n_bits": n_bits,
                      "kind": "matvec" if matvec else "matmul", "dtype": dt}

    # ------------------------------------------------------------ products (extra seeded)
    def operand(rng, shape, dt):
        x = rng.standard_normal(shape)
        if dt == "float64":
            return x
        if dt == "float32":
            return x.astype(np.float32)
        return rk._f32_to_bf16_bits(x.astype(np.float32))

    shapes_mv = [(1, 1), (3, 9), (64, 8), (17, 137), (9, 257), (33, 128), (5, 1000)]
    n = 0
    for (rows, bits) in shapes_mv:
        for dt in ("float64", "float32", "bfloat16"):
            rng = np.random.default_rng(7000 + n)
            factor = rng.choice(np.array([-1, 1], dtype=np.int8), size=(rows, bits))
            p = rk.pack_bits(factor, backend=NR)
            v = operand(rng, (bits,), dt)
            key = f"xmv{n}"
            prod[key + "_packed"], prod[key + "_operand"] = p, v
            prod[key + "_result"] = rk.packed_matvec(p, bits, v, dtype=dt, backend=NR)
            pmeta[key] = {"scenario": f"seeded_matvec_{rows}x{bits}_{dt}", "n_bits": bits,
                          "kind": "matvec", "dtype": dt}
            n += 1
    n = 0
    for (rows, bits, cols) in [(7, 40, 5), (4, 13, 1), (19, 130, 17), (2, 64, 33)]:
        for dt in ("float64", "float32", "bfloat16"):
            rng = np.random.default_rng(7100 + n)
            factor = rng.choice(np.array([-1, 1], dtype=np.int8), size=(rows, bits))
            p = rk.pack_bits(factor, backend=NR)
            m = operand(rng, (bits, cols), dt)
            key = f"xmm{n}"
            prod[key + "_packed"], prod[key + "_operand"] = p, m
            prod[key + "_result"] = rk.packed_matmul(p, bits, m, dtype=dt, backend=NR)
            pmeta[key] = {"scenario": f"seeded_matmul_{rows}x{bits}x{cols}_{dt}", "n_bits": bits,
                          "kind": "matmul", "dtype": dt}
            n += 1

    itq, imeta = joint_itq_cases(rk, load)

    # ------------------------------------------------------------ factorized linear
    # engine/mod.rs:393-460 expressed through the reference's NumPy products.
    lay: dict[str, np.ndarray] = {}
    lmeta: dict[str, dict] = {}

    def layer_case(key, dout, din, r, seed, with_bias, big=False):
        rng = np.random.default_rng(seed)
        ub = rng.random((dout, r)) < 0.5
        vb = rng.random((din, r)) < 0.5
        s1 = (np.abs(rng.standard_normal(dout)) * 0.02 + 1e-3).astype(np.float32)
        s2 = (np.abs(rng.standard_normal(din)) * 0.02 + 1e-3).astype(np.float32)
        x = rng.standard_normal(din).astype(np.float32)
        bias = (rng.standard_normal(dout) * 0.1).astype(np.float32) if with_bias else None
        ub_rows = np.packbits(ub, axis=1, bitorder="little")
        vb_t_rows = np.packbits(vb.T, axis=1, bitorder="little")
        if not big:
            assert np.array_equal(ub_rows, rk.pack_bits(np.where(ub, 1, -1), backend=NR))
        b32 = bias if bias is not None else np.zeros(dout, np.float32)
        # fp32 serving
        z = (s2 * x).astype(np.float32).astype(np.float64)
        t = rk.packed_matvec(vb_t_rows, din, z, backend=NR)
        u = rk.packed_matvec(ub_rows, r, t, backend=NR)
        y32 = (u.astype(np.float32) * s1 + b32).astype(np.float32)
        # bf16 serving
        zb = rk._f32_to_bf16_bits((s2 * x).astype(np.float32))
        tb = rk.packed_matvec(vb_t_rows, din, zb, dtype="bfloat16", backend=NR)
        ubf = rk.packed_matvec(ub_rows, r, tb, dtype="bfloat16", backend=NR)
        y16 = (rk._bf16_bits_to_f32(ubf) * s1 + b32).astype(np.float32)
        if not big:
            lay[key + "_ub_rows"], lay[key + "_vb_t_rows"] = ub_rows, vb_t_rows
            lay[key + "_s1"], lay[key + "_s2"] = s1, s2
            if bias is not None:
                lay[key + "_bias"] = bias
        lay[key + "_x"], lay[key + "_y_f32"], lay[key + "_y_bf16"] = x, y32, y16
        lay[key + "_t_f64"] = t
        lmeta[key] = {"dout": dout, "din": din, "r": r, "seed": seed, "bias": with_bias,
                      "stored_factors": not big,
                      "generator": "rng=default_rng(seed); ub=rng.random((dout,r))<0.5; "
                                   "vb=rng.random((din,r))<0.5; s1,s2=|N(0,1)|*0.02+1e-3 f32; "
                                   "x=N(0,1) f32; bias=N(0,1)*0.1 f32 if bias"}

    layer_case("small", 96, 160, 72, 11, True)
    layer_case("odd", 50, 77, 35, 12, False)      # r % 8 != 0, din % 8 != 0
    layer_case("mid", 256, 512, 128, 13, True)
    t0 = time.time()
    layer_case("config0", 4096, 4096, 1024, 0, False, big=True)
    print(f"config0 layer through the NumPy reference: {time.time() - t0:.1f}s")

    # ------------------------------------------------------------ attention
    att: dict[str, np.ndarray] = {}
    ameta: dict[str, dict] = {}
    for i, rec in enumerate(load("attention_tiled")):
        key = f"tiled{i}"
        sh = rec["shape"]
        qs = (sh["batch"], sh["n_heads"], sh["seq"], sh["head_dim"])
        ks = (sh["batch"], sh["n_kv_heads"], sh["seq"], sh["head_dim"])
        vs = (sh["batch"], sh["n_kv_heads"], sh["seq"], sh["val_dim"])
        q = np.asarray(rec["inputs"]["query"], np.float32).reshape(qs)
        k = np.asarray(rec["inputs"]["key"], np.float32).reshape(ks)
        v = np.asarray(rec["inputs"]["value"], np.float32).reshape(vs)
        want = np.asarray(rec["faces"][NR]["out"], np.float64).reshape(qs[:3] + (sh["val_dim"],))
        got = attention_tiled(q, k, v, causal=rec["causal"])
        assert np.allclose(got, want, rtol=1e-12, atol=1e-14), rec["scenario"]
        att[key + "_q"], att[key + "_k"], att[key + "_v"], att[key + "_out"] = q, k, v, want
        ameta[key] = {"scenario": rec["scenario"], "causal": rec["causal"], "seed": rec["seed"]}
    for i, rec in enumerate(load("attention_sage")):
        key = f"sage{i}"
        sh = rec["shape"]
        qs = (sh["batch"], sh["n_heads"], sh["seq"], sh["head_dim"])
        ks = (sh["batch"], sh["n_kv_heads"], sh["seq"], sh["head_dim"])
        vs = (sh["batch"], sh["n_kv_heads"], sh["seq"], sh["val_dim"])
        q = np.asarray(rec["inputs"]["query"], np.float32).reshape(qs)
        k = np.asarray(rec["inputs"]["key"], np.float32).reshape(ks)
        v = np.asarray(rec["inputs"]["value"], np.float32).reshape(vs)
        os_ = qs[:3] + (sh["val_dim"],)
        want = np.asarray(rec["faces"]["quantized-reference"]["out"], np.float64).reshape(os_)
        exact = np.asarray(rec["faces"]["exact"]["out"], np.float64).reshape(os_)
        got = attention_sage(q, k, v, causal=rec["causal"], block_size=rec["block_size"])
        assert np.allclose(got, want, rtol=1e-12, atol=1e-14), rec["scenario"]
        att[key + "_q"], att[key + "_k"], att[key + "_v"] = q, k, v
        att[key + "_out"], att[key + "_exact"] = want, exact
        ameta[key] = {"scenario": rec["scenario"], "causal": rec["causal"], "seed": rec["seed"],
                      "block_size": rec["block_size"],
                      "reference_metrics": rec["reference_metrics"]}
    # extra seeded shapes through the reference functions (ragged tiles, GQA, d=64/128)
    extra = [(1, 4, 2, 200, 64, 64, True, 64), (2, 4, 4, 97, 32, 48, False, 32),
             (1, 8, 2, 130, 128, 128, True, 64), (1, 2, 1, 65, 16, 16, True, 1)]
    for i, (b, h, kvh, s, d, dv, causal, blk) in enumerate(extra):
        key = f"xatt{i}"
        rng = np.random.default_rng(9200 + i)
        q = rng.standard_normal((b, h, s, d)).astype(np.float32)
        k = (rng.standard_normal((b, kvh, s, d)) + 2.0 * rng.standard_normal((1, kvh, 1, d))
             ).astype(np.float32)
        v = rng.standard_normal((b, kvh, s, dv)).astype(np.float32)
        att[key + "_q"], att[key + "_k"], att[key + "_v"] = q, k, v
        att[key + "_out_tiled"] = attention_tiled(q, k, v, causal=causal, block_size=blk)
        att[key + "_out_sage"] = attention_sage(q, k, v, causal=causal, block_size=blk)
        ameta[key] = {"scenario": f"seeded_{b}x{h}/{kvh}x{s}x{d}->{dv}", "causal": causal,
                      "block_size": blk, "seed": 9200 + i}

    dump("bitplanes", out, meta)
    dump("products", prod, pmeta)
    dump("joint_itq", itq, imeta)
    dump("layer", lay, lmeta)
    dump("attention", att, ameta)
    copy_parity_tiny(ref_root)


if __name__ == "__main__":
    if len(sys.argv) not in (2, 3):
        raise SystemExit("usage: make_golden.py <path of the reference checkout> [joint_itq|parity_tiny]")
    main(*sys.argv[1:])
