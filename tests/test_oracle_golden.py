"""The CPU oracle against the reference's golden vectors (no GPU needed).

Pins oracle/qk_oracle.c and oracle/attention_np.py: every vector here was produced by
the reference's NumPy implementation or is one of the reference's committed fixtures
(tests/golden/make_golden.py).
"""

import numpy as np
import pytest

import oracle
from oracle import attention_np as anp
from conftest import golden, make_layer


def test_pack_unpack_bit_exact():
    g = golden("bitplanes")
    for key in g.cases("pack"):
        factor, packed = g[key + "_factor"], g[key + "_packed"]
        n_bits = g.meta[key]["n_bits"]
        assert np.array_equal(oracle.pack_bits(factor).reshape(packed.shape), packed), key
        if factor.size:
            assert np.array_equal(oracle.unpack_bits(packed, n_bits), factor.reshape(-1, n_bits))
        if g.has(key + "_expected_bytes"):
            assert np.array_equal(packed.ravel(), g[key + "_expected_bytes"].ravel())


def test_pack_rejects_non_binary():
    with pytest.raises(ValueError, match=r"got 0 at row 1, column 2"):
        oracle.pack_bits(np.array([[1, -1, 1], [1, 1, 0]], dtype=np.int8))


def test_sign_estimate():
    g = golden("bitplanes")
    for key in g.cases("sign"):
        for name in g.meta[key]["inputs"]:
            x = g[f"{key}_{name}"]
            assert np.array_equal(oracle.sign_estimate(x), g[f"{key}_{name}_signs"].ravel())


def test_products_bit_identical_to_reference():
    g = golden("products")
    n = 0
    for key, m in g.meta.items():
        fn = oracle.packed_matvec if m["kind"] == "matvec" else oracle.packed_matmul
        if key.startswith("refmv"):
            for variant, res in (("packed", "result"), ("packed_dirty", "result_dirty")):
                if g.has(f"{key}_{variant}"):
                    got = fn(g[f"{key}_{variant}"], m["n_bits"], g[key + "_vec"], m["dtype"])
                    assert np.array_equal(got, g[f"{key}_{res}"]), (key, variant)
                    n += 1
            continue
        opnd = g[key + "_mat"] if g.has(key + "_mat") else g[key + "_operand"]
        got = fn(g[key + "_packed"], m["n_bits"], opnd, m["dtype"])
        want = g[key + "_result"]
        assert got.dtype == want.dtype and np.array_equal(got, want), m["scenario"]
        n += 1
    assert n >= 40


def test_fast_face_backward_bound():
    # fast.rs:10-18: |fast - scalar| <= 1e-12 * sum|v_k|, and thread-count independent
    rng = np.random.default_rng(5)
    for rows, bits in [(1, 1), (257, 73), (1024, 137), (64, 8), (130, 4096)]:
        p = np.packbits(rng.random((rows, bits)) < 0.5, axis=1, bitorder="little")
        v = rng.standard_normal(bits)
        ref = oracle.packed_matvec(p, bits, v)
        one = oracle.fast_packed_matvec(p, bits, v, 1)
        many = oracle.fast_packed_matvec(p, bits, v, 4)
        assert np.array_equal(one, many)
        assert np.abs(one - ref).max() <= 1e-12 * np.abs(v).sum()


def test_vectorised_product_matches_sequential():
    rng = np.random.default_rng(6)
    p = np.packbits(rng.random((40, 333)) < 0.5, axis=1, bitorder="little")
    m = rng.standard_normal((333, 7))
    seq = oracle.packed_matmul(p, 333, m)
    vec = oracle.packed_matmul_exact(p, 333, m)
    assert np.abs(seq - vec).max() <= 1e-13 * np.abs(m).sum(axis=0).max()


def test_container_repack():
    rng = np.random.default_rng(8)
    for n_rows, r in [(5, 7), (4, 16), (9, 35)]:
        bits = rng.random((n_rows, r)) < 0.5
        stream = np.packbits(bits.ravel(), bitorder="little")
        assert np.array_equal(oracle.container_to_rows(stream, n_rows, r),
                              np.packbits(bits, axis=1, bitorder="little"))
        assert np.array_equal(oracle.container_to_rows_transposed(stream, n_rows, r),
                              np.packbits(bits.T, axis=1, bitorder="little"))


@pytest.mark.parametrize("key", ["small", "odd", "mid"])
def test_layer_apply_matches_reference(key):
    g = golden("layer")
    m = g.meta[key]
    bias = g[key + "_bias"] if m["bias"] else None
    args = (g[key + "_ub_rows"], g[key + "_vb_t_rows"], m["dout"], m["din"], m["r"],
            g[key + "_s1"], g[key + "_s2"], bias, g[key + "_x"])
    assert np.array_equal(oracle.layer_apply(*args, serving="float32"), g[key + "_y_f32"])
    assert np.array_equal(oracle.layer_apply(*args, serving="bfloat16"), g[key + "_y_bf16"])


def test_layer_apply_config0_matches_reference():
    g = golden("layer")
    m = g.meta["config0"]
    L = make_layer(m["dout"], m["din"], m["r"], m["seed"])
    assert np.array_equal(L["x"], g["config0_x"])
    y = oracle.layer_apply(L["ub_rows"], L["vb_t_rows"], m["dout"], m["din"], m["r"], L["s1"],
                           L["s2"], None, L["x"], serving="float32")
    assert np.array_equal(y, g["config0_y_f32"])
    yb = oracle.layer_apply(L["ub_rows"], L["vb_t_rows"], m["dout"], m["din"], m["r"], L["s1"],
                            L["s2"], None, L["x"], serving="bfloat16")
    assert np.array_equal(yb, g["config0_y_bf16"])
    yf = oracle.layer_apply(L["ub_rows"], L["vb_t_rows"], m["dout"], m["din"], m["r"], L["s1"],
                            L["s2"], None, L["x"], serving="float32", use_fast=True, n_threads=4)
    assert np.abs(yf - y).max() <= 1e-6 * np.abs(y).max()


def test_attention_exact_matches_reference():
    g = golden("attention")
    for key in g.cases("tiled"):
        got = anp.attention_exact(g[key + "_q"], g[key + "_k"], g[key + "_v"],
                                  causal=g.meta[key]["causal"])
        assert np.allclose(got, g[key + "_out"], rtol=1e-11, atol=1e-13), key
    for key in g.cases("xatt"):
        got = anp.attention_exact(g[key + "_q"], g[key + "_k"], g[key + "_v"],
                                  causal=g.meta[key]["causal"])
        assert np.allclose(got, g[key + "_out_tiled"], rtol=1e-10, atol=1e-12), key


def test_attention_sage_matches_reference():
    g = golden("attention")
    for key in g.cases("sage"):
        m = g.meta[key]
        got = anp.attention_sage(g[key + "_q"], g[key + "_k"], g[key + "_v"], causal=m["causal"],
                                 block_size=m["block_size"])
        assert np.allclose(got, g[key + "_out"], rtol=1e-11, atol=1e-13), key
        cos, rel_l1, _ = anp.quality_metrics(got, g[key + "_exact"])
        assert abs(cos - m["reference_metrics"]["cosine"]) < 1e-9
        assert abs(rel_l1 - m["reference_metrics"]["relative_l1"]) < 1e-9
    for key in g.cases("xatt"):
        m = g.meta[key]
        got = anp.attention_sage(g[key + "_q"], g[key + "_k"], g[key + "_v"], causal=m["causal"],
                                 block_size=m["block_size"])
        assert np.allclose(got, g[key + "_out_sage"], rtol=1e-10, atol=1e-12), key


def test_attention_sage_row_subset_and_f32_codes():
    g = golden("attention")
    key = "xatt0"
    m = g.meta[key]
    q, k, v = g[key + "_q"], g[key + "_k"], g[key + "_v"]
    rows = np.array([0, 63, 64, 150, 199])
    sub = anp.attention_sage(q, k, v, causal=m["causal"], block_size=m["block_size"], rows=rows)
    assert np.allclose(sub, g[key + "_out_sage"][:, :, rows], rtol=1e-10, atol=1e-12)
    o64, c64 = anp.attention_sage(q, k, v, causal=True, block_size=64, return_codes=True)
    o32, c32 = anp.attention_sage(q, k, v, causal=True, block_size=64, return_codes=True,
                                  ft=np.float32)
    # float32 and float64 quantisers may differ only where a value sits on a rounding tie
    assert np.mean(c64[0] != c32[0]) < 1e-3
    # a flipped code moves one P or V entry by 1/127 of its scale, so outputs agree to a
    # few 1e-3 at worst and to ~1e-6 where no code flipped
    assert np.abs(o64 - o32).max() < 2e-2
    assert np.median(np.abs(o64 - o32)) < 1e-6


def test_gqa_attention_scalar_matches_exact():
    rng = np.random.default_rng(3)
    n_heads, n_kv, d, n_pos = 8, 2, 32, 77
    q = rng.standard_normal(n_heads * d).astype(np.float32)
    keys = rng.standard_normal((n_pos, n_kv * d)).astype(np.float32)
    vals = rng.standard_normal((n_pos, n_kv * d)).astype(np.float32)
    got = oracle.gqa_attention_scalar(q, keys, vals, n_heads, n_kv, d)
    k4 = keys.reshape(n_pos, n_kv, d).transpose(1, 0, 2)[None]
    v4 = vals.reshape(n_pos, n_kv, d).transpose(1, 0, 2)[None]
    want = anp.attention_exact(q.reshape(1, n_heads, 1, d), k4, v4, causal=True)
    assert np.abs(got - want.ravel()).max() < 1e-5


def test_joint_itq_oracle_matches_reference():
    from oracle import itq_np
    g = golden("joint_itq")
    assert len(g.cases("itq")) >= 11
    for key in g.cases("itq"):
        meta = g.meta[key]
        u_t, v_t, n_iter, converged = itq_np.joint_itq(g[key + "_u_hat"], g[key + "_v_hat"],
                                                       **meta["kwargs"])
        assert np.array_equal(u_t, g[key + "_u_t"]), meta["scenario"]
        assert np.array_equal(v_t, g[key + "_v_t"]), meta["scenario"]
        assert (n_iter, converged) == (meta["n_iter"], meta["converged"]), meta["scenario"]
