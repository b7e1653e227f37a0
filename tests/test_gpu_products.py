"""GPU parity of the packed products through the C ABI: bit-identical to the
reference's vectors for float64, float32 and bfloat16."""

import numpy as np
import pytest

import oracle
from conftest import golden
from quantibbler_b200 import kernels

pytestmark = pytest.mark.gpu


def test_golden_products_bit_identical():
    g = golden("products")
    n = 0
    for key, m in g.meta.items():
        mv = m["kind"] == "matvec"
        fn = kernels.packed_matvec_dtype if mv else kernels.packed_matmul_dtype
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
        assert got.dtype == want.dtype and got.shape == want.shape, m["scenario"]
        assert np.array_equal(got, want), m["scenario"]
        n += 1
    assert n >= 40


@pytest.mark.parametrize("rows,bits", [(1, 1), (257, 73), (1024, 137), (64, 8), (300, 4096)])
def test_gpu_context_matvec_f64_bit_identical_and_repeatable(gpu_ctx, rows, bits):
    # crates/quantibbler-kernels/tests/gpu_parity.rs:49-150
    rng = np.random.default_rng(rows * 7 + bits)
    p = np.packbits(rng.random((rows, bits)) < 0.5, axis=1, bitorder="little")
    v = rng.standard_normal(bits)
    want = oracle.packed_matvec(p, bits, v)
    got = gpu_ctx.packed_matvec(p, rows, bits, v)
    assert np.array_equal(got, want)
    for _ in range(2):
        assert np.array_equal(gpu_ctx.packed_matvec(p, rows, bits, v), got)


@pytest.mark.parametrize("dtype", ["float64", "float32", "bfloat16"])
def test_matmul_mid_size_bit_identical(dtype):
    rng = np.random.default_rng(21)
    rows, bits, cols = 200, 1000, 9
    p = np.packbits(rng.random((rows, bits)) < 0.5, axis=1, bitorder="little")
    m = rng.standard_normal((bits, cols))
    if dtype == "float32":
        m = m.astype(np.float32)
    elif dtype == "bfloat16":
        m = oracle.f32_to_bf16_bits(m.astype(np.float32))
    want = oracle.packed_matmul(p, bits, m, dtype)
    got = kernels.packed_matmul_dtype(p, bits, m, dtype)
    assert np.array_equal(got, want)
    # the declared tolerance against the exact float64 product (parity.rs:955-974)
    as_f64 = oracle.bf16_bits_to_f32(m).astype(np.float64) if dtype == "bfloat16" else m.astype(np.float64)
    got64 = oracle.bf16_bits_to_f32(got).astype(np.float64) if dtype == "bfloat16" else got.astype(np.float64)
    exact = oracle.packed_matmul_exact(p, bits, as_f64)
    tol = {"float64": 1e-12, "float32": 1e-6, "bfloat16": 1e-2}[dtype]
    assert (np.abs(got64 - exact) / np.abs(as_f64).sum(axis=0)).max() <= tol


def test_reference_dispatch_uses_this_module(monkeypatch):
    # With the drop-in on sys.path the products raise the reference's texts unchanged.
    import quantibbler_kernels as qk
    p = np.zeros((6, 2), np.uint8)
    with pytest.raises(ValueError, match="vec must have length 13, got 3"):
        qk.packed_matvec(p, 13, np.zeros(3))
