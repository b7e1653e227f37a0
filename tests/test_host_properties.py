"""Property tests of the host-side functions of the library (no GPU): random shapes and
seeds instead of hand-picked ones.  The oracles are NumPy one-liners or ``oracle/``."""

import numpy as np
from hypothesis import given, settings
from hypothesis import strategies as st

from oracle import itq_np
from quantibbler_b200 import kernels


@settings(max_examples=60, deadline=None, derandomize=True, database=None)
@given(st.integers(0, 9), st.integers(0, 70), st.integers(0, 2**32 - 1))
def test_pack_unpack_round_trip_and_bit_order(rows, cols, seed):
    rng = np.random.default_rng(seed)
    signs = np.where(rng.random((rows, cols)) < 0.5, 1, -1).astype(np.int8)
    packed = kernels.pack_bits(signs)
    assert packed.shape == (rows, (cols + 7) // 8) and packed.dtype == np.uint8
    # element 8j+k of a row sits at bit k of byte j; +1 -> 1; pad bits zero (core.rs:129-162)
    assert np.array_equal(packed, np.packbits(signs > 0, axis=1, bitorder="little").reshape(
        rows, (cols + 7) // 8))
    assert np.array_equal(kernels.unpack_bits(packed, cols), signs)
    assert np.array_equal(kernels.pack_bits(signs.astype(np.float64)), packed)
    if cols % 8 and rows:       # pad bits are ignored on the way back (core.rs:166-189)
        dirty = packed.copy()
        dirty[:, -1] |= np.uint8(0xFF << (cols % 8) & 0xFF)
        assert np.array_equal(kernels.unpack_bits(dirty, cols), signs)


@settings(max_examples=40, deadline=None, derandomize=True, database=None)
@given(st.lists(st.floats(allow_nan=False, width=64), max_size=40))
def test_sign_estimate_is_the_closed_sign(values):
    x = np.asarray(values, dtype=np.float64)
    got = kernels.sign_estimate(x)
    assert np.array_equal(got, np.where(x >= 0.0, 1, -1).astype(np.int8))   # core.rs:193-197


@settings(max_examples=25, deadline=None, derandomize=True, database=None)
@given(st.integers(1, 40), st.integers(0, 40), st.integers(1, 9), st.integers(0, 2**64 - 1),
       st.integers(0, 12))
def test_joint_itq_equals_the_numpy_oracle(dout, din, rank, seed, max_iter):
    rng = np.random.default_rng(seed % (2**32))
    u_hat = rng.standard_normal((dout, rank))
    v_hat = rng.standard_normal((din, rank))
    want = itq_np.joint_itq(u_hat, v_hat, max_iter=max_iter, seed=seed, return_margin=True)
    got = kernels.joint_itq(u_hat, v_hat, max_iter=max_iter, seed=seed)
    differ = np.concatenate([got[0], got[1]]) != np.concatenate([want[0], want[1]])
    # the two SVDs agree to rounding: a sign may differ only where Z R vanishes to rounding,
    # and then the later iterations may part ways too - so compare only runs that agree
    if differ.any():
        assert np.all(np.abs(want[4][differ]) < 1e-9)
    else:
        assert got[2] == want[2] and got[3] == want[3]
