"""Python face of the kernels: the nine functions of the reference's PyO3 module.

Mirrors crates/quantibbler-kernels/src/lib.rs:86-402 (``quantibbler_kernels``): the same
names, argument order, accepted dtypes, returned shapes and ``ValueError`` texts, so
that ``src/quantibbler/kernels/__init__.py`` can import this module in place of the
Rust extension.  Like the PyO3 face it only converts boundary types; pack/unpack and
sign are exact integer work done on the host by the shared library, and the products
run on the GPU through the C ABI (they raise if no device is usable).
"""

from __future__ import annotations

import numpy as np

from . import _lib
from ._lib import DTYPE_TAGS, KernelError, check

__all__ = [
    "backend_version", "pack_bits", "unpack_bits", "sign_estimate", "packed_matvec",
    "packed_matmul", "packed_matvec_dtype", "packed_matmul_dtype", "joint_itq",
]

DEFAULT_MAX_ITER = 50     # core.rs DEFAULT_MAX_ITER
DEFAULT_TOL = 1e-12       # core.rs DEFAULT_TOL


def _ptr(a: np.ndarray):
    return a.ctypes.data


def _rows_cols(shape) -> tuple[int, int]:
    # lib.rs:68-72
    n_cols = int(shape[-1]) if len(shape) else 0
    n_rows = int(np.prod(shape[:-1], dtype=np.int64)) if len(shape) else 1
    return n_rows, n_cols


def _typed(obj, dtype, what: str) -> np.ndarray:
    arr = np.asarray(obj)
    if arr.dtype != np.dtype(dtype):
        raise TypeError(f"{what} must be a {np.dtype(dtype).name} array, got {arr.dtype.name}")
    return np.ascontiguousarray(arr)


def backend_version() -> str:
    return _lib.lib().qk_backend_version().decode()


def pack_bits(factor) -> np.ndarray:
    """±1 factor (float64 or int8, any dimensionality) -> (n_rows, ceil(n_cols/8)) uint8."""
    arr = np.asarray(factor)
    if arr.ndim == 0:
        raise KernelError("pack_bits expects an array with at least one dimension")
    if arr.dtype == np.float64:
        fn = _lib.lib().qk_pack_bits_f64
    elif arr.dtype == np.int8:
        fn = _lib.lib().qk_pack_bits
    else:
        raise TypeError(f"pack_bits accepts float64 or int8 arrays, got {arr.dtype.name}")
    arr = np.ascontiguousarray(arr)
    n_rows, n_cols = _rows_cols(arr.shape)
    out = np.zeros((n_rows, (n_cols + 7) // 8), dtype=np.uint8)
    check(fn(_ptr(arr), arr.size, n_rows, n_cols, _ptr(out), out.size))
    return out


def unpack_bits(packed, n_bits: int, dtype: str = "int8") -> np.ndarray:
    p = _typed(packed, np.uint8, "packed")
    n_rows, n_words = _rows_cols(p.shape)
    n_bits = int(n_bits)
    if n_bits < 0:
        raise OverflowError("can't convert negative int to unsigned")
    if n_bits > n_words * 8:
        raise KernelError(
            f"n_bits={n_bits} exceeds the packed width {n_words} ({n_words * 8} bits)")
    if dtype not in ("int8", "float64"):
        raise KernelError(f'unpack_bits dtype must be \'int8\' or \'float64\', got "{dtype}"')
    out = np.zeros((n_rows, n_bits), dtype=np.int8)
    check(_lib.lib().qk_unpack_bits(_ptr(p), p.size, n_rows, n_bits, _ptr(out), out.size))
    return out if dtype == "int8" else out.astype(np.float64)


def sign_estimate(x) -> np.ndarray:
    xf = _typed(x, np.float64, "x")
    out = np.zeros(xf.size, dtype=np.int8)
    check(_lib.lib().qk_sign_estimate(_ptr(xf), xf.size, _ptr(out)))
    return out


_NP_OF_TAG = {"float64": np.float64, "float32": np.float32, "bfloat16": np.uint16}


def _tag(dtype: str) -> int:
    # resolve through the library so that the refusal text is the reference's
    import ctypes
    tag = ctypes.c_int32(-1)
    check(_lib.lib().qk_dtype_from_name(str(dtype).encode(), ctypes.byref(tag)))
    return tag.value


def packed_matvec_dtype(packed, n_bits: int, vec, dtype: str) -> np.ndarray:
    p = _typed(packed, np.uint8, "packed")
    n_rows, _ = _rows_cols(p.shape)
    tag = _tag(dtype)  # before touching the operand (lib.rs:303-305)
    v = _typed(vec, _NP_OF_TAG[dtype], "vec")
    out = np.zeros(n_rows, dtype=_NP_OF_TAG[dtype])
    check(_lib.lib().qk_packed_matvec(None, _ptr(p), p.size, n_rows, int(n_bits), tag, _ptr(v),
                                      v.size, _ptr(out)))
    return out


def packed_matmul_dtype(packed, n_bits: int, mat, dtype: str) -> np.ndarray:
    p = _typed(packed, np.uint8, "packed")
    n_rows, _ = _rows_cols(p.shape)
    tag = _tag(dtype)
    m = _typed(mat, _NP_OF_TAG[dtype], "mat")
    n_bits = int(n_bits)
    n_cols = int(m.shape[-1]) if m.ndim else 0
    k_cols = m.size // n_bits if n_bits else m.size
    out = np.zeros((n_rows, k_cols), dtype=_NP_OF_TAG[dtype])
    check(_lib.lib().qk_packed_matmul(None, _ptr(p), p.size, n_rows, n_bits, tag, _ptr(m), m.size,
                                      n_cols, _ptr(out), out.size))
    return out


def packed_matvec(packed, n_bits: int, vec) -> np.ndarray:
    """float64 product; the v0.1 name (lib.rs:170-183)."""
    return packed_matvec_dtype(packed, n_bits, vec, "float64")


def packed_matmul(packed, n_bits: int, mat) -> np.ndarray:
    return packed_matmul_dtype(packed, n_bits, mat, "float64")


def _unsigned(value, what: str, bits: int) -> int:
    v = int(value)
    if v < 0:
        raise OverflowError("can't convert negative int to unsigned")
    if v >= 1 << bits:
        raise OverflowError(f"{what} does not fit in {bits} bits")
    return v


def joint_itq(u_hat, v_hat, *, max_iter=None, tol=None, seed=None):
    """Alternating Procrustes over ``Z = [u_hat; v_hat]`` (lib.rs:197-234, core.rs:327-424).

    Returns ``(u_t, v_t, n_iter, converged)`` with int8 ±1 factors of the operands' row
    counts.  As in the PyO3 face the defaults are 50 iterations, tolerance 1e-12 and seed 0.
    Host work in the shared library (this is compressor-side code in the reference too).
    """
    import ctypes
    u = _typed(u_hat, np.float64, "u_hat")
    v = _typed(v_hat, np.float64, "v_hat")
    dout, rank = _rows_cols(u.shape)
    din, rank_v = _rows_cols(v.shape)
    if rank != rank_v:
        raise KernelError(f"joint_itq rank mismatch: u_hat r={rank}, v_hat r={rank_v}")
    iters = DEFAULT_MAX_ITER if max_iter is None else _unsigned(max_iter, "max_iter", 64)
    tolerance = DEFAULT_TOL if tol is None else float(tol)
    seed64 = 0 if seed is None else _unsigned(seed, "seed", 64)
    u_t = np.zeros((dout, rank), dtype=np.int8)
    v_t = np.zeros((din, rank), dtype=np.int8)
    n_iter = ctypes.c_size_t(0)
    converged = ctypes.c_int32(0)
    check(_lib.lib().qk_joint_itq(_ptr(u), u.size, _ptr(v), v.size, dout, din, rank, iters,
                                  tolerance, seed64, _ptr(u_t), _ptr(v_t),
                                  ctypes.byref(n_iter), ctypes.byref(converged)))
    return u_t, v_t, int(n_iter.value), bool(converged.value)
