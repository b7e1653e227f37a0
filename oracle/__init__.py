"""CPU oracle for the quantibbler-kernels hot path.  TEST INFRASTRUCTURE ONLY.

The oracle is the checker: parity tests, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` are the only callers.
The product library never imports, links or executes anything in this package.

Parity status: PINNED against the reference's committed golden vectors and against
outputs of the reference's NumPy implementation (``tests/golden/``).

``qk_oracle.c`` restates ``crates/quantibbler-kernels/src/{core,fast}.rs`` and the
factorized-linear apply of ``crates/quantibbler-server/src/engine/mod.rs``;
``attention_np.py`` restates ``src/quantibbler/kernels/attention_{tiled,sage}.py``.
"""

from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libqk_oracle.so")
_lib = None

c_sz = ctypes.c_size_t
_u8p = ctypes.POINTER(ctypes.c_uint8)


def build(force: bool = False) -> str:
    """Compile ``qk_oracle.c`` with the Makefile beside it (gcc only)."""
    src = os.path.join(_HERE, "qk_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
        _lib.qko_bf16_to_f32.restype = ctypes.c_float
        _lib.qko_bf16_to_f32.argtypes = [ctypes.c_uint16]
        _lib.qko_f32_to_bf16.restype = ctypes.c_uint16
        _lib.qko_f32_to_bf16.argtypes = [ctypes.c_float]
    return _lib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=dtype))


# ---------------------------------------------------------------- bitplanes
def pack_bits(factor) -> np.ndarray:
    f = _c(factor, np.int8)
    n_cols = f.shape[-1]
    n_rows = int(np.prod(f.shape[:-1], dtype=np.int64))
    out = np.zeros((n_rows, (n_cols + 7) // 8), dtype=np.uint8)
    bad_v = ctypes.c_int(0)
    bad_r = c_sz(0)
    bad_c = c_sz(0)
    rc = lib().qko_pack_bits(_ptr(f), c_sz(n_rows), c_sz(n_cols), _ptr(out),
                             ctypes.byref(bad_v), ctypes.byref(bad_r), ctypes.byref(bad_c))
    if rc:
        raise ValueError(
            f"pack_bits expects values in {{-1, +1}}; got {bad_v.value} at row {bad_r.value}, "
            f"column {bad_c.value}")
    return out


def unpack_bits(packed, n_bits: int) -> np.ndarray:
    p = _c(packed, np.uint8)
    n_rows = p.shape[0]
    out = np.zeros((n_rows, n_bits), dtype=np.int8)
    lib().qko_unpack_bits(_ptr(p), c_sz(n_rows), c_sz(n_bits), _ptr(out))
    return out


def sign_estimate(x) -> np.ndarray:
    xf = _c(x, np.float64)
    out = np.zeros(xf.size, dtype=np.int8)
    lib().qko_sign_estimate(_ptr(xf), c_sz(xf.size), _ptr(out))
    return out


def container_to_rows(packed, n_rows: int, r: int) -> np.ndarray:
    p = _c(packed, np.uint8).ravel()
    out = np.zeros((n_rows, (r + 7) // 8), dtype=np.uint8)
    lib().qko_container_to_rows(_ptr(p), c_sz(n_rows), c_sz(r), _ptr(out))
    return out


def container_to_rows_transposed(packed, din: int, r: int) -> np.ndarray:
    p = _c(packed, np.uint8).ravel()
    out = np.zeros((r, (din + 7) // 8), dtype=np.uint8)
    lib().qko_container_to_rows_transposed(_ptr(p), c_sz(din), c_sz(r), _ptr(out))
    return out


# ---------------------------------------------------------------- products
_NP = {"float64": np.float64, "float32": np.float32, "bfloat16": np.uint16}
_SUFFIX = {"float64": "f64", "float32": "f32", "bfloat16": "bf16"}


def packed_matvec(packed, n_bits: int, vec, dtype: str = "float64") -> np.ndarray:
    """Sequential scalar product (core.rs:247-260); bf16 as uint16 bit patterns."""
    p = _c(packed, np.uint8)
    v = _c(vec, _NP[dtype])
    assert v.shape == (n_bits,), (v.shape, n_bits)
    n_rows = p.shape[0]
    out = np.zeros(n_rows, dtype=_NP[dtype])
    getattr(lib(), "qko_packed_matvec_" + _SUFFIX[dtype])(
        _ptr(p), c_sz(n_rows), c_sz(n_bits), _ptr(v), _ptr(out))
    return out


def packed_matmul(packed, n_bits: int, mat, dtype: str = "float64") -> np.ndarray:
    """Sequential scalar column-batched product (core.rs:288-317)."""
    p = _c(packed, np.uint8)
    m = _c(mat, _NP[dtype])
    n_rows = p.shape[0]
    n_cols = m.shape[-1]
    kc = m.size // n_bits if n_bits else m.size
    out = np.zeros((n_rows, kc), dtype=_NP[dtype])
    getattr(lib(), "qko_packed_matmul_" + _SUFFIX[dtype])(
        _ptr(p), c_sz(n_rows), c_sz(n_bits), _ptr(m), c_sz(m.size), c_sz(n_cols), _ptr(out))
    return out


def fast_packed_matvec(packed, n_bits: int, vec, n_threads: int = 1) -> np.ndarray:
    """The reference's SIMD + row-parallel f64 face (fast.rs:85-110)."""
    p = _c(packed, np.uint8)
    v = _c(vec, np.float64)
    n_rows = p.shape[0]
    out = np.zeros(n_rows, dtype=np.float64)
    lib().qko_fast_packed_matvec_f64(_ptr(p), c_sz(n_rows), c_sz(n_bits), _ptr(v), _ptr(out),
                                     ctypes.c_int(n_threads))
    return out


def layer_apply(ub_rows, vb_t_rows, dout, din, r, s1, s2, bias, x, serving="float32",
                use_fast=False, n_threads=1) -> np.ndarray:
    """One factorized linear on one token (engine/mod.rs:393-460)."""
    ub = _c(ub_rows, np.uint8)
    vbt = _c(vb_t_rows, np.uint8)
    s1 = _c(s1, np.float32)
    s2 = _c(s2, np.float32)
    x = _c(x, np.float32)
    b = None if bias is None else _c(bias, np.float32)
    y = np.zeros(dout, dtype=np.float32)
    bp = _ptr(b) if b is not None else None
    if serving == "float32":
        rc = lib().qko_layer_apply_f32(_ptr(ub), _ptr(vbt), c_sz(dout), c_sz(din), c_sz(r),
                                       _ptr(s1), _ptr(s2), bp, _ptr(x), _ptr(y),
                                       ctypes.c_int(int(use_fast)), ctypes.c_int(n_threads))
    elif serving == "bfloat16":
        rc = lib().qko_layer_apply_bf16(_ptr(ub), _ptr(vbt), c_sz(dout), c_sz(din), c_sz(r),
                                        _ptr(s1), _ptr(s2), bp, _ptr(x), _ptr(y))
    else:
        raise ValueError(serving)
    if rc:
        raise MemoryError("oracle layer_apply")
    return y


def gqa_attention_scalar(q, keys, vals, n_heads, n_kv_heads, head_dim) -> np.ndarray:
    """Single-position decode attention (engine/mod.rs:1074-1121), f32."""
    q = _c(q, np.float32)
    keys = _c(keys, np.float32)
    vals = _c(vals, np.float32)
    n_pos = keys.size // (n_kv_heads * head_dim)
    out = np.zeros(n_heads * head_dim, dtype=np.float32)
    scratch = np.zeros(n_pos, dtype=np.float32)
    lib().qko_gqa_attention_scalar(_ptr(q), _ptr(keys), _ptr(vals), c_sz(n_pos), c_sz(n_heads),
                                   c_sz(n_kv_heads), c_sz(head_dim), _ptr(out), _ptr(scratch))
    return out


# ---------------------------------------------------------------- bf16 helpers
def f32_to_bf16_bits(x) -> np.ndarray:
    """kernels/__init__.py:233-245: round-to-nearest-even in integer space."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> np.uint64(16)) & np.uint64(1)
    return (((u + np.uint64(0x7FFF) + lsb) >> np.uint64(16)) & np.uint64(0xFFFF)).astype(np.uint16)


def bf16_bits_to_f32(bits) -> np.ndarray:
    """kernels/__init__.py:227-230."""
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


# ---------------------------------------------------------------- vectorised products
def unpack_signs(packed, n_bits: int, dtype=np.float64) -> np.ndarray:
    """±1 matrix of a packed array (vectorised; LSB-first within each byte)."""
    p = np.asarray(packed, dtype=np.uint8)
    bits = np.unpackbits(p, axis=-1, bitorder="little")[..., :n_bits]
    return bits.astype(dtype) * 2 - 1


def packed_matmul_exact(packed, n_bits: int, mat) -> np.ndarray:
    """Vectorised f64 product for sizes the sequential loops cannot reach.

    Not bit-identical to the sequential order (BLAS reassociates); used as the
    "exact f64 product" that the reference's backward-error gates compare against
    (crates/quantibbler-kernels/tests/parity.rs:955-974).
    """
    return unpack_signs(packed, n_bits) @ np.asarray(mat, dtype=np.float64)
