"""NumPy oracle for joint_itq.  TEST INFRASTRUCTURE ONLY.

Parity status: PINNED.  Reproduces the reference's committed vectors
(crates/quantibbler-kernels/tests/fixtures/joint_itq.json, re-emitted under tests/golden/
with further seeded cases run through the reference's NumPy implementation), signs,
iteration counts and convergence flags.

Follows src/quantibbler/kernels/__init__.py:345-512 (``_splitmix_matrix``,
``_gram_schmidt``, ``_matmul_lr``, ``_matmul_at_b_lr``, ``_numpy_joint_itq``).  The
reference writes every product as three nested Python loops so that each element is summed
left to right; here the loop over the summation index is kept and the two free indices are
vectorised, which leaves every element's order of additions unchanged and makes sizes of a
few thousand rows run in seconds.  The r x r SVD is ``np.linalg.svd``, as in the reference.
"""

from __future__ import annotations

import math

import numpy as np

_MASK64 = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15
_MIX1 = 0xBF58476D1CE4E5B9
_MIX2 = 0x94D049BB133111EB


def splitmix_matrix(seed: int, rank: int) -> np.ndarray:
    """kernels/__init__.py:345-362: rank x rank float64 in [-1, 1), filled row-major."""
    state = int(seed) & _MASK64
    out = np.empty(rank * rank, dtype=np.float64)
    for i in range(rank * rank):
        state = (state + _GOLDEN) & _MASK64
        z = state
        z = ((z ^ (z >> 30)) * _MIX1) & _MASK64
        z = ((z ^ (z >> 27)) * _MIX2) & _MASK64
        z ^= z >> 31
        out[i] = (z >> 11) / 9007199254740992.0 * 2.0 - 1.0
    return out.reshape(rank, rank)


def _dot_lr(a: np.ndarray, b: np.ndarray) -> float:
    acc = 0.0
    for x, y in zip(a.tolist(), b.tolist()):
        acc += x * y
    return acc


def gram_schmidt(a: np.ndarray) -> np.ndarray:
    """kernels/__init__.py:365-390: modified Gram-Schmidt over columns, sums left to right."""
    rank = a.shape[0]
    r0 = np.array(a, dtype=np.float64, copy=True)
    for j in range(rank):
        v = r0[:, j].copy()
        for i in range(j):
            d = _dot_lr(r0[:, i], v)
            v -= d * r0[:, i]
        nrm = math.sqrt(_dot_lr(v, v))
        if nrm == 0.0:
            raise ValueError("joint_itq produced a degenerate zero column building R0")
        r0[:, j] = v / nrm
    return r0


def matmul_lr(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """kernels/__init__.py:393-404: a @ b, element (i, j) summed over t = 0, 1, ... in order."""
    out = np.zeros((a.shape[0], b.shape[1]), dtype=np.float64)
    for t in range(a.shape[1]):
        out += a[:, t:t + 1] * b[t:t + 1, :]
    return out


def matmul_at_b_lr(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """kernels/__init__.py:407-418: a.T @ b, element (i, j) summed over the rows in order."""
    out = np.zeros((a.shape[1], b.shape[1]), dtype=np.float64)
    for t in range(a.shape[0]):
        out += a[t][:, None] * b[t][None, :]
    return out


def joint_itq(u_hat, v_hat, *, max_iter: int = 50, tol: float = 1e-12, seed: int = 0,
              return_margin: bool = False):
    """kernels/__init__.py:420-512.  ``return_margin`` adds the final ``Z R`` so that a test
    can tell a sign that hangs on the last bits of the rotation from a real difference."""
    u = np.asarray(u_hat, dtype=np.float64)
    v = np.asarray(v_hat, dtype=np.float64)
    if u.ndim != 2 or v.ndim != 2:
        raise ValueError("joint_itq expects 2-D inputs u_hat (dout, r), v_hat (din, r)")
    dout, rank = u.shape
    din, rank_v = v.shape
    if rank != rank_v:
        raise ValueError(f"joint_itq rank mismatch: u_hat r={rank}, v_hat r={rank_v}")
    if rank == 0 or dout + din == 0:
        raise ValueError("joint_itq expects non-empty factors")
    rr = gram_schmidt(splitmix_matrix(seed, rank))
    z = np.concatenate([u, v], axis=0)
    n_iter, converged = 0, False
    for it in range(1, int(max_iter) + 1):
        b = (matmul_lr(z, rr) >= 0.0).astype(np.float64) * 2.0 - 1.0
        umat, _s, vt = np.linalg.svd(matmul_at_b_lr(b, z), full_matrices=True)
        r_new = matmul_lr(np.ascontiguousarray(vt.T), np.ascontiguousarray(umat.T))
        delta = math.sqrt(_dot_lr((r_new - rr).ravel(), (r_new - rr).ravel()))
        rr = r_new
        n_iter = it
        if tol > 0.0 and delta <= tol:
            converged = True
            break
    zr = matmul_lr(z, rr)
    signs = np.where(zr >= 0.0, np.int8(1), np.int8(-1)).astype(np.int8)
    res = (signs[:dout].copy(), signs[dout:].copy(), n_iter, converged)
    return res + (zr,) if return_margin else res
