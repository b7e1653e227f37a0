"""NumPy oracle for the two attention kernels.  TEST INFRASTRUCTURE ONLY.

Parity status: PINNED.  ``attention_exact`` and ``attention_sage`` reproduce the
reference's committed vectors (crates/quantibbler-kernels/tests/fixtures/
attention_tiled.json and attention_sage.json, re-emitted under tests/golden/) and the
outputs of the reference's own NumPy functions on seeded inputs.

``attention_exact`` follows src/quantibbler/kernels/attention_tiled.py:76-180 (the
dense softmax(QK^T/sqrt(d))V it tiles, GQA head h -> kv head h // group, causal
positions removed before the row maximum), extended to seq_q != seq_kv with the
bottom-right alignment of the device contract
(crates/quantibbler-kernels/src/gpu_attention.rs:451-570: key j is masked for query i
when j + seq_q > i + seq_kv).

``attention_sage`` follows src/quantibbler/kernels/attention_sage.py:136-350 stage by
stage without recording per-tile statistics, so it runs at sequence lengths where the
reference's stats list would not fit in memory, and it can restrict itself to a subset
of query rows: a row's result depends only on that row and on the key blocks, never on
the other rows of its query tile.
"""

from __future__ import annotations

import math

import numpy as np

INT8_MAX = 127


def attention_exact(q, k, v, *, causal=False, rows=None) -> np.ndarray:
    """Dense f64 attention.  q (B,H,Sq,d), k (B,KV,Skv,d), v (B,KV,Skv,dv).

    ``rows`` optionally restricts the computed query positions; the result then has
    shape (B,H,len(rows),dv).
    """
    q = np.asarray(q, dtype=np.float64)
    k = np.asarray(k, dtype=np.float64)
    v = np.asarray(v, dtype=np.float64)
    b, h, sq, d = q.shape
    kvh, skv = k.shape[1], k.shape[2]
    group = h // kvh
    idx = np.arange(sq) if rows is None else np.asarray(rows)
    out = np.zeros((b, h, len(idx), v.shape[3]), dtype=np.float64)
    scale = 1.0 / math.sqrt(d)
    cols = np.arange(skv)
    for bi in range(b):
        for hi in range(h):
            kv = hi // group
            s = (q[bi, hi, idx] @ k[bi, kv].T) * scale
            if causal:
                blocked = cols[None, :] + sq > idx[:, None] + skv
                s = np.where(blocked, -np.inf, s)
            m = s.max(axis=-1, keepdims=True)
            p = np.exp(s - m)
            out[bi, hi] = (p @ v[bi, kv]) / p.sum(axis=-1, keepdims=True)
    return out


def _dynamic_scale(peak, ft):
    # attention_sage.py:148-161: delta = max|A|/127, zero range -> 1.0
    return np.where(peak > 0, peak / ft(INT8_MAX), ft(1.0)).astype(ft)


def quantize_per_token(x, ft=np.float64):
    """attention_sage.py:164-174."""
    x = np.asarray(x, dtype=ft)
    delta = _dynamic_scale(np.max(np.abs(x), axis=-1, keepdims=True), ft)
    hat = np.clip(np.rint(x / delta), -INT8_MAX, INT8_MAX)
    return hat.astype(np.int8), delta


def quantize_per_channel(x, ft=np.float64):
    """attention_sage.py:177-189 (scale over the token axis of the tile)."""
    x = np.asarray(x, dtype=ft)
    delta = _dynamic_scale(np.max(np.abs(x), axis=-2, keepdims=True), ft)
    hat = np.clip(np.rint(x / delta), -INT8_MAX, INT8_MAX)
    return hat.astype(np.int8), delta


def attention_sage(q, k, v, *, causal=False, block_size=64, rows=None, ft=np.float64,
                   return_codes=False):
    """[SA] section-4 INT8 attention as the reference computes it.

    ``ft`` is the float type of every non-integer stage: float64 reproduces
    attention_sage.py; float32 is the arithmetic of the device kernel
    (gpu_attention.rs:67-397) and is what INT8 codes are compared bit-for-bit against.
    With ``return_codes`` also returns (q_hat, k_hat, v_hat) for the visited tiles.
    """
    q = np.asarray(q, dtype=ft)
    k = np.asarray(k, dtype=ft)
    v = np.asarray(v, dtype=ft)
    b, h, s, d = q.shape
    kvh = k.shape[1]
    assert k.shape[2] == s and v.shape[2] == s, "sage attention is self-attention"
    group = h // kvh
    idx = np.arange(s) if rows is None else np.asarray(rows)
    dv = v.shape[3]
    inv_sqrt_d = ft(1.0 / math.sqrt(d)) if ft is np.float64 else ft(1.0) / np.sqrt(ft(d))
    q_hat, q_scale = quantize_per_token(q[:, :, idx] * inv_sqrt_d, ft)
    q_deq = q_hat.astype(ft) * q_scale
    out = np.zeros((b, h, len(idx), dv), dtype=ft)
    kv_index = np.repeat(np.arange(kvh), group)
    p_scale = ft(1.0) / ft(127.0)

    m = np.full((b, h, len(idx), 1), -np.inf, dtype=ft)
    ell = np.zeros((b, h, len(idx), 1), dtype=ft)
    acc = np.zeros((b, h, len(idx), dv), dtype=ft)
    j_hi = (int(idx.max()) + 1) if causal else s
    k_codes, v_codes = [], []
    for j0 in range(0, j_hi, block_size):
        j1 = min(j0 + block_size, s)
        cols = np.arange(j0, j1)
        kb = k[:, :, j0:j1]
        if ft is np.float64:
            k_mean = kb.mean(axis=-2, keepdims=True)
        else:
            # the device kernel sums the block's tokens one by one in float32 and divides
            # once (gpu_attention.rs:197-209); reproduce that order so codes can match
            ssum = np.zeros(kb.shape[:2] + (1, d), dtype=ft)
            for jj in range(kb.shape[2]):
                ssum = (ssum + kb[:, :, jj:jj + 1]).astype(ft)
            k_mean = (ssum / ft(kb.shape[2])).astype(ft)
        k_hat, k_scale = quantize_per_token(kb - k_mean, ft)
        dot = np.matmul(q_hat.astype(np.int32), k_hat[:, kv_index].astype(np.int32).swapaxes(-1, -2))
        scores = dot.astype(ft) * q_scale * k_scale[:, kv_index].swapaxes(-1, -2) \
            + q_deq @ k_mean[:, kv_index].swapaxes(-1, -2)
        if causal:
            scores = np.where(cols[None, :] > idx[:, None], ft(-np.inf), scores)
        m_new = np.maximum(m, scores.max(axis=-1, keepdims=True))
        empty = np.isneginf(m_new)
        with np.errstate(invalid="ignore"):
            alpha = np.where(empty, ft(0), np.exp(m - m_new))
            p = np.where(empty, ft(0), np.exp(scores - m_new)).astype(ft)
        ell = alpha * ell + p.sum(axis=-1, keepdims=True, dtype=ft)
        p_hat = np.clip(np.rint(p / p_scale), 0, INT8_MAX).astype(np.int32)
        v_hat, v_scale = quantize_per_channel(v[:, :, j0:j1], ft)
        pv = np.matmul(p_hat, v_hat[:, kv_index].astype(np.int32))
        contrib = pv.astype(ft) * p_scale * v_scale[:, kv_index]
        acc = alpha * acc + np.where(empty, ft(0), contrib)
        m = m_new
        if return_codes:
            k_codes.append(k_hat)
            v_codes.append(v_hat)
    with np.errstate(invalid="ignore", divide="ignore"):
        out = acc / ell
    if return_codes:
        return out, (q_hat, k_codes, v_codes)
    return out


def parity_two_part(got, want, row_len, rtol, band):
    """The reference's two-part gate (tests/gpu_attention_parity.rs:81-127).

    Returns (inf-norm relative error, worst per-element relative error among elements
    at least ``band`` x their row's max magnitude).
    """
    got = np.asarray(got, dtype=np.float64).reshape(-1, row_len)
    want = np.asarray(want, dtype=np.float64).reshape(-1, row_len)
    norm = max(np.abs(want).max(), np.abs(got).max())
    inf_rel = np.abs(got - want).max() / norm
    row_max = np.abs(want).max(axis=1, keepdims=True)
    sel = (np.abs(want) >= band * row_max) & (np.abs(want) > 0)
    worst = float((np.abs(got - want)[sel] / np.abs(want)[sel]).max()) if sel.any() else 0.0
    return float(inf_rel), worst


def quality_metrics(got, want):
    """cosine, relative L1, RMSE (tests/gpu_attention_sage.rs:147-165)."""
    g = np.asarray(got, dtype=np.float64).ravel()
    w = np.asarray(want, dtype=np.float64).ravel()
    cos = float(g @ w / (np.linalg.norm(g) * np.linalg.norm(w)))
    rel_l1 = float(np.abs(g - w).sum() / np.abs(w).sum())
    rmse = float(np.sqrt(np.mean((g - w) ** 2)))
    return cos, rel_l1, rmse


def attention_sage_block(q, k, v, *, causal=False, rows=None):
    """The benchmark specification's wording of Sage, restated: NOT the reference's arithmetic,
    and pinned to nothing (the reference holds no implementation, fixture or golden vector of
    it: parity unpinned).  "Q and K use per-64-token-block INT8 symmetric quantisation [with K
    mean-smoothing]; PV is computed in bf16 with fp32 online-softmax accumulation."

    Q / sqrt(d) gets one scale per block of 64 queries; K has its 64-key block's channel mean
    removed (as the reference's gamma does per block, attention_sage.py:164-198) and then one
    scale per block; scores = dQ dK (Qhat . Khat) + (dQ Qhat) . mean; the softmax is exact here
    (float64), V is rounded to bfloat16, P is NOT rounded: what the device adds on top is the
    bfloat16 rounding of P and float32 accumulation, which the test's tolerance covers.
    float32 is used where the device forms the quantities that decide an INT8 code.
    """
    ft = np.float32
    q = np.asarray(q, dtype=ft)
    k = np.asarray(k, dtype=ft)
    v = np.asarray(v, dtype=ft)
    b, h, s, d = q.shape
    kvh = k.shape[1]
    assert k.shape[2] == s and v.shape[2] == s, "sage attention is self-attention"
    group = h // kvh
    kv_index = np.repeat(np.arange(kvh), group)
    blk = 64
    inv_sqrt_d = ft(1.0) / np.sqrt(ft(d))
    qs = (q * inv_sqrt_d).astype(ft)
    q_hat = np.zeros(q.shape, dtype=np.int32)
    q_scale = np.zeros((b, h, s, 1), dtype=ft)
    for i0 in range(0, s, blk):
        part = qs[:, :, i0:i0 + blk]
        peak = np.abs(part).max(axis=(-1, -2), keepdims=True)
        delta = np.where(peak > 0, peak / ft(127.0), ft(1.0)).astype(ft)
        q_hat[:, :, i0:i0 + blk] = np.clip(np.rint(part / delta), -INT8_MAX, INT8_MAX).astype(np.int32)
        q_scale[:, :, i0:i0 + blk] = delta
    q_deq = q_hat.astype(ft) * q_scale
    idx = np.arange(s) if rows is None else np.asarray(rows)
    scores = np.full((b, h, len(idx), s), -np.inf, dtype=np.float64)
    for j0 in range(0, s, blk):
        j1 = min(j0 + blk, s)
        kb = k[:, :, j0:j1]
        ssum = np.zeros(kb.shape[:2] + (1, d), dtype=ft)
        for jj in range(kb.shape[2]):          # the device's order: token by token in float32
            ssum = (ssum + kb[:, :, jj:jj + 1]).astype(ft)
        k_mean = (ssum / ft(kb.shape[2])).astype(ft)
        cen = (kb - k_mean).astype(ft)
        peak = np.abs(cen).max(axis=(-1, -2), keepdims=True)
        delta = np.where(peak > 0, peak / ft(127.0), ft(1.0)).astype(ft)
        k_hat = np.clip(np.rint(cen / delta), -INT8_MAX, INT8_MAX).astype(np.int32)
        dot = np.matmul(q_hat[:, :, idx], k_hat[:, kv_index].swapaxes(-1, -2))
        sc = dot.astype(np.float64) * q_scale[:, :, idx].astype(np.float64) * delta[:, kv_index].astype(np.float64) \
            + q_deq[:, :, idx].astype(np.float64) @ k_mean[:, kv_index].astype(np.float64).swapaxes(-1, -2)
        scores[..., j0:j1] = sc
    if causal:
        scores = np.where(np.arange(s)[None, :] > idx[:, None], -np.inf, scores)
    scores = scores - scores.max(axis=-1, keepdims=True)
    p = np.exp(scores)
    p /= p.sum(axis=-1, keepdims=True)
    u = v.view(np.uint32).astype(np.uint64)     # V rounded to bfloat16 (ties to even)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    v_bf = u.view(np.float32).astype(np.float64)
    return np.matmul(p, v_bf[:, kv_index]).astype(np.float32)
