"""Tensor-parallel partitioning of a factorized-linear decoder (host-side, NumPy only).

The reference has no parallelism of any kind; this is the partitioning the benchmark
specification prescribes for the path: column-parallel layers (q, k, v, gate, up) split the
rows of Ub, s1 and the bias by output feature and replicate Vb^T and s2; row-parallel
layers (o, down) split the columns of Vb^T and s2 by input feature and replicate Ub and s1,
so their outputs are partial sums that one all-reduce per attention block and one per MLP
block complete.  Attention shards by KV head; the LM head by vocabulary rows.
"""

from __future__ import annotations

import numpy as np


def _range(n: int, rank: int, size: int) -> tuple[int, int]:
    if n % size:
        raise ValueError(f"dimension {n} is not divisible by tensor-parallel size {size}")
    step = n // size
    return rank * step, (rank + 1) * step


def _with_rows(layer: dict) -> dict:
    """A plain copy that holds the row bitplanes (a model directory's layer makes them on
    first use) and not the container streams, which describe the whole layer only."""
    layer["ub_rows"], layer["vb_t_rows"]  # noqa: B018  (touch: see model_dir._Factors)
    return {k: v for k, v in layer.items() if k not in ("ub_packed", "vb_packed")}


def shard_column_parallel(layer: dict, rank: int, size: int) -> dict:
    """Rows of Ub, s1 and bias for output features [lo, hi); Vb^T and s2 whole."""
    lo, hi = _range(layer["dout"], rank, size)
    out = _with_rows(layer)
    out["ub_rows"] = np.ascontiguousarray(layer["ub_rows"][lo:hi])
    out["s1"] = np.ascontiguousarray(layer["s1"][lo:hi])
    out["bias"] = None if layer.get("bias") is None else np.ascontiguousarray(layer["bias"][lo:hi])
    out["dout"] = hi - lo
    return out


def shard_row_parallel(layer: dict, rank: int, size: int) -> dict:
    """Columns of Vb^T and s2 for input features [lo, hi); Ub and s1 whole.  The bias is
    kept on rank 0 only, so that the all-reduce adds it once."""
    lo, hi = _range(layer["din"], rank, size)
    if lo % 8 or hi % 8:
        raise ValueError(f"row-parallel shard [{lo}, {hi}) must fall on byte boundaries")
    out = _with_rows(layer)
    out["vb_t_rows"] = np.ascontiguousarray(layer["vb_t_rows"][:, lo // 8:hi // 8])
    out["s2"] = np.ascontiguousarray(layer["s2"][lo:hi])
    out["din"] = hi - lo
    if rank != 0:
        out["bias"] = None
    return out


def shard_model(weights: dict, cfg, rank: int, size: int) -> dict:
    """The slice of a whole-model weight dict that rank `rank` of `size` holds."""
    if size == 1:
        return weights
    if cfg.n_kv_heads % size or cfg.n_heads % size or cfg.d_ff % size or cfg.vocab % size:
        raise ValueError(f"tensor-parallel size {size} must divide kv heads {cfg.n_kv_heads}, "
                         f"heads {cfg.n_heads}, d_ff {cfg.d_ff} and vocabulary {cfg.vocab}")
    out = {k: v for k, v in weights.items() if k != "layers"}
    out["layers"] = []
    for lw in weights["layers"]:
        s = {k: v for k, v in lw.items()
             if k not in ("q", "k", "v", "o", "gate", "up", "down")}
        for name in ("q", "k", "v", "gate", "up"):
            s[name] = shard_column_parallel(lw[name], rank, size)
        for name in ("o", "down"):
            s[name] = shard_row_parallel(lw[name], rank, size)
        out["layers"].append(s)
    lo, hi = _range(cfg.vocab, rank, size)
    head = weights["lm_head"][lo:hi]
    out["lm_head"] = np.ascontiguousarray(head) if isinstance(head, np.ndarray) else head
    out["vocab_offset"] = lo
    return out
