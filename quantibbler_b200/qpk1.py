"""Reader of the qpk1 layer stream, over the C ABI (host only).

Mirrors ``parse`` of crates/quantibbler-qpk1/src/lib.rs:229-320 (the server's reader of the
format written by src/quantibbler/qpk1.py:150-208): fail-closed, same messages, raised as
``ValueError``.  The binary factors stay packed (container bit streams); use
``PackedLayer.from_qpk1`` to put the layer on the GPU.
"""

from __future__ import annotations

import ctypes

import numpy as np

from . import _lib
from ._lib import check


class _Info(ctypes.Structure):
    _fields_ = [("version", ctypes.c_uint32), ("dtype_tag", ctypes.c_uint32)] + [
        (n, ctypes.c_size_t) for n in ("dout", "din", "r", "s1_offset", "s2_offset", "bias_offset",
                                       "ub_offset", "ub_len", "vb_offset", "vb_len")]


def parse(data) -> dict:
    """Header fields, float32 scales / bias and the packed factor streams of one layer.
    ``bias`` is ``None`` for a version-1 (pre-bias) stream."""
    raw = np.frombuffer(bytes(data), dtype=np.uint8) if not isinstance(data, np.ndarray) else data
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    info = _Info()
    check(_lib.lib().qk_qpk1_parse(raw.ctypes.data, raw.size, ctypes.byref(info)))
    s1 = np.zeros(info.dout, np.float32)
    s2 = np.zeros(info.din, np.float32)
    bias = np.zeros(info.dout, np.float32)
    check(_lib.lib().qk_qpk1_scales(raw.ctypes.data, raw.size, s1.ctypes.data, s2.ctypes.data,
                                    bias.ctypes.data))
    return {"version": int(info.version),
            "dtype": "float16" if info.dtype_tag == 1 else "float32",
            "dout": int(info.dout), "din": int(info.din), "r": int(info.r),
            "s1": s1, "s2": s2, "bias": bias if info.bias_offset else None,
            "ub_packed": raw[info.ub_offset:info.ub_offset + info.ub_len].copy(),
            "vb_packed": raw[info.vb_offset:info.vb_offset + info.vb_len].copy()}
