"""Host-side mirror of the reference's device face and factorized-linear layer.

``GpuContext`` mirrors crates/quantibbler-kernels/src/gpu.rs:76-184 (``init``,
``init_at``, ``packed_matvec``) and gpu_attention.rs:451-756 (``attention``,
``attention_sage``); ``AttentionShape`` mirrors gpu_attention.rs:402-411;
``PackedLayer`` mirrors crates/quantibbler-server/src/engine/mod.rs:313-480.  Names,
argument meaning and error behaviour follow the reference; the arithmetic runs in
libqk_kernels.so.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np

from . import _lib
from ._lib import QK_BF16, QK_F32, DeviceError, KernelError, check

GPU_INDEX_CEILING = 0xFFFFFFFF  # gpu.rs:42-45


def gpu_init_hint() -> str:
    """gpu.rs:36-40 (GPU_INIT_HINT), naming the CUDA requirements."""
    return _lib.lib().qk_gpu_init_hint().decode()


def gpu_available() -> bool:
    """gpu.rs:187-189."""
    return bool(_lib.lib().qk_gpu_available())


@dataclass(frozen=True)
class AttentionShape:
    """gpu_attention.rs:402-411."""
    batch: int
    n_heads: int
    n_kv_heads: int
    seq_q: int
    seq_kv: int
    head_dim: int
    val_dim: int


def _f(a, dtype):
    return np.ascontiguousarray(np.asarray(a, dtype=dtype))


class GpuContext:
    """A live CUDA context on one device (gpu.rs:76-113).

    Construction fails closed: every failure raises ``DeviceError`` with
    ``gpu_init_hint()`` embedded.  Safe to share between host threads.
    """

    def __init__(self, handle):
        self._h = handle

    @classmethod
    def init_at(cls, device_index: int) -> "GpuContext":
        h = ctypes.c_void_p()
        check(_lib.lib().qk_gpu_init_at(int(device_index), ctypes.byref(h)))
        return cls(h)

    @classmethod
    def init(cls) -> "GpuContext":
        return cls.init_at(0)

    def close(self) -> None:
        if self._h:
            _lib.lib().qk_gpu_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self):
        return self._h

    def synchronize(self) -> None:
        check(_lib.lib().qk_gpu_synchronize(self._h))

    @property
    def stream(self) -> int:
        return int(_lib.lib().qk_gpu_stream(self._h) or 0)

    def set_stream(self, cuda_stream: int | None) -> None:
        """Launch on a caller-owned stream; ``None`` restores the context's own stream.
        The legacy default stream has the numeric handle 0, which the C ABI reads as
        "restore": pass it as cudaStreamLegacy (1) instead."""
        if cuda_stream is None:
            handle = 0
        else:
            handle = int(cuda_stream) or 1
        check(_lib.lib().qk_gpu_set_stream(self._h, ctypes.c_void_p(handle)))

    def container_to_rows(self, stream, n_rows: int, r: int, transposed: bool = False) -> np.ndarray:
        """The container repack of engine/mod.rs:258-289 run by the device's kernels (the ones
        ``PackedLayer.from_container`` uses): ``stream`` holds an ``n_rows x r`` sign matrix
        bit by bit; the result is its rows (``n_rows x ceil(r/8)`` bytes) or, transposed, its
        columns (``r x ceil(n_rows/8)``)."""
        s = _f(stream, np.uint8).ravel()
        rows, bits = (int(r), int(n_rows)) if transposed else (int(n_rows), int(r))
        out = np.zeros((rows, (bits + 7) // 8), np.uint8)
        check(_lib.lib().qk_gpu_container_to_rows(self._h, s.ctypes.data, s.size, int(n_rows),
                                                  int(r), int(bool(transposed)),
                                                  out.ctypes.data, out.size))
        return out

    def set_gemv_kernel(self, which: int) -> int:
        return int(_lib.lib().qk_set_gemv_kernel(self._h, int(which)))

    @property
    def launch_count(self) -> int:
        return int(_lib.lib().qk_gpu_launch_count(self._h))

    def packed_matvec(self, packed, n_rows: int, n_bits: int, vec) -> np.ndarray:
        """float64 ``unpack(packed) @ vec`` on the device (gpu.rs:116-183)."""
        p = _f(packed, np.uint8).ravel()
        v = _f(vec, np.float64).ravel()
        out = np.zeros(int(n_rows), dtype=np.float64)
        check(_lib.lib().qk_gpu_packed_matvec(self._h, p.ctypes.data, p.size, int(n_rows),
                                              int(n_bits), v.ctypes.data, v.size,
                                              out.ctypes.data))
        return out


class _ShapeStruct(ctypes.Structure):
    _fields_ = [(n, ctypes.c_size_t) for n in ("batch", "n_heads", "n_kv_heads", "seq_q", "seq_kv",
                                               "head_dim", "val_dim")]


def _attention(self, fn_name, shape, query, key, value, causal, block_size=None):
    q = _f(query, np.float32).ravel()
    k = _f(key, np.float32).ravel()
    v = _f(value, np.float32).ravel()
    st = _ShapeStruct(shape.batch, shape.n_heads, shape.n_kv_heads, shape.seq_q, shape.seq_kv,
                      shape.head_dim, shape.val_dim)
    out = np.zeros(shape.batch * shape.n_heads * shape.seq_q * shape.val_dim, dtype=np.float32)
    fn = getattr(_lib.lib(), fn_name)
    args = [self._h, ctypes.byref(st), q.ctypes.data, q.size, k.ctypes.data, k.size, v.ctypes.data,
            v.size, int(bool(causal))]
    if block_size is not None:
        args.append(int(block_size))
    check(fn(*args, out.ctypes.data, out.size))
    return out


def _gpu_attention(self, shape: AttentionShape, query, key, value, causal: bool) -> np.ndarray:
    """Exact tiled attention, flat float32 in and out (gpu_attention.rs:451-570)."""
    return _attention(self, "qk_gpu_attention", shape, query, key, value, causal)


def _gpu_attention_sage(self, shape: AttentionShape, query, key, value, causal: bool,
                        block_size: int) -> np.ndarray:
    """Sage INT8 attention (gpu_attention.rs:589-756)."""
    if block_size < 0:
        raise OverflowError("can't convert negative int to unsigned")
    return _attention(self, "qk_gpu_attention_sage", shape, query, key, value, causal, block_size)


def _gpu_attention_dev(self, shape: AttentionShape, q_ptr: int, k_ptr: int, v_ptr: int,
                       causal: bool, out_ptr: int, block_size: int | None = None) -> None:
    """Either attention face on float32 device buffers, asynchronous on the context's stream
    (``block_size`` given: the Sage face)."""
    st = _ShapeStruct(shape.batch, shape.n_heads, shape.n_kv_heads, shape.seq_q, shape.seq_kv,
                      shape.head_dim, shape.val_dim)
    ptrs = [ctypes.c_void_p(p) for p in (q_ptr, k_ptr, v_ptr)]
    if block_size is None:
        check(_lib.lib().qk_gpu_attention_dev(self._h, ctypes.byref(st), *ptrs, int(bool(causal)),
                                              ctypes.c_void_p(out_ptr)))
    else:
        check(_lib.lib().qk_gpu_attention_sage_dev(self._h, ctypes.byref(st), *ptrs,
                                                   int(bool(causal)), int(block_size),
                                                   ctypes.c_void_p(out_ptr)))


def _gpu_attention_sage_block_dev(self, shape: AttentionShape, q_ptr: int, k_ptr: int, v_ptr: int,
                                  causal: bool, out_ptr: int) -> None:
    """The benchmark specification's Sage variant (one INT8 scale per 64-token block for Q and K,
    bfloat16 P and V) on float32 device buffers; NOT the reference's arithmetic.  Asynchronous."""
    st = _ShapeStruct(shape.batch, shape.n_heads, shape.n_kv_heads, shape.seq_q, shape.seq_kv,
                      shape.head_dim, shape.val_dim)
    check(_lib.lib().qk_gpu_attention_sage_block_dev(
        self._h, ctypes.byref(st), ctypes.c_void_p(q_ptr), ctypes.c_void_p(k_ptr), ctypes.c_void_p(v_ptr),
        int(bool(causal)), ctypes.c_void_p(out_ptr)))


def _set_sage_kernel(self, which: int) -> int:
    """2: the tcgen05 Sage kernel where the shape allows (default), else as 1; 1: the mma.sync
    INT8 tensor-core kernel where the shape allows, else as 0; 0: the dp4a kernel.  Returns the
    previous choice."""
    return int(_lib.lib().qk_set_sage_kernel(self._h, int(which)))


def _set_decode_attention_kernel(self, which: int) -> int:
    """1: tensor-core decode attention where the cache allows (default); 0: the scalar kernel;
    anything else only reads the choice.  Returns the previous choice."""
    return int(_lib.lib().qk_set_decode_attention_kernel(self._h, int(which)))


def _gpu_sage_quantize(self, shape: AttentionShape, query, key, value, block_size: int) -> dict:
    """The INT8 codes and scales the Sage face computes before its integer products
    (attention_sage.py:164-198 as applied by gpu_attention.rs:132-260), in plain layouts:
    ``q_codes [B,H,S,d]``, ``q_scale [B,H,S]``, ``k_codes [B,KV,S,d]``, ``k_scale [B,KV,S]``,
    ``k_mean [B,KV,blocks,d]``, ``v_codes [B,KV,S,dv]``, ``v_scale [B,KV,blocks,dv]``."""
    q = _f(query, np.float32).ravel()
    k = _f(key, np.float32).ravel()
    v = _f(value, np.float32).ravel()
    st = _ShapeStruct(shape.batch, shape.n_heads, shape.n_kv_heads, shape.seq_q, shape.seq_kv,
                      shape.head_dim, shape.val_dim)
    B, H, KV, S, d, dv = (shape.batch, shape.n_heads, shape.n_kv_heads, shape.seq_kv,
                          shape.head_dim, shape.val_dim)
    blocks = -(-S // min(int(block_size), S)) if block_size > 0 and S > 0 else 0
    out = dict(q_codes=np.zeros((B, H, S, d), np.int8), q_scale=np.zeros((B, H, S), np.float32),
               k_codes=np.zeros((B, KV, S, d), np.int8), k_scale=np.zeros((B, KV, S), np.float32),
               k_mean=np.zeros((B, KV, blocks, d), np.float32),
               v_codes=np.zeros((B, KV, S, dv), np.int8),
               v_scale=np.zeros((B, KV, blocks, dv), np.float32))
    check(_lib.lib().qk_gpu_sage_quantize(
        self._h, ctypes.byref(st), q.ctypes.data, q.size, k.ctypes.data, k.size, v.ctypes.data,
        v.size, int(block_size), *[out[n].ctypes.data for n in (
            "q_codes", "q_scale", "k_codes", "k_scale", "k_mean", "v_codes", "v_scale")]))
    return out


GpuContext.sage_quantize = _gpu_sage_quantize
GpuContext.attention = _gpu_attention
GpuContext.attention_sage = _gpu_attention_sage
GpuContext.attention_dev = _gpu_attention_dev
GpuContext.attention_sage_block_dev = _gpu_attention_sage_block_dev
GpuContext.set_sage_kernel = _set_sage_kernel
GpuContext.set_decode_attention_kernel = _set_decode_attention_kernel


def _set_wait_limit(self, polls: int) -> int:
    """Polls a device-side wait makes before it gives up (0: the default); returns the
    previous value."""
    return int(_lib.lib().qk_set_wait_limit(self._h, int(polls)))


GpuContext.set_wait_limit = _set_wait_limit


def _set_dependent_launch(self, on: bool) -> bool:
    """Programmatic dependent launch of the decoder-path kernels (default on); returns the
    previous setting."""
    return bool(_lib.lib().qk_set_dependent_launch(self._h, int(bool(on))))


GpuContext.set_dependent_launch = _set_dependent_launch


class PackedLayer:
    """Device-resident factorized linear (engine/mod.rs:313-381).

    ``ub_rows`` is ``dout x ceil(r/8)`` and ``vb_t_rows`` is ``r x ceil(din/8)`` uint8, the
    per-row bitplanes the reference's ``PackedLayer`` holds; ``serving`` is ``"float32"``
    or ``"bfloat16"`` (``ServingDtype``).
    """

    def __init__(self, ctx: GpuContext, ub_rows, vb_t_rows, dout: int, din: int, r: int, s1, s2,
                 bias=None, serving: str = "float32", name: str = ""):
        if serving not in ("float32", "bfloat16"):
            raise KernelError(f"serving dtype must be float32 or bfloat16, got {serving!r}")
        self.ctx, self.name = ctx, name
        self.dout, self.din, self.r, self.serving = int(dout), int(din), int(r), serving
        ub = _f(ub_rows, np.uint8).ravel()
        vbt = _f(vb_t_rows, np.uint8).ravel()
        s1 = _f(s1, np.float32).ravel()
        s2 = _f(s2, np.float32).ravel()
        if s1.size != self.dout or s2.size != self.din:
            raise KernelError(f"layer {name}: scale lengths {s1.size}/{s2.size} do not match "
                              f"dout={dout}, din={din}")
        b = None
        if bias is not None and np.size(bias):
            b = _f(bias, np.float32).ravel()
            if b.size != self.dout:  # engine/mod.rs:357-363
                raise KernelError(
                    f"layer {name}: bias has {b.size} entries; expected dout={dout}")
        h = ctypes.c_void_p()
        check(_lib.lib().qk_layer_create(
            ctx.handle, ub.ctypes.data, ub.size, vbt.ctypes.data, vbt.size, self.dout, self.din,
            self.r, s1.ctypes.data, s2.ctypes.data, b.ctypes.data if b is not None else None,
            QK_F32 if serving == "float32" else QK_BF16, ctypes.byref(h)))
        self._h = h

    @classmethod
    def from_container(cls, ctx, ub_packed, vb_packed, dout, din, r, s1, s2, bias=None,
                       serving="float32", name=""):
        """engine/mod.rs:342-381 (from_layer) from the container's bit streams of Ub
        (dout x r) and Vb (din x r): uploaded as they are, the rows of Ub and of Vb^T are
        separated on the device (the repack of engine/mod.rs:258-289)."""
        if serving not in ("float32", "bfloat16"):
            raise KernelError(f"serving dtype must be float32 or bfloat16, got {serving!r}")
        self = cls.__new__(cls)
        self.ctx, self.name, self.serving = ctx, name, serving
        self.dout, self.din, self.r = int(dout), int(din), int(r)
        ub = _f(ub_packed, np.uint8).ravel()
        vb = _f(vb_packed, np.uint8).ravel()
        s1 = _f(s1, np.float32).ravel()
        s2 = _f(s2, np.float32).ravel()
        if s1.size != self.dout or s2.size != self.din:
            raise KernelError(f"layer {name}: scale lengths {s1.size}/{s2.size} do not match "
                              f"dout={dout}, din={din}")
        b = None
        if bias is not None and np.size(bias):
            b = _f(bias, np.float32).ravel()
            if b.size != self.dout:  # engine/mod.rs:357-363
                raise KernelError(
                    f"layer {name}: bias has {b.size} entries; expected dout={dout}")
        h = ctypes.c_void_p()
        check(_lib.lib().qk_layer_create_from_streams(
            ctx.handle, ub.ctypes.data, ub.size, vb.ctypes.data, vb.size, self.dout, self.din,
            self.r, s1.ctypes.data, s2.ctypes.data, b.ctypes.data if b is not None else None,
            QK_F32 if serving == "float32" else QK_BF16, ctypes.byref(h)))
        self._h = h
        return self

    @classmethod
    def from_qpk1(cls, ctx, data, serving="float32", name=""):
        """A layer straight from its qpk1 stream (crates/quantibbler-qpk1/src/lib.rs:229-320
        parse + engine/mod.rs:342-381 from_layer); a malformed stream raises the reader's
        ``ValueError`` text."""
        from . import qpk1
        raw = np.frombuffer(bytes(data), dtype=np.uint8)
        info = qpk1.parse(raw)
        self = cls.__new__(cls)
        self.ctx, self.name, self.serving = ctx, name, serving
        self.dout, self.din, self.r = info["dout"], info["din"], info["r"]
        h = ctypes.c_void_p()
        check(_lib.lib().qk_layer_from_qpk1(ctx.handle, raw.ctypes.data, raw.size,
                                            QK_F32 if serving == "float32" else QK_BF16,
                                            ctypes.byref(h)))
        self._h = h
        return self

    def close(self) -> None:
        if getattr(self, "_h", None):
            _lib.lib().qk_layer_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self):
        return self._h

    def apply(self, x) -> np.ndarray:
        """``y = s1*(Ub(Vb^T(s2*x))) + bias`` for one token, host arrays in and out
        (engine/mod.rs:393-437 and :449-460)."""
        xv = _f(x, np.float32).ravel()
        if xv.size != self.din:
            raise KernelError(
                f"layer {self.name} expects input dim {self.din}, got {xv.size}")
        y = np.zeros(self.dout, dtype=np.float32)
        check(_lib.lib().qk_layer_apply_host(self.ctx.handle, self._h, xv.ctypes.data, xv.size,
                                             y.ctypes.data, y.size))
        return y

    def apply_prefill(self, x_ptr: int, n_tokens: int, y_ptr: int) -> None:
        """Many tokens at once on the tensor cores (bfloat16 serving only).  Asynchronous on the
        context's stream; ``ctx.synchronize()`` reports an expired in-kernel wait."""
        check(_lib.lib().qk_layer_apply_prefill(self.ctx.handle, self._h, ctypes.c_void_p(x_ptr),
                                                int(n_tokens), ctypes.c_void_p(y_ptr)))

    def apply_device(self, x_ptr: int, n_tokens: int, y_ptr: int) -> None:
        """Asynchronous apply on device buffers (float32, row-major tokens)."""
        check(_lib.lib().qk_layer_apply(self.ctx.handle, self._h, ctypes.c_void_p(x_ptr),
                                        int(n_tokens), ctypes.c_void_p(y_ptr)))


def apply_prefill_many(layers, x_ptr: int, n_tokens: int, y_ptrs) -> None:
    """Up to four bfloat16-serving layers that read the same input (q, k, v or gate, up) through
    the tensor-core GEMM with one launch per stage for all of them.  Asynchronous."""
    n = len(layers)
    handles = (ctypes.c_void_p * n)(*[layer._h for layer in layers])
    outs = (ctypes.c_void_p * n)(*[ctypes.c_void_p(p) for p in y_ptrs])
    check(_lib.lib().qk_layers_apply_prefill(layers[0].ctx.handle, handles, n, ctypes.c_void_p(x_ptr),
                                             int(n_tokens), outs))


def apply_prefill_many_gated(layers, gate_ptr: int, up_ptr: int, n_tokens: int, y_ptrs) -> None:
    """``apply_prefill_many`` on ``silu(gate) * up`` (the down projection behind the SwiGLU),
    the activation formed inside the GEMM's scaling kernel.  Asynchronous."""
    n = len(layers)
    handles = (ctypes.c_void_p * n)(*[layer._h for layer in layers])
    outs = (ctypes.c_void_p * n)(*[ctypes.c_void_p(p) for p in y_ptrs])
    check(_lib.lib().qk_layers_apply_prefill_gated(layers[0].ctx.handle, handles, n, ctypes.c_void_p(gate_ptr),
                                                   ctypes.c_void_p(up_ptr), int(n_tokens), outs))


def apply_noalloc(layer: PackedLayer, x_ptr: int, y_ptr: int) -> None:
    """One token through ``layer`` with the library allocating nothing: for hosts that own
    all device memory themselves (for example a server whose KV cache took what was left
    at start-up).  Same values as ``apply_device(x, 1, y)``; limited to r <= 8192 and
    din <= 16384; calls that overlap on the GPU share one built-in scratch and race."""
    check(_lib.lib().qk_layer_apply_noalloc(layer.ctx.handle, layer.handle, ctypes.c_void_p(x_ptr),
                                            ctypes.c_void_p(y_ptr)))


def apply_group(ctx: GpuContext, layers, x_ptr: int, y_ptr: int) -> None:
    """Same-shape layers in one pair of launches; layer i reads x + i*din floats."""
    arr = (ctypes.c_void_p * len(layers))(*[l.handle for l in layers])
    check(_lib.lib().qk_layers_apply_group(ctx.handle, arr, len(layers), ctypes.c_void_p(x_ptr),
                                           ctypes.c_void_p(y_ptr)))


class LayerGroup:
    """Same-shape layers bound once to device buffers (layer i reads x + i*din floats and
    writes y + i*dout floats); ``apply`` is two kernel launches."""

    def __init__(self, ctx: GpuContext, layers, x_ptr: int, y_ptr: int):
        self.ctx, self.layers = ctx, list(layers)
        arr = (ctypes.c_void_p * len(self.layers))(*[l.handle for l in self.layers])
        h = ctypes.c_void_p()
        check(_lib.lib().qk_group_create(ctx.handle, arr, len(self.layers), ctypes.c_void_p(x_ptr),
                                         ctypes.c_void_p(y_ptr), ctypes.byref(h)))
        self._h = h

    def apply(self) -> None:
        check(_lib.lib().qk_group_apply(self.ctx.handle, self._h))

    def close(self) -> None:
        if getattr(self, "_h", None):
            _lib.lib().qk_group_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class HostLayerGroup:
    """Same-shape layers applied to HOST inputs in one step.  The per-layer host call
    (``PackedLayer.apply``, the shape of the reference's ``PackedLayer::apply``) pays two
    copies, two launches and a synchronisation per layer; a caller that has many independent
    applies ready (all layers of a step, or one layer for many requests) hands them over
    together.  The layers are cut into a few sub-groups that run as a pipeline on three
    streams - inputs up, launch, outputs down - so that the upload of one sub-group, the
    kernels of the previous one and the download of the one before overlap (the link is full
    duplex).  ``x_host`` is ``[n_layers, din]`` and ``y_host`` ``[n_layers, dout]`` float32
    torch CPU tensors; pinned memory makes both copies asynchronous DMA."""

    def __init__(self, ctx: GpuContext, layers, n_parts: int | None = None, bounds=None):
        import torch
        self.torch, self.ctx, self.layers = torch, ctx, list(layers)
        first = self.layers[0]
        n = len(self.layers)
        self.x_dev = torch.zeros((n, first.din), dtype=torch.float32, device="cuda")
        self.y_dev = torch.zeros((n, first.dout), dtype=torch.float32, device="cuda")
        # sub-groups of at least ~300 layers keep every launch in its many-instance form
        # (measured on 2368 config-0 layers: 4 parts 2200 GB/s, 8 parts 2550, 12 parts 2120;
        # uneven splits given through `bounds` - a short first or last sub-group, tapered
        # sizes, 16 x 148 - all measured below the even 8 x 296: 2310-2585 against 2595)
        if n_parts is None:
            n_parts = max(1, min(8, n // 296))
        if bounds is None:
            bounds = [n * i // n_parts for i in range(n_parts + 1)]
        bounds = [int(b) for b in bounds]
        if bounds[0] != 0 or bounds[-1] != n or any(a >= b for a, b in zip(bounds, bounds[1:])):
            raise KernelError(f"sub-group bounds must rise from 0 to {n}, got {bounds}")
        n_parts = len(bounds) - 1
        self.parts = []
        for lo, hi in zip(bounds[:-1], bounds[1:]):
            self.parts.append(LayerGroup(ctx, self.layers[lo:hi], self.x_dev[lo:hi].data_ptr(),
                                         self.y_dev[lo:hi].data_ptr()))
        self._groups = (ctypes.c_void_p * n_parts)(*[g._h for g in self.parts])
        self._rows = (ctypes.c_size_t * (n_parts + 1))(*bounds)

    def apply(self, x_host, y_host) -> None:
        """``y_host[i] = layer_i(x_host[i])`` for every layer; returns when ``y_host`` is valid.
        One library call (``qk_groups_apply_host``) queues the whole pipeline."""
        if tuple(x_host.shape) != tuple(self.x_dev.shape) or tuple(y_host.shape) != tuple(
                self.y_dev.shape):
            raise KernelError(f"host buffers must be {tuple(self.x_dev.shape)} and "
                              f"{tuple(self.y_dev.shape)}, got {tuple(x_host.shape)} and "
                              f"{tuple(y_host.shape)}")
        if not (x_host.is_contiguous() and y_host.is_contiguous()):
            raise KernelError("host buffers must be contiguous")
        check(_lib.lib().qk_groups_apply_host(
            self.ctx.handle, self._groups, self._rows, len(self.parts), ctypes.c_void_p(x_host.data_ptr()),
            ctypes.c_void_p(y_host.data_ptr()), ctypes.c_void_p(self.x_dev.data_ptr()),
            ctypes.c_void_p(self.y_dev.data_ptr()), self.layers[0].din, self.layers[0].dout))

    def close(self) -> None:
        for group in self.parts:
            group.close()


class Feed(ctypes.Structure):
    """The C ABI's ``qk_feed``: up to four arrays of feed targets and, for each, how many
    consecutive targets read one token."""
    _fields_ = [("targets", ctypes.c_void_p * 4), ("per_token", ctypes.c_size_t * 4),
                ("n_arrays", ctypes.c_size_t)]


def make_feed(pairs) -> Feed:
    """``pairs``: [(fed LayerPlan, targets per token), ...]."""
    f = Feed()
    for i, (plan, per_token) in enumerate(pairs):
        ptr, n = plan.feed_targets()
        if n % per_token:
            raise KernelError(f"a plan of {n} instances cannot be fed {per_token} per token")
        f.targets[i] = ptr
        f.per_token[i] = per_token
    f.n_arrays = len(pairs)
    return f


class StepBlock(ctypes.Structure):
    """The C ABI's ``qk_step_block``: one transformer block's layers, norm weights and caches."""
    _fields_ = [(n, ctypes.c_void_p) for n in ("q", "k", "v", "o", "gate", "up", "down", "input_norm",
                                               "post_norm", "cache_k", "cache_v")]


class StepBuffers(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in ("x", "x2", "q", "k", "v", "attn", "delta_attn", "delta_mlp",
                                               "gate", "up", "att_scratch", "cos_sin", "positions",
                                               "seq_index", "kv_len")]


class StepDesc(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_size_t) for n in ("n_blocks", "n_tokens", "d_model", "n_heads", "n_kv_heads",
                                                "head_dim", "d_ff", "s_max", "n_seq", "n_splits")] +
                [("rms_eps", ctypes.c_float), ("serving_dtype", ctypes.c_int32), ("kv_dtype", ctypes.c_int32),
                 ("blocks", ctypes.POINTER(StepBlock)), ("buf", StepBuffers)])


class DecodeStep:
    """All transformer blocks of one decode step as one cooperative kernel
    (``qk_decode_step_create`` / ``qk_decode_step_run``).  ``blocks``: per block a dict with the
    seven PackedLayers under their names, ``input_norm`` / ``post_norm`` / ``cache_k`` / ``cache_v``
    device pointers; ``buffers``: the names of ``StepBuffers`` mapped to device pointers;
    ``dims``: the size fields of ``StepDesc``.  Raises KernelError when the configuration is
    outside what the kernel takes."""

    def __init__(self, ctx: GpuContext, blocks, buffers: dict, serving_tag: int, kv_tag: int, rms_eps: float,
                 **dims):
        self.ctx = ctx
        self._keep = [b[n] for b in blocks for n in ("q", "k", "v", "o", "gate", "up", "down")]
        arr = (StepBlock * len(blocks))()
        for dst, b in zip(arr, blocks):
            for n in ("q", "k", "v", "o", "gate", "up", "down"):
                setattr(dst, n, b[n].handle)
            for n in ("input_norm", "post_norm", "cache_k", "cache_v"):
                setattr(dst, n, b[n])
        desc = StepDesc(n_blocks=len(blocks), rms_eps=rms_eps, serving_dtype=serving_tag, kv_dtype=kv_tag,
                        blocks=arr, **dims)
        for n, _ in StepBuffers._fields_:
            setattr(desc.buf, n, buffers[n])
        h = ctypes.c_void_p()
        check(_lib.lib().qk_decode_step_create(ctx.handle, ctypes.byref(desc), ctypes.byref(h)))
        self._h = h

    def run(self) -> None:
        check(_lib.lib().qk_decode_step_run(self.ctx.handle, self._h))

    def trace(self, stamps_ptr: int | None, capacity: int = 0) -> None:
        """Later runs record the device timer at kernel start, after every grid barrier and at
        the end into ``capacity`` uint64 entries at ``stamps_ptr`` (None: off)."""
        check(_lib.lib().qk_decode_step_trace(self._h, ctypes.c_void_p(stamps_ptr or 0), capacity))

    def close(self) -> None:
        if getattr(self, "_h", None):
            _lib.lib().qk_decode_step_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class LayerPlan(LayerGroup):
    """Instances (layer, x pointer, y pointer) bound once; ``apply`` is two kernel launches
    (one when there are at least as many instances as SMs).  The layers may differ in shape
    while the plan is small (q beside k and v at a small batch).  With ``gated`` the instances
    are (layer, gate pointer, up pointer, y pointer) and the layer is applied to
    SwiGLU(gate, up)."""

    def __init__(self, ctx: GpuContext, instances, gated: bool = False):
        self.ctx = ctx
        self.layers = [i[0] for i in instances]
        n = len(instances)
        larr = (ctypes.c_void_p * n)(*[i[0].handle for i in instances])
        xarr = (ctypes.c_void_p * n)(*[ctypes.c_void_p(i[1]) for i in instances])
        yarr = (ctypes.c_void_p * n)(*[ctypes.c_void_p(i[-1]) for i in instances])
        h = ctypes.c_void_p()
        if gated:
            uarr = (ctypes.c_void_p * n)(*[ctypes.c_void_p(i[2]) for i in instances])
            check(_lib.lib().qk_plan_create_gated(ctx.handle, larr, xarr, uarr, yarr, n,
                                                  ctypes.byref(h)))
        else:
            check(_lib.lib().qk_plan_create(ctx.handle, larr, xarr, yarr, n, ctypes.byref(h)))
        self._h = h

    def set_norm(self, residuals, norm_weight: int, eps: float, x_outs) -> None:
        """Makes ``apply`` start with the RMSNorm of its input (``qk_plan_set_norm``): instance k
        reads its x pointer as the residual stream, adds ``residuals[k]`` (a device pointer or
        None) and applies its layer to the normed vector; where ``x_outs[k]`` is not None it
        also writes the updated stream there (one instance per token; never the input buffer).
        Raises KernelError, leaving the plan as it was, when the plan does not fit that form."""
        n = len(self.layers)
        rarr = (ctypes.c_void_p * n)(*[ctypes.c_void_p(r) for r in residuals])
        oarr = (ctypes.c_void_p * n)(*[ctypes.c_void_p(o) for o in x_outs])
        check(_lib.lib().qk_plan_set_norm(self.ctx.handle, self._h, rarr, ctypes.c_void_p(norm_weight),
                                          ctypes.c_float(eps), oarr))

    def set_allreduce(self, gather: bool, inbox_bases, rank: int, world: int, total_words: int, tokens,
                      d: int, state_ptr: int) -> None:
        """Tensor parallel (``qk_plan_set_allreduce``).  ``gather=False``: the plan's last stage
        pushes its outputs into the inboxes of all ranks (``inbox_bases``: one device address per
        rank) instead of storing them.  ``gather=True``: this normed plan takes the sum of what
        arrived in this rank's inbox (``inbox_bases[0]``) as the residual of its norm.
        ``tokens[k]``: the token instance k belongs to; ``total_words``: tokens x d words per
        source rank; ``state_ptr``: the two uint32 the process's all-reduces share."""
        n = len(self.layers)
        bases = np.ascontiguousarray(inbox_bases, dtype=np.uint64)
        toks = np.ascontiguousarray(tokens, dtype=np.uint32)
        assert toks.size == n
        check(_lib.lib().qk_plan_set_allreduce(self.ctx.handle, self._h, 1 if gather else 0, bases.ctypes.data,
                                               int(rank), int(world), int(total_words), toks.ctypes.data,
                                               int(d), ctypes.c_void_p(state_ptr)))

    def feed_targets(self):
        """Turns the plan into a fed plan (the digit tables of its stage-1 inputs are then
        written by the ``*_feed`` call that produces those inputs, and every ``apply`` must follow
        such a call) and returns (device pointer to the per-instance targets, their number)."""
        ptr, n = ctypes.c_void_p(), ctypes.c_size_t()
        check(_lib.lib().qk_plan_feed_targets(self.ctx.handle, self._h, ctypes.byref(ptr),
                                              ctypes.byref(n)))
        return ptr.value, n.value


__all__ = ["apply_noalloc", "DecodeStep", "Feed", "make_feed", "LayerPlan", "LayerGroup", "HostLayerGroup", "GpuContext", "AttentionShape", "PackedLayer", "apply_group", "gpu_available",
           "gpu_init_hint", "GPU_INDEX_CEILING", "KernelError", "DeviceError"]
