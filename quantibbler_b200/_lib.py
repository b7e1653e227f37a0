"""ctypes binding of libqk_kernels.so (the C ABI declared in include/qk_kernels.h).

The library is the product; this module only loads it and maps status codes to
exceptions.  There is no fallback: if the shared library is missing the import of any
product function fails with an error that says how to build it.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_double, c_float, c_int32, c_size_t, c_uint64, c_void_p

from . import _build

QK_OK, QK_ERR_VALUE, QK_ERR_INIT, QK_ERR_CUDA, QK_ERR_TIMEOUT, QK_ERR_ALLOC = range(6)
QK_F64, QK_F32, QK_BF16 = 0, 1, 2
DTYPE_TAGS = {"float64": QK_F64, "float32": QK_F32, "bfloat16": QK_BF16}


class KernelError(ValueError):
    """The reference's ``KernelError`` (crates/quantibbler-kernels/src/core.rs:31-44).

    It subclasses ``ValueError`` because that is what the reference's Python face raises
    for it (crates/quantibbler-kernels/src/lib.rs:34-36).
    """


class DeviceError(RuntimeError):
    """A CUDA failure or the absence of a usable device (no CPU fallback exists)."""


_SIGNATURES = {
    "qk_last_error": (c_char_p, []),
    "qk_backend_version": (c_char_p, []),
    "qk_gpu_init_hint": (c_char_p, []),
    "qk_pack_bits": (c_int32, [c_void_p, c_size_t, c_size_t, c_size_t, c_void_p, c_size_t]),
    "qk_pack_bits_f64": (c_int32, [c_void_p, c_size_t, c_size_t, c_size_t, c_void_p, c_size_t]),
    "qk_unpack_bits": (c_int32, [c_void_p, c_size_t, c_size_t, c_size_t, c_void_p, c_size_t]),
    "qk_sign_estimate": (c_int32, [c_void_p, c_size_t, c_void_p]),
    "qk_joint_itq": (c_int32, [c_void_p, c_size_t, c_void_p, c_size_t, c_size_t, c_size_t, c_size_t,
                               c_size_t, c_double, c_uint64, c_void_p, c_void_p,
                               POINTER(c_size_t), POINTER(c_int32)]),
    "qk_validate_packed": (c_int32, [c_size_t, c_size_t, c_size_t, POINTER(c_size_t)]),
    "qk_dtype_from_name": (c_int32, [c_char_p, POINTER(c_int32)]),
    "qk_dtype_name": (c_char_p, [c_int32]),
    "qk_container_to_rows": (c_int32, [c_void_p, c_size_t, c_size_t, c_size_t, c_void_p, c_size_t]),
    "qk_container_to_rows_transposed": (c_int32, [c_void_p, c_size_t, c_size_t, c_size_t, c_void_p,
                                                  c_size_t]),
    "qk_gpu_available": (c_int32, []),
    "qk_gpu_init_at": (c_int32, [c_size_t, POINTER(c_void_p)]),
    "qk_gpu_init": (c_int32, [POINTER(c_void_p)]),
    "qk_gpu_free": (None, [c_void_p]),
    "qk_gpu_synchronize": (c_int32, [c_void_p]),
    "qk_gpu_stream": (c_void_p, [c_void_p]),
    "qk_gpu_set_stream": (c_int32, [c_void_p, c_void_p]),
    "qk_gpu_packed_matvec": (c_int32, [c_void_p, c_void_p, c_size_t, c_size_t, c_size_t, c_void_p,
                                       c_size_t, c_void_p]),
    "qk_packed_matvec": (c_int32, [c_void_p, c_void_p, c_size_t, c_size_t, c_size_t, c_int32,
                                   c_void_p, c_size_t, c_void_p]),
    "qk_packed_matmul": (c_int32, [c_void_p, c_void_p, c_size_t, c_size_t, c_size_t, c_int32,
                                   c_void_p, c_size_t, c_size_t, c_void_p, c_size_t]),
    "qk_gpu_attention": (c_int32, [c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_size_t,
                                   c_void_p, c_size_t, c_int32, c_void_p, c_size_t]),
    "qk_gpu_attention_sage": (c_int32, [c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_size_t,
                                        c_void_p, c_size_t, c_int32, c_size_t, c_void_p, c_size_t]),
    "qk_layer_create": (c_int32, [c_void_p, c_void_p, c_size_t, c_void_p, c_size_t, c_size_t,
                                  c_size_t, c_size_t, c_void_p, c_void_p, c_void_p, c_int32,
                                  POINTER(c_void_p)]),
    "qk_layer_free": (None, [c_void_p]),
    "qk_layer_apply": (c_int32, [c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "qk_layer_apply_prefill": (c_int32, [c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "qk_layers_apply_prefill": (c_int32, [c_void_p, c_void_p, c_size_t, c_void_p, c_size_t, c_void_p]),
    "qk_prefill_work_split": (c_int32, [c_size_t, c_void_p, c_void_p, c_size_t, c_void_p, c_size_t, c_void_p]),
    "qk_layers_apply_prefill_gated": (c_int32, [c_void_p, c_void_p, c_size_t, c_void_p, c_void_p, c_size_t,
                                                c_void_p]),
    "qk_layer_apply_noalloc": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p]),
    "qk_layer_apply_host": (c_int32, [c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_size_t]),
    "qk_layers_apply_group": (c_int32, [c_void_p, POINTER(c_void_p), c_size_t, c_void_p, c_void_p]),
    "qk_group_create": (c_int32, [c_void_p, POINTER(c_void_p), c_size_t, c_void_p, c_void_p,
                                  POINTER(c_void_p)]),
    "qk_plan_create": (c_int32, [c_void_p, POINTER(c_void_p), POINTER(c_void_p), POINTER(c_void_p),
                                 c_size_t, POINTER(c_void_p)]),
    "qk_plan_create_gated": (c_int32, [c_void_p, POINTER(c_void_p), POINTER(c_void_p),
                                       POINTER(c_void_p), POINTER(c_void_p), c_size_t,
                                       POINTER(c_void_p)]),
    "qk_plan_set_norm": (c_int32, [c_void_p, c_void_p, POINTER(c_void_p), c_void_p, ctypes.c_float,
                                   POINTER(c_void_p)]),
    "qk_plan_set_allreduce": (c_int32, [c_void_p, c_void_p, c_int32, c_void_p, c_int32, c_int32, c_size_t,
                                        c_void_p, c_size_t, c_void_p]),
    "qk_group_apply": (c_int32, [c_void_p, c_void_p]),
    "qk_plan_feed_targets": (c_int32, [c_void_p, c_void_p, POINTER(c_void_p), POINTER(c_size_t)]),
    "qk_decode_attention_rope_scratch": (c_size_t, [c_size_t, c_size_t, c_size_t, c_size_t, c_size_t]),
    "qk_decode_attention_rope": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_void_p, c_int32, c_void_p, c_size_t, c_size_t, c_size_t,
                                           c_size_t, c_size_t, c_size_t, c_size_t, c_void_p, c_void_p]),
    "qk_groups_apply_host": (c_int32, [c_void_p, POINTER(c_void_p), POINTER(c_size_t), c_size_t, c_void_p,
                                       c_void_p, c_void_p, c_void_p, c_size_t, c_size_t]),
    "qk_decode_step_create": (c_int32, [c_void_p, c_void_p, POINTER(c_void_p)]),
    "qk_decode_step_run": (c_int32, [c_void_p, c_void_p]),
    "qk_decode_step_free": (None, [c_void_p]),
    "qk_decode_step_trace": (c_int32, [c_void_p, c_void_p, c_size_t]),
    "qk_rmsnorm_feed": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_size_t, c_float,
                                  c_int32, c_void_p, c_void_p, c_void_p]),
    "qk_allreduce_rmsnorm_feed": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32,
                                            c_void_p, c_void_p, c_size_t, c_size_t, c_float, c_int32,
                                            c_void_p, c_void_p, c_void_p]),
    "qk_decode_attention_feed": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_void_p,
                                           c_size_t, c_size_t, c_size_t, c_size_t, c_size_t, c_size_t,
                                           c_void_p, c_void_p, c_int32, c_void_p]),
    "qk_swiglu_feed": (c_int32, [c_void_p, c_void_p, c_void_p, c_size_t, c_size_t, c_int32, c_void_p]),
    "qk_group_free": (None, [c_void_p]),
    "qk_rmsnorm": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_size_t, c_float,
                             c_int32, c_void_p, c_void_p]),
    "qk_rope_cache": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_void_p, c_int32, c_size_t, c_size_t,
                                c_size_t, c_size_t, c_size_t, c_size_t]),
    "qk_decode_attention_scratch": (c_size_t, [c_size_t, c_size_t, c_size_t, c_size_t]),
    "qk_decode_attention": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_void_p,
                                      c_size_t, c_size_t, c_size_t, c_size_t, c_size_t, c_size_t,
                                      c_void_p, c_void_p]),
    "qk_prefill_attention": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_size_t,
                                       c_size_t, c_size_t, c_size_t, c_size_t, c_size_t, c_size_t,
                                       c_void_p]),
    "qk_swiglu": (c_int32, [c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "qk_add": (c_int32, [c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "qk_embed": (c_int32, [c_void_p, c_void_p, c_int32, c_void_p, c_size_t, c_size_t, c_size_t,
                           c_void_p]),
    "qk_lm_head": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_size_t, c_size_t, c_size_t,
                             c_size_t, c_void_p]),
    "qk_argmax_first": (c_int32, [c_void_p, c_void_p, c_size_t, c_size_t, c_size_t, c_int32,
                                  c_void_p, c_void_p]),
    "qk_set_gemv_kernel": (c_int32, [c_void_p, c_int32]),
    "qk_qpk1_parse": (c_int32, [c_void_p, c_size_t, c_void_p]),
    "qk_qpk1_scales": (c_int32, [c_void_p, c_size_t, c_void_p, c_void_p, c_void_p]),
    "qk_layer_create_from_streams": (c_int32, [c_void_p, c_void_p, c_size_t, c_void_p, c_size_t,
                                               c_size_t, c_size_t, c_size_t, c_void_p, c_void_p,
                                               c_void_p, c_int32, POINTER(c_void_p)]),
    "qk_gpu_container_to_rows": (c_int32, [c_void_p, c_void_p, c_size_t, c_size_t, c_size_t,
                                           c_int32, c_void_p, c_size_t]),
    "qk_layer_from_qpk1": (c_int32, [c_void_p, c_void_p, c_size_t, c_int32, c_void_p]),
    "qk_set_sage_kernel": (c_int32, [c_void_p, c_int32]),
    "qk_allreduce_rmsnorm": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_void_p,
                                       c_void_p, c_size_t, c_size_t, c_float, c_int32, c_void_p, c_void_p]),
    "qk_set_decode_attention_kernel": (c_int32, [c_void_p, c_int32]),
    "qk_gpu_attention_dev": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32,
                                       c_void_p]),
    "qk_gpu_attention_sage_dev": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                            c_int32, c_size_t, c_void_p]),
    "qk_gpu_attention_sage_block_dev": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32,
                                                  c_void_p]),
    "qk_gpu_launch_count": (c_uint64, [c_void_p]),
    "qk_gpu_sage_quantize": (c_int32, [c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_size_t,
                                       c_void_p, c_size_t, c_size_t, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_void_p, c_void_p]),
    "qk_set_wait_limit": (ctypes.c_uint32, [c_void_p, ctypes.c_uint32]),
    "qk_set_dependent_launch": (c_int32, [c_void_p, c_int32]),
}

_lib = None


def exported_symbols() -> list[str]:
    """Every entry point include/qk_kernels.h declares."""
    return sorted(_SIGNATURES)


def lib() -> ctypes.CDLL:
    """Load the shared library, rebuilding it first when a source is newer than it (the build
    is incremental); a stale library that cannot be rebuilt is refused, not loaded."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB_PATH
    try:
        # incremental by modification time: a no-op when the library is newer than its sources
        _build.build()
    except Exception as exc:  # no nvcc, or a compile error
        if not os.path.exists(path):
            raise ImportError(
                f"libqk_kernels.so is not built ({path}); run `python -m quantibbler_b200._build` "
                f"on a machine with nvcc. There is no CPU fallback. Cause: {exc}") from exc
        if _build.stale():
            raise ImportError(
                f"{path} is older than its sources and could not be rebuilt: {exc}") from exc
    handle = ctypes.CDLL(path)
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(handle, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = handle
    return _lib


def last_error() -> str:
    return lib().qk_last_error().decode("utf-8", "replace")


def check(status: int) -> None:
    """Raise the exception that a non-zero status stands for."""
    if status == QK_OK:
        return
    msg = last_error()
    if status == QK_ERR_VALUE:
        raise KernelError(msg)
    raise DeviceError(msg)
