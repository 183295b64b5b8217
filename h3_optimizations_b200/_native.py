"""ctypes binding of ``libh3sparse.so`` (the C ABI declared in include/h3sparse.h).

There is no fallback: if the library is missing or an entry point returns a
non-zero status, a ``NativeError`` is raised.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libh3sparse.so"

H3S_F32, H3S_BF16, H3S_F16, H3S_F64 = 0, 1, 2, 3
DTYPE_CODES = {
    torch.float32: H3S_F32,
    torch.bfloat16: H3S_BF16,
    torch.float16: H3S_F16,
    torch.float64: H3S_F64,
}

ABI_VERSION = 1


class QKVCarriers(ctypes.Structure):
    """``h3s_qkv_carriers`` of include/h3sparse.h."""

    _fields_ = [
        ("q8", c_void_p), ("q_scale", c_void_p), ("q_summary", c_void_p),
        ("k8", c_void_p), ("k_scale", c_void_p), ("k_summary", c_void_p),
        ("k_stage", c_void_p), ("v_stage", c_void_p), ("stats", c_void_p),
        ("summary_dtype", c_int), ("sequence_total", c_int), ("row_start", c_int),
    ]


class NativeError(RuntimeError):
    """The native library is missing, mismatched, or a call failed."""

    def __init__(self, message, code=None):
        super().__init__(message)
        self.code = code


# name -> (restype, argtypes); mirrors include/h3sparse.h one to one
PROTOTYPES = {
    "h3s_abi_version": (c_int, []),
    "h3s_last_error": (c_char_p, []),
    "h3s_device_capability": (c_int, []),
    "h3s_set_wait_budget_ns": (c_int, [ctypes.c_ulonglong]),
    "h3s_get_wait_budget_ns": (ctypes.c_ulonglong, []),
    "h3s_column_stats_scratch_bytes": (c_size_t, [c_int]),
    "h3s_column_stats": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int, c_int,
                                 c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p]),
    "h3s_column_stats_static": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int, c_int,
                                        c_int, c_float, c_void_p, c_void_p, c_void_p]),
    "h3s_quant_qk_blocks": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "h3s_quant_v_fp8": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p, c_int, c_int,
                                c_int, c_int, c_float, c_void_p]),
    "h3s_convrot_quant_rows": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "h3s_qkv_gemm_chunk": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                   c_int64, c_void_p, c_void_p]),
    "h3s_qkv_gemm_chunk_norm_rope": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                             c_void_p, c_int64, c_void_p, c_void_p, c_float, c_void_p, c_int,
                                             c_void_p, c_void_p, c_void_p]),
    "h3s_qkv_gemm_chunk_carriers": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                            ctypes.POINTER(QKVCarriers), c_void_p, c_void_p, c_float, c_void_p,
                                            c_int, c_void_p, c_void_p, c_void_p]),
    "h3s_dense_gemm": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                               c_void_p, c_int, c_void_p, c_int64, c_void_p, c_void_p]),
    "h3s_quant_rows_fp8": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "h3s_column_stats_finalize": (c_int, [c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p]),
    "h3s_route_topk": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                               c_int, c_int, c_void_p, c_void_p]),
    "h3s_route_to_delta_lut": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                       c_void_p, c_void_p]),
    "h3s_sparse_attn_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int64, c_int64,
                                    c_int, c_int, c_int, c_void_p, c_void_p]),
    "h3s_sparse_attn_fwd_scatter": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                            c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int,
                                            c_int64, c_int64, c_int, c_int, c_int, c_void_p, c_void_p]),
    "h3s_sparse_attn_fwd_mma": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int64,
                                        c_int64, c_int, c_int, c_int, c_void_p]),
}

_lib = None


def load(path=None):
    """Load the shared library and bind every prototype (idempotent)."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    target = Path(path) if path is not None else LIB_PATH
    if not target.exists():
        raise NativeError(
            "native library %s is missing: build it with `python -m h3_optimizations_b200.build` "
            "(there is no CPU fallback)" % target
        )
    lib = ctypes.CDLL(str(target))
    for name, (restype, argtypes) in PROTOTYPES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise NativeError("native library %s does not export %s" % (target, name)) from exc
        fn.restype = restype
        fn.argtypes = argtypes
    version = lib.h3s_abi_version()
    if version != ABI_VERSION:
        raise NativeError("native library ABI %d does not match the binding's %d" % (version, ABI_VERSION))
    if path is None:
        _lib = lib
    return lib


def check(status, what):
    if status != 0:
        message = load().h3s_last_error().decode("utf-8", "replace")
        raise NativeError("%s failed (%d): %s" % (what, status, message), code=status)


def ptr(tensor):
    return None if tensor is None else c_void_p(tensor.data_ptr())


def stream_ptr(device=None):
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def dtype_code(dtype):
    try:
        return DTYPE_CODES[dtype]
    except KeyError:
        raise NativeError("unsupported element type %s" % dtype) from None
