"""ctypes binding of libgca_b200.so (the C ABI declared in include/gca_b200.h).

The library is built in-tree by ``long_context_modeling_b200.build``.  There is no
fallback of any kind: if the shared object is missing, or a call is rejected, an
exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
# GCA_B200_LIB names another build of the same library (a profiling build, or the test build
# whose forward withholds a copy so that a bounded wait expires); default: the in-tree build.
LIB_PATH = os.environ.get("GCA_B200_LIB") or os.path.join(_HERE, "libgca_b200.so")

BF16, F32 = 0, 1
ALGO_AUTO, ALGO_SIMT, ALGO_TC, ALGO_TC_UNPAIRED = 0, 1, 2, 3
ABI_VERSION = 2
STATUS_BAD_INDEX, STATUS_TIMEOUT = 1, 2

_i64x4 = C.c_int64 * 4


class GcaFwdArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
        ("indices", C.c_void_p), ("weights", C.c_void_p), ("out", C.c_void_p),
        ("lse", C.c_void_p), ("status", C.c_void_p),
        ("q_stride", _i64x4), ("o_stride", _i64x4), ("k_stride", _i64x4), ("v_stride", _i64x4),
        ("N", C.c_int32), ("J", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("S", C.c_int32),
        ("L", C.c_int32), ("D", C.c_int32), ("K", C.c_int32), ("C", C.c_int32),
        ("dtype", C.c_int32), ("algo", C.c_int32), ("sm_scale", C.c_float), ("off_by_one", C.c_float),
    ]


class GcaBwdArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
        ("indices", C.c_void_p), ("weights", C.c_void_p), ("dout", C.c_void_p), ("lse", C.c_void_p),
        ("dq", C.c_void_p), ("dk_cache", C.c_void_p), ("dv_cache", C.c_void_p), ("dw", C.c_void_p),
        ("workspace", C.c_void_p), ("status", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("q_stride", _i64x4), ("do_stride", _i64x4), ("dq_stride", _i64x4),
        ("k_stride", _i64x4), ("v_stride", _i64x4), ("dk_stride", _i64x4), ("dv_stride", _i64x4),
        ("N", C.c_int32), ("J", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("S", C.c_int32),
        ("L", C.c_int32), ("D", C.c_int32), ("K", C.c_int32), ("C", C.c_int32),
        ("dtype", C.c_int32), ("algo", C.c_int32), ("sm_scale", C.c_float), ("off_by_one", C.c_float),
    ]


class LmkTopkArgs(C.Structure):
    _fields_ = [
        ("lmk_q", C.c_void_p), ("lmk_k", C.c_void_p), ("noise", C.c_void_p),
        ("out_keys", C.c_void_p), ("out_indices", C.c_void_p), ("out_scores", C.c_void_p),
        ("out_weights", C.c_void_p), ("out_nvalid", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("q_batch_stride", C.c_int64), ("q_row_stride", C.c_int64),
        ("k_batch_stride", C.c_int64), ("k_row_stride", C.c_int64),
        ("q_pos0", C.c_int64), ("e_base", C.c_int64),
        ("N", C.c_int32), ("Cq", C.c_int32), ("E", C.c_int32), ("D", C.c_int32), ("K", C.c_int32),
        ("head_dim", C.c_int32), ("score_round", C.c_int32), ("splits", C.c_int32),
    ]


class LmkMergeArgs(C.Structure):
    _fields_ = [
        ("keys", C.c_void_p), ("out_keys", C.c_void_p), ("out_indices", C.c_void_p),
        ("out_scores", C.c_void_p), ("out_weights", C.c_void_p), ("out_nvalid", C.c_void_p),
        ("R", C.c_int32), ("P", C.c_int32), ("K", C.c_int32),
    ]


class CacheAppendArgs(C.Structure):
    _fields_ = [
        ("new_k", C.c_void_p), ("new_v", C.c_void_p), ("new_lmk", C.c_void_p),
        ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("lmk_cache", C.c_void_p),
        ("new_batch_stride", C.c_int64), ("cache_batch_stride", C.c_int64),
        ("new_lmk_batch_stride", C.c_int64), ("lmk_cache_batch_stride", C.c_int64),
        ("N", C.c_int32), ("count", C.c_int32), ("pos", C.c_int32), ("L", C.c_int32),
        ("HD", C.c_int32), ("Dm", C.c_int32), ("dtype", C.c_int32), ("zero_landmark", C.c_int32),
        ("capacity", C.c_int32), ("lmk_capacity", C.c_int32),
    ]


class LmkExchangeArgs(C.Structure):
    _fields_ = [
        ("local_keys", C.c_void_p), ("mailboxes", C.c_void_p),
        ("out_keys", C.c_void_p), ("out_indices", C.c_void_p), ("out_scores", C.c_void_p),
        ("out_weights", C.c_void_p), ("out_nvalid", C.c_void_p), ("status", C.c_void_p),
        ("R", C.c_int32), ("K", C.c_int32), ("world", C.c_int32), ("rank", C.c_int32),
        ("R_max", C.c_int32), ("wait_ms", C.c_int32),
    ]


class KvProjectArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("wk", C.c_void_p), ("wv", C.c_void_p),
        ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("lmk_cache", C.c_void_p), ("status", C.c_void_p),
        ("cache_batch_stride", C.c_int64), ("lmk_cache_batch_stride", C.c_int64),
        ("N", C.c_int32), ("count", C.c_int32), ("pos", C.c_int32), ("D", C.c_int32),
        ("capacity", C.c_int32), ("lmk_capacity", C.c_int32), ("zero_landmark", C.c_int32),
    ]


class RowRmsArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("row_scale", C.c_void_p), ("M", C.c_int64), ("x_stride", C.c_int64),
                ("D", C.c_int32), ("eps", C.c_float)]


class LinearArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("w", C.c_void_p), ("out", C.c_void_p), ("residual", C.c_void_p), ("row_scale", C.c_void_p),
        ("status", C.c_void_p), ("M", C.c_int64),
        ("x_stride", C.c_int64), ("w_stride", C.c_int64), ("out_stride", C.c_int64), ("residual_stride", C.c_int64),
        ("N", C.c_int32), ("K", C.c_int32),
    ]


class WindowDecodeArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("alibi_slopes", C.c_void_p), ("out", C.c_void_p),
        ("q_stride", C.c_int64 * 3), ("o_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3), ("v_stride", C.c_int64 * 3),
        ("N", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("Sq", C.c_int32), ("T", C.c_int32), ("window", C.c_int32),
        ("sm_scale", C.c_float),
    ]


class WindowRingDecodeArgs(C.Structure):
    _fields_ = [("attn", WindowDecodeArgs), ("k_new", C.c_void_p), ("v_new", C.c_void_p), ("rows_written", C.c_void_p),
                ("new_stride", C.c_int64 * 2)]


class LinearCeArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("w", C.c_void_p), ("targets", C.c_void_p), ("row_scale", C.c_void_p), ("loss", C.c_void_p),
        ("lse", C.c_void_p), ("workspace", C.c_void_p), ("status", C.c_void_p), ("M", C.c_int64),
        ("x_stride", C.c_int64), ("w_stride", C.c_int64), ("workspace_bytes", C.c_int64), ("N", C.c_int32), ("K", C.c_int32),
    ]


class WindowAppendArgs(C.Structure):
    _fields_ = [("k_window", C.c_void_p), ("v_window", C.c_void_p), ("k_new", C.c_void_p), ("v_new", C.c_void_p),
                ("window_stride", C.c_int64 * 2), ("new_stride", C.c_int64 * 2), ("N", C.c_int32), ("H", C.c_int32), ("T", C.c_int32)]

EXPORTS = {
    "gca_fwd": (C.c_int, [C.POINTER(GcaFwdArgs), C.c_void_p]),
    "gca_decode": (C.c_int, [C.POINTER(GcaFwdArgs), C.c_void_p]),
    "gca_bwd": (C.c_int, [C.POINTER(GcaBwdArgs), C.c_void_p]),
    "gca_bwd_workspace_bytes": (C.c_size_t, [C.POINTER(GcaBwdArgs)]),
    "gca_bwd_stages": (C.c_int, [C.POINTER(GcaBwdArgs), C.c_uint, C.c_void_p]),
    "lmk_score_topk": (C.c_int, [C.POINTER(LmkTopkArgs), C.c_void_p]),
    "lmk_topk_workspace_bytes": (C.c_size_t, [C.POINTER(LmkTopkArgs)]),
    "lmk_score_topk_static": (C.c_int, [C.POINTER(LmkTopkArgs), C.c_void_p]),
    "lmk_topk_merge": (C.c_int, [C.POINTER(LmkMergeArgs), C.c_void_p]),
    "gca_cache_append": (C.c_int, [C.POINTER(CacheAppendArgs), C.c_void_p]),
    "gca_kv_project_append": (C.c_int, [C.POINTER(KvProjectArgs), C.c_void_p]),
    "gca_row_rms": (C.c_int, [C.POINTER(RowRmsArgs), C.c_void_p]),
    "gca_linear": (C.c_int, [C.POINTER(LinearArgs), C.c_void_p]),
    "gca_silu_mul": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int64, C.c_int64, C.c_void_p]),
    "gca_window_decode": (C.c_int, [C.POINTER(WindowDecodeArgs), C.c_void_p]),
    "gca_window_shift_append": (C.c_int, [C.POINTER(WindowAppendArgs), C.c_void_p]),
    "gca_window_ring_decode": (C.c_int, [C.POINTER(WindowRingDecodeArgs), C.c_void_p]),
    "gca_linear_ce_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int32]),
    "gca_linear_cross_entropy": (C.c_int, [C.POINTER(LinearCeArgs), C.c_void_p]),
    "lmk_exchange_mailbox_bytes": (C.c_size_t, [C.c_int, C.c_int]),
    "lmk_exchange_mailbox_create": (C.c_int, [C.c_int, C.c_int, C.POINTER(C.c_void_p), C.c_void_p]),
    "lmk_exchange_mailbox_open": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "lmk_exchange_mailbox_close": (C.c_int, [C.c_void_p]),
    "lmk_exchange_mailbox_destroy": (C.c_int, [C.c_void_p]),
    "lmk_exchange_mailbox_reset": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "lmk_topk_exchange": (C.c_int, [C.POINTER(LmkExchangeArgs), C.c_void_p]),
    "gca_vmem_granularity": (C.c_size_t, [C.c_int]),
    "gca_vmem_reserve": (C.c_int, [C.c_size_t, C.c_size_t, C.POINTER(C.c_void_p)]),
    "gca_vmem_map": (C.c_int, [C.c_void_p, C.c_size_t, C.c_int, C.POINTER(C.c_ulonglong)]),
    "gca_vmem_unmap": (C.c_int, [C.c_void_p, C.c_size_t, C.c_ulonglong]),
    "gca_vmem_free": (C.c_int, [C.c_void_p, C.c_size_t]),
    "gca_strerror": (C.c_char_p, [C.c_int]),
    "gca_abi_version": (C.c_int, []),
    "gca_sizeof": (C.c_size_t, [C.c_int]),
}

_lib: Optional[C.CDLL] = None


def lib() -> C.CDLL:
    """Load the shared library once.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m long_context_modeling_b200.build` "
                "(there is no fallback path)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, argtypes) in EXPORTS.items():
            fn = getattr(handle, name)          # AttributeError if a symbol is missing
            fn.restype = res
            fn.argtypes = argtypes
        if handle.gca_abi_version() != ABI_VERSION:
            raise RuntimeError("libgca_b200.so has an unexpected ABI version")
        for which, struct in enumerate((GcaFwdArgs, GcaBwdArgs, LmkTopkArgs, LmkMergeArgs, CacheAppendArgs, LmkExchangeArgs,
                                       KvProjectArgs, RowRmsArgs, LinearArgs, WindowDecodeArgs, LinearCeArgs, WindowAppendArgs,
                                       WindowRingDecodeArgs)):
            if handle.gca_sizeof(which) != C.sizeof(struct):
                raise RuntimeError(f"struct layout mismatch for {struct.__name__}: "
                                   f"library {handle.gca_sizeof(which)} vs binding {C.sizeof(struct)}")
        _lib = handle
    return _lib


class GcaError(RuntimeError):
    pass


_nvtx = False


def set_nvtx(enabled: bool) -> None:
    """Wrap every call into the library in an NVTX range named after the entry point (for timelines of
    a host program; off by default)."""
    global _nvtx
    _nvtx = bool(enabled)


def call(name: str, *args) -> None:
    """``check(lib().<name>(*args), name)`` with the optional NVTX range around the launch."""
    fn = getattr(lib(), name)
    if _nvtx:
        import torch
        torch.cuda.nvtx.range_push(name)
        try:
            code = fn(*args)
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        code = fn(*args)
    check(code, name)


def check(code: int, what: str) -> None:
    """0 -> ok; negative -> ValueError (argument rejected); positive -> CUDA runtime error."""
    if code == 0:
        return
    msg = lib().gca_strerror(code).decode()
    if code < 0:
        raise ValueError(f"{what}: {msg} (code {code})")
    raise GcaError(f"{what}: CUDA error {code}: {msg}")


def strides4(*vals) -> "_i64x4":
    return _i64x4(*[int(v) for v in vals])
