"""ctypes binding of ``libh3attn.so`` (the C ABI declared in ``include/h3attn.h``).

There is no fallback: if the shared library is missing or a call returns a non-zero status the
binding raises.  Build the library with ``python -m pika_h3_flex_b200.build``.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
# H3A_LIBRARY names another build of the library (for example one compiled with different tuning macros)
LIB_PATH = os.environ.get("H3A_LIBRARY") or os.path.join(_HERE, "libh3attn.so")

# status codes / enums (mirror include/h3attn.h)
H3A_OK = 0
H3A_ERR_ARG, H3A_ERR_ALIGN, H3A_ERR_SHAPE, H3A_ERR_ARCH = -1, -2, -3, -4
H3A_ERR_LAUNCH, H3A_ERR_TIMEOUT, H3A_ERR_WORKSPACE, H3A_ERR_DRIVER = -5, -6, -7, -8
H3A_ERR_STATIC_SCRATCH = -9
H3A_ERR_INDEX = -10
H3A_ERR_BOUND = -11
MODE_DENSE_BF16, MODE_FP8_QK, MODE_BLOCK_SPARSE = 0, 1, 2
ROPE_INTERLEAVED, ROPE_HALF = 0, 1
PREP_FP8 = 1
PREP_NO_NORM = 2
KERNEL_CTA_PAIRS, KERNEL_FIXED_REFERENCE, KERNEL_SPLIT_LAST_WAVE, KERNEL_ONLINE_TWO_LAUNCH, KERNEL_PERSISTENT = 1, 2, 4, 8, 16
MAX_RANKS = 8
PEER_HANDLE_BYTES = 64

EXPORTS = (
    "h3a_version",
    "h3a_status_string",
    "h3a_attn_workspace_bytes",
    "h3a_attn_fwd",
    "h3a_qk_prep",
    "h3a_rope_table",
    "h3a_build_block_index",
    "h3a_read_device_status",
    "h3a_attn_fwd_sparse_static",
    "h3a_static_scratch_capacity",
    "h3a_memcpy2d_async",
    "h3a_selftest_wait_timeout",
    "h3a_proj_fwd",
    "h3a_adaln_norm",
    "h3a_qk_prep_scatter",
    "h3a_attn_kernel_choice",
    "h3a_peer_alloc",
    "h3a_peer_open",
    "h3a_peer_close",
    "h3a_peer_free",
)


class AttnParams(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p),
        ("q_stride_l", C.c_int64), ("q_stride_h", C.c_int64),
        ("k_stride_l", C.c_int64), ("k_stride_h", C.c_int64),
        ("v_stride_l", C.c_int64), ("v_stride_h", C.c_int64),
        ("o_stride_l", C.c_int64), ("o_stride_h", C.c_int64),
        ("Lq", C.c_int32), ("Lk", C.c_int32), ("H", C.c_int32), ("d", C.c_int32),
        ("B", C.c_int32), ("mode", C.c_int32), ("softmax_scale", C.c_float),
        ("q_scale", C.c_void_p), ("k_scale", C.c_void_p),
        ("row_ptr", C.c_void_p), ("col_idx", C.c_void_p), ("nnz", C.c_int32),
        ("lse", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("status_word", C.c_void_p), ("wait_limit_ns", C.c_int64), ("logit_bound", C.c_float), ("sparse_heavy_pairs", C.c_int32),
        ("o_rank_base", C.c_void_p * MAX_RANKS), ("o_n_ranks", C.c_int32), ("o_rank_rows", C.c_int32),
    ]


class HeadScatter(C.Structure):
    _fields_ = [
        ("base", C.c_void_p * MAX_RANKS), ("n_ranks", C.c_int32), ("heads_per_rank", C.c_int32), ("round_robin", C.c_int32),
        ("head0", C.c_int32), ("row_offset", C.c_int32), ("L_total", C.c_int32), ("start_head", C.c_int32),
    ]


class PrepParams(C.Structure):
    _fields_ = [
        ("q_in", C.c_void_p), ("k_in", C.c_void_p), ("q_out", C.c_void_p), ("k_out", C.c_void_p),
        ("q_scale", C.c_void_p), ("k_scale", C.c_void_p),
        ("q_stride_l", C.c_int64), ("q_stride_h", C.c_int64), ("k_stride_l", C.c_int64), ("k_stride_h", C.c_int64),
        ("Lq", C.c_int32), ("Lk", C.c_int32), ("H", C.c_int32), ("d", C.c_int32),
        ("q_rope", C.c_void_p), ("k_rope", C.c_void_p), ("q_weight", C.c_void_p), ("k_weight", C.c_void_p),
        ("eps", C.c_float), ("rope_mode", C.c_int32), ("flags", C.c_uint32),
    ]


class ProjParams(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("w", C.c_void_p), ("lora_t", C.c_void_p), ("lora_bs", C.c_void_p),
        ("bias", C.c_void_p), ("rope", C.c_void_p), ("norm_weight", C.c_void_p), ("out", C.c_void_p), ("out_scale", C.c_void_p),
        ("x_stride_l", C.c_int64), ("w_stride_n", C.c_int64), ("lora_t_stride_l", C.c_int64), ("lora_bs_stride_n", C.c_int64),
        ("out_stride_l", C.c_int64), ("out_stride_h", C.c_int64),
        ("L", C.c_int32), ("K", C.c_int32), ("N", C.c_int32), ("R", C.c_int32),
        ("epilogue", C.c_int32), ("rope_mode", C.c_int32), ("eps", C.c_float),
        ("status_word", C.c_void_p), ("wait_limit_ns", C.c_int64), ("out_to", C.c_void_p),
    ]


PROJ_STORE, PROJ_PREP, PROJ_PREP_FP8 = 0, 1, 2


class AdaLnParams(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("y", C.c_void_p), ("scale", C.c_void_p), ("shift", C.c_void_p),
        ("idx", C.c_void_p), ("weight", C.c_void_p), ("bias", C.c_void_p),
        ("x_stride", C.c_int64), ("y_stride", C.c_int64), ("scale_stride", C.c_int64), ("shift_stride", C.c_int64),
        ("L", C.c_int32), ("D", C.c_int32), ("T", C.c_int32), ("rms", C.c_int32), ("eps", C.c_float),
    ]


class H3AError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: {status_string(status)} (status {status})")


_lib: Optional[C.CDLL] = None


def load() -> C.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} not found: the CUDA library is required (no CPU fallback). "
            "Build it with `python -m pika_h3_flex_b200.build`."
        )
    lib = C.CDLL(LIB_PATH)
    lib.h3a_version.argtypes = [C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    lib.h3a_version.restype = C.c_int32
    lib.h3a_status_string.argtypes = [C.c_int32]
    lib.h3a_status_string.restype = C.c_char_p
    lib.h3a_attn_workspace_bytes.argtypes = [C.POINTER(AttnParams), C.POINTER(C.c_size_t)]
    lib.h3a_attn_workspace_bytes.restype = C.c_int32
    lib.h3a_attn_fwd.argtypes = [C.POINTER(AttnParams), C.c_void_p]
    lib.h3a_attn_fwd.restype = C.c_int32
    lib.h3a_qk_prep.argtypes = [C.POINTER(PrepParams), C.c_void_p]
    lib.h3a_qk_prep.restype = C.c_int32
    lib.h3a_rope_table.argtypes = [C.c_void_p, C.c_int32, C.POINTER(C.c_int32), C.c_float, C.c_void_p, C.c_void_p]
    lib.h3a_rope_table.restype = C.c_int32
    lib.h3a_build_block_index.argtypes = [C.c_int32] * 7 + [C.c_void_p, C.c_void_p, C.POINTER(C.c_int64)]
    lib.h3a_build_block_index.restype = C.c_int32
    lib.h3a_read_device_status.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_int32)]
    lib.h3a_read_device_status.restype = C.c_int32
    lib.h3a_attn_fwd_sparse_static.argtypes = [C.POINTER(AttnParams), C.c_void_p]
    lib.h3a_attn_fwd_sparse_static.restype = C.c_int32
    lib.h3a_static_scratch_capacity.argtypes = [C.POINTER(C.c_size_t)]
    lib.h3a_static_scratch_capacity.restype = C.c_int32
    lib.h3a_memcpy2d_async.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_int32, C.c_void_p]
    lib.h3a_memcpy2d_async.restype = C.c_int32
    lib.h3a_selftest_wait_timeout.argtypes = [C.c_void_p, C.c_int64, C.c_void_p]
    lib.h3a_selftest_wait_timeout.restype = C.c_int32
    lib.h3a_proj_fwd.argtypes = [C.POINTER(ProjParams), C.c_void_p]
    lib.h3a_proj_fwd.restype = C.c_int32
    lib.h3a_adaln_norm.argtypes = [C.POINTER(AdaLnParams), C.c_void_p]
    lib.h3a_adaln_norm.restype = C.c_int32
    lib.h3a_attn_kernel_choice.argtypes = [C.POINTER(AttnParams), C.POINTER(C.c_int32)]
    lib.h3a_attn_kernel_choice.restype = C.c_int32
    lib.h3a_qk_prep_scatter.argtypes = [C.POINTER(PrepParams), C.POINTER(HeadScatter), C.POINTER(HeadScatter), C.c_void_p]
    lib.h3a_qk_prep_scatter.restype = C.c_int32
    lib.h3a_peer_alloc.argtypes = [C.c_size_t, C.POINTER(C.c_void_p), C.c_char_p]
    lib.h3a_peer_alloc.restype = C.c_int32
    lib.h3a_peer_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
    lib.h3a_peer_open.restype = C.c_int32
    lib.h3a_peer_close.argtypes = [C.c_void_p]
    lib.h3a_peer_close.restype = C.c_int32
    lib.h3a_peer_free.argtypes = [C.c_void_p]
    lib.h3a_peer_free.restype = C.c_int32
    _lib = lib
    return lib


def status_string(status: int) -> str:
    return load().h3a_status_string(int(status)).decode()


def check(status: int, where: str) -> None:
    if status != H3A_OK:
        raise H3AError(status, where)


def version() -> tuple:
    a, b = C.c_int32(), C.c_int32()
    check(load().h3a_version(C.byref(a), C.byref(b)), "h3a_version")
    return a.value, b.value
