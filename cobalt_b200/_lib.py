"""ctypes binding of libcobalt_b200.so (the C ABI declared in include/cobalt_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint32, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcobalt_b200.so")


class CobaltMat(Structure):
    """Mirror of ``struct CobaltMat``."""
    _fields_ = [
        ("tiles", c_void_p),
        ("tile_off", c_void_p),
        ("col_scale", c_void_p),
        ("K", c_int32), ("N", c_int32),
        ("bits", c_int32), ("group", c_int32),
        ("n_row_blocks", c_int32), ("n_col_tiles", c_int32),
        ("max_tile_bytes", c_uint32), ("max_tile_nnz", c_uint32),
        ("nnz", c_int64),
    ]


class CobaltPeerSlots(Structure):
    """Mirror of ``struct CobaltPeerSlots``."""
    _fields_ = [
        ("peer_base", c_void_p),
        ("rank", c_int32), ("world", c_int32),
        ("slot_stride_bytes", c_size_t), ("flags_off_bytes", c_size_t),
    ]


class CobaltStagedInput(Structure):
    """Mirror of ``struct CobaltStagedInput``."""
    _fields_ = [
        ("kind", c_int32), ("flavor", c_int32),
        ("a", c_void_p), ("b", c_void_p),
        ("ld", c_int64),
        ("w", c_void_p), ("w_branch", c_void_p), ("h_out", c_void_p),
        ("eps", c_float),
        ("b_slots", POINTER(CobaltPeerSlots)),
    ]


IN_PLAIN, IN_GLU, IN_ADDNORM = 0, 1, 2
EUNSUPPORTED = -7


class CobaltError(RuntimeError):
    def __init__(self, fn: str, status: int, text: str):
        super().__init__(f"{fn} failed with status {status}: {text}")
        self.status = status


EXPORTS = {
    # name: (restype, argtypes)
    "cobalt_version": (c_int, []),
    "cobalt_strerror": (c_char_p, [c_int]),
    "cobalt_gemv": (c_int, [POINTER(CobaltMat), c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int, c_void_p,
                            c_size_t, c_void_p]),
    "cobalt_gemv_scratch_bytes": (c_size_t, [POINTER(CobaltMat), c_int]),
    "cobalt_gemv_static": (c_int, [POINTER(CobaltMat), c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int, c_void_p]),
    "cobalt_gemv_fused": (c_int, [c_int, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_size_t,
                                  c_void_p]),
    "cobalt_gemv_fused_scratch_bytes": (c_size_t, [c_int, c_void_p, c_int]),
    "cobalt_gemv_fused_staged": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                         c_void_p, c_size_t, c_void_p]),
    "cobalt_gemv_fused_host_async": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_size_t,
                                             c_void_p]),
    "cobalt_peer_sum": (c_int, [c_void_p, c_size_t, c_void_p, c_int, c_void_p, c_void_p]),
    "cobalt_gemv_rowwalk": (c_int, [POINTER(CobaltMat), c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int,
                                    c_void_p]),
    "cobalt_gemm": (c_int, [POINTER(CobaltMat), c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int, c_void_p,
                            c_size_t, c_void_p]),
    "cobalt_gemm_scratch_bytes": (c_size_t, [POINTER(CobaltMat), c_int]),
    "cobalt_linear_f32": (c_int, [POINTER(CobaltMat), c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p, c_size_t,
                                  c_void_p]),
    "cobalt_dequant": (c_int, [POINTER(CobaltMat), c_void_p, c_void_p]),
    "cobalt_unpack": (c_int, [POINTER(CobaltMat), c_void_p, c_void_p, c_void_p]),
    "cobalt_linear_host": (c_int, [POINTER(CobaltMat), c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                   c_void_p, c_size_t, c_void_p]),
    "cobalt_linear_host_async": (c_int, [POINTER(CobaltMat), c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                   c_void_p, c_size_t, c_void_p]),
    "cobalt_add_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p,
                                   c_void_p]),
    "cobalt_rope_kv": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                               c_int, c_void_p, c_void_p, c_float, c_int64, c_void_p]),
    "cobalt_swiglu": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "cobalt_attn_decode_scratch_bytes": (c_size_t, [c_int, c_int, c_int]),
    "cobalt_attn_decode": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_int, c_int, c_int, c_int,
                                   c_int, c_float, c_int, c_int64, c_void_p]),
    "cobalt_attn_decode_fused": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_int, c_int, c_int,
                                         c_int, c_int, c_float, c_int, c_int64, c_void_p]),
    "cobalt_attn_decode_fused_scratch_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "cobalt_allreduce_peer": (c_int, [c_void_p, c_int, c_int, c_size_t, c_size_t, c_size_t, c_void_p, c_int, c_void_p,
                                      c_void_p]),
    "cobalt_device_status": (c_int, [c_void_p, c_void_p, POINTER(c_uint32)]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m cobalt_b200.build` (needs nvcc); "
                "cobalt_b200 has no fallback path")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in EXPORTS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(fn: str, status: int) -> None:
    if status != 0:
        text = load().cobalt_strerror(status).decode()
        raise CobaltError(fn, status, text)
