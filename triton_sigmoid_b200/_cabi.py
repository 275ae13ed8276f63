"""ctypes binding of the C ABI in ``include/sigattn_b200.h``.

There is no fallback: if the shared library is missing, loading fails with instructions
to build it, and every call reports the library's own error text.
"""

from __future__ import annotations

import ctypes
import os
import threading

from ._paths import LIB_PATH

SIGATTN_FP16 = 0
SIGATTN_BF16 = 1
SIGATTN_FP32 = 2
SIGATTN_CAUSAL = 1
SIGATTN_ACCURATE = 2
SIGATTN_BWD_SPLIT = 4
SIGATTN_BIAS_NEG_LOG_LK = 8
SIGATTN_STATIC_SCRATCH_ELEMS = 8 * 1024 * 1024

Q_ABI_VERSION, Q_SM_ARCH, Q_MAX_HEAD_DIM, Q_PARAMS_SIZE = 0, 1, 2, 3

EXPORTED_SYMBOLS = (
    "sigattn_fwd",
    "sigattn_bwd",
    "sigattn_bwd_static_scratch",
    "sigattn_bwd_workspace_bytes",
    "sigattn_last_error",
    "sigattn_query",
    "sigattn_device_status",
    "sigattn_selftest_bounded_wait",
)


class SigAttnParams(ctypes.Structure):
    """Field-for-field mirror of ``struct SigAttnParams``."""

    _fields_ = [
        ("struct_bytes", ctypes.c_uint32),
        ("dtype", ctypes.c_int32),
        ("B", ctypes.c_int32),
        ("H", ctypes.c_int32),
        ("D", ctypes.c_int32),
        ("Tq", ctypes.c_int32),
        ("Tk", ctypes.c_int32),
        ("flags", ctypes.c_uint32),
        ("scale", ctypes.c_float),
        ("bias_scalar", ctypes.c_float),
        ("device", ctypes.c_int32),
        ("reserved0", ctypes.c_int32),
        ("q", ctypes.c_void_p),
        ("k", ctypes.c_void_p),
        ("v", ctypes.c_void_p),
        ("o", ctypes.c_void_p),
        ("dout", ctypes.c_void_p),
        ("dq", ctypes.c_void_p),
        ("dk", ctypes.c_void_p),
        ("dv", ctypes.c_void_p),
        ("q_strides", ctypes.c_int64 * 3),
        ("k_strides", ctypes.c_int64 * 3),
        ("v_strides", ctypes.c_int64 * 3),
        ("o_strides", ctypes.c_int64 * 3),
        ("do_strides", ctypes.c_int64 * 3),
        ("dq_strides", ctypes.c_int64 * 3),
        ("dk_strides", ctypes.c_int64 * 3),
        ("dv_strides", ctypes.c_int64 * 3),
        ("seq_lens_q", ctypes.c_void_p),
        ("seq_lens_k", ctypes.c_void_p),
        ("bias", ctypes.c_void_p),
        ("score_mod", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("stream", ctypes.c_void_p),
        ("ev_main_start", ctypes.c_void_p),
        ("ev_main_stop", ctypes.c_void_p),
        ("cu_seqlens_q", ctypes.c_void_p),
        ("cu_seqlens_k", ctypes.c_void_p),
        ("total_q", ctypes.c_int32),
        ("total_k", ctypes.c_int32),
    ]


_lib = None
_lock = threading.Lock()


def load() -> ctypes.CDLL:
    """Load (once) and type the shared library."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = os.environ.get("SIGATTN_B200_LIB", LIB_PATH)  # explicit override of the library location
        if not os.path.exists(path):
            raise ImportError(
                f"{path} is missing: build it with `python -m triton_sigmoid_b200.build` "
                "(needs nvcc with sm_100a support). This package has no other execution path."
            )
        lib = ctypes.CDLL(path)
        lib.sigattn_fwd.argtypes = [ctypes.POINTER(SigAttnParams)]
        lib.sigattn_fwd.restype = ctypes.c_int
        lib.sigattn_bwd.argtypes = [ctypes.POINTER(SigAttnParams)]
        lib.sigattn_bwd.restype = ctypes.c_int
        lib.sigattn_bwd_static_scratch.argtypes = [ctypes.POINTER(SigAttnParams)]
        lib.sigattn_bwd_static_scratch.restype = ctypes.c_int
        lib.sigattn_bwd_workspace_bytes.argtypes = [ctypes.c_int32] * 4
        lib.sigattn_bwd_workspace_bytes.restype = ctypes.c_size_t
        lib.sigattn_last_error.argtypes = []
        lib.sigattn_last_error.restype = ctypes.c_char_p
        lib.sigattn_query.argtypes = [ctypes.c_int]
        lib.sigattn_query.restype = ctypes.c_int
        lib.sigattn_device_status.argtypes = [ctypes.c_int]
        lib.sigattn_device_status.restype = ctypes.c_int
        lib.sigattn_selftest_bounded_wait.argtypes = [ctypes.c_int, ctypes.c_int]
        lib.sigattn_selftest_bounded_wait.restype = ctypes.c_int
        if lib.sigattn_query(Q_PARAMS_SIZE) != ctypes.sizeof(SigAttnParams):
            raise ImportError(
                f"SigAttnParams layout mismatch: library {lib.sigattn_query(Q_PARAMS_SIZE)} bytes, "
                f"binding {ctypes.sizeof(SigAttnParams)} bytes; rebuild the library"
            )
        _lib = lib
    return _lib


def last_error() -> str:
    return load().sigattn_last_error().decode("utf-8", "replace")


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed (code {rc}): {last_error()}")
