"""ctypes binding of libb200s.so (declared in include/b200s.h).

The library is the only compute path: loading fails loudly when the shared object is missing
and no function here falls back to torch or the CPU.
"""
from __future__ import annotations

import ctypes
import os
import threading

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
# B200S_LIBRARY names another build of the same library (A/B comparisons of kernel variants).
LIB_PATH = os.environ.get("B200S_LIBRARY") or os.path.join(PKG_DIR, "libb200s.so")

# enums of include/b200s.h
BF16, FP16, FP32 = 0, 1, 2
K_MAJOR, MN_MAJOR = 0, 1
ALGO_AUTO, ALGO_DENSE, ALGO_CLASSIC, ALGO_WINOGRAD = 0, 1, 2, 3
PREC_TF32, PREC_3XTF32 = 0, 1

OK = 0
ERR_NULL_POINTER = -1
ERR_BAD_SHAPE = -2
ERR_BAD_STRIDE = -3
ERR_BAD_ALIGNMENT = -4
ERR_BAD_DTYPE = -5
ERR_BAD_ALGO = -6
ERR_BAD_DEPTH = -7
ERR_WORKSPACE_TOO_SMALL = -8
ERR_CUDA = -9
ERR_NO_DEVICE = -10
ERR_DEVICE_TIMEOUT = -11
ERR_TUNER_IO = -12
ERR_TOO_LARGE = -13


class Problem(ctypes.Structure):
    """Mirror of ``struct b200s_problem``."""

    _fields_ = [
        ("M", ctypes.c_int64), ("N", ctypes.c_int64), ("K", ctypes.c_int64),
        ("batch", ctypes.c_int64),
        ("lda", ctypes.c_int64), ("ldb", ctypes.c_int64), ("ldc", ctypes.c_int64),
        ("strideA", ctypes.c_int64), ("strideB", ctypes.c_int64), ("strideC", ctypes.c_int64),
        ("a_major", ctypes.c_int32), ("b_major", ctypes.c_int32),
        ("in_dtype", ctypes.c_int32), ("out_dtype", ctypes.c_int32),
        ("algo", ctypes.c_int32), ("depth", ctypes.c_int32), ("beta", ctypes.c_int32),
        ("prod_dtype", ctypes.c_int32), ("precision", ctypes.c_int32), ("tile_variant", ctypes.c_int32),
        ("pipeline", ctypes.c_int32), ("b_blocks_ready", ctypes.c_int32), ("fuse", ctypes.c_int32),
    ]


class B200SError(RuntimeError):
    """A libb200s.so call returned a negative status."""

    def __init__(self, status: int, text: str):
        super().__init__(f"b200s status {status}: {text}")
        self.status = status


# name -> (restype, argtypes); every symbol include/b200s.h declares.
_P = ctypes.POINTER
SIGNATURES = {
    "b200s_version": (ctypes.c_int, []),
    "b200s_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "b200s_last_cuda_error": (ctypes.c_char_p, []),
    "b200s_workspace_bytes": (ctypes.c_int, [_P(Problem), _P(ctypes.c_size_t)]),
    "b200s_matmul": (ctypes.c_int, [_P(Problem), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                    ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "b200s_matmul_bias": (ctypes.c_int, [_P(Problem), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                         ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "b200s_matmul_static": (ctypes.c_int, [_P(Problem), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                           ctypes.c_void_p]),
    "b200s_resolve": (ctypes.c_int, [_P(Problem), _P(ctypes.c_int32), _P(ctypes.c_int32)]),
    "b200s_tuner_clear": (ctypes.c_int, []),
    "b200s_tuner_record": (ctypes.c_int, [ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int32,
                                          ctypes.c_int32, ctypes.c_int32]),
    "b200s_tuner_load": (ctypes.c_int, [ctypes.c_char_p]),
    "b200s_tuner_save": (ctypes.c_int, [ctypes.c_char_p]),
    "b200s_tuner_lookup": (ctypes.c_int, [ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int32,
                                          _P(ctypes.c_int32), _P(ctypes.c_int32)]),
    "b200s_tuner_record_schedule": (ctypes.c_int, [ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int32,
                                                   ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]),
    "b200s_tuner_lookup_schedule": (ctypes.c_int, [ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int32,
                                                   _P(ctypes.c_int32), _P(ctypes.c_int32), _P(ctypes.c_int32)]),
    "b200s_device_status": (ctypes.c_int, [ctypes.c_void_p, _P(ctypes.c_int32), _P(ctypes.c_int32)]),
    "b200s_wait_probe": (ctypes.c_int, [ctypes.c_uint64, ctypes.c_void_p]),
    "b200s_static_status": (ctypes.c_int, [ctypes.c_void_p, _P(ctypes.c_int32), _P(ctypes.c_int32)]),
    "b200s_launch_count": (ctypes.c_int64, []),
    "b200s_profile_begin": (ctypes.c_int, [ctypes.c_int]),
    "b200s_profile_end": (ctypes.c_int, [_P(ctypes.c_float), _P(ctypes.c_int32)]),
    "b200s_preadd": (ctypes.c_int, [_P(Problem), ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "b200s_combine_peers": (ctypes.c_int, [_P(Problem), ctypes.c_void_p, _P(ctypes.c_void_p), ctypes.c_int,
                                           ctypes.c_void_p]),
    "b200s_matmul_peers": (ctypes.c_int, [_P(Problem), ctypes.c_void_p, ctypes.c_void_p, _P(ctypes.c_void_p), ctypes.c_int,
                                          ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "b200s_matmul_multicast": (ctypes.c_int, [_P(Problem), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                              ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "b200s_peer_barrier": (ctypes.c_int, [_P(ctypes.c_void_p), ctypes.c_int, ctypes.c_int, ctypes.c_uint32,
                                          ctypes.c_uint64, ctypes.c_void_p]),
    "b200s_push_rows": (ctypes.c_int, [ctypes.c_void_p, _P(ctypes.c_void_p), ctypes.c_int, ctypes.c_size_t,
                                       ctypes.c_void_p]),
    "b200s_set_product_sms": (ctypes.c_int, [ctypes.c_int]),
    "b200s_set_sender_sms": (ctypes.c_int, [ctypes.c_int]),
    "b200s_push_panel": (ctypes.c_int, [ctypes.c_void_p, _P(ctypes.c_void_p), ctypes.c_int, ctypes.c_void_p,
                                        ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]),
    "b200s_combine": (ctypes.c_int, [_P(Problem), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
}

_lib = None
_lock = threading.Lock()


def load() -> ctypes.CDLL:
    """Load libb200s.so once and attach the prototypes. Raises if the library was not built."""
    global _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise ImportError(
                    f"{LIB_PATH} is missing: build it with `python -m strassen_triton_b200.build` "
                    "(there is no fallback path)")
            lib = ctypes.CDLL(LIB_PATH)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
            # measured (M, N, K) -> (algo, depth) table shipped beside the library; a missing or
            # corrupt file leaves the library's built-in thresholds in force
            table = os.path.join(PKG_DIR, "tuner_table.txt")
            if os.path.exists(table):
                lib.b200s_tuner_load(table.encode())
            _lib = lib
    return _lib


def status_string(status: int) -> str:
    return load().b200s_status_string(status).decode()


def check(status: int) -> None:
    """Map a negative status to the exception type the reference raises for that mistake:
    shape problems are ValueError (strassen.py:757-762), everything else B200SError."""
    if status == OK:
        return
    text = status_string(status)
    if status == ERR_CUDA:
        text += ": " + load().b200s_last_cuda_error().decode()
    if status in (ERR_BAD_SHAPE, ERR_BAD_DEPTH):
        raise ValueError(f"b200s status {status}: {text}")
    raise B200SError(status, text)
