"""ctypes binding of libapk.so (C ABI in include/apk.h).

The shared library is built in-tree by ``autoparallel_b200.build.build_native`` (nvcc, sm_100a).
There is no fallback: if the library is missing, ``lib()`` raises and every op that needs it
fails loudly.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

APK_MAX_B = 4
APK_MAX_WORLD = 8

APK_OK = 0
APK_ERR_ARG = -1
APK_ERR_CUDA = -2
APK_ERR_SIZE = -3
APK_ERR_TIMEOUT = -4

APK_BF16 = 0
APK_E4M3 = 1
APK_F32 = 2
APK_F16 = 3

APK_SCALE_NONE = 0
APK_SCALE_SCALAR = 1
APK_SCALE_VECTOR = 2
APK_SCALE_ROWS_REPLICATED = 3

APK_REDUCE_SUM = 0
APK_REDUCE_AVG = 1

CSRC_DIR = Path(__file__).resolve().parent / "csrc"
LIB_PATH = CSRC_DIR / "libapk.so"

# Every symbol include/apk.h declares; the CPU test-suite checks that the library exports them.
EXPORTED_SYMBOLS = (
    "apk_abi_version",
    "apk_last_error",
    "apk_symm_alloc",
    "apk_symm_free",
    "apk_symm_export",
    "apk_symm_import",
    "apk_symm_unimport",
    "apk_ag_gemm_arena_bytes",
    "apk_gemm_rs_arena_bytes",
    "apk_ctrl_bytes",
    "apk_ag_gemm",
    "apk_gemm_rs",
    "apk_ag_gemm_static",
    "apk_all_gather",
    "apk_reduce_scatter",
    "apk_debug_schedule",
    "apk_debug_set_rs_lag",
    "apk_check_status",
    "apk_launch_count",
    "apk_pair_launch_count",
    "apk_pair_refusal_count",
    "apk_set_trace",
)


class ApkComm(C.Structure):
    _fields_ = [
        ("rank", C.c_int32),
        ("world", C.c_int32),
        ("data", C.c_void_p * APK_MAX_WORLD),
        ("flags", C.c_void_p * APK_MAX_WORLD),
        ("data_bytes", C.c_uint64),
        ("flag_bytes", C.c_uint64),
        ("ctrl", C.c_void_p),
        ("ctrl_bytes", C.c_uint64),
        ("status", C.c_void_p),
        ("epoch", C.c_uint32),
        ("reserved", C.c_uint32),
        ("timeout_s", C.c_double),
    ]


class ApkOperand(C.Structure):
    _fields_ = [
        ("B", C.c_void_p),
        ("ldb", C.c_int64),
        ("n_major", C.c_int32),
        ("N", C.c_int32),
        ("out", C.c_void_p),
        ("ldo", C.c_int64),
        ("out_dtype", C.c_int32),
        ("b_scale_mode", C.c_int32),
        ("b_scale", C.c_void_p),
        ("bias", C.c_void_p),
        ("bias_dtype", C.c_int32),
        ("reserved", C.c_int32),
        ("result_scale", C.c_void_p),
    ]


class ApkAgGemmArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32),
        ("rows_per_rank", C.c_int32),
        ("K", C.c_int32),
        ("nB", C.c_int32),
        ("A_shard", C.c_void_p),
        ("lda", C.c_int64),
        ("Bs", ApkOperand * APK_MAX_B),
        ("A_gathered", C.c_void_p),
        ("return_A", C.c_int32),
        ("a_scale_mode", C.c_int32),
        ("A_scale", C.c_void_p),
        ("A_scale_gathered", C.c_void_p),
        ("gather_k", C.c_int32),
        ("reserved", C.c_int32),
    ]


class ApkGemmRsArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32),
        ("M", C.c_int32),
        ("K", C.c_int32),
        ("reduce_op", C.c_int32),
        ("A", C.c_void_p),
        ("lda", C.c_int64),
        ("B", ApkOperand),
        ("a_scale_mode", C.c_int32),
        ("scatter_cols", C.c_int32),
        ("A_scale", C.c_void_p),
    ]


class ApkError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"libapk error {code}: {message}")
        self.code = code


_lib = None


def lib() -> C.CDLL:
    """Load libapk.so (once) and declare the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    path = Path(os.environ.get("APK_LIB", LIB_PATH))
    if not path.exists():
        raise RuntimeError(
            f"{path} not found: build it with `python -m autoparallel_b200.build` "
            "(needs nvcc; there is no CPU or PyTorch fallback for the fused ops)"
        )
    L = C.CDLL(str(path))
    L.apk_abi_version.restype = C.c_int
    L.apk_last_error.restype = C.c_char_p
    L.apk_symm_alloc.argtypes = [C.c_uint64, C.POINTER(C.c_void_p)]
    L.apk_symm_free.argtypes = [C.c_void_p]
    L.apk_symm_export.argtypes = [C.c_void_p, C.c_char_p]
    L.apk_symm_import.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
    L.apk_symm_unimport.argtypes = [C.c_void_p]
    L.apk_ag_gemm_arena_bytes.argtypes = [C.POINTER(ApkAgGemmArgs), C.c_int32]
    L.apk_ag_gemm_arena_bytes.restype = C.c_uint64
    L.apk_gemm_rs_arena_bytes.argtypes = [C.POINTER(ApkGemmRsArgs), C.c_int32]
    L.apk_gemm_rs_arena_bytes.restype = C.c_uint64
    L.apk_ctrl_bytes.argtypes = [C.c_int32, C.c_int32]
    L.apk_ctrl_bytes.restype = C.c_uint64
    L.apk_ag_gemm.argtypes = [C.POINTER(ApkComm), C.POINTER(ApkAgGemmArgs), C.c_void_p]
    L.apk_gemm_rs.argtypes = [C.POINTER(ApkComm), C.POINTER(ApkGemmRsArgs), C.c_void_p]
    L.apk_ag_gemm_static.argtypes = [C.POINTER(ApkComm), C.POINTER(ApkAgGemmArgs), C.c_void_p]
    L.apk_ag_gemm_static.restype = C.c_int
    L.apk_all_gather.argtypes = [C.POINTER(ApkComm), C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p]
    L.apk_all_gather.restype = C.c_int
    L.apk_reduce_scatter.argtypes = [C.POINTER(ApkComm), C.c_void_p, C.c_void_p, C.c_uint64, C.c_int32, C.c_int32, C.c_void_p]
    L.apk_reduce_scatter.restype = C.c_int
    L.apk_debug_schedule.argtypes = [C.c_int32] * 5 + [C.POINTER(C.c_int32)] + [C.c_int32] * 3 + [C.POINTER(C.c_int32), C.c_int32]
    L.apk_debug_schedule.restype = C.c_int
    L.apk_debug_set_rs_lag.argtypes = [C.c_int32]
    L.apk_debug_set_rs_lag.restype = None
    L.apk_check_status.argtypes = [C.POINTER(ApkComm), C.c_void_p, C.POINTER(C.c_uint32)]
    L.apk_launch_count.restype = C.c_uint64
    L.apk_pair_launch_count.restype = C.c_uint64
    L.apk_pair_refusal_count.restype = C.c_uint64
    L.apk_set_trace.argtypes = [C.c_void_p, C.c_uint64]
    L.apk_set_trace.restype = C.c_int
    for name in ("apk_symm_alloc", "apk_symm_free", "apk_symm_export", "apk_symm_import", "apk_symm_unimport",
                 "apk_ag_gemm", "apk_gemm_rs", "apk_check_status"):
        getattr(L, name).restype = C.c_int
    if L.apk_abi_version() != 1:
        raise RuntimeError("libapk.so ABI version mismatch; rebuild it")
    _lib = L
    return L


def check(rc: int) -> None:
    if rc != APK_OK:
        raise ApkError(rc, lib().apk_last_error().decode(errors="replace"))
