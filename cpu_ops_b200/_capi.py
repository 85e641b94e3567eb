"""ctypes binding of the C ABI declared in ``include/cpu_ops_b200.h``.

The shared library is built in-tree (``cpu_ops_b200/libcpu_ops_b200.so``) by
``cpu_ops_b200/build.py``.  There is no fallback: if the library is missing,
``load()`` raises, and every GEMM entry point goes through it.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "libcpu_ops_b200.so"

MAX_OPS = 8

STATUS_SUCCESS = 0
STATUS_INVALID_PROBLEM = 1
STATUS_INVALID_ARGUMENTS = 2
STATUS_UNSUPPORTED = 3
STATUS_NO_DEVICE = 4
STATUS_CUDA_ERROR = 5
STATUS_DEVICE_TIMEOUT = 6
STATUS_BAD_DESCRIPTOR = 7

FMT_U8, FMT_S8, FMT_E4M3, FMT_E5M2, FMT_E2M1 = 0, 1, 2, 3, 4
KIND_I8, KIND_MX = 0, 1
ACT_NONE, ACT_RELU = 0, 1
OP_RELU, OP_CLAMP, OP_BIAS_ADD, OP_SCALE_PER_ROW, OP_SCALE_PER_COL, OP_GELU, OP_SILU = range(1, 8)
MEM_AUTO, MEM_HOST, MEM_DEVICE = 0, 1, 2
FLAG_ASYNC = 1
FLAG_PAIR_ON, FLAG_PAIR_OFF = 2, 4
NOALLOC_SCRATCH_BYTES = 8 << 20

# Every symbol include/cpu_ops_b200.h declares.
EXPORTED_SYMBOLS = (
    "cpuops_b200_gemm",
    "cpuops_b200_gemm_i8_noalloc",
    "cpuops_b200_relayout_scales",
    "cpuops_b200_scale_layout_bytes",
    "cpuops_b200_shard_rows",
    "cpuops_b200_stream_status",
    "cpuops_b200_set_sm_limit",
    "cpuops_b200_set_wait_budget_us",
    "cpuops_b200_selftest_wait_timeout",
    "cpuops_b200_profile",
    "cpuops_b200_profile_collect",
    "cpuops_b200_launch_count",
    "cpuops_b200_last_plan",
    "cpuops_b200_prepare_b",
    "cpuops_b200_release_b",
    "cpuops_b200_last_error",
    "cpuops_b200_abi_version",
    "cpuops_b200_device_count",
)


class Plan(C.Structure):
    """cpuops_b200_plan: what the last GEMM call launched (diagnostics)."""
    _fields_ = [("swapped", C.c_int32), ("tile_n", C.c_int32), ("pair", C.c_int32),
                ("slices", C.c_int32), ("stages", C.c_int32), ("grid", C.c_int32),
                ("c_ring", C.c_int32), ("prepared_b", C.c_int32),
                ("epilogue_warps", C.c_int32), ("narrow_last", C.c_int32), ("decode", C.c_int32)]


class Scalar(C.Union):
    _fields_ = [("i32", C.c_int32), ("f32", C.c_float)]


class EpilogueOp(C.Structure):
    _fields_ = [("opcode", C.c_int32), ("reserved", C.c_int32), ("ptr", C.c_void_p),
                ("lo", Scalar), ("hi", Scalar)]


class GemmDesc(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("kind", C.c_int32), ("a_format", C.c_int32),
        ("b_format", C.c_int32), ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32),
        ("a_row_major", C.c_int32), ("b_row_major", C.c_int32), ("c_row_major", C.c_int32),
        ("a", C.c_void_p), ("b", C.c_void_p), ("a_scales", C.c_void_p), ("b_scales", C.c_void_p),
        ("lda", C.c_int32), ("ldb", C.c_int32), ("ld_scales_a", C.c_int32),
        ("ld_scales_b", C.c_int32), ("c", C.c_void_p), ("d", C.c_void_p), ("ldc", C.c_int32),
        ("ldd", C.c_int32), ("alpha", Scalar), ("beta", Scalar), ("activation", C.c_int32),
        ("n_ops", C.c_int32), ("ops", EpilogueOp * MAX_OPS), ("split_k_slices", C.c_int32),
        ("memory_space", C.c_int32), ("stream", C.c_void_p), ("flags", C.c_uint32),
        ("device", C.c_int32), ("tile_n", C.c_int32),
    ]


_lib = None


def load() -> C.CDLL:
    """Load the CUDA library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m cpu_ops_b200.build` "
            "(nvcc, sm_100a).  cpu_ops_b200 has no CPU fallback.")
    lib = C.CDLL(str(LIB_PATH))
    lib.cpuops_b200_gemm.restype = C.c_int
    lib.cpuops_b200_gemm.argtypes = [C.POINTER(GemmDesc)]
    lib.cpuops_b200_gemm_i8_noalloc.restype = C.c_int
    lib.cpuops_b200_gemm_i8_noalloc.argtypes = [C.POINTER(GemmDesc)]
    lib.cpuops_b200_relayout_scales.restype = C.c_int
    lib.cpuops_b200_relayout_scales.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                                C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
    lib.cpuops_b200_scale_layout_bytes.restype = C.c_size_t
    lib.cpuops_b200_scale_layout_bytes.argtypes = [C.c_int32] * 4
    lib.cpuops_b200_shard_rows.restype = C.c_int
    lib.cpuops_b200_shard_rows.argtypes = [C.c_int32, C.c_int32, C.c_int32,
                                           C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    lib.cpuops_b200_stream_status.restype = C.c_int
    lib.cpuops_b200_stream_status.argtypes = [C.c_void_p]
    lib.cpuops_b200_set_sm_limit.restype = C.c_int
    lib.cpuops_b200_set_sm_limit.argtypes = [C.c_int32, C.c_int32]
    lib.cpuops_b200_set_wait_budget_us.restype = C.c_int
    lib.cpuops_b200_set_wait_budget_us.argtypes = [C.c_uint32]
    lib.cpuops_b200_selftest_wait_timeout.restype = C.c_int
    lib.cpuops_b200_selftest_wait_timeout.argtypes = [C.c_uint32, C.c_void_p]
    lib.cpuops_b200_profile.restype = C.c_int
    lib.cpuops_b200_profile.argtypes = [C.c_int]
    lib.cpuops_b200_profile_collect.restype = C.c_int
    lib.cpuops_b200_profile_collect.argtypes = [C.POINTER(C.c_double), C.POINTER(C.c_int32)]
    lib.cpuops_b200_launch_count.restype = C.c_uint64
    lib.cpuops_b200_prepare_b.restype = C.c_int
    lib.cpuops_b200_prepare_b.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
    lib.cpuops_b200_release_b.restype = C.c_int
    lib.cpuops_b200_release_b.argtypes = [C.c_void_p]
    lib.cpuops_b200_last_plan.restype = C.c_int
    lib.cpuops_b200_last_plan.argtypes = [C.POINTER(Plan)]
    lib.cpuops_b200_last_error.restype = C.c_char_p
    lib.cpuops_b200_abi_version.restype = C.c_int
    lib.cpuops_b200_device_count.restype = C.c_int
    _lib = lib
    return lib


def last_plan() -> Plan:
    plan = Plan()
    load().cpuops_b200_last_plan(C.byref(plan))
    return plan


def last_error() -> str:
    return load().cpuops_b200_last_error().decode(errors="replace")
