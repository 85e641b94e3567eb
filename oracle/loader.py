"""ctypes bindings for the test-side checkers (TEST INFRASTRUCTURE ONLY).

Two libraries, both built by ``oracle/Makefile``:

* ``_build/libquant_gemm_oracle.so`` -- the plain-C restatement
  (``quant_gemm_oracle.c``) of the reference's quantized-GEMM arithmetic;
* ``_ref/libcpu_ops_ref_<isa>.so`` -- the unmodified reference headers behind
  ``ref_shim.cc`` (absent where the reference checkout was not available at
  build time; callers must then skip).

Only ``tests/``, the smoke check and the benchmark's CPU-baseline leg import
this module.  The product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ORACLE_SO = HERE / "_build" / "libquant_gemm_oracle.so"
REF_DIR = HERE / "_ref"

FMT_E4M3, FMT_E5M2, FMT_E2M1, FMT_E8M0 = 2, 3, 4, 5
OP_RELU, OP_CLAMP, OP_BIAS_ADD, OP_SCALE_PER_ROW, OP_SCALE_PER_COL, OP_GELU, OP_SILU = range(1, 8)


class _LoHi(C.Union):
    _fields_ = [("i", C.c_int32), ("f", C.c_float)]


class OracleOp(C.Structure):
    _fields_ = [("opcode", C.c_int32), ("pad", C.c_int32), ("ptr", C.c_void_p),
                ("lo", _LoHi), ("hi", _LoHi)]


def build_oracle(force: bool = False) -> Path:
    """Compile the C restatement (gcc only; seconds)."""
    src = HERE / "quant_gemm_oracle.c"
    if force or not ORACLE_SO.exists() or ORACLE_SO.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "oracle"], check=True, capture_output=True)
    return ORACLE_SO


def reference_checkout() -> str:
    """Path of the reference checkout: the environment variable CPU_OPS_REFERENCE, else a
    directory named `reference` beside this repository (empty string when neither exists)."""
    import os
    for cand in (os.environ.get("CPU_OPS_REFERENCE", ""), str(HERE.parent.parent / "reference")):
        if cand and Path(cand, "include", "cpu_ops").is_dir():
            return cand
    return ""


def build_ref(reference: str = "") -> bool:
    """Compile the reference shim and the reference's own test programs (against this
    repository's headers and library) when the reference checkout is present."""
    reference = reference or reference_checkout()
    if not reference:
        return False
    subprocess.run(["make", "-C", str(HERE), "ref", f"REFERENCE={reference}"], check=True,
                   capture_output=True)
    res = subprocess.run(["make", "-C", str(HERE), "upstream_tests", f"REFERENCE={reference}"],
                         capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("the reference's test programs no longer compile against include/:\n" +
                           res.stdout[-3000:] + res.stderr[-3000:])
    return True


def _ptr(a, ctype=C.c_void_p):
    if a is None:
        return None
    return a.ctypes.data_as(ctype)


def _ops_array(ops, is_int, keep):
    """ops: list of (opcode, vector-or-None, lo, hi)."""
    arr = (OracleOp * max(1, len(ops)))()
    for t, (code, vec, lo, hi) in enumerate(ops):
        arr[t].opcode = code
        if vec is not None:
            vec = np.ascontiguousarray(vec, dtype=np.int32 if is_int else np.float32)
            keep.append(vec)
            arr[t].ptr = vec.ctypes.data
        if is_int:
            arr[t].lo.i, arr[t].hi.i = int(lo or 0), int(hi or 0)
        else:
            arr[t].lo.f, arr[t].hi.f = float(lo or 0.0), float(hi or 0.0)
    return arr


class Oracle:
    """The C restatement."""

    def __init__(self):
        self.lib = C.CDLL(str(build_oracle()))
        L = self.lib
        for name in ("oracle_decode_e4m3", "oracle_decode_e5m2", "oracle_decode_e2m1",
                     "oracle_decode_e8m0"):
            getattr(L, name).restype = C.c_float
            getattr(L, name).argtypes = [C.c_uint8]
        for name in ("oracle_encode_e4m3", "oracle_encode_e5m2", "oracle_encode_e2m1",
                     "oracle_encode_e8m0"):
            getattr(L, name).restype = C.c_uint8
            getattr(L, name).argtypes = [C.c_float]
        i, p, f = C.c_int, C.c_void_p, C.c_float
        L.oracle_gemm_u8s8s32.restype = i
        L.oracle_gemm_u8s8s32.argtypes = [i, i, i, p, i, i, p, i, i, p, i, p, i, i, C.c_int32,
                                          C.c_int32, i, i, p]
        L.oracle_gemm_mx.restype = i
        L.oracle_gemm_mx.argtypes = [i, i, i, i, p, p, i, i, i, p, p, i, i, p, i, p, i, i, f, f,
                                     i, i, p, i, i]
        L.oracle_gemm_mx_f64.restype = i
        L.oracle_gemm_mx_f64.argtypes = [i, i, i, i, p, p, i, i, i, p, p, i, i, p, i, i, f, f, p, p]
        L.oracle_gemm_mx_f64_sampled.restype = i
        L.oracle_gemm_mx_f64_sampled.argtypes = [i, i, p, p, i, i, i, p, p, i, i, p, i, i, f, f,
                                                 i, p, p, p, p]
        L.oracle_gemm_u8s8s32_sampled.restype = i
        L.oracle_gemm_u8s8s32_sampled.argtypes = [i, p, i, i, p, i, i, p, i, i, C.c_int32,
                                                  C.c_int32, i, i, p, i, p, p, p]

    def resolve_k_slices(self, m, n, k, kc, requested, threads):
        """Slice count the reference would use (run_blocked.h:100-117)."""
        return self.lib.oracle_resolve_k_slices(m, n, k, kc, requested, threads)

    # -- formats ---------------------------------------------------------------
    def decode(self, fmt, code):
        fn = {FMT_E4M3: self.lib.oracle_decode_e4m3, FMT_E5M2: self.lib.oracle_decode_e5m2,
              FMT_E2M1: self.lib.oracle_decode_e2m1, FMT_E8M0: self.lib.oracle_decode_e8m0}[fmt]
        return fn(int(code) & 0xFF)

    def encode(self, fmt, x):
        fn = {FMT_E4M3: self.lib.oracle_encode_e4m3, FMT_E5M2: self.lib.oracle_encode_e5m2,
              FMT_E2M1: self.lib.oracle_encode_e2m1, FMT_E8M0: self.lib.oracle_encode_e8m0}[fmt]
        return fn(float(x))

    def decode_table(self, fmt):
        n = 16 if fmt == FMT_E2M1 else 256
        return np.array([self.decode(fmt, c) for c in range(n)], dtype=np.float32)

    # -- GEMMs -----------------------------------------------------------------
    def gemm_u8s8s32(self, m, n, k, A, lda, a_rm, B, ldb, b_rm, Cm, ldc, D, ldd, c_rm, alpha=1,
                     beta=0, activation=0, ops=()):
        keep = []
        arr = _ops_array(list(ops), True, keep)
        return self.lib.oracle_gemm_u8s8s32(m, n, k, _ptr(A), lda, int(a_rm), _ptr(B), ldb,
                                            int(b_rm), _ptr(Cm), ldc, _ptr(D), ldd, int(c_rm),
                                            alpha, beta, activation, len(ops),
                                            C.cast(arr, C.c_void_p))

    def gemm_mx(self, m, n, k, fmt_a, A, SA, lda, ldsa, fmt_b, B, SB, ldb, ldsb, Cm, ldc, D, ldd,
                c_rm=True, alpha=1.0, beta=0.0, activation=0, ops=(), kc=512, slices=1):
        keep = []
        arr = _ops_array(list(ops), False, keep)
        return self.lib.oracle_gemm_mx(m, n, k, fmt_a, _ptr(A), _ptr(SA), lda, ldsa, fmt_b,
                                       _ptr(B), _ptr(SB), ldb, ldsb, _ptr(Cm), ldc, _ptr(D), ldd,
                                       int(c_rm), alpha, beta, activation, len(ops),
                                       C.cast(arr, C.c_void_p), kc, slices)

    def gemm_mx_f64(self, m, n, k, fmt_a, A, SA, lda, ldsa, fmt_b, B, SB, ldb, ldsb, Cm, ldc,
                    c_rm=True, alpha=1.0, beta=0.0):
        want = np.zeros((m, n), dtype=np.float64)
        bound = np.zeros((m, n), dtype=np.float64)
        self.lib.oracle_gemm_mx_f64(m, n, k, fmt_a, _ptr(A), _ptr(SA), lda, ldsa, fmt_b, _ptr(B),
                                    _ptr(SB), ldb, ldsb, _ptr(Cm), ldc, int(c_rm), alpha, beta,
                                    _ptr(want), _ptr(bound))
        return want, bound

    def gemm_mx_f64_sampled(self, k, fmt_a, A, SA, lda, ldsa, fmt_b, B, SB, ldb, ldsb, Cm, ldc,
                            c_rm, alpha, beta, rows, cols):
        rows = np.ascontiguousarray(rows, dtype=np.int32)
        cols = np.ascontiguousarray(cols, dtype=np.int32)
        want = np.zeros(len(rows), dtype=np.float64)
        bound = np.zeros(len(rows), dtype=np.float64)
        self.lib.oracle_gemm_mx_f64_sampled(k, fmt_a, _ptr(A), _ptr(SA), lda, ldsa, fmt_b,
                                            _ptr(B), _ptr(SB), ldb, ldsb, _ptr(Cm), ldc,
                                            int(c_rm), alpha, beta, len(rows), _ptr(rows),
                                            _ptr(cols), _ptr(want), _ptr(bound))
        return want, bound

    def gemm_u8s8s32_sampled(self, k, A, lda, a_rm, B, ldb, b_rm, Cm, ldc, c_rm, alpha, beta,
                             activation, ops, rows, cols):
        keep = []
        arr = _ops_array(list(ops), True, keep)
        rows = np.ascontiguousarray(rows, dtype=np.int32)
        cols = np.ascontiguousarray(cols, dtype=np.int32)
        out = np.zeros(len(rows), dtype=np.int32)
        self.lib.oracle_gemm_u8s8s32_sampled(k, _ptr(A), lda, int(a_rm), _ptr(B), ldb, int(b_rm),
                                             _ptr(Cm), ldc, int(c_rm), alpha, beta, activation,
                                             len(ops), C.cast(arr, C.c_void_p), len(rows),
                                             _ptr(rows), _ptr(cols), _ptr(out))
        return out


def _cpu_flags():
    try:
        with open("/proc/cpuinfo") as fh:
            for line in fh:
                if line.startswith("flags"):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def ref_library_path():
    """Widest prebuilt reference variant the running CPU supports, or None."""
    flags = _cpu_flags()
    order = []
    if {"avx512f", "avx512bw", "avx512vl", "avx512dq", "avx512cd", "avx512_vnni",
            "avx512_bf16"} <= flags:
        order.append("avx512")
    if {"avx2", "fma", "f16c", "bmi2"} <= flags:
        order.append("avx2")
    order.append("scalar")
    forced = os.environ.get("CPU_OPS_REF_ISA")
    if forced:
        order = [forced]
    for isa in order:
        p = REF_DIR / f"libcpu_ops_ref_{isa}.so"
        if p.exists():
            return p
    return None


class Reference:
    """The unmodified reference headers behind ref_shim.cc."""

    def __init__(self, path=None):
        path = path or ref_library_path()
        if path is None:
            raise FileNotFoundError("oracle/_ref is not built (run `make -C oracle ref`)")
        self.path = Path(path)
        self.lib = C.CDLL(str(path))
        L = self.lib
        i, p, f = C.c_int, C.c_void_p, C.c_float
        L.ref_gemm_u8s8s32.restype = i
        L.ref_gemm_u8s8s32.argtypes = [i, i, i, i, p, i, p, i, p, i, p, i, C.c_int32, C.c_int32,
                                       i, i, i]
        L.ref_gemm_u8s8s32_bias_relu_clamp.restype = i
        L.ref_gemm_u8s8s32_bias_relu_clamp.argtypes = [i, i, i, p, i, p, i, p, i, p, i, C.c_int32,
                                                       C.c_int32, p, C.c_int32, C.c_int32, i, i]
        L.ref_gemm_mx.restype = i
        L.ref_gemm_mx.argtypes = [i, i, i, i, i, i, p, p, i, i, p, p, i, i, p, i, p, i, f, f, i,
                                  i, i]
        L.ref_gemm_mx_chain.restype = i
        L.ref_gemm_mx_chain.argtypes = [i, i, i, i, i, p, p, i, i, p, p, i, i, p, i, p, i, f, f,
                                        p, p, f, f, i, i]
        L.ref_decode.restype = f
        L.ref_decode.argtypes = [i, C.c_uint8]
        L.ref_encode.restype = C.c_uint8
        L.ref_encode.argtypes = [i, f]
        L.ref_isa.restype = C.c_char_p
        L.ref_mx_kc.restype = i
        L.ref_pool_threads.restype = i

    @property
    def isa(self):
        return self.lib.ref_isa().decode()

    @property
    def mx_kc(self):
        return self.lib.ref_mx_kc()

    @property
    def pool_threads(self):
        return self.lib.ref_pool_threads()

    def decode(self, fmt, code):
        return self.lib.ref_decode(fmt, int(code) & 0xFF)

    def encode(self, fmt, x):
        return self.lib.ref_encode(fmt, float(x))

    def gemm_u8s8s32(self, m, n, k, A, lda, a_rm, B, ldb, b_rm, Cm, ldc, D, ldd, c_rm, alpha=1,
                     beta=0, relu=False, split_k=0, threads=0):
        layouts = int(a_rm) | (int(b_rm) << 1) | (int(c_rm) << 2)
        return self.lib.ref_gemm_u8s8s32(layouts, m, n, k, _ptr(A), lda, _ptr(B), ldb, _ptr(Cm),
                                         ldc, _ptr(D), ldd, alpha, beta, int(relu), split_k,
                                         threads)

    def gemm_u8s8s32_bias_relu_clamp(self, m, n, k, A, lda, B, ldb, Cm, ldc, D, ldd, alpha, beta,
                                     bias, lo, hi, split_k=0, threads=0):
        return self.lib.ref_gemm_u8s8s32_bias_relu_clamp(m, n, k, _ptr(A), lda, _ptr(B), ldb,
                                                         _ptr(Cm), ldc, _ptr(D), ldd, alpha, beta,
                                                         _ptr(bias), lo, hi, split_k, threads)

    def gemm_mx(self, m, n, k, fmt_a, A, SA, lda, ldsa, fmt_b, B, SB, ldb, ldsb, Cm, ldc, D, ldd,
                c_rm=True, alpha=1.0, beta=0.0, relu=False, split_k=0, threads=0):
        return self.lib.ref_gemm_mx(fmt_a, fmt_b, int(c_rm), m, n, k, _ptr(A), _ptr(SA), lda,
                                    ldsa, _ptr(B), _ptr(SB), ldb, ldsb, _ptr(Cm), ldc, _ptr(D),
                                    ldd, alpha, beta, int(relu), split_k, threads)

    def gemm_mx_chain(self, fmt, chain_id, m, n, k, A, SA, lda, ldsa, B, SB, ldb, ldsb, Cm, ldc,
                      D, ldd, alpha=1.0, beta=0.0, vec0=None, vec1=None, lo=0.0, hi=0.0,
                      split_k=0, threads=0):
        return self.lib.ref_gemm_mx_chain(fmt, chain_id, m, n, k, _ptr(A), _ptr(SA), lda, ldsa,
                                          _ptr(B), _ptr(SB), ldb, ldsb, _ptr(Cm), ldc, _ptr(D),
                                          ldd, alpha, beta, _ptr(vec0), _ptr(vec1), lo, hi,
                                          split_k, threads)


def have_reference():
    return ref_library_path() is not None
