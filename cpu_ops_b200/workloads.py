"""Seeded synthetic operands for the quantized-GEMM configurations.

The reference's tests and benchmark draw their inputs from ``std::mt19937``
through library-specific distributions (test/test_gemm_int8.cc:65-68,
test/test_gemm_mx.cc:133-148, examples/01_benchmark.cc:84-88), which are not
portable.  These generators use numpy's ``Philox`` counter-based stream
instead and hand the *same buffers* to the GPU path and to the CPU checker, so
parity never depends on reproducing a C++ distribution.  Value ranges follow
the configuration that is being generated.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import _capi

FMT_BYTES_PER_ELEM = {_capi.FMT_E4M3: 1.0, _capi.FMT_E5M2: 1.0, _capi.FMT_E2M1: 0.5}


def rng_for(seed: int, stream: int = 0) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[seed & 0xFFFFFFFFFFFFFFFF, stream]))


def mx_elements(fmt: int, rows: int, k: int, ld: int, rng: np.random.Generator,
                finite_only: bool = True) -> np.ndarray:
    """`rows` rows of `ld` elements (k valid), uniform over the code space.

    e4m3: the 254 non-NaN codes; e5m2: codes without Inf/NaN; e2m1: all 16 codes
    in both nibbles.  Returned as a flat uint8 array of the storage bytes.
    """
    del k
    if fmt == _capi.FMT_E2M1:
        assert ld % 2 == 0, "fp4 needs an even leading dimension"
        return rng.integers(0, 256, size=rows * ld // 2, dtype=np.uint8)
    raw = rng.integers(0, 256, size=rows * ld, dtype=np.uint8)
    if not finite_only:
        return raw
    if fmt == _capi.FMT_E4M3:
        bad = (raw & 0x7F) == 0x7F
        raw[bad] = (raw[bad] & 0x80) | rng.integers(0, 0x7F, size=int(bad.sum()), dtype=np.uint8)
    else:
        bad = (raw & 0x7C) == 0x7C
        raw[bad] = (raw[bad] & 0x83) | (rng.integers(0, 31, size=int(bad.sum()), dtype=np.uint8) << 2)
    return raw


def mx_scales(rows: int, ld_scales: int, lo: int, hi: int, rng: np.random.Generator) -> np.ndarray:
    """E8M0 exponent bytes, uniform in [lo, hi]."""
    return rng.integers(lo, hi + 1, size=rows * ld_scales, dtype=np.uint8)


@dataclass
class Int8Problem:
    m: int
    n: int
    k: int
    a_row_major: bool
    b_row_major: bool
    c_row_major: bool
    lda: int
    ldb: int
    ldc: int
    A: np.ndarray
    B: np.ndarray
    C: np.ndarray


def int8_problem(m, n, k, a_rm=True, b_rm=True, c_rm=True, pad=0, seed=0, full_range=True,
                 c_range=1000) -> Int8Problem:
    """u8 x s8 operands; full_range draws A in [0,255], B in [-128,127] (the
    reference's own tests stay in [0,15] x [-8,8], test_gemm_int8.cc:66-67)."""
    lda = (k if a_rm else m) + pad
    ldb = (n if b_rm else k) + pad
    ldc = (n if c_rm else m) + pad
    r = rng_for(seed, 1)
    if full_range:
        A = r.integers(0, 256, size=(m if a_rm else k) * lda, dtype=np.uint8)
        B = r.integers(-128, 128, size=(k if b_rm else n) * ldb, dtype=np.int8)
    else:
        A = r.integers(0, 16, size=(m if a_rm else k) * lda, dtype=np.uint8)
        B = r.integers(-8, 9, size=(k if b_rm else n) * ldb, dtype=np.int8)
    Cm = r.integers(-c_range, c_range + 1, size=(m if c_rm else n) * ldc, dtype=np.int32)
    return Int8Problem(m, n, k, a_rm, b_rm, c_rm, lda, ldb, ldc, A, B, Cm)


@dataclass
class MxProblem:
    m: int
    n: int
    k: int
    fmt_a: int
    fmt_b: int
    c_row_major: bool
    lda: int
    ldb: int
    ldsa: int
    ldsb: int
    ldc: int
    A: np.ndarray
    SA: np.ndarray
    B: np.ndarray
    SB: np.ndarray
    C: np.ndarray


def mx_problem(fmt, m, n, k, c_rm=True, pad=0, scale_lo=124, scale_hi=130, seed=0, fmt_b=None,
               c_sigma=1.0, finite_only=True, lds=None) -> MxProblem:
    """MX operands in the TN layout (A: m rows of k, B: n rows of k).  `lds` overrides the
    leading dimension of both scale arrays (default: ceil(k/32), one more when padded)."""
    fmt_b = fmt if fmt_b is None else fmt_b
    even = 1 if (fmt == _capi.FMT_E2M1 or fmt_b == _capi.FMT_E2M1) else 0
    ld = k + pad
    if even and (ld & 1):
        ld += 1
    kg = (k + 31) // 32
    lds = (kg + (1 if pad else 0)) if lds is None else int(lds)
    assert lds >= kg
    ldc = (n if c_rm else m) + pad
    r = rng_for(seed, 2)
    A = mx_elements(fmt, m, k, ld, r, finite_only)
    SA = mx_scales(m, lds, scale_lo, scale_hi, r)
    B = mx_elements(fmt_b, n, k, ld, r, finite_only)
    SB = mx_scales(n, lds, scale_lo, scale_hi, r)
    Cm = (r.standard_normal((m if c_rm else n) * ldc) * c_sigma).astype(np.float32)
    return MxProblem(m, n, k, fmt, fmt_b, c_rm, ld, ld, lds, lds, ldc, A, SA, B, SB, Cm)


# The five headline configurations (shapes, layouts, value ranges, epilogues).
CONFIGS = {
    "int8_2048": dict(kind="int8", m=2048, n=2048, k=2048, alpha=1, beta=1, split_k=1),
    "mxfp8_e4m3_4096": dict(kind="mx", fmt=_capi.FMT_E4M3, m=4096, n=4096, k=4096, alpha=1.0,
                            beta=0.5, scale_lo=122, scale_hi=132),
    "mxfp4_decode": dict(kind="mx", fmt=_capi.FMT_E2M1, m=(1, 8, 32), n=14336, k=4096, alpha=1.0,
                         beta=0.0, scale_lo=124, scale_hi=130),
    "int8_8192_chain": dict(kind="int8", m=8192, n=8192, k=16384, alpha=1, beta=0, split_k=0,
                            chain="bias_relu_clamp", bias_range=1 << 15, clamp=(0, 1 << 20)),
    "mx_16384": dict(kind="mx", fmt=(_capi.FMT_E5M2, _capi.FMT_E2M1), m=16384, n=16384, k=16384,
                     alpha=1.0, beta=0.0, scale_lo=120, scale_hi=134),
}


def gemm_ops(m: int, n: int, k: int) -> float:
    """Algorithmic work, the reference's convention: one multiply-add = 2 ops
    (examples/01_benchmark.cc:101,173)."""
    return 2.0 * m * n * k


def gemm_min_bytes(m, n, k, a_bytes_per_elem, b_bytes_per_elem, mx: bool, beta_nonzero: bool,
                   bias: bool = False) -> float:
    """Compulsory traffic: operands + MX scales + D (+ C if beta != 0) (+ bias)."""
    total = m * k * a_bytes_per_elem + n * k * b_bytes_per_elem + m * n * 4
    if mx:
        total += (m + n) * ((k + 31) // 32)
    if beta_nonzero:
        total += m * n * 4
    if bias:
        total += n * 4
    return float(total)
