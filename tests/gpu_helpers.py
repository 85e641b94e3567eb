"""Helpers shared by the GPU parity tests: run a problem through the C ABI and
through the CPU oracle on the same buffers."""
import numpy as np

import cpu_ops_b200 as c
from cpu_ops_b200 import _capi

STORAGE = {_capi.FMT_E4M3: c.fp8e4m3_t, _capi.FMT_E5M2: c.fp8e5m2_t, _capi.FMT_E2M1: c.fp4e2m1_t}
INT32_MIN = np.iinfo(np.int32).min


def layout(row_major):
    return c.RowMajor if row_major else c.ColumnMajor


def run_int8_gpu(P, alpha=1, beta=0, relu=False, chain=(), split=0, tile_n=0, D=None, in_place=False,
                 bufs=None, pair=None):
    """P: workloads.Int8Problem.  Returns (status, D)."""
    op = c.GemmU8S8S32(layout(P.a_row_major), layout(P.b_row_major), layout(P.c_row_major),
                       tile_n=tile_n, pair=pair)
    if D is None:
        D = P.C.copy() if in_place else np.full_like(P.C, INT32_MIN)  # poison: all must be written
    Cbuf = D if in_place else P.C
    b = bufs or {}
    epi = c.LinearCombinationFused(alpha, beta, list(chain),
                                   c.Activation.kRelu if relu else c.Activation.kNone)
    args = op.Arguments(c.GemmCoord(P.m, P.n, P.k), c.TensorRef(b.get("A", P.A), P.lda),
                        c.TensorRef(b.get("B", P.B), P.ldb), c.TensorRef(b.get("C", Cbuf), P.ldc),
                        c.TensorRef(b.get("D", D), P.ldc), epi, split)
    return op(args), D


def run_int8_oracle(oracle, P, alpha=1, beta=0, relu=False, ops=()):
    D = np.full_like(P.C, INT32_MIN)
    st = oracle.gemm_u8s8s32(P.m, P.n, P.k, P.A, P.lda, P.a_row_major, P.B, P.ldb, P.b_row_major,
                             P.C, P.ldc, D, P.ldc, P.c_row_major, alpha, beta, int(relu), list(ops))
    assert st == 0
    return D


def run_mx_gpu(P, alpha=1.0, beta=0.0, relu=False, chain=(), split=0, tile_n=0, in_place=False,
               pair=None):
    op = c.GemmMx(STORAGE[P.fmt_a], STORAGE[P.fmt_b], layout(P.c_row_major), tile_n=tile_n, pair=pair)
    D = P.C.copy() if in_place else np.full_like(P.C, np.nan)   # NaN poison
    Cbuf = D if in_place else P.C
    epi = c.LinearCombinationFused(alpha, beta, list(chain),
                                   c.Activation.kRelu if relu else c.Activation.kNone)
    args = op.Arguments(c.GemmCoord(P.m, P.n, P.k), c.MxTensorRef(P.A, P.SA, P.lda, P.ldsa),
                        c.MxTensorRef(P.B, P.SB, P.ldb, P.ldsb), c.TensorRef(Cbuf, P.ldc),
                        c.TensorRef(D, P.ldc), epi, split)
    return op(args), D


def run_mx_oracle(oracle, P, alpha=1.0, beta=0.0, relu=False, ops=(), kc=512, slices=1):
    D = np.full_like(P.C, np.nan)
    st = oracle.gemm_mx(P.m, P.n, P.k, P.fmt_a, P.A, P.SA, P.lda, P.ldsa, P.fmt_b, P.B, P.SB, P.ldb,
                        P.ldsb, P.C, P.ldc, D, P.ldc, P.c_row_major, alpha, beta, int(relu),
                        list(ops), kc, slices)
    assert st == 0
    return D


def mx_f64(oracle, P, alpha=1.0, beta=0.0):
    return oracle.gemm_mx_f64(P.m, P.n, P.k, P.fmt_a, P.A, P.SA, P.lda, P.ldsa, P.fmt_b, P.B, P.SB,
                              P.ldb, P.ldsb, P.C, P.ldc, P.c_row_major, alpha, beta)


def gather(flat, m, n, ld, row_major):
    ii, jj = np.meshgrid(np.arange(m), np.arange(n), indexing="ij")
    off = ii * ld + jj if row_major else jj * ld + ii
    return flat[off]


def normwise(got, want):
    got = np.asarray(got, np.float64); want = np.asarray(want, np.float64)
    den = np.linalg.norm(want)
    return np.linalg.norm(got - want) / (den if den > 0 else 1.0)


MX_TOL = 1e-5  # normwise tolerance of the MX paths vs the reference f32 result and vs double


def check_mx(oracle, P, D, alpha, beta, relu=False, tol=MX_TOL):
    """Normwise error vs the f32 oracle and vs the double reference, plus the
    reference test's per-element bound (test/test_gemm_mx.cc:217-226)."""
    m, n, k = P.m, P.n, P.k
    ref32 = run_mx_oracle(oracle, P, alpha, beta, relu)
    G = gather(D, m, n, P.ldc, P.c_row_major)
    R = gather(ref32, m, n, P.ldc, P.c_row_major)
    assert not np.isnan(G).any(), "an output element was not written"
    assert normwise(G, R) <= tol, f"vs reference f32: {normwise(G, R):.3e}"
    if not relu:
        want, bound = mx_f64(oracle, P, alpha, beta)
        assert normwise(G, want) <= tol, f"vs double: {normwise(G, want):.3e}"
        eps = np.finfo(np.float32).eps
        allowed = 8.0 * k * eps * bound + 16.0 * eps * np.abs(want) + 1e-12
        assert np.all(np.abs(G.astype(np.float64) - want) <= allowed), "outside the reference test's bound"
