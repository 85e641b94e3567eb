"""The headline configurations at their full sizes.  Where the scalar oracle
would take too long the checks are (a) the unmodified reference (oracle/_ref)
when that library is present, (b) the oracle at sampled output positions and
(c) size-independent properties: exact power-of-two linearity, row-block
consistency (the multi-GPU sharding invariant) and run-to-run determinism."""
import numpy as np
import pytest

import cpu_ops_b200 as c
from cpu_ops_b200 import _capi, workloads as W
from oracle.loader import (FMT_E2M1, FMT_E4M3, FMT_E5M2, OP_BIAS_ADD, OP_CLAMP, OP_RELU, Reference,
                           have_reference)
from tests.gpu_helpers import MX_TOL, normwise, run_int8_gpu, run_mx_gpu

pytestmark = pytest.mark.gpu


def _sample(m, n, count, seed):
    r = W.rng_for(seed, 6)
    return r.integers(0, m, size=count), r.integers(0, n, size=count)


def test_mxfp8_e4m3_4096(gpu, oracle):
    """GemmMxE4M3, TN, M = N = K = 4096, non-NaN e4m3 codes, scales in [122, 132],
    C ~ N(0, 1), alpha = 1, beta = 0.5."""
    m = n = k = 4096
    P = W.mx_problem(FMT_E4M3, m, n, k, True, scale_lo=122, scale_hi=132, seed=0xC0FFEE12)
    st, D = run_mx_gpu(P, 1.0, 0.5)
    assert st == c.Status.kSuccess, _capi.last_error()
    assert not np.isnan(D).any()
    rows, cols = _sample(m, n, 4096, 1)
    want, bound = oracle.gemm_mx_f64_sampled(k, FMT_E4M3, P.A, P.SA, k, P.ldsa, FMT_E4M3, P.B, P.SB, k,
                                             P.ldsb, P.C, n, True, 1.0, 0.5, rows, cols)
    got = D.reshape(m, n)[rows, cols].astype(np.float64)
    assert normwise(got, want) <= MX_TOL
    eps = np.finfo(np.float32).eps
    assert np.all(np.abs(got - want) <= 8.0 * k * eps * bound + 16 * eps * np.abs(want) + 1e-12)
    if have_reference():
        R = np.zeros_like(P.C)
        Reference().gemm_mx(m, n, k, FMT_E4M3, P.A, P.SA, k, P.ldsa, FMT_E4M3, P.B, P.SB, k, P.ldsb,
                            P.C, n, R, n, True, 1.0, 0.5, False, 0, 0)
        assert normwise(D, R) <= MX_TOL
    st, D2 = run_mx_gpu(P, 1.0, 0.5)
    assert np.array_equal(D.view(np.uint32), D2.view(np.uint32))


@pytest.mark.parametrize("m", [1, 8, 32])
def test_mxfp4_decode_full_width(gpu, oracle, m):
    """GemmMxE2M1, M in {1, 8, 32}, N = 14336, K = 4096, beta = 0."""
    n, k = 14336, 4096
    P = W.mx_problem(FMT_E2M1, m, n, k, True, scale_lo=124, scale_hi=130, seed=0xC0FFEE20 + m)
    st, D = run_mx_gpu(P, 1.0, 0.0)
    assert st == c.Status.kSuccess, _capi.last_error()
    want = np.zeros_like(P.C)
    oracle.gemm_mx(m, n, k, FMT_E2M1, P.A, P.SA, k, P.ldsa, FMT_E2M1, P.B, P.SB, k, P.ldsb, P.C, n,
                   want, n, True, 1.0, 0.0)
    assert normwise(D, want) <= MX_TOL
    # every partial sum of e2m1 products with these scales is exact in f32
    assert np.array_equal(D.view(np.uint32), want.view(np.uint32))


def test_int8_8192x8192x16384_chain(gpu, oracle):
    """u8 x s8 -> s32 with BiasAdd -> Relu -> Clamp[0, 2^20], split_k_slices = 0,
    full-range operands (|acc| < 2^31: no wrap)."""
    m = n = 8192
    k = 16384
    P = W.int8_problem(m, n, k, seed=0xC0FFEE40)
    bias = W.rng_for(0xC0FFEE40, 9).integers(-(1 << 15), (1 << 15) + 1, size=n, dtype=np.int32)
    chain = [c.BiasAdd(bias), c.Relu(), c.Clamp(0, 1 << 20)]
    ops = [(OP_BIAS_ADD, bias, 0, 0), (OP_RELU, None, 0, 0), (OP_CLAMP, None, 0, 1 << 20)]
    st, D = run_int8_gpu(P, 1, 0, chain=chain, split=0)
    assert st == c.Status.kSuccess, _capi.last_error()
    rows, cols = _sample(m, n, 8192, 2)
    want = oracle.gemm_u8s8s32_sampled(k, P.A, k, True, P.B, n, True, P.C, n, True, 1, 0, 0, ops, rows,
                                       cols)
    assert np.array_equal(D.reshape(m, n)[rows, cols], want)
    # the clamp saturates most outputs; check the raw accumulators too (no chain)
    st, Draw = run_int8_gpu(P, 1, 0, split=0)
    raw = oracle.gemm_u8s8s32_sampled(k, P.A, k, True, P.B, n, True, P.C, n, True, 1, 0, 0, (), rows, cols)
    assert np.array_equal(Draw.reshape(m, n)[rows, cols], raw)
    if have_reference():
        R = np.zeros_like(P.C)
        Reference().gemm_u8s8s32_bias_relu_clamp(m, n, k, P.A, k, P.B, n, P.C, n, R, n, 1, 0, bias, 0,
                                                 1 << 20, 0, 0)
        assert np.array_equal(D, R)
    # a forced two-stage split must give the same bits
    st, D3 = run_int8_gpu(P, 1, 0, chain=chain, split=2)
    assert st == c.Status.kSuccess and np.array_equal(D, D3)


@pytest.mark.parametrize("fmt", [FMT_E5M2, FMT_E2M1])
def test_mx_16384(gpu, oracle, fmt):
    """M = N = K = 16384, TN, finite codes, scales in [120, 134], alpha = 1, beta = 0."""
    m = n = k = 16384
    P = W.mx_problem(fmt, m, n, k, True, scale_lo=120, scale_hi=134, seed=0xC0FFEE50 + fmt)
    st, D = run_mx_gpu(P, 1.0, 0.0)
    assert st == c.Status.kSuccess, _capi.last_error()
    rows, cols = _sample(m, n, 2048, 3)
    want, bound = oracle.gemm_mx_f64_sampled(k, fmt, P.A, P.SA, P.lda, P.ldsa, fmt, P.B, P.SB, P.ldb,
                                             P.ldsb, P.C, n, True, 1.0, 0.0, rows, cols)
    got = D.reshape(m, n)[rows, cols].astype(np.float64)
    assert normwise(got, want) <= MX_TOL
    eps = np.finfo(np.float32).eps
    assert np.all(np.abs(got - want) <= 8.0 * k * eps * bound + 16 * eps * np.abs(want) + 1e-12)
    # linearity in a power of two is exact: D(alpha = 4) == 4 * D(alpha = 1), bit for bit
    rb = 1024
    Q = W.MxProblem(rb, n, k, fmt, fmt, True, P.lda, P.ldb, P.ldsa, P.ldsb, n,
                    P.A[: rb * (P.lda // (2 if fmt == FMT_E2M1 else 1))], P.SA[: rb * P.ldsa], P.B, P.SB,
                    P.C[: rb * n])
    st, Dq = run_mx_gpu(Q, 4.0, 0.0)
    assert st == c.Status.kSuccess
    # row-block consistency: the first 1024 rows computed alone equal the full run's rows
    assert np.array_equal((Dq.reshape(rb, n) / np.float32(4.0)).view(np.uint32),
                          D.reshape(m, n)[:rb].view(np.uint32))
