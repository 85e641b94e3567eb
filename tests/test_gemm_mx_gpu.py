"""GPU parity of GemmMx (e4m3 / e5m2 / e2m1 + E8M0 scales) against the CPU
oracle.  Tolerance: normwise error <= 1e-5 against the reference's f32 result
and against a double reference, plus the reference test's own per-element
bound 8*k*eps*sum|a*b| + 16*eps*|want| (test/test_gemm_mx.cc:217-226).  Cases
follow test/test_gemm_mx.cc:376-479: padded ld / ld_scales, NaN-poisoned D,
k not a multiple of 32, both C layouts, several (alpha, beta), split-k."""
import numpy as np
import pytest

import cpu_ops_b200 as c
from cpu_ops_b200 import _capi, workloads as W
from oracle.loader import (FMT_E2M1, FMT_E4M3, FMT_E5M2, OP_BIAS_ADD, OP_CLAMP, OP_GELU, OP_RELU,
                           OP_SCALE_PER_COL, OP_SCALE_PER_ROW, OP_SILU)
from tests.gpu_helpers import (MX_TOL, check_mx, gather, normwise, run_mx_gpu, run_mx_oracle)

pytestmark = pytest.mark.gpu

SHAPES = [(1, 1, 32), (5, 7, 96), (16, 6, 33), (64, 64, 64), (65, 63, 67), (31, 17, 258),
          (128, 256, 96)]


def _case(oracle, fmt, m, n, k, c_rm, alpha, beta, split=0, tile_n=0, pad=3, lo=124, hi=130, seed=None):
    P = W.mx_problem(fmt, m, n, k, c_rm, pad=pad, scale_lo=lo, scale_hi=hi,
                     seed=(m * 131 + n * 17 + k) if seed is None else seed)
    st, D = run_mx_gpu(P, alpha, beta, split=split, tile_n=tile_n)
    assert st == c.Status.kSuccess, _capi.last_error()
    check_mx(oracle, P, D, alpha, beta)
    return P, D


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_reference_shapes(gpu, oracle, m, n, k):
    _case(oracle, FMT_E4M3, m, n, k, True, 1.0, 0.0)
    _case(oracle, FMT_E4M3, m, n, k, False, 2.0, -0.5)
    _case(oracle, FMT_E5M2, m, n, k, True, 1.0, 0.25)
    _case(oracle, FMT_E2M1, m, n, k & ~1, True, 1.0, 0.0)
    _case(oracle, FMT_E2M1, m, n, k & ~1, False, 0.5, -0.5)


def test_odd_k_fp4(gpu, oracle):
    """The reference accepts an odd k for fp4 as long as ld is even
    (gemm_mx.h:105-108); the nibble after the last element must not leak in."""
    for (m, n, k) in [(16, 6, 33), (65, 63, 67), (5, 130, 257)]:
        _case(oracle, FMT_E2M1, m, n, k, True, 1.0, 0.5)


def test_split_k(gpu, oracle):
    for fmt in (FMT_E4M3, FMT_E2M1):
        _case(oracle, fmt, 32, 32, 4096, True, 1.0, 0.5)           # automatic
    _case(oracle, FMT_E4M3, 24, 40, 3000, True, 1.25, 0.5, split=7)
    _case(oracle, FMT_E5M2, 24, 40, 3000, True, 1.25, 0.5, split=7)
    _case(oracle, FMT_E2M1, 24, 40, 2998, True, 1.25, 0.5, split=7)
    _case(oracle, FMT_E4M3, 200, 300, 2048, False, 1.0, 0.5, split=4)


@pytest.mark.parametrize("fmt", [FMT_E4M3, FMT_E5M2, FMT_E2M1])
def test_every_tile_width(gpu, oracle, fmt):
    for tile_n in (32, 64, 128, 192, 224, 256):
        _case(oracle, fmt, 300, 700, 1024, True, 1.0, 0.5, tile_n=tile_n, pad=0)


def test_run_to_run_determinism(gpu, oracle):
    P = W.mx_problem(FMT_E4M3, 257, 515, 4100, True, seed=21)
    for split in (1, 5):
        outs = [run_mx_gpu(P, 1.0, 0.5, split=split)[1] for _ in range(3)]
        assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))
        assert np.array_equal(outs[0].view(np.uint32), outs[2].view(np.uint32))


def test_small_magnitude_beta(gpu, oracle):
    """With scales around 2^0 the product term dwarfs beta*C; here the scales are
    tiny so that a wrong beta, a missing C or a C read at the wrong place is
    visible at 1e-5."""
    P = W.mx_problem(FMT_E4M3, 96, 160, 256, True, pad=3, scale_lo=110, scale_hi=112, seed=22,
                     c_sigma=1.0)
    st, D = run_mx_gpu(P, 1.0, 0.5)
    assert st == c.Status.kSuccess
    check_mx(oracle, P, D, 1.0, 0.5)
    wrong = run_mx_oracle(oracle, P, 1.0, 0.25)
    G = gather(D, P.m, P.n, P.ldc, True)
    assert normwise(G, gather(wrong, P.m, P.n, P.ldc, True)) > 1e-2  # the test can see beta
    st, D2 = run_mx_gpu(P, 1.0, 0.5, in_place=True)
    assert st == c.Status.kSuccess
    assert np.array_equal(gather(D2, P.m, P.n, P.ldc, True), G)


def test_beta_zero_never_reads_c(gpu, oracle):
    P = W.mx_problem(FMT_E5M2, 40, 50, 160, True, seed=23)
    P.C[:] = np.nan
    st, D = run_mx_gpu(P, 1.0, 0.0)
    assert st == c.Status.kSuccess
    check_mx(oracle, P, D, 1.0, 0.0)


def test_fused_float_chains(gpu, oracle):
    """BiasAdd/Relu/ScalePerRow/ScalePerCol/Clamp are exact f32 ops (same bits as
    applying them to the GEMM result); Gelu/Silu are compared with a tolerance."""
    m, n, k = 70, 150, 320
    # scales 2^-8..2^-5 keep the results O(1), where test_fusion.cc's tolerance applies
    P = W.mx_problem(FMT_E4M3, m, n, k, True, pad=3, seed=24, scale_lo=119, scale_hi=122)
    r = W.rng_for(24, 4)
    v0 = r.standard_normal(max(m, n)).astype(np.float32)
    v1 = (1.0 + 0.1 * r.standard_normal(max(m, n))).astype(np.float32)
    alpha, beta = 1.0, 0.5
    st, plain = run_mx_gpu(P, alpha, beta)
    assert st == c.Status.kSuccess
    acc_scale = float(np.abs(gather(plain, m, n, P.ldc, True)).max())
    chains = [
        ([c.BiasAdd(v0), c.Relu()], [(OP_BIAS_ADD, v0, 0, 0), (OP_RELU, None, 0, 0)], True),
        ([c.ScalePerRow(v0)], [(OP_SCALE_PER_ROW, v0, 0, 0)], True),
        ([c.BiasAdd(v0), c.ScalePerCol(v1), c.Clamp(-0.5, 2.0)],
         [(OP_BIAS_ADD, v0, 0, 0), (OP_SCALE_PER_COL, v1, 0, 0), (OP_CLAMP, None, -0.5, 2.0)], True),
        ([c.Gelu()], [(OP_GELU, None, 0, 0)], False),
        ([c.Silu()], [(OP_SILU, None, 0, 0)], False),
    ]
    for gpu_chain, ops, exact in chains:
        for split in (1, 3):
            st, D = run_mx_gpu(P, alpha, beta, chain=gpu_chain, split=split)
            assert st == c.Status.kSuccess, _capi.last_error()
            want = run_mx_oracle(oracle, P, alpha, beta, ops=ops)
            G = gather(D, m, n, P.ldc, True); R = gather(want, m, n, P.ldc, True)
            # test/test_fusion.cc:89-93 allows 1e-5 * max(1, |ref|) on O(1) data; where
            # a bias cancels a large accumulator the error scales with the accumulator
            tol = 1e-5 * np.maximum(1.0, np.abs(R)) + 1e-6 * acc_scale
            assert np.all(np.abs(G - R) <= tol), float(np.max(np.abs(G - R) / tol))
            if exact and split == 1:
                # chain(plain result) computed on the host from the GPU's own unfused output
                ref_chain = _apply_chain_host(gather(plain, m, n, P.ldc, True), ops)
                assert np.array_equal(G.view(np.uint32), ref_chain.view(np.uint32))


def _apply_chain_host(x, ops):
    x = x.copy()
    m, n = x.shape
    for code, vec, lo, hi in ops:
        if code == OP_RELU:
            x = np.where(x < 0, np.float32(0), x)
        elif code == OP_CLAMP:
            x = np.where(x < np.float32(lo), np.float32(lo), np.where(np.float32(hi) < x, np.float32(hi), x))
        elif code == OP_BIAS_ADD:
            x = x + vec[None, :n]
        elif code == OP_SCALE_PER_ROW:
            x = x * vec[:m, None]
        elif code == OP_SCALE_PER_COL:
            x = x * vec[None, :n]
    return x.astype(np.float32)


def test_special_values_propagate(gpu, oracle):
    """NaN elements, Inf elements and a NaN scale (0xFF) poison exactly the rows /
    columns they touch, as in IEEE arithmetic on the decoded operands."""
    m, n, k = 40, 48, 128
    P = W.mx_problem(FMT_E5M2, m, n, k, True, seed=25)
    P.A[3 * P.lda + 5] = 0x7D            # NaN in row 3 of A
    P.B[7 * P.ldb + 9] = 0x7C            # +Inf in column 7 of B
    P.SA[11 * P.ldsa + 1] = 0xFF         # NaN scale for row 11, block 1
    st, D = run_mx_gpu(P, 1.0, 0.0)
    assert st == c.Status.kSuccess
    want = run_mx_oracle(oracle, P, 1.0, 0.0)
    G = gather(D, m, n, P.ldc, True); R = gather(want, m, n, P.ldc, True)
    assert np.array_equal(np.isnan(G), np.isnan(R))
    assert np.array_equal(np.isinf(G), np.isinf(R))
    fin = np.isfinite(R)
    assert normwise(G[fin], R[fin]) <= MX_TOL
    # e4m3 NaN codes
    Q = W.mx_problem(FMT_E4M3, m, n, k, True, seed=26)
    Q.B[2 * Q.ldb + 100] = 0xFF
    st, D = run_mx_gpu(Q, 1.0, 0.0)
    want = run_mx_oracle(oracle, Q, 1.0, 0.0)
    G = gather(D, m, n, Q.ldc, True); R = gather(want, m, n, Q.ldc, True)
    assert np.array_equal(np.isnan(G), np.isnan(R)) and np.isnan(G[:, 2]).all()


def test_padding_never_meets_a_nan_scale(gpu, oracle):
    """k = 33 with scale entries past ceil(k/32) set to 0xFF: those entries are
    outside the problem (gemm_mx.h:97-99) and must not be read or multiplied."""
    m, n, k = 20, 24, 33
    P = W.mx_problem(FMT_E4M3, m, n, k, True, pad=3, seed=27)
    kg = (k + 31) // 32
    SA = P.SA.reshape(m, P.ldsa); SA[:, kg:] = 0xFF
    SB = P.SB.reshape(n, P.ldsb); SB[:, kg:] = 0xFF
    st, D = run_mx_gpu(P, 1.0, 0.0)
    assert st == c.Status.kSuccess
    check_mx(oracle, P, D, 1.0, 0.0)


def test_extreme_scales(gpu, oracle):
    """Scale exponents over the whole configured range of the large sweep
    ([120, 134]) and e5m2 elements over their whole finite range."""
    _case(oracle, FMT_E5M2, 130, 140, 512, True, 1.0, 0.0, lo=120, hi=134, pad=0)
    _case(oracle, FMT_E2M1, 130, 140, 512, True, 1.0, 0.0, lo=120, hi=134, pad=0)


@pytest.mark.parametrize("m", [1, 8, 32])
def test_decode_shapes(gpu, oracle, m):
    """Decode-shaped mxfp4: M in {1, 8, 32}, K = 4096, all 16 codes in both
    nibbles, scales in [124, 130], beta = 0 (N reduced so the scalar oracle
    finishes quickly; the full N = 14336 runs in the full-size test)."""
    P, D = _case(oracle, FMT_E2M1, m, 1792, 4096, True, 1.0, 0.0, pad=0)
    # e2m1 products with power-of-two scales are exact in f32 at this depth
    want = run_mx_oracle(oracle, P, 1.0, 0.0)
    assert np.array_equal(D.view(np.uint32), want.view(np.uint32))


def test_device_resident_operands(gpu, oracle):
    import torch
    P = W.mx_problem(FMT_E4M3, 300, 520, 1024, True, seed=28, scale_lo=122, scale_hi=132)
    dev = {k_: torch.from_numpy(getattr(P, k_)).cuda() for k_ in ("A", "SA", "B", "SB", "C")}
    dD = torch.full_like(dev["C"], float("nan"))
    op = c.GemmMxE4M3()
    st = op(op.Arguments(c.GemmCoord(P.m, P.n, P.k), c.MxTensorRef(dev["A"], dev["SA"], P.lda, P.ldsa),
                         c.MxTensorRef(dev["B"], dev["SB"], P.ldb, P.ldsb), c.TensorRef(dev["C"], P.ldc),
                         c.TensorRef(dD, P.ldc), c.LinearCombination(1.0, 0.5)))
    assert st == c.Status.kSuccess, _capi.last_error()
    check_mx(oracle, P, dD.cpu().numpy(), 1.0, 0.5)


MIXED = [(FMT_E4M3, FMT_E5M2), (FMT_E5M2, FMT_E4M3), (FMT_E4M3, FMT_E2M1), (FMT_E2M1, FMT_E4M3),
         (FMT_E2M1, FMT_E5M2), (FMT_E5M2, FMT_E2M1)]


@pytest.mark.parametrize("fa,fb", MIXED)
def test_mixed_operand_formats(gpu, oracle, fa, fb):
    """GemmMx<SA, SB> takes any storage pair (gemm/device/gemm_mx.h:44-47).  Shapes cover
    the in-place path (k a multiple of 128, aligned rows), the repacked path (padded
    leading dimension, k not a multiple of 128, odd k), small m (operands swapped), the
    CTA-pair kernel and split-k."""
    cases = [(64, 96, 256, 0, 0, None), (70, 150, 320, 3, 0, None), (33, 47, 77, 3, 0, None),
             (5, 200, 512, 0, 0, None), (300, 260, 1024, 0, 0, True), (130, 140, 2048, 0, 3, None)]
    for m, n, k, pad, split, pair in cases:
        P = W.mx_problem(fa, m, n, k, True, pad=pad, seed=m * 131 + n * 17 + k, fmt_b=fb)
        st, D = run_mx_gpu(P, 1.0, 0.5, split=split, pair=pair)
        assert st == c.Status.kSuccess, (_capi.last_error(), m, n, k)
        if split == 0:
            check_mx(oracle, P, D, 1.0, 0.5)
        else:
            ref = run_mx_oracle(oracle, P, 1.0, 0.5)
            G, R = gather(D, m, n, P.ldc, True), gather(ref, m, n, P.ldc, True)
            assert normwise(G, R) <= MX_TOL


def test_mixed_formats_device_resident_in_place(gpu, oracle):
    """Device operands with k % 128 == 0 and 32-byte aligned rows are read in place
    (no repack launch): exactly two launches per call."""
    import torch
    m, n, k = 256, 384, 1024
    P = W.mx_problem(FMT_E2M1, m, n, k, True, seed=99, fmt_b=FMT_E4M3)
    dev = torch.device("cuda", 0)
    t = {name: torch.from_numpy(getattr(P, name)).to(dev) for name in ("A", "SA", "B", "SB", "C")}
    Dd = torch.full((P.C.size,), float("nan"), device=dev, dtype=torch.float32)
    op = c.GemmMx(c.fp4e2m1_t, c.fp8e4m3_t)
    args = op.Arguments(c.GemmCoord(m, n, k), c.MxTensorRef(t["A"], t["SA"], P.lda, P.ldsa),
                        c.MxTensorRef(t["B"], t["SB"], P.ldb, P.ldsb), c.TensorRef(t["C"], P.ldc),
                        c.TensorRef(Dd, P.ldc), c.LinearCombination(1.0, 0.0), 1)  # one k slice
    before = c.launch_count()
    assert op(args) == c.Status.kSuccess, _capi.last_error()
    assert c.launch_count() - before == 2  # scale re-layout + GEMM, no repack
    check_mx(oracle, P, Dd.cpu().numpy(), 1.0, 0.0)
