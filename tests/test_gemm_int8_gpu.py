"""GPU parity of GemmU8S8S32 against the CPU oracle, bit for bit.  The cases
follow the reference's own test (test/test_gemm_int8.cc:153-229): every layout
combination, padded leading dimensions, poisoned D, in-place C == D, k residues
and k-block boundaries, alpha/beta/relu, k == 0, split-k, determinism -- plus
what it leaves out: full-range operands, s32 fused chains, wrap-around."""
import numpy as np
import pytest

import cpu_ops_b200 as c
from cpu_ops_b200 import _capi, workloads as W
from oracle.loader import OP_BIAS_ADD, OP_CLAMP, OP_RELU, OP_SCALE_PER_COL, OP_SCALE_PER_ROW
from tests.gpu_helpers import INT32_MIN, run_int8_gpu, run_int8_oracle

pytestmark = pytest.mark.gpu

SHAPES = [(1, 1, 1), (1, 1, 5), (6, 16, 4), (5, 7, 9), (3, 5, 7), (16, 16, 16), (64, 64, 64),
          (65, 63, 67), (31, 17, 255), (17, 31, 257), (128, 256, 96)]


def _check(oracle, P, alpha, beta, relu=False, split=0, tile_n=0):
    want = run_int8_oracle(oracle, P, alpha, beta, relu)
    st, D = run_int8_gpu(P, alpha, beta, relu, split=split, tile_n=tile_n)
    assert st == c.Status.kSuccess, _capi.last_error()
    assert np.array_equal(D, want)
    st, D2 = run_int8_gpu(P, alpha, beta, relu, split=split, tile_n=tile_n, in_place=True)
    assert st == c.Status.kSuccess, _capi.last_error()
    # in place: padding elements keep C's values, the m x n window must match
    mask = want != INT32_MIN
    assert np.array_equal(D2[mask], want[mask])


@pytest.mark.parametrize("lay", range(8))
def test_all_layouts_small_shapes(gpu, oracle, lay):
    a_rm, b_rm, c_rm = bool(lay & 1), bool(lay & 2), bool(lay & 4)
    for (m, n, k) in SHAPES:
        for full in (False, True):
            P = W.int8_problem(m, n, k, a_rm, b_rm, c_rm, pad=3, seed=m * 131 + n * 17 + k,
                               full_range=full, c_range=100)
            _check(oracle, P, 1, 0)
            _check(oracle, P, 3, -2)
    P = W.int8_problem(64, 64, 64, a_rm, b_rm, c_rm, pad=3, seed=1)
    _check(oracle, P, 1, 1, relu=True)
    P = W.int8_problem(16, 24, 0, a_rm, b_rm, c_rm, pad=3, seed=2)   # k == 0: D = beta * C
    _check(oracle, P, 1, 5)


@pytest.mark.parametrize("lay", range(8))
def test_split_k(gpu, oracle, lay):
    a_rm, b_rm, c_rm = bool(lay & 1), bool(lay & 2), bool(lay & 4)
    P = W.int8_problem(16, 16, 4096, a_rm, b_rm, c_rm, pad=3, seed=3)
    _check(oracle, P, 3, -2, split=0)
    _check(oracle, P, 3, -2, split=5)
    P = W.int8_problem(32, 32, 8192, a_rm, b_rm, c_rm, pad=3, seed=4)
    _check(oracle, P, 1, 1, relu=True, split=0)
    _check(oracle, P, 1, 1, relu=True, split=7)


def test_results_do_not_depend_on_slices_or_tiles(gpu, oracle):
    """Integer arithmetic: every slice count and tile shape gives the same bits
    (the reference checks 1 vs 8 threads, test_gemm_int8.cc:125-149)."""
    P = W.int8_problem(129, 255, 1097, seed=11)
    want = run_int8_oracle(oracle, P, 3, -2)
    for split in (1, 2, 3, 8):
        for tile_n in (0, 128, 256):
            st, D = run_int8_gpu(P, 3, -2, split=split, tile_n=tile_n)
            assert st == c.Status.kSuccess and np.array_equal(D, want), (split, tile_n)
    P = W.int8_problem(129, 255, 97, True, False, True, seed=12)   # k-major B: every tile width
    want = run_int8_oracle(oracle, P, 3, -2)
    for tile_n in (32, 64, 128, 192, 256):
        st, D = run_int8_gpu(P, 3, -2, tile_n=tile_n)
        assert st == c.Status.kSuccess and np.array_equal(D, want), tile_n


def test_wrap_around_matches_twos_complement(gpu, oracle):
    """alpha/beta large enough to overflow s32: both sides wrap modulo 2^32."""
    P = W.int8_problem(40, 72, 300, seed=13, c_range=2 ** 30)
    want = run_int8_oracle(oracle, P, 70001, 12345)
    st, D = run_int8_gpu(P, 70001, 12345)
    assert st == c.Status.kSuccess and np.array_equal(D, want)


def test_beta_zero_never_reads_c(gpu, oracle):
    P = W.int8_problem(33, 65, 129, seed=14)
    P.C[:] = INT32_MIN  # garbage that would show up if it were multiplied in
    want = run_int8_oracle(oracle, P, 2, 0)
    st, D = run_int8_gpu(P, 2, 0)
    assert st == c.Status.kSuccess and np.array_equal(D, want)


@pytest.mark.parametrize("c_rm", [True, False])
def test_fused_s32_chains(gpu, oracle, c_rm):
    """BiasAdd / Relu / Clamp / ScalePerRow / ScalePerCol on s32 accumulators
    (epilogue/fusion.h:31-129), unsplit and split."""
    m, n, k = 70, 150, 700
    P = W.int8_problem(m, n, k, True, True, c_rm, pad=3, seed=15)
    r = W.rng_for(15, 4)
    bias = r.integers(-(1 << 15), (1 << 15) + 1, size=n, dtype=np.int32)
    rs = r.integers(-3, 4, size=m, dtype=np.int32)
    cs = r.integers(-3, 4, size=n, dtype=np.int32)
    chains = [
        ([c.BiasAdd(bias), c.Relu(), c.Clamp(0, 1 << 20)],
         [(OP_BIAS_ADD, bias, 0, 0), (OP_RELU, None, 0, 0), (OP_CLAMP, None, 0, 1 << 20)]),
        ([c.ScalePerRow(rs), c.BiasAdd(bias)], [(OP_SCALE_PER_ROW, rs, 0, 0), (OP_BIAS_ADD, bias, 0, 0)]),
        ([c.ScalePerCol(cs), c.Clamp(-5000, 7000)], [(OP_SCALE_PER_COL, cs, 0, 0), (OP_CLAMP, None, -5000, 7000)]),
        ([], []),
    ]
    for gpu_chain, oracle_ops in chains:
        for split in (1, 3):
            want = run_int8_oracle(oracle, P, 1, 1, ops=oracle_ops)
            st, D = run_int8_gpu(P, 1, 1, chain=gpu_chain, split=split)
            assert st == c.Status.kSuccess, _capi.last_error()
            assert np.array_equal(D, want)


def test_small_m_uses_swapped_operands(gpu, oracle):
    """m <= 64 puts B on the tensor cores' M side; per-column and per-row chain
    vectors must still index the caller's columns and rows."""
    m, n, k = 8, 1000, 512
    P = W.int8_problem(m, n, k, seed=16)
    r = W.rng_for(16, 4)
    bias = r.integers(-1000, 1000, size=n, dtype=np.int32)
    rs = r.integers(1, 5, size=m, dtype=np.int32)
    want = run_int8_oracle(oracle, P, 1, 1, ops=[(OP_BIAS_ADD, bias, 0, 0), (OP_SCALE_PER_ROW, rs, 0, 0)])
    st, D = run_int8_gpu(P, 1, 1, chain=[c.BiasAdd(bias), c.ScalePerRow(rs)])
    assert st == c.Status.kSuccess and np.array_equal(D, want)


def test_device_resident_operands_and_determinism(gpu, oracle):
    import torch
    P = W.int8_problem(384, 640, 2048, seed=17)
    want = run_int8_oracle(oracle, P, 1, 1)
    dev = {k_: torch.from_numpy(getattr(P, k_)).cuda() for k_ in ("A", "B", "C")}
    outs = []
    for _ in range(2):
        dD = torch.full_like(dev["C"], INT32_MIN)
        st, _ = run_int8_gpu(P, 1, 1, bufs=dict(A=dev["A"], B=dev["B"], C=dev["C"], D=dD), D=P.C)
        assert st == c.Status.kSuccess
        outs.append(dD.cpu().numpy())
    assert np.array_equal(outs[0], want) and np.array_equal(outs[0], outs[1])
    # in place on the device
    dD = dev["C"].clone()
    st, _ = run_int8_gpu(P, 1, 1, bufs=dict(A=dev["A"], B=dev["B"], C=dD, D=dD), D=P.C)
    assert st == c.Status.kSuccess and np.array_equal(dD.cpu().numpy(), want)


def test_unaligned_device_operands_are_repacked(gpu, oracle):
    """Leading dimensions and bases that TMA cannot address (ld = dim + 3, odd
    offsets) on device memory go through the repack kernel."""
    import torch
    for lay in (7, 0, 5):
        a_rm, b_rm, c_rm = bool(lay & 1), bool(lay & 2), bool(lay & 4)
        P = W.int8_problem(65, 63, 67, a_rm, b_rm, c_rm, pad=3, seed=18)
        want = run_int8_oracle(oracle, P, 3, -2)
        # shift every buffer by 1 element so that even the base is unaligned
        dA = torch.zeros(P.A.size + 1, dtype=torch.uint8, device="cuda"); dA[1:] = torch.from_numpy(P.A).cuda()
        dB = torch.zeros(P.B.size + 1, dtype=torch.int8, device="cuda"); dB[1:] = torch.from_numpy(P.B).cuda()
        dC = torch.from_numpy(P.C).cuda()
        dD = torch.full_like(dC, INT32_MIN)
        st, _ = run_int8_gpu(P, 3, -2, bufs=dict(A=dA[1:], B=dB[1:], C=dC, D=dD), D=P.C)
        assert st == c.Status.kSuccess, _capi.last_error()
        assert np.array_equal(dD.cpu().numpy(), want)


def test_config_int8_2048_bit_exact(gpu, oracle):
    """M = N = K = 2048, all row-major, full-range u8/s8, C in [-1000, 1000],
    alpha = beta = 1, split_k_slices = 1: D bit-exact against the CPU path."""
    from oracle.loader import Reference, have_reference
    P = W.int8_problem(2048, 2048, 2048, seed=0xC0FFEE)
    st, D = run_int8_gpu(P, 1, 1, split=1)
    assert st == c.Status.kSuccess, _capi.last_error()
    if have_reference():
        want = np.zeros_like(P.C)
        Reference().gemm_u8s8s32(2048, 2048, 2048, P.A, 2048, True, P.B, 2048, True, P.C, 2048, want,
                                 2048, True, 1, 1, False, 1, 0)
        assert np.array_equal(D, want)
    r = W.rng_for(5, 5)
    rows = r.integers(0, 2048, size=4096); cols = r.integers(0, 2048, size=4096)
    got = D.reshape(2048, 2048)[rows, cols]
    want_s = oracle.gemm_u8s8s32_sampled(2048, P.A, 2048, True, P.B, 2048, True, P.C, 2048, True, 1, 1,
                                         0, (), rows, cols)
    assert np.array_equal(got, want_s)
