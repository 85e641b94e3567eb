"""GPU parity of the two-CTA form of the GEMM kernel (clusters of two CTAs on one
256-row tile, tcgen05 cta_group::2), forced on through the descriptor flag so that
small shapes reach it: every layout it supports, ragged m / n / k, split-k slabs,
chains, the C ring, and bit-identity with the one-CTA kernel."""
import numpy as np
import pytest

import cpu_ops_b200 as c
from cpu_ops_b200 import _capi, workloads as W
from oracle.loader import FMT_E2M1, FMT_E4M3, FMT_E5M2, OP_BIAS_ADD, OP_CLAMP, OP_RELU, OP_SCALE_PER_ROW
from tests.gpu_helpers import (check_mx, gather, run_int8_gpu, run_int8_oracle, run_mx_gpu,
                               run_mx_oracle)

pytestmark = pytest.mark.gpu


def _assert_pair(expected=1):
    assert _capi.last_plan().pair == expected


@pytest.mark.parametrize("m,n,k", [(256, 256, 128), (300, 260, 1000), (129, 70, 96), (640, 512, 4096),
                                   (1000, 1000, 333)])
@pytest.mark.parametrize("a_rm,b_rm", [(1, 0), (0, 0)])
def test_int8_pair_k_major_b(gpu, oracle, m, n, k, a_rm, b_rm):
    """B column-major (k contiguous): any tile width; A row- or column-major."""
    for c_rm in (1, 0):
        P = W.int8_problem(m, n, k, a_rm, b_rm, c_rm, pad=3, seed=m + n + k)
        st, D = run_int8_gpu(P, alpha=3, beta=-2, pair=True)
        assert st == c.Status.kSuccess, _capi.last_error()
        _assert_pair()
        want = run_int8_oracle(oracle, P, alpha=3, beta=-2)
        assert np.array_equal(gather(D, m, n, P.ldc, c_rm), gather(want, m, n, P.ldc, c_rm))


@pytest.mark.parametrize("m,n,k", [(256, 256, 128), (384, 700, 520), (1000, 513, 256)])
def test_int8_pair_row_major_b_needs_256_wide_tiles(gpu, oracle, m, n, k):
    """B row-major (n contiguous) is staged in 128-column chunks, one per CTA: tile_n 256."""
    for a_rm in (1, 0):
        P = W.int8_problem(m, n, k, a_rm, 1, 1, pad=0, seed=7 * m + n)
        st, D = run_int8_gpu(P, alpha=1, beta=1, pair=True, tile_n=256)
        assert st == c.Status.kSuccess, _capi.last_error()
        _assert_pair()
        assert np.array_equal(D, run_int8_oracle(oracle, P, alpha=1, beta=1))
        # any other width falls back to one CTA per tile
        st, D = run_int8_gpu(P, alpha=1, beta=1, pair=True, tile_n=128)
        assert st == c.Status.kSuccess, _capi.last_error()
        _assert_pair(0)
        assert np.array_equal(D, run_int8_oracle(oracle, P, alpha=1, beta=1))


@pytest.mark.parametrize("tile_n", [64, 96, 128, 160, 192, 224, 256])
def test_int8_pair_every_tile_width_and_split_k(gpu, oracle, tile_n):
    P = W.int8_problem(520, 600, 2048, 1, 0, 1, seed=tile_n)
    want = run_int8_oracle(oracle, P, alpha=1, beta=1)
    for split in (1, 3):
        st, D = run_int8_gpu(P, alpha=1, beta=1, pair=True, tile_n=tile_n, split=split)
        assert st == c.Status.kSuccess, _capi.last_error()
        _assert_pair()
        assert _capi.last_plan().slices == split
        assert np.array_equal(D, want)


def test_int8_pair_chain(gpu, oracle):
    m, n, k = 700, 520, 640
    P = W.int8_problem(m, n, k, 1, 0, 1, seed=5)
    r = W.rng_for(5, 4)
    bias = r.integers(-(1 << 15), 1 << 15, size=n, dtype=np.int32)
    rows = r.integers(-3, 4, size=m, dtype=np.int32)
    chain = [c.BiasAdd(bias), c.ScalePerRow(rows), c.Relu(), c.Clamp(0, 1 << 20)]
    ops = [(OP_BIAS_ADD, bias, 0, 0), (OP_SCALE_PER_ROW, rows, 0, 0), (OP_RELU, None, 0, 0),
           (OP_CLAMP, None, 0, 1 << 20)]
    st, D = run_int8_gpu(P, alpha=1, beta=0, chain=chain, pair=True)
    assert st == c.Status.kSuccess, _capi.last_error()
    _assert_pair()
    assert np.array_equal(D, run_int8_oracle(oracle, P, alpha=1, beta=0, ops=ops))


@pytest.mark.parametrize("fmt", [FMT_E4M3, FMT_E5M2, FMT_E2M1])
@pytest.mark.parametrize("m,n,k", [(256, 224, 128), (300, 500, 1000), (513, 450, 4096), (129, 33, 70)])
def test_mx_pair_matches_oracle_and_single_cta_bits(gpu, oracle, fmt, m, n, k):
    for c_rm, beta in ((True, 0.5), (False, 0.0)):
        P = W.mx_problem(fmt, m, n, k, c_rm, pad=3, seed=m * 131 + n * 17 + k)
        st, D = run_mx_gpu(P, 1.0, beta, pair=True)
        assert st == c.Status.kSuccess, _capi.last_error()
        _assert_pair()
        check_mx(oracle, P, D, 1.0, beta)
        st, D1 = run_mx_gpu(P, 1.0, beta, pair=False)
        assert st == c.Status.kSuccess, _capi.last_error()
        _assert_pair(0)
        G, G1 = gather(D, m, n, P.ldc, c_rm), gather(D1, m, n, P.ldc, c_rm)
        assert np.array_equal(G.view(np.uint32), G1.view(np.uint32))


@pytest.mark.parametrize("tile_n", [64, 128, 192, 224, 256])
def test_mx_pair_tile_widths_and_split_k(gpu, oracle, tile_n):
    P = W.mx_problem(FMT_E4M3, 400, 520, 2048, True, seed=tile_n)
    for split in (1, 2):
        st, D = run_mx_gpu(P, 1.0, 0.5, pair=True, tile_n=tile_n, split=split)
        assert st == c.Status.kSuccess, _capi.last_error()
        _assert_pair()
        ref = run_mx_oracle(oracle, P, 1.0, 0.5, slices=1)
        G, R = gather(D, P.m, P.n, P.ldc, True), gather(ref, P.m, P.n, P.ldc, True)
        assert np.linalg.norm(G.astype(np.float64) - R) <= 1e-5 * np.linalg.norm(R)


def _int8_on_device(P, **kw):
    """The whole problem resident on the device: one kernel launch, no host row panels."""
    import torch
    dev = torch.device("cuda", 0)
    bufs = {name: torch.from_numpy(getattr(P, name)).to(dev) for name in ("A", "B", "C")}
    bufs["D"] = torch.full((P.C.size,), -(1 << 31), device=dev, dtype=torch.int32)
    st, _ = run_int8_gpu(P, bufs=bufs, **kw)
    return st, bufs["D"].cpu().numpy()


@pytest.mark.parametrize("pair", [False, True])
def test_narrow_last_column_over_several_rounds(gpu, oracle, pair):
    """More tiles than workers and a ragged last tile column: that column is computed at
    its own width and its tiles are dealt to the late work slots.  Every tile must still be
    computed exactly once: int8 bit-exact, MX within the tolerance."""
    m, n, k = 4096, 1300, 256            # 256-wide tiles: five full columns + one of 20
    P = W.int8_problem(m, n, k, 1, 0, 1, pad=4, seed=91)
    st, D = _int8_on_device(P, alpha=2, beta=1, pair=pair, tile_n=256)
    assert st == c.Status.kSuccess, _capi.last_error()
    _assert_pair(1 if pair else 0)
    plan = _capi.last_plan()
    assert plan.narrow_last == 1 and plan.grid == 148      # 192 (96) tiles on 148 CTAs (74 pairs)
    want = run_int8_oracle(oracle, P, alpha=2, beta=1)
    assert np.array_equal(gather(D, m, n, P.ldc, 1), gather(want, m, n, P.ldc, 1))
    Q = W.mx_problem(FMT_E4M3, m, 1100, 512, True, pad=0, seed=92)
    st, D = run_mx_gpu(Q, 1.0, 0.5, pair=pair, tile_n=192)           # five full columns + 140 -> 160 wide
    assert st == c.Status.kSuccess, _capi.last_error()
    _assert_pair(1 if pair else 0)
    assert _capi.last_plan().narrow_last == 1
    check_mx(oracle, Q, D, 1.0, 0.5)


def test_epilogue_warp_count_follows_the_launch_shape(gpu, oracle):
    """Eight epilogue warps when no CTA gets a second tile or the k loop is short, four
    otherwise; both forms must give the oracle's bits."""
    for (m, n, k), want_warps in (((1024, 1024, 512), 8),      # 32 tiles on 148 SMs: a single wave
                                  ((4096, 2048, 512), 8),      # several waves, 4 k-blocks per tile
                                  ((4096, 2048, 4096), 4)):    # several waves, 32 k-blocks per tile
        P = W.int8_problem(m, n, k, 1, 0, 1, seed=m + k)
        st, D = _int8_on_device(P, alpha=1, beta=1, tile_n=256)
        assert st == c.Status.kSuccess, _capi.last_error()
        assert _capi.last_plan().epilogue_warps == want_warps, (m, n, k)
        assert np.array_equal(D, run_int8_oracle(oracle, P, alpha=1, beta=1))
