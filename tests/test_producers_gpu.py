"""GPU parity of the k-block dealing between the two TMA producer warps of the GEMM kernel.

Producer j loads the k-blocks whose running index (over all tiles of its CTA) is j modulo 2.
The cases here make that index do everything it can: several tiles per CTA with an odd
number of k-blocks each (the producers swap roles from tile to tile), split-k slices of
unequal length, a single k-block per tile, a ring shorter than four stages (one producer
only), a ragged k tail, both kernel forms.  The kernels are held to eight SMs
(cpuops_b200_set_sm_limit) so that small problems give every CTA several tiles.  int8 is
compared bit for bit with the oracle, MX within the tolerance of the other MX tests."""
import numpy as np
import pytest

import cpu_ops_b200 as c
from cpu_ops_b200 import _capi, workloads as W
from oracle.loader import FMT_E2M1, FMT_E4M3
from tests.gpu_helpers import check_mx, gather, run_int8_gpu, run_int8_oracle, run_mx_gpu

pytestmark = pytest.mark.gpu

SMS = 8  # CTAs (four pairs) the kernels may use in this file


@pytest.fixture(autouse=True)
def eight_sms(gpu):
    lib = _capi.load()
    assert lib.cpuops_b200_set_sm_limit(-1, SMS) == 0
    yield
    assert lib.cpuops_b200_set_sm_limit(-1, 0) == 0


def _int8_on_device(P, **kw):
    import torch
    dev = torch.device("cuda", 0)
    bufs = {name: torch.from_numpy(getattr(P, name)).to(dev) for name in ("A", "B", "C")}
    bufs["D"] = torch.full((P.C.size,), -(1 << 31), device=dev, dtype=torch.int32)
    st, _ = run_int8_gpu(P, bufs=bufs, **kw)
    return st, bufs["D"].cpu().numpy()


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("k", [128, 640, 896 + 33, 1920])
def test_int8_odd_k_block_counts_over_several_tiles_per_cta(gpu, oracle, pair, k):
    """768 x 1280 in 256-wide tiles: 30 (15) tiles on 8 CTAs (4 pairs), so every CTA walks
    three or four tiles; with 1, 5, 8 (one ragged) or 15 k-blocks per tile the producers'
    parities alternate between tiles in every possible way."""
    m, n = 768, 1280
    P = W.int8_problem(m, n, k, 1, 0, 1, pad=0, seed=7 + k)
    st, D = _int8_on_device(P, alpha=1, beta=1, pair=pair, tile_n=256, split=1)
    assert st == c.Status.kSuccess, _capi.last_error()
    plan = _capi.last_plan()
    assert plan.pair == (1 if pair else 0) and plan.grid == SMS and plan.slices == 1
    want = run_int8_oracle(oracle, P, alpha=1, beta=1)
    assert np.array_equal(gather(D, m, n, P.ldc, 1), gather(want, m, n, P.ldc, 1))


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("slices", [2, 3, 5])
def test_int8_uneven_split_k_ranges(gpu, oracle, pair, slices):
    """k = 13 k-blocks cut into 2, 3 or 5 slices: ranges of 7+6, 5+4+4, 3+3+3+2+2 k-blocks,
    many work items per CTA."""
    m, n, k = 512, 640, 13 * 128
    P = W.int8_problem(m, n, k, 1, 0, 1, pad=16, seed=31 + slices)
    st, D = _int8_on_device(P, alpha=2, beta=-1, pair=pair, split=slices, tile_n=128)
    assert st == c.Status.kSuccess, _capi.last_error()
    assert _capi.last_plan().slices == slices
    want = run_int8_oracle(oracle, P, alpha=2, beta=-1)
    assert np.array_equal(gather(D, m, n, P.ldc, 1), gather(want, m, n, P.ldc, 1))


@pytest.mark.parametrize("fmt", [FMT_E4M3, FMT_E2M1])
@pytest.mark.parametrize("pair", [False, True])
def test_mx_odd_k_block_counts_over_several_tiles_per_cta(gpu, oracle, fmt, pair):
    """The MX kinds carry two more loads per k-block (the scale atoms): 3 and 7 k-blocks per
    tile, three to five tiles per CTA, beta != 0."""
    per_block = 256 if fmt == FMT_E2M1 else 128
    for kb in (3, 7):
        m, n, k = 512, 1344, kb * per_block
        P = W.mx_problem(fmt, m, n, k, True, pad=0, seed=50 + kb)
        st, D = run_mx_gpu(P, 1.0, 0.5, pair=pair, tile_n=224 if pair else 128, split=1)
        assert st == c.Status.kSuccess, _capi.last_error()
        assert _capi.last_plan().pair == (1 if pair else 0)
        check_mx(oracle, P, D, 1.0, 0.5)


def test_results_do_not_depend_on_which_producer_loaded_a_k_block(gpu, oracle):
    """The same MX problem as one launch and as three forced k slices reads every k-block
    through a different producer and ring stage; int8 gives identical bits, and two runs of
    the same MX call give identical bits."""
    P = W.int8_problem(768, 1024, 11 * 128, 1, 0, 1, pad=0, seed=77)
    st, D1 = _int8_on_device(P, alpha=1, beta=0, split=1)
    assert st == c.Status.kSuccess, _capi.last_error()
    st, D3 = _int8_on_device(P, alpha=1, beta=0, split=3)
    assert st == c.Status.kSuccess, _capi.last_error()
    assert np.array_equal(D1, D3)
    Q = W.mx_problem(FMT_E4M3, 512, 1792, 9 * 128, True, pad=0, seed=78)
    st, Da = run_mx_gpu(Q, 1.0, 0.0, split=1)
    assert st == c.Status.kSuccess, _capi.last_error()
    st, Db = run_mx_gpu(Q, 1.0, 0.0, split=1)
    assert st == c.Status.kSuccess, _capi.last_error()
    assert np.array_equal(Da.view(np.uint32), Db.view(np.uint32))
    check_mx(oracle, Q, Da, 1.0, 0.0)
