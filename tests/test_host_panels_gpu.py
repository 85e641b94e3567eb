"""GPU parity of the host-operand path for large m: the library stages the B side
once and runs the output rows as panels on three streams so that uploads, GEMMs and
downloads overlap.  The panels must be invisible in the result: bit-exact for int8,
and for MX the very bits the device-resident (unsplit) call produces."""
import numpy as np
import pytest
import torch

import cpu_ops_b200 as c
from cpu_ops_b200 import _capi, workloads as W
from oracle.loader import FMT_E2M1, FMT_E4M3, OP_BIAS_ADD, OP_CLAMP, OP_RELU, OP_SCALE_PER_ROW
from tests.gpu_helpers import (MX_TOL, STORAGE, check_mx, gather, layout, run_int8_gpu,
                               run_int8_oracle, run_mx_gpu, run_mx_oracle)

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("lay", [(1, 1, 1), (0, 1, 0), (1, 0, 0), (0, 0, 1)])
def test_int8_panels_all_layouts_ragged_last_panel(gpu, oracle, lay):
    """m = 1100 gives panels of 640 + 460 rows; padded leading dimensions."""
    a_rm, b_rm, c_rm = lay
    P = W.int8_problem(1100, 200, 300, a_rm, b_rm, c_rm, pad=5, seed=71)
    st, D = run_int8_gpu(P, alpha=2, beta=-1)
    assert st == c.Status.kSuccess, _capi.last_error()
    want = run_int8_oracle(oracle, P, alpha=2, beta=-1)
    assert np.array_equal(gather(D, P.m, P.n, P.ldc, c_rm), gather(want, P.m, P.n, P.ldc, c_rm))


def test_int8_panels_chain_with_host_vectors(gpu, oracle):
    m, n, k = 2048 + 64, 256, 512
    P = W.int8_problem(m, n, k, seed=72)
    r = W.rng_for(72, 5)
    bias = r.integers(-(1 << 15), 1 << 15, size=n, dtype=np.int32)
    rows = r.integers(-3, 4, size=m, dtype=np.int32)
    chain = [c.BiasAdd(bias), c.ScalePerRow(rows), c.Relu(), c.Clamp(0, 1 << 20)]
    ops = [(OP_BIAS_ADD, bias, 0, 0), (OP_SCALE_PER_ROW, rows, 0, 0), (OP_RELU, None, 0, 0),
           (OP_CLAMP, None, 0, 1 << 20)]
    st, D = run_int8_gpu(P, alpha=1, beta=0, chain=chain)
    assert st == c.Status.kSuccess, _capi.last_error()
    want = run_int8_oracle(oracle, P, alpha=1, beta=0, ops=ops)
    assert np.array_equal(D, want)


@pytest.mark.parametrize("fmt,c_rm", [(FMT_E4M3, True), (FMT_E4M3, False), (FMT_E2M1, True)])
def test_mx_panels_match_oracle_and_device_call_bits(gpu, oracle, fmt, c_rm):
    m, n, k = 1536 + 100, 320, 1024
    P = W.mx_problem(fmt, m, n, k, c_rm, pad=3, seed=73)
    alpha, beta = 1.0, 0.5
    st, D = run_mx_gpu(P, alpha, beta)                      # host operands: panels
    assert st == c.Status.kSuccess, _capi.last_error()
    check_mx(oracle, P, D, alpha, beta)
    # the same problem with every operand resident on the device: one unsplit call
    dev = torch.device("cuda", 0)
    t = {name: torch.from_numpy(getattr(P, name)).to(dev) for name in ("A", "SA", "B", "SB", "C")}
    Dd = torch.full((P.C.size,), float("nan"), device=dev, dtype=torch.float32)
    op = c.GemmMx(STORAGE[P.fmt_a], STORAGE[P.fmt_b], layout(c_rm))
    args = op.Arguments(c.GemmCoord(m, n, k), c.MxTensorRef(t["A"], t["SA"], P.lda, P.ldsa),
                        c.MxTensorRef(t["B"], t["SB"], P.ldb, P.ldsb), c.TensorRef(t["C"], P.ldc),
                        c.TensorRef(Dd, P.ldc), c.LinearCombination(alpha, beta), 0)
    assert op(args) == c.Status.kSuccess, _capi.last_error()
    G = gather(D, m, n, P.ldc, c_rm)
    Gd = gather(Dd.cpu().numpy(), m, n, P.ldc, c_rm)
    assert np.array_equal(G.view(np.uint32), Gd.view(np.uint32))


def test_mx_panels_leave_padding_untouched(gpu, oracle):
    """Bytes of D between the rows (ld > n) keep their poison."""
    m, n, k = 1280, 130, 256
    P = W.mx_problem(FMT_E4M3, m, n, k, True, pad=6, seed=74)
    st, D = run_mx_gpu(P, 1.0, 0.0)
    assert st == c.Status.kSuccess, _capi.last_error()
    full = D[: (m - 1) * P.ldc + n].copy()
    pad = np.ones(full.size, bool)
    ii, jj = np.meshgrid(np.arange(m), np.arange(n), indexing="ij")
    pad[(ii * P.ldc + jj).ravel()] = False
    assert np.isnan(full[pad]).all()
    assert not np.isnan(full[~pad]).any()
