"""GPU test of the prepared-B service: a decode loop registers its MX weights' scale
array once (cpuops_b200_prepare_b) and every later call with those weights reuses the
kept tile-ordered copy.  Results must be the bits of the unprepared call."""
import numpy as np
import pytest
import torch

import cpu_ops_b200 as c
from cpu_ops_b200 import _capi, workloads as W
from oracle.loader import FMT_E2M1, FMT_E4M3
from tests.gpu_helpers import STORAGE, check_mx

pytestmark = pytest.mark.gpu


def _device_args(op, P, t, D):
    return op.Arguments(c.GemmCoord(P.m, P.n, P.k), c.MxTensorRef(t["A"], t["SA"], P.lda, P.ldsa),
                        c.MxTensorRef(t["B"], t["SB"], P.ldb, P.ldsb), c.TensorRef(t["C"], P.ldc),
                        c.TensorRef(D, P.ldc), c.LinearCombination(1.0, 0.0), 0)


@pytest.mark.parametrize("fmt,m,n,k", [(FMT_E2M1, 8, 1024, 2048), (FMT_E4M3, 1, 640, 1024),
                                      (FMT_E4M3, 300, 500, 1024), (FMT_E2M1, 33, 300, 4096 + 96),
                                      (FMT_E4M3, 64, 1792, 1000), (FMT_E2M1, 1, 14336, 4096)])
def test_prepared_b_gives_the_same_bits(gpu, oracle, fmt, m, n, k):
    dev = torch.device("cuda", 0)
    P = W.mx_problem(fmt, m, n, k, True, seed=n + k)
    t = {name: torch.from_numpy(getattr(P, name)).to(dev) for name in ("A", "SA", "B", "SB", "C")}
    op = c.GemmMx(STORAGE[fmt], STORAGE[fmt])
    D0 = torch.full((P.C.size,), float("nan"), device=dev)
    assert op(_device_args(op, P, t, D0)) == c.Status.kSuccess, _capi.last_error()
    assert _capi.last_plan().prepared_b == 0
    check_mx(oracle, P, D0.cpu().numpy(), 1.0, 0.0)
    with c.PreparedB(op, _device_args(op, P, t, D0)):
        for step in range(3):  # fresh activations, same weights
            P2 = W.mx_problem(fmt, m, n, k, True, seed=1000 + step)
            t["A"].copy_(torch.from_numpy(P2.A)); t["SA"].copy_(torch.from_numpy(P2.SA))
            D1 = torch.full((P.C.size,), float("nan"), device=dev)
            assert op(_device_args(op, P, t, D1)) == c.Status.kSuccess, _capi.last_error()
            # (the small-m kernel reads the raw scales itself and has no use for a kept copy)
            plan = _capi.last_plan()
            assert plan.prepared_b == (0 if plan.decode else 1)

            # reference: the same operands with the weights not registered (other address)
            sb_copy = t["SB"].clone()
            t2 = dict(t, SB=sb_copy)
            D2 = torch.full((P.C.size,), float("nan"), device=dev)
            assert op(_device_args(op, P, t2, D2)) == c.Status.kSuccess
            assert _capi.last_plan().prepared_b == 0
            assert torch.equal(D1.view(torch.int32), D2.view(torch.int32))
    # released: the next call re-lays the scales out again
    D3 = torch.full((P.C.size,), float("nan"), device=dev)
    assert op(_device_args(op, P, t, D3)) == c.Status.kSuccess
    assert _capi.last_plan().prepared_b == 0


def test_prepare_b_rejects_bad_descriptions(gpu):
    dev = torch.device("cuda", 0)
    op = c.GemmU8S8S32()
    a = torch.zeros(64, dtype=torch.uint8, device=dev)
    args = op.Arguments(c.GemmCoord(8, 8, 8), c.TensorRef(a, 8), c.TensorRef(a, 8), c.TensorRef(a, 8),
                        c.TensorRef(a, 8), c.LinearCombination(1, 0), 0)
    with pytest.raises(RuntimeError):
        c.PreparedB(op, args)  # int8 operands carry no scales
    mx = c.GemmMxE4M3()
    host = np.zeros(64, np.uint8)
    margs = mx.Arguments(c.GemmCoord(8, 8, 32), c.MxTensorRef(a, a, 32, 1), c.MxTensorRef(a, host, 32, 1),
                         c.TensorRef(a, 8), c.TensorRef(a, 8), c.LinearCombination(1.0, 0.0), 0)
    with pytest.raises(RuntimeError):
        c.PreparedB(mx, margs)  # scales in host memory
