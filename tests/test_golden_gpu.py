"""The CUDA path against the committed golden fixtures (inputs + outputs of the
unmodified reference, tests/golden/make_golden.py): int8 bit for bit, MX within
1e-5 normwise of the reference's f32 result."""
import numpy as np
import pytest

import cpu_ops_b200 as c
from cpu_ops_b200 import _capi, workloads as W
from tests import golden_io
from tests.gpu_helpers import MX_TOL, gather, normwise, run_int8_gpu, run_mx_gpu

pytestmark = pytest.mark.gpu


def test_int8_golden(gpu):
    cases, z = golden_io.int8_cases()
    for cs in cases:
        lay = cs["layouts"]
        P = W.Int8Problem(cs["m"], cs["n"], cs["k"], bool(lay & 1), bool(lay & 2), bool(lay & 4),
                          cs["lda"], cs["ldb"], cs["ldc"], cs["A"], cs["B"], cs["C"])
        st, D = run_int8_gpu(P, cs["alpha"], cs["beta"], bool(cs["relu"]), split=cs["split"])
        assert st == c.Status.kSuccess, _capi.last_error()
        assert np.array_equal(D, cs["D"]), (cs["m"], cs["n"], cs["k"], lay)
    m, n, k = (int(x) for x in z["chain_shape"])
    P = W.Int8Problem(m, n, k, True, True, True, k, n, n, z["chain_A"], z["chain_B"], z["chain_C"])
    for split in (0, 3):
        st, D = run_int8_gpu(P, 1, 0, chain=[c.BiasAdd(z["chain_bias"]), c.Relu(), c.Clamp(0, 1 << 20)],
                             split=split)
        assert st == c.Status.kSuccess and np.array_equal(D, z["chain_D"])


def test_mx_golden(gpu):
    cases, z = golden_io.mx_cases()
    for cs in cases:
        P = W.MxProblem(cs["m"], cs["n"], cs["k"], cs["fmt"], cs["fmt"], bool(cs["c_rm"]), cs["lda"],
                        cs["ldb"], cs["ldsa"], cs["ldsb"], cs["ldc"], cs["A"], cs["SA"], cs["B"],
                        cs["SB"], cs["C"])
        st, D = run_mx_gpu(P, cs["alpha"], cs["beta"], bool(cs["relu"]), split=cs["split"])
        assert st == c.Status.kSuccess, _capi.last_error()
        G = gather(D, P.m, P.n, P.ldc, P.c_row_major)
        R = gather(cs["D"], P.m, P.n, P.ldc, P.c_row_major)
        assert not np.isnan(G).any()
        assert normwise(G, R) <= MX_TOL, (cs["fmt"], P.m, P.n, P.k, normwise(G, R))
    m, n, k = (int(x) for x in z["ch_shape"])
    kg = (k + 31) // 32
    P = W.MxProblem(m, n, k, _capi.FMT_E4M3, _capi.FMT_E4M3, True, k, k, kg, kg, n, z["ch_A"],
                    z["ch_SA"], z["ch_B"], z["ch_SB"], z["ch_C"])
    v0, v1 = z["ch_vec0"], z["ch_vec1"]
    chains = {1: [c.BiasAdd(v0), c.Relu()], 2: [c.ScalePerRow(v0)],
              3: [c.BiasAdd(v0), c.ScalePerCol(v1), c.Clamp(-0.5, 2.0)], 4: [c.Gelu()], 5: [c.Silu()]}
    acc_scale = float(np.abs(z["ch_D1"]).max())
    for cid, chain in chains.items():
        st, D = run_mx_gpu(P, 0.01, 0.5, chain=chain)
        assert st == c.Status.kSuccess, _capi.last_error()
        want = z[f"ch_D{cid}"]
        # 1e-5 * max(1, |ref|) as in test/test_fusion.cc:89-93, plus a term for outputs
        # where the bias cancels an accumulator of the data's overall magnitude
        tol = 1e-5 * np.maximum(1.0, np.abs(want)) + 1e-6 * acc_scale
        assert np.all(np.abs(D - want) <= tol), (cid, float(np.max(np.abs(D - want) / tol)))
