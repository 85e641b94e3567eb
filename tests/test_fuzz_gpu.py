"""Seeded random sweep over shapes, layouts, paddings, tiles, split-k and both kernel
forms, against the CPU oracle: int8 bit-exact, MX within the normwise tolerance.  The
sweep exists to reach combinations the hand-written cases do not name (tails in every
dimension at once, TMA-unaligned leading dimensions with the CTA-pair kernel, ...)."""
import numpy as np
import pytest

import cpu_ops_b200 as c
from cpu_ops_b200 import _capi, workloads as W
from oracle.loader import FMT_E2M1, FMT_E4M3, FMT_E5M2
from tests.gpu_helpers import MX_TOL, gather, normwise, run_int8_gpu, run_int8_oracle, run_mx_gpu, run_mx_oracle

pytestmark = pytest.mark.gpu


def _dims(r, big):
    hi = 900 if big else 300
    return int(r.integers(1, hi)), int(r.integers(1, hi)), int(r.integers(1, 1500))


@pytest.mark.parametrize("seed", range(6))
def test_int8_random_configurations(gpu, oracle, seed):
    r = np.random.default_rng(1000 + seed)
    for case in range(10):
        m, n, k = _dims(r, case % 3 == 0)
        a_rm, b_rm, c_rm = (bool(x) for x in r.integers(0, 2, 3))
        pad = int(r.choice([0, 0, 1, 3, 4, 16]))
        alpha, beta = int(r.integers(-3, 4)), int(r.choice([0, 1, -2]))
        split = int(r.choice([0, 0, 1, 2, 5]))
        pair = [None, True, False][int(r.integers(0, 3))]
        tile_n = int(r.choice([0, 0, 0, 64, 128, 256]))
        if tile_n and not b_rm and r.integers(0, 2):
            tile_n = int(r.choice([96, 160, 224]))  # odd widths need k-contiguous B
        if b_rm and tile_n not in (0, 128, 256):
            tile_n = 0
        if m <= 64:
            tile_n = 0  # operands are swapped: the forced width would apply to the other operand's layout
        P = W.int8_problem(m, n, k, a_rm, b_rm, c_rm, pad=pad, seed=seed * 100 + case)
        relu = bool(r.integers(0, 2))
        st, D = run_int8_gpu(P, alpha=alpha, beta=beta, split=split, tile_n=tile_n, pair=pair, relu=relu)
        tag = (m, n, k, a_rm, b_rm, c_rm, pad, alpha, beta, split, pair, tile_n, relu)
        assert st == c.Status.kSuccess, (tag, _capi.last_error())
        want = run_int8_oracle(oracle, P, alpha=alpha, beta=beta, relu=relu)
        assert np.array_equal(gather(D, m, n, P.ldc, c_rm), gather(want, m, n, P.ldc, c_rm)), tag


@pytest.mark.parametrize("seed", range(6))
def test_mx_random_configurations(gpu, oracle, seed):
    r = np.random.default_rng(2000 + seed)
    fmts = [FMT_E4M3, FMT_E5M2, FMT_E2M1]
    for case in range(6):
        m, n, k = _dims(r, case % 3 == 0)
        fa, fb = fmts[int(r.integers(0, 3))], fmts[int(r.integers(0, 3))]
        c_rm = bool(r.integers(0, 2))
        pad = int(r.choice([0, 0, 3, 16]))
        alpha, beta = float(r.choice([1.0, 0.5, -2.0])), float(r.choice([0.0, 0.5, -1.0]))
        split = int(r.choice([0, 0, 1, 3]))
        pair = [None, True, False][int(r.integers(0, 3))]
        tile_n = int(r.choice([0, 0, 0, 64, 128, 192, 224]))
        P = W.mx_problem(fa, m, n, k, c_rm, pad=pad, seed=seed * 100 + case, fmt_b=fb)
        st, D = run_mx_gpu(P, alpha, beta, split=split, tile_n=tile_n, pair=pair)
        tag = (m, n, k, fa, fb, c_rm, pad, alpha, beta, split, pair, tile_n)
        assert st == c.Status.kSuccess, (tag, _capi.last_error())
        ref = run_mx_oracle(oracle, P, alpha, beta)
        G, R = gather(D, m, n, P.ldc, c_rm), gather(ref, m, n, P.ldc, c_rm)
        assert not np.isnan(G).any(), tag
        assert normwise(G, R) <= MX_TOL, (tag, normwise(G, R))
