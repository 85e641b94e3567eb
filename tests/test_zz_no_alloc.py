"""The allocation-free entry point, cpuops_b200_gemm_i8_noalloc.

Who needs it: a process that handed all device memory to its own pool at start-up,
or a latency-critical serving loop in which a cudaMalloc inside a library call would
stall the whole device.  The regular entry point may grow its cached workspace with
cudaMalloc; this one keeps its split-k partial sums in a fixed array inside the
library and must give the same bits.

This file is collected last on purpose: if it fails under `pytest -x`, every other
test has already run.  It also has to pass alone in a fresh process, where its first
call is the first CUDA call of the process.
"""
import numpy as np
import pytest

import cpu_ops_b200 as c
from cpu_ops_b200 import _capi, workloads as W
from oracle.loader import OP_BIAS_ADD, OP_CLAMP, OP_RELU
from tests.gpu_helpers import run_int8_oracle

pytestmark = pytest.mark.gpu


def _device_problem(m, n, k, seed, lay=7):
    import torch
    a_rm, b_rm, c_rm = bool(lay & 1), bool(lay & 2), bool(lay & 4)
    P = W.int8_problem(m, n, k, a_rm, b_rm, c_rm, seed=seed)
    dev = {name: torch.from_numpy(getattr(P, name)).cuda() for name in ("A", "B", "C")}
    return P, dev


def _run_both(P, dev, alpha, beta, chain_host, split):
    import torch
    layout = lambda rm: c.RowMajor if rm else c.ColumnMajor
    op = c.GemmU8S8S32(layout(P.a_row_major), layout(P.b_row_major), layout(P.c_row_major))
    chain = []
    keep = []
    for kind, vec, lo, hi in chain_host:
        if kind == "bias":
            t = torch.from_numpy(vec).cuda(); keep.append(t); chain.append(c.BiasAdd(t))
        elif kind == "relu":
            chain.append(c.Relu())
        elif kind == "clamp":
            chain.append(c.Clamp(lo, hi))
    epi = c.LinearCombinationFused(alpha, beta, chain)
    outs = []
    for entry in ("regular", "noalloc"):
        dD = torch.full_like(dev["C"], np.iinfo(np.int32).min)   # poison: all must be written
        args = op.Arguments(c.GemmCoord(P.m, P.n, P.k), c.TensorRef(dev["A"], P.lda),
                            c.TensorRef(dev["B"], P.ldb), c.TensorRef(dev["C"], P.ldc),
                            c.TensorRef(dD, P.ldc), epi, split)
        st = op(args) if entry == "regular" else op.call_noalloc(args)
        assert st == c.Status.kSuccess, (entry, _capi.last_error())
        outs.append(dD.cpu().numpy())
    return outs


def test_noalloc_matches_regular_entry_point_twice_in_a_row(gpu, oracle):
    # first call: all row-major, fused chain, 4 slices
    P1, dev1 = _device_problem(384, 512, 2048, seed=101)
    bias = W.rng_for(101, 9).integers(-(1 << 15), (1 << 15) + 1, size=P1.n, dtype=np.int32)
    reg, noa = _run_both(P1, dev1, 1, 1, [("bias", bias, 0, 0), ("relu", None, 0, 0),
                                           ("clamp", None, 0, 1 << 20)], split=4)
    assert np.array_equal(reg, noa)
    # ... and both are the CPU oracle's bits, so this file stands on its own
    want = run_int8_oracle(oracle, P1, 1, 1, ops=[(OP_BIAS_ADD, bias, 0, 0), (OP_RELU, None, 0, 0),
                                                  (OP_CLAMP, None, 0, 1 << 20)])
    assert np.array_equal(noa, want)
    # second call right after it: another shape and layout, more slices, so stale partial
    # sums from the first call sit in the shared scratch array and must not leak in
    P2, dev2 = _device_problem(256, 320, 4096, seed=102, lay=0b001)  # A row-, B/C column-major
    reg, noa = _run_both(P2, dev2, 3, -2, [], split=7)
    assert np.array_equal(reg, noa)
    # and the first problem again, automatic slice count
    reg, noa = _run_both(P1, dev1, 1, 0, [], split=0)
    assert np.array_equal(reg, noa)


def test_noalloc_automatic_slice_count_fits_the_array(gpu, oracle):
    """split_k_slices = 0 on a 1024 x 1024 result (4 MiB per slab): eight slices would not
    fit the 8 MiB array, two do; the automatic mode must pick what fits instead of failing."""
    P, dev = _device_problem(1024, 1024, 1024, seed=104)
    reg, noa = _run_both(P, dev, 1, 1, [], split=0)
    assert np.array_equal(reg, noa)
    assert np.array_equal(noa, run_int8_oracle(oracle, P, 1, 1))


def test_noalloc_rejects_what_it_cannot_hold(gpu):
    import torch
    # 8 slices of a 2048 x 2048 s32 result = 128 MiB of partial sums: over the limit
    P, dev = _device_problem(2048, 2048, 1024, seed=103)
    op = c.GemmU8S8S32()
    dD = torch.empty_like(dev["C"])
    args = op.Arguments(c.GemmCoord(P.m, P.n, P.k), c.TensorRef(dev["A"], P.lda),
                        c.TensorRef(dev["B"], P.ldb), c.TensorRef(dev["C"], P.ldc),
                        c.TensorRef(dD, P.ldc), c.LinearCombination(1, 0), 8)
    assert op.call_noalloc(args) == c.Status.kErrorInvalidArguments
    msg = _capi.last_error()
    assert str(_capi.NOALLOC_SCRATCH_BYTES) in msg and "scratch" in msg
    # host operands would need staging memory
    args = op.Arguments(c.GemmCoord(64, 64, 128), c.TensorRef(np.zeros(64 * 128, np.uint8), 128),
                        c.TensorRef(np.zeros(128 * 64, np.int8), 64),
                        c.TensorRef(np.zeros(64 * 64, np.int32), 64),
                        c.TensorRef(np.zeros(64 * 64, np.int32), 64), c.LinearCombination(1, 0), 2)
    assert op.call_noalloc(args) == c.Status.kErrorInvalidArguments
    assert "device pointers only" in _capi.last_error()
