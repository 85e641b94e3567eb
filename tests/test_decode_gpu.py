"""The small-m MX kernel (one launch, raw scales read by TMA, every SM streaming an equal
share of the weights, partial sums added in ascending k order) against the CPU oracle.
The reference has no kernel of its own for these shapes: its GEMV-like calls run the
general blocked path (gemm/kernel/run_blocked.h:79-174), which the oracle restates."""
import numpy as np
import pytest

import cpu_ops_b200 as c
from cpu_ops_b200 import _capi, workloads as W
from oracle.loader import FMT_E2M1, FMT_E4M3, FMT_E5M2, OP_BIAS_ADD, OP_CLAMP, OP_RELU, OP_SCALE_PER_ROW
from tests.gpu_helpers import MX_TOL, STORAGE, check_mx, gather, layout, normwise, run_mx_gpu, run_mx_oracle

pytestmark = pytest.mark.gpu


def lds16(k):
    """A scale leading dimension the kernel's TMA boxes can address (multiple of 16)."""
    return -(-((k + 31) // 32) // 16) * 16


@pytest.mark.parametrize("fmt", [FMT_E2M1, FMT_E4M3, FMT_E5M2])
@pytest.mark.parametrize("m,n,k", [(1, 128, 256), (8, 384, 1024), (32, 1000, 512), (33, 2048, 2048),
                                   (64, 640, 4096), (3, 14336 // 8, 1280), (17, 130, 544)])
def test_shapes_against_the_oracle(gpu, oracle, fmt, m, n, k):
    """Tile counts below, at and above the SM count; n not a multiple of 128; k with a
    ragged last 128-byte block and (k = 544) a ragged last 32-element scale block."""
    P = W.mx_problem(fmt, m, n, k, True, lds=lds16(k), seed=0xD0 + m + n + k)
    st, D = run_mx_gpu(P, 1.0, 0.0)
    assert st == c.Status.kSuccess, _capi.last_error()
    plan = _capi.last_plan()
    assert plan.decode == 1 and plan.swapped == 1, "the small-m kernel did not run"
    check_mx(oracle, P, D, 1.0, 0.0)
    st, D2 = run_mx_gpu(P, 1.0, 0.0)
    assert np.array_equal(D.view(np.uint32), D2.view(np.uint32)), "run-to-run bits differ"


def test_mixed_fp8_formats(gpu, oracle):
    P = W.mx_problem(FMT_E4M3, 8, 512, 1024, True, lds=32, fmt_b=FMT_E5M2, seed=5)
    st, D = run_mx_gpu(P, 0.5, 0.0)
    assert st == c.Status.kSuccess and _capi.last_plan().decode == 1
    check_mx(oracle, P, D, 0.5, 0.0)


@pytest.mark.parametrize("c_rm", [True, False])
def test_epilogue_forms(gpu, oracle, c_rm):
    """beta != 0, activation, and a chain whose vectors are indexed by the caller's column
    (the kernel's row) and by the caller's row (the kernel's column)."""
    m, n, k = 8, 1536, 2048
    P = W.mx_problem(FMT_E2M1, m, n, k, c_rm, lds=64, scale_lo=118, scale_hi=122, seed=77)
    st, D = run_mx_gpu(P, 2.0, -0.75)
    assert st == c.Status.kSuccess and _capi.last_plan().decode == 1
    check_mx(oracle, P, D, 2.0, -0.75)
    st, D = run_mx_gpu(P, 1.0, 1.0, in_place=True)
    assert st == c.Status.kSuccess
    check_mx(oracle, P, D, 1.0, 1.0)
    r = W.rng_for(9, 3)
    bias = r.standard_normal(n).astype(np.float32)
    rows = (1.0 + r.random(m)).astype(np.float32)
    chain = [c.BiasAdd(bias), c.Relu(), c.ScalePerRow(rows), c.Clamp(0.0, 3.0)]
    ops = [(OP_BIAS_ADD, bias, 0.0, 0.0), (OP_RELU, None, 0.0, 0.0), (OP_SCALE_PER_ROW, rows, 0.0, 0.0),
           (OP_CLAMP, None, 0.0, 3.0)]
    st, D = run_mx_gpu(P, 1.0, 0.5, chain=chain)
    assert st == c.Status.kSuccess and _capi.last_plan().decode == 1
    want = run_mx_oracle(oracle, P, 1.0, 0.5, ops=ops)
    G = gather(D, m, n, P.ldc, c_rm)
    R = gather(want, m, n, P.ldc, c_rm)
    assert not np.isnan(G).any()
    assert normwise(G, R) <= MX_TOL


def test_never_split_keeps_whole_tiles(gpu, oracle):
    """split_k_slices = 1: every CTA takes whole weight tiles (no partial sums)."""
    P = W.mx_problem(FMT_E2M1, 8, 14336 // 4, 4096, True, lds=128, seed=3)
    st, D = run_mx_gpu(P, 1.0, 0.0, split=1)
    assert st == c.Status.kSuccess
    plan = _capi.last_plan()
    assert plan.decode == 1 and plan.slices == 1
    want = run_mx_oracle(oracle, P, 1.0, 0.0)
    assert np.array_equal(D.view(np.uint32), want.view(np.uint32))
    st, D0 = run_mx_gpu(P, 1.0, 0.0, split=0)
    assert st == c.Status.kSuccess and _capi.last_plan().slices > 1
    # exact partial sums with these scales: cutting k changes no bit
    assert np.array_equal(D0.view(np.uint32), want.view(np.uint32))


def test_scale_arrays_tma_cannot_address_take_the_general_kernel(gpu, oracle):
    """A scale leading dimension that is not a multiple of 16 is legal (mx_formats.h:280-295
    only asks ld_scales >= ceil(k/32)); the call then runs the general kernel."""
    P = W.mx_problem(FMT_E4M3, 4, 256, 1024 + 32, True, lds=33, seed=21)
    st, D = run_mx_gpu(P, 1.0, 0.0)
    assert st == c.Status.kSuccess and _capi.last_plan().decode == 0
    check_mx(oracle, P, D, 1.0, 0.0)


def test_special_values_do_not_leak_between_rows(gpu, oracle):
    """A NaN scale on one weight row and an Inf element on one activation row poison only
    their own output column / row; rows that do not exist (m < tile width) stay out."""
    m, n, k = 5, 256, 512
    P = W.mx_problem(FMT_E5M2, m, n, k, True, lds=16, seed=31)
    P.SB[7 * P.ldsb + 3] = 0xFF          # weight row 7: NaN scale
    P.A[2 * P.lda + 100] = 0x7C          # activation row 2: +Inf
    st, D = run_mx_gpu(P, 1.0, 0.0)
    assert st == c.Status.kSuccess and _capi.last_plan().decode == 1
    want = run_mx_oracle(oracle, P, 1.0, 0.0)
    G, R = D.reshape(m, n), want.reshape(m, n)
    assert np.array_equal(np.isnan(G), np.isnan(R))
    assert np.array_equal(np.isinf(G), np.isinf(R))
    ok = np.isfinite(R)
    assert normwise(G[ok], R[ok]) <= MX_TOL


def test_device_operands_async_back_to_back(gpu, oracle):
    """Device-resident operands, asynchronous calls back to back on one stream: each call's
    CTAs may start while the call before it is still finishing.  D of one call is never an
    input of the next here, but every call rewrites the D buffer of the call three steps
    before it."""
    import torch
    m, n, k = 8, 14336 // 2, 4096
    probs = [W.mx_problem(FMT_E2M1, m, n, k, True, lds=128, seed=100 + i) for i in range(3)]
    dev = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=dev)
    op = c.GemmMx(STORAGE[FMT_E2M1], STORAGE[FMT_E2M1], layout(True), stream=stream.cuda_stream,
                  asynchronous=True, memory_space=_capi.MEM_DEVICE)
    bufs, outs = [], []
    with torch.cuda.stream(stream):
        for P in probs:
            t = {k_: torch.from_numpy(getattr(P, k_)).to(dev) for k_ in ("A", "SA", "B", "SB", "C")}
            t["D"] = torch.full((m * n,), float("nan"), device=dev)
            bufs.append(t)
        stream.synchronize()
        for rep in range(2):
            for P, t in zip(probs, bufs):
                args = op.Arguments(c.GemmCoord(m, n, k), c.MxTensorRef(t["A"], t["SA"], P.lda, P.ldsa),
                                    c.MxTensorRef(t["B"], t["SB"], P.ldb, P.ldsb), c.TensorRef(t["C"], n),
                                    c.TensorRef(t["D"], n), c.LinearCombination(1.0, 0.0))
                assert op(args) == c.Status.kSuccess, _capi.last_error()
        assert c.stream_status(stream.cuda_stream) == c.Status.kSuccess, _capi.last_error()
    assert _capi.last_plan().decode == 1
    for P, t in zip(probs, bufs):
        want = run_mx_oracle(oracle, P, 1.0, 0.0)
        assert np.array_equal(t["D"].cpu().numpy().view(np.uint32), want.view(np.uint32))


def test_a_call_may_consume_what_the_call_before_it_wrote(gpu, oracle):
    """Four calls back to back on one stream accumulate into one buffer (C = D, beta = 1):
    every call's epilogue reads what the previous call's epilogue wrote.  The kernels
    overlap at their edges (programmatic launch), so this is the ordering the device-side
    dependency wait has to provide."""
    import torch
    m, n, k = 16, 14336 // 4, 2048
    probs = [W.mx_problem(FMT_E4M3, m, n, k, True, lds=64, seed=200 + i) for i in range(4)]
    dev = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=dev)
    op = c.GemmMx(STORAGE[FMT_E4M3], STORAGE[FMT_E4M3], layout(True), stream=stream.cuda_stream,
                  asynchronous=True, memory_space=_capi.MEM_DEVICE)
    acc = torch.from_numpy(probs[0].C.copy()).to(dev)
    keep = []
    with torch.cuda.stream(stream):
        for P in probs:
            t = {k_: torch.from_numpy(getattr(P, k_)).to(dev) for k_ in ("A", "SA", "B", "SB")}
            keep.append(t)
        stream.synchronize()
        for P, t in zip(probs, keep):
            args = op.Arguments(c.GemmCoord(m, n, k), c.MxTensorRef(t["A"], t["SA"], P.lda, P.ldsa),
                                c.MxTensorRef(t["B"], t["SB"], P.ldb, P.ldsb), c.TensorRef(acc, n),
                                c.TensorRef(acc, n), c.LinearCombination(1.0, 1.0))
            assert op(args) == c.Status.kSuccess, _capi.last_error()
        assert c.stream_status(stream.cuda_stream) == c.Status.kSuccess, _capi.last_error()
    want = probs[0].C.copy()
    for P in probs:
        Q = W.MxProblem(m, n, k, P.fmt_a, P.fmt_b, True, P.lda, P.ldb, P.ldsa, P.ldsb, n, P.A, P.SA, P.B, P.SB,
                        want.copy())
        want = run_mx_oracle(oracle, Q, 1.0, 1.0)
    got = acc.cpu().numpy()
    assert not np.isnan(got).any()
    assert normwise(got, want) <= MX_TOL
