"""Runtime behaviour around the kernels, on a device: the bounded-wait failure path (made to
run out without faulting anything), per-stream workspaces under two streams and under CUDA
graph capture, and the current-device contract."""
import ctypes as C

import numpy as np
import pytest
import torch

import cpu_ops_b200 as c
from cpu_ops_b200 import _capi, workloads as W
from oracle.loader import FMT_E4M3
from tests.gpu_helpers import MX_TOL, normwise, run_int8_gpu, run_int8_oracle, run_mx_oracle

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_becomes_a_status_and_the_device_stays_usable(gpu, lib, oracle):
    """One warp waits 2 ms on a barrier nothing arrives on: the wait gives up, the kernel
    records its code in the device error word and returns; the host reads it, reports
    DEVICE_TIMEOUT and clears it.  Nothing traps, faults or hangs, and the next GEMM on
    the same stream is bit-exact."""
    stream = torch.cuda.Stream()
    st = lib.cpuops_b200_selftest_wait_timeout(2000, C.c_void_p(stream.cuda_stream))
    assert st == _capi.STATUS_DEVICE_TIMEOUT
    assert "timed out (code 1)" in _capi.last_error()          # kErrProducerWait
    assert c.stream_status(stream.cuda_stream) == c.Status.kSuccess   # the word was cleared
    assert lib.cpuops_b200_selftest_wait_timeout(0, None) == _capi.STATUS_INVALID_ARGUMENTS
    P = W.int8_problem(300, 260, 1024, seed=5)
    dev = {k_: torch.from_numpy(getattr(P, k_)).cuda() for k_ in ("A", "B", "C")}
    D = torch.full_like(dev["C"], -1)
    op = c.GemmU8S8S32(stream=stream.cuda_stream)
    args = op.Arguments(c.GemmCoord(P.m, P.n, P.k), c.TensorRef(dev["A"], P.lda), c.TensorRef(dev["B"], P.ldb),
                        c.TensorRef(dev["C"], P.ldc), c.TensorRef(D, P.ldc), c.LinearCombination(1, 1))
    assert op(args) == c.Status.kSuccess, _capi.last_error()
    assert np.array_equal(D.cpu().numpy(), run_int8_oracle(oracle, P, 1, 1))


def test_wait_budget_is_a_setting(gpu, lib, oracle):
    """A short (but ample) budget changes nothing for a healthy launch; 0 restores the default."""
    assert lib.cpuops_b200_set_wait_budget_us(200000) == 0
    try:
        P = W.int8_problem(512, 512, 2048, seed=6)
        st, D = run_int8_gpu(P, 1, 0)
        assert st == c.Status.kSuccess and np.array_equal(D, run_int8_oracle(oracle, P, 1, 0))
    finally:
        assert lib.cpuops_b200_set_wait_budget_us(0) == 0


def _device_int8(P):
    t = {k_: torch.from_numpy(getattr(P, k_)).cuda() for k_ in ("A", "B", "C")}
    t["D"] = torch.full_like(t["C"], -7)
    return t


def _int8_args(op, P, t, split):
    return op.Arguments(c.GemmCoord(P.m, P.n, P.k), c.TensorRef(t["A"], P.lda), c.TensorRef(t["B"], P.ldb),
                        c.TensorRef(t["C"], P.ldc), c.TensorRef(t["D"], P.ldc), c.LinearCombination(1, 1), split)


def test_two_streams_each_with_its_own_growing_workspace(gpu, oracle):
    """Asynchronous calls on two caller streams; on each stream the second call needs a
    larger workspace (more split-k slabs) than the first, so the buffer is re-allocated
    while the other stream's work is in flight."""
    small = W.int8_problem(256, 256, 4096, seed=21)      # 4 slabs of 256 KB
    large = W.int8_problem(1024, 768, 8192, seed=22)     # 8 slabs of 3 MB
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    work = []
    for s in streams:
        op = c.GemmU8S8S32(stream=s.cuda_stream, asynchronous=True, memory_space=_capi.MEM_DEVICE)
        with torch.cuda.stream(s):
            for P, split in ((small, 4), (large, 8), (small, 3)):
                t = _device_int8(P)
                assert op(_int8_args(op, P, t, split)) == c.Status.kSuccess, _capi.last_error()
                work.append((P, t))
    for s in streams:
        assert c.stream_status(s.cuda_stream) == c.Status.kSuccess, _capi.last_error()
    want = {id(small): run_int8_oracle(oracle, small, 1, 1), id(large): run_int8_oracle(oracle, large, 1, 1)}
    for P, t in work:
        assert np.array_equal(t["D"].cpu().numpy(), want[id(P)])


def test_graph_capture_and_later_workspace_growth(gpu, oracle):
    """A call that would have to allocate during stream capture is refused with a message
    and leaves the capture intact; after one eager call on the stream the same call is
    captured; a later, larger call on that stream must not free the buffer the graph uses."""
    small = W.int8_problem(256, 256, 4096, seed=31)
    large = W.int8_problem(1024, 1024, 8192, seed=32)
    s = torch.cuda.Stream()
    op = c.GemmU8S8S32(stream=s.cuda_stream, asynchronous=True, memory_space=_capi.MEM_DEVICE)
    ts, tl = _device_int8(small), _device_int8(large)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        # (a) nothing ran on this stream yet: the split-k slabs would need a fresh workspace
        with torch.cuda.graph(g, stream=s, capture_error_mode="relaxed"):
            st = op(_int8_args(op, small, ts, 4))
        assert st == c.Status.kErrorInvalidArguments and "outside stream capture" in _capi.last_error()
        # (b) once eagerly, then captured
        assert op(_int8_args(op, small, ts, 4)) == c.Status.kSuccess, _capi.last_error()
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s, capture_error_mode="relaxed"):
            assert op(_int8_args(op, small, ts, 4)) == c.Status.kSuccess, _capi.last_error()
        # (c) a larger call grows the stream's workspace; the graph's buffer must survive it
        assert op(_int8_args(op, large, tl, 8)) == c.Status.kSuccess, _capi.last_error()
        ts["D"].fill_(-7)
        g.replay()
        s.synchronize()
    assert c.stream_status(s.cuda_stream) == c.Status.kSuccess
    assert np.array_equal(ts["D"].cpu().numpy(), run_int8_oracle(oracle, small, 1, 1))
    assert np.array_equal(tl["D"].cpu().numpy(), run_int8_oracle(oracle, large, 1, 1))


def test_short_last_panel_joins_its_neighbour(gpu, oracle):
    """Host A / D with m = 2561: five panels of 640 rows would leave a last panel of one row,
    which used to be launched as a small-m problem with a different plan (a 160 ... 224 wide
    tile is not usable for an n-contiguous swapped operand).  Column-major A and B."""
    P = W.int8_problem(2561, 2240, 384, a_rm=False, b_rm=False, c_rm=True, seed=41)
    st, D = run_int8_gpu(P, alpha=1, beta=1)
    assert st == c.Status.kSuccess, _capi.last_error()
    assert np.array_equal(D, run_int8_oracle(oracle, P, 1, 1))


def test_the_callers_current_device_is_left_alone(gpu, oracle):
    """A descriptor may name a device; the calling thread's current device is unchanged
    afterwards (one device here: the call must simply not disturb it)."""
    before = torch.cuda.current_device()
    P = W.mx_problem(FMT_E4M3, 70, 200, 256, True, seed=51)
    op = c.GemmMxE4M3(device=0)
    D = np.full_like(P.C, np.nan)
    args = op.Arguments(c.GemmCoord(P.m, P.n, P.k), c.MxTensorRef(P.A, P.SA, P.lda, P.ldsa),
                        c.MxTensorRef(P.B, P.SB, P.ldb, P.ldsb), c.TensorRef(P.C, P.ldc), c.TensorRef(D, P.ldc),
                        c.LinearCombination(1.0, 0.0))
    assert op(args) == c.Status.kSuccess, _capi.last_error()
    assert torch.cuda.current_device() == before
    assert normwise(D, run_mx_oracle(oracle, P, 1.0, 0.0)) <= MX_TOL


def test_sm_limit_leaves_sms_free_and_changes_no_result(gpu, lib, oracle):
    """cpuops_b200_set_sm_limit: the persistent kernels launch at most that many CTAs (so that
    a communication kernel on another stream finds free SMs); the int8 result keeps its bits,
    the MX result stays inside the tolerance, and 0 restores the default."""
    P = W.int8_problem(2048, 2304, 1024, seed=61)          # 16 x 9 tiles: more than any limit below
    Q = W.mx_problem(FMT_E4M3, 1536, 2048, 2048, True, seed=62)
    want_i8 = run_int8_oracle(oracle, P, 1, 1)
    want_mx = run_mx_oracle(oracle, Q, 1.0, 0.5)
    try:
        for limit in (64, 101, 132):
            assert lib.cpuops_b200_set_sm_limit(-1, limit) == 0
            st, D = run_int8_gpu(P, 1, 1)
            assert st == c.Status.kSuccess, _capi.last_error()
            assert _capi.last_plan().grid <= limit
            assert np.array_equal(D, want_i8)
            from tests.gpu_helpers import run_mx_gpu
            st, D = run_mx_gpu(Q, 1.0, 0.5, split=1)
            assert st == c.Status.kSuccess, _capi.last_error()
            assert _capi.last_plan().grid <= limit
            assert normwise(D, want_mx) <= MX_TOL
    finally:
        assert lib.cpuops_b200_set_sm_limit(-1, 0) == 0
    st, D = run_int8_gpu(P, 1, 1)
    assert st == c.Status.kSuccess and np.array_equal(D, want_i8)
