"""The C entry points are re-entrant from the caller's view, like the reference's
operator() (concurrent calls serialise inside the library, as they do on the CPU
library's pool mutex, thread_pool.h:93-96): several host threads calling at once, with
host and device operands, must each get their own correct result."""
import threading

import numpy as np
import pytest

import cpu_ops_b200 as c
from cpu_ops_b200 import _capi, workloads as W
from oracle.loader import FMT_E4M3
from tests.gpu_helpers import MX_TOL, normwise, run_int8_gpu, run_int8_oracle, run_mx_gpu, run_mx_oracle

pytestmark = pytest.mark.gpu


def test_concurrent_callers(gpu, oracle):
    errors = []

    def int8_worker(seed):
        try:
            for rep in range(4):
                P = W.int8_problem(100 + 37 * seed, 90 + 11 * rep, 256 + 64 * seed, seed=seed * 10 + rep)
                st, D = run_int8_gpu(P, alpha=1, beta=1)
                assert st == c.Status.kSuccess, _capi.last_error()
                assert np.array_equal(D, run_int8_oracle(oracle, P, alpha=1, beta=1))
        except Exception as exc:  # noqa: BLE001 - reported by the main thread
            errors.append(exc)

    def mx_worker(seed):
        try:
            for rep in range(3):
                P = W.mx_problem(FMT_E4M3, 1100 if rep == 0 else 64, 200, 512, True, seed=seed * 10 + rep)
                st, D = run_mx_gpu(P, 1.0, 0.5)   # the first shape takes the host row-panel path
                assert st == c.Status.kSuccess, _capi.last_error()
                assert normwise(D, run_mx_oracle(oracle, P, 1.0, 0.5)) <= MX_TOL
        except Exception as exc:  # noqa: BLE001
            errors.append(exc)

    threads = [threading.Thread(target=int8_worker, args=(s,)) for s in range(3)]
    threads += [threading.Thread(target=mx_worker, args=(s,)) for s in range(3)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors[0]
