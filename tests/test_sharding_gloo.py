"""The N > 1 host path on CPU: two gloo ranks each own a row block of the
output (computed here by the CPU oracle in place of the GPU), assemble the
replicated D with sharding.all_gather_rows, and must reproduce the unsharded
result bit for bit."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist
    from cpu_ops_b200 import _capi, sharding, workloads as W
    from oracle.loader import Oracle

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    o = Oracle()
    m, n, k = 300, 48, 96          # 3 tiles of 128 rows -> blocks of 256 and 44 rows
    P = W.mx_problem(_capi.FMT_E4M3, m, n, k, True, seed=77)
    sh = sharding.shard_rows(m, world, rank)
    r0, rn = sh.row_begin, sh.row_count
    D_local = np.zeros((rn, n), np.float32)
    if rn:
        o.gemm_mx(rn, n, k, P.fmt_a, P.A[r0 * P.lda:], P.SA[r0 * P.ldsa:], P.lda, P.ldsa, P.fmt_b,
                  P.B, P.SB, P.ldb, P.ldsb, P.C[r0 * P.ldc:], P.ldc, D_local, n, True, 1.0, 0.5)
    full = sharding.all_gather_rows(torch.from_numpy(D_local), m)
    want = np.zeros((m, n), np.float32)
    o.gemm_mx(m, n, k, P.fmt_a, P.A, P.SA, P.lda, P.ldsa, P.fmt_b, P.B, P.SB, P.ldb, P.ldsb, P.C,
              P.ldc, want, n, True, 1.0, 0.5)
    ok = np.array_equal(full.numpy().view(np.uint32), want.view(np.uint32))
    Path(out_dir, f"rank{rank}.ok").write_text("1" if ok else "0")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_row_sharded_gemm_two_ranks(tmp_path):
    import torch.multiprocessing as mp
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "rank0.ok").read_text() == "1"
    assert (tmp_path / "rank1.ok").read_text() == "1"
