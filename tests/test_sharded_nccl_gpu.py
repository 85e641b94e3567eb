"""Row-block sharding on real devices: one process per GPU computes its block of D through
the C ABI, the blocks are assembled with sharding.all_gather_rows over NCCL, and the result
must be, bit for bit, what one GPU computes alone -- including uneven blocks and a rank
whose block is empty.  The MX calls fix split_k_slices = 1: the automatic slice count
depends on the number of rows a call sees, and a different number of k slices sums the f32
partial results in a different order (int8 is exact for any slice count).  Needs two or
more GPUs (skipped otherwise); plain NCCL all-gather only, no peer-memory operands reach
the kernels."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, out_dir):
    try:
        _worker_body(rank, world, port, out_dir)
    except Exception:  # noqa: BLE001 - the parent reports it
        import traceback
        Path(out_dir, f"rank{rank}.ok").write_text("exception:\n" + traceback.format_exc())
        raise


def _worker_body(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch
    import torch.distributed as dist
    import cpu_ops_b200 as c
    from cpu_ops_b200 import _capi, sharding, workloads as W
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    ok, notes = True, []
    # (kind, m, n, k): m = 700 -> 6 tiles over 2 ranks = 384 + 316 rows; m = 100 -> one tile,
    # every rank but the first owns nothing
    for kind, m, n, k in (("int8", 700, 256, 512), ("mx", 700, 384, 1024), ("int8", 100, 128, 256),
                          ("mx", 1280, 512, 2048)):
        sh = sharding.shard_rows(m, world, rank)
        r0, rn = sh.row_begin, sh.row_count
        if kind == "int8":
            P = W.int8_problem(m, n, k, seed=900 + m)
            A, B, Cm = (torch.from_numpy(x).to(dev) for x in (P.A, P.B, P.C))
            op = c.GemmU8S8S32()

            def run(lo, cnt, D):
                args = op.Arguments(c.GemmCoord(cnt, n, k), c.TensorRef(A[lo * k:], k), c.TensorRef(B, n),
                                    c.TensorRef(Cm[lo * n:], n), c.TensorRef(D, n), c.LinearCombination(2, -1))
                return op(args)
            dtype = torch.int32
        else:
            P = W.mx_problem(_capi.FMT_E4M3, m, n, k, True, seed=900 + m)
            A, SA, B, SB, Cm = (torch.from_numpy(x).to(dev) for x in (P.A, P.SA, P.B, P.SB, P.C))
            op = c.GemmMxE4M3()

            def run(lo, cnt, D):
                args = op.Arguments(c.GemmCoord(cnt, n, k), c.MxTensorRef(A[lo * P.lda:], SA[lo * P.ldsa:], P.lda, P.ldsa),
                                    c.MxTensorRef(B, SB, P.ldb, P.ldsb), c.TensorRef(Cm[lo * n:], n),
                                    c.TensorRef(D, n), c.LinearCombination(1.0, 0.5), 1)
                return op(args)
            dtype = torch.float32
        D_local = torch.zeros((rn, n), dtype=dtype, device=dev)
        alone = torch.zeros((m, n), dtype=dtype, device=dev)
        # the calls below run on the library's own stream, which is not ordered after torch's:
        # the operands and the zero fills above must have landed first
        torch.cuda.synchronize()
        if rn:
            st = run(r0, rn, D_local)
            if st != c.Status.kSuccess:
                notes.append(f"{kind} {m}x{n}x{k}: {st!r} {_capi.last_error()}")
            ok = ok and st == c.Status.kSuccess
        full = sharding.all_gather_rows(D_local, m)
        ok = ok and run(0, m, alone) == c.Status.kSuccess
        same = bool(torch.equal(full.view(torch.int32), alone.view(torch.int32)))
        if not same:
            notes.append(f"{kind} {m}x{n}x{k}: assembled D differs from the single-GPU D")
        ok = ok and same
    Path(out_dir, f"rank{rank}.ok").write_text("1" if ok else "0 " + "; ".join(notes))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_sharded_blocks_assemble_to_the_single_gpu_result(gpu, tmp_path):
    import torch
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two or more GPUs")
    import torch.multiprocessing as mp
    port = 29700 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}.ok").read_text() == "1", f"rank {r}"
