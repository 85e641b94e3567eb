"""GPU test of cpuops_b200_relayout_scales: row-major E8M0 scales -> the tile-ordered
512-byte atoms the tensor cores read ([32 lanes][4 row groups][4 scale blocks] per atom,
atoms ordered [tile][k-block][atom along k][128-row group]); positions outside the
matrix hold 127 (scale 1.0)."""
import ctypes as C

import numpy as np
import pytest
import torch

from cpu_ops_b200 import _capi

pytestmark = pytest.mark.gpu


def expected_layout(scales, rows, k, ld, tile_rows, bps):
    kblocks = (k + 31) // 32
    tiles = -(-rows // tile_rows)
    stages = -(-k // (bps * 32))
    nb128 = -(-tile_rows // 128)
    ka = bps // 4
    out = np.full(tiles * stages * ka * nb128 * 512, 127, np.uint8)
    for tile in range(tiles):
        for stage in range(stages):
            for a in range(ka):
                for nb in range(nb128):
                    base = ((tile * stages + stage) * (ka * nb128) + a * nb128 + nb) * 512
                    for g in range(4):
                        for lane in range(32):
                            r_in_tile = nb * 128 + g * 32 + lane
                            row = tile * tile_rows + r_in_tile
                            if r_in_tile >= tile_rows or row >= rows:
                                continue
                            for b in range(4):
                                kb = stage * bps + a * 4 + b
                                if kb < kblocks:
                                    out[base + lane * 16 + g * 4 + b] = scales[row * ld + kb]
    return out


@pytest.mark.parametrize("rows,k,pad,tile_rows,bps", [(128, 128, 0, 128, 4), (300, 1000, 3, 128, 4),
                                                     (70, 4096, 0, 224, 8), (500, 333, 5, 256, 8),
                                                     (33, 96, 1, 32, 4), (1, 4096, 0, 64, 8)])
def test_relayout_matches_the_documented_atom_layout(gpu, rows, k, pad, tile_rows, bps):
    lib = _capi.load()
    ld = (k + 31) // 32 + pad
    rng = np.random.default_rng(rows * 7 + k)
    scales = rng.integers(1, 255, size=rows * ld, dtype=np.uint8)
    nbytes = lib.cpuops_b200_scale_layout_bytes(rows, k, tile_rows, bps)
    want = expected_layout(scales, rows, k, ld, tile_rows, bps)
    assert nbytes == want.size
    dev = torch.device("cuda", 0)
    src = torch.from_numpy(scales).to(dev)
    dst = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    st = lib.cpuops_b200_relayout_scales(C.c_void_p(src.data_ptr()), rows, k, ld, tile_rows, bps,
                                         C.c_void_p(dst.data_ptr()), None)
    assert st == 0, _capi.last_error()
    assert np.array_equal(dst.cpu().numpy(), want)
