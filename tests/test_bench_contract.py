"""The bench harness's reference arm runs on CPU only: its JSON line must carry the
keys the measurement contract asks for, on a workload small enough for a test."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

from oracle.loader import have_reference

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.skipif(not have_reference(), reason="oracle/_ref is not built")
def test_reference_arm_line_has_the_contract_keys():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "1", "--workload", "int8_2048"], capture_output=True, text=True,
                         timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["config"]["workload"] == "int8_2048"
    assert line["cpu_baseline"]["kind"] == "reference" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["value"] > 0 and line["unit"] == "TOP/s"


def test_without_a_gpu_the_product_arm_refuses_to_run():
    """No CPU fallback: bench.py's own arm needs a CUDA device."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode != 0
    assert "no CPU fallback" in (out.stderr + out.stdout)


@pytest.mark.parametrize("fmt_name", ["e4m3", "e5m2", "e2m1"])
def test_the_bench_s_own_double_reference_agrees_with_the_oracle(oracle, fmt_name):
    """bench.py checks its multi-GPU leg against a float64 reference written in numpy inside
    bench.py (it may not lean on the test-side oracle there); that reference must itself be
    the oracle's double reference, code for code, including special values."""
    import numpy as np
    sys.path.insert(0, str(ROOT))
    import bench
    from cpu_ops_b200 import _capi, workloads as W
    fmt = {"e4m3": _capi.FMT_E4M3, "e5m2": _capi.FMT_E5M2, "e2m1": _capi.FMT_E2M1}[fmt_name]
    m, n, k = 5, 7, 96
    P = W.mx_problem(fmt, m, n, k, True, scale_lo=118, scale_hi=135, seed=3, finite_only=True)
    wl = bench.Workload("mx_e5m2_16384")
    wl.fmt, wl.k, wl.alpha = fmt, k, 1.0
    per = 2 if fmt == _capi.FMT_E2M1 else 1
    got = bench.sampled_f64_reference(wl, P.A.reshape(m, k // per), P.SA.reshape(m, k // 32),
                                      P.B.reshape(n, k // per), P.SB.reshape(n, k // 32))
    want, _ = oracle.gemm_mx_f64(m, n, k, fmt, P.A, P.SA, P.lda, P.ldsa, fmt, P.B, P.SB, P.ldb, P.ldsb,
                                 np.zeros(m * n, np.float32), n, True, 1.0, 0.0)
    # (float64 sums in another order: equal to rounding of the double accumulation)
    scale = np.abs(want).max()
    assert np.all(np.abs(got - want) <= 1e-12 * scale)
    # every code of the element format decodes as the oracle decodes it
    codes = np.arange(16 if fmt == _capi.FMT_E2M1 else 256, dtype=np.uint8)
    dec = {"e4m3": oracle.lib.oracle_decode_e4m3, "e5m2": oracle.lib.oracle_decode_e5m2,
           "e2m1": oracle.lib.oracle_decode_e2m1}[fmt_name]
    ref = np.array([dec(int(c_)) for c_ in codes], dtype=np.float64)
    mine = bench._decode_f64(fmt, codes)
    finite = np.isfinite(ref)
    assert np.array_equal(mine[finite], ref[finite])


def test_roofline_bound_follows_the_arithmetic_intensity():
    sys.path.insert(0, str(ROOT))
    import bench
    peaks = {"hbm_gbs": 6450.6, "bf16_tflops": 1646.6, "bf16_tflops_sustained": 1385.7}
    r = bench.Workload("int8_2048").roofline(20e-6, peaks, "measured")
    assert r["bound"] == "hbm" and r["unit"] == "GB/s" and abs(r["intensity_ops_per_byte"] - 409.2) < 1
    r = bench.Workload("mxfp8_e4m3_4096").roofline(70e-6, peaks, "measured")
    assert r["bound"] == "tensor" and abs(r["peak"] - 3293.2) < 0.1 and r["peak_nominal"] == 4500.0
    assert abs(r["frac"] - 137438953472 / 70e-6 / 1e12 / 3293.2) < 1e-9 and "frac_sustained" in r
    r = bench.Workload("mxfp4_decode_m8").roofline(9e-6, peaks, "measured")
    assert r["bound"] == "hbm" and r["algorithmic_per_launch"] == 31671296.0
