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
