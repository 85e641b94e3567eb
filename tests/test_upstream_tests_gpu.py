"""The reference's OWN test programs, unchanged, against this repository's drop-in headers
and CUDA library.  oracle/Makefile (target upstream_tests) compiles
test/test_gemm_int8.cc and test/test_gemm_mx.cc of the reference checkout, from where they
lie, with -I include and -lcpu_ops_b200; the binaries land in oracle/_ref/ (built
artefacts, kept out of history).  They call the operators with host std::vector buffers,
leading dimensions of dim + 3, k = 1, 5, 7, 33, 67, 258 ..., all eight int8 layout
combinations and every policy / config tag the reference spells.

test_gemm_mx.cc also holds cases for the reference's lossy MX-VNNI policy (its lines
236-344 and 427-475): they compare against operands re-quantised to int8 per block.  This
library computes the exact product for every policy tag, so those cases differ from their
re-quantised expectation by the quantisation error for fp8 -- by design -- and agree for
fp4 e2m1, which re-quantises exactly.  Everything else must pass."""
import re
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

REF_DIR = Path(__file__).resolve().parent.parent / "oracle" / "_ref"


def _run(name):
    exe = REF_DIR / name
    if not exe.exists():
        pytest.skip(f"{exe} is not built: `make -C oracle upstream_tests` needs the reference checkout "
                    "(CPU_OPS_REFERENCE)")
    return subprocess.run([str(exe)], capture_output=True, text=True, timeout=1200)


def test_reference_test_gemm_int8_passes_unchanged(gpu):
    res = _run("upstream_test_gemm_int8")
    assert res.returncode == 0, res.stdout[-4000:] + res.stderr[-2000:]
    m = re.search(r"test_gemm_int8: (\d+) cases, (\d+) failures", res.stdout)
    assert m, res.stdout[-2000:]
    assert int(m.group(1)) == 501 and int(m.group(2)) == 0


def test_reference_test_gemm_mx_passes_outside_the_lossy_policy(gpu):
    res = _run("upstream_test_gemm_mx")
    m = re.search(r"test_gemm_mx: (\d+) cases, (\d+) failures", res.stdout)
    assert m, res.stdout[-2000:] + res.stderr[-2000:]
    assert int(m.group(1)) == 212
    fails = [ln for ln in res.stdout.splitlines() if ln.startswith("FAIL")]
    assert len(fails) == int(m.group(2))
    unexpected = [ln for ln in fails if not re.search(r": vnni e(4m3|5m2) ", ln)]
    assert not unexpected, "\n".join(unexpected[:20])
