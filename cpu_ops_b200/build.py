"""Builds ``libcpu_ops_b200.so`` in-tree with nvcc for sm_100a.

``python -m cpu_ops_b200.build`` cross-compiles without a GPU.  The library is
kept next to the package (not installed) so that the file that is loaded is
the one that was built from this tree.
"""
from __future__ import annotations

import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OUT = PKG_DIR / "libcpu_ops_b200.so"
# The same sources with -DCPUOPS_B200_INSTRUMENT: per-role cycle counters in the GEMM kernel,
# launch-policy overrides read from CPUOPS_B200_* environment variables, and the exports
# the launch-policy tests call.  Never loaded by the package itself.
OUT_INSTRUMENT = PKG_DIR / "libcpu_ops_b200_instrument.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared",
]


def sources():
    return sorted(CSRC.glob("*.cu"))


def needs_build(out: Path = OUT) -> bool:
    if not out.exists():
        return True
    newest = max(p.stat().st_mtime for p in list(CSRC.glob("*")) +
                 [PKG_DIR.parent / "include" / "cpu_ops_b200.h"])
    return out.stat().st_mtime < newest


def build(force: bool = False, verbose: bool = False, instrument: bool = False) -> Path:
    out = OUT_INSTRUMENT if instrument else OUT
    if not force and not needs_build(out):
        return out
    cmd = ["nvcc", *NVCC_FLAGS, *(["-DCPUOPS_B200_INSTRUMENT"] if instrument else []),
           *(["-Xptxas", "-v"] if verbose else []), "-o", str(out), *map(str, sources()), "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv,
                instrument="--instrument" in sys.argv))
