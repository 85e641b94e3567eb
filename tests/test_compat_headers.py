"""The C++17 drop-in headers under include/cpu_ops/.  A translation unit written
like the reference's own tests (tests/cpp/compat_call_sites.cc: positional
aggregate initialisation of Arguments, the same aliases and epilogue types) is
compiled with g++ against this repository's headers and linked with the CUDA
library.  Without a GPU: argument validation / Status codes, and the element
codecs against the reference's tables (tests/golden/format_tables.npz).  With a
GPU: the GEMM cases against exact references computed in the same program."""
import subprocess
from pathlib import Path

import numpy as np
import pytest

from tests import golden_io

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def compat_binary(lib, tmp_path_factory):
    out = tmp_path_factory.mktemp("compat") / "compat_call_sites"
    pkg = ROOT / "cpu_ops_b200"
    cmd = ["g++", "-std=c++17", "-O2", "-Wall", "-Wextra", "-Werror", f"-I{ROOT / 'include'}",
           str(ROOT / "tests" / "cpp" / "compat_call_sites.cc"), f"-L{pkg}", "-lcpu_ops_b200",
           f"-Wl,-rpath,{pkg}", "-o", str(out)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return out


def test_status_codes_through_the_cpp_headers(compat_binary, lib):
    if lib.cpuops_b200_device_count() > 0:
        pytest.skip("the no-GPU expectations apply to machines without a device")
    res = subprocess.run([str(compat_binary), "--status"], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "0 failures" in res.stdout


def test_codecs_match_the_reference_tables(compat_binary, tmp_path):
    t = golden_io.format_tables()
    xs = t["encode_inputs"].astype(np.float32)
    (tmp_path / "in.bin").write_bytes(xs.tobytes())
    res = subprocess.run([str(compat_binary), "--codecs", str(tmp_path / "in.bin"),
                          str(tmp_path / "out.bin")], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    raw = (tmp_path / "out.bin").read_bytes()
    tables = np.frombuffer(raw[: (256 + 256 + 16 + 256) * 4], dtype=np.float32)
    enc = np.frombuffer(raw[(256 + 256 + 16 + 256) * 4:], dtype=np.uint8).reshape(-1, 4)
    off = 0
    for name, count in (("e4m3", 256), ("e5m2", 256), ("e2m1", 16), ("e8m0", 256)):
        got = tables[off: off + count]
        want = t["decode_" + name]
        # NaN payloads are not part of the contract; everything else is bit-exact
        both_nan = np.isnan(got) & np.isnan(want)
        assert np.array_equal(got.view(np.uint32)[~both_nan], want.view(np.uint32)[~both_nan]), name
        off += count
    assert enc.shape[0] == xs.size
    for col, name in enumerate(("e4m3", "e5m2", "e2m1", "e8m0")):
        assert np.array_equal(enc[:, col], t["encode_" + name]), name


@pytest.mark.gpu
def test_reference_style_call_sites_on_gpu(compat_binary, gpu):
    res = subprocess.run([str(compat_binary), "--gpu"], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-4000:] + res.stderr[-2000:]
    assert "0 failures" in res.stdout
