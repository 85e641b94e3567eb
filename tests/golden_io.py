"""Readers for the fixtures written by tests/golden/make_golden.py."""
from pathlib import Path

import numpy as np

GOLDEN = Path(__file__).resolve().parent / "golden"
GOLDEN_KC = 256   # KC of the reference build (AVX2) that produced the fixtures
GOLDEN_THREADS = 8  # thread count passed to the reference when they were made


def _cases(path):
    z = np.load(path, allow_pickle=False)
    n = int(z["n_cases"])
    out = []
    for i in range(n):
        pre = f"c{i}_"
        d = {}
        for key in z.files:
            if key.startswith(pre):
                v = z[key]
                d[key[len(pre):]] = v.item() if v.ndim == 0 else v
        out.append(d)
    return out, z


def int8_cases():
    return _cases(GOLDEN / "int8_cases.npz")


def mx_cases():
    return _cases(GOLDEN / "mx_cases.npz")


def format_tables():
    return np.load(GOLDEN / "format_tables.npz")
