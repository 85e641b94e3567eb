"""Generates tests/golden/*.npz: small seeded inputs together with the outputs
of the UNMODIFIED reference (oracle/_ref, built from the reference headers by
oracle/Makefile) on those inputs.  Run in a container that has the reference
checkout:

    make -C oracle ref && python tests/golden/make_golden.py

The fixtures pin both the C oracle (tests/test_oracle_pins.py, no GPU) and the
CUDA path (tests/test_golden_gpu.py).  Outputs are produced with the AVX2 + FMA
build of the reference (-march=x86-64-v3: KC = 256, fused multiply-add
mainloop, the arithmetic the reference documents); the `meta` entry of each
file records the ISA line and KC.  The forced-scalar build is not used here:
without FMA instructions its generic `a*b+c` mainloop rounds twice.
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from cpu_ops_b200 import _capi, workloads as W  # noqa: E402
from oracle.loader import REF_DIR, Reference  # noqa: E402

OUT = Path(__file__).resolve().parent


def main():
    ref = Reference(REF_DIR / "libcpu_ops_ref_avx2.so")
    meta = dict(isa=ref.isa, mx_kc=ref.mx_kc)

    # ---- u8 x s8 -> s32 ----------------------------------------------------------
    cases = []
    for (m, n, k, lay, alpha, beta, relu, split, full) in [
        (65, 63, 67, 7, 3, -2, 0, 0, 1), (65, 63, 67, 0, 3, -2, 0, 0, 1),
        (17, 31, 257, 5, 1, 0, 0, 0, 1), (129, 255, 97, 2, 1, 1, 1, 0, 0),
        (16, 16, 4096, 7, 1, 1, 1, 0, 1), (16, 24, 0, 7, 1, 5, 0, 0, 1),
    ]:
        a_rm, b_rm, c_rm = bool(lay & 1), bool(lay & 2), bool(lay & 4)
        P = W.int8_problem(m, n, k, a_rm, b_rm, c_rm, pad=3, seed=m * 131 + n * 17 + k,
                           full_range=bool(full))
        D = np.full_like(P.C, np.iinfo(np.int32).min)
        st = ref.gemm_u8s8s32(m, n, k, P.A, P.lda, a_rm, P.B, P.ldb, b_rm, P.C, P.ldc, D, P.ldc,
                              c_rm, alpha, beta, bool(relu), split, 8)
        assert st == 0
        cases.append(dict(m=m, n=n, k=k, layouts=lay, alpha=alpha, beta=beta, relu=relu,
                          split=split, lda=P.lda, ldb=P.ldb, ldc=P.ldc, A=P.A, B=P.B, C=P.C, D=D))
    # fused chain BiasAdd -> Relu -> Clamp, forced split
    m, n, k = 48, 64, 1100
    P = W.int8_problem(m, n, k, seed=99)
    bias = W.rng_for(99, 9).integers(-(1 << 15), (1 << 15) + 1, size=n, dtype=np.int32)
    D = np.zeros_like(P.C)
    st = ref.gemm_u8s8s32_bias_relu_clamp(m, n, k, P.A, P.lda, P.B, P.ldb, P.C, P.ldc, D, P.ldc, 1,
                                          0, bias, 0, 1 << 20, 3, 8)
    assert st == 0
    np.savez_compressed(OUT / "int8_cases.npz", n_cases=len(cases), meta=str(meta),
                        **{f"c{i}_{k_}": v for i, cs in enumerate(cases) for k_, v in cs.items()},
                        chain_A=P.A, chain_B=P.B, chain_C=P.C, chain_bias=bias, chain_D=D,
                        chain_shape=np.array([m, n, k]))

    # ---- MX ------------------------------------------------------------------------
    cases = []
    for (fmt, m, n, k, c_rm, alpha, beta, relu, split, lo, hi) in [
        (_capi.FMT_E4M3, 31, 17, 258, 1, 1.0, 0.25, 0, 0, 124, 130),
        (_capi.FMT_E4M3, 65, 63, 67, 0, 2.0, -0.5, 0, 0, 124, 130),
        (_capi.FMT_E5M2, 16, 6, 33, 1, 1.0, 0.25, 0, 0, 124, 130),
        (_capi.FMT_E5M2, 64, 64, 640, 1, 1.25, 0.5, 1, 0, 120, 134),
        (_capi.FMT_E2M1, 65, 63, 66, 1, 1.0, 0.0, 0, 0, 124, 130),
        (_capi.FMT_E2M1, 31, 17, 258, 0, 0.5, -0.5, 0, 0, 124, 130),
        (_capi.FMT_E4M3, 24, 40, 1600, 1, 1.25, 0.5, 0, 3, 122, 132),
        (_capi.FMT_E2M1, 8, 40, 4096, 1, 1.0, 0.0, 0, 0, 124, 130),
    ]:
        P = W.mx_problem(fmt, m, n, k, bool(c_rm), pad=3, scale_lo=lo, scale_hi=hi,
                         seed=m * 131 + n * 17 + k + fmt)
        D = np.full_like(P.C, np.nan)
        st = ref.gemm_mx(m, n, k, fmt, P.A, P.SA, P.lda, P.ldsa, fmt, P.B, P.SB, P.ldb, P.ldsb, P.C,
                         P.ldc, D, P.ldc, bool(c_rm), alpha, beta, bool(relu), split, 8)
        assert st == 0
        cases.append(dict(fmt=fmt, m=m, n=n, k=k, c_rm=c_rm, alpha=alpha, beta=beta, relu=relu,
                          split=split, lda=P.lda, ldb=P.ldb, ldsa=P.ldsa, ldsb=P.ldsb, ldc=P.ldc,
                          A=P.A, SA=P.SA, B=P.B, SB=P.SB, C=P.C, D=D))
    # fused float chains on the MX path (RowMajor C)
    chains = []
    m, n, k = 40, 72, 320
    P = W.mx_problem(_capi.FMT_E4M3, m, n, k, True, pad=0, seed=4242)
    r = W.rng_for(4242, 5)
    vec0 = (r.standard_normal(max(m, n)) * 4).astype(np.float32)
    vec1 = (1.0 + 0.1 * r.standard_normal(max(m, n))).astype(np.float32)
    for chain_id in (1, 2, 3, 4, 5):
        D = np.full_like(P.C, np.nan)
        st = ref.gemm_mx_chain(_capi.FMT_E4M3, chain_id, m, n, k, P.A, P.SA, P.lda, P.ldsa, P.B, P.SB,
                               P.ldb, P.ldsb, P.C, P.ldc, D, P.ldc, 0.01, 0.5, vec0, vec1, -0.5, 2.0,
                               0, 8)
        assert st == 0
        chains.append(D)
    np.savez_compressed(OUT / "mx_cases.npz", n_cases=len(cases), meta=str(meta),
                        **{f"c{i}_{k_}": v for i, cs in enumerate(cases) for k_, v in cs.items()},
                        ch_A=P.A, ch_SA=P.SA, ch_B=P.B, ch_SB=P.SB, ch_C=P.C, ch_vec0=vec0,
                        ch_vec1=vec1, ch_shape=np.array([m, n, k]),
                        **{f"ch_D{cid}": D for cid, D in zip((1, 2, 3, 4, 5), chains)})

    # ---- format tables ---------------------------------------------------------------
    tabs = {}
    for name, fmt, ncodes in (("e4m3", 2, 256), ("e5m2", 3, 256), ("e2m1", 4, 16), ("e8m0", 5, 256)):
        tabs["decode_" + name] = np.array([ref.decode(fmt, c_) for c_ in range(ncodes)],
                                          dtype=np.float32)
    xs = np.concatenate([np.linspace(-8, 8, 4001), np.linspace(-500, 500, 2001),
                         np.logspace(-12, 6, 400), -np.logspace(-12, 6, 400),
                         [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, np.inf, -np.inf, 448, 449, 464, 480,
                          57344, 61440, 65536, 1e-30, 2.0 ** -127]]).astype(np.float32)
    tabs["encode_inputs"] = xs
    for name, fmt in (("e4m3", 2), ("e5m2", 3), ("e2m1", 4), ("e8m0", 5)):
        tabs["encode_" + name] = np.array([ref.encode(fmt, float(x)) for x in xs], dtype=np.uint8)
    np.savez_compressed(OUT / "format_tables.npz", **tabs)
    for f in sorted(OUT.glob("*.npz")):
        print(f.name, f.stat().st_size)


if __name__ == "__main__":
    main()
