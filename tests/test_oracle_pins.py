"""Pins the CPU oracle (oracle/quant_gemm_oracle.c) without a GPU:
  * the reference's known-answer decode values (test/test_gemm_mx.cc:38-67),
  * its encode/decode round trips (test/test_gemm_mx.cc:69-91),
  * golden inputs/outputs produced by the unmodified reference
    (tests/golden/*.npz, see tests/golden/make_golden.py),
  * live comparison with oracle/_ref where that library is present, and
  * the reference test's own double-precision bound (test/test_gemm_mx.cc:179-227).
"""
import math

import numpy as np
import pytest

from cpu_ops_b200 import workloads as W
from oracle.loader import (FMT_E2M1, FMT_E4M3, FMT_E5M2, FMT_E8M0, OP_BIAS_ADD, OP_CLAMP, OP_GELU,
                           OP_RELU, OP_SCALE_PER_COL, OP_SCALE_PER_ROW, OP_SILU)
from tests import golden_io


def test_decode_known_answers(oracle):
    d = oracle.decode
    assert d(FMT_E4M3, 0x00) == 0.0 and d(FMT_E4M3, 0x38) == 1.0 and d(FMT_E4M3, 0x7E) == 448.0
    assert math.isnan(d(FMT_E4M3, 0x7F)) and math.isnan(d(FMT_E4M3, 0xFF))
    assert d(FMT_E4M3, 0x01) == 2.0 ** -9 and d(FMT_E4M3, 0xB8) == -1.0
    assert math.copysign(1.0, d(FMT_E4M3, 0x80)) == -1.0 and d(FMT_E4M3, 0x80) == 0.0
    assert d(FMT_E5M2, 0x3C) == 1.0 and d(FMT_E5M2, 0x7B) == 57344.0
    assert d(FMT_E5M2, 0x7C) == math.inf and math.isnan(d(FMT_E5M2, 0x7D))
    assert d(FMT_E5M2, 0x01) == 2.0 ** -16
    assert [d(FMT_E2M1, c) for c in (0x0, 0x1, 0x2, 0x7, 0xF)] == [0.0, 0.5, 1.0, 6.0, -6.0]
    assert d(FMT_E8M0, 127) == 1.0 and d(FMT_E8M0, 128) == 2.0
    assert d(FMT_E8M0, 0) == 2.0 ** -127 and d(FMT_E8M0, 254) == 2.0 ** 127
    assert math.isnan(d(FMT_E8M0, 255))


@pytest.mark.parametrize("fmt,ncodes", [(FMT_E4M3, 256), (FMT_E5M2, 256), (FMT_E2M1, 16)])
def test_encode_decode_round_trip(oracle, fmt, ncodes):
    for v in range(ncodes // 2):  # non-negative half of the code space
        f = oracle.decode(fmt, v)
        if math.isnan(f) or math.isinf(f):
            continue
        assert oracle.encode(fmt, f) == v, (fmt, v, f)


def test_e8m0_round_trip(oracle):
    for e in range(-127, 128):
        assert oracle.encode(FMT_E8M0, math.ldexp(1.0, e)) == e + 127


def test_format_tables_match_reference_fixture(oracle):
    t = golden_io.format_tables()
    for name, fmt in (("e4m3", FMT_E4M3), ("e5m2", FMT_E5M2), ("e2m1", FMT_E2M1), ("e8m0", FMT_E8M0)):
        got = oracle.decode_table(fmt) if fmt != FMT_E8M0 else np.array(
            [oracle.decode(fmt, c) for c in range(256)], dtype=np.float32)
        assert np.array_equal(got.view(np.uint32), t["decode_" + name].view(np.uint32)), name
        enc = np.array([oracle.encode(fmt, float(x)) for x in t["encode_inputs"]], dtype=np.uint8)
        assert np.array_equal(enc, t["encode_" + name]), name


def test_int8_golden(oracle):
    cases, z = golden_io.int8_cases()
    assert len(cases) >= 6
    for cs in cases:
        lay = cs["layouts"]
        a_rm, b_rm, c_rm = bool(lay & 1), bool(lay & 2), bool(lay & 4)
        D = np.full_like(cs["C"], np.iinfo(np.int32).min)
        st = oracle.gemm_u8s8s32(cs["m"], cs["n"], cs["k"], cs["A"], cs["lda"], a_rm, cs["B"],
                                 cs["ldb"], b_rm, cs["C"], cs["ldc"], D, cs["ldc"], c_rm,
                                 cs["alpha"], cs["beta"], cs["relu"])
        assert st == 0
        assert np.array_equal(D, cs["D"]), (cs["m"], cs["n"], cs["k"], lay)
    m, n, k = (int(x) for x in z["chain_shape"])
    D = np.zeros_like(z["chain_C"])
    ops = [(OP_BIAS_ADD, z["chain_bias"], 0, 0), (OP_RELU, None, 0, 0), (OP_CLAMP, None, 0, 1 << 20)]
    oracle.gemm_u8s8s32(m, n, k, z["chain_A"], k, True, z["chain_B"], n, True, z["chain_C"], n, D, n,
                        True, 1, 0, 0, ops)
    assert np.array_equal(D, z["chain_D"])


def test_mx_golden_bit_exact(oracle):
    """The oracle reproduces the reference's f32 results bit for bit when given
    the reference's KC and slice count."""
    cases, z = golden_io.mx_cases()
    assert len(cases) >= 8
    for cs in cases:
        m, n, k = cs["m"], cs["n"], cs["k"]
        slices = oracle.resolve_k_slices(m, n, k, golden_io.GOLDEN_KC, cs["split"],
                                         golden_io.GOLDEN_THREADS)
        D = np.full_like(cs["C"], np.nan)
        st = oracle.gemm_mx(m, n, k, cs["fmt"], cs["A"], cs["SA"], cs["lda"], cs["ldsa"], cs["fmt"],
                            cs["B"], cs["SB"], cs["ldb"], cs["ldsb"], cs["C"], cs["ldc"], D,
                            cs["ldc"], bool(cs["c_rm"]), cs["alpha"], cs["beta"], cs["relu"], (),
                            golden_io.GOLDEN_KC, slices)
        assert st == 0
        assert np.array_equal(D.view(np.uint32), cs["D"].view(np.uint32)), (cs["fmt"], m, n, k)


def test_mx_chain_golden(oracle):
    _, z = golden_io.mx_cases()
    m, n, k = (int(x) for x in z["ch_shape"])
    kg = (k + 31) // 32
    v0, v1 = z["ch_vec0"], z["ch_vec1"]
    chains = {
        1: [(OP_BIAS_ADD, v0, 0, 0), (OP_RELU, None, 0, 0)],
        2: [(OP_SCALE_PER_ROW, v0, 0, 0)],
        3: [(OP_BIAS_ADD, v0, 0, 0), (OP_SCALE_PER_COL, v1, 0, 0), (OP_CLAMP, None, -0.5, 2.0)],
        4: [(OP_GELU, None, 0, 0)],
        5: [(OP_SILU, None, 0, 0)],
    }
    for cid, ops in chains.items():
        D = np.full_like(z["ch_C"], np.nan)
        oracle.gemm_mx(m, n, k, FMT_E4M3, z["ch_A"], z["ch_SA"], k, kg, FMT_E4M3, z["ch_B"],
                       z["ch_SB"], k, kg, z["ch_C"], n, D, n, True, 0.01, 0.5, 0, ops,
                       golden_io.GOLDEN_KC, 1)
        want = z[f"ch_D{cid}"]
        if cid in (4, 5):
            # the reference evaluates Gelu/Silu with a polynomial on full tiles and in
            # double precision on edge tiles (epilogue/fusion.h:43-78); the oracle uses
            # the double form everywhere: compare with a tolerance
            assert np.allclose(D, want, rtol=2e-6, atol=2e-6), cid
        else:
            assert np.array_equal(D.view(np.uint32), want.view(np.uint32)), cid


def test_oracle_meets_reference_test_bound(oracle):
    """The f32 oracle stays inside the bound the reference's own test allows
    against a double reference (test/test_gemm_mx.cc:217-226)."""
    eps = np.finfo(np.float32).eps
    for fmt, (m, n, k) in ((FMT_E4M3, (31, 17, 258)), (FMT_E5M2, (65, 63, 67)), (FMT_E2M1, (16, 6, 34))):
        P = W.mx_problem(fmt, m, n, k, True, pad=3, seed=5)
        D = np.full_like(P.C, np.nan)
        oracle.gemm_mx(m, n, k, fmt, P.A, P.SA, P.lda, P.ldsa, fmt, P.B, P.SB, P.ldb, P.ldsb, P.C,
                       P.ldc, D, P.ldc, True, 1.0, 0.25)
        want, bound = oracle.gemm_mx_f64(m, n, k, fmt, P.A, P.SA, P.lda, P.ldsa, fmt, P.B, P.SB,
                                         P.ldb, P.ldsb, P.C, P.ldc, True, 1.0, 0.25)
        got = D.reshape(m, P.ldc)[:, :n].astype(np.float64)
        allowed = 8.0 * k * eps * bound + 16.0 * eps * np.abs(want) + 1e-12
        assert np.all(np.abs(got - want) <= allowed)


def test_status_codes(oracle):
    """gemm/device/gemm.h:100-122, gemm_mx.h:79-112; test/test_gemm_mx.cc:346-372."""
    A = np.zeros(64, np.uint8); B = np.zeros(64, np.int8); C = np.zeros(64, np.int32)
    assert oracle.gemm_u8s8s32(-1, 4, 4, A, 4, 1, B, 4, 1, C, 4, C, 4, 1) == 1
    assert oracle.gemm_u8s8s32(0, 4, 4, None, 4, 1, None, 4, 1, None, 4, None, 4, 1) == 0
    assert oracle.gemm_u8s8s32(4, 4, 4, None, 4, 1, B, 4, 1, C, 4, C, 4, 1) == 2
    assert oracle.gemm_u8s8s32(4, 4, 4, A, 3, 1, B, 4, 1, C, 4, C, 4, 1) == 2
    data = np.zeros(64, np.uint8); sc = np.full(8, 127, np.uint8); c = np.zeros(64, np.float32)
    ok = oracle.gemm_mx(4, 4, 32, FMT_E2M1, data, sc, 32, 1, FMT_E2M1, data, sc, 32, 1, c, 4, c, 4)
    assert ok == 0
    assert oracle.gemm_mx(4, 4, 32, FMT_E2M1, data, None, 32, 1, FMT_E2M1, data, sc, 32, 1, c, 4, c, 4) == 2
    assert oracle.gemm_mx(4, 4, 32, FMT_E2M1, data, sc, 33, 1, FMT_E2M1, data, sc, 32, 1, c, 4, c, 4) == 2
    assert oracle.gemm_mx(-1, 4, 32, FMT_E2M1, data, sc, 32, 1, FMT_E2M1, data, sc, 32, 1, c, 4, c, 4) == 1


# ---- live comparison with the real reference, where oracle/_ref exists ----------

def test_live_int8_matches_reference(oracle, reference):
    for (m, n, k) in [(5, 7, 9), (65, 63, 67), (17, 31, 257)]:
        for lay in range(8):
            a_rm, b_rm, c_rm = bool(lay & 1), bool(lay & 2), bool(lay & 4)
            P = W.int8_problem(m, n, k, a_rm, b_rm, c_rm, pad=3, seed=lay + m)
            D1 = np.zeros_like(P.C); D2 = np.zeros_like(P.C)
            for alpha, beta, relu in ((1, 0, 0), (3, -2, 0), (70001, 12345, 1)):
                oracle.gemm_u8s8s32(m, n, k, P.A, P.lda, a_rm, P.B, P.ldb, b_rm, P.C, P.ldc, D1,
                                    P.ldc, c_rm, alpha, beta, relu)
                reference.gemm_u8s8s32(m, n, k, P.A, P.lda, a_rm, P.B, P.ldb, b_rm, P.C, P.ldc, D2,
                                       P.ldc, c_rm, alpha, beta, bool(relu), 0, 0)
                assert np.array_equal(D1, D2)


def test_live_mx_matches_reference_bit_for_bit(oracle, reference):
    kc = reference.mx_kc
    threads = min(8, reference.pool_threads)
    for fmt in (FMT_E4M3, FMT_E5M2, FMT_E2M1):
        for (m, n, k, split) in [(5, 7, 96, 0), (16, 6, 34, 0), (31, 17, 258, 0), (8, 8, 2050, 3),
                                 (32, 32, 4608, 0)]:
            P = W.mx_problem(fmt, m, n, k, True, pad=3, seed=fmt * 7 + m)
            D1 = np.full_like(P.C, np.nan); D2 = np.full_like(P.C, np.nan)
            slices = oracle.resolve_k_slices(m, n, k, kc, split, threads)
            oracle.gemm_mx(m, n, k, fmt, P.A, P.SA, P.lda, P.ldsa, fmt, P.B, P.SB, P.ldb, P.ldsb,
                           P.C, P.ldc, D1, P.ldc, True, 1.25, 0.5, 0, (), kc, slices)
            reference.gemm_mx(m, n, k, fmt, P.A, P.SA, P.lda, P.ldsa, fmt, P.B, P.SB, P.ldb, P.ldsb,
                              P.C, P.ldc, D2, P.ldc, True, 1.25, 0.5, False, split, threads)
            assert np.array_equal(D1.view(np.uint32), D2.view(np.uint32)), (fmt, m, n, k, split)
