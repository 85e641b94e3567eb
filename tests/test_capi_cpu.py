"""Host-side checks that need no GPU: the library loads, exports every symbol
include/cpu_ops_b200.h declares, validates arguments in the reference's order
(gemm/device/gemm.h:100-122, gemm_mx.h:79-112) before touching a device, and
its host-only helpers (shard plan, scale layout size) are right."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

import cpu_ops_b200 as c
from cpu_ops_b200 import _capi, sharding

ROOT = Path(__file__).resolve().parent.parent


def test_product_library_has_no_probe_exports(lib):
    """The launch-policy probes and cycle counters exist only in the instrumented build."""
    for name in ("cpuops_b200_debug_slot_to_tile", "cpuops_b200_debug_pick_tile_width",
                 "cpuops_b200_debug_clock"):
        assert not hasattr(lib, name), name


def test_library_exports_every_declared_symbol(lib):
    header = (ROOT / "include" / "cpu_ops_b200.h").read_text()
    declared = set(re.findall(r"CPUOPS_B200_API\s+[\w\s\*]+?\b(cpuops_b200_\w+)\s*\(", header))
    assert declared, "no declarations found in the header"
    assert declared == set(_capi.EXPORTED_SYMBOLS)
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.cpuops_b200_abi_version() == 1


def test_descriptor_size_is_checked(lib):
    d = _capi.GemmDesc()
    d.struct_size = C.sizeof(_capi.GemmDesc) - 8
    assert lib.cpuops_b200_gemm(C.byref(d)) == _capi.STATUS_BAD_DESCRIPTOR
    assert lib.cpuops_b200_gemm(None) == _capi.STATUS_BAD_DESCRIPTOR


def _i8_args(op, m, n, k, lda=None, ldb=None, ldc=None, a=True, b=True, cc=True, d=True):
    A = np.zeros(max(1, m * k), np.uint8); B = np.zeros(max(1, k * n), np.int8)
    Cm = np.zeros(max(1, m * n), np.int32)
    return op.Arguments(c.GemmCoord(m, n, k), c.TensorRef(A if a else None, lda if lda is not None else k),
                        c.TensorRef(B if b else None, ldb if ldb is not None else n),
                        c.TensorRef(Cm if cc else None, ldc if ldc is not None else n),
                        c.TensorRef(Cm if d else None, ldc if ldc is not None else n)), (A, B, Cm)


def test_int8_validation_order(lib):
    op = c.GemmU8S8S32()
    args, keep = _i8_args(op, -1, 4, 4)
    assert op(args) == c.Status.kErrorInvalidProblem
    # m == 0 or n == 0 succeeds before any pointer check
    args, keep = _i8_args(op, 0, 4, 4, a=False, b=False, cc=False, d=False)
    assert op(args) == c.Status.kSuccess
    # null operands (C must be non-null even though beta == 0)
    for kw in (dict(a=False), dict(b=False), dict(cc=False), dict(d=False)):
        args, keep = _i8_args(op, 4, 4, 4, **kw)
        assert op(args) == c.Status.kErrorInvalidArguments, kw
    # leading dimensions
    for kw in (dict(lda=3), dict(ldb=3), dict(ldc=3)):
        args, keep = _i8_args(op, 4, 4, 4, **kw)
        assert op(args) == c.Status.kErrorInvalidArguments, kw
    # column-major A needs lda >= m
    opc = c.GemmU8S8S32(c.ColumnMajor, c.RowMajor, c.RowMajor)
    args, keep = _i8_args(opc, 8, 4, 4, lda=4)
    assert opc(args) == c.Status.kErrorInvalidArguments


def test_mx_validation_order(lib):
    """test/test_gemm_mx.cc:346-372."""
    op = c.GemmMxE2M1()
    data = np.zeros(64, np.uint8); scales = np.full(8, 127, np.uint8); cm = np.zeros(64, np.float32)

    def args(**kw):
        a = op.Arguments(c.GemmCoord(4, 4, 32), c.MxTensorRef(data, scales, 32, 1),
                         c.MxTensorRef(data, scales, 32, 1), c.TensorRef(cm, 4), c.TensorRef(cm, 4))
        for k_, v in kw.items():
            obj, attr = k_.split("__")
            setattr(getattr(a, obj), attr, v)
        return a

    assert op(args(ref_A__scales=None)) == c.Status.kErrorInvalidArguments
    assert op(args(ref_A__ld=33)) == c.Status.kErrorInvalidArguments      # odd fp4 ld
    assert op(args(ref_B__ld=31)) == c.Status.kErrorInvalidArguments      # ld < k
    assert op(args(ref_B__ld_scales=0)) == c.Status.kErrorInvalidArguments
    assert op(args(ref_C__ld=3)) == c.Status.kErrorInvalidArguments
    a = args(); a.problem_size = c.GemmCoord(-1, 4, 32)
    assert op(a) == c.Status.kErrorInvalidProblem
    a = args(); a.problem_size = c.GemmCoord(0, 4, 32)
    assert op(a) == c.Status.kSuccess


def test_no_device_is_reported_not_emulated(lib):
    """Without a GPU a valid problem must fail loudly (no CPU fallback)."""
    if lib.cpuops_b200_device_count() > 0:
        pytest.skip("a device is present")
    op = c.GemmU8S8S32()
    args, keep = _i8_args(op, 4, 4, 4)
    assert op(args) == c.Status.kErrorNoDevice
    assert "no CPU fallback" in _capi.last_error()


def test_shard_rows_partitions_whole_tiles():
    for m in (1, 127, 128, 129, 4096, 16384, 5000):
        for world in (1, 2, 3, 4, 8):
            plan = sharding.shard_plan(m, world)
            assert plan[0].row_begin == 0
            assert sum(s.row_count for s in plan) == m
            for a, b in zip(plan, plan[1:]):
                assert a.row_begin + a.row_count == b.row_begin
                assert b.row_begin % 128 == 0 or b.row_count == 0
            counts = [s.row_count for s in plan]
            # balanced to within one tile, plus the ragged last tile
            assert max(counts) - min(counts) < 256 or min(counts) == 0
    with pytest.raises(ValueError):
        sharding.shard_rows(16, 2, 2)


def test_scale_layout_bytes(lib):
    f = lib.cpuops_b200_scale_layout_bytes
    assert f(4096, 4096, 128, 4) == 4096 * 128        # exact fit: one byte per scale
    assert f(4096, 4096, 256, 4) == 4096 * 128
    assert f(100, 4096, 128, 4) == 128 * 128           # rows padded to the tile
    assert f(128, 33, 128, 4) == 128 * 4               # k padded to one stage of 4 blocks
    assert f(192, 256, 192, 8) == 2 * 512 * 2          # 192-row tile = two 128-row atoms, 8 blocks
    assert f(0, 10, 128, 4) == 0 and f(10, 10, 128, 5) == 0


def test_prepare_b_validates_before_touching_a_device(lib):
    """cpuops_b200_prepare_b: int8 operands carry no scales; a bad scale description
    is rejected; without a device a valid registration fails loudly."""
    handle = C.c_void_p()
    d = _capi.GemmDesc()
    d.struct_size = C.sizeof(_capi.GemmDesc)
    d.kind = _capi.KIND_I8
    assert lib.cpuops_b200_prepare_b(C.byref(d), C.byref(handle)) == _capi.STATUS_UNSUPPORTED
    d.kind = _capi.KIND_MX
    d.n, d.k, d.ld_scales_b = 8, 64, 1          # needs two scale entries per row
    scales = np.zeros(16, np.uint8)
    d.b_scales = scales.ctypes.data
    assert lib.cpuops_b200_prepare_b(C.byref(d), C.byref(handle)) == _capi.STATUS_INVALID_ARGUMENTS
    d.ld_scales_b = 2
    d.struct_size = 8
    assert lib.cpuops_b200_prepare_b(C.byref(d), C.byref(handle)) == _capi.STATUS_BAD_DESCRIPTOR
    d.struct_size = C.sizeof(_capi.GemmDesc)
    if lib.cpuops_b200_device_count() == 0:
        assert lib.cpuops_b200_prepare_b(C.byref(d), C.byref(handle)) == _capi.STATUS_NO_DEVICE
    assert lib.cpuops_b200_release_b(None) == _capi.STATUS_INVALID_ARGUMENTS


def test_last_plan_is_readable_before_any_call(lib):
    plan = _capi.Plan()
    assert lib.cpuops_b200_last_plan(C.byref(plan)) == 0
    assert lib.cpuops_b200_last_plan(None) == _capi.STATUS_INVALID_ARGUMENTS


@pytest.mark.parametrize("workers", [1, 3, 74, 148])
def test_narrow_column_work_order_is_a_permutation_and_balances(lib_instrument, workers):
    """A launch whose last tile column is narrower deals those cheaper tiles to the work
    slots (slot v runs on worker v % workers in round v // workers) so that no worker ends
    a whole wide tile late.  The map must hit every tile exactly once, keep the wide tiles
    in ascending order, and never load a worker more than the plain order would."""
    f = lib_instrument.cpuops_b200_debug_slot_to_tile
    f.argtypes = [C.c_int32] * 4 + [C.POINTER(C.c_int32)] * 2
    f.restype = C.c_int

    def loads(wide, narrow, order):
        out = [0.0] * workers
        for v, is_narrow in enumerate(order):
            out[v % workers] += 0.67 if is_narrow else 1.0
        return max(out)

    for narrow in (0, 1, 2, 16, 33):
        for wide in (0, 1, 73, 74, 147, 288, 301):
            if wide + narrow == 0:
                continue
            wide_seen, narrow_seen, order = [], set(), []
            for v in range(wide + narrow):
                a, b = C.c_int32(), C.c_int32()
                assert f(v, wide, narrow, workers, C.byref(a), C.byref(b)) == 0
                order.append(bool(a.value))
                if a.value:
                    assert 0 <= b.value < narrow and b.value not in narrow_seen
                    narrow_seen.add(b.value)
                else:
                    wide_seen.append(b.value)
            assert wide_seen == list(range(wide))
            assert len(narrow_seen) == narrow
            plain = [False] * wide + [True] * narrow
            assert loads(wide, narrow, order) <= loads(wide, narrow, plain) + 1e-9
    a, b = C.c_int32(), C.c_int32()
    assert f(5, 2, 3, workers, C.byref(a), C.byref(b)) == 1      # slot out of range


def test_tile_width_choice_for_the_configured_workloads(lib_instrument):
    """The launcher's cost model (148 SMs): 256-wide tiles for int8, 224-wide for MX (two
    accumulators plus the scale slots must fit in tensor memory), also for 4096^3 where a
    64-wide last column evens the rounds out; an n-contiguous B only allows 128 or 256."""
    f = lib_instrument.cpuops_b200_debug_pick_tile_width
    f.argtypes = [C.c_int32] * 7
    f.restype = C.c_int
    sms = 148
    #            Mk     Nk     k-blocks  mx beta  n-contiguous B
    assert f(4096, 4096, 32, 1, sms, 1, 0) == 224          # mxfp8 4096^3, beta = 0.5
    assert f(8192, 8192, 64, 1, sms, 0, 0) == 224          # mxfp8 8192^3
    assert f(16384, 16384, 64, 1, sms, 0, 0) == 224        # mxfp4 16384^3
    assert f(8192, 8192, 64, 0, sms, 0, 1) == 256          # int8 8192^3, row-major B
    assert f(8192, 8192, 128, 0, sms, 0, 1) == 256         # int8 8192 x 8192 x 16384
    assert f(2048, 2048, 16, 0, sms, 1, 1) == 256          # int8 2048^3
    # mid-size shapes whose choice was checked against forced widths on a B200
    assert f(2048, 2048, 16, 1, sms, 0, 0) == 256          # MX 2048^3: one wave of 128 tiles
    assert f(1024, 4096, 32, 1, sms, 0, 0) == 256          # 224 would be 152 tiles on 148 SMs
    assert f(4096, 1024, 32, 1, sms, 1, 0) == 256
    assert f(3000, 5000, 16, 1, sms, 0, 0) == 224
    assert f(1024, 8192, 16, 1, sms, 0, 0) == 224
    assert f(2560, 2560, 64, 1, sms, 0, 0) in (192, 224)   # not 128-wide pairs: 15 % slower
    assert f(1024, 4096, 32, 0, sms, 0, 1) == 256
    for nk in (129, 500, 1000, 3000, 5000):
        for mk in (128, 1000, 5000):
            assert f(mk, nk, 16, 0, sms, 0, 1) in (128, 256)
            assert f(mk, nk, 16, 1, sms, 1, 0) in (128, 160, 192, 224, 256)
