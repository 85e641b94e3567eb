"""Python mirror of the reference's device-level GEMM operators, over the C ABI.

Names and argument meaning follow ``include/cpu_ops/gemm/device/gemm.h`` and
``gemm_mx.h`` of napplesty/cpu_ops: ``GemmCoord``, ``TensorRef`` /
``MxTensorRef`` (pointer + leading dimension), ``LinearCombination`` /
``LinearCombinationFused`` epilogue parameters, ``Arguments`` with the same
field order, and a callable operator returning the reference's ``Status``.
Buffers may be numpy arrays (host memory), torch tensors (host or CUDA) or raw
integer addresses.  All work is done by ``libcpu_ops_b200.so``; nothing here
computes.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass, field
from typing import Any, Optional, Sequence

from . import _capi


class Status(enum.IntEnum):
    """cpu_ops::Status (status.h:5-9) plus the GPU-runtime codes of the C ABI."""
    kSuccess = 0
    kErrorInvalidProblem = 1
    kErrorInvalidArguments = 2
    kErrorUnsupported = 3
    kErrorNoDevice = 4
    kErrorCuda = 5
    kErrorDeviceTimeout = 6
    kErrorBadDescriptor = 7


class RowMajor:
    """layout::RowMajor (layout/matrix.h:9-15)."""
    kIsRowMajor = True

    @staticmethod
    def offset(row, col, ld):
        return row * ld + col


class ColumnMajor:
    """layout::ColumnMajor (layout/matrix.h:17-22)."""
    kIsRowMajor = False

    @staticmethod
    def offset(row, col, ld):
        return col * ld + row


class fp8e4m3_t:
    fmt = _capi.FMT_E4M3
    elems_per_byte = 1


class fp8e5m2_t:
    fmt = _capi.FMT_E5M2
    elems_per_byte = 1


class fp4e2m1_t:
    fmt = _capi.FMT_E2M1
    elems_per_byte = 2


def data_ptr(buf: Any) -> Optional[int]:
    """Address of a numpy array, torch tensor, ctypes object or int; None stays None."""
    if buf is None:
        return None
    if isinstance(buf, int):
        return buf or None
    if hasattr(buf, "data_ptr"):
        return int(buf.data_ptr()) or None
    if hasattr(buf, "ctypes"):
        return int(buf.ctypes.data) or None
    return C.addressof(buf)


def _settle_torch_operands(args) -> None:
    """A call without a stream runs on the library's own stream, which is not ordered after
    torch's: if an operand is a CUDA torch tensor, wait for torch's current stream first so
    that fills and copies enqueued there have landed (the C ABI leaves this to the caller)."""
    for ref in (args.ref_A, args.ref_B, args.ref_C, args.ref_D):
        buf = getattr(ref, "data", None)
        if getattr(buf, "is_cuda", False):
            import torch
            torch.cuda.current_stream(buf.device).synchronize()
            return


@dataclass
class GemmCoord:
    """gemm_coord.h:6-13."""
    m: int = 0
    n: int = 0
    k: int = 0


@dataclass
class TensorRef:
    """tensor_ref.h:6-27: non-owning pointer + leading dimension (elements)."""
    data: Any = None
    ld: int = 0


@dataclass
class MxTensorRef:
    """mx_formats.h:280-295: packed elements + E8M0 scales, ld in elements,
    ld_scales in scale entries."""
    data: Any = None
    scales: Any = None
    ld: int = 0
    ld_scales: int = 0


class Activation(enum.IntEnum):
    kNone = 0
    kRelu = 1


# ---- fused chain ops (epilogue/fusion.h:31-129) --------------------------------
@dataclass
class Relu:
    opcode = _capi.OP_RELU


@dataclass
class Gelu:
    opcode = _capi.OP_GELU


@dataclass
class Silu:
    opcode = _capi.OP_SILU


@dataclass
class Clamp:
    lo: Any = 0
    hi: Any = 0
    opcode = _capi.OP_CLAMP


@dataclass
class BiasAdd:
    bias: Any = None
    opcode = _capi.OP_BIAS_ADD


@dataclass
class ScalePerRow:
    scale: Any = None
    opcode = _capi.OP_SCALE_PER_ROW


@dataclass
class ScalePerCol:
    scale: Any = None
    opcode = _capi.OP_SCALE_PER_COL


@dataclass
class LinearCombination:
    """LinearCombination<T>::Params (epilogue/linear_combination.h:72-76)."""
    alpha: Any = 1
    beta: Any = 0
    activation: Activation = Activation.kNone
    chain: Sequence[Any] = ()


@dataclass
class LinearCombinationFused:
    """LinearCombinationFused<T, Ops...>::Params (epilogue/fusion.h:170-174)."""
    alpha: Any = 1
    beta: Any = 0
    chain: Sequence[Any] = ()
    activation: Activation = Activation.kNone


@dataclass
class GemmArguments:
    """Gemm::Arguments (gemm.h:84-94); field order as in the reference."""
    problem_size: GemmCoord = field(default_factory=GemmCoord)
    ref_A: TensorRef = field(default_factory=TensorRef)
    ref_B: TensorRef = field(default_factory=TensorRef)
    ref_C: TensorRef = field(default_factory=TensorRef)
    ref_D: TensorRef = field(default_factory=TensorRef)
    epilogue: Any = field(default_factory=LinearCombination)
    split_k_slices: int = 0


@dataclass
class GemmMxArguments:
    """GemmMx::Arguments (gemm_mx.h:65-74)."""
    problem_size: GemmCoord = field(default_factory=GemmCoord)
    ref_A: MxTensorRef = field(default_factory=MxTensorRef)
    ref_B: MxTensorRef = field(default_factory=MxTensorRef)
    ref_C: TensorRef = field(default_factory=TensorRef)
    ref_D: TensorRef = field(default_factory=TensorRef)
    epilogue: Any = field(default_factory=LinearCombination)
    split_k_slices: int = 0


def _fill_epilogue(desc: _capi.GemmDesc, epi, is_int: bool):
    if is_int:
        desc.alpha.i32, desc.beta.i32 = int(epi.alpha), int(epi.beta)
    else:
        desc.alpha.f32, desc.beta.f32 = float(epi.alpha), float(epi.beta)
    desc.activation = int(getattr(epi, "activation", Activation.kNone))
    chain = list(getattr(epi, "chain", ()) or ())
    if len(chain) > _capi.MAX_OPS:
        raise ValueError(f"at most {_capi.MAX_OPS} chain ops")
    desc.n_ops = len(chain)
    for t, op in enumerate(chain):
        rec = desc.ops[t]
        rec.opcode = op.opcode
        rec.ptr = data_ptr(getattr(op, "bias", None) if hasattr(op, "bias")
                           else getattr(op, "scale", None))
        if isinstance(op, Clamp):
            if is_int:
                rec.lo.i32, rec.hi.i32 = int(op.lo), int(op.hi)
            else:
                rec.lo.f32, rec.hi.f32 = float(op.lo), float(op.hi)


class _Operator:
    """Shared call plumbing.  Stateless, like the reference functors."""

    def __init__(self, *, stream: Optional[int] = None, asynchronous: bool = False,
                 memory_space: int = _capi.MEM_AUTO, device: int = -1, tile_n: int = 0,
                 pair: Optional[bool] = None):
        # A raw handle of 0 is CUDA's legacy default stream (what torch reports for its
        # default stream); the C ABI reserves NULL for "the library's own stream", so
        # pass the explicit legacy-stream handle instead.
        self._stream = 1 if stream == 0 else stream
        self._async = asynchronous
        self._memory_space = memory_space
        self._device = device
        self._tile_n = tile_n
        # testing/tuning: True/False force/forbid the two-CTA kernel, None lets the library decide
        self._pair_flag = 0 if pair is None else (_capi.FLAG_PAIR_ON if pair else _capi.FLAG_PAIR_OFF)
        self._gemm = _capi.load().cpuops_b200_gemm

    def run(self, desc: _capi.GemmDesc) -> Status:
        """Issues one call with a descriptor built earlier by ``describe``.

        A C++ caller of the reference builds ``Arguments`` on the stack for free; a
        Python loop that issues the same GEMM repeatedly (a decode loop) can keep the
        descriptor instead of paying for its construction on every call.
        """
        return Status(self._gemm(C.byref(desc)))

    def __call__(self, args, num_threads: int = 0) -> Status:
        del num_threads  # accepted for source compatibility; the GPU grid replaces the pool
        desc = self.describe(args)
        if self._stream is None:
            _settle_torch_operands(args)
        return self.run(desc)

    def _finish(self, desc: _capi.GemmDesc, args) -> _capi.GemmDesc:
        desc.struct_size = C.sizeof(_capi.GemmDesc)
        desc.split_k_slices = int(args.split_k_slices)
        desc.memory_space = self._memory_space
        desc.stream = self._stream
        desc.flags = (_capi.FLAG_ASYNC if self._async else 0) | self._pair_flag
        desc.device = self._device
        desc.tile_n = self._tile_n
        return desc


class GemmU8S8S32(_Operator):
    """gemm::device::GemmU8S8S32<LayoutA, LayoutB, LayoutC> (gemm.h:130-142):
    u8 x s8 -> s32, D = epilogue(alpha * A*B + beta * C), wrap-around s32."""

    Arguments = GemmArguments

    def __init__(self, layout_a=RowMajor, layout_b=RowMajor, layout_c=RowMajor, **kw):
        super().__init__(**kw)
        self.LayoutA, self.LayoutB, self.LayoutC = layout_a, layout_b, layout_c

    def describe(self, args: GemmArguments) -> _capi.GemmDesc:
        """The C-ABI descriptor of one call (pointers are read now, not at run time)."""
        desc = _capi.GemmDesc()
        desc.kind = _capi.KIND_I8
        desc.a_format, desc.b_format = _capi.FMT_U8, _capi.FMT_S8
        ps = args.problem_size
        desc.m, desc.n, desc.k = int(ps.m), int(ps.n), int(ps.k)
        desc.a_row_major = int(self.LayoutA.kIsRowMajor)
        desc.b_row_major = int(self.LayoutB.kIsRowMajor)
        desc.c_row_major = int(self.LayoutC.kIsRowMajor)
        desc.a, desc.lda = data_ptr(args.ref_A.data), int(args.ref_A.ld)
        desc.b, desc.ldb = data_ptr(args.ref_B.data), int(args.ref_B.ld)
        desc.c, desc.ldc = data_ptr(args.ref_C.data), int(args.ref_C.ld)
        desc.d, desc.ldd = data_ptr(args.ref_D.data), int(args.ref_D.ld)
        _fill_epilogue(desc, args.epilogue, True)
        return self._finish(desc, args)


    def call_noalloc(self, args: GemmArguments) -> Status:
        """The same GEMM through ``cpuops_b200_gemm_i8_noalloc``: the two-stage split-k
        path with its partial sums in the library's built-in scratch array, for hosts
        that must not trigger a device allocation (a serving process that owns all
        device memory through its own pool; a latency-critical loop where cudaMalloc
        would stall the device).  Device operands only; see the C header for limits."""
        desc = _capi.GemmDesc()
        desc.kind = _capi.KIND_I8
        desc.a_format, desc.b_format = _capi.FMT_U8, _capi.FMT_S8
        ps = args.problem_size
        desc.m, desc.n, desc.k = int(ps.m), int(ps.n), int(ps.k)
        desc.a_row_major = int(self.LayoutA.kIsRowMajor)
        desc.b_row_major = int(self.LayoutB.kIsRowMajor)
        desc.c_row_major = int(self.LayoutC.kIsRowMajor)
        desc.a, desc.lda = data_ptr(args.ref_A.data), int(args.ref_A.ld)
        desc.b, desc.ldb = data_ptr(args.ref_B.data), int(args.ref_B.ld)
        desc.c, desc.ldc = data_ptr(args.ref_C.data), int(args.ref_C.ld)
        desc.d, desc.ldd = data_ptr(args.ref_D.data), int(args.ref_D.ld)
        _fill_epilogue(desc, args.epilogue, True)
        desc.struct_size = C.sizeof(_capi.GemmDesc)
        desc.split_k_slices = int(args.split_k_slices)
        desc.memory_space = self._memory_space
        desc.stream = self._stream
        desc.device = self._device
        return Status(_capi.load().cpuops_b200_gemm_i8_noalloc(C.byref(desc)))


class GemmMx(_Operator):
    """gemm::device::GemmMx<StorageA, StorageB, LayoutC> (gemm_mx.h:44-118):
    OCP MX fp8/fp4 elements with one E8M0 scale per 32 k-elements, f32 output."""

    Arguments = GemmMxArguments

    def __init__(self, storage_a=fp8e4m3_t, storage_b=None, layout_c=RowMajor, **kw):
        super().__init__(**kw)
        self.StorageA = storage_a
        self.StorageB = storage_b or storage_a
        self.LayoutC = layout_c

    def describe(self, args: GemmMxArguments) -> _capi.GemmDesc:
        """The C-ABI descriptor of one call (pointers are read now, not at run time)."""
        desc = _capi.GemmDesc()
        desc.kind = _capi.KIND_MX
        desc.a_format, desc.b_format = self.StorageA.fmt, self.StorageB.fmt
        ps = args.problem_size
        desc.m, desc.n, desc.k = int(ps.m), int(ps.n), int(ps.k)
        desc.a_row_major, desc.b_row_major = 1, 0
        desc.c_row_major = int(self.LayoutC.kIsRowMajor)
        a, b = args.ref_A, args.ref_B
        desc.a, desc.a_scales = data_ptr(a.data), data_ptr(a.scales)
        desc.lda, desc.ld_scales_a = int(a.ld), int(a.ld_scales)
        desc.b, desc.b_scales = data_ptr(b.data), data_ptr(b.scales)
        desc.ldb, desc.ld_scales_b = int(b.ld), int(b.ld_scales)
        desc.c, desc.ldc = data_ptr(args.ref_C.data), int(args.ref_C.ld)
        desc.d, desc.ldd = data_ptr(args.ref_D.data), int(args.ref_D.ld)
        _fill_epilogue(desc, args.epilogue, False)
        return self._finish(desc, args)


class PreparedB:
    """Keeps the tile-ordered copy of an MX weight operand's scales across calls
    (``cpuops_b200_prepare_b``): a decode loop registers its weights once."""

    def __init__(self, op: "GemmMx", args: "GemmMxArguments"):
        self._handle = C.c_void_p()
        desc = op.describe(args)
        st = _capi.load().cpuops_b200_prepare_b(C.byref(desc), C.byref(self._handle))
        if st != 0:
            raise RuntimeError(f"prepare_b failed ({st}): {_capi.last_error()}")

    def release(self) -> None:
        if self._handle:
            _capi.load().cpuops_b200_release_b(self._handle)
            self._handle = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.release()


def GemmMxE4M3(layout_c=RowMajor, **kw):
    """gemm_mx.h:121-122."""
    return GemmMx(fp8e4m3_t, fp8e4m3_t, layout_c, **kw)


def GemmMxE5M2(layout_c=RowMajor, **kw):
    """gemm_mx.h:123-124."""
    return GemmMx(fp8e5m2_t, fp8e5m2_t, layout_c, **kw)


def GemmMxE2M1(layout_c=RowMajor, **kw):
    """gemm_mx.h:125-127."""
    return GemmMx(fp4e2m1_t, fp4e2m1_t, layout_c, **kw)


def stream_status(stream: Optional[int] = None) -> Status:
    """Synchronise `stream` and report device-side errors of asynchronous calls."""
    return Status(_capi.load().cpuops_b200_stream_status(1 if stream == 0 else stream))


def launch_count() -> int:
    return int(_capi.load().cpuops_b200_launch_count())
