"""cpu_ops_b200: the quantized-GEMM path of napplesty/cpu_ops on NVIDIA B200.

``gemm`` mirrors the reference's device-level operators (GemmU8S8S32,
GemmMxE4M3 / E5M2 / E2M1) over the C ABI of ``libcpu_ops_b200.so``;
``sharding`` spreads output row blocks over one process per GPU;
``workloads`` generates the seeded synthetic inputs used by tests and bench.
"""
from . import _capi  # noqa: F401
from .gemm import (  # noqa: F401
    Activation, BiasAdd, Clamp, ColumnMajor, Gelu, GemmArguments, GemmCoord, GemmMx,
    GemmMxArguments, GemmMxE2M1, GemmMxE4M3, GemmMxE5M2, GemmU8S8S32, LinearCombination,
    LinearCombinationFused, MxTensorRef, PreparedB, Relu, RowMajor, ScalePerCol, ScalePerRow, Silu, Status,
    TensorRef, fp4e2m1_t, fp8e4m3_t, fp8e5m2_t, launch_count, stream_status,
)

__version__ = "0.1.0"
