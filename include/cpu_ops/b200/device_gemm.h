// gemm::device::Gemm / GemmMx with the reference's template surface and
// Arguments (include/cpu_ops/gemm/device/gemm.h:57-127, gemm_mx.h:44-118), for
// translation units that move from the CPU library to the B200 library without
// source changes.  operator() flattens Arguments into the C-ABI descriptor and
// calls cpuops_b200_gemm(); validation order and Status codes are the
// reference's (the C ABI re-checks them).  Config and MmaPolicy template
// arguments are accepted as tags and ignored: tile shapes are chosen by the
// library.  num_threads is accepted and ignored.
#ifndef CPU_OPS_B200_DEVICE_GEMM_H_
#define CPU_OPS_B200_DEVICE_GEMM_H_

#include <cstdint>
#include <cstring>
#include <type_traits>

#include "cpu_ops/b200/core_types.h"
#include "cpu_ops/b200/epilogue_types.h"
#include "cpu_ops/b200/mx_types.h"
#include "cpu_ops_b200.h"

namespace cpu_ops {

// Tag types callers may spell as Config / MmaPolicy template arguments.
namespace mma {
template <int VLEN = 8>
struct VnniPolicy {
  using ElemA = uint8_t;
  using ElemB = int8_t;
  using AccT = int32_t;
};
struct Vnni512GemmConfig {};
struct Fma512GemmConfig {};
struct AmxGemmConfig {};
struct AmxPolicy {
  using ElemA = uint8_t;
  using ElemB = int8_t;
  using AccT = int32_t;
};
template <typename StorageA, typename StorageB, int VLEN = 8>
struct MxPolicy {
  using ElemA = StorageA;
  using ElemB = StorageB;
  using AccT = float;
};
template <typename StorageA, typename StorageB, int VLEN = 8>
struct MxVnniPolicy {
  using ElemA = StorageA;
  using ElemB = StorageB;
  using AccT = float;
};
}  // namespace mma

namespace b200_detail {

template <typename T>
struct MxFormat;
template <>
struct MxFormat<fp8e4m3_t> {
  static constexpr int value = CPUOPS_B200_FMT_E4M3;
};
template <>
struct MxFormat<fp8e5m2_t> {
  static constexpr int value = CPUOPS_B200_FMT_E5M2;
};
template <>
struct MxFormat<fp4e2m1_t> {
  static constexpr int value = CPUOPS_B200_FMT_E2M1;
};

inline Status to_status(int rc) {
  switch (rc) {
    case CPUOPS_B200_STATUS_SUCCESS: return Status::kSuccess;
    case CPUOPS_B200_STATUS_INVALID_PROBLEM: return Status::kErrorInvalidProblem;
    case CPUOPS_B200_STATUS_INVALID_ARGUMENTS: return Status::kErrorInvalidArguments;
    default: return Status::kErrorInternal;  // cpuops_b200_last_error() has the detail
  }
}

inline cpuops_b200_gemm_desc blank_desc() {
  cpuops_b200_gemm_desc d;
  std::memset(&d, 0, sizeof d);
  d.struct_size = sizeof d;
  d.device = -1;
  return d;
}

}  // namespace b200_detail

namespace gemm {
namespace device {

template <typename T>
struct GemmConfig {};  // tile-shape tag of the CPU library; ignored here

namespace detail {
// Default Config / Policy tags, spelled by callers that pass them explicitly
// (gemm.h:33-51, gemm_mx.h:27-42 of the reference).
template <typename T>
struct GemmDefaults {
  using Config = GemmConfig<T>;
  using Policy = mma::VnniPolicy<>;
};
template <typename StorageA, typename StorageB>
struct GemmMxDefaults {
  using Config = GemmConfig<float>;
  using Policy = mma::MxPolicy<StorageA, StorageB>;
};
}  // namespace detail

// D = epilogue(alpha * A * B + beta * C).  Only the quantized instantiation
// (uint8_t x int8_t -> int32_t) exists in this library.
template <typename ElementA_, typename LayoutA_, typename ElementB_, typename LayoutB_,
          typename ElementC_, typename LayoutC_, typename ElementAccumulator_ = ElementC_,
          typename Epilogue_ = epilogue::LinearCombination<ElementC_>,
          typename Config_ = GemmConfig<ElementC_>, typename MmaPolicy_ = mma::VnniPolicy<>>
class Gemm {
 public:
  using ElementA = ElementA_;
  using LayoutA = LayoutA_;
  using ElementB = ElementB_;
  using LayoutB = LayoutB_;
  using ElementC = ElementC_;
  using LayoutC = LayoutC_;
  using ElementAccumulator = ElementAccumulator_;
  using Epilogue = Epilogue_;
  using Config = Config_;
  using MmaPolicy = MmaPolicy_;

  static_assert(std::is_same<ElementA, uint8_t>::value && std::is_same<ElementB, int8_t>::value &&
                    std::is_same<ElementC, int32_t>::value &&
                    std::is_same<ElementAccumulator, int32_t>::value,
                "the B200 library provides the quantized path only: uint8_t x int8_t -> int32_t "
                "(float / half GEMMs stay with the CPU library)");

  struct Arguments {
    GemmCoord problem_size;
    TensorRef<const ElementA, LayoutA> ref_A;
    TensorRef<const ElementB, LayoutB> ref_B;
    TensorRef<const ElementC, LayoutC> ref_C;
    TensorRef<ElementC, LayoutC> ref_D;
    typename Epilogue::Params epilogue;
    int split_k_slices = 0;  // 0 automatic, 1 never, > 1 forced
  };

  Gemm() = default;

  Status operator()(const Arguments& args, int /*num_threads*/ = 0) const {
    cpuops_b200_gemm_desc d = b200_detail::blank_desc();
    d.kind = CPUOPS_B200_KIND_I8;
    d.a_format = CPUOPS_B200_FMT_U8;
    d.b_format = CPUOPS_B200_FMT_S8;
    d.m = args.problem_size.m;
    d.n = args.problem_size.n;
    d.k = args.problem_size.k;
    d.a_row_major = LayoutA::kIsRowMajor;
    d.b_row_major = LayoutB::kIsRowMajor;
    d.c_row_major = LayoutC::kIsRowMajor;
    d.a = args.ref_A.data();
    d.lda = args.ref_A.ld();
    d.b = args.ref_B.data();
    d.ldb = args.ref_B.ld();
    d.c = args.ref_C.data();
    d.ldc = args.ref_C.ld();
    d.d = args.ref_D.data();
    d.ldd = args.ref_D.ld();
    b200_detail::EpilogueToDesc<Epilogue>::fill(args.epilogue, &d);
    d.split_k_slices = args.split_k_slices;
    return b200_detail::to_status(cpuops_b200_gemm(&d));
  }
};

template <typename LayoutA, typename LayoutB, typename LayoutC>
using GemmU8S8S32 = Gemm<uint8_t, LayoutA, int8_t, LayoutB, int32_t, LayoutC, int32_t,
                         epilogue::LinearCombination<int32_t>, GemmConfig<int32_t>, mma::VnniPolicy<>>;

// D = epilogue(alpha * (A .* scalesA)(B .* scalesB) + beta * C), f32 C/D, "TN".
template <typename StorageA_, typename StorageB_, typename LayoutC_ = layout::RowMajor,
          typename Epilogue_ = epilogue::LinearCombination<float>, typename Config_ = GemmConfig<float>,
          typename MmaPolicy_ = mma::MxPolicy<StorageA_, StorageB_>>
class GemmMx {
 public:
  using StorageA = StorageA_;
  using StorageB = StorageB_;
  using LayoutC = LayoutC_;
  using Epilogue = Epilogue_;
  using Config = Config_;
  using MmaPolicy = MmaPolicy_;

  struct Arguments {
    GemmCoord problem_size;
    MxTensorRef<StorageA> ref_A;  // m rows of k
    MxTensorRef<StorageB> ref_B;  // n rows of k
    TensorRef<const float, LayoutC> ref_C;
    TensorRef<float, LayoutC> ref_D;
    typename Epilogue::Params epilogue;
    int split_k_slices = 0;
  };

  GemmMx() = default;

  Status operator()(const Arguments& args, int /*num_threads*/ = 0) const {
    cpuops_b200_gemm_desc d = b200_detail::blank_desc();
    d.kind = CPUOPS_B200_KIND_MX;
    d.a_format = b200_detail::MxFormat<StorageA>::value;
    d.b_format = b200_detail::MxFormat<StorageB>::value;
    d.m = args.problem_size.m;
    d.n = args.problem_size.n;
    d.k = args.problem_size.k;
    d.a_row_major = 1;
    d.b_row_major = 0;
    d.c_row_major = LayoutC::kIsRowMajor;
    d.a = args.ref_A.data;
    d.a_scales = args.ref_A.scales;
    d.lda = args.ref_A.ld;
    d.ld_scales_a = args.ref_A.ld_scales;
    d.b = args.ref_B.data;
    d.b_scales = args.ref_B.scales;
    d.ldb = args.ref_B.ld;
    d.ld_scales_b = args.ref_B.ld_scales;
    d.c = args.ref_C.data();
    d.ldc = args.ref_C.ld();
    d.d = args.ref_D.data();
    d.ldd = args.ref_D.ld();
    b200_detail::EpilogueToDesc<Epilogue>::fill(args.epilogue, &d);
    d.split_k_slices = args.split_k_slices;
    return b200_detail::to_status(cpuops_b200_gemm(&d));
  }
};

template <typename LayoutC = layout::RowMajor>
using GemmMxE4M3 = GemmMx<fp8e4m3_t, fp8e4m3_t, LayoutC>;
template <typename LayoutC = layout::RowMajor>
using GemmMxE5M2 = GemmMx<fp8e5m2_t, fp8e5m2_t, LayoutC>;
template <typename LayoutC = layout::RowMajor>
using GemmMxE2M1 = GemmMx<fp4e2m1_t, fp4e2m1_t, LayoutC>;

// The CPU library's opt-in lossy int8-requantising MX variants
// (gemm_mx.h:132-158) have no separate implementation here: the names forward to
// the exact block-scaled path.
template <typename LayoutC = layout::RowMajor>
using GemmMxE4M3Vnni = GemmMxE4M3<LayoutC>;
template <typename LayoutC = layout::RowMajor>
using GemmMxE5M2Vnni = GemmMxE5M2<LayoutC>;
template <typename LayoutC = layout::RowMajor>
using GemmMxE2M1Vnni = GemmMxE2M1<LayoutC>;

// Int8 GEMM with a fused chain, spelled like the reference's float GemmFusedF32
// (gemm_fused.h:15-18).
template <typename LayoutA, typename LayoutB, typename LayoutC, typename... Ops>
using GemmFusedU8S8S32 =
    Gemm<uint8_t, LayoutA, int8_t, LayoutB, int32_t, LayoutC, int32_t,
         epilogue::LinearCombinationFused<int32_t, Ops...>>;

}  // namespace device
}  // namespace gemm
}  // namespace cpu_ops

#endif  // CPU_OPS_B200_DEVICE_GEMM_H_
