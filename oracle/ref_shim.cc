// TEST INFRASTRUCTURE ONLY.  C-ABI shim over the UNMODIFIED reference headers
// (napplesty/cpu_ops, include/cpu_ops/...), compiled by oracle/Makefile from the
// sources where they lie (-I$(REFERENCE)/include) into oracle/_ref/.  It exists
// so that (a) the C restatement in quant_gemm_oracle.c can be pinned against
// the real reference and (b) the benchmark can time the reference's own CPU
// path on the host cores.  No reference source is copied: this file only
// instantiates the reference's public templates
//   gemm::device::Gemm<uint8_t,..,int8_t,..,int32_t,..>   (gemm/device/gemm.h:57-127)
//   gemm::device::GemmMx<SA,SB,LC,...>                    (gemm/device/gemm_mx.h:44-118)
//   epilogue::LinearCombination / LinearCombinationFused   (epilogue/*.h)
// the way test/test_gemm_int8.cc:70-84 and test/test_gemm_mx.cc:199-211 do.
// The product library never links or loads this.

#include <cstdint>
#include <cstring>
#include <thread>

#include "cpu_ops/epilogue/fusion.h"
#include "cpu_ops/epilogue/linear_combination.h"
#include "cpu_ops/gemm/device/gemm.h"
#include "cpu_ops/gemm/device/gemm_fused.h"
#include "cpu_ops/gemm/device/gemm_mx.h"
#include "cpu_ops/mx_formats.h"

using cpu_ops::layout::ColumnMajor;
using cpu_ops::layout::RowMajor;
namespace epi = cpu_ops::epilogue;
namespace dev = cpu_ops::gemm::device;

namespace {

// Default tile configuration and policy of the GemmU8S8S32 alias for the ISA
// this TU is compiled for (gemm/device/gemm.h:130-142).
#if defined(CPU_OPS_SIMD_AVX512VNNI)
using I8Config = cpu_ops::mma::Vnni512GemmConfig;
#else
using I8Config = dev::GemmConfig<int32_t>;
#endif
using I8Policy = cpu_ops::mma::VnniPolicy<>;

template <typename LA, typename LB, typename LC>
int run_i8(int m, int n, int k, const uint8_t* A, int lda, const int8_t* B, int ldb,
           const int32_t* C, int ldc, int32_t* D, int ldd, int32_t alpha, int32_t beta,
           int relu, int split_k, int threads) {
  using Op = dev::GemmU8S8S32<LA, LB, LC>;
  typename Op::Arguments args{{m, n, k},
                              {A, lda},
                              {B, ldb},
                              {C, ldc},
                              {D, ldd},
                              {alpha, beta,
                               relu ? epi::Activation::kRelu : epi::Activation::kNone},
                              split_k};
  Op op;
  return static_cast<int>(op(args, threads));
}

template <typename SA, typename SB, typename LC>
int run_mx(int m, int n, int k, const uint8_t* A, const uint8_t* SAp, int lda, int ldsa,
           const uint8_t* B, const uint8_t* SBp, int ldb, int ldsb, const float* C, int ldc,
           float* D, int ldd, float alpha, float beta, int relu, int split_k, int threads) {
  using Op = dev::GemmMx<SA, SB, LC>;
  typename Op::Arguments args;
  args.problem_size = {m, n, k};
  args.ref_A = {A, SAp, lda, ldsa};
  args.ref_B = {B, SBp, ldb, ldsb};
  args.ref_C = {C, ldc};
  args.ref_D = {D, ldd};
  args.epilogue = {alpha, beta, relu ? epi::Activation::kRelu : epi::Activation::kNone};
  args.split_k_slices = split_k;
  Op op;
  return static_cast<int>(op(args, threads));
}

template <typename SA, typename SB>
int run_mx_lc(int c_row_major, int m, int n, int k, const uint8_t* A, const uint8_t* SAp,
              int lda, int ldsa, const uint8_t* B, const uint8_t* SBp, int ldb, int ldsb,
              const float* C, int ldc, float* D, int ldd, float alpha, float beta, int relu,
              int split_k, int threads) {
  if (c_row_major)
    return run_mx<SA, SB, RowMajor>(m, n, k, A, SAp, lda, ldsa, B, SBp, ldb, ldsb, C, ldc, D,
                                    ldd, alpha, beta, relu, split_k, threads);
  return run_mx<SA, SB, ColumnMajor>(m, n, k, A, SAp, lda, ldsa, B, SBp, ldb, ldsb, C, ldc, D,
                                     ldd, alpha, beta, relu, split_k, threads);
}

template <typename T, typename... Ops>
int run_mx_chain(int m, int n, int k, const uint8_t* A, const uint8_t* SAp, int lda, int ldsa,
                 const uint8_t* B, const uint8_t* SBp, int ldb, int ldsb, const float* C,
                 int ldc, float* D, int ldd, float alpha, float beta, epi::Chain<Ops...> chain,
                 int split_k, int threads) {
  using Op = dev::GemmMx<T, T, RowMajor, epi::LinearCombinationFused<float, Ops...>>;
  typename Op::Arguments args{{m, n, k},          {A, SAp, lda, ldsa}, {B, SBp, ldb, ldsb},
                              {C, ldc},           {D, ldd},            {alpha, beta, chain},
                              split_k};
  Op op;
  return static_cast<int>(op(args, threads));
}

template <typename T>
int run_mx_chain_id(int chain_id, int m, int n, int k, const uint8_t* A, const uint8_t* SAp,
                    int lda, int ldsa, const uint8_t* B, const uint8_t* SBp, int ldb, int ldsb,
                    const float* C, int ldc, float* D, int ldd, float alpha, float beta,
                    const float* vec0, const float* vec1, float lo, float hi, int split_k,
                    int threads) {
#define MX_ARGS m, n, k, A, SAp, lda, ldsa, B, SBp, ldb, ldsb, C, ldc, D, ldd, alpha, beta
  switch (chain_id) {
    case 1:
      return run_mx_chain<T>(MX_ARGS,
                             epi::Chain<epi::BiasAdd<float>, epi::Relu>{
                                 epi::BiasAdd<float>{vec0}, epi::Relu{}},
                             split_k, threads);
    case 2:
      return run_mx_chain<T>(
          MX_ARGS, epi::Chain<epi::ScalePerRow<float>>{epi::ScalePerRow<float>{vec0}}, split_k,
          threads);
    case 3:
      return run_mx_chain<T>(
          MX_ARGS,
          epi::Chain<epi::BiasAdd<float>, epi::ScalePerCol<float>, epi::Clamp<float>>{
              epi::BiasAdd<float>{vec0}, epi::ScalePerCol<float>{vec1},
              epi::Clamp<float>{lo, hi}},
          split_k, threads);
    case 4:
      return run_mx_chain<T>(MX_ARGS, epi::Chain<epi::Gelu>{epi::Gelu{}}, split_k, threads);
    case 5:
      return run_mx_chain<T>(MX_ARGS, epi::Chain<epi::Silu>{epi::Silu{}}, split_k, threads);
    default:
      return -1;
  }
#undef MX_ARGS
}

}  // namespace

extern "C" {

// layouts: bit 0 = A row-major, bit 1 = B row-major, bit 2 = C/D row-major.
__attribute__((visibility("default"))) int ref_gemm_u8s8s32(
    int layouts, int m, int n, int k, const uint8_t* A, int lda, const int8_t* B, int ldb,
    const int32_t* C, int ldc, int32_t* D, int ldd, int32_t alpha, int32_t beta, int relu,
    int split_k, int threads) {
#define I8_ARGS m, n, k, A, lda, B, ldb, C, ldc, D, ldd, alpha, beta, relu, split_k, threads
  switch (layouts & 7) {
    case 0: return run_i8<ColumnMajor, ColumnMajor, ColumnMajor>(I8_ARGS);
    case 1: return run_i8<RowMajor, ColumnMajor, ColumnMajor>(I8_ARGS);
    case 2: return run_i8<ColumnMajor, RowMajor, ColumnMajor>(I8_ARGS);
    case 3: return run_i8<RowMajor, RowMajor, ColumnMajor>(I8_ARGS);
    case 4: return run_i8<ColumnMajor, ColumnMajor, RowMajor>(I8_ARGS);
    case 5: return run_i8<RowMajor, ColumnMajor, RowMajor>(I8_ARGS);
    case 6: return run_i8<ColumnMajor, RowMajor, RowMajor>(I8_ARGS);
    default: return run_i8<RowMajor, RowMajor, RowMajor>(I8_ARGS);
  }
#undef I8_ARGS
}

// All-RowMajor u8 x s8 -> s32 with the fused chain BiasAdd -> Relu -> Clamp
// spelled out as a caller of the reference would (gemm/device/gemm.h:57-61
// with epilogue/fusion.h:168-195).
__attribute__((visibility("default"))) int ref_gemm_u8s8s32_bias_relu_clamp(
    int m, int n, int k, const uint8_t* A, int lda, const int8_t* B, int ldb, const int32_t* C,
    int ldc, int32_t* D, int ldd, int32_t alpha, int32_t beta, const int32_t* bias, int32_t lo,
    int32_t hi, int split_k, int threads) {
  using Epi = epi::LinearCombinationFused<int32_t, epi::BiasAdd<int32_t>, epi::Relu,
                                          epi::Clamp<int32_t>>;
  using Op = dev::Gemm<uint8_t, RowMajor, int8_t, RowMajor, int32_t, RowMajor, int32_t, Epi,
                       I8Config, I8Policy>;
  typename Op::Arguments args{
      {m, n, k},
      {A, lda},
      {B, ldb},
      {C, ldc},
      {D, ldd},
      {alpha, beta,
       epi::Chain<epi::BiasAdd<int32_t>, epi::Relu, epi::Clamp<int32_t>>{
           epi::BiasAdd<int32_t>{bias}, epi::Relu{}, epi::Clamp<int32_t>{lo, hi}}},
      split_k};
  Op op;
  return static_cast<int>(op(args, threads));
}

// fmt: 2 = e4m3, 3 = e5m2, 4 = e2m1 (fp4 packed two per byte).
__attribute__((visibility("default"))) int ref_gemm_mx(
    int fmt_a, int fmt_b, int c_row_major, int m, int n, int k, const uint8_t* A,
    const uint8_t* SA, int lda, int ldsa, const uint8_t* B, const uint8_t* SB, int ldb,
    int ldsb, const float* C, int ldc, float* D, int ldd, float alpha, float beta, int relu,
    int split_k, int threads) {
  using cpu_ops::fp4e2m1_t;
  using cpu_ops::fp8e4m3_t;
  using cpu_ops::fp8e5m2_t;
#define MX_ARGS \
  c_row_major, m, n, k, A, SA, lda, ldsa, B, SB, ldb, ldsb, C, ldc, D, ldd, alpha, beta, relu, \
      split_k, threads
  const int key = fmt_a * 10 + fmt_b;
  switch (key) {
    case 22: return run_mx_lc<fp8e4m3_t, fp8e4m3_t>(MX_ARGS);
    case 23: return run_mx_lc<fp8e4m3_t, fp8e5m2_t>(MX_ARGS);
    case 24: return run_mx_lc<fp8e4m3_t, fp4e2m1_t>(MX_ARGS);
    case 32: return run_mx_lc<fp8e5m2_t, fp8e4m3_t>(MX_ARGS);
    case 33: return run_mx_lc<fp8e5m2_t, fp8e5m2_t>(MX_ARGS);
    case 34: return run_mx_lc<fp8e5m2_t, fp4e2m1_t>(MX_ARGS);
    case 42: return run_mx_lc<fp4e2m1_t, fp8e4m3_t>(MX_ARGS);
    case 43: return run_mx_lc<fp4e2m1_t, fp8e5m2_t>(MX_ARGS);
    case 44: return run_mx_lc<fp4e2m1_t, fp4e2m1_t>(MX_ARGS);
    default: return -1;
  }
#undef MX_ARGS
}

// Same-format MX GEMM, RowMajor C, with one of the fused float chains:
//   1 BiasAdd(vec0) -> Relu            2 ScalePerRow(vec0)
//   3 BiasAdd(vec0) -> ScalePerCol(vec1) -> Clamp[lo,hi]
//   4 Gelu                              5 Silu
__attribute__((visibility("default"))) int ref_gemm_mx_chain(
    int fmt, int chain_id, int m, int n, int k, const uint8_t* A, const uint8_t* SA, int lda,
    int ldsa, const uint8_t* B, const uint8_t* SB, int ldb, int ldsb, const float* C, int ldc,
    float* D, int ldd, float alpha, float beta, const float* vec0, const float* vec1, float lo,
    float hi, int split_k, int threads) {
#define CH_ARGS \
  chain_id, m, n, k, A, SA, lda, ldsa, B, SB, ldb, ldsb, C, ldc, D, ldd, alpha, beta, vec0, \
      vec1, lo, hi, split_k, threads
  switch (fmt) {
    case 2: return run_mx_chain_id<cpu_ops::fp8e4m3_t>(CH_ARGS);
    case 3: return run_mx_chain_id<cpu_ops::fp8e5m2_t>(CH_ARGS);
    case 4: return run_mx_chain_id<cpu_ops::fp4e2m1_t>(CH_ARGS);
    default: return -1;
  }
#undef CH_ARGS
}

__attribute__((visibility("default"))) float ref_decode(int fmt, uint8_t code) {
  switch (fmt) {
    case 2: return cpu_ops::fp8e4m3_t::to_float(code);
    case 3: return cpu_ops::fp8e5m2_t::to_float(code);
    case 4: return cpu_ops::fp4e2m1_t::to_float(code);
    default: return cpu_ops::e8m0_to_float(code);
  }
}

__attribute__((visibility("default"))) uint8_t ref_encode(int fmt, float x) {
  switch (fmt) {
    case 2: return cpu_ops::fp8e4m3_t::from_float(x);
    case 3: return cpu_ops::fp8e5m2_t::from_float(x);
    case 4: return cpu_ops::fp4e2m1_t::from_float(x);
    default: return cpu_ops::e8m0_from_float(x);
  }
}

// The ISA line the reference benchmark prints (examples/01_benchmark.cc:188-202).
__attribute__((visibility("default"))) const char* ref_isa(void) {
#if defined(CPU_OPS_SIMD_AVX512BF16)
  return "AVX-512F + VNNI + BF16";
#elif defined(CPU_OPS_SIMD_AVX512VNNI)
  return "AVX-512F + VNNI";
#elif defined(CPU_OPS_SIMD_AVX512F)
  return "AVX-512F";
#elif defined(CPU_OPS_SIMD_VNNI)
  return "AVX2 + VNNI";
#elif defined(CPU_OPS_SIMD_AVX2)
  return "AVX2";
#else
  return "scalar";
#endif
}

// KC of the MX path for this build (gemm/device/gemm_mx.h:31-40).
__attribute__((visibility("default"))) int ref_mx_kc(void) {
  return dev::detail::GemmMxDefaults<cpu_ops::fp8e4m3_t, cpu_ops::fp8e4m3_t>::Config::kKC;
}

// Size of the reference's global pool (thread/thread_pool.h:27-29).
__attribute__((visibility("default"))) int ref_pool_threads(void) {
  return cpu_ops::thread::ThreadPool::global().num_threads();
}

}  // extern "C"
