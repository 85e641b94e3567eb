// Call sites written the way the reference's own tests write them
// (test/test_gemm_int8.cc:46-109, test/test_gemm_mx.cc:150-227, :346-372),
// compiled against include/cpu_ops/ of THIS repository and linked with
// libcpu_ops_b200.so.  Modes:
//   compat_call_sites --status                 argument validation only (no GPU needed)
//   compat_call_sites --codecs in.bin out.bin  dump decode tables + encode the floats in in.bin
//   compat_call_sites --gpu                    run the GEMM cases on the GPU against in-file
//                                              exact (int64) / double references
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <limits>
#include <random>
#include <string>
#include <type_traits>
#include <vector>

#include "cpu_ops/cpu_ops.h"

namespace {

int g_failures = 0;
int g_cases = 0;

#define CHECK(cond, ...)                                 \
  do {                                                   \
    if (!(cond)) {                                       \
      ++g_failures;                                      \
      std::printf("FAIL %s:%d: ", __FILE__, __LINE__);   \
      std::printf(__VA_ARGS__);                          \
      std::printf("\n");                                 \
    }                                                    \
  } while (0)

using cpu_ops::Status;
using cpu_ops::fp4e2m1_t;
using cpu_ops::fp8e4m3_t;
using cpu_ops::fp8e5m2_t;
using cpu_ops::layout::ColumnMajor;
using cpu_ops::layout::RowMajor;
namespace epilogue = cpu_ops::epilogue;

template <typename LA, typename LB, typename LC>
void int8_case(int m, int n, int k, int32_t alpha, int32_t beta, bool relu) {
  ++g_cases;
  const int lda = (LA::kIsRowMajor ? k : m) + 3;
  const int ldb = (LB::kIsRowMajor ? n : k) + 3;
  const int ldc = (LC::kIsRowMajor ? n : m) + 3;
  std::vector<uint8_t> A(static_cast<size_t>(LA::kIsRowMajor ? m : k) * lda);
  std::vector<int8_t> B(static_cast<size_t>(LB::kIsRowMajor ? k : n) * ldb);
  std::vector<int32_t> C(static_cast<size_t>(LC::kIsRowMajor ? m : n) * ldc);
  std::vector<int32_t> D(C.size(), INT32_MIN), want(C.size(), INT32_MIN);
  std::mt19937 rng(static_cast<unsigned>(m * 131 + n * 17 + k));
  for (auto& x : A) x = static_cast<uint8_t>(rng() & 0xFF);
  for (auto& x : B) x = static_cast<int8_t>(rng() & 0xFF);
  for (auto& x : C) x = static_cast<int32_t>(rng() % 2001) - 1000;
  for (int i = 0; i < m; ++i)
    for (int j = 0; j < n; ++j) {
      int64_t acc = 0;
      for (int p = 0; p < k; ++p)
        acc += int64_t{A[LA::offset(i, p, lda)]} * int64_t{B[LB::offset(p, j, ldb)]};
      int64_t v = int64_t{alpha} * acc + int64_t{beta} * C[LC::offset(i, j, ldc)];
      if (relu && v < 0) v = 0;
      want[LC::offset(i, j, ldc)] = static_cast<int32_t>(v);
    }
  using Gemm = cpu_ops::gemm::device::GemmU8S8S32<LA, LB, LC>;
  typename Gemm::Arguments args{{m, n, k},
                                {A.data(), lda},
                                {B.data(), ldb},
                                {C.data(), ldc},
                                {D.data(), ldc},
                                {alpha, beta,
                                 relu ? epilogue::Activation::kRelu : epilogue::Activation::kNone}};
  Gemm op;
  CHECK(op(args, 8) == Status::kSuccess, "int8 %dx%dx%d: bad status (%s)", m, n, k,
        cpuops_b200_last_error());
  CHECK(D == want, "int8 %dx%dx%d a=%d b=%d relu=%d: result differs", m, n, k, alpha, beta, (int)relu);
  // in place
  std::vector<int32_t> D2 = C;
  typename Gemm::Arguments args2{{m, n, k}, {A.data(), lda}, {B.data(), ldb},
                                 {D2.data(), ldc}, {D2.data(), ldc}, args.epilogue};
  CHECK(op(args2) == Status::kSuccess, "int8 in-place: bad status");
  for (int i = 0; i < m; ++i)
    for (int j = 0; j < n; ++j)
      CHECK(D2[LC::offset(i, j, ldc)] == want[LC::offset(i, j, ldc)], "int8 in-place (%d,%d)", i, j);
}

void int8_fused_case(int m, int n, int k) {
  ++g_cases;
  std::vector<uint8_t> A(static_cast<size_t>(m) * k);
  std::vector<int8_t> B(static_cast<size_t>(k) * n);
  std::vector<int32_t> C(static_cast<size_t>(m) * n, 0), D(C.size(), INT32_MIN), bias(n);
  std::mt19937 rng(7);
  for (auto& x : A) x = static_cast<uint8_t>(rng() & 0xFF);
  for (auto& x : B) x = static_cast<int8_t>(rng() & 0xFF);
  for (auto& x : bias) x = static_cast<int32_t>(rng() % 65537) - 32768;
  using Fused = cpu_ops::gemm::device::Gemm<
      uint8_t, RowMajor, int8_t, RowMajor, int32_t, RowMajor, int32_t,
      epilogue::LinearCombinationFused<int32_t, epilogue::BiasAdd<int32_t>, epilogue::Relu,
                                       epilogue::Clamp<int32_t>>,
      cpu_ops::mma::Vnni512GemmConfig, cpu_ops::mma::VnniPolicy<>>;
  typename Fused::Arguments args{
      {m, n, k}, {A.data(), k}, {B.data(), n}, {C.data(), n}, {D.data(), n},
      {1, 0,
       epilogue::Chain<epilogue::BiasAdd<int32_t>, epilogue::Relu, epilogue::Clamp<int32_t>>{
           epilogue::BiasAdd<int32_t>{bias.data()}, epilogue::Relu{},
           epilogue::Clamp<int32_t>{0, 1 << 20}}}};
  Fused op;
  CHECK(op(args) == Status::kSuccess, "fused int8: bad status (%s)", cpuops_b200_last_error());
  for (int i = 0; i < m; ++i)
    for (int j = 0; j < n; ++j) {
      int64_t acc = 0;
      for (int p = 0; p < k; ++p) acc += int64_t{A[size_t(i) * k + p]} * int64_t{B[size_t(p) * n + j]};
      int64_t v = acc + bias[j];
      v = v < 0 ? 0 : v;
      v = v > (1 << 20) ? (1 << 20) : v;
      CHECK(D[size_t(i) * n + j] == static_cast<int32_t>(v), "fused int8 (%d,%d): got %d want %lld", i,
            j, D[size_t(i) * n + j], (long long)v);
    }
}

template <typename T>
float decode_elem(const uint8_t* base, int row, int k, int ld) {
  if constexpr (std::is_same<T, fp4e2m1_t>::value) {
    const uint8_t byte = base[(static_cast<size_t>(row) * ld + k) / 2];
    return fp4e2m1_t::to_float((k & 1) ? (byte >> 4) : (byte & 0xF));
  } else {
    return T::to_float(base[static_cast<size_t>(row) * ld + k]);
  }
}

template <typename TA, typename TB, typename LC>
void mx_case(int m, int n, int k, float alpha, float beta, int split_k_slices = 0) {
  ++g_cases;
  const bool a_fp4 = std::is_same<TA, fp4e2m1_t>::value, b_fp4 = std::is_same<TB, fp4e2m1_t>::value;
  const int ld = (k + 3) & ~((a_fp4 || b_fp4) ? 1 : 0);
  const int ldc = (LC::kIsRowMajor ? n : m) + 3;
  const int kg = (k + 31) / 32, lds = kg + 1;
  std::vector<uint8_t> A(static_cast<size_t>(m) * (ld / (a_fp4 ? 2 : 1)), 0);
  std::vector<uint8_t> B(static_cast<size_t>(n) * (ld / (b_fp4 ? 2 : 1)), 0);
  std::vector<uint8_t> SA(static_cast<size_t>(m) * lds), SB(static_cast<size_t>(n) * lds);
  const size_t size_c = static_cast<size_t>(LC::kIsRowMajor ? m : n) * ldc;
  std::vector<float> C(size_c), D(size_c, std::numeric_limits<float>::quiet_NaN());
  std::mt19937 rng(static_cast<unsigned>(m * 131 + n * 17 + k));
  auto fill = [&](std::vector<uint8_t>& data, std::vector<uint8_t>& scales, bool e4m3, bool e5m2) {
    for (auto& b : data) {
      b = static_cast<uint8_t>(rng() & 0xFF);
      if (e4m3 && (b & 0x7F) == 0x7F) b &= 0xF7;
      if (e5m2 && (b & 0x7C) == 0x7C) b &= 0xBF;
    }
    for (auto& s : scales) s = static_cast<uint8_t>(124 + rng() % 7);
  };
  fill(A, SA, std::is_same<TA, fp8e4m3_t>::value, std::is_same<TA, fp8e5m2_t>::value);
  fill(B, SB, std::is_same<TB, fp8e4m3_t>::value, std::is_same<TB, fp8e5m2_t>::value);
  for (auto& x : C) x = static_cast<float>(static_cast<int>(rng() % 2001) - 1000) * 0.001f;

  using Op = cpu_ops::gemm::device::GemmMx<TA, TB, LC>;
  typename Op::Arguments args;
  args.problem_size = {m, n, k};
  args.ref_A = {A.data(), SA.data(), ld, lds};
  args.ref_B = {B.data(), SB.data(), ld, lds};
  args.ref_C = {C.data(), ldc};
  args.ref_D = {D.data(), ldc};
  args.epilogue = {alpha, beta};
  args.split_k_slices = split_k_slices;
  Op op;
  CHECK(op(args, 8) == Status::kSuccess, "mx %dx%dx%d: bad status (%s)", m, n, k,
        cpuops_b200_last_error());
  const double eps = std::numeric_limits<float>::epsilon();
  for (int i = 0; i < m; ++i)
    for (int j = 0; j < n; ++j) {
      double acc = 0.0, bnd = 0.0;
      for (int p = 0; p < k; ++p) {
        const double a = double(decode_elem<TA>(A.data(), i, p, ld)) *
                         cpu_ops::e8m0_to_float(SA[size_t(i) * lds + (p >> 5)]);
        const double b = double(decode_elem<TB>(B.data(), j, p, ld)) *
                         cpu_ops::e8m0_to_float(SB[size_t(j) * lds + (p >> 5)]);
        acc += a * b;
        bnd += std::fabs(a * b);
      }
      double want = double(alpha) * acc;
      if (beta != 0.f) want += double(beta) * C[LC::offset(i, j, ldc)];
      const double allowed = 8.0 * k * eps * bnd + 16.0 * eps * std::fabs(want) + 1e-12;
      const double got = D[LC::offset(i, j, ldc)];
      CHECK(std::fabs(got - want) <= allowed, "mx %dx%dx%d (%d,%d): got %g want %g", m, n, k, i, j, got,
            want);
    }
}

void status_cases(bool expect_device) {
  ++g_cases;
  using Op = cpu_ops::gemm::device::GemmMx<fp4e2m1_t, fp4e2m1_t, RowMajor>;
  Op op;
  std::vector<uint8_t> data(64, 0), scales(8, 127);
  std::vector<float> c(64, 0.f);
  typename Op::Arguments args;
  args.problem_size = {4, 4, 32};
  args.ref_A = {data.data(), scales.data(), 32, 1};
  args.ref_B = {data.data(), scales.data(), 32, 1};
  args.ref_C = {c.data(), 4};
  args.ref_D = {c.data(), 4};
  if (expect_device) {
    CHECK(op(args, 1) == Status::kSuccess, "valid fp4 problem rejected");
  } else {
    CHECK(op(args, 1) == Status::kErrorInternal, "without a GPU a valid problem must fail loudly");
  }
  args.ref_A.scales = nullptr;
  CHECK(op(args, 1) == Status::kErrorInvalidArguments, "null scales accepted");
  args.ref_A.scales = scales.data();
  args.ref_A.ld = 33;
  CHECK(op(args, 1) == Status::kErrorInvalidArguments, "odd fp4 ld accepted");
  args.ref_A.ld = 32;
  args.problem_size = {-1, 4, 32};
  CHECK(op(args, 1) == Status::kErrorInvalidProblem, "negative dim accepted");

  using I8 = cpu_ops::gemm::device::GemmU8S8S32<RowMajor, RowMajor, RowMajor>;
  std::vector<uint8_t> a(16);
  std::vector<int8_t> b(16);
  std::vector<int32_t> cc(16);
  I8 gi;
  typename I8::Arguments ia{{4, 4, 4}, {a.data(), 3}, {b.data(), 4}, {cc.data(), 4}, {cc.data(), 4}, {1, 0}};
  CHECK(gi(ia) == Status::kErrorInvalidArguments, "short lda accepted");
  typename I8::Arguments ib{{0, 4, 4}, {nullptr, 0}, {nullptr, 0}, {nullptr, 0}, {nullptr, 0}, {1, 0}};
  CHECK(gi(ib) == Status::kSuccess, "empty problem must succeed before pointer checks");
  typename I8::Arguments ic{{4, 4, 4}, {a.data(), 4}, {b.data(), 4}, {nullptr, 4}, {cc.data(), 4}, {1, 0}};
  CHECK(gi(ic) == Status::kErrorInvalidArguments, "null C accepted (it must be non-null even when beta == 0)");
}

int dump_codecs(const char* in_path, const char* out_path) {
  std::FILE* fi = std::fopen(in_path, "rb");
  std::FILE* fo = std::fopen(out_path, "wb");
  if (!fi || !fo) return 2;
  for (int c = 0; c < 256; ++c) { float f = fp8e4m3_t::to_float(uint8_t(c)); std::fwrite(&f, 4, 1, fo); }
  for (int c = 0; c < 256; ++c) { float f = fp8e5m2_t::to_float(uint8_t(c)); std::fwrite(&f, 4, 1, fo); }
  for (int c = 0; c < 16; ++c) { float f = fp4e2m1_t::to_float(uint8_t(c)); std::fwrite(&f, 4, 1, fo); }
  for (int c = 0; c < 256; ++c) { float f = cpu_ops::e8m0_to_float(uint8_t(c)); std::fwrite(&f, 4, 1, fo); }
  float x;
  while (std::fread(&x, 4, 1, fi) == 1) {
    const uint8_t enc[4] = {fp8e4m3_t::from_float(x), fp8e5m2_t::from_float(x), fp4e2m1_t::from_float(x),
                            cpu_ops::e8m0_from_float(x)};
    std::fwrite(enc, 1, 4, fo);
  }
  std::fclose(fi);
  std::fclose(fo);
  return 0;
}

}  // namespace

int main(int argc, char** argv) {
  const std::string mode = argc > 1 ? argv[1] : "--status";
  if (mode == "--codecs" && argc == 4) return dump_codecs(argv[2], argv[3]);
  if (mode == "--status") {
    status_cases(false);
  } else if (mode == "--gpu") {
    status_cases(true);
    int8_case<RowMajor, RowMajor, RowMajor>(65, 63, 67, 3, -2, false);
    int8_case<RowMajor, ColumnMajor, ColumnMajor>(17, 31, 257, 1, 0, false);
    int8_case<ColumnMajor, RowMajor, RowMajor>(129, 255, 97, 1, 1, true);
    int8_case<ColumnMajor, ColumnMajor, ColumnMajor>(5, 7, 9, 3, -2, false);
    int8_case<RowMajor, RowMajor, RowMajor>(16, 24, 0, 1, 5, false);
    int8_case<RowMajor, RowMajor, RowMajor>(32, 32, 8192, 1, 1, true);
    int8_fused_case(96, 160, 700);
    mx_case<fp8e4m3_t, fp8e4m3_t, RowMajor>(65, 63, 67, 1.0f, 0.0f);
    mx_case<fp8e4m3_t, fp8e4m3_t, ColumnMajor>(31, 17, 258, 2.0f, -0.5f);
    mx_case<fp8e5m2_t, fp8e5m2_t, RowMajor>(16, 6, 33, 1.0f, 0.25f);
    mx_case<fp4e2m1_t, fp4e2m1_t, RowMajor>(128, 256, 96, 1.0f, 0.0f);
    mx_case<fp4e2m1_t, fp4e2m1_t, ColumnMajor>(31, 17, 258, 0.5f, -0.5f);
    mx_case<fp8e4m3_t, fp8e4m3_t, RowMajor>(24, 40, 3000, 1.25f, 0.5f, 7);
    // any storage pair (gemm_mx.h:44-47)
    mx_case<fp8e4m3_t, fp8e5m2_t, RowMajor>(33, 47, 77, 1.0f, 0.5f);
    mx_case<fp8e4m3_t, fp4e2m1_t, RowMajor>(65, 63, 131, 1.0f, 0.0f);
    mx_case<fp4e2m1_t, fp8e5m2_t, ColumnMajor>(40, 24, 256, 0.5f, 0.25f);
  } else {
    std::printf("usage: compat_call_sites --status | --gpu | --codecs in out\n");
    return 2;
  }
  std::printf("compat_call_sites: %d cases, %d failures\n", g_cases, g_failures);
  return g_failures == 0 ? 0 : 1;
}
