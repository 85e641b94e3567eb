// Source-compatible value types of the cpu_ops call surface, for callers that
// build against the B200 library instead of the CPU headers.  Same names,
// namespaces, members and enumerator values as the reference:
//   Status        include/cpu_ops/status.h:5-9
//   GemmCoord     include/cpu_ops/gemm_coord.h:6-13
//   layout::*     include/cpu_ops/layout/matrix.h:9-22
//   TensorRef     include/cpu_ops/tensor_ref.h:6-27
#ifndef CPU_OPS_B200_CORE_TYPES_H_
#define CPU_OPS_B200_CORE_TYPES_H_

#include <cstdint>

namespace cpu_ops {

// The first three values are the reference's; kErrorInternal is appended for
// failures that only a GPU runtime can have (no device, CUDA error, device-side
// timeout, feature not built), so existing values keep their numbers.
enum class Status {
  kSuccess = 0,
  kErrorInvalidProblem,
  kErrorInvalidArguments,
  kErrorInternal,
};

struct GemmCoord {
  int m = 0, n = 0, k = 0;
  GemmCoord() = default;
  constexpr GemmCoord(int rows, int cols, int depth) : m(rows), n(cols), k(depth) {}
};

namespace layout {

struct RowMajor {
  static constexpr bool kIsRowMajor = true;
  static constexpr int64_t offset(int row, int col, int ld) {
    return int64_t{row} * ld + col;
  }
};

struct ColumnMajor {
  static constexpr bool kIsRowMajor = false;
  static constexpr int64_t offset(int row, int col, int ld) {
    return int64_t{col} * ld + row;
  }
};

}  // namespace layout

// Borrowed pointer + leading dimension (in elements).  Host or device memory.
template <typename T, typename Layout>
class TensorRef {
 public:
  using Element = T;
  using LayoutType = Layout;

  TensorRef() = default;
  TensorRef(T* ptr, int ld) : ptr_(ptr), ld_(ld) {}

  T* data() const { return ptr_; }
  int ld() const { return ld_; }
  // Element access is only meaningful for host memory.
  T& at(int row, int col) const { return ptr_[Layout::offset(row, col, ld_)]; }
  TensorRef subrect(int row, int col) const {
    return TensorRef(ptr_ + Layout::offset(row, col, ld_), ld_);
  }

 private:
  T* ptr_ = nullptr;
  int ld_ = 0;
};

}  // namespace cpu_ops

#endif  // CPU_OPS_B200_CORE_TYPES_H_
