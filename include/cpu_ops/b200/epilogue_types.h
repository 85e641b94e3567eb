// Epilogue parameter types of the cpu_ops call surface, as plain descriptors:
//   Activation, LinearCombination<T>::Params     epilogue/linear_combination.h:12-15,70-76
//   Relu, Gelu, Silu, Clamp<T>, BiasAdd<T>, ScalePerRow<T>, ScalePerCol<T>,
//   Chain<Ops...>, LinearCombinationFused<T, Ops...>::Params
//                                                 epilogue/fusion.h:31-195
// In the CPU library these are functors applied inside the mainloop; here they
// only carry their parameters to the GPU epilogue, which applies the same
// arithmetic (see cpu_ops_b200/csrc/epilogue.cuh).  User-defined functors cannot
// cross the C ABI and are rejected at compile time.
#ifndef CPU_OPS_B200_EPILOGUE_TYPES_H_
#define CPU_OPS_B200_EPILOGUE_TYPES_H_

#include <cstddef>
#include <cstring>
#include <tuple>
#include <type_traits>
#include <utility>

#include "cpu_ops_b200.h"

namespace cpu_ops {
namespace epilogue {

enum class Activation {
  kNone,
  kRelu,
};

template <typename T>
struct LinearCombination {
  using ElementType = T;
  struct Params {
    T alpha = T(1);
    T beta = T(0);
    Activation activation = Activation::kNone;
  };
  Params params;
  LinearCombination() = default;
  explicit LinearCombination(const Params& p) : params(p) {}
};

struct Relu {};
struct Gelu {};
struct Silu {};

template <typename T>
struct Clamp {
  T lo;
  T hi;
};

template <typename T>
struct BiasAdd {
  const T* bias = nullptr;
};

template <typename T>
struct ScalePerRow {
  const T* scale = nullptr;
};

template <typename T>
struct ScalePerCol {
  const T* scale = nullptr;
};

template <typename... Ops>
struct Chain {
  std::tuple<Ops...> ops;
  Chain(Ops... o) : ops(std::move(o)...) {}
};

template <typename T, typename... Ops>
struct LinearCombinationFused {
  using ElementType = T;
  struct Params {
    T alpha = T(1);
    T beta = T(0);
    Chain<Ops...> chain{};
  };
  Params params;
  LinearCombinationFused() = default;
  explicit LinearCombinationFused(const Params& p) : params(p) {}
};

}  // namespace epilogue

namespace b200_detail {

template <typename T>
inline void store_scalar(cpuops_b200_scalar* dst, T value) {
  static_assert(sizeof(T) == 4, "s32 or f32 accumulators");
  std::memcpy(dst, &value, 4);
}

// One chain op -> one C-ABI record.  Unknown op types fail to compile.
template <typename T, typename Op>
struct OpRecord {
  static_assert(sizeof(Op) == 0,
                "this epilogue op is not one of Relu, Gelu, Silu, Clamp, BiasAdd, ScalePerRow, "
                "ScalePerCol: user functors cannot be forwarded to the GPU library");
};
template <typename T>
struct OpRecord<T, epilogue::Relu> {
  static void fill(const epilogue::Relu&, cpuops_b200_epilogue_op* r) { r->opcode = CPUOPS_B200_OP_RELU; }
};
template <typename T>
struct OpRecord<T, epilogue::Gelu> {
  static_assert(std::is_same<T, float>::value, "Gelu needs f32 accumulators");
  static void fill(const epilogue::Gelu&, cpuops_b200_epilogue_op* r) { r->opcode = CPUOPS_B200_OP_GELU; }
};
template <typename T>
struct OpRecord<T, epilogue::Silu> {
  static_assert(std::is_same<T, float>::value, "Silu needs f32 accumulators");
  static void fill(const epilogue::Silu&, cpuops_b200_epilogue_op* r) { r->opcode = CPUOPS_B200_OP_SILU; }
};
template <typename T, typename U>
struct OpRecord<T, epilogue::Clamp<U>> {
  static void fill(const epilogue::Clamp<U>& op, cpuops_b200_epilogue_op* r) {
    r->opcode = CPUOPS_B200_OP_CLAMP;
    store_scalar(&r->lo, static_cast<T>(op.lo));
    store_scalar(&r->hi, static_cast<T>(op.hi));
  }
};
template <typename T>
struct OpRecord<T, epilogue::BiasAdd<T>> {
  static void fill(const epilogue::BiasAdd<T>& op, cpuops_b200_epilogue_op* r) {
    r->opcode = CPUOPS_B200_OP_BIAS_ADD;
    r->ptr = op.bias;
  }
};
template <typename T>
struct OpRecord<T, epilogue::ScalePerRow<T>> {
  static void fill(const epilogue::ScalePerRow<T>& op, cpuops_b200_epilogue_op* r) {
    r->opcode = CPUOPS_B200_OP_SCALE_PER_ROW;
    r->ptr = op.scale;
  }
};
template <typename T>
struct OpRecord<T, epilogue::ScalePerCol<T>> {
  static void fill(const epilogue::ScalePerCol<T>& op, cpuops_b200_epilogue_op* r) {
    r->opcode = CPUOPS_B200_OP_SCALE_PER_COL;
    r->ptr = op.scale;
  }
};

template <typename T, typename... Ops, std::size_t... I>
inline void fill_chain(const epilogue::Chain<Ops...>& chain, cpuops_b200_gemm_desc* d,
                       std::index_sequence<I...>) {
  static_assert(sizeof...(Ops) <= CPUOPS_B200_MAX_OPS, "too many ops in the epilogue chain");
  (OpRecord<T, Ops>::fill(std::get<I>(chain.ops), &d->ops[I]), ...);
  d->n_ops = static_cast<int32_t>(sizeof...(Ops));
}

// Epilogue::Params -> descriptor fields, for the two epilogue templates.
template <typename Epilogue>
struct EpilogueToDesc {
  static_assert(sizeof(Epilogue) == 0,
                "Epilogue must be epilogue::LinearCombination<T> or "
                "epilogue::LinearCombinationFused<T, Ops...>");
};
template <typename T>
struct EpilogueToDesc<epilogue::LinearCombination<T>> {
  static void fill(const typename epilogue::LinearCombination<T>::Params& p, cpuops_b200_gemm_desc* d) {
    store_scalar(&d->alpha, p.alpha);
    store_scalar(&d->beta, p.beta);
    d->activation = p.activation == epilogue::Activation::kRelu ? CPUOPS_B200_ACT_RELU : CPUOPS_B200_ACT_NONE;
    d->n_ops = 0;
  }
};
template <typename T, typename... Ops>
struct EpilogueToDesc<epilogue::LinearCombinationFused<T, Ops...>> {
  static void fill(const typename epilogue::LinearCombinationFused<T, Ops...>::Params& p,
                   cpuops_b200_gemm_desc* d) {
    store_scalar(&d->alpha, p.alpha);
    store_scalar(&d->beta, p.beta);
    d->activation = CPUOPS_B200_ACT_NONE;
    fill_chain<T>(p.chain, d, std::index_sequence_for<Ops...>{});
  }
};

}  // namespace b200_detail
}  // namespace cpu_ops

#endif  // CPU_OPS_B200_EPILOGUE_TYPES_H_
