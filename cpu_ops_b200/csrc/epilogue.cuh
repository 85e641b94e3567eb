// Device-side epilogue: D = chain(act(alpha * acc + beta * C)).
//
// Arithmetic contract (what the CPU library computes, element by element):
//   s32: alpha*acc + beta*C in wrap-around 32-bit arithmetic; C is not read
//        when beta == 0  (epilogue/linear_combination.h:33-38, integer branch)
//   f32: beta != 0 ? fma(beta, C, alpha*acc) : alpha*acc   (:27-31)
//   then Activation::kRelu (:85-87), then the chain ops in order
//   (epilogue/fusion.h:31-129, 136-166).
// Gelu/Silu are evaluated in f32 (tanhf / expf); the CPU library itself mixes
// a polynomial vector form and a double-precision scalar form for them, so
// they are compared with a tolerance, never bit for bit.
#pragma once

#include "gemm_params.h"

namespace b200 {

template <bool kInt>
__device__ __forceinline__ uint32_t linear_combine_bits(const EpilogueParams& e, uint32_t acc,
                                                        uint32_t src) {
  if constexpr (kInt) {
    uint32_t v = e.alpha * acc;
    if (e.beta_nonzero) v += e.beta * src;
    if (e.activation == 1 && static_cast<int32_t>(v) < 0) v = 0;
    return v;
  } else {
    const float a = __uint_as_float(e.alpha), b = __uint_as_float(e.beta);
    float v = __fmul_rn(a, __uint_as_float(acc));
    if (e.beta_nonzero) v = __fmaf_rn(b, __uint_as_float(src), v);
    if (e.activation == 1) v = v < 0.0f ? 0.0f : v;
    return __float_as_uint(v);
  }
}

template <bool kInt>
__device__ __forceinline__ uint32_t apply_op_bits(const EpilogueOp& op, uint32_t x, int krow,
                                                  int kcol) {
  const int idx = op.index_by_krow ? krow : kcol;
  if constexpr (kInt) {
    int32_t v = static_cast<int32_t>(x);
    switch (op.opcode) {
      case kOpRelu: v = v < 0 ? 0 : v; break;
      case kOpClamp: {
        const int32_t lo = static_cast<int32_t>(op.lo), hi = static_cast<int32_t>(op.hi);
        v = v < lo ? lo : (hi < v ? hi : v);
        break;
      }
      case kOpBiasAdd:
        v = static_cast<int32_t>(static_cast<uint32_t>(v) +
                                 static_cast<uint32_t>(__ldg(static_cast<const int32_t*>(op.ptr) + idx)));
        break;
      case kOpScalePerRow:
      case kOpScalePerCol:
        v = static_cast<int32_t>(static_cast<uint32_t>(v) *
                                 static_cast<uint32_t>(__ldg(static_cast<const int32_t*>(op.ptr) + idx)));
        break;
      default: break;
    }
    return static_cast<uint32_t>(v);
  } else {
    float v = __uint_as_float(x);
    switch (op.opcode) {
      case kOpRelu: v = v < 0.0f ? 0.0f : v; break;
      case kOpClamp: {
        const float lo = __uint_as_float(op.lo), hi = __uint_as_float(op.hi);
        v = v < lo ? lo : (hi < v ? hi : v);
        break;
      }
      case kOpBiasAdd: v = __fadd_rn(v, __ldg(static_cast<const float*>(op.ptr) + idx)); break;
      case kOpScalePerRow:
      case kOpScalePerCol: v = __fmul_rn(v, __ldg(static_cast<const float*>(op.ptr) + idx)); break;
      case kOpGelu: {
        const float inner = 0.7978845608028654f * (v + 0.044715f * v * v * v);
        v = 0.5f * (v * (1.0f + tanhf(inner)));
        break;
      }
      case kOpSilu: v = v / (1.0f + expf(-v)); break;
      default: break;
    }
    return __float_as_uint(v);
  }
}

// One element, all steps (used by the split-k reduce and k == 0 kernels).
template <bool kInt>
__device__ __forceinline__ uint32_t epilogue_element(const EpilogueParams& e, uint32_t acc,
                                                     int krow, int kcol) {
  uint32_t src = 0;
  if (e.beta_nonzero) {
    // plain load: C may alias D, which this kernel writes
    src = static_cast<const uint32_t*>(e.C)[krow * e.c_sr + kcol * e.c_sc];
  }
  uint32_t v = linear_combine_bits<kInt>(e, acc, src);
  for (int t = 0; t < e.n_ops; ++t) v = apply_op_bits<kInt>(e.ops[t], v, krow, kcol);
  return v;
}

}  // namespace b200
