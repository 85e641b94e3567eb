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

// One chain op on a 32-column chunk of one accumulator row (registers r[0..32)).  The
// opcode is uniform over the kernel, so it is dispatched once per chunk, outside the
// element loop; a vector indexed by column is fetched as eight 16-byte loads (the same
// addresses in every lane: one broadcast transaction each), a vector indexed by row as
// one load.  Columns at or beyond `ncols` are computed on harmlessly and never stored.
// The arithmetic per element is exactly apply_op_bits'.
template <bool kInt>
__device__ __forceinline__ void apply_op_chunk(const EpilogueOp& op, uint32_t (&r)[32], int krow,
                                               int kcol0, int ncols) {
  const int code = op.opcode;
  if (code == kOpBiasAdd || code == kOpScalePerRow || code == kOpScalePerCol) {
    uint32_t v[32];
    const uint32_t* vec = static_cast<const uint32_t*>(op.ptr);
    if (op.index_by_krow) {
      const uint32_t x = __ldg(vec + krow);
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = x;
    } else if (ncols == 32 && (reinterpret_cast<uintptr_t>(vec + kcol0) & 15u) == 0) {
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(vec + kcol0 + i));
        v[i] = q.x; v[i + 1] = q.y; v[i + 2] = q.z; v[i + 3] = q.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = i < ncols ? __ldg(vec + kcol0 + i) : 0u;
    }
    if constexpr (kInt) {
      if (code == kOpBiasAdd) {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] += v[i];
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] *= v[i];
      }
    } else {
      if (code == kOpBiasAdd) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          r[i] = __float_as_uint(__fadd_rn(__uint_as_float(r[i]), __uint_as_float(v[i])));
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          r[i] = __float_as_uint(__fmul_rn(__uint_as_float(r[i]), __uint_as_float(v[i])));
      }
    }
  } else if (code == kOpRelu) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if constexpr (kInt) {
        r[i] = static_cast<int32_t>(r[i]) < 0 ? 0u : r[i];
      } else {
        r[i] = __uint_as_float(r[i]) < 0.0f ? 0u : r[i];  // x < 0 ? +0.0f : x (NaN and -0.0 pass)
      }
    }
  } else if (code == kOpClamp) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if constexpr (kInt) {
        const int32_t lo = static_cast<int32_t>(op.lo), hi = static_cast<int32_t>(op.hi);
        const int32_t x = static_cast<int32_t>(r[i]);
        r[i] = static_cast<uint32_t>(x < lo ? lo : (hi < x ? hi : x));
      } else {
        const float lo = __uint_as_float(op.lo), hi = __uint_as_float(op.hi);
        const float x = __uint_as_float(r[i]);
        r[i] = __float_as_uint(x < lo ? lo : (hi < x ? hi : x));
      }
    }
  } else if (code == kOpGelu || code == kOpSilu) {
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = apply_op_bits<kInt>(op, r[i], krow, kcol0 + i);
  }
}

// Reads every field of the epilogue parameters once.  Kernel parameters live in constant
// memory, and a field's first read on an SM misses the constant cache (measured: about
// 0.6 us).  The epilogue warps call this while they are still waiting for their first
// accumulator, so that the misses are not paid between the last MMA and the first store.
__device__ __forceinline__ void warm_epilogue_params(const EpilogueParams& e) {
  uint32_t sink = e.alpha ^ e.beta ^ static_cast<uint32_t>(e.beta_nonzero) ^ static_cast<uint32_t>(e.activation) ^
                  static_cast<uint32_t>(e.n_ops) ^ static_cast<uint32_t>(reinterpret_cast<uintptr_t>(e.D)) ^
                  static_cast<uint32_t>(reinterpret_cast<uintptr_t>(e.C)) ^ static_cast<uint32_t>(e.d_sr) ^
                  static_cast<uint32_t>(e.d_sc) ^ static_cast<uint32_t>(e.c_sr) ^ static_cast<uint32_t>(e.c_sc);
#pragma unroll
  for (int t = 0; t < kMaxOps; ++t)
    sink ^= static_cast<uint32_t>(e.ops[t].opcode) ^ static_cast<uint32_t>(reinterpret_cast<uintptr_t>(e.ops[t].ptr)) ^
            e.ops[t].lo ^ e.ops[t].hi;
  asm volatile("" ::"r"(sink));
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
