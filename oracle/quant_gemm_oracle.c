/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement ("oracle") of the quantized-GEMM
 * path of napplesty/cpu_ops. Nothing in the product library links, loads or
 * calls this file; only the test-suite, the smoke check and the benchmark's
 * CPU-baseline leg do, as the checker.
 *
 * Parity status: PINNED. Every entry point below is checked (see
 * tests/test_oracle_pins.py) against
 *   - the known-answer decode values of the reference's own test
 *     (test/test_gemm_mx.cc:38-67), and
 *   - outputs of the unmodified reference headers compiled into
 *     oracle/_ref (oracle/ref_shim.cc), committed as tests/golden fixtures.
 *
 * Each function cites the reference file:line it restates (paths relative to
 * the reference project root).  Plain C99, scalar, single threaded; compile
 * with -ffp-contract=off so that only the explicit fmaf() calls fuse.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* Element formats: include/cpu_ops/mx_formats.h                             */
/* ------------------------------------------------------------------------- */

static float bits_to_float(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static uint32_t float_to_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}

/* e4m3: bias 7, no infinity, S.1111.111 is NaN, denormals m * 2^-9.
 * mx_formats.h:30-56. */
ORACLE_API float oracle_decode_e4m3(uint8_t v) {
  const uint32_t sign = (uint32_t)(v >> 7) << 31;
  const int exp = (v >> 3) & 0xF;
  const int mant = v & 0x7;
  if (exp == 0) {
    const float mag = ldexpf((float)mant, -9);
    return bits_to_float(float_to_bits(mag) | sign);
  }
  if (exp == 15 && mant == 7) return bits_to_float(sign | 0x7FC00000u);
  return bits_to_float(sign | ((uint32_t)(exp - 7 + 127) << 23) | ((uint32_t)mant << 20));
}

/* e5m2: bias 15, inf (exp 31, mant 0) and NaN, denormals m * 2^-16.
 * mx_formats.h:60-88. */
ORACLE_API float oracle_decode_e5m2(uint8_t v) {
  const uint32_t sign = (uint32_t)(v >> 7) << 31;
  const int exp = (v >> 2) & 0x1F;
  const int mant = v & 0x3;
  if (exp == 0) {
    const float mag = ldexpf((float)mant, -16);
    return bits_to_float(float_to_bits(mag) | sign);
  }
  if (exp == 31) return bits_to_float(sign | 0x7F800000u | ((uint32_t)mant << 21));
  return bits_to_float(sign | ((uint32_t)(exp - 15 + 127) << 23) | ((uint32_t)mant << 21));
}

/* e2m1: +-{0, .5, 1, 1.5, 2, 3, 4, 6}.  mx_formats.h:91-107. */
ORACLE_API float oracle_decode_e2m1(uint8_t nibble) {
  static const float mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
  const float m = mag[nibble & 7];
  return (nibble & 8) ? -m : m;
}

/* E8M0: 2^(e-127); e == 0 is the f32 denormal 2^-127, 0xFF is NaN.
 * mx_formats.h:253-263. */
ORACLE_API float oracle_decode_e8m0(uint8_t e) {
  if (e == 0) return bits_to_float(0x00400000u);
  if (e == 0xFF) return bits_to_float(0x7FC00000u);
  return bits_to_float((uint32_t)e << 23);
}

/* Encoders (host-side data preparation in the reference's tests).
 * e4m3: RNE, saturating to +-448, NaN -> NaN.  mx_formats.h:123-153. */
ORACLE_API uint8_t oracle_encode_e4m3(float x) {
  const uint32_t f = float_to_bits(x);
  const uint32_t sign = (f >> 24) & 0x80;
  const uint32_t fexp = (f >> 23) & 0xFF;
  const uint32_t mant = f & 0x7FFFFF;
  if (fexp == 0xFF) return (uint8_t)(sign | (mant ? 0x7F : 0x7E));
  const int e = (int)fexp - 127 + 7;
  if (e > 15) return (uint8_t)(sign | 0x7E);
  if (e <= 0) {
    const int e_unb = (int)fexp - 127;
    if (e_unb < -10) return (uint8_t)sign;
    const uint32_t mant24 = mant | 0x800000;
    const int shift = 14 - e_unb;
    uint32_t m3 = mant24 >> shift;
    const uint32_t rem = mant24 & ((1u << shift) - 1);
    const uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (m3 & 1))) ++m3;
    return (uint8_t)(sign | m3);
  }
  uint32_t half = ((uint32_t)e << 3) | (mant >> 20);
  const uint32_t rem = mant & 0xFFFFF;
  if (rem > 0x80000 || (rem == 0x80000 && (half & 1))) ++half;
  if (half > 0x7E) half = 0x7E;
  return (uint8_t)(sign | half);
}

/* e5m2: RNE, overflow to infinity.  mx_formats.h:173-199. */
ORACLE_API uint8_t oracle_encode_e5m2(float x) {
  const uint32_t f = float_to_bits(x);
  const uint32_t sign = (f >> 24) & 0x80;
  const uint32_t fexp = (f >> 23) & 0xFF;
  const uint32_t mant = f & 0x7FFFFF;
  if (fexp == 0xFF) return (uint8_t)(sign | 0x7C | (mant ? 0x2 : 0));
  const int e = (int)fexp - 127 + 15;
  if (e >= 31) return (uint8_t)(sign | 0x7C);
  if (e <= 0) {
    const int e_unb = (int)fexp - 127;
    if (e_unb < -17) return (uint8_t)sign;
    const uint32_t mant24 = mant | 0x800000;
    const int shift = 7 - e_unb;
    uint32_t m2 = mant24 >> shift;
    const uint32_t rem = mant24 & ((1u << shift) - 1);
    const uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (m2 & 1))) ++m2;
    return (uint8_t)(sign | m2);
  }
  uint32_t half = ((uint32_t)e << 2) | (mant >> 21);
  const uint32_t rem = mant & 0x1FFFFF;
  if (rem > 0x100000 || (rem == 0x100000 && (half & 1))) ++half;
  return (uint8_t)(sign | half);
}

/* e2m1: RNE with ties to the even code, NaN -> 0, saturating at 6.
 * mx_formats.h:212-249 (the thresholds are the midpoints of the value grid). */
ORACLE_API uint8_t oracle_encode_e2m1(float x) {
  if (x != x) return 0;
  const uint8_t sign = signbit(x) ? 0x8 : 0x0;
  const float a = fabsf(x);
  /* midpoints between consecutive magnitudes; a tie picks the even code */
  static const float mid[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f};
  uint8_t code = 7;
  for (int i = 0; i < 7; ++i) {
    if (a < mid[i]) { code = (uint8_t)i; break; }
    if (a == mid[i]) { code = (uint8_t)((i & 1) ? i + 1 : i); break; }
  }
  return (uint8_t)(sign | code);
}

/* E8M0 encoder: nearest power of two, ties up, clamp.  mx_formats.h:265-278. */
ORACLE_API uint8_t oracle_encode_e8m0(float x) {
  const uint32_t f = float_to_bits(x);
  if ((f & 0x7FFFFFFF) > 0x7F800000) return 0xFF;
  const uint32_t fexp = (f >> 23) & 0xFF;
  if (fexp == 0) return 0;
  const int e = (int)fexp - 127;
  const uint32_t mant = f & 0x7FFFFF;
  int r = e + (mant > 0x3504F3 ? 1 : 0);
  if (r < -127) r = -127;
  if (r > 127) r = 127;
  return (uint8_t)(r + 127);
}

/* ------------------------------------------------------------------------- */
/* Epilogue: epilogue/linear_combination.h, epilogue/fusion.h                */
/* ------------------------------------------------------------------------- */

enum {
  ORACLE_OP_RELU = 1,          /* fusion.h:31-40   x < 0 ? 0 : x          */
  ORACLE_OP_CLAMP = 2,         /* fusion.h:82-93   x<lo?lo:(hi<x?hi:x)    */
  ORACLE_OP_BIAS_ADD = 3,      /* fusion.h:96-105  x + bias[col]          */
  ORACLE_OP_SCALE_PER_ROW = 4, /* fusion.h:108-117 x * scale[row]         */
  ORACLE_OP_SCALE_PER_COL = 5, /* fusion.h:120-129 x * scale[col]         */
  ORACLE_OP_GELU = 6,          /* fusion.h:43-60   scalar (double) form   */
  ORACLE_OP_SILU = 7           /* fusion.h:63-78   scalar (double) form   */
};

typedef struct oracle_op {
  int32_t opcode;
  int32_t pad;
  const void* ptr; /* bias / scale vector (element type of the accumulator) */
  union { int32_t i; float f; } lo;
  union { int32_t i; float f; } hi;
} oracle_op;

static int64_t c_offset(int row_major, int64_t i, int64_t j, int64_t ld) {
  /* layout/matrix.h:9-22 */
  return row_major ? i * ld + j : j * ld + i;
}

/* Integer chain in wrap-around s32 (computed in uint32 to stay defined). */
static int32_t chain_s32(int32_t x, int n_ops, const oracle_op* ops, int row, int col) {
  for (int t = 0; t < n_ops; ++t) {
    const oracle_op* op = &ops[t];
    switch (op->opcode) {
      case ORACLE_OP_RELU: x = x < 0 ? 0 : x; break;
      case ORACLE_OP_CLAMP: x = x < op->lo.i ? op->lo.i : (op->hi.i < x ? op->hi.i : x); break;
      case ORACLE_OP_BIAS_ADD:
        x = (int32_t)((uint32_t)x + (uint32_t)((const int32_t*)op->ptr)[col]);
        break;
      case ORACLE_OP_SCALE_PER_ROW:
        x = (int32_t)((uint32_t)x * (uint32_t)((const int32_t*)op->ptr)[row]);
        break;
      case ORACLE_OP_SCALE_PER_COL:
        x = (int32_t)((uint32_t)x * (uint32_t)((const int32_t*)op->ptr)[col]);
        break;
      default: break;
    }
  }
  return x;
}

static float chain_f32(float x, int n_ops, const oracle_op* ops, int row, int col) {
  for (int t = 0; t < n_ops; ++t) {
    const oracle_op* op = &ops[t];
    switch (op->opcode) {
      case ORACLE_OP_RELU: x = x < 0.0f ? 0.0f : x; break;
      case ORACLE_OP_CLAMP: x = x < op->lo.f ? op->lo.f : (op->hi.f < x ? op->hi.f : x); break;
      case ORACLE_OP_BIAS_ADD: x = x + ((const float*)op->ptr)[col]; break;
      case ORACLE_OP_SCALE_PER_ROW: x = x * ((const float*)op->ptr)[row]; break;
      case ORACLE_OP_SCALE_PER_COL: x = x * ((const float*)op->ptr)[col]; break;
      case ORACLE_OP_GELU: {
        const double d = (double)x;
        const double inner = 0.7978845608028654 * (d + 0.044715 * d * d * d);
        x = (float)(0.5 * (d * (1.0 + tanh(inner))));
        break;
      }
      case ORACLE_OP_SILU: {
        const double d = (double)x;
        x = (float)(d / (1.0 + exp(-d)));
        break;
      }
      default: break;
    }
  }
  return x;
}

/* ------------------------------------------------------------------------- */
/* u8 x s8 -> s32                                                            */
/* ------------------------------------------------------------------------- */

/*
 * gemm/device/gemm.h:99-127 (validation order and status codes),
 * gemm/threadblock/mma_policy_vnni.h:80-95 + arch/simd.h:119-133 (the
 * non-saturating 4-way u8*s8 dot product, wrap-around s32),
 * epilogue/linear_combination.h:26-39 (integer branch) and
 * gemm/kernel/run_blocked.h:30-36 (k == 0).  In Z/2^32 the reference's
 * per-k-block update  D = alpha*acc0 + beta*C ; D += alpha*acc_b  equals
 * alpha*acc + beta*C evaluated once, for any blocking or split-k, so the
 * oracle reduces fully first.  activation: 0 none, 1 relu
 * (linear_combination.h:80-89).  Returns the reference Status value:
 * 0 success, 1 invalid problem, 2 invalid arguments.
 */
ORACLE_API int oracle_gemm_u8s8s32(int m, int n, int k, const uint8_t* A, int lda,
                                   int a_row_major, const int8_t* B, int ldb,
                                   int b_row_major, const int32_t* C, int ldc, int32_t* D,
                                   int ldd, int c_row_major, int32_t alpha, int32_t beta,
                                   int activation, int n_ops, const oracle_op* ops) {
  if (m < 0 || n < 0 || k < 0) return 1;
  if (m == 0 || n == 0) return 0;
  if (k > 0) {
    if (!A || !B || !C || !D) return 2;
    if (lda < (a_row_major ? k : m) || ldb < (b_row_major ? n : k) ||
        ldc < (c_row_major ? n : m) || ldd < (c_row_major ? n : m))
      return 2;
  }
  for (int i = 0; i < m; ++i) {
    for (int j = 0; j < n; ++j) {
      uint32_t acc = 0;
      for (int p = 0; p < k; ++p) {
        const int32_t a = A[c_offset(a_row_major, i, p, lda)];
        const int32_t b = B[c_offset(b_row_major, p, j, ldb)];
        acc += (uint32_t)(a * b);
      }
      uint32_t v = (uint32_t)alpha * acc;
      if (beta != 0) v += (uint32_t)beta * (uint32_t)C[c_offset(c_row_major, i, j, ldc)];
      int32_t x = (int32_t)v;
      if (activation == 1) x = x < 0 ? 0 : x;
      x = chain_s32(x, n_ops, ops, i, j);
      D[c_offset(c_row_major, i, j, ldd)] = x;
    }
  }
  return 0;
}

/* ------------------------------------------------------------------------- */
/* MX (block-scaled) GEMM                                                    */
/* ------------------------------------------------------------------------- */

enum { ORACLE_FMT_E4M3 = 2, ORACLE_FMT_E5M2 = 3, ORACLE_FMT_E2M1 = 4 };

/* Element (row, kk) of an MX operand, decoded and block-scaled in f32:
 * gemm/threadblock/mma_policy_mx.h:171-198 (decode * scale, one f32 multiply)
 * and mx_formats.h:280-295 (addressing: data[(row*ld+kk)/elems_per_byte],
 * scales[row*ld_scales + kk/32]; fp4 even index in the low nibble). */
static float mx_elem(int fmt, const uint8_t* data, const uint8_t* scales, int64_t ld,
                     int64_t ld_scales, int row, int kk) {
  float e;
  if (fmt == ORACLE_FMT_E2M1) {
    const uint8_t byte = data[((int64_t)row * ld + kk) >> 1];
    e = oracle_decode_e2m1((kk & 1) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 0xF));
  } else if (fmt == ORACLE_FMT_E4M3) {
    e = oracle_decode_e4m3(data[(int64_t)row * ld + kk]);
  } else {
    e = oracle_decode_e5m2(data[(int64_t)row * ld + kk]);
  }
  return e * oracle_decode_e8m0(scales[(int64_t)row * ld_scales + (kk >> 5)]);
}

/* threadblock_swizzle.h:31-37: balanced contiguous split of `count`. */
static void split_range(int count, int parts, int idx, int* begin, int* length) {
  const int base = count / parts;
  const int rem = count % parts;
  *begin = idx * base + (idx < rem ? idx : rem);
  *length = base + (idx < rem ? 1 : 0);
}

static int mx_validate(int m, int n, int k, const void* A, const void* SA, int lda, int ldsa,
                       int fmt_a, const void* B, const void* SB, int ldb, int ldsb,
                       int fmt_b, const void* C, int ldc, const void* D, int ldd,
                       int c_row_major) {
  /* gemm/device/gemm_mx.h:78-112 */
  if (m < 0 || n < 0 || k < 0) return 1;
  if (m == 0 || n == 0) return 0;
  if (k == 0) return 0;
  if (!A || !SA || !B || !SB || !C || !D) return 2;
  const int sld = (k + 31) / 32;
  if (lda < k || ldb < k || ldsa < sld || ldsb < sld) return 2;
  if ((fmt_a == ORACLE_FMT_E2M1 && (lda & 1)) || (fmt_b == ORACLE_FMT_E2M1 && (ldb & 1))) return 2;
  const int ldc_min = c_row_major ? n : m;
  if (ldc < ldc_min || ldd < ldc_min) return 2;
  return 0;
}

/*
 * D = chain(alpha * (A.sA)(B.sB) + beta * C) with the reference's f32
 * arithmetic order:
 *   - per KC-block, per output element, acc = fmaf(a'_k, b'_k, acc) for
 *     ascending k, one accumulator per element (arch/mma_atom.h:29-38);
 *   - first block: beta != 0 ? fmaf(beta, C, alpha*acc) : alpha*acc;
 *     later blocks: fmaf(alpha, acc, D)   (epilogue/linear_combination.h:26-39,
 *     invoked per KC block by gemm/threadblock/block_gemm.h:65-78,119-150);
 *   - activation / chain on the last block only;
 *   - split-k (slices > 1): slice s reduces its k range (balanced contiguous
 *     split, threadblock_swizzle.h:75-78) into a slab with PartialSum
 *     (epilogue/partial_sum.h:19-28), slabs are summed ((w0+w1)+w2)+... and
 *     the epilogue runs once with first=last=true (run_blocked.h:40-75);
 *   - k == 0: D = epilogue(0, C)  (run_blocked.h:30-36).
 * kc is the reference's KC (512 on AVX-512 hosts, 256 otherwise:
 * gemm_mx.h:31-40).  slices <= 1 means unsplit.  B is stored as n rows of k.
 */
ORACLE_API int oracle_gemm_mx(int m, int n, int k, int fmt_a, const uint8_t* A,
                              const uint8_t* SA, int lda, int ldsa, int fmt_b,
                              const uint8_t* B, const uint8_t* SB, int ldb, int ldsb,
                              const float* C, int ldc, float* D, int ldd, int c_row_major,
                              float alpha, float beta, int activation, int n_ops,
                              const oracle_op* ops, int kc, int slices) {
  const int st = mx_validate(m, n, k, A, SA, lda, ldsa, fmt_a, B, SB, ldb, ldsb, fmt_b, C,
                             ldc, D, ldd, c_row_major);
  if (st != 0 || m == 0 || n == 0) return st;
  if (kc <= 0) kc = 512;
  if (slices < 1) slices = 1;
  if (slices > k && k > 0) slices = k;
  float* arow = (float*)malloc(sizeof(float) * (size_t)(k > 0 ? k : 1));
  float* brow = (float*)malloc(sizeof(float) * (size_t)(k > 0 ? k : 1));
  /* decode each B column once per (i) would be O(m n k) decodes; cache all of
   * B decoded instead (n*k floats) when small enough, else decode per use. */
  const size_t bcache_elems = (size_t)n * (size_t)(k > 0 ? k : 1);
  float* bcache = bcache_elems <= ((size_t)1 << 28) ? (float*)malloc(bcache_elems * 4) : NULL;
  if (bcache) {
    for (int j = 0; j < n; ++j)
      for (int p = 0; p < k; ++p)
        bcache[(size_t)j * k + p] = mx_elem(fmt_b, B, SB, ldb, ldsb, j, p);
  }
  for (int i = 0; i < m; ++i) {
    for (int p = 0; p < k; ++p) arow[p] = mx_elem(fmt_a, A, SA, lda, ldsa, i, p);
    for (int j = 0; j < n; ++j) {
      const float* bp;
      if (bcache) {
        bp = bcache + (size_t)j * k;
      } else {
        for (int p = 0; p < k; ++p) brow[p] = mx_elem(fmt_b, B, SB, ldb, ldsb, j, p);
        bp = brow;
      }
      const float src = C[c_offset(c_row_major, i, j, ldc)];
      float out;
      if (k == 0) {
        out = beta != 0.0f ? fmaf(beta, src, alpha * 0.0f) : alpha * 0.0f;
      } else if (slices == 1) {
        out = 0.0f;
        for (int k0 = 0; k0 < k; k0 += kc) {
          const int k1 = k0 + kc < k ? k0 + kc : k;
          float acc = 0.0f;
          for (int p = k0; p < k1; ++p) acc = fmaf(arow[p], bp[p], acc);
          if (k0 == 0) {
            out = beta != 0.0f ? fmaf(beta, src, alpha * acc) : alpha * acc;
          } else {
            out = fmaf(alpha, acc, out);
          }
        }
      } else {
        float total = 0.0f;
        for (int s = 0; s < slices; ++s) {
          int kb, kl;
          split_range(k, slices, s, &kb, &kl);
          float slab = 0.0f;
          for (int k0 = kb; k0 < kb + kl; k0 += kc) {
            const int k1 = k0 + kc < kb + kl ? k0 + kc : kb + kl;
            float acc = 0.0f;
            for (int p = k0; p < k1; ++p) acc = fmaf(arow[p], bp[p], acc);
            slab = (k0 == kb) ? acc : slab + acc;
          }
          total = (s == 0) ? slab : total + slab;
        }
        out = beta != 0.0f ? fmaf(beta, src, alpha * total) : alpha * total;
      }
      if (activation == 1) out = out < 0.0f ? 0.0f : out;
      out = chain_f32(out, n_ops, ops, i, j);
      D[c_offset(c_row_major, i, j, ldd)] = out;
    }
  }
  free(arow);
  free(brow);
  free(bcache);
  return 0;
}

/*
 * Double-precision reference over exactly decoded operands, and the
 * reference test's own per-element error bound (test/test_gemm_mx.cc:179-227):
 *   want  = alpha * sum_k a_k*b_k (+ beta*C if beta != 0), in double
 *   bound = sum_k |a_k*b_k|
 * No activation / chain.  want and bound are m*n row-major (ld = n).
 */
ORACLE_API int oracle_gemm_mx_f64(int m, int n, int k, int fmt_a, const uint8_t* A,
                                  const uint8_t* SA, int lda, int ldsa, int fmt_b,
                                  const uint8_t* B, const uint8_t* SB, int ldb, int ldsb,
                                  const float* C, int ldc, int c_row_major, float alpha,
                                  float beta, double* want, double* bound) {
  if (m <= 0 || n <= 0) return 0;
  double* arow = (double*)malloc(sizeof(double) * (size_t)(k > 0 ? k : 1));
  for (int i = 0; i < m; ++i) {
    for (int p = 0; p < k; ++p) {
      /* the reference multiplies the f32 decode by the f32 scale in double */
      float e;
      if (fmt_a == ORACLE_FMT_E2M1) {
        const uint8_t byte = A[((int64_t)i * lda + p) >> 1];
        e = oracle_decode_e2m1((p & 1) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 0xF));
      } else {
        e = fmt_a == ORACLE_FMT_E4M3 ? oracle_decode_e4m3(A[(int64_t)i * lda + p])
                                     : oracle_decode_e5m2(A[(int64_t)i * lda + p]);
      }
      arow[p] = (double)e * (double)oracle_decode_e8m0(SA[(int64_t)i * ldsa + (p >> 5)]);
    }
    for (int j = 0; j < n; ++j) {
      double acc = 0.0, bnd = 0.0;
      for (int p = 0; p < k; ++p) {
        float e;
        if (fmt_b == ORACLE_FMT_E2M1) {
          const uint8_t byte = B[((int64_t)j * ldb + p) >> 1];
          e = oracle_decode_e2m1((p & 1) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 0xF));
        } else {
          e = fmt_b == ORACLE_FMT_E4M3 ? oracle_decode_e4m3(B[(int64_t)j * ldb + p])
                                       : oracle_decode_e5m2(B[(int64_t)j * ldb + p]);
        }
        const double b = (double)e * (double)oracle_decode_e8m0(SB[(int64_t)j * ldsb + (p >> 5)]);
        acc += arow[p] * b;
        bnd += fabs(arow[p] * b);
      }
      double v = (double)alpha * acc;
      if (beta != 0.0f) v += (double)beta * (double)C[c_offset(c_row_major, i, j, ldc)];
      want[(size_t)i * n + j] = v;
      if (bound) bound[(size_t)i * n + j] = bnd;
    }
  }
  free(arow);
  return 0;
}

/* Samples `count` output positions (rows[i], cols[i]) of the double reference;
 * used for the full-size configurations where an O(mnk) scalar pass is too
 * slow.  Same arithmetic as oracle_gemm_mx_f64. */
ORACLE_API int oracle_gemm_mx_f64_sampled(int k, int fmt_a, const uint8_t* A, const uint8_t* SA,
                                          int lda, int ldsa, int fmt_b, const uint8_t* B,
                                          const uint8_t* SB, int ldb, int ldsb, const float* C,
                                          int ldc, int c_row_major, float alpha, float beta,
                                          int count, const int32_t* rows, const int32_t* cols,
                                          double* want, double* bound) {
  for (int t = 0; t < count; ++t) {
    const int i = rows[t], j = cols[t];
    double acc = 0.0, bnd = 0.0;
    for (int p = 0; p < k; ++p) {
      float ea, eb;
      if (fmt_a == ORACLE_FMT_E2M1) {
        const uint8_t byte = A[((int64_t)i * lda + p) >> 1];
        ea = oracle_decode_e2m1((p & 1) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 0xF));
      } else {
        ea = fmt_a == ORACLE_FMT_E4M3 ? oracle_decode_e4m3(A[(int64_t)i * lda + p])
                                      : oracle_decode_e5m2(A[(int64_t)i * lda + p]);
      }
      if (fmt_b == ORACLE_FMT_E2M1) {
        const uint8_t byte = B[((int64_t)j * ldb + p) >> 1];
        eb = oracle_decode_e2m1((p & 1) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 0xF));
      } else {
        eb = fmt_b == ORACLE_FMT_E4M3 ? oracle_decode_e4m3(B[(int64_t)j * ldb + p])
                                      : oracle_decode_e5m2(B[(int64_t)j * ldb + p]);
      }
      const double a = (double)ea * (double)oracle_decode_e8m0(SA[(int64_t)i * ldsa + (p >> 5)]);
      const double b = (double)eb * (double)oracle_decode_e8m0(SB[(int64_t)j * ldsb + (p >> 5)]);
      acc += a * b;
      bnd += fabs(a * b);
    }
    double v = (double)alpha * acc;
    if (beta != 0.0f) v += (double)beta * (double)C[c_offset(c_row_major, i, j, ldc)];
    want[t] = v;
    if (bound) bound[t] = bnd;
  }
  return 0;
}

/* Sampled exact int8 reference for the full-size configurations: the same
 * arithmetic as oracle_gemm_u8s8s32 at `count` positions (before activation
 * and chain; callers apply those through oracle_chain_s32). */
ORACLE_API int oracle_gemm_u8s8s32_sampled(int k, const uint8_t* A, int lda, int a_row_major,
                                           const int8_t* B, int ldb, int b_row_major,
                                           const int32_t* C, int ldc, int c_row_major,
                                           int32_t alpha, int32_t beta, int activation,
                                           int n_ops, const oracle_op* ops, int count,
                                           const int32_t* rows, const int32_t* cols,
                                           int32_t* out) {
  for (int t = 0; t < count; ++t) {
    const int i = rows[t], j = cols[t];
    uint32_t acc = 0;
    for (int p = 0; p < k; ++p) {
      const int32_t a = A[c_offset(a_row_major, i, p, lda)];
      const int32_t b = B[c_offset(b_row_major, p, j, ldb)];
      acc += (uint32_t)(a * b);
    }
    uint32_t v = (uint32_t)alpha * acc;
    if (beta != 0) v += (uint32_t)beta * (uint32_t)C[c_offset(c_row_major, i, j, ldc)];
    int32_t x = (int32_t)v;
    if (activation == 1) x = x < 0 ? 0 : x;
    out[t] = chain_s32(x, n_ops, ops, i, j);
  }
  return 0;
}

/* The reference's split-k decision, gemm/kernel/run_blocked.h:100-117: only
 * with more than one thread; a forced count is used as given, the automatic
 * one needs k >= 8*KC and is bounded by 2*p and by a 4 MiB slab budget; both
 * are clamped to k/KC so no slice is shallower than one KC block. */
ORACLE_API int oracle_resolve_k_slices(int m, int n, int k, int kc, int requested, int p) {
  int k_slices = 1;
  if (p > 1) {
    const int depth_cap = k / kc > 1 ? k / kc : 1;
    if (requested > 0) {
      k_slices = requested;
    } else if (k >= 8 * kc) {
      const uint64_t slab_bytes = (uint64_t)m * (uint64_t)n * 4u;
      uint64_t ws_cap = ((uint64_t)4 << 20) / (slab_bytes > 0 ? slab_bytes : 1);
      if (ws_cap < 1) ws_cap = 1;
      if (ws_cap > 0x7FFFFFFF) ws_cap = 0x7FFFFFFF;
      k_slices = 2 * p < (int)ws_cap ? 2 * p : (int)ws_cap;
    }
    if (k_slices > depth_cap) k_slices = depth_cap;
    if (k_slices < 1) k_slices = 1;
  }
  return k_slices;
}

ORACLE_API int oracle_abi_version(void) { return 1; }
