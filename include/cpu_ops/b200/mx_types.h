// OCP MX storage types of the cpu_ops call surface (include/cpu_ops/mx_formats.h):
// fp8e4m3_t (:107-153), fp8e5m2_t (:157-199), fp4e2m1_t (:204-249), the E8M0
// scale helpers (:253-278) and MxTensorRef (:280-295).  The codecs are host-side
// data-preparation helpers (the GPU consumes the raw bytes); they are written
// arithmetically here and checked code-by-code against the reference's tables
// by the test-suite.
#ifndef CPU_OPS_B200_MX_TYPES_H_
#define CPU_OPS_B200_MX_TYPES_H_

#include <algorithm>
#include <array>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>

namespace cpu_ops {

namespace b200_detail {

inline uint32_t f32_to_bits(float x) {
  uint32_t u;
  std::memcpy(&u, &x, sizeof u);
  return u;
}

// Decode of a small float: `ebits` exponent bits, `mbits` mantissa bits, `bias`.
inline float decode_minifloat(unsigned code, int ebits, int mbits, int bias) {
  const unsigned mant = code & ((1u << mbits) - 1);
  const unsigned expo = (code >> mbits) & ((1u << ebits) - 1);
  const bool neg = (code >> (ebits + mbits)) & 1u;
  const float mag = expo == 0 ? std::ldexp(static_cast<float>(mant), 1 - bias - mbits)
                              : std::ldexp(static_cast<float>(mant | (1u << mbits)),
                                           static_cast<int>(expo) - bias - mbits);
  return neg ? -mag : mag;
}

// Round-to-nearest-even encode of |x| onto a minifloat grid; returns the code
// without sign, possibly one past `max_code` (the caller saturates or overflows).
inline unsigned encode_minifloat_rne(float ax, int mbits, int bias) {
  if (ax == 0.0f) return 0;
  int e;
  std::frexp(ax, &e);            // ax = f * 2^e, f in [0.5, 1)
  int expo = e - 1 + bias;       // biased exponent of the leading one
  if (expo < 1) expo = 0;        // subnormal grid: unit 2^(1 - bias - mbits)
  const int unit = (expo == 0 ? 1 : expo) - bias - mbits;
  const float scaled = std::ldexp(ax, -unit);               // in units of the grid step
  float r = std::nearbyint(scaled);                          // default rounding mode: RNE
  unsigned q = static_cast<unsigned>(r);
  // q counts grid steps from the start of the binade (normal: includes the hidden one)
  if (expo == 0) return q;                                   // may carry into the first normal
  if (q >= (2u << mbits)) return (static_cast<unsigned>(expo + 1) << mbits);  // carried up a binade
  return (static_cast<unsigned>(expo) << mbits) | (q - (1u << mbits));
}

// Decode table of a storage type, filled from its to_float (the reference keeps constexpr
// tables, mx_formats.h:30-102; callers and its tests use them as T::kLut[code] and
// T::kLut.size()).
template <typename T, size_t N>
inline std::array<float, N> make_decode_table() {
  std::array<float, N> t{};
  for (size_t c = 0; c < N; ++c) t[c] = T::to_float(static_cast<uint8_t>(c));
  return t;
}

}  // namespace b200_detail

// Declared because the reference's umbrella header exports the name (callers write
// `using cpu_ops::bfloat16_t;`); no operator of this library takes it.
struct bfloat16_t {
  uint16_t bits = 0;
};

// 1-4-3, bias 7, no infinity; S.1111.111 is NaN.
struct fp8e4m3_t {
  uint8_t bits = 0;
  fp8e4m3_t() = default;
  fp8e4m3_t(float f) : bits(from_float(f)) {}
  struct Raw {};
  constexpr fp8e4m3_t(uint8_t raw_bits, Raw) : bits(raw_bits) {}
  operator float() const { return to_float(bits); }

  static float to_float(uint8_t b) {
    if ((b & 0x7F) == 0x7F) return std::numeric_limits<float>::quiet_NaN();
    return b200_detail::decode_minifloat(b, 4, 3, 7);
  }
  // RNE, saturating at +-448; NaN stays NaN, infinity saturates.
  static uint8_t from_float(float x) {
    const uint8_t sign = std::signbit(x) ? 0x80 : 0x00;
    if (x != x) return sign | 0x7F;
    const float ax = std::fabs(x);
    if (ax >= 480.0f) return sign | 0x7E;  // past the midpoint above 448 (or inf)
    unsigned code = b200_detail::encode_minifloat_rne(ax, 3, 7);
    if (code > 0x7E) code = 0x7E;
    return static_cast<uint8_t>(sign | code);
  }
  static const std::array<float, 256> kLut;  // kLut[code] == to_float(code)
};
inline const std::array<float, 256> fp8e4m3_t::kLut = b200_detail::make_decode_table<fp8e4m3_t, 256>();

// 1-5-2, bias 15, IEEE-like infinities and NaNs.
struct fp8e5m2_t {
  uint8_t bits = 0;
  fp8e5m2_t() = default;
  fp8e5m2_t(float f) : bits(from_float(f)) {}
  struct Raw {};
  constexpr fp8e5m2_t(uint8_t raw_bits, Raw) : bits(raw_bits) {}
  operator float() const { return to_float(bits); }

  static float to_float(uint8_t b) {
    if ((b & 0x7C) == 0x7C) {
      if (b & 0x03) return std::numeric_limits<float>::quiet_NaN();
      return (b & 0x80) ? -std::numeric_limits<float>::infinity()
                        : std::numeric_limits<float>::infinity();
    }
    return b200_detail::decode_minifloat(b, 5, 2, 15);
  }
  // RNE; overflow rounds to infinity.
  static uint8_t from_float(float x) {
    const uint8_t sign = std::signbit(x) ? 0x80 : 0x00;
    if (x != x) return sign | 0x7E;
    const float ax = std::fabs(x);
    if (std::isinf(ax)) return sign | 0x7C;
    unsigned code = b200_detail::encode_minifloat_rne(ax, 2, 15);
    if (code > 0x7C) code = 0x7C;
    return static_cast<uint8_t>(sign | code);
  }
  static const std::array<float, 256> kLut;
};
inline const std::array<float, 256> fp8e5m2_t::kLut = b200_detail::make_decode_table<fp8e5m2_t, 256>();

// 1-2-1, bias 1: +-{0, .5, 1, 1.5, 2, 3, 4, 6}.  Nibble-level helpers only; two
// elements share a byte, the even element index in the low nibble.
struct fp4e2m1_t {
  static float to_float(uint8_t nibble) {
    return b200_detail::decode_minifloat(nibble & 0xF, 2, 1, 1);
  }
  // RNE with ties to the even code; NaN maps to 0; saturates at 6.
  static uint8_t from_float(float x) {
    if (x != x) return 0;
    const uint8_t sign = std::signbit(x) ? 0x8 : 0x0;
    const float ax = std::fabs(x);
    if (ax > 5.0f) return sign | 0x7;
    unsigned code = b200_detail::encode_minifloat_rne(ax, 1, 1);
    if (code > 7) code = 7;
    return static_cast<uint8_t>(sign | code);
  }
  static const std::array<float, 16> kLut;
};
inline const std::array<float, 16> fp4e2m1_t::kLut = b200_detail::make_decode_table<fp4e2m1_t, 16>();

// E8M0 block scale: 2^(e - 127); e == 0 is 2^-127, 0xFF is NaN.
inline float e8m0_to_float(uint8_t e) {
  if (e == 0xFF) return std::numeric_limits<float>::quiet_NaN();
  return std::ldexp(1.0f, static_cast<int>(e) - 127);
}

// Nearest power of two (ties up: mantissa above sqrt(2) rounds up), clamped to
// [2^-127, 2^127]; NaN gives 0xFF, zero and f32 denormals give 0.
inline uint8_t e8m0_from_float(float x) {
  const uint32_t u = b200_detail::f32_to_bits(x);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0xFF;
  const int biased = static_cast<int>((u >> 23) & 0xFF);
  if (biased == 0) return 0;
  int r = biased - 127 + ((u & 0x7FFFFFu) > 0x3504F3u ? 1 : 0);
  if (r < -127) r = -127;
  if (r > 127) r = 127;
  return static_cast<uint8_t>(r + 127);
}

// One MX operand: packed elements plus one E8M0 scale per 32 elements along k.
//   element (i, k): data[(i * ld + k) / elems_per_byte]
//   scale (i, k/32): scales[i * ld_scales + k / 32]
template <typename T>
struct MxTensorRef {
  const uint8_t* data = nullptr;
  const uint8_t* scales = nullptr;
  int ld = 0;         // leading dimension in elements
  int ld_scales = 0;  // leading dimension in scale entries
};

namespace mma {
namespace mxvnni_detail {

// Host-side helper of the reference's lossy MX-VNNI policy
// (gemm/threadblock/mma_policy_mx_vnni.h:55-78), kept because callers and the reference's
// tests build their own expected values with it: re-quantises up to 32 unscaled values to
// int8 codes on the grid 2^qexp, qexp = floor(log2(max |v|)) - 6, round to nearest even,
// clamped to [-128, 127]; q[len..32) is zero; returns qexp (-127 for an all-zero block).
// The GEMMs of this library never re-quantise: MxVnniPolicy forwards to the exact path.
inline int quantize_block_i8(const float* v, int len, int8_t* q) {
  float peak = 0.0f;
  for (int t = 0; t < len; ++t) peak = std::max(peak, std::fabs(v[t]));
  std::fill(q, q + 32, static_cast<int8_t>(0));
  if (peak == 0.0f) return -127;
  const int qexp = static_cast<int>((b200_detail::f32_to_bits(peak) >> 23) & 0xFF) - 127 - 6;
  const uint32_t inv_bits = static_cast<uint32_t>(127 - qexp) << 23;  // 2^-qexp
  float inv;
  std::memcpy(&inv, &inv_bits, sizeof inv);
  for (int t = 0; t < len; ++t) {
    const float code = std::nearbyint(v[t] * inv);  // default rounding mode: nearest even
    q[t] = static_cast<int8_t>(code > 127.0f ? 127 : (code < -128.0f ? -128 : static_cast<int>(code)));
  }
  return qexp;
}

}  // namespace mxvnni_detail
}  // namespace mma

}  // namespace cpu_ops

#endif  // CPU_OPS_B200_MX_TYPES_H_
