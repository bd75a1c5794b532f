// Shared device math of the block-fp8 kernels.
//
// Bit-exact contract (per_block_cast_to_fp8 run by PyTorch on the CPU):
//   amax  = max |x| over the 128x128 block, NaN-propagating
//   scale = max(amax, 1e-4) / 448                    (fp32, true division)
//   q     = e4m3( fp32(x / scale) )                  (true division, round to nearest even)
//
// The division per element is the expensive part.  It is avoided without
// giving up exactness: with r = 1 / scale, the two products x * r * (1 - 2^-20)
// and x * r * (1 + 2^-20) bracket the correctly rounded quotient; conversion to
// e4m3 is monotonic, so when both ends convert to the same byte that byte is
// the exact answer.  Only when they differ (the quotient sits within 2^-19 of
// a rounding boundary, about one element in 30 000) is the division done.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <cstdint>

namespace awex {

struct QuantScale {
  float s;     // the scale written out
  float r_lo;  // (1 / s) * (1 - 2^-20)
  float r_hi;  // (1 / s) * (1 + 2^-20)
};

__device__ __forceinline__ QuantScale make_quant_scale(float amax, bool ue8m0) {
  float s = (amax < 1e-4f ? 1e-4f : amax) / 448.0f;  // NaN stays NaN
  if (ue8m0) {
    // Round up to a power of two: the value of fp32 log2 -> ceil -> exp2, which is
    // exact for every scale a 16-bit amax can produce.  Done on the bits (a
    // non-zero mantissa bumps the exponent; an exponent that overflows is
    // infinity, as exp2(128) is), so no rounding of a logarithm is involved.
    const float c = s < 1e-10f ? 1e-10f : s;  // NaN stays NaN
    uint32_t b = __float_as_uint(c);
    if (c == c && (b & 0x007FFFFFu)) b = (b & 0x7F800000u) + 0x00800000u;
    s = __uint_as_float(b);
  }
  const float r = __frcp_rn(s);
  QuantScale q;
  q.s = s;
  q.r_lo = r * 0.99999904632568359375f;  // 1 - 2^-20
  q.r_hi = r * 1.00000095367431640625f;  // 1 + 2^-20
  return q;
}

// Two values -> two e4m3 bytes (low byte = a).
__device__ __forceinline__ uint32_t quant_pair(float a, float b, const QuantScale& q) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a * q.r_lo, b * q.r_lo), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(a * q.r_hi, b * q.r_hi), __NV_SATFINITE, __NV_E4M3);
  if (lo == hi) return lo;
  return __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(a, q.s), __fdiv_rn(b, q.s)), __NV_SATFINITE, __NV_E4M3);
}

// NaN-propagating maximum of |x| kept as ordered integer bits.  For IEEE
// formats the magnitude bits order like unsigned integers and every NaN sorts
// above infinity, so an integer max is the NaN-propagating amax.
__device__ __forceinline__ uint32_t amax_bits_bf16x2(uint32_t m, uint32_t packed) { return __vmaxu2(m, packed & 0x7FFF7FFFu); }

__device__ __forceinline__ float amax_from_bf16x2(uint32_t m) {
  const uint32_t top = max(m & 0xFFFFu, m >> 16);
  return __uint_as_float(top << 16);
}
__device__ __forceinline__ float amax_from_f16x2(uint32_t m) {
  const uint32_t top = max(m & 0xFFFFu, m >> 16);
  return __half2float(__ushort_as_half(static_cast<unsigned short>(top)));
}
__device__ __forceinline__ uint32_t amax_bits_f32(uint32_t m, float x) { return max(m, __float_as_uint(x) & 0x7FFFFFFFu); }

// 8 bf16 / fp16 values (one 16-byte chunk) -> 8 e4m3 bytes.
template <bool kBf16>
__device__ __forceinline__ uint2 quant_chunk16(const uint4& raw, const QuantScale& q) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t out[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float a, b;
    if (kBf16) {
      a = __uint_as_float(w[i] << 16);
      b = __uint_as_float(w[i] & 0xFFFF0000u);
    } else {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      a = f.x;
      b = f.y;
    }
    out[i] = quant_pair(a, b, q);
  }
  return make_uint2(out[0] | (out[1] << 16), out[2] | (out[3] << 16));
}

}  // namespace awex
