// Shared device math of the block-fp8 kernels.
//
// Bit-exact contract (per_block_cast_to_fp8 of the reference, awex/converter/weights_converter.py:42-61,
// run by PyTorch on the CPU):
//   amax  = max |x| over the 128x128 block, NaN-propagating
//   scale = max(amax, 1e-4) / 448                    (fp32, true division)
//   q     = e4m3( fp32(x / scale) )                  (true division, round to nearest even)
//
// The division per element is the expensive part.  It is avoided without
// giving up exactness, in one of two ways.
//
//  * 16-bit sources (bf16, fp16): with r = RN(1 / scale), one correction step
//        q0 = x * r;  e = fma(-q0, scale, x);  q = fma(e, r, q0)
//    yields the quotient to within what e4m3 can tell apart (the residual e is
//    exact, and adding e * r to a quotient that is off by at most an ulp lands on
//    RN(x / scale) except in rare cases far from any e4m3 rounding boundary).  The
//    scale is positive, so each byte takes its sign from x: that only matters for
//    x = -0, which the correction step alone would turn into +0.
//    A block's scale comes from its own maximum, so |x / scale| <= 448 and
//    nothing overflows; results too small to be normal numbers round to zero in
//    e4m3 either way.  That the resulting byte equals the true division's for
//    EVERY value a 16-bit tensor can hold against EVERY scale its blocks can have
//    is checked exhaustively on the device (fp8_quotient_check_kernel in fp8_block.cu, run
//    by the GPU tests), not taken on trust.  Scales that are not finite (a block
//    holding an infinity or a NaN) take the division.
//  * fp32 sources: the two products x * r * (1 - 2^-20) and x * r * (1 + 2^-20)
//    bracket the correctly rounded quotient; conversion to e4m3 is monotonic,
//    so when both ends convert to the same byte that byte is the exact answer.
//    Only when they differ (the quotient sits within 2^-19 of a rounding
//    boundary, about one element in 30 000) is the division done.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <cstdint>

namespace awex {

struct QuantScale {
  float s;     // the scale written out
  float r;     // RN(1 / s)
  float r_lo;  // r * (1 - 2^-20)
  float r_hi;  // r * (1 + 2^-20)
  bool finite; // s is a finite number: the division-free forms apply
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
  q.r = r;
  q.r_lo = r * 0.99999904632568359375f;  // 1 - 2^-20
  q.r_hi = r * 1.00000095367431640625f;  // 1 + 2^-20
  q.finite = (__float_as_uint(s) & 0x7F800000u) != 0x7F800000u;
  return q;
}

// Two values -> two e4m3 bytes (low byte = a): the bracketing form, for any fp32 input.
__device__ __forceinline__ uint32_t quant_pair(float a, float b, const QuantScale& q) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a * q.r_lo, b * q.r_lo), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(a * q.r_hi, b * q.r_hi), __NV_SATFINITE, __NV_E4M3);
  if (lo == hi) return lo;
  return __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(a, q.s), __fdiv_rn(b, q.s)), __NV_SATFINITE, __NV_E4M3);
}

// x / s correctly rounded for a finite s, by one correction step on x * RN(1 / s).
__device__ __forceinline__ float quotient_corrected(float x, const QuantScale& q) {
  const float q0 = x * q.r;
  const float e = __fmaf_rn(-q0, q.s, x);
  return __fmaf_rn(e, q.r, q0);  // (turns x = -0 into +0: callers restore the sign)
}

// Two values that came from a 16-bit type and a finite scale -> two e4m3 bytes (low
// byte = a), signs not yet restored.
__device__ __forceinline__ uint32_t quant_pair16_finite(float a, float b, const QuantScale& q) {
  return __nv_cvt_float2_to_fp8x2(make_float2(quotient_corrected(a, q), quotient_corrected(b, q)), __NV_SATFINITE, __NV_E4M3);
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
    out[i] = q.finite ? quant_pair16_finite(a, b, q)
                      : __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(a, q.s), __fdiv_rn(b, q.s)), __NV_SATFINITE, __NV_E4M3);
  }
  uint2 r = make_uint2(out[0] | (out[1] << 16), out[2] | (out[3] << 16));
  if (q.finite) {
    // every byte takes the sign of its source value: the top byte of each 16-bit
    // element (bytes 1 and 3 of a word) holds it in bit 7
    r.x = (r.x & 0x7F7F7F7Fu) | (__byte_perm(raw.x, raw.y, 0x7531) & 0x80808080u);
    r.y = (r.y & 0x7F7F7F7Fu) | (__byte_perm(raw.z, raw.w, 0x7531) & 0x80808080u);
  }
  return r;
}

}  // namespace awex
