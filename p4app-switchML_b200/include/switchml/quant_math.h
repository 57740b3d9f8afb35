// The block fixed-point arithmetic of SwitchML, written once for host and device.
//
// For a block of float32 values shared by `n` workers:
//   local exponent   e  = biased_exponent(max|x|) - 126      (so that 2^e > max|x|)
//   global exponent  E  = max over workers of e              (done by the aggregator)
//   scale            sf = float( K / (n * 2^E) ),  K = 2^31-1
//   quantise         q  = round_to_nearest_even(x * sf)      (int32)
//   aggregate        Q  = sum over workers of q              (wrapping int32 add)
//   dequantise       y  = float(Q) / sf
// Reference: client_lib/src/prepostprocessors/cpu_exponent_quantizer_ppp.cc:88-156
// (quantise, exponent) and :200-260 (dequantise, scale from the global exponent).
//
// Deliberate differences, identical on CPU and GPU so that both produce the same bits:
//  * rounding is nearest-even everywhere (the reference mixes nearest-even in its vector
//    loop with half-away-from-zero in its scalar tail);
//  * the conversion saturates to the int32 range and maps NaN to 0 (the behaviour of
//    cvt.rni.s32.f32); the reference's conversion is undefined there;
//  * E is clamped to [-90, 127]: below -90 the scale would overflow float32 (an all-zero
//    block has e = -126 and gives 0 * inf = NaN in the reference), above 127 the
//    exponent byte would wrap;
//  * when n is not a power of two, K = 2^31-1-256 so that n rounded-up addends cannot
//    exceed int32 (for powers of two the scale is exact and K = 2^31-1 is already safe).
#ifndef SWITCHML_QUANT_MATH_H_
#define SWITCHML_QUANT_MATH_H_

#include <math.h>
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define SML_HD __host__ __device__ __forceinline__
#else
#define SML_HD inline
#endif

namespace switchml {
namespace quant {

static const int kMinExponent = -90;
static const int kMaxExponent = 127;
// Exponent reported for an empty or all-zero block.
static const int kZeroExponent = -126;

SML_HD uint32_t FloatBits(float x) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(x);
#else
  uint32_t u;
  memcpy(&u, &x, 4);
  return u;
#endif
}

// Exponent byte for a block whose largest magnitude is `maxabs` (>= 0, may be inf).
SML_HD int LocalExponent(float maxabs) {
  int e = static_cast<int>((FloatBits(maxabs) & 0x7f800000u) >> 23) - 126;
  return e > kMaxExponent ? kMaxExponent : e;
}

SML_HD int ClampExponent(int e) {
  return e < kMinExponent ? kMinExponent : (e > kMaxExponent ? kMaxExponent : e);
}

SML_HD float ScaleFactor(int global_exponent, int num_workers) {
  int e = ClampExponent(global_exponent);
  bool pow2 = (num_workers & (num_workers - 1)) == 0;
  double k = pow2 ? 2147483647.0 : 2147483647.0 - 256.0;
  // ldexp is exact in double for this range; one rounding when narrowing to float.
  return static_cast<float>(ldexp(k / static_cast<double>(num_workers), -e));
}

// The same scale factor without double precision in the hot path: `base` = QuantBase(n) is
// computed once per context, the power of two is applied with exact float multiplications
// (two steps, so that every intermediate stays a normal number). Bit-identical to
// ScaleFactor(): scaling by a power of two commutes with the rounding to float.
SML_HD float QuantBase(int num_workers) {
  bool pow2 = (num_workers & (num_workers - 1)) == 0;
  double k = pow2 ? 2147483647.0 : 2147483647.0 - 256.0;
  return static_cast<float>(k / static_cast<double>(num_workers));
}

SML_HD float ScaleFactorFromBase(int global_exponent, float base) {
  int e = ClampExponent(global_exponent);
  int h = e / 2;
#if defined(__CUDA_ARCH__)
  float s1 = __int_as_float((127 - h) << 23);        // 2^-h
  float s2 = __int_as_float((127 - (e - h)) << 23);  // 2^-(e-h)
#else
  float s1 = ldexpf(1.0f, -h);
  float s2 = ldexpf(1.0f, -(e - h));
#endif
  return base * s1 * s2;
}

SML_HD int32_t Quantize(float x, float sf) {
#if defined(__CUDA_ARCH__)
  return __float2int_rn(x * sf);  // cvt.rni.s32.f32: nearest-even, saturating, NaN -> 0
#else
  float p = x * sf;
  if (p != p) return 0;
  if (p >= 2147483648.0f) return INT32_MAX;
  if (p <= -2147483648.0f) return INT32_MIN;
  return static_cast<int32_t>(nearbyintf(p));  // default rounding mode: nearest-even
#endif
}

SML_HD float Dequantize(int32_t q, float sf) {
#if defined(__CUDA_ARCH__)
  return __fdiv_rn(__int2float_rn(q), sf);
#else
  return static_cast<float>(q) / sf;
#endif
}

}  // namespace quant
}  // namespace switchml
#endif  // SWITCHML_QUANT_MATH_H_
