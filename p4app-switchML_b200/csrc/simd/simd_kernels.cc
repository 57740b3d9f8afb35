// See simd_kernels.h.
#include "simd/simd_kernels.h"

#include <arpa/inet.h>
#include <immintrin.h>

#include <atomic>
#include <cmath>
#include <cstdlib>
#include <cstring>

#include "switchml/quant_math.h"

namespace switchml {
namespace simd {

namespace {

bool Detect() {
  const char* off = getenv("SWITCHML_NO_SIMD");
  if (off && *off && *off != '0') return false;
  return __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw");
}

std::atomic<int> g_enabled{-1};

#define SML_AVX512 __attribute__((target("avx512f,avx512bw")))

SML_AVX512 inline __m512i Bswap32(__m512i v) {
  const __m512i pattern = _mm512_set_epi8(
      12, 13, 14, 15, 8, 9, 10, 11, 4, 5, 6, 7, 0, 1, 2, 3, 12, 13, 14, 15, 8, 9, 10, 11, 4, 5, 6, 7, 0, 1, 2, 3,
      12, 13, 14, 15, 8, 9, 10, 11, 4, 5, 6, 7, 0, 1, 2, 3, 12, 13, 14, 15, 8, 9, 10, 11, 4, 5, 6, 7, 0, 1, 2, 3);
  return _mm512_shuffle_epi8(v, pattern);
}

SML_AVX512 inline __mmask16 TailMask(size_t left) {
  return left >= 16 ? static_cast<__mmask16>(0xffff) : static_cast<__mmask16>((1u << left) - 1u);
}

SML_AVX512 float BlockMaxAbs512(const float* x, size_t n) {
  __m512 m = _mm512_setzero_ps();
  for (size_t i = 0; i < n; i += 16) {
    __m512 v = _mm512_abs_ps(_mm512_maskz_loadu_ps(TailMask(n - i), x + i));
    m = _mm512_max_ps(v, m);  // the second operand is returned when the first is a NaN
  }
  return _mm512_reduce_max_ps(m);
}

SML_AVX512 void QuantizeToWire512(const float* x, size_t n, float sf, int32_t* wire) {
  const __m512 vsf = _mm512_set1_ps(sf);
  const __m512 top = _mm512_set1_ps(2147483648.0f);
  const __m512i int_max = _mm512_set1_epi32(INT32_MAX);
  for (size_t i = 0; i < n; i += 16) {
    const __mmask16 k = TailMask(n - i);
    __m512 p = _mm512_mul_ps(_mm512_maskz_loadu_ps(k, x + i), vsf);
    // Nearest-even under the default rounding mode; NaN and anything out of range come back
    // as 0x80000000, which is already right for the negative side.
    __m512i q = _mm512_cvtps_epi32(p);
    q = _mm512_mask_mov_epi32(q, _mm512_cmp_ps_mask(p, top, _CMP_GE_OQ), int_max);
    q = _mm512_mask_mov_epi32(q, _mm512_cmp_ps_mask(p, p, _CMP_UNORD_Q), _mm512_setzero_si512());
    _mm512_mask_storeu_epi32(wire + i, k, Bswap32(q));
  }
}

SML_AVX512 void DequantizeFromWire512(const int32_t* wire, size_t n, float sf, float* y) {
  const __m512 vsf = _mm512_set1_ps(sf);
  for (size_t i = 0; i < n; i += 16) {
    const __mmask16 k = TailMask(n - i);
    __m512i q = Bswap32(_mm512_maskz_loadu_epi32(k, wire + i));
    _mm512_mask_storeu_ps(y + i, k, _mm512_div_ps(_mm512_cvtepi32_ps(q), vsf));
  }
}

SML_AVX512 void Swap32_512(const int32_t* in, size_t n, int32_t* out) {
  for (size_t i = 0; i < n; i += 16) {
    const __mmask16 k = TailMask(n - i);
    _mm512_mask_storeu_epi32(out + i, k, Bswap32(_mm512_maskz_loadu_epi32(k, in + i)));
  }
}

SML_AVX512 void AddWire512(const uint8_t* wire, size_t n, int32_t* acc) {
  for (size_t i = 0; i < n; i += 16) {
    const __mmask16 k = TailMask(n - i);
    __m512i v = Bswap32(_mm512_maskz_loadu_epi32(k, wire + 4 * i));
    __m512i a = _mm512_maskz_loadu_epi32(k, acc + i);
    _mm512_mask_storeu_epi32(acc + i, k, _mm512_add_epi32(a, v));
  }
}

}  // namespace

bool Enabled() {
  int e = g_enabled.load(std::memory_order_relaxed);
  if (e < 0) {
    e = Detect() ? 1 : 0;
    g_enabled.store(e, std::memory_order_relaxed);
  }
  return e == 1;
}

void Enable(bool on) { g_enabled.store(on && Detect() ? 1 : 0, std::memory_order_relaxed); }

float BlockMaxAbs(const float* x, size_t n) {
  if (Enabled()) return BlockMaxAbs512(x, n);
  float m = 0.0f;
  for (size_t i = 0; i < n; i++) {
    float v = fabsf(x[i]);
    if (v > m) m = v;
  }
  return m;
}

void QuantizeToWire(const float* x, size_t n, float sf, int32_t* wire) {
  if (Enabled()) return QuantizeToWire512(x, n, sf, wire);
  for (size_t i = 0; i < n; i++) wire[i] = static_cast<int32_t>(htonl(static_cast<uint32_t>(quant::Quantize(x[i], sf))));
}

void DequantizeFromWire(const int32_t* wire, size_t n, float sf, float* y) {
  if (Enabled()) return DequantizeFromWire512(wire, n, sf, y);
  for (size_t i = 0; i < n; i++)
    y[i] = quant::Dequantize(static_cast<int32_t>(ntohl(static_cast<uint32_t>(wire[i]))), sf);
}

void Swap32(const int32_t* in, size_t n, int32_t* out) {
  if (Enabled()) return Swap32_512(in, n, out);
  for (size_t i = 0; i < n; i++) out[i] = static_cast<int32_t>(htonl(static_cast<uint32_t>(in[i])));
}

void AddWire(const uint8_t* wire, size_t n, int32_t* acc) {
  if (Enabled()) return AddWire512(wire, n, acc);
  for (size_t i = 0; i < n; i++) {
    uint32_t be;
    memcpy(&be, wire + 4 * i, 4);
    acc[i] = static_cast<int32_t>(static_cast<uint32_t>(acc[i]) + ntohl(be));
  }
}

}  // namespace simd
}  // namespace switchml
