// The element loops of the CPU data path, with AVX-512 versions chosen at run time.
//
// The reference vectorises its quantiser with Agner Fog's vector class library built for
// AVX-512 (prepostprocessors/cpu_exponent_quantizer_ppp.cc:30-37,88-109,130-146,215-247:
// Vec16f max(abs()), roundi(x * sf), permute-based byte swap, to_float / sf). Here the same
// loops are written with intrinsics in functions compiled for AVX-512 (target attribute, so
// the rest of the library keeps the default instruction set) and picked when the CPU has
// avx512f and avx512bw; otherwise, or with SWITCHML_NO_SIMD=1, the scalar loops run. Both
// give the same bits: every step is a single correctly rounded IEEE operation in either
// form (multiply, convert with round-to-nearest-even, divide), and the special cases of
// quant::Quantize (NaN -> 0, saturation) are applied with masks.
//
// "Wire" order is big-endian 32-bit words, as the packets carry them.
#ifndef SWITCHML_SIMD_KERNELS_H_
#define SWITCHML_SIMD_KERNELS_H_

#include <stddef.h>
#include <stdint.h>

namespace switchml {
namespace simd {

// True if the AVX-512 versions are in use.
bool Enabled();
// For tests: force the scalar (false) or the automatic (true) choice.
void Enable(bool on);

// max |x[i]|, 0 for n == 0; a NaN never becomes the maximum.
float BlockMaxAbs(const float* x, size_t n);
// wire[i] = big-endian(quant::Quantize(x[i], sf))
void QuantizeToWire(const float* x, size_t n, float sf, int32_t* wire);
// y[i] = quant::Dequantize(host-order(wire[i]), sf)
void DequantizeFromWire(const int32_t* wire, size_t n, float sf, float* y);
// out[i] = byte-swapped in[i] (host <-> wire; the buffers may be the same)
void Swap32(const int32_t* in, size_t n, int32_t* out);
// acc[i] += host-order(wire[i]) with wrapping 32-bit addition; `wire` may be unaligned
void AddWire(const uint8_t* wire, size_t n, int32_t* acc);

}  // namespace simd
}  // namespace switchml
#endif  // SWITCHML_SIMD_KERNELS_H_
