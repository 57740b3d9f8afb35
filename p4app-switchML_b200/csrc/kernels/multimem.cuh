// Thin wrappers over the NVLink SHARP instructions. An address inside a multicast
// mapping names the same offset in every rank's bound memory: ld_reduce returns the
// reduction of all copies computed in the NVSwitch, st writes all copies at once.
#ifndef SWITCHML_MULTIMEM_CUH_
#define SWITCHML_MULTIMEM_CUH_

#include <stdint.h>

namespace switchml {
namespace kernels {

__device__ __forceinline__ float4 MultimemLdReduceAddF32x4(const void* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc) : "memory");
  return v;
}

// 8 bf16 values per call, summed in float32 inside the switch, returned as bf16 pairs.
__device__ __forceinline__ uint4 MultimemLdReduceAddBf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}

// Integer reductions have no vector form: one 32-bit lane per instruction.
__device__ __forceinline__ int MultimemLdReduceAddS32(const void* mc) {
  int v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.s32 %0, [%1];" : "=r"(v) : "l"(mc) : "memory");
  return v;
}

__device__ __forceinline__ int MultimemLdReduceMaxS32(const void* mc) {
  int v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.max.s32 %0, [%1];" : "=r"(v) : "l"(mc) : "memory");
  return v;
}

// 16 bytes to every copy. Stores are bitwise, so one spelling serves all element types.
__device__ __forceinline__ void MultimemStore16(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               ::"l"(mc), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)),
                 "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w)) : "memory");
}

__device__ __forceinline__ void MultimemStore4(void* mc, unsigned v) {
  asm volatile("multimem.st.relaxed.sys.global.b32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}

}  // namespace kernels
}  // namespace switchml
#endif  // SWITCHML_MULTIMEM_CUH_
