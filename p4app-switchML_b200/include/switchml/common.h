// Basic vocabulary types shared by every layer of the library.
//
// Parity: reference client_lib/src/common.h:40-116 (JobId, WorkerTid, Numel, DataType,
// DataTypeSize, Tensor, Tensor::OffsetPtrs). Additions for the GPU backend: BFLOAT16 as a
// third element type (gradient buckets of bf16 models) and a memory-space tag so a job
// can say whether its pointers are host or device addresses.
#ifndef SWITCHML_COMMON_H_
#define SWITCHML_COMMON_H_

#include <stdint.h>

#include <chrono>
#include <cstddef>

namespace switchml {

typedef uint64_t JobId;
typedef int16_t WorkerTid;
typedef uint64_t Numel;
typedef std::chrono::steady_clock clock;

enum DataType {
  FLOAT32 = 0,   // IEEE binary32
  INT32 = 1,     // two's complement, wrapping add
  BFLOAT16 = 2,  // GPU backends only; accumulated in float32
  UINT8 = 3,     // travels widened to int32 and is narrowed (wrapping) on return, like the
                 // reference's NCCL plugin does for PyTorch's uint8 flag reductions
                 // (nccl_plugin/switchml_plugin.cc:328-337,371-377)
};

static inline uint16_t DataTypeSize(DataType t) {
  switch (t) {
    case FLOAT32:
    case INT32:
      return 4;
    case BFLOAT16:
      return 2;
    case UINT8:
      return 1;
  }
  return 0;
}

static inline const char* DataTypeName(DataType t) {
  switch (t) {
    case FLOAT32: return "float32";
    case INT32: return "int32";
    case BFLOAT16: return "bfloat16";
    case UINT8: return "uint8";
  }
  return "?";
}

// A flat, contiguous 1-D view. `in_ptr` is only read; results go to `out_ptr`, which
// may alias `in_ptr` (in-place reduction).
struct Tensor {
  void* in_ptr = nullptr;
  void* out_ptr = nullptr;
  Numel numel = 0;
  DataType data_type = FLOAT32;

  // Advance both pointers by `n` elements (used when a job is cut into slices).
  inline void OffsetPtrs(Numel n) {
    size_t bytes = static_cast<size_t>(n) * DataTypeSize(data_type);
    in_ptr = static_cast<char*>(in_ptr) + bytes;
    out_ptr = static_cast<char*>(out_ptr) + bytes;
  }
};

}  // namespace switchml
#endif  // SWITCHML_COMMON_H_
