// See cpu_exponent_quantizer_ppp.h. The arithmetic itself lives in switchml/quant_math.h
// so that the GPU kernels and this file cannot drift apart.
#include "ppp/cpu_exponent_quantizer_ppp.h"

#include <arpa/inet.h>

#include <algorithm>
#include <cmath>

#include "simd/simd_kernels.h"
#include "switchml/log.h"
#include "switchml/quant_math.h"

namespace switchml {

namespace {
inline float BlockMaxAbs(const float* x, Numel n) {
  float m = 0.0f;
  for (Numel i = 0; i < n; i++) {
    float v = fabsf(x[i]);
    if (v > m) m = v;  // NaN never wins the comparison, as in the reference loop
  }
  return m;
}
}  // namespace

CpuExponentQuantizerPPP::CpuExponentQuantizerPPP(Config& config, WorkerTid worker_tid,
                                                 Numel ltu_size, Numel batch_num_ltus)
    : PrePostProcessor(config, worker_tid, ltu_size, batch_num_ltus),
      batch_max_num_ltus_(batch_num_ltus),
      batch_(batch_num_ltus) {}

uint64_t CpuExponentQuantizerPPP::SetupJobSlice(JobSlice* job_slice) {
  job_slice_ = job_slice;
  ltu_numel_ = ltu_size_ / 4;
  total_ltus_ = (job_slice->slice.numel + ltu_numel_ - 1) / ltu_numel_;
  batch_ = std::min<Numel>(total_ltus_, batch_max_num_ltus_);
  scale_.clear();
  if (job_slice->slice.data_type == FLOAT32) scale_.assign(total_ltus_, 0.0f);
  return total_ltus_;
}

bool CpuExponentQuantizerPPP::NeedsExtraBatch() {
  return job_slice_->slice.data_type == FLOAT32;
}

Numel CpuExponentQuantizerPPP::LtuNumel(uint64_t k) const {
  Numel off = k * ltu_numel_;
  return std::min<Numel>(ltu_numel_, job_slice_->slice.numel - off);
}

void CpuExponentQuantizerPPP::PreprocessSingle(uint64_t ltu_id, void* entries_ptr,
                                               void* extra_info) {
  int32_t* wire = static_cast<int32_t*>(entries_ptr);
  const Tensor& t = job_slice_->slice;
  if (t.data_type == FLOAT32) {
    const float* in = static_cast<const float*>(t.in_ptr);
    if (ltu_id >= batch_) {
      // Payload: the LTU one batch behind, whose global exponent is known by now.
      uint64_t k = ltu_id - batch_;
      const float* x = in + k * ltu_numel_;
      Numel n = LtuNumel(k);
      simd::QuantizeToWire(x, n, scale_[k], wire);
    }
    if (ltu_id < total_ltus_) {
      // Exponent: of the LTU with this id, sent one batch early.
      float m = simd::BlockMaxAbs(in + ltu_id * ltu_numel_, LtuNumel(ltu_id));
      *static_cast<int8_t*>(extra_info) = static_cast<int8_t>(quant::LocalExponent(m));
    }
  } else if (t.data_type == INT32) {
    const int32_t* x = static_cast<const int32_t*>(t.in_ptr) + ltu_id * ltu_numel_;
    simd::Swap32(x, LtuNumel(ltu_id), wire);
  } else {
    SML_LOG(FATAL) << "worker thread " << worker_tid_ << ": unsupported data type "
                   << DataTypeName(t.data_type);
  }
}

void CpuExponentQuantizerPPP::PostprocessSingle(uint64_t ltu_id, void* entries_ptr,
                                                void* extra_info) {
  const int32_t* wire = static_cast<const int32_t*>(entries_ptr);
  const Tensor& t = job_slice_->slice;
  if (t.data_type == FLOAT32) {
    if (ltu_id >= batch_) {
      uint64_t k = ltu_id - batch_;
      float* y = static_cast<float*>(t.out_ptr) + k * ltu_numel_;
      Numel n = LtuNumel(k);
      simd::DequantizeFromWire(wire, n, scale_[k], y);
    }
    if (ltu_id < total_ltus_) {
      int e = *static_cast<const int8_t*>(extra_info);
      scale_[ltu_id] = quant::ScaleFactor(e, config_.general_.num_workers);
    }
  } else if (t.data_type == INT32) {
    int32_t* y = static_cast<int32_t*>(t.out_ptr) + ltu_id * ltu_numel_;
    simd::Swap32(wire, LtuNumel(ltu_id), y);
  } else {
    SML_LOG(FATAL) << "worker thread " << worker_tid_ << ": unsupported data type "
                   << DataTypeName(t.data_type);
  }
}

void CpuExponentQuantizerPPP::CleanupJobSlice() {
  scale_.clear();
  job_slice_ = nullptr;
}

void OracleQuantAllReduce(const float* const* inputs, int num_workers, Numel numel,
                          Numel block_numel, float* out) {
  for (Numel off = 0; off < numel; off += block_numel) {
    Numel n = std::min<Numel>(block_numel, numel - off);
    int e = quant::kZeroExponent;
    for (int w = 0; w < num_workers; w++) {
      e = std::max(e, quant::LocalExponent(BlockMaxAbs(inputs[w] + off, n)));
    }
    float sf = quant::ScaleFactor(e, num_workers);
    for (Numel i = 0; i < n; i++) {
      uint32_t acc = 0;  // unsigned: wrapping add without UB
      for (int w = 0; w < num_workers; w++) {
        acc += static_cast<uint32_t>(quant::Quantize(inputs[w][off + i], sf));
      }
      out[off + i] = quant::Dequantize(static_cast<int32_t>(acc), sf);
    }
  }
}

void OracleIntAllReduce(const int32_t* const* inputs, int num_workers, Numel numel,
                        int32_t* out) {
  for (Numel i = 0; i < numel; i++) {
    uint32_t acc = 0;
    for (int w = 0; w < num_workers; w++) acc += static_cast<uint32_t>(inputs[w][i]);
    out[i] = static_cast<int32_t>(acc);
  }
}

}  // namespace switchml
