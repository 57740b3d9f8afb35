// CPU block-exponent quantiser: float32 <-> int32 fixed point around the aggregator.
//
// Parity: reference prepostprocessors/cpu_exponent_quantizer_ppp.{h,cc}. The exponent
// of LTU k is computed while LTU k-batch is quantised and travels with it; the global
// exponent of LTU k comes back with the result of LTU k-batch. Float slices therefore
// need one extra leading batch whose payload is ignored. INT32 slices skip all of it
// and are only converted to network byte order.
#ifndef SWITCHML_CPU_EXPONENT_QUANTIZER_PPP_H_
#define SWITCHML_CPU_EXPONENT_QUANTIZER_PPP_H_

#include <vector>

#include "switchml/prepostprocessor.h"

namespace switchml {

class CpuExponentQuantizerPPP : public PrePostProcessor {
 public:
  CpuExponentQuantizerPPP(Config& config, WorkerTid worker_tid, Numel ltu_size,
                          Numel batch_num_ltus);
  uint64_t SetupJobSlice(JobSlice* job_slice) override;
  bool NeedsExtraBatch() override;
  void PreprocessSingle(uint64_t ltu_id, void* entries_ptr, void* extra_info = nullptr) override;
  void PostprocessSingle(uint64_t ltu_id, void* entries_ptr, void* extra_info = nullptr) override;
  void CleanupJobSlice() override;

 private:
  // Elements of LTU `k` that lie inside the slice (the last one may be short).
  Numel LtuNumel(uint64_t k) const;

  JobSlice* job_slice_ = nullptr;
  Numel ltu_numel_ = 0;          // elements per full LTU
  Numel batch_max_num_ltus_;     // slots of this worker thread
  Numel batch_;                  // min(slots, LTUs of the slice)
  uint64_t total_ltus_ = 0;
  std::vector<float> scale_;     // per LTU, known once its global exponent arrived
};

// ---- stand-alone oracle (tests, benchmarks) -------------------------------------------
// Block-quantised SUM of `num_workers` float tensors exactly as the aggregation pipeline
// computes it (blocks of `block_numel` elements, the last one short).
void OracleQuantAllReduce(const float* const* inputs, int num_workers, Numel numel,
                          Numel block_numel, float* out);
// Wrapping int32 SUM.
void OracleIntAllReduce(const int32_t* const* inputs, int num_workers, Numel numel, int32_t* out);

}  // namespace switchml
#endif  // SWITCHML_CPU_EXPONENT_QUANTIZER_PPP_H_
