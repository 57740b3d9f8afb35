// PrePostProcessor (PPP): the only component that touches user data on the CPU
// backends. It turns a job slice into "logical transmission units" (LTUs, here one
// packet payload each) on the way out and writes results back on the way in.
//
// Parity: reference client_lib/src/prepostprocessor.h:44-150 and prepostprocessor.cc
// (factory by name: cpu_exponent_quantizer | bypass), prepostprocessors/bypass_ppp.h.
#ifndef SWITCHML_PREPOSTPROCESSOR_H_
#define SWITCHML_PREPOSTPROCESSOR_H_

#include <memory>

#include "switchml/common.h"
#include "switchml/config.h"
#include "switchml/job.h"

namespace switchml {

class PrePostProcessor {
 public:
  // `ltu_size` in bytes, `batch_num_ltus` = slots of the calling worker thread.
  static std::shared_ptr<PrePostProcessor> CreateInstance(Config& config, WorkerTid worker_tid,
                                                          Numel ltu_size, Numel batch_num_ltus);
  virtual ~PrePostProcessor() = default;

  // Prepare for a slice; returns how many LTUs carry its payload.
  virtual uint64_t SetupJobSlice(JobSlice* job_slice) = 0;
  // True when one extra leading batch is needed (exponents travel one batch ahead).
  virtual bool NeedsExtraBatch() = 0;
  // Fill the payload (and the 1-byte exponent in `extra_info`) of LTU `ltu_id`.
  virtual void PreprocessSingle(uint64_t ltu_id, void* entries_ptr, void* extra_info = nullptr) = 0;
  // Consume the aggregated payload / exponent of LTU `ltu_id`.
  virtual void PostprocessSingle(uint64_t ltu_id, void* entries_ptr, void* extra_info = nullptr) = 0;
  virtual void CleanupJobSlice() = 0;

 protected:
  PrePostProcessor(Config& config, WorkerTid worker_tid, Numel ltu_size, Numel batch_num_ltus)
      : config_(config), worker_tid_(worker_tid), ltu_size_(ltu_size), batch_num_ltus_(batch_num_ltus) {}
  Config& config_;
  WorkerTid worker_tid_;
  Numel ltu_size_;
  Numel batch_num_ltus_;
};

// Does nothing to the data: isolates the transport from the numerics.
class BypassPPP : public PrePostProcessor {
 public:
  BypassPPP(Config& config, WorkerTid worker_tid, Numel ltu_size, Numel batch_num_ltus)
      : PrePostProcessor(config, worker_tid, ltu_size, batch_num_ltus) {}
  uint64_t SetupJobSlice(JobSlice* job_slice) override {
    uint64_t bytes = job_slice->slice.numel * DataTypeSize(job_slice->slice.data_type);
    return (bytes + ltu_size_ - 1) / ltu_size_;
  }
  bool NeedsExtraBatch() override { return false; }
  void PreprocessSingle(uint64_t, void*, void* = nullptr) override {}
  void PostprocessSingle(uint64_t, void*, void* = nullptr) override {}
  void CleanupJobSlice() override {}
};

}  // namespace switchml
#endif  // SWITCHML_PREPOSTPROCESSOR_H_
