// Backend and PrePostProcessor factories.
// Parity: reference client_lib/src/backend.cc:40-64, prepostprocessor.cc:32-41.
#include "switchml/backend.h"

#include "backends/cuda/cuda_backend.h"
#include "backends/dummy/dummy_backend.h"
#include "backends/softswitch/udp_backend.h"
#include "ppp/cpu_exponent_quantizer_ppp.h"
#include "switchml/log.h"
#include "switchml/prepostprocessor.h"

namespace switchml {

int Backend::NumSchedulerConsumers() const { return config_.general_.num_worker_threads; }

std::unique_ptr<Backend> Backend::CreateInstance(Context& context, Config& config) {
  const std::string& name = config.general_.backend;
  if (name == "dummy") return std::unique_ptr<Backend>(new DummyBackend(context, config));
  if (name == "udp") return std::unique_ptr<Backend>(new UdpBackend(context, config));
  if (name == "cuda") return std::unique_ptr<Backend>(CreateCudaBackend(context, config));
  SML_LOG(FATAL) << "'" << name << "' is not a valid backend.";
  return nullptr;
}

std::shared_ptr<PrePostProcessor> PrePostProcessor::CreateInstance(Config& config,
                                                                   WorkerTid worker_tid,
                                                                   Numel ltu_size,
                                                                   Numel batch_num_ltus) {
  const std::string& name = config.general_.prepostprocessor;
  if (name == "cpu_exponent_quantizer") {
    return std::make_shared<CpuExponentQuantizerPPP>(config, worker_tid, ltu_size, batch_num_ltus);
  }
  if (name == "bypass") {
    return std::make_shared<BypassPPP>(config, worker_tid, ltu_size, batch_num_ltus);
  }
  SML_LOG(FATAL) << "'" << name << "' is not a valid prepostprocessor.";
  return nullptr;
}

}  // namespace switchml
