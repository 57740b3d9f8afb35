// DummyBackend: runs the whole software stack without any communication.
//
// Parity: reference backends/dummy/dummy_backend.{h,cc} and dummy_worker_thread.{h,cc}.
// Sent packets are parked; "receiving" hands back a random number of them in random
// order (so out-of-order completion of the slot pipeline is exercised), optionally
// multiplies every int32 payload by num_workers to imitate an N-way sum of identical
// data (dummy_backend.cc:72-84), and sleeps to model `bandwidth` Mbps shared by the
// worker threads (dummy_backend.cc:124-133). Workers never see each other's data here.
#ifndef SWITCHML_DUMMY_BACKEND_H_
#define SWITCHML_DUMMY_BACKEND_H_

#include <thread>
#include <vector>

#include "switchml/backend.h"

namespace switchml {

class DummyBackend : public Backend {
 public:
  DummyBackend(Context& context, Config& config);
  ~DummyBackend() override;
  void SetupWorker() override;
  void CleanupWorker() override;

 private:
  void WorkerLoop(WorkerTid tid);
  std::vector<std::thread> threads_;
};

}  // namespace switchml
#endif  // SWITCHML_DUMMY_BACKEND_H_
