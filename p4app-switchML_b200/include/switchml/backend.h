// Backend: owns the transport and the worker threads that drive it.
// Parity: reference client_lib/src/backend.h:43-93 and backend.cc:40-64 (factory by
// name, SetupWorker / CleanupWorker). Names here: dummy | udp | cuda.
#ifndef SWITCHML_BACKEND_H_
#define SWITCHML_BACKEND_H_

#include <memory>

#include "switchml/config.h"
#include "switchml/job.h"

namespace switchml {

class Context;

class Backend {
 public:
  static std::unique_ptr<Backend> CreateInstance(Context& context, Config& config);
  virtual ~Backend() = default;
  Backend(const Backend&) = delete;
  void operator=(const Backend&) = delete;

  // Bring up the transport and start the worker threads.
  virtual void SetupWorker() = 0;
  // Stop and join the worker threads, release the transport.
  virtual void CleanupWorker() = 0;
  // How many threads of this backend pull slices from the scheduler.
  virtual int NumSchedulerConsumers() const;
  // Called in the submitting thread before the job is enqueued. The cuda backend
  // records the producer event here, or launches the job itself in inline mode, in
  // which case it returns true and the scheduler is bypassed.
  virtual bool OnSubmit(const std::shared_ptr<Job>& job) { (void)job; return false; }
  // Backend-specific counters appended to the stats report (JSON object text).
  virtual std::string ExtraStatsJson() { return "{}"; }

 protected:
  Backend(Context& context, Config& config) : context_(context), config_(config) {}
  Context& context_;
  Config& config_;
};

}  // namespace switchml
#endif  // SWITCHML_BACKEND_H_
