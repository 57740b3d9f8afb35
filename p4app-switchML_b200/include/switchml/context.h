// switchml::Context — the public entry point of the library.
//
// Parity: reference client_lib/src/context.h:53-233 and context.cc:36-197 — a process
// singleton with the lifecycle CREATED → STARTING → RUNNING → STOPPING → STOPPED;
// Start() loads/validates/prints the config, initialises stats, creates the scheduler
// and the backend and starts the workers; AllReduceAsync() returns a Job handle at once;
// AllReduce() waits for it; WaitForAllJobs(); Stop() fails whatever is still queued,
// joins the workers and logs the stats; the destructor stops a running context.
// Calling the job API while the context is not RUNNING is a fatal error.
//
// Extensions (no counterpart in the reference): a context can be started again after
// Stop(); pointers may be device addresses when backend = cuda, optionally with the
// CUDA stream that produces the input; symmetric (peer-mapped, multicast-bound) device
// buffers can be allocated for zero-copy reduction.
#ifndef SWITCHML_CONTEXT_H_
#define SWITCHML_CONTEXT_H_

#include <atomic>
#include <condition_variable>
#include <memory>
#include <mutex>

#include "switchml/backend.h"
#include "switchml/common.h"
#include "switchml/config.h"
#include "switchml/job.h"
#include "switchml/scheduler.h"
#include "switchml/stats.h"

namespace switchml {

class Context {
 public:
  enum ContextState { CREATED, STARTING, RUNNING, STOPPING, STOPPED };

  Context(const Context&) = delete;
  void operator=(const Context&) = delete;

  static Context& GetInstance();

  // `config` == nullptr: Config::LoadFromFile() with the default search order.
  bool Start(Config* config = nullptr);
  void Stop();

  std::shared_ptr<Job> AllReduceAsync(void* in_ptr, void* out_ptr, uint64_t numel,
                                      DataType data_type, AllReduceOperation op);
  // Same, for device pointers whose contents are produced by work already enqueued on
  // `stream` (a cudaStream_t; nullptr = legacy default stream).
  std::shared_ptr<Job> AllReduceAsync(void* in_ptr, void* out_ptr, uint64_t numel,
                                      DataType data_type, AllReduceOperation op, void* stream);
  std::shared_ptr<Job> AllReduce(void* in_ptr, void* out_ptr, uint64_t numel, DataType data_type,
                                 AllReduceOperation op);
  // Every worker's `ptr` ends up with the values of rank `root` (a job type the reference
  // declares but does not implement). Done with the one collective the fabric has: the
  // other workers contribute zeros to a sum. Exact for INT32 and with mode = float_sum; with
  // the quantised mode all workers, the root included, get the same values rounded to the
  // block's fixed-point grid. The buffer of a non-root worker is overwritten at once.
  // FLOAT32, INT32 and (cuda) BFLOAT16; the dummy backend has no peers and fails the job
  // unless there is one worker.
  std::shared_ptr<Job> BroadcastAsync(void* ptr, uint64_t numel, DataType data_type, int root,
                                      void* stream = nullptr);
  void WaitForAllJobs();

  ContextState GetContextState();
  const Config& GetConfig();
  Stats& GetStats();
  Backend* GetBackend() { return backend_.get(); }

  // ---- used by backend worker threads (friends in the reference, context.h:183-203) ----
  bool GetJobSlice(WorkerTid worker_thread_id, JobSlice& job_slice);
  void NotifyJobSliceCompletion(WorkerTid worker_thread_id, const JobSlice& job_slice);
  // Finalise a job that bypassed the scheduler (inline-launched GPU jobs).
  void NotifyJobCompletion(const std::shared_ptr<Job>& job, bool ok, const std::string& why = "");

 private:
  Context();
  ~Context();
  void FinishJob(const std::shared_ptr<Job>& job, bool ok, const std::string& why);

  std::atomic<ContextState> context_state_;  // read by worker threads while Start/Stop write it
  Config config_;
  Stats stats_;
  std::unique_ptr<Backend> backend_;
  std::unique_ptr<Scheduler> scheduler_;
  std::mutex context_mutex_;           // serialises Start/Stop
  uint64_t number_of_current_jobs_;
  std::mutex jobs_mutex_;
  std::condition_variable all_jobs_finished_event_;
};

}  // namespace switchml
#endif  // SWITCHML_CONTEXT_H_
