// Scheduler: hands job slices to worker threads.
//
// Parity: reference client_lib/src/scheduler.h:47-133 (abstract interface + factory by
// name) and schedulers/fifo_scheduler.{h,cc} (one FIFO of jobs; every worker thread
// takes one slice of the same job; static slicing numel/threads with the remainder
// spread one element each over the first threads; a job finishes when every thread
// reported its slice; Stop() fails everything still queued).
#ifndef SWITCHML_SCHEDULER_H_
#define SWITCHML_SCHEDULER_H_

#include <condition_variable>
#include <deque>
#include <map>
#include <memory>
#include <mutex>

#include "switchml/common.h"
#include "switchml/config.h"
#include "switchml/job.h"
#include "switchml/utils.h"

namespace switchml {

class Scheduler {
 public:
  // `consumers` = number of threads that will call GetJobSlice (0: num_worker_threads).
  static std::unique_ptr<Scheduler> CreateInstance(Config& config, int consumers = 0);
  virtual ~Scheduler() = default;
  Scheduler(const Scheduler&) = delete;
  void operator=(const Scheduler&) = delete;

  // Add a job; false if the scheduler was stopped (the job is marked FAILED).
  virtual bool EnqueueJob(std::shared_ptr<Job> job) = 0;
  // Blocking. Gives worker thread `tid` its slice of the current job. False = stopped.
  virtual bool GetJobSlice(WorkerTid tid, JobSlice& job_slice) = 0;
  // Called by a worker when its slice is done. True when this was the job's last slice,
  // in which case the caller (Context) finalises the job.
  virtual bool NotifyJobSliceCompletion(WorkerTid tid, const JobSlice& job_slice) = 0;
  // Wake every blocked worker and fail all queued jobs.
  virtual void Stop();

 protected:
  Scheduler(Config& config, int consumers);
  int consumers_;
  std::mutex access_mutex_;
  std::condition_variable job_submitted_event_;
  bool stopped_ = false;
  Config& config_;
};

// Slice `index` of `parts` over a tensor: numel/parts each, the first numel%parts slices
// one element longer. Exposed for tests and for the cuda backend's channel split.
void StaticSlice(Numel numel, int parts, int index, Numel* offset, Numel* length);

class FifoScheduler : public Scheduler {
 public:
  FifoScheduler(Config& config, int consumers);
  bool EnqueueJob(std::shared_ptr<Job> job) override;
  bool GetJobSlice(WorkerTid tid, JobSlice& job_slice) override;
  bool NotifyJobSliceCompletion(WorkerTid tid, const JobSlice& job_slice) override;
  void Stop() override;

 private:
  std::deque<std::shared_ptr<Job>> queue_;
  // job id -> slices not yet handed out / slices completed
  std::map<JobId, int> undispatched_;
  std::map<JobId, int> finished_;
  // All worker threads step to the next job together so that thread t of every worker
  // process talks to the same slots of the aggregator.
  Barrier barrier_;
};

}  // namespace switchml
#endif  // SWITCHML_SCHEDULER_H_
