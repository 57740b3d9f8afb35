// Job: one submitted collective and its lifecycle.
//
// Parity: reference client_lib/src/job.h:37-148 and job.cc:29-57 — JobType
// {ALLREDUCE, BROADCAST (only declared in the reference, implemented here)},
// AllReduceOperation {SUM},
// monotone JobStatus INIT→QUEUED→RUNNING→FINISHED|FAILED (going backwards is a fatal
// error), ids from a process-wide counter, WaitToComplete() blocking on a condition
// variable, JobSlice = (job, sub-tensor).
//
// Added for the GPU backend: a job may carry the CUDA stream whose earlier work
// produces `in_ptr`, and exposes a "launched" milestone so that a consumer stream can
// be ordered after the job on the device instead of blocking the host.
#ifndef SWITCHML_JOB_H_
#define SWITCHML_JOB_H_

#include <atomic>
#include <condition_variable>
#include <memory>
#include <mutex>
#include <string>

#include <functional>

#include "switchml/common.h"

namespace switchml {

enum JobType {
  ALLREDUCE = 0,
  BROADCAST = 1,  // "Not yet supported" in the reference (job.h:39); here: the root's values reach every
                  // worker as a sum in which all other workers contribute zeros
};

enum AllReduceOperation {
  SUM = 0,
};

union ExtraJobInfo {
  AllReduceOperation allreduce_operation;
  int broadcast_root;  // BROADCAST jobs: rank whose values are handed out
};

enum JobStatus {
  INIT = 0,
  QUEUED = 1,
  RUNNING = 2,
  FINISHED = 3,
  FAILED = 4,
};

const char* JobStatusName(JobStatus s);

// Device-side ordering hooks attached by the cuda backend (opaque here so that the
// core stays free of CUDA headers).
struct DeviceJobState {
  virtual ~DeviceJobState() {}
  // Make `stream` (a cudaStream_t) wait for the job's device work.
  virtual void StreamWait(void* stream) = 0;
};

class Job {
 public:
  Job(Tensor tensor, JobType job_type, ExtraJobInfo extra_job_info);
  ~Job() = default;
  Job(const Job&) = delete;
  void operator=(const Job&) = delete;

  // Block until the job is FINISHED or FAILED.
  void WaitToComplete();
  // Same with a limit; returns false on timeout.
  bool WaitToCompleteFor(double milliseconds);
  JobStatus GetJobStatus();
  void SetJobStatus(JobStatus job_status);

  // GPU jobs: block (microseconds) until the kernels are enqueued, then order `stream`
  // after them. No-op for CPU backends or finished jobs. Returns false if the job failed
  // before it was launched.
  bool StreamWait(void* stream);
  void SetDeviceState(std::shared_ptr<DeviceJobState> st);

  const JobId id_;
  const Tensor tensor_;
  const JobType job_type_;
  const ExtraJobInfo extra_job_info_;
  // CUDA stream (cudaStream_t) that produces the input, or nullptr for the legacy
  // default stream / host memory.
  void* producer_stream_ = nullptr;
  // Event (cudaEvent_t) recorded on producer_stream_ at submission; owned by the backend.
  void* ready_event_ = nullptr;
  // Human-readable reason when FAILED.
  std::string failure_reason_;
  // Run once by the context right before a successful job turns FINISHED (uint8 jobs on
  // host memory narrow their int32 working copy into the caller's buffer here).
  std::function<void()> on_success_;

 private:
  static std::atomic<JobId> next_id_;
  JobStatus job_status_;
  std::mutex access_mutex_;
  std::condition_variable job_event_;
  std::shared_ptr<DeviceJobState> device_state_;
  bool launched_ = false;
};

struct JobSlice {
  std::shared_ptr<Job> job;
  Tensor slice;
};

}  // namespace switchml
#endif  // SWITCHML_JOB_H_
