// Job lifecycle. Parity: reference client_lib/src/job.cc:29-57.
#include "switchml/job.h"

#include <chrono>

#include "switchml/log.h"

namespace switchml {

std::atomic<JobId> Job::next_id_{0};

const char* JobStatusName(JobStatus s) {
  switch (s) {
    case INIT: return "INIT";
    case QUEUED: return "QUEUED";
    case RUNNING: return "RUNNING";
    case FINISHED: return "FINISHED";
    case FAILED: return "FAILED";
  }
  return "?";
}

Job::Job(Tensor tensor, JobType job_type, ExtraJobInfo extra_job_info)
    : id_(next_id_.fetch_add(1)),
      tensor_(tensor),
      job_type_(job_type),
      extra_job_info_(extra_job_info),
      job_status_(INIT) {}

void Job::WaitToComplete() {
  std::unique_lock<std::mutex> lk(access_mutex_);
  job_event_.wait(lk, [this] { return job_status_ == FINISHED || job_status_ == FAILED; });
}

bool Job::WaitToCompleteFor(double milliseconds) {
  std::unique_lock<std::mutex> lk(access_mutex_);
  return job_event_.wait_for(lk, std::chrono::duration<double, std::milli>(milliseconds),
                             [this] { return job_status_ == FINISHED || job_status_ == FAILED; });
}

JobStatus Job::GetJobStatus() {
  std::lock_guard<std::mutex> lk(access_mutex_);
  return job_status_;
}

void Job::SetJobStatus(JobStatus job_status) {
  {
    std::lock_guard<std::mutex> lk(access_mutex_);
    // FINISHED and FAILED are both terminal; everything else only moves forward.
    bool terminal = job_status_ == FINISHED || job_status_ == FAILED;
    if (terminal || job_status < job_status_) {
      SML_LOG(FATAL) << "Job " << id_ << " cannot go from " << JobStatusName(job_status_) << " to "
                     << JobStatusName(job_status);
    }
    job_status_ = job_status;
  }
  job_event_.notify_all();
}

void Job::SetDeviceState(std::shared_ptr<DeviceJobState> st) {
  {
    std::lock_guard<std::mutex> lk(access_mutex_);
    device_state_ = std::move(st);
    launched_ = true;
  }
  job_event_.notify_all();
}

bool Job::StreamWait(void* stream) {
  std::shared_ptr<DeviceJobState> st;
  {
    std::unique_lock<std::mutex> lk(access_mutex_);
    job_event_.wait(lk, [this] {
      return launched_ || job_status_ == FINISHED || job_status_ == FAILED;
    });
    if (job_status_ == FAILED) return false;
    st = device_state_;
  }
  if (st) st->StreamWait(stream);
  return true;
}

}  // namespace switchml
