// Scheduler factory and the FIFO scheduler.
// Parity: reference client_lib/src/scheduler.cc:30-37, schedulers/fifo_scheduler.cc:30-146.
#include "switchml/scheduler.h"

#include "switchml/log.h"

namespace switchml {

std::unique_ptr<Scheduler> Scheduler::CreateInstance(Config& config, int consumers) {
  if (consumers <= 0) consumers = config.general_.num_worker_threads;
  if (config.general_.scheduler == "fifo") {
    return std::unique_ptr<Scheduler>(new FifoScheduler(config, consumers));
  }
  SML_LOG(FATAL) << "'" << config.general_.scheduler << "' is not a valid scheduler.";
  return nullptr;
}

Scheduler::Scheduler(Config& config, int consumers) : consumers_(consumers), config_(config) {}

void Scheduler::Stop() {
  {
    std::lock_guard<std::mutex> lk(access_mutex_);
    stopped_ = true;
  }
  job_submitted_event_.notify_all();
}

void StaticSlice(Numel numel, int parts, int index, Numel* offset, Numel* length) {
  Numel base = numel / parts;
  Numel rem = numel % parts;
  Numel i = static_cast<Numel>(index);
  *length = base + (i < rem ? 1 : 0);
  *offset = base * i + (i < rem ? i : rem);
}

FifoScheduler::FifoScheduler(Config& config, int consumers)
    : Scheduler(config, consumers), barrier_(consumers) {}

bool FifoScheduler::EnqueueJob(std::shared_ptr<Job> job) {
  {
    std::lock_guard<std::mutex> lk(access_mutex_);
    if (stopped_) {
      job->failure_reason_ = "scheduler stopped";
      job->SetJobStatus(FAILED);
      return false;
    }
    job->SetJobStatus(QUEUED);
    undispatched_[job->id_] = consumers_;
    finished_[job->id_] = 0;
    queue_.push_back(job);
  }
  job_submitted_event_.notify_all();
  return true;
}

bool FifoScheduler::GetJobSlice(WorkerTid tid, JobSlice& job_slice) {
  // Everybody finishes job k before anybody starts job k+1.
  if (!barrier_.Wait()) return false;
  std::unique_lock<std::mutex> lk(access_mutex_);
  job_submitted_event_.wait(lk, [this] { return stopped_ || !queue_.empty(); });
  if (stopped_) return false;
  std::shared_ptr<Job> job = queue_.front();
  if (--undispatched_[job->id_] == 0) {
    queue_.pop_front();
    undispatched_.erase(job->id_);
  }
  job_slice.job = job;
  job_slice.slice = job->tensor_;
  Numel off, len;
  StaticSlice(job->tensor_.numel, consumers_, tid, &off, &len);
  job_slice.slice.OffsetPtrs(off);
  job_slice.slice.numel = len;
  if (job->GetJobStatus() == QUEUED) job->SetJobStatus(RUNNING);
  return true;
}

bool FifoScheduler::NotifyJobSliceCompletion(WorkerTid, const JobSlice& job_slice) {
  std::lock_guard<std::mutex> lk(access_mutex_);
  JobId id = job_slice.job->id_;
  auto it = finished_.find(id);
  if (it == finished_.end()) return false;  // already failed by Stop()
  if (++it->second == consumers_) {
    finished_.erase(it);
    return true;
  }
  return false;
}

void FifoScheduler::Stop() {
  Scheduler::Stop();
  barrier_.Destroy();
  std::deque<std::shared_ptr<Job>> drop;
  {
    std::lock_guard<std::mutex> lk(access_mutex_);
    drop.swap(queue_);
    undispatched_.clear();
    // Slices already handed out keep their finished_ entry so the job still completes
    // (or is failed by Context) when its workers return.
    for (auto& j : drop) finished_.erase(j->id_);
  }
  for (auto& j : drop) {
    JobStatus s = j->GetJobStatus();
    if (s != FINISHED && s != FAILED) {
      j->failure_reason_ = "context stopped before the job ran";
      j->SetJobStatus(FAILED);
    }
  }
}

}  // namespace switchml
