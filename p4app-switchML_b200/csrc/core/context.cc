// Context lifecycle and job submission.
// Parity: reference client_lib/src/context.cc:36-197.
#include "switchml/context.h"

#include <cstring>
#include <string>
#include <vector>

#include "switchml/log.h"
#include "switchml/version.h"

namespace switchml {

Context& Context::GetInstance() {
  static Context instance;
  return instance;
}

Context::Context() : context_state_(CREATED), number_of_current_jobs_(0) {
  SML_VLOG(1) << "switchml-b200 " << SWITCHML_VERSION << " (" << SWITCHML_BUILD_INFO << ")";
}

Context::~Context() {
  try {
    if (context_state_ == RUNNING) Stop();
  } catch (...) {
  }
}

bool Context::Start(Config* config) {
  std::lock_guard<std::mutex> lk(context_mutex_);
  SML_CHECK(context_state_ == CREATED || context_state_ == STOPPED)
      << "Start() called on a context that is already started";
  context_state_ = STARTING;
  try {
    if (config == nullptr) {
      config_ = Config();
      if (!config_.LoadFromFile()) {
        context_state_ = STOPPED;
        return false;
      }
      config_.ApplyEnvOverrides();
    } else {
      config_ = *config;
    }
    config_.Validate();
    config_.PrintConfig();

    stats_.InitStats(config_.general_.num_worker_threads);
    backend_ = Backend::CreateInstance(*this, config_);
    scheduler_ = Scheduler::CreateInstance(config_, backend_->NumSchedulerConsumers());
    {
      std::lock_guard<std::mutex> jl(jobs_mutex_);
      number_of_current_jobs_ = 0;
    }
    // Workers test the state in their loops, so it must read RUNNING before they exist.
    context_state_ = RUNNING;
    backend_->SetupWorker();
  } catch (const std::exception& e) {
    SML_LOG(ERROR) << "Context::Start failed: " << e.what();
    if (scheduler_) scheduler_->Stop();
    try {
      if (backend_) backend_->CleanupWorker();
    } catch (...) {
    }
    backend_.reset();
    scheduler_.reset();
    context_state_ = STOPPED;
    return false;
  }
  return true;
}

void Context::Stop() {
  std::lock_guard<std::mutex> lk(context_mutex_);
  SML_CHECK(context_state_ == RUNNING) << "Stop() called on a context that is not running";
  context_state_ = STOPPING;
  SML_VLOG(1) << "Stopping the context";
  scheduler_->Stop();         // wakes the workers and fails queued jobs
  backend_->CleanupWorker();  // joins them
  stats_.LogStats();
  backend_.reset();
  scheduler_.reset();
  context_state_ = STOPPED;
  {
    std::lock_guard<std::mutex> jl(jobs_mutex_);
    number_of_current_jobs_ = 0;
  }
  all_jobs_finished_event_.notify_all();
}

std::shared_ptr<Job> Context::AllReduceAsync(void* in_ptr, void* out_ptr, uint64_t numel,
                                             DataType data_type, AllReduceOperation op) {
  return AllReduceAsync(in_ptr, out_ptr, numel, data_type, op, nullptr);
}

std::shared_ptr<Job> Context::AllReduceAsync(void* in_ptr, void* out_ptr, uint64_t numel,
                                             DataType data_type, AllReduceOperation op,
                                             void* stream) {
  SML_CHECK(context_state_ == RUNNING)
      << "AllReduceAsync called while the context is not running";
  Tensor t;
  t.in_ptr = in_ptr;
  t.out_ptr = out_ptr;
  t.numel = numel;
  t.data_type = data_type;
  ExtraJobInfo extra;
  extra.allreduce_operation = op;
  // uint8 on host memory (CPU backends): the job works on an int32 copy, which is narrowed
  // into `out_ptr` when the job succeeds. The cuda backend widens on the device itself.
  std::shared_ptr<std::vector<int32_t>> widened;
  if (data_type == UINT8 && config_.general_.backend != "cuda") {
    const uint8_t* src = static_cast<const uint8_t*>(in_ptr);
    widened = std::make_shared<std::vector<int32_t>>(src, src + numel);
    t.in_ptr = t.out_ptr = widened->data();
    t.data_type = INT32;
  }
  std::shared_ptr<Job> job = std::make_shared<Job>(t, ALLREDUCE, extra);
  job->producer_stream_ = stream;
  if (widened) {
    uint8_t* dst = static_cast<uint8_t*>(out_ptr);
    job->on_success_ = [widened, dst] {
      for (size_t i = 0; i < widened->size(); i++) dst[i] = static_cast<uint8_t>((*widened)[i]);
    };
  }
  {
    std::lock_guard<std::mutex> jl(jobs_mutex_);
    number_of_current_jobs_++;
  }
  stats_.IncJobsSubmittedNum();
  stats_.AppendJobSubmittedNumel(numel);
  if (data_type == BFLOAT16 && config_.general_.backend != "cuda") {
    FinishJob(job, false, "bfloat16 tensors need backend = cuda");
    return job;
  }
  bool taken = backend_->OnSubmit(job);
  if (!taken && !scheduler_->EnqueueJob(job)) {
    FinishJob(job, false, "scheduler stopped");
  }
  return job;
}

std::shared_ptr<Job> Context::BroadcastAsync(void* ptr, uint64_t numel, DataType data_type, int root,
                                             void* stream) {
  SML_CHECK(context_state_ == RUNNING) << "BroadcastAsync called while the context is not running";
  const GeneralConfig& g = config_.general_;
  Tensor t;
  t.in_ptr = t.out_ptr = ptr;
  t.numel = numel;
  t.data_type = data_type;
  ExtraJobInfo extra;
  extra.broadcast_root = root;
  std::shared_ptr<Job> job = std::make_shared<Job>(t, BROADCAST, extra);
  job->producer_stream_ = stream;
  {
    std::lock_guard<std::mutex> jl(jobs_mutex_);
    number_of_current_jobs_++;
  }
  stats_.IncJobsSubmittedNum();
  stats_.AppendJobSubmittedNumel(numel);
  const bool cuda = g.backend == "cuda";
  if (root < 0 || root >= static_cast<int>(g.num_workers)) {
    FinishJob(job, false, "broadcast root " + std::to_string(root) + " is not a rank of this session");
  } else if (data_type == UINT8 || (data_type == BFLOAT16 && !cuda)) {
    FinishJob(job, false, std::string("broadcast does not take ") + DataTypeName(data_type) + " tensors here");
  } else if (g.num_workers == 1) {
    job->SetJobStatus(JobStatus::RUNNING);
    FinishJob(job, true, "");
  } else if (g.backend == "dummy") {
    // No peers to hear from: the root keeps what it has, anybody else cannot be served.
    if (static_cast<int>(g.rank) == root) {
      job->SetJobStatus(JobStatus::RUNNING);
      FinishJob(job, true, "");
    } else {
      FinishJob(job, false, "the dummy backend has no peers to receive a broadcast from");
    }
  } else {
    // Host memory: the zeros are written here; device memory: the cuda backend enqueues the
    // clearing in stream order in front of the kernel.
    if (!cuda && static_cast<int>(g.rank) != root) memset(ptr, 0, numel * DataTypeSize(data_type));
    bool taken = backend_->OnSubmit(job);
    if (!taken && !scheduler_->EnqueueJob(job)) FinishJob(job, false, "scheduler stopped");
  }
  return job;
}

std::shared_ptr<Job> Context::AllReduce(void* in_ptr, void* out_ptr, uint64_t numel,
                                        DataType data_type, AllReduceOperation op) {
  SML_CHECK(context_state_ == RUNNING) << "AllReduce called while the context is not running";
  std::shared_ptr<Job> job = AllReduceAsync(in_ptr, out_ptr, numel, data_type, op);
  job->WaitToComplete();
  return job;
}

void Context::WaitForAllJobs() {
  SML_CHECK(context_state_ == RUNNING || context_state_ == STOPPING || context_state_ == STOPPED)
      << "WaitForAllJobs called on a context that was never started";
  std::unique_lock<std::mutex> jl(jobs_mutex_);
  all_jobs_finished_event_.wait(jl, [this] { return number_of_current_jobs_ == 0; });
}

Context::ContextState Context::GetContextState() { return context_state_; }
const Config& Context::GetConfig() { return config_; }
Stats& Context::GetStats() { return stats_; }

bool Context::GetJobSlice(WorkerTid tid, JobSlice& job_slice) {
  if (context_state_ != RUNNING || !scheduler_) return false;
  return scheduler_->GetJobSlice(tid, job_slice);
}

void Context::FinishJob(const std::shared_ptr<Job>& job, bool ok, const std::string& why) {
  JobStatus s = job->GetJobStatus();
  if (s != FINISHED && s != FAILED) {
    if (ok) {
      if (job->on_success_) {
        job->on_success_();
        job->on_success_ = nullptr;
      }
      stats_.IncJobsFinishedNum();
      job->SetJobStatus(FINISHED);
    } else {
      stats_.IncJobsFailedNum();
      job->failure_reason_ = why;
      job->SetJobStatus(FAILED);
    }
  }
  bool none_left = false;
  {
    std::lock_guard<std::mutex> jl(jobs_mutex_);
    if (number_of_current_jobs_ > 0) number_of_current_jobs_--;
    none_left = number_of_current_jobs_ == 0;
  }
  if (none_left) all_jobs_finished_event_.notify_all();
}

void Context::NotifyJobSliceCompletion(WorkerTid tid, const JobSlice& job_slice) {
  if (!scheduler_) return;
  bool last = scheduler_->NotifyJobSliceCompletion(tid, job_slice);
  if (last) {
    bool ok = context_state_ == RUNNING && job_slice.job->failure_reason_.empty();
    FinishJob(job_slice.job, ok,
              ok ? "" : (job_slice.job->failure_reason_.empty() ? "context stopped during the job"
                                                                 : job_slice.job->failure_reason_));
  }
}

void Context::NotifyJobCompletion(const std::shared_ptr<Job>& job, bool ok,
                                  const std::string& why) {
  FinishJob(job, ok, why);
}

}  // namespace switchml
