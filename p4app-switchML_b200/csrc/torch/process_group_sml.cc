// torch_switchml: the c10d backend "sml" as a native PyTorch extension.
//
// Counterpart of the reference's pytorch_plugin (ProcessGroupSML.{hpp,cpp}): the
// constructor starts the SwitchML context, allreduce() takes exactly one tensor with
// ReduceOp::SUM (float32, int32, and here also bfloat16 on the GPU), every other
// collective is left to the base class, which reports it as unsupported. Unlike the
// reference, a CUDA tensor is reduced where it is (no copy to pinned host memory), the
// work object returns immediately, and it has a future, so DDP communication hooks can
// be built on it.
//
//   import torch, torch.distributed as dist
//   import switchml_b200.parallel.native_process_group   # loads this module, registers "sml_native"
//   dist.init_process_group("sml_native", ...)
//
// The configuration comes from the usual switchml.cfg search (or $SWITCHML_CONFIG); rank
// and world size of the process group override the file.
#include <torch/extension.h>
#include <pybind11/chrono.h>

#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Types.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>

#ifdef SWITCHML_TORCH_CUDA
#include <c10/cuda/CUDAStream.h>
#endif

#include <chrono>
#include <cstdlib>
#include <string>

#include "switchml/context.h"
#include "switchml/log.h"

namespace {

switchml::DataType ToSwitchML(const at::Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return switchml::FLOAT32;
    case at::kInt: return switchml::INT32;
    case at::kByte: return switchml::UINT8;  // PyTorch reduces uint8 flags across workers
    case at::kBFloat16:
      TORCH_CHECK(t.is_cuda(), "SwitchML reduces bfloat16 tensors only on the GPU");
      return switchml::BFLOAT16;
    default:
      TORCH_CHECK(false, "SwitchML supports float32, int32, uint8 and (CUDA) bfloat16 tensors, got ", t.scalar_type());
  }
}

void* CurrentStream(const at::Tensor& t) {
#ifdef SWITCHML_TORCH_CUDA
  if (t.is_cuda()) return c10::cuda::getCurrentCUDAStream(t.device().index()).stream();
#endif
  (void)t;
  return nullptr;
}

class WorkSML : public c10d::Work {
 public:
  WorkSML(std::shared_ptr<switchml::Job> job, std::vector<at::Tensor> tensors, int rank)
      : c10d::Work(rank, c10d::OpType::ALLREDUCE), job_(std::move(job)), tensors_(std::move(tensors)) {}

  bool isCompleted() override {
    switchml::JobStatus s = job_->GetJobStatus();
    return s == switchml::FINISHED || s == switchml::FAILED;
  }
  bool isSuccess() const override { return job_->GetJobStatus() == switchml::FINISHED; }

  // CUDA tensors: order the caller's current stream after the reduction (no host block).
  // CPU tensors: block until the job is done.
  bool wait(std::chrono::milliseconds timeout = kNoTimeout) override {
    (void)timeout;
    const at::Tensor& t = tensors_[0];
    if (t.is_cuda()) {
      TORCH_CHECK(job_->StreamWait(CurrentStream(t)), "SwitchML allreduce failed: ", job_->failure_reason_);
    } else {
      job_->WaitToComplete();
      TORCH_CHECK(job_->GetJobStatus() == switchml::FINISHED, "SwitchML allreduce failed: ",
                  job_->failure_reason_);
    }
    return true;
  }
  void synchronize() override { wait(); }
  std::vector<at::Tensor> result() override { return tensors_; }

  c10::intrusive_ptr<c10::ivalue::Future> getFuture() override {
    if (!future_) {
      const at::Tensor& t = tensors_[0];
      std::vector<c10::Device> devices;
      if (t.is_cuda()) devices.push_back(t.device());
      future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()), devices);
      wait();  // CUDA: the current stream now follows the job; the future records it
      future_->markCompleted(c10::IValue(tensors_));
    }
    return future_;
  }

 private:
  std::shared_ptr<switchml::Job> job_;
  std::vector<at::Tensor> tensors_;
  c10::intrusive_ptr<c10::ivalue::Future> future_;
};

class BackendSML : public c10d::Backend {
 public:
  BackendSML(int rank, int size) : c10d::Backend(rank, size) {
    switchml::Context& ctx = switchml::Context::GetInstance();
    if (ctx.GetContextState() != switchml::Context::RUNNING) {
      switchml::Config cfg;
      TORCH_CHECK(cfg.LoadFromFile(), "SwitchML: no switchml.cfg found (set SWITCHML_CONFIG)");
      cfg.ApplyEnvOverrides();
      cfg.general_.rank = static_cast<uint16_t>(rank);
      cfg.general_.num_workers = static_cast<uint16_t>(size);
      TORCH_CHECK(ctx.Start(&cfg), "SwitchML: the context did not start");
      started_here_ = true;
    }
  }
  ~BackendSML() override {
    try {
      switchml::Context& ctx = switchml::Context::GetInstance();
      if (started_here_ && ctx.GetContextState() == switchml::Context::RUNNING) ctx.Stop();
    } catch (...) {
    }
  }

  const std::string getBackendName() const override { return "sml_native"; }

  c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor>& tensors,
                                           const c10d::AllreduceOptions& opts = c10d::AllreduceOptions()) override {
    TORCH_CHECK(tensors.size() == 1, "SwitchML reduces exactly one tensor per call (one GPU per worker)");
    TORCH_CHECK(opts.reduceOp == c10d::ReduceOp::SUM, "SwitchML implements ReduceOp.SUM only");
    at::Tensor& t = tensors[0];
    TORCH_CHECK(t.is_contiguous(), "SwitchML needs a contiguous tensor");
    switchml::Context& ctx = switchml::Context::GetInstance();
    std::shared_ptr<switchml::Job> job = ctx.AllReduceAsync(
        t.data_ptr(), t.data_ptr(), static_cast<uint64_t>(t.numel()), ToSwitchML(t), switchml::SUM, CurrentStream(t));
    return c10::make_intrusive<WorkSML>(std::move(job), tensors, getRank());
  }

  static c10::intrusive_ptr<c10d::Backend> Create(const c10::intrusive_ptr<c10d::Store>& /*store*/, int rank,
                                                  int size, const std::chrono::duration<float>& /*timeout*/) {
    return c10::make_intrusive<BackendSML>(rank, size);
  }

 private:
  bool started_here_ = false;
};

}  // namespace

PYBIND11_MODULE(torch_switchml, m) {
  m.doc() = "SwitchML c10d backend (native)";
  m.def("create_backend", &BackendSML::Create, "Factory for torch.distributed.Backend.register_backend");
}
