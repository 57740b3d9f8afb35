// See cuda_backend.h.
#include "backends/cuda/cuda_backend.h"

#include <cuda_runtime.h>
#if __has_include(<nvtx3/nvToolsExt.h>)
#include <nvtx3/nvToolsExt.h>
#define SML_NVTX_PUSH(name) nvtxRangePushA(name)
#define SML_NVTX_POP() nvtxRangePop()
#else
#define SML_NVTX_PUSH(name) ((void)0)
#define SML_NVTX_POP() ((void)0)
#endif

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cctype>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <mutex>
#include <sstream>
#include <thread>
#include <vector>

#include "backends/cuda/fd_channel.h"
#include "backends/cuda/symmetric_memory.h"
#include "kernels/allreduce_kernels.h"
#include "rendezvous/control.h"
#include "switchml/context.h"
#include "switchml/log.h"
#include "switchml/quant_math.h"

namespace switchml {

namespace {

#define SML_CUDA_CHECK(call)                                                        \
  do {                                                                              \
    cudaError_t _e = (call);                                                        \
    SML_CHECK(_e == cudaSuccess) << #call << ": " << cudaGetErrorString(_e);        \
  } while (0)

// Recycles CUDA events; shared with the jobs so that an event outlives the backend if a
// caller still holds the job.
struct EventPool {
  std::mutex mu;
  std::vector<cudaEvent_t> free_list;
  cudaEvent_t Get() {
    {
      std::lock_guard<std::mutex> lk(mu);
      if (!free_list.empty()) {
        cudaEvent_t e = free_list.back();
        free_list.pop_back();
        return e;
      }
    }
    cudaEvent_t e = nullptr;
    cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
    return e;
  }
  void Put(cudaEvent_t e) {
    if (!e) return;
    std::lock_guard<std::mutex> lk(mu);
    free_list.push_back(e);
  }
  ~EventPool() {
    for (cudaEvent_t e : free_list) cudaEventDestroy(e);
  }
};

struct EventState : public DeviceJobState {
  cudaEvent_t done = nullptr;
  std::shared_ptr<EventPool> pool;
  ~EventState() override {
    if (pool) pool->Put(done);
  }
  void StreamWait(void* stream) override {
    cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), done, 0);
  }
};

struct InFlight {
  std::shared_ptr<Job> job;
  bool via_scheduler = false;
  JobSlice slice;
  cudaEvent_t done = nullptr;
  cudaEvent_t ready = nullptr;
  int status_slot = 0;
  unsigned long long tiles = 0;
  std::string launch_error;
};

static const int kStatusSlots = 4096;

class CudaBackend : public CudaBackendInterface {
 public:
  CudaBackend(Context& context, Config& config) : CudaBackendInterface(context, config) {}
  ~CudaBackend() override { CleanupWorker(); }

  int NumSchedulerConsumers() const override { return 1; }

  void SetupWorker() override;
  void CleanupWorker() override;
  bool OnSubmit(const std::shared_ptr<Job>& job) override;
  std::string ExtraStatsJson() override;

  void* SymmetricAlloc(size_t bytes) override;
  void SymmetricReset() override;
  bool UsesMultimem() const override { return ctx_.use_multimem != 0; }
  bool SymmetricHeapInfo(void** local, void** peers, void** multicast, size_t* bytes) override {
    if (!heap_.local) return false;
    *local = heap_.local;
    for (int p = 0; p < n_; p++) peers[p] = heap_.peers[p];
    *multicast = heap_.multicast;
    *bytes = heap_.bytes;
    return true;
  }
  int Device() const override { return device_; }
  int RunWaitProbe(double budget_ms) override;

 private:
  void LauncherLoop();
  void CompletionLoop();
  void BindServiceThread(const char* what);
  // Enqueue the kernels of `job` on `stream`; fills `f`. Caller holds launch_mu_.
  // `capturing`: the stream is being captured into a CUDA graph; nothing that belongs to
  // this one submission (events, status slot, buffer parity) may end up in the launch.
  void LaunchJob(const std::shared_ptr<Job>& job, cudaStream_t stream, InFlight* f, bool capturing = false);
  cudaEvent_t GetEvent() { return events_->Get(); }
  void PutEvent(cudaEvent_t e) { events_->Put(e); }

  int device_ = 0;
  int rank_ = 0, n_ = 1;
  bool inline_launch_ = false;
  bool set_up_ = false;
  std::unique_ptr<ControlServer> server_;
  ControlClient client_;
  FdChannel fds_;
  std::unique_ptr<SymmetricAllocator> allocator_;
  SymmetricRegion staging_;
  SymmetricRegion heap_;
  size_t heap_used_ = 0;
  kernels::RankCtx ctx_;
  int max_channels_ = 1;
  cudaStream_t comm_stream_ = nullptr;
  int* dev_status_ = nullptr;
  unsigned long long* dev_counters_ = nullptr;
  unsigned long long* dev_trace_ = nullptr;  // kTraceWords, only with [backend.cuda] trace
  unsigned long long* dev_epochs_ = nullptr;  // per-channel epochs, advanced by the kernels themselves
  int* host_status_ = nullptr;  // pinned ring of status words

  std::mutex launch_mu_;  // serialises launches: one job order on every rank
  // launch = inline: all jobs share the staging slots, the flag pad and the per-channel
  // epochs, so two jobs must never run on the GPU at the same time. A job submitted on a
  // stream other than the previous job's is ordered after that job through this event.
  cudaEvent_t order_event_ = nullptr;
  cudaStream_t order_stream_ = nullptr;
  bool order_valid_ = false;
  unsigned long long epoch_base_ = 0;
  int oneshot_parity_ = 0;
  unsigned long long launched_jobs_ = 0;
  uint64_t oneshot_limit_ = 0;  // messages up to this many bytes take the one-barrier kernel
  unsigned long long kernel_launches_ = 0;  // kernels of this library enqueued so far (under launch_mu_)

  std::shared_ptr<EventPool> events_ = std::make_shared<EventPool>();

  std::thread launcher_, completer_;
  std::mutex q_mu_;
  std::condition_variable q_cv_;
  std::deque<InFlight> inflight_;
  bool stop_completer_ = false;
  std::atomic<bool> failed_{false};
};

void CudaBackend::SetupWorker() {
  const GeneralConfig& g = config_.general_;
  const CudaBackendConfig& c = config_.backend_.cuda;
  rank_ = g.rank;
  n_ = g.num_workers;
  SML_CHECK(n_ <= kernels::kMaxRanks)
      << "the cuda backend serves one NVSwitch domain of at most " << kernels::kMaxRanks
      << " GPUs, got num_workers = " << n_;
  inline_launch_ = c.launch == "inline";

  int ndev = 0;
  cudaError_t e = cudaGetDeviceCount(&ndev);
  SML_CHECK(e == cudaSuccess && ndev > 0)
      << "backend = cuda needs a GPU: " << cudaGetErrorString(e);
  device_ = c.device;
  if (device_ < 0) {
    const char* lr = getenv("LOCAL_RANK");
    device_ = (lr && *lr) ? atoi(lr) : static_cast<int>(g.rank);
    device_ %= ndev;
  }
  SML_CHECK(device_ < ndev) << "backend.cuda.device " << device_ << " does not exist";
  SML_CUDA_CHECK(cudaSetDevice(device_));
  cudaDeviceProp prop;
  SML_CUDA_CHECK(cudaGetDeviceProperties(&prop, device_));
  SML_CHECK(prop.major >= 9) << "device " << device_ << " (" << prop.name << ", sm_" << prop.major
                             << prop.minor << ") is too old for this library (built for sm_100a)";

  uint64_t session = static_cast<uint64_t>(
      std::chrono::duration_cast<std::chrono::nanoseconds>(
          std::chrono::system_clock::now().time_since_epoch()).count());
  if (n_ > 1) {
    if (rank_ == 0) {
      server_.reset(new ControlServer());
      SML_CHECK(server_->Start(g.controller_ip_str, g.controller_port, 0))
          << "cannot start the in-process controller on " << g.controller_ip_str << ":"
          << g.controller_port;
    }
    SML_CHECK(client_.Connect(g.controller_ip_str, g.controller_port)) << "controller unreachable";
    SML_CHECK(client_.Broadcast(n_, rank_, 0, &session)) << "session broadcast failed";
    SML_CHECK(fds_.Listen(session, rank_, c.rendezvous_dir)) << "cannot open the fd channel";
    SML_CHECK(client_.Barrier(n_)) << "barrier failed";
  }
  allocator_.reset(new SymmetricAllocator(rank_, n_, device_, &client_, &fds_));

  // Co-residency bound: every CTA of a job must be able to run at the same time.
  max_channels_ = prop.multiProcessorCount;
  if (c.channels > 0 && static_cast<int>(c.channels) < max_channels_) max_channels_ = c.channels;
  if (max_channels_ > kernels::kMaxChannels) max_channels_ = kernels::kMaxChannels;

  memset(&ctx_, 0, sizeof(ctx_));
  ctx_.rank = rank_;
  ctx_.nranks = n_;
  ctx_.slot_bytes = c.slot_bytes;
  ctx_.slots_per_channel = c.slots_per_channel;
  ctx_.sc_fence = c.signal_fence == "sc" ? 1 : 0;
  ctx_.exp_ring = kernels::ExpRingDepth(static_cast<int>(c.slots_per_channel));
  ctx_.exp_lookahead = kernels::ExpLookahead(static_cast<int>(c.slots_per_channel), static_cast<int>(c.exponent_lookahead));
  ctx_.block_numel = static_cast<int>(g.packet_numel);
  ctx_.quant_base = quant::QuantBase(n_);
  // The one-barrier kernel sends every rank's whole message to every rank, n-1 times the
  // traffic of the streaming algorithms: the fewer the ranks, the longer it stays the faster
  // one. The configured limit is the one for eight workers.
  oneshot_limit_ = c.oneshot_max_bytes * 8 / static_cast<uint64_t>(n_ < 2 ? 2 : n_);
  ctx_.oneshot_bytes = (oneshot_limit_ + 255) / 256 * 256;
  ctx_.timeout_ns = static_cast<unsigned long long>(c.wait_timeout_ms * 1e6);
  size_t bytes = kernels::StagingBytes(ctx_.slot_bytes, ctx_.slots_per_channel, ctx_.block_numel,
                                       max_channels_, ctx_.oneshot_bytes, n_, &ctx_.data_offset,
                                       &ctx_.exp_offset, &ctx_.oneshot_offset);
  ctx_.stage_bytes = kernels::ReportedStageBytes(bytes);
  // Two GPUs exchange less data with plain peer loads/stores (N bytes each way) than
  // through the switch (1.5 N); from three GPUs on the in-switch reduction wins.
  bool want_mc = c.transport == "nvls" || (c.transport == "auto" && n_ > 2);
  std::string err;
  SML_CHECK(allocator_->Create(bytes, want_mc, &staging_, &err))
      << "cannot create the symmetric staging region (" << (bytes >> 20) << " MiB): " << err;
  SML_CHECK(!(c.transport == "nvls" && n_ > 1 && !staging_.multicast))
      << "backend.cuda.transport = nvls but NVLink multicast is not available";
  for (int p = 0; p < n_; p++) ctx_.stage_peer[p] = static_cast<char*>(staging_.peers[p]);
  ctx_.stage_mc = static_cast<char*>(staging_.multicast);
  ctx_.use_multimem = staging_.multicast != nullptr;

  if (c.symm_heap_mb > 0) {
    SML_CHECK(allocator_->Create(static_cast<size_t>(c.symm_heap_mb) << 20, ctx_.use_multimem != 0,
                                 &heap_, &err))
        << "cannot create the symmetric heap: " << err;
    if (ctx_.use_multimem && !heap_.multicast) {
      SML_LOG(WARNING) << "symmetric heap has no multicast mapping; zero-copy jobs use peer loads";
    }
  }
  heap_used_ = 0;

  int lo = 0, hi = 0;
  cudaDeviceGetStreamPriorityRange(&lo, &hi);
  SML_CUDA_CHECK(cudaStreamCreateWithPriority(&comm_stream_, cudaStreamNonBlocking, hi));
  SML_CUDA_CHECK(cudaEventCreateWithFlags(&order_event_, cudaEventDisableTiming));
  order_valid_ = false;
  SML_CUDA_CHECK(cudaMalloc(&dev_counters_, 16 * sizeof(unsigned long long)));
  SML_CUDA_CHECK(cudaMemset(dev_counters_, 0, 16 * sizeof(unsigned long long)));
  SML_CUDA_CHECK(cudaMalloc(&dev_epochs_, kernels::kMaxChannels * sizeof(unsigned long long)));
  SML_CUDA_CHECK(cudaMemset(dev_epochs_, 0, kernels::kMaxChannels * sizeof(unsigned long long)));
  // Status words live in pinned host memory that the device can write: a kernel stores
  // its error code there directly, so a job costs no extra copy or memset on the stream.
  SML_CUDA_CHECK(cudaHostAlloc(&host_status_, kStatusSlots * sizeof(int), cudaHostAllocMapped));
  memset(host_status_, 0, kStatusSlots * sizeof(int));
  SML_CUDA_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&dev_status_), host_status_, 0));
  ctx_.status = dev_status_;
  ctx_.counters = dev_counters_;
  if (c.trace) {
    SML_CUDA_CHECK(cudaMalloc(&dev_trace_, kernels::kTraceWords * sizeof(unsigned long long)));
    SML_CUDA_CHECK(cudaMemset(dev_trace_, 0, kernels::kTraceWords * sizeof(unsigned long long)));
  }
  ctx_.trace = dev_trace_;
  ctx_.epoch_words = dev_epochs_;
  epoch_base_ = 0;
  oneshot_parity_ = 0;
  launched_jobs_ = 0;
  kernel_launches_ = 0;
  failed_ = false;
  SML_CUDA_CHECK(cudaDeviceSynchronize());
  if (n_ > 1) SML_CHECK(client_.Barrier(n_)) << "barrier failed";

  SML_VLOG(0) << "cuda backend ready: rank " << rank_ << "/" << n_ << " on device " << device_
              << " (" << prop.name << "), transport "
              << (n_ == 1 ? "local" : (ctx_.use_multimem ? "nvls (multimem)" : "p2p (peer memory)"))
              << ", staging " << (bytes >> 20) << " MiB, up to " << max_channels_ << " channels, launch "
              << c.launch;
  stop_completer_ = false;
  set_up_ = true;
  completer_ = std::thread(&CudaBackend::CompletionLoop, this);
  if (!inline_launch_) launcher_ = std::thread(&CudaBackend::LauncherLoop, this);
}

void CudaBackend::CleanupWorker() {
  if (!set_up_) return;
  set_up_ = false;
  if (launcher_.joinable()) launcher_.join();
  {
    std::lock_guard<std::mutex> lk(q_mu_);
    stop_completer_ = true;
  }
  q_cv_.notify_all();
  if (completer_.joinable()) completer_.join();
  cudaSetDevice(device_);
  cudaDeviceSynchronize();
  bool peers_alive = !failed_.load();
  if (server_) server_->StopAccepting();
  if (n_ > 1 && peers_alive && !client_.Barrier(n_, 10000)) peers_alive = false;
  if (heap_.local) allocator_->Destroy(&heap_, peers_alive);
  if (staging_.local) allocator_->Destroy(&staging_, peers_alive);
  if (comm_stream_) cudaStreamDestroy(comm_stream_);
  comm_stream_ = nullptr;
  if (order_event_) cudaEventDestroy(order_event_);
  order_event_ = nullptr;
  order_valid_ = false;
  if (dev_counters_) cudaFree(dev_counters_);
  if (dev_trace_) cudaFree(dev_trace_);
  if (dev_epochs_) cudaFree(dev_epochs_);
  dev_epochs_ = nullptr;
  if (host_status_) cudaFreeHost(host_status_);
  dev_status_ = nullptr;
  dev_counters_ = nullptr;
  dev_trace_ = nullptr;
  host_status_ = nullptr;
  fds_.Close();
  client_.Close();
  if (server_) {
    server_->Stop();
    server_.reset();
  }
}

void* CudaBackend::SymmetricAlloc(size_t bytes) {
  if (!heap_.local) return nullptr;
  size_t need = (bytes + 255) / 256 * 256;
  std::lock_guard<std::mutex> lk(launch_mu_);
  if (heap_used_ + need > heap_.bytes) return nullptr;
  void* p = static_cast<char*>(heap_.local) + heap_used_;
  heap_used_ += need;
  return p;
}

void CudaBackend::SymmetricReset() {
  std::lock_guard<std::mutex> lk(launch_mu_);
  heap_used_ = 0;
}

// nullptr if kernels may dereference `p`, else the reason why not.
static const char* GpuCannotAccess(const void* p) {
  if (p == nullptr) return "null pointer";
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
    cudaGetLastError();
    return "the address is unknown to CUDA";
  }
  if (at.type == cudaMemoryTypeUnregistered) return "the address is ordinary (pageable) host memory";
  return nullptr;
}

void CudaBackend::LaunchJob(const std::shared_ptr<Job>& job, cudaStream_t stream, InFlight* f, bool capturing) {
  const CudaBackendConfig& c = config_.backend_.cuda;
  Tensor t = job->tensor_;
  const Tensor& user = job->tensor_;
  // The kernels dereference both pointers on the GPU: refuse anything the GPU cannot be
  // trusted to reach (ordinary malloc'ed host memory) instead of launching into a fault.
  // Device, managed and pinned (cudaHostAlloc / cudaHostRegister) memory pass.
  if (t.numel > 0) {
    const char* why = GpuCannotAccess(t.in_ptr);
    if (!why && t.out_ptr != t.in_ptr) why = GpuCannotAccess(t.out_ptr);
    if (why) {
      f->launch_error = std::string("backend = cuda needs device, managed or pinned memory: ") + why;
      return;
    }
  }
  // uint8: widen into int32 scratch of the stream's memory pool, reduce that in place,
  // narrow into the caller's output. With one worker the sum is the input itself.
  void* widened = nullptr;
  if (t.data_type == UINT8 && n_ > 1 && t.numel > 0) {
    if (capturing) {
      f->launch_error = "uint8 jobs cannot be captured into a CUDA graph";
      return;
    }
    cudaError_t we = cudaMallocAsync(&widened, t.numel * 4, stream);
    if (we == cudaSuccess) we = kernels::LaunchWidenU8(t.in_ptr, widened, t.numel, stream);
    if (we != cudaSuccess) {
      f->launch_error = std::string("uint8 staging failed: ") + cudaGetErrorString(we);
      cudaGetLastError();
      if (widened) cudaFreeAsync(widened, stream);
      return;
    }
    t.in_ptr = t.out_ptr = widened;
    t.data_type = INT32;
  }
  const bool integer = t.data_type == INT32 || t.data_type == UINT8;
  // A broadcast is a sum to which everybody but the root contributes zeros: clear this
  // rank's buffer in stream order, in front of the kernel; never average.
  const bool broadcast = job->job_type_ == BROADCAST;
  if (broadcast && rank_ != job->extra_job_info_.broadcast_root && t.numel > 0) {
    cudaError_t ce = cudaMemsetAsync(t.in_ptr, 0, t.numel * DataTypeSize(t.data_type), stream);
    if (ce != cudaSuccess) {
      f->launch_error = std::string("broadcast: clearing the buffer failed: ") + cudaGetErrorString(ce);
      cudaGetLastError();
      return;
    }
  }
  kernels::JobArgs a;
  memset(&a, 0, sizeof(a));
  a.in = t.in_ptr;
  a.out = t.out_ptr;
  a.numel = t.numel;
  a.elem_type = t.data_type == FLOAT32 ? kernels::ELEM_F32
              : t.data_type == BFLOAT16 ? kernels::ELEM_BF16 : kernels::ELEM_I32;
  a.mode = (!integer && c.mode == "int32_quant") ? kernels::MODE_QUANT : kernels::MODE_SUM;
  a.post_scale = c.average && !integer && !broadcast ? 1.0f / static_cast<float>(n_) : 1.0f;
  size_t esz = DataTypeSize(t.data_type);
  size_t bytes = t.numel * esz;
  a.bulk_copy = t.numel > 0 && kernels::DeviceMemory(t.in_ptr) && kernels::DeviceMemory(t.out_ptr);

  // Pick the algorithm (identically on every rank: it depends on sizes and on whether the
  // pointers sit in the symmetric heap, which is allocated in lock step).
  auto in_heap = [&](const void* p) {
    return heap_.local && p >= heap_.local &&
           static_cast<const char*>(p) + bytes <= static_cast<const char*>(heap_.local) + heap_.bytes;
  };
  auto heap_usable = [&](const void* p) {
    return in_heap(p) && (reinterpret_cast<uintptr_t>(p) & 15) == 0 && (!ctx_.use_multimem || heap_.multicast);
  };
  const bool out_in_heap = n_ > 1 && heap_usable(t.out_ptr);
  const bool heap_ok = out_in_heap && heap_usable(t.in_ptr);
  auto describe_heap = [&] {
    for (int p = 0; p < n_; p++) a.user_peer[p] = static_cast<char*>(heap_.peers[p]);
    a.user_mc = static_cast<char*>(heap_.multicast);
    a.user_bytes = heap_.bytes;
    a.in_offset = static_cast<const char*>(t.in_ptr) - static_cast<const char*>(heap_.local);
    a.out_offset = static_cast<const char*>(t.out_ptr) - static_cast<const char*>(heap_.local);
  };
  // Peer-memory transport moves large messages with posted stores only, unless told otherwise.
  const bool push = n_ > 1 && !ctx_.use_multimem && c.p2p_algo == "push" &&
                    kernels::PushTileCapacity(ctx_, a.elem_type, a.mode) > 0;
  // (Tensors of the symmetric heap are reduced where they lie when the switch can do it;
  // over plain peer memory small ones are quicker through the one-barrier kernel.)
  // Plain sums through the switch leave the one-barrier kernel at a quarter of the configured
  // size already (measured at four GPUs: 4 MiB take 40 us there against 36 us streamed).
  const uint64_t oneshot_limit = (ctx_.use_multimem && a.mode == kernels::MODE_SUM) ? c.oneshot_max_bytes / 4 : oneshot_limit_;
  if (bytes <= oneshot_limit && !(a.mode == kernels::MODE_SUM && heap_ok && ctx_.use_multimem)) {
    a.algo = kernels::ALGO_ONESHOT;
    a.oneshot_parity = oneshot_parity_;
    if (!capturing) oneshot_parity_ ^= 1;
  } else if (push) {
    a.algo = kernels::ALGO_PUSH;
    if (out_in_heap) {  // results go straight into every rank's output
      a.out_zero_copy = 1;
      describe_heap();
    }
  } else if (a.mode == kernels::MODE_SUM && heap_ok) {
    a.algo = kernels::ALGO_ZEROCOPY;
    describe_heap();
  } else {
    a.algo = kernels::ALGO_STAGED;
    if (a.mode == kernels::MODE_QUANT && out_in_heap) {
      a.out_zero_copy = 1;
      describe_heap();
    }
  }
  kernels::LaunchPlan plan = kernels::PlanLaunch(ctx_, a, c.channels, max_channels_);
  a.tile_elems = plan.tile_elems;
  a.epochs = plan.epochs;
  if (capturing && a.algo == kernels::ALGO_ONESHOT) {
    a.trailing_barrier = 1;  // a replayed launch cannot alternate buffers: meet again instead,
    a.oneshot_parity = 2;    // in a buffer set of its own, apart from the alternating pair
    a.epochs = 2;
  }
  epoch_base_ += a.epochs;
  f->tiles = plan.tiles;
  // Replays of a captured launch share one status word that nobody waits on; a timeout in
  // a replay still shows up in the device counters.
  f->status_slot = capturing ? kStatusSlots - 2 : static_cast<int>(launched_jobs_++ % (kStatusSlots - 2));
  f->done = capturing ? nullptr : GetEvent();

  cudaError_t e = cudaSuccess;
  host_status_[f->status_slot] = kernels::STATUS_OK;  // the ring is far longer than the queue
  kernels::RankCtx job_ctx = ctx_;
  job_ctx.status = dev_status_ + f->status_slot;
  // A single worker reducing in place has nothing to do (float_sum: the sum of one term;
  // quantised mode still runs, because quantise/dequantise rounds the values).
  bool nothing_to_do = n_ == 1 && t.in_ptr == t.out_ptr && a.mode == kernels::MODE_SUM && a.post_scale == 1.0f;
  // One NVTX range per job: shows up in timeline tools, costs nothing without one.
  char range[96];
  snprintf(range, sizeof(range), "switchml job %llu: %llu x %s", static_cast<unsigned long long>(job->id_),
           static_cast<unsigned long long>(t.numel), DataTypeName(user.data_type));
  SML_NVTX_PUSH(range);
  bool plain_copy = n_ == 1 && a.mode == kernels::MODE_SUM && a.post_scale == 1.0f && !nothing_to_do;
  // One worker in the exact mode: one pass that rounds every value to its block's grid.
  const bool local_quant = n_ == 1 && a.mode == kernels::MODE_QUANT && a.elem_type == kernels::ELEM_F32 && t.numel > 0 &&
                           ((reinterpret_cast<uintptr_t>(t.in_ptr) | reinterpret_cast<uintptr_t>(t.out_ptr)) & 15) == 0;
  if (local_quant)
    e = kernels::LaunchLocalQuant(t.in_ptr, t.out_ptr, t.numel, ctx_.block_numel, ctx_.quant_base, a.post_scale, stream);
  else if (t.numel > 0 && plain_copy) e = kernels::LaunchLocalCopy(t.in_ptr, t.out_ptr, bytes, stream);
  else if (t.numel > 0 && !nothing_to_do) e = kernels::LaunchAllReduce(job_ctx, a, plan, stream);
  if (t.numel > 0 && !nothing_to_do && e == cudaSuccess) kernel_launches_ += widened ? 3 : 1;
  SML_NVTX_POP();
  if (widened) {
    if (e == cudaSuccess) e = kernels::LaunchNarrowI32(widened, user.out_ptr, user.numel, stream);
    cudaFreeAsync(widened, stream);
  }
  if (e == cudaSuccess && f->done) e = cudaEventRecord(f->done, stream);
  if (e != cudaSuccess) {
    f->launch_error = std::string("kernel launch failed: ") + cudaGetErrorString(e);
    cudaGetLastError();
  }
  SML_VLOG(2) << "job " << job->id_ << ": " << t.numel << " x " << DataTypeName(user.data_type)
              << " algo " << a.algo << " mode " << a.mode << " channels " << plan.channels
              << " epochs " << plan.epochs;
  if (f->done) {
    auto st = std::make_shared<EventState>();
    st->done = f->done;
    st->pool = events_;
    job->SetDeviceState(st);
  } else {
    job->SetDeviceState(nullptr);  // captured: the work is ordered by the graph itself
  }
}

bool CudaBackend::OnSubmit(const std::shared_ptr<Job>& job) {
  if (job->job_type_ != ALLREDUCE && job->job_type_ != BROADCAST) {
    context_.NotifyJobCompletion(job, false, "only ALLREDUCE and BROADCAST jobs are supported");
    return true;
  }
  if (config_.general_.instant_job_completion) {
    job->SetJobStatus(RUNNING);
    context_.NotifyJobCompletion(job, true);
    return true;
  }
  cudaSetDevice(device_);
  if (!inline_launch_) {
    // Remember where the producer stream is now; the launcher orders the job after it.
    cudaEvent_t ready = GetEvent();
    cudaEventRecord(ready, static_cast<cudaStream_t>(job->producer_stream_));
    job->ready_event_ = ready;
    return false;  // goes through the scheduler
  }
  InFlight f;
  f.job = job;
  cudaStream_t user_stream = static_cast<cudaStream_t>(job->producer_stream_);
  cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(user_stream, &capture) != cudaSuccess) {
    capture = cudaStreamCaptureStatusNone;
    cudaGetLastError();
  }
  const bool capturing = capture == cudaStreamCaptureStatusActive;
  {
    std::lock_guard<std::mutex> lk(launch_mu_);
    job->SetJobStatus(QUEUED);
    job->SetJobStatus(RUNNING);
    // Not while capturing: an event recorded outside the capture cannot be waited on inside
    // it. A captured job is ordered by the graph it becomes part of; whoever replays that
    // graph next to other jobs of this context orders the two.
    if (!capturing && order_valid_ && order_stream_ != user_stream)
      cudaStreamWaitEvent(user_stream, order_event_, 0);
    LaunchJob(job, user_stream, &f, capturing);
    if (!capturing && cudaEventRecord(order_event_, user_stream) == cudaSuccess) {
      order_stream_ = user_stream;
      order_valid_ = true;
    } else if (!capturing) {
      cudaGetLastError();
    }
  }
  if (capturing) {
    // The kernels now live in the graph under capture and run whenever it is replayed;
    // as far as this submission goes the job is done.
    context_.NotifyJobCompletion(job, f.launch_error.empty(), f.launch_error);
    return true;
  }
  {
    std::lock_guard<std::mutex> lk(q_mu_);
    inflight_.push_back(std::move(f));
  }
  q_cv_.notify_all();
  return true;
}

// [backend.cuda] numa_bind: keep a service thread on the cores next to the GPU (the reference
// pins its RDMA worker threads to the NIC's NUMA node, rdma_worker_thread.cc:77).
void CudaBackend::BindServiceThread(const char* what) {
  if (!config_.backend_.cuda.numa_bind) return;
  char bus[32] = {0};
  if (cudaDeviceGetPCIBusId(bus, sizeof(bus), device_) != cudaSuccess) {
    cudaGetLastError();
    return;
  }
  for (char* p = bus; *p; ++p) *p = static_cast<char>(tolower(*p));  // sysfs spells bus ids in lower case
  int node = GetDeviceNuma(bus);
  if (node < 0 || !BindToNumaNode(node)) {
    SML_VLOG(1) << what << " thread: no NUMA binding (device " << bus << ", node " << node << ")";
  } else {
    SML_VLOG(1) << what << " thread bound to NUMA node " << node << " of device " << bus;
  }
}

void CudaBackend::LauncherLoop() {
  cudaSetDevice(device_);
  BindServiceThread("launcher");
  JobSlice js;
  while (context_.GetContextState() == Context::RUNNING && context_.GetJobSlice(0, js)) {
    InFlight f;
    f.job = js.job;
    f.via_scheduler = true;
    f.slice = js;
    f.ready = static_cast<cudaEvent_t>(js.job->ready_event_);
    {
      std::lock_guard<std::mutex> lk(launch_mu_);
      if (f.ready) cudaStreamWaitEvent(comm_stream_, f.ready, 0);
      LaunchJob(js.job, comm_stream_, &f);
    }
    {
      std::lock_guard<std::mutex> lk(q_mu_);
      inflight_.push_back(std::move(f));
    }
    q_cv_.notify_all();
    // The scheduler's barrier (one consumer) lets us take the next job at once: jobs are
    // queued back to back on the stream and complete in order.
  }
}

void CudaBackend::CompletionLoop() {
  cudaSetDevice(device_);
  BindServiceThread("completion");
  Stats& stats = context_.GetStats();
  for (;;) {
    InFlight f;
    {
      std::unique_lock<std::mutex> lk(q_mu_);
      q_cv_.wait(lk, [this] { return stop_completer_ || !inflight_.empty(); });
      if (inflight_.empty()) return;  // stop requested and nothing left
      f = std::move(inflight_.front());
      inflight_.pop_front();
    }
    bool ok = f.launch_error.empty();
    std::string why = f.launch_error;
    if (ok) {
      cudaError_t e = cudaEventSynchronize(f.done);
      if (e != cudaSuccess) {
        ok = false;
        why = std::string("device error: ") + cudaGetErrorString(e);
        failed_ = true;
      } else {
        int st = *reinterpret_cast<volatile int*>(host_status_ + f.status_slot);
        if (st != kernels::STATUS_OK) {
          ok = false;
          std::ostringstream o;
          if ((st & 0xf) == kernels::STATUS_TIMEOUT) {
            o << "a peer did not arrive within " << config_.backend_.cuda.wait_timeout_ms
              << " ms (channel " << (st >> 8) << ", phase " << ((st >> 4) & 0xf) << ")";
            stats.AddTimeouts(0, 1);
          } else if ((st & 0xf) == kernels::STATUS_BOUNDS) {
            o << "checked build: a tile of channel " << (st >> 8) << " would reach outside its region";
          } else {
            o << "kernel status " << st;
          }
          why = o.str();
          failed_ = true;
        }
      }
    }
    stats.AddTotalPktsSent(0, f.tiles);
    if (ok) stats.AddCorrectPktsReceived(0, f.tiles);
    PutEvent(f.ready);
    // f.done belongs to the job's EventState and returns to the pool with the job.
    if (f.via_scheduler) {
      if (!ok) f.job->failure_reason_ = why;
      context_.NotifyJobSliceCompletion(0, f.slice);
    } else {
      context_.NotifyJobCompletion(f.job, ok, why);
    }
  }
}

std::string CudaBackend::ExtraStatsJson() {
  unsigned long long c[16] = {0};
  if (dev_counters_) {
    cudaSetDevice(device_);
    cudaMemcpy(c, dev_counters_, sizeof(c), cudaMemcpyDeviceToHost);
  }
  std::ostringstream o;
  o << "{\"device\":" << device_ << ",\"multimem\":" << (ctx_.use_multimem ? "true" : "false")
    << ",\"tiles\":" << c[0] << ",\"wait_spins\":" << c[1] << ",\"device_timeouts\":" << c[2]
    << ",\"jobs_launched\":" << launched_jobs_ << ",\"kernel_launches\":" << kernel_launches_
    << ",\"epoch\":" << epoch_base_
    << ",\"channel0_ns\":{\"loader_wait\":" << c[3] << ",\"loader_work\":" << c[4] + c[9] + c[10] + c[11]
    << ",\"loader_scale_factors\":" << c[9] << ",\"loader_payload\":" << c[10] << ",\"loader_exponents_ahead\":" << c[11]
    << ",\"loader_signal\":" << c[4]
    << ",\"reducer_wait\":" << c[5] << ",\"reducer_work\":" << c[6] << ",\"storer_wait\":" << c[7]
    << ",\"storer_work\":" << c[8] << "}";
  if (dev_trace_) {
    // The last job's timeline on channel 0, in ns after the kernel's start: for each role, when its
    // waits for a tile were over and when it had finished the tile (0 = the job had no such tile).
    std::vector<unsigned long long> t(kernels::kTraceWords);
    cudaMemcpy(t.data(), dev_trace_, t.size() * sizeof(t[0]), cudaMemcpyDeviceToHost);
    const unsigned long long t0 = t[6 * kernels::kTraceTiles];
    static const char* names[6] = {"loader_began", "loader_finished", "reducer_began", "reducer_finished",
                                   "storer_began", "storer_finished"};
    o << ",\"channel0_trace_ns\":{";
    for (int row = 0; row < 6; row++) {
      o << (row ? "," : "") << "\"" << names[row] << "\":[";
      for (int k = 0; k < kernels::kTraceTiles; k++) {
        unsigned long long v = t[row * kernels::kTraceTiles + k];
        o << (k ? "," : "") << (v > t0 ? v - t0 : 0);
      }
      o << "]";
    }
    o << "}";
  }
  o << "}";
  return o.str();
}

int CudaBackend::RunWaitProbe(double budget_ms) {
  cudaSetDevice(device_);
  std::lock_guard<std::mutex> lk(launch_mu_);
  kernels::RankCtx probe = ctx_;
  probe.timeout_ns = static_cast<unsigned long long>(budget_ms * 1e6);
  cudaStream_t s = comm_stream_;
  int st = -1;
  int slot = kStatusSlots - 1;
  host_status_[slot] = kernels::STATUS_OK;
  probe.status = dev_status_ + slot;
  cudaError_t e = kernels::LaunchWaitProbe(probe, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e == cudaSuccess) st = *reinterpret_cast<volatile int*>(host_status_ + slot);
  return e == cudaSuccess ? st : -static_cast<int>(e);
}

}  // namespace

Backend* CreateCudaBackend(Context& context, Config& config) {
  return new CudaBackend(context, config);
}

// ---------------------------------------------------------------------------------------

bool KernelsCheckedBuild() { return kernels::CheckedBuild(); }

int ConvertU8OnDevice(bool widen, const void* in, void* out, unsigned long long numel, void* stream,
                      std::string* error) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = widen ? kernels::LaunchWidenU8(in, out, numel, s) : kernels::LaunchNarrowI32(in, out, numel, s);
  if (e != cudaSuccess) {
    if (error) *error = cudaGetErrorString(e);
    cudaGetLastError();
  }
  return static_cast<int>(e);
}

int EmulatedAllReduce(int nranks, void* const* in_ptrs, void* const* out_ptrs,
                      unsigned long long numel, int elem_type, int mode, int algo, int block_numel,
                      size_t slot_bytes, int slots_per_channel, int channels, float post_scale,
                      int repeats, int exponent_lookahead, std::string* error) {
  using namespace kernels;
  auto fail = [&](const std::string& m, int code) {
    if (error) *error = m;
    return code;
  };
  if (nranks < 1 || nranks > kMaxRanks) return fail("nranks out of range", -1);
  if (algo == ALGO_ZEROCOPY) return fail("zero-copy needs real symmetric memory", -1);
  if (slot_bytes / 4 / block_numel * slots_per_channel > 8192)
    return fail("slots_per_channel * slot_bytes / (4 * block_numel) exceeds 8192", -1);
  int dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return fail("no CUDA device", -2);
  int esz = elem_type == ELEM_BF16 ? 2 : 4;
  size_t oneshot_bytes = algo == ALGO_ONESHOT ? (numel * esz + 255) / 256 * 256 : 256;
  int max_channels = prop.multiProcessorCount / nranks;  // all virtual ranks share the GPU
  if (max_channels < 1) max_channels = 1;
  if (channels > 0 && channels < max_channels) max_channels = channels;

  RankCtx proto;
  memset(&proto, 0, sizeof(proto));
  proto.nranks = nranks;
  proto.slot_bytes = slot_bytes;
  proto.slots_per_channel = slots_per_channel;
  proto.sc_fence = 0;
  proto.exp_ring = ExpRingDepth(slots_per_channel);
  proto.exp_lookahead = ExpLookahead(slots_per_channel, exponent_lookahead < 0 ? kDefaultExpLookahead : exponent_lookahead);
  proto.block_numel = block_numel;
  proto.quant_base = quant::QuantBase(nranks);
  proto.oneshot_bytes = oneshot_bytes;
  proto.timeout_ns = 2000000000ull;  // 2 s: generous for one GPU, still bounded
  size_t bytes = StagingBytes(slot_bytes, slots_per_channel, block_numel, max_channels,
                              oneshot_bytes, nranks, &proto.data_offset, &proto.exp_offset,
                              &proto.oneshot_offset);
  proto.stage_bytes = ReportedStageBytes(bytes);
  std::vector<char*> stage(nranks, nullptr);
  int* status = nullptr;
  unsigned long long* counters = nullptr;
  RankCtx* d_ctx = nullptr;
  JobArgs* d_job = nullptr;
  unsigned long long* epochs = nullptr;
  int result = 0;
  cudaError_t e = cudaSuccess;
  auto cleanup = [&] {
    for (char* p : stage) if (p) cudaFree(p);
    if (status) cudaFree(status);
    if (counters) cudaFree(counters);
    if (epochs) cudaFree(epochs);
    if (d_ctx) cudaFree(d_ctx);
    if (d_job) cudaFree(d_job);
  };
  for (int r = 0; r < nranks && e == cudaSuccess; r++) {
    e = cudaMalloc(&stage[r], bytes);
    if (e == cudaSuccess) e = cudaMemset(stage[r], 0, bytes);
  }
  if (e == cudaSuccess) e = cudaMalloc(&status, nranks * sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(status, 0, nranks * sizeof(int));
  if (e == cudaSuccess) e = cudaMalloc(&counters, nranks * 16 * sizeof(unsigned long long));
  if (e == cudaSuccess) e = cudaMemset(counters, 0, nranks * 16 * sizeof(unsigned long long));
  if (e == cudaSuccess) e = cudaMalloc(&epochs, nranks * kMaxChannels * sizeof(unsigned long long));
  if (e == cudaSuccess) e = cudaMemset(epochs, 0, nranks * kMaxChannels * sizeof(unsigned long long));
  if (e == cudaSuccess) e = cudaMalloc(&d_ctx, nranks * sizeof(RankCtx));
  if (e == cudaSuccess) e = cudaMalloc(&d_job, nranks * sizeof(JobArgs));
  if (e != cudaSuccess) {
    cleanup();
    return fail(std::string("allocation failed: ") + cudaGetErrorString(e), -3);
  }
  if (algo == ALGO_PUSH && PushTileCapacity(proto, elem_type, mode) == 0) {
    cleanup();
    return fail("ALGO_PUSH needs at least two ranks and slots of about twice nranks * max(block, 128) * 4 bytes", -1);
  }
  std::vector<RankCtx> ctxs(nranks, proto);
  std::vector<JobArgs> jobs(nranks);
  unsigned long long epoch = 0;
  for (int it = 0; it < (repeats < 1 ? 1 : repeats) && result == 0; it++) {
    LaunchPlan plan;
    for (int r = 0; r < nranks; r++) {
      ctxs[r].rank = r;
      for (int p = 0; p < nranks; p++) ctxs[r].stage_peer[p] = stage[p];
      ctxs[r].status = status + r;
      ctxs[r].counters = counters + r * 16;
      ctxs[r].epoch_words = epochs + static_cast<size_t>(r) * kMaxChannels;
      JobArgs& j = jobs[r];
      memset(&j, 0, sizeof(j));
      j.in = in_ptrs[r];
      j.out = out_ptrs[r];
      j.numel = numel;
      j.elem_type = elem_type;
      j.mode = mode;
      j.algo = algo;
      j.post_scale = post_scale;
      j.bulk_copy = DeviceMemory(j.in) && DeviceMemory(j.out);
      j.oneshot_parity = it & 1;
    }
    plan = PlanLaunch(ctxs[0], jobs[0], channels, max_channels);
    for (int r = 0; r < nranks; r++) {
      jobs[r].tile_elems = plan.tile_elems;
      jobs[r].epochs = plan.epochs;
    }
    epoch += plan.epochs;
    cudaMemcpy(d_ctx, ctxs.data(), nranks * sizeof(RankCtx), cudaMemcpyHostToDevice);
    cudaMemcpy(d_job, jobs.data(), nranks * sizeof(JobArgs), cudaMemcpyHostToDevice);
    e = LaunchAllReduceEmulated(d_ctx, d_job, jobs[0], nranks, plan, 0);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
      result = fail(std::string("emulated launch failed: ") + cudaGetErrorString(e), -4);
      break;
    }
    std::vector<int> st(nranks);
    cudaMemcpy(st.data(), status, nranks * sizeof(int), cudaMemcpyDeviceToHost);
    for (int r = 0; r < nranks; r++) {
      if (st[r] != STATUS_OK) result = fail("kernel status " + std::to_string(st[r]) + " on rank " + std::to_string(r), st[r]);
    }
  }
  cleanup();
  return result;
}

}  // namespace switchml
