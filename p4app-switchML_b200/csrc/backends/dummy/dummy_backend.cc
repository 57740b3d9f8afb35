// See dummy_backend.h.
#include "backends/dummy/dummy_backend.h"

#include <arpa/inet.h>
#include <time.h>

#include <algorithm>
#include <random>

#include "backends/slot_window.h"
#include "switchml/context.h"
#include "switchml/log.h"
#include "switchml/prepostprocessor.h"

namespace switchml {

namespace {

class DummyTransport : public SlotTransport {
 public:
  DummyTransport(const Config& cfg, WorkerTid tid)
      : cfg_(cfg), rng_(0x9e3779b97f4a7c15ull ^ static_cast<uint64_t>(tid)) {}

  void Send(const SlotPacket& p, bool) override { pending_.push_back(p.slot); }

  bool Poll(std::vector<SlotPacket>& slots, std::vector<int>* ready) override {
    if (pending_.empty()) return true;
    // A random, non-empty subset in random order.
    std::shuffle(pending_.begin(), pending_.end(), rng_);
    size_t n = 1 + rng_() % pending_.size();
    uint64_t bytes = 0;
    for (size_t i = 0; i < n; i++) {
      int s = pending_.back();
      pending_.pop_back();
      SlotPacket& p = slots[s];
      if (cfg_.backend_.dummy.process_packets) {
        uint32_t nw = cfg_.general_.num_workers;
        for (uint16_t j = 0; j < p.numel; j++) {
          uint32_t v = ntohl(static_cast<uint32_t>(p.payload[j]));
          p.payload[j] = static_cast<int32_t>(htonl(v * nw));  // two's complement product
        }
      }
      bytes += static_cast<uint64_t>(p.numel) * 4;
      ready->push_back(s);
    }
    float mbps = cfg_.backend_.dummy.bandwidth;
    if (mbps > 0) {
      // All worker threads share the modelled link.
      double ns = static_cast<double>(bytes) * 8.0 * cfg_.general_.num_worker_threads / mbps * 1e3;
      struct timespec ts;
      ts.tv_sec = static_cast<time_t>(ns / 1e9);
      ts.tv_nsec = static_cast<long>(ns - ts.tv_sec * 1e9);
      nanosleep(&ts, nullptr);
    }
    return true;
  }

 private:
  const Config& cfg_;
  std::mt19937_64 rng_;
  std::vector<int> pending_;
};

}  // namespace

DummyBackend::DummyBackend(Context& context, Config& config) : Backend(context, config) {}
DummyBackend::~DummyBackend() { CleanupWorker(); }

void DummyBackend::SetupWorker() {
  for (WorkerTid t = 0; t < static_cast<WorkerTid>(config_.general_.num_worker_threads); t++) {
    threads_.emplace_back(&DummyBackend::WorkerLoop, this, t);
  }
}

void DummyBackend::CleanupWorker() {
  for (auto& t : threads_) {
    if (t.joinable()) t.join();
  }
  threads_.clear();
}

void DummyBackend::WorkerLoop(WorkerTid tid) {
  const GeneralConfig& g = config_.general_;
  int window = static_cast<int>(g.max_outstanding_packets / g.num_worker_threads);
  int packet_numel = static_cast<int>(g.packet_numel);
  auto ppp = PrePostProcessor::CreateInstance(config_, tid, g.packet_numel * 4, window);
  DummyTransport transport(config_, tid);
  std::vector<int32_t> pool;
  Stats& stats = context_.GetStats();
  auto running = [this] { return context_.GetContextState() == Context::RUNNING; };
  JobSlice js;
  while (running() && context_.GetJobSlice(tid, js)) {
    SML_VLOG(2) << "worker thread " << tid << " got a slice of job " << js.job->id_ << " with "
                << js.slice.numel << " elements";
    if (js.slice.numel > 0 && !g.instant_job_completion) {
      SlotWindowResult r = RunSlotWindow(js, *ppp, transport, window, packet_numel, pool, running);
      stats.AddTotalPktsSent(tid, r.sent);
      stats.AddCorrectPktsReceived(tid, r.received);
      stats.AddWrongPktsReceived(tid, r.wrong);
      if (!r.ok) js.job->failure_reason_ = "context stopped during the job";
    }
    context_.NotifyJobSliceCompletion(tid, js);
  }
  SML_VLOG(1) << "worker thread " << tid << " exiting";
}

}  // namespace switchml
