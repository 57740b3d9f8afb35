// Statistics report. Parity: reference client_lib/src/stats.cc:58-186 (same fields,
// '#'-delimited values, sum/mean/max/min/median/stdev of job sizes).
#include "switchml/stats.h"

#include <algorithm>
#include <cmath>
#include <numeric>

#include "switchml/log.h"

namespace switchml {

Stats::Stats() {}
Stats::~Stats() {}

void Stats::InitStats(WorkerTid n) {
  num_worker_threads_ = n;
  total_pkts_sent_.reset(new std::atomic<uint64_t>[n]);
  wrong_pkts_received_.reset(new std::atomic<uint64_t>[n]);
  correct_pkts_received_.reset(new std::atomic<uint64_t>[n]);
  timeouts_num_.reset(new std::atomic<uint64_t>[n]);
  ResetStats();
}

void Stats::ResetStats() {
  jobs_submitted_num_ = 0;
  jobs_finished_num_ = 0;
  jobs_failed_num_ = 0;
  {
    std::lock_guard<std::mutex> lk(list_mu_);
    jobs_submitted_numel_.clear();
  }
  for (WorkerTid i = 0; i < num_worker_threads_; i++) {
    total_pkts_sent_[i] = 0;
    wrong_pkts_received_[i] = 0;
    correct_pkts_received_[i] = 0;
    timeouts_num_[i] = 0;
  }
}

void Stats::AppendJobSubmittedNumel(uint64_t size) {
  std::lock_guard<std::mutex> lk(list_mu_);
  jobs_submitted_numel_.push_back(size);
}

template <typename T>
static std::string Describe(std::vector<T> v) {
  std::ostringstream o;
  if (v.empty()) return "Sum: #0# Mean: #0# Max: #0# Min: #0# Median: #0# Stdev: #0#";
  std::sort(v.begin(), v.end());
  long double sum = 0;
  for (const T& x : v) sum += x;
  long double mean = sum / v.size();
  long double var = 0;
  for (const T& x : v) var += (x - mean) * (x - mean);
  var /= v.size();
  long double median = v.size() % 2 ? static_cast<long double>(v[v.size() / 2])
                                    : (static_cast<long double>(v[v.size() / 2 - 1]) + v[v.size() / 2]) / 2;
  o << "Sum: #" << static_cast<double>(sum) << "# Mean: #" << static_cast<double>(mean)
    << "# Max: #" << v.back() << "# Min: #" << v.front() << "# Median: #"
    << static_cast<double>(median) << "# Stdev: #" << static_cast<double>(std::sqrt(var)) << "#";
  return o.str();
}

std::string Stats::DescribeIntList(std::vector<uint64_t> list) { return Describe(std::move(list)); }
std::string Stats::DescribeFloatList(std::vector<double> list) { return Describe(std::move(list)); }

std::string Stats::Report() {
  std::ostringstream o;
  std::vector<uint64_t> numels;
  {
    std::lock_guard<std::mutex> lk(list_mu_);
    numels = jobs_submitted_numel_;
  }
  std::vector<uint64_t> sent, ok, wrong, to;
  for (WorkerTid i = 0; i < num_worker_threads_; i++) {
    sent.push_back(total_pkts_sent_[i]);
    ok.push_back(correct_pkts_received_[i]);
    wrong.push_back(wrong_pkts_received_[i]);
    to.push_back(timeouts_num_[i]);
  }
  auto total = [](const std::vector<uint64_t>& v) {
    return std::accumulate(v.begin(), v.end(), uint64_t(0));
  };
  o << "Stats:"
    << "\n    Submitted jobs: #" << jobs_submitted_num_.load() << "#"
    << "\n    Submitted jobs sizes: #" << List2Str(numels) << "#"
    << "\n    Submitted jobs sizes distribution: " << DescribeIntList(numels)
    << "\n    Finished jobs: #" << jobs_finished_num_.load() << "#"
    << "\n    Failed jobs: #" << jobs_failed_num_.load() << "#"
    << "\n    Worker threads:"
    << "\n        Total packets sent: #" << List2Str(sent) << "# Sum: #" << total(sent) << "#"
    << "\n        Correct packets received: #" << List2Str(ok) << "# Sum: #" << total(ok) << "#"
    << "\n        Wrong packets received: #" << List2Str(wrong) << "# Sum: #" << total(wrong) << "#"
    << "\n        Number of timeouts: #" << List2Str(to) << "# Sum: #" << total(to) << "#";
  return o.str();
}

std::string Stats::ToJson() {
  std::ostringstream o;
  std::vector<uint64_t> numels;
  {
    std::lock_guard<std::mutex> lk(list_mu_);
    numels = jobs_submitted_numel_;
  }
  auto arr = [&](const std::unique_ptr<std::atomic<uint64_t>[]>& a) {
    std::ostringstream s;
    s << "[";
    for (WorkerTid i = 0; i < num_worker_threads_; i++) s << (i ? "," : "") << a[i].load();
    s << "]";
    return s.str();
  };
  o << "{\"jobs_submitted\":" << jobs_submitted_num_.load()
    << ",\"jobs_finished\":" << jobs_finished_num_.load()
    << ",\"jobs_failed\":" << jobs_failed_num_.load() << ",\"jobs_submitted_numel\":[";
  for (size_t i = 0; i < numels.size(); i++) o << (i ? "," : "") << numels[i];
  o << "],\"total_pkts_sent\":" << arr(total_pkts_sent_)
    << ",\"correct_pkts_received\":" << arr(correct_pkts_received_)
    << ",\"wrong_pkts_received\":" << arr(wrong_pkts_received_)
    << ",\"timeouts\":" << arr(timeouts_num_) << "}";
  return o.str();
}

void Stats::LogStats() { SML_VLOG(1) << Report(); }

}  // namespace switchml
