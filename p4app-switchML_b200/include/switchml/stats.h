// Counters collected while a context runs.
//
// Parity: reference client_lib/src/stats.h:40-167 and stats.cc:58-186 — jobs
// submitted/finished, list of submitted sizes, per-worker-thread packets sent, correct
// and wrong packets received, timeouts; InitStats/ResetStats/LogStats with '#'-delimited
// values for scraping; DescribeIntList/DescribeFloatList/List2Str helpers. On the cuda
// backend a "packet" is one staged tile of a channel. Unlike the reference the counters
// are atomics, so the report is coherent when read while jobs run.
#ifndef SWITCHML_STATS_H_
#define SWITCHML_STATS_H_

#include <atomic>
#include <memory>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

#include "switchml/common.h"

namespace switchml {

class Stats {
 public:
  Stats();
  ~Stats();
  Stats(const Stats&) = delete;
  void operator=(const Stats&) = delete;

  void InitStats(WorkerTid num_worker_threads);
  void LogStats();
  void ResetStats();
  // The same report LogStats() prints, as a string / as JSON.
  std::string Report();
  std::string ToJson();

  std::string DescribeIntList(std::vector<uint64_t> list);
  std::string DescribeFloatList(std::vector<double> list);
  template <typename T>
  std::string List2Str(std::vector<T> list) {
    std::ostringstream o;
    o << "[";
    for (size_t i = 0; i < list.size(); i++) o << (i ? ", " : "") << list[i];
    o << "]";
    return o.str();
  }

  inline void IncJobsSubmittedNum() { jobs_submitted_num_++; }
  void AppendJobSubmittedNumel(uint64_t size);
  inline void IncJobsFinishedNum() { jobs_finished_num_++; }
  inline void IncJobsFailedNum() { jobs_failed_num_++; }
  inline void AddTotalPktsSent(WorkerTid t, uint64_t n) { total_pkts_sent_[t] += n; }
  inline void AddCorrectPktsReceived(WorkerTid t, uint64_t n) { correct_pkts_received_[t] += n; }
  inline void AddWrongPktsReceived(WorkerTid t, uint64_t n) { wrong_pkts_received_[t] += n; }
  inline void AddTimeouts(WorkerTid t, uint64_t n) { timeouts_num_[t] += n; }

  uint64_t jobs_submitted_num() const { return jobs_submitted_num_; }
  uint64_t jobs_finished_num() const { return jobs_finished_num_; }
  uint64_t jobs_failed_num() const { return jobs_failed_num_; }
  uint64_t total_pkts_sent(WorkerTid t) const { return total_pkts_sent_[t]; }
  uint64_t correct_pkts_received(WorkerTid t) const { return correct_pkts_received_[t]; }
  uint64_t wrong_pkts_received(WorkerTid t) const { return wrong_pkts_received_[t]; }
  uint64_t timeouts_num(WorkerTid t) const { return timeouts_num_[t]; }
  WorkerTid num_worker_threads() const { return num_worker_threads_; }

 private:
  WorkerTid num_worker_threads_ = 0;
  std::atomic<uint64_t> jobs_submitted_num_{0};
  std::atomic<uint64_t> jobs_finished_num_{0};
  std::atomic<uint64_t> jobs_failed_num_{0};
  std::mutex list_mu_;
  std::vector<uint64_t> jobs_submitted_numel_;
  std::unique_ptr<std::atomic<uint64_t>[]> total_pkts_sent_;
  std::unique_ptr<std::atomic<uint64_t>[]> wrong_pkts_received_;
  std::unique_ptr<std::atomic<uint64_t>[]> correct_pkts_received_;
  std::unique_ptr<std::atomic<uint64_t>[]> timeouts_num_;
};

}  // namespace switchml
#endif  // SWITCHML_STATS_H_
