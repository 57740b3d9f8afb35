// TimeoutQueue: constant-time bookkeeping of which outstanding slot expires next.
//
// Every entry gets the same time-to-live, so insertion order equals expiry order and a
// doubly linked list addressed by slot index gives O(1) Push/Remove/Check. After
// `threshold` expiries the time-to-live doubles and the threshold grows by `increment`
// (exponential back-off), like the reference (backends/rdma/rdma_timeout_queue.cc:55-135
// and dpdk_worker_thread_utils.inc:225-265).
#ifndef SWITCHML_TIMEOUT_QUEUE_H_
#define SWITCHML_TIMEOUT_QUEUE_H_

#include <chrono>
#include <cstdint>
#include <vector>

namespace switchml {

class TimeoutQueue {
 public:
  typedef std::chrono::steady_clock::time_point TimePoint;

  TimeoutQueue(int num_entries, double timeout_ms, uint64_t threshold, uint64_t increment)
      : nodes_(num_entries), timeout_us_(static_cast<int64_t>(timeout_ms * 1000.0)),
        threshold_(threshold), increment_(increment) {}

  // (Re)arm entry `i` at time `now`; it becomes the youngest entry.
  void Push(int i, TimePoint now) {
    if (nodes_[i].linked) Unlink(i);
    Node& n = nodes_[i];
    n.stamp = now;
    n.prev = tail_;
    n.next = -1;
    n.linked = true;
    if (tail_ >= 0) nodes_[tail_].next = i; else head_ = i;
    tail_ = i;
  }
  void Remove(int i) {
    if (nodes_[i].linked) Unlink(i);
  }
  // Index of the oldest entry if it has expired at `now`, else -1. The entry stays
  // armed; the caller re-Pushes it when it retransmits.
  int Check(TimePoint now) {
    if (head_ < 0) return -1;
    int64_t age = std::chrono::duration_cast<std::chrono::microseconds>(now - nodes_[head_].stamp).count();
    if (age < timeout_us_) return -1;
    if (++timeouts_ >= threshold_) {
      timeout_us_ *= 2;
      threshold_ += increment_;
    }
    return head_;
  }
  bool Empty() const { return head_ < 0; }
  uint64_t timeouts() const { return timeouts_; }
  double timeout_ms() const { return timeout_us_ / 1000.0; }

 private:
  struct Node {
    TimePoint stamp;
    int prev = -1, next = -1;
    bool linked = false;
  };
  void Unlink(int i) {
    Node& n = nodes_[i];
    if (n.prev >= 0) nodes_[n.prev].next = n.next; else head_ = n.next;
    if (n.next >= 0) nodes_[n.next].prev = n.prev; else tail_ = n.prev;
    n.linked = false;
    n.prev = n.next = -1;
  }
  std::vector<Node> nodes_;
  int head_ = -1, tail_ = -1;
  int64_t timeout_us_;
  uint64_t threshold_, increment_, timeouts_ = 0;
};

}  // namespace switchml
#endif  // SWITCHML_TIMEOUT_QUEUE_H_
