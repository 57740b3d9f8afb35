// SoftSwitch: the aggregation pipeline of the programmable switch as a CPU state machine.
//
// It reproduces, per incoming packet, what the reference P4 program does in its ingress
// pipeline (p4/switchml.p4:96-192): drop simulator → worker bitmap update/check
// (bitmap_checker.p4:82-154) → worker counter (workers_counter.p4:25-111) → exponent max
// (exponents.p4:32-111) → 32-bit adders (processor.p4:32-127) → next step
// (next_step_selector.p4:112-204): consume, multicast the finished slot, or answer a
// retransmission from the retained copy of the slot. Every slot exists twice ("sets");
// using one set acknowledges the other, which is what makes retransmissions idempotent.
//
// The class has no sockets: Process() takes one packet and appends the packets to emit.
// The UDP front end lives in rendezvous/control.cc; tests drive it directly.
//
// Process() may be called from several threads at once (the front end can run several
// "pipes", each with its own socket, like the pipes of the switch ASIC): the session state
// is read under a shared lock, every slot belongs to one of 64 lock stripes, and the
// counters are atomic. Opening or resetting a session takes the state lock exclusively.
#ifndef SWITCHML_SOFT_SWITCH_H_
#define SWITCHML_SOFT_SWITCH_H_

#include <atomic>
#include <cstdint>
#include <mutex>
#include <random>
#include <shared_mutex>
#include <string>
#include <vector>

#include "backends/softswitch/wire.h"

namespace switchml {

struct SwitchOutput {
  int dest_worker;
  int dest_thread;
  std::vector<uint8_t> bytes;  // WireHeader + payload
  bool to_sender = false;      // send to the address the input came from (echo replies)
};

// A 64-bit event counter that several pipes may bump at once; reads and copies are
// snapshots (relaxed: the numbers are statistics, nothing synchronises on them).
struct Counter {
  std::atomic<uint64_t> v{0};
  Counter() {}
  Counter(uint64_t x) : v(x) {}
  Counter(const Counter& o) : v(o.v.load(std::memory_order_relaxed)) {}
  Counter& operator=(const Counter& o) {
    v.store(o.v.load(std::memory_order_relaxed), std::memory_order_relaxed);
    return *this;
  }
  void operator++(int) { v.fetch_add(1, std::memory_order_relaxed); }
  void operator+=(uint64_t x) { v.fetch_add(x, std::memory_order_relaxed); }
  operator uint64_t() const { return v.load(std::memory_order_relaxed); }
};

struct SwitchCounters {
  // per slot and set, like the counters behind the reference CLI's show_statistics
  Counter broadcast, retransmit, consumed, ignored;
  Counter ingress_dropped, egress_dropped, malformed;
  Counter echo_replies, forwarded, flooded;
};

struct WorkerCounters {
  Counter rx_packets, rx_bytes, tx_packets, tx_bytes;
  // packets of this worker lost to the drop simulator (reference: per-queue-pair dropped
  // counter of p4/drop_simulator.p4, shown by the CLI's show_dropped_packets)
  Counter ingress_dropped, egress_dropped;
};

// Per (worker, worker thread): the counterpart of the reference's per-queue-pair counters
// (controller/rdma_receiver.py:199-286: packets, messages, sequence violations). A thread's
// endpoint plays the role of a queue pair; a packet for a slot use that was already absorbed
// or finished is what a sequence violation is there: a packet outside the expected order.
struct EndpointCounters {
  Counter rx_packets, rx_messages, out_of_order, results, retransmitted_results;  // a message ends with its exponent-carrying packet
};

class SoftSwitch {
 public:
  explicit SoftSwitch(uint32_t num_slots = 16384);

  // Forget every worker and clear all registers (rank 0 does this when a session starts;
  // reference controller/grpc_server.py:234-236,332-334).
  void Reset(uint64_t session_id, int num_workers, int packet_numel);
  // Register a worker in the current session; false if the rank is out of range.
  bool AddWorker(int rank);
  int num_workers() const { return num_workers_; }
  uint64_t session_id() const { return session_id_; }

  // Feed one datagram; results (0, 1 or num_workers packets) are appended to `out`.
  void Process(const uint8_t* data, size_t len, std::vector<SwitchOutput>* out);

  // Fault injection: probability in [0,1] of dropping a packet on ingress / each copy on
  // egress (reference p4/drop_simulator.p4:24-71, controller/drop_simulator.py:45-93).
  void SetDropProbabilities(double ingress, double egress, uint64_t seed = 0);
  void GetDropProbabilities(double* ingress, double* egress) const;

  SwitchCounters counters() const;
  WorkerCounters worker_counters(int rank) const;
  EndpointCounters endpoint_counters(int rank, int thread) const;
  uint32_t Bitmap(uint32_t slot, int set) const;
  // Human-readable tables for the CLI.
  std::string DescribeWorkers() const;
  std::string DescribeStatistics() const;
  std::string DescribeDropped() const;
  // One slot: bitmap, missing packets and the per-slot counters of both sets (the reference
  // keeps four counters per slot and set in the next-step selector,
  // p4/next_step_selector.p4:37-40, shown by the CLI's show_statistics).
  std::string DescribeSlot(uint32_t slot) const;
  std::string DescribeEndpoints() const;

 private:
  struct SlotSet {
    uint32_t bitmap = 0;     // workers whose packet for this use has been absorbed
    uint32_t remaining = 0;  // packets still missing; 0 = idle or complete
    int8_t exponent = 0;
    uint16_t numel = 0;
    uint32_t pkt_id = 0;
    uint8_t job_tag = 0;
    bool complete = false;   // values hold a finished aggregate (the retained copy)
    // per slot and set: finished aggregates sent out, answers to retransmissions, packets
    // absorbed while waiting for others, duplicates ignored (reset with the session)
    uint32_t n_broadcast = 0, n_retransmit = 0, n_consumed = 0, n_ignored = 0;
    std::vector<int32_t> values;  // host order
  };

  void Emit(const SlotSet& s, uint16_t pool_index, int dest_worker, int dest_thread, uint8_t type,
            std::vector<SwitchOutput>* out);
  bool Roll(double p);
  // Echo and forwarding: everything that is not aggregation traffic.
  void ProcessOther(const WireHeader& h, const uint8_t* data, size_t len, std::vector<SwitchOutput>* out);

  static const int kStripes = 64;
  mutable std::shared_mutex state_mu_;        // session state: shared in Process(), exclusive to change it
  mutable std::mutex slot_mu_[kStripes];      // slot s is guarded by stripe s % kStripes
  std::mutex rng_mu_;
  uint32_t num_slots_;
  std::vector<SlotSet> sets_[2];
  int num_workers_ = 0;
  int packet_numel_ = 0;
  uint64_t session_id_ = 0;
  uint32_t registered_ = 0;
  double drop_ingress_ = 0, drop_egress_ = 0;
  std::mt19937_64 rng_;
  SwitchCounters counters_;
  WorkerCounters worker_counters_[kMaxWorkers];
  EndpointCounters endpoint_counters_[kMaxWorkers][kMaxThreads];
};

}  // namespace switchml
#endif  // SWITCHML_SOFT_SWITCH_H_
