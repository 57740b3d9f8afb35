// See soft_switch.h.
#include "backends/softswitch/soft_switch.h"

#include <arpa/inet.h>

#include <cstddef>
#include <cstring>

#include "simd/simd_kernels.h"
#include <sstream>

namespace switchml {

SoftSwitch::SoftSwitch(uint32_t num_slots) : num_slots_(num_slots), rng_(0x5eed) {
  sets_[0].resize(num_slots_);
  sets_[1].resize(num_slots_);
}

void SoftSwitch::Reset(uint64_t session_id, int num_workers, int packet_numel) {
  std::unique_lock<std::shared_mutex> lk(state_mu_);
  for (int k = 0; k < 2; k++) {
    for (SlotSet& s : sets_[k]) s = SlotSet();
  }
  session_id_ = session_id;
  num_workers_ = num_workers;
  packet_numel_ = packet_numel;
  registered_ = 0;
  counters_ = SwitchCounters();
  for (WorkerCounters& w : worker_counters_) w = WorkerCounters();
  for (auto& row : endpoint_counters_)
    for (EndpointCounters& e : row) e = EndpointCounters();
}

bool SoftSwitch::AddWorker(int rank) {
  std::unique_lock<std::shared_mutex> lk(state_mu_);
  if (rank < 0 || rank >= num_workers_ || rank >= kMaxWorkers) return false;
  registered_ |= 1u << rank;
  return true;
}

void SoftSwitch::SetDropProbabilities(double ingress, double egress, uint64_t seed) {
  std::unique_lock<std::shared_mutex> lk(state_mu_);
  drop_ingress_ = ingress < 0 ? 0 : (ingress > 1 ? 1 : ingress);
  drop_egress_ = egress < 0 ? 0 : (egress > 1 ? 1 : egress);
  if (seed) rng_.seed(seed);
}

void SoftSwitch::GetDropProbabilities(double* ingress, double* egress) const {
  std::shared_lock<std::shared_mutex> lk(state_mu_);
  *ingress = drop_ingress_;
  *egress = drop_egress_;
}

bool SoftSwitch::Roll(double p) {
  if (p <= 0) return false;
  std::lock_guard<std::mutex> lk(rng_mu_);
  return std::uniform_real_distribution<double>(0.0, 1.0)(rng_) < p;
}

void SoftSwitch::Emit(const SlotSet& s, uint16_t pool_index, int dest_worker, int dest_thread,
                      uint8_t type, std::vector<SwitchOutput>* out) {
  if (Roll(drop_egress_)) {
    counters_.egress_dropped++;
    worker_counters_[dest_worker].egress_dropped++;
    return;
  }
  if (dest_thread < kMaxThreads) {
    EndpointCounters& e = endpoint_counters_[dest_worker][dest_thread];
    if (type == WIRE_RESULT_RETX) e.retransmitted_results++;
    else e.results++;
  }
  SwitchOutput o;
  o.dest_worker = dest_worker;
  o.dest_thread = dest_thread;
  o.bytes.resize(sizeof(WireHeader) + s.numel * 4u);
  WireHeader h;
  h.magic = htonl(kWireMagic);
  h.type = type;
  h.job_tag = s.job_tag;
  h.worker_id = htons(static_cast<uint16_t>(dest_worker));
  h.pkt_id = htonl(s.pkt_id);
  h.pool_index = htons(pool_index);
  h.numel = htons(s.numel);
  h.exponent = s.exponent;
  h.thread_id = static_cast<uint8_t>(dest_thread);
  h.session_lo = htons(static_cast<uint16_t>(session_id_));
  memcpy(o.bytes.data(), &h, sizeof(h));
  simd::Swap32(s.values.data(), s.numel, reinterpret_cast<int32_t*>(o.bytes.data() + sizeof(h)));
  worker_counters_[dest_worker].tx_packets++;
  worker_counters_[dest_worker].tx_bytes += o.bytes.size();
  out->push_back(std::move(o));
}

void SoftSwitch::Process(const uint8_t* data, size_t len, std::vector<SwitchOutput>* out) {
  std::shared_lock<std::shared_mutex> state(state_mu_);
  WireHeader h;
  if (len < sizeof(h)) { counters_.malformed++; return; }
  memcpy(&h, data, sizeof(h));
  uint16_t numel = ntohs(h.numel);
  int worker = ntohs(h.worker_id);
  uint16_t pool_index = ntohs(h.pool_index);
  if (ntohl(h.magic) == kWireMagic && (h.type == WIRE_ECHO_REQUEST || h.type == WIRE_FORWARD)) {
    ProcessOther(h, data, len, out);
    return;
  }
  const bool last_packet = h.type == WIRE_DATA;  // carries the message's exponent
  if (ntohl(h.magic) != kWireMagic || (h.type != WIRE_DATA && h.type != WIRE_DATA_MORE) || numel > kMaxPacketNumel ||
      len != sizeof(h) + numel * 4u || worker >= num_workers_ || worker >= kMaxWorkers ||
      h.thread_id >= kMaxThreads ||  // the return port is looked up by (worker, thread): refuse what the table cannot hold
      !(registered_ & (1u << worker)) || ntohs(h.session_lo) != static_cast<uint16_t>(session_id_) ||
      (pool_index & ~kSetBit) >= num_slots_) {
    counters_.malformed++;
    return;
  }
  worker_counters_[worker].rx_packets++;
  worker_counters_[worker].rx_bytes += len;
  if (Roll(drop_ingress_)) {
    counters_.ingress_dropped++;
    worker_counters_[worker].ingress_dropped++;
    return;
  }
  EndpointCounters* ep = &endpoint_counters_[worker][h.thread_id];
  ep->rx_packets++;
  if (last_packet) ep->rx_messages++;

  int k = (pool_index & kSetBit) ? 1 : 0;
  uint32_t slot = pool_index & ~kSetBit;
  std::lock_guard<std::mutex> slot_lock(slot_mu_[slot % kStripes]);  // both sets of the slot
  SlotSet& cur = sets_[k][slot];
  SlotSet& other = sets_[1 - k][slot];
  uint32_t bit = 1u << worker;

  // Bitmap stage: note the arrival in this set and acknowledge the other set.
  bool seen = (cur.bitmap & bit) != 0;
  cur.bitmap |= bit;
  other.bitmap &= ~bit;

  if (seen) {
    ep->out_of_order++;
    // A retransmission. If the slot is finished the worker lost the result: send it again
    // from the retained copy, to that worker only. Otherwise the first copy was already
    // absorbed and the aggregate is still waiting for others: nothing to do.
    if (cur.complete) {
      counters_.retransmit++;
      cur.n_retransmit++;
      Emit(cur, pool_index, worker, h.thread_id, WIRE_RESULT_RETX, out);
    } else {
      counters_.ignored++;
      cur.n_ignored++;
    }
    return;
  }

  const uint8_t* payload = data + sizeof(h);
  if (cur.remaining == 0) {
    // First packet of a new use of this slot set: overwrite.
    cur.values.assign(numel, 0);
    simd::AddWire(payload, numel, cur.values.data());
    cur.exponent = last_packet ? h.exponent : static_cast<int8_t>(-128);
    cur.numel = numel;
    cur.pkt_id = ntohl(h.pkt_id);
    cur.job_tag = h.job_tag;
    cur.complete = false;
    cur.remaining = static_cast<uint32_t>(num_workers_ - 1);
  } else {
    uint16_t n = numel < cur.numel ? numel : cur.numel;
    simd::AddWire(payload, n, cur.values.data());  // wrapping add, as the switch register ALUs do
    if (last_packet && h.exponent > cur.exponent) cur.exponent = h.exponent;
    cur.remaining--;
  }

  if (cur.remaining == 0) {
    cur.complete = true;
    counters_.broadcast++;
    cur.n_broadcast++;
    for (int w = 0; w < num_workers_; w++) Emit(cur, pool_index, w, h.thread_id, WIRE_RESULT, out);
  } else {
    counters_.consumed++;
    cur.n_consumed++;
  }
}

void SoftSwitch::ProcessOther(const WireHeader& h, const uint8_t* data, size_t len,
                              std::vector<SwitchOutput>* out) {
  int worker = ntohs(h.worker_id);
  if (worker >= kMaxWorkers || h.thread_id >= kMaxThreads || len > static_cast<size_t>(kWireMaxBytes)) {
    counters_.malformed++;
    return;
  }
  if (h.type == WIRE_ECHO_REQUEST) {
    // Answered for anyone who asks, registered or not, like a ping to the switch's address.
    SwitchOutput o;
    o.dest_worker = worker;
    o.dest_thread = h.thread_id;
    o.bytes.assign(data, data + len);
    o.bytes[offsetof(WireHeader, type)] = WIRE_ECHO_REPLY;
    o.to_sender = true;
    counters_.echo_replies++;
    out->push_back(std::move(o));
    return;
  }
  // WIRE_FORWARD: only between registered workers of the current session.
  uint16_t dest = ntohs(h.pool_index);
  int dest_worker = dest >> 8, dest_thread = dest & 0xff;
  if (worker >= num_workers_ || !(registered_ & (1u << worker)) ||
      ntohs(h.session_lo) != static_cast<uint16_t>(session_id_) || dest_thread >= kMaxThreads) {
    counters_.malformed++;
    return;
  }
  if (dest_worker == kFloodWorker) {
    counters_.flooded++;
    for (int w = 0; w < num_workers_; w++) {
      if (w == worker || !(registered_ & (1u << w))) continue;
      SwitchOutput o;
      o.dest_worker = w;
      o.dest_thread = dest_thread;
      o.bytes.assign(data, data + len);
      out->push_back(std::move(o));
    }
    return;
  }
  if (dest_worker >= num_workers_ || !(registered_ & (1u << dest_worker))) {
    counters_.malformed++;
    return;
  }
  counters_.forwarded++;
  SwitchOutput o;
  o.dest_worker = dest_worker;
  o.dest_thread = dest_thread;
  o.bytes.assign(data, data + len);
  out->push_back(std::move(o));
}

SwitchCounters SoftSwitch::counters() const {
  std::shared_lock<std::shared_mutex> lk(state_mu_);
  return counters_;
}

WorkerCounters SoftSwitch::worker_counters(int rank) const {
  std::shared_lock<std::shared_mutex> lk(state_mu_);
  return worker_counters_[rank];
}

EndpointCounters SoftSwitch::endpoint_counters(int rank, int thread) const {
  std::shared_lock<std::shared_mutex> lk(state_mu_);
  if (rank < 0 || rank >= kMaxWorkers || thread < 0 || thread >= kMaxThreads) return EndpointCounters();
  return endpoint_counters_[rank][thread];
}

uint32_t SoftSwitch::Bitmap(uint32_t slot, int set) const {
  std::shared_lock<std::shared_mutex> lk(state_mu_);
  std::lock_guard<std::mutex> slot_lock(slot_mu_[(slot % num_slots_) % kStripes]);
  return sets_[set & 1][slot % num_slots_].bitmap;
}

std::string SoftSwitch::DescribeWorkers() const {
  std::shared_lock<std::shared_mutex> lk(state_mu_);
  std::ostringstream o;
  o << "session " << session_id_ << ": " << num_workers_ << " worker(s), packet_numel "
    << packet_numel_ << "\n rank  registered  rx_pkts  rx_bytes  tx_pkts  tx_bytes\n";
  for (int w = 0; w < num_workers_; w++) {
    const WorkerCounters& c = worker_counters_[w];
    o << " " << w << "  " << ((registered_ >> w) & 1 ? "yes" : "no") << "  " << c.rx_packets << "  "
      << c.rx_bytes << "  " << c.tx_packets << "  " << c.tx_bytes << "\n";
  }
  return o.str();
}

std::string SoftSwitch::DescribeStatistics() const {
  std::shared_lock<std::shared_mutex> lk(state_mu_);
  std::ostringstream o;
  o << "broadcast " << counters_.broadcast << "\nretransmit " << counters_.retransmit
    << "\nconsumed " << counters_.consumed << "\nignored " << counters_.ignored
    << "\ningress_dropped " << counters_.ingress_dropped << "\negress_dropped "
    << counters_.egress_dropped << "\nmalformed " << counters_.malformed << "\necho_replies "
    << counters_.echo_replies << "\nforwarded " << counters_.forwarded << "\nflooded "
    << counters_.flooded << "\n";
  return o.str();
}

std::string SoftSwitch::DescribeSlot(uint32_t slot) const {
  std::shared_lock<std::shared_mutex> lk(state_mu_);
  slot %= num_slots_;
  std::lock_guard<std::mutex> slot_lock(slot_mu_[slot % kStripes]);
  std::ostringstream o;
  o << " set  bitmap  missing  complete  broadcast  retransmit  consumed  ignored\n";
  for (int k = 0; k < 2; k++) {
    const SlotSet& s = sets_[k][slot];
    o << " " << k << "  " << s.bitmap << "  " << s.remaining << "  " << (s.complete ? "yes" : "no") << "  "
      << s.n_broadcast << "  " << s.n_retransmit << "  " << s.n_consumed << "  " << s.n_ignored << "\n";
  }
  return o.str();
}

std::string SoftSwitch::DescribeDropped() const {
  std::shared_lock<std::shared_mutex> lk(state_mu_);
  std::ostringstream o;
  o << " rank  ingress_dropped  egress_dropped\n";
  for (int w = 0; w < num_workers_; w++)
    o << " " << w << "  " << worker_counters_[w].ingress_dropped << "  " << worker_counters_[w].egress_dropped
      << "\n";
  o << " total  " << counters_.ingress_dropped << "  " << counters_.egress_dropped << "\n";
  return o.str();
}

std::string SoftSwitch::DescribeEndpoints() const {
  std::shared_lock<std::shared_mutex> lk(state_mu_);
  std::ostringstream o;
  o << " rank  thread  rx_pkts  rx_msgs  out_of_order  results  retransmitted_results\n";
  for (int w = 0; w < num_workers_; w++) {
    for (int t = 0; t < kMaxThreads; t++) {
      const EndpointCounters& e = endpoint_counters_[w][t];
      if (e.rx_packets == 0 && e.results == 0 && e.retransmitted_results == 0) continue;
      o << " " << w << "  " << t << "  " << e.rx_packets << "  " << e.rx_messages << "  " << e.out_of_order << "  " << e.results << "  "
        << e.retransmitted_results << "\n";
    }
  }
  return o.str();
}

}  // namespace switchml
