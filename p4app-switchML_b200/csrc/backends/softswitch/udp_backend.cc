// See udp_backend.h.
#include "backends/softswitch/udp_backend.h"

#include <arpa/inet.h>
#include <errno.h>
#include <netinet/in.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <chrono>
#include <cstring>

#include "backends/slot_window.h"
#include "backends/softswitch/wire.h"
#include "backends/timeout_queue.h"
#include "switchml/context.h"
#include "switchml/log.h"
#include "switchml/prepostprocessor.h"
#include "switchml/utils.h"

namespace switchml {

namespace {

class UdpTransport : public SlotTransport {
 public:
  // `window` slots of one message each; a message is `pkts_per_msg` datagrams of packet_numel
  // elements on consecutive pool indices (reference rdma_worker_thread.cc:116-124).
  UdpTransport(const Config& cfg, WorkerTid tid, int fd, uint64_t session_id, int window, int pkts_per_msg)
      : cfg_(cfg), tid_(tid), fd_(fd), session_id_(session_id), window_(window), pkts_per_msg_(pkts_per_msg),
        packet_numel_(static_cast<int>(cfg.general_.packet_numel)),
        all_packets_(pkts_per_msg == 64 ? ~0ull : (1ull << pkts_per_msg) - 1),
        set_bits_(window, 0), answered_(window, 0), missing_(window, 0) {
    tx_headers_.resize(kBurst);
    tx_iov_.resize(2 * kBurst);
    tx_msgs_.resize(kBurst);
    rx_buf_.resize(static_cast<size_t>(kBurst) * kRxStride);
    rx_iov_.resize(kBurst);
    rx_msgs_.resize(kBurst);
    for (int i = 0; i < kBurst; i++) {
      rx_iov_[i].iov_base = rx_buf_.data() + static_cast<size_t>(i) * kRxStride;
      rx_iov_[i].iov_len = kRxStride;
      memset(&rx_msgs_[i], 0, sizeof(mmsghdr));
      rx_msgs_[i].msg_hdr.msg_iov = &rx_iov_[i];
      rx_msgs_[i].msg_hdr.msg_iovlen = 1;
    }
  }

  void BeginSlice(const JobSlice& js, uint64_t, int batch) override {
    job_tag_ = static_cast<uint8_t>(js.job->id_ & 0xff);
    foreign_tags_ = 0;
    batch_ = batch;
    timers_.reset(new TimeoutQueue(batch, cfg_.general_.timeout, cfg_.general_.timeout_threshold,
                                   cfg_.general_.timeout_threshold_increment));
  }

  void EndSlice() override {
    // Later jobs start at a different place of the pool so that a late packet of this
    // job cannot be mistaken for one of the next (reference dpdk_worker_thread.cc:100,392).
    shift_ = (shift_ + batch_) % window_;
  }

  void Send(const SlotPacket& p, bool retransmission) override {
    int phys = (p.slot + shift_) % window_;
    if (!retransmission) {
      set_bits_[phys] ^= 1;  // every new use takes the other set
      answered_[p.slot] = 0;
      missing_[p.slot] = all_packets_;
    }
    // Header and payload leave as two pieces of one datagram (no copy); the burst goes out
    // with one system call in Flush(). A retransmission repeats only the packets of the
    // message that are still unanswered.
    for (int j = 0; j < pkts_per_msg_; j++) {
      if (!(missing_[p.slot] >> j & 1)) continue;
      const bool last = j == pkts_per_msg_ - 1;
      uint16_t pool_index = static_cast<uint16_t>((tid_ * window_ + phys) * pkts_per_msg_ + j) |
                            (set_bits_[phys] ? kSetBit : 0);
      if (tx_count_ == kBurst) Flush();
      WireHeader& h = tx_headers_[tx_count_];
      h.magic = htonl(kWireMagic);
      h.type = last ? WIRE_DATA : WIRE_DATA_MORE;  // the message's one exponent rides on its last packet
      h.job_tag = job_tag_;
      h.worker_id = htons(cfg_.general_.rank);
      h.pkt_id = htonl(p.pkt_id * static_cast<uint32_t>(pkts_per_msg_) + static_cast<uint32_t>(j));
      h.pool_index = htons(pool_index);
      h.numel = htons(static_cast<uint16_t>(packet_numel_));
      h.exponent = last ? p.exponent : 0;
      h.thread_id = static_cast<uint8_t>(tid_);
      h.session_lo = htons(static_cast<uint16_t>(session_id_));
      iovec* v = &tx_iov_[2 * tx_count_];
      v[0].iov_base = &h;
      v[0].iov_len = sizeof(h);
      v[1].iov_base = p.payload + static_cast<size_t>(j) * packet_numel_;
      v[1].iov_len = packet_numel_ * 4u;
      memset(&tx_msgs_[tx_count_], 0, sizeof(mmsghdr));
      tx_msgs_[tx_count_].msg_hdr.msg_iov = v;
      tx_msgs_[tx_count_].msg_hdr.msg_iovlen = 2;
      tx_count_++;
    }
    timers_->Push(p.slot, std::chrono::steady_clock::now());
  }

  void Flush() override {
    int done = 0;
    while (done < tx_count_) {
      int r = sendmmsg(fd_, tx_msgs_.data() + done, static_cast<unsigned>(tx_count_ - done), 0);
      if (r <= 0) {
        if (r < 0 && (errno == EINTR)) continue;
        break;  // a lost datagram is what the retransmission timers are for
      }
      done += r;
    }
    tx_count_ = 0;
  }

  bool Poll(std::vector<SlotPacket>& slots, std::vector<int>* ready) override {
    struct pollfd pf = {fd_, POLLIN, 0};
    int r = poll(&pf, 1, 1);
    if (r < 0 && errno != EINTR) return false;
    if (r <= 0) return true;
    int got = recvmmsg(fd_, rx_msgs_.data(), kBurst, MSG_DONTWAIT, nullptr);
    for (int m = 0; m < got; m++) {
      const uint8_t* data = rx_buf_.data() + static_cast<size_t>(m) * kRxStride;
      size_t n = rx_msgs_[m].msg_len;
      WireHeader h;
      if (n < sizeof(h)) { ready->push_back(-1); continue; }
      memcpy(&h, data, sizeof(h));
      uint16_t numel = ntohs(h.numel);
      uint16_t pool_index = ntohs(h.pool_index);
      const int index = static_cast<int>(pool_index & ~kSetBit) - tid_ * window_ * pkts_per_msg_;
      const int phys = index >= 0 ? index / pkts_per_msg_ : -1, j = index >= 0 ? index % pkts_per_msg_ : 0;
      bool ok = ntohl(h.magic) == kWireMagic && (h.type == WIRE_RESULT || h.type == WIRE_RESULT_RETX) &&
                n == sizeof(h) + numel * 4u && numel == packet_numel_ && phys >= 0 && phys < window_;
      if (ok && h.job_tag != job_tag_) {
        // The switch stamps a result with the tag of the first packet that reached the slot, so
        // the workers' job counters must agree. A result that fits in every other respect but
        // carries another tag, again and again, means they do not (one worker submitted a job
        // that the others never saw): say so instead of retransmitting in silence.
        int ss = (phys - shift_ % window_ + window_) % window_;
        if (ss < static_cast<int>(slots.size()) && !answered(ss) &&
            slots[ss].pkt_id * static_cast<uint32_t>(pkts_per_msg_) + static_cast<uint32_t>(j) == ntohl(h.pkt_id) &&
            ++foreign_tags_ == 16) {
          SML_LOG(ERROR) << "worker thread " << tid_ << ": results for the packets of job tag " << int(job_tag_)
                         << " keep arriving with tag " << int(h.job_tag)
                         << ": the workers have not submitted the same sequence of jobs";
        }
        ok = false;
      }
      int s = -1;
      if (ok) {
        s = (phys - shift_ % window_ + window_) % window_;
        ok = s < static_cast<int>(slots.size()) && !answered(s) && (missing_[s] >> j & 1) &&
             slots[s].pkt_id * static_cast<uint32_t>(pkts_per_msg_) + static_cast<uint32_t>(j) == ntohl(h.pkt_id) &&
             ((pool_index & kSetBit) != 0) == (set_bits_[phys] != 0);
      }
      if (!ok) { ready->push_back(-1); continue; }  // duplicate, stale job or foreign packet
      SlotPacket& p = slots[s];
      memcpy(p.payload + static_cast<size_t>(j) * packet_numel_, data + sizeof(h), numel * 4u);
      if (j == pkts_per_msg_ - 1) p.exponent = h.exponent;
      missing_[s] &= ~(1ull << j);
      if (missing_[s] == 0) {  // the whole message is back
        mark_answered(s);
        ready->push_back(s);
      }
    }
    return true;
  }

  void OnAnswered(int slot) override { timers_->Remove(slot); }

  uint64_t OnIdle(std::vector<SlotPacket>& slots) override {
    uint64_t fired = 0;
    auto now = std::chrono::steady_clock::now();
    for (int s = timers_->Check(now); s >= 0; s = timers_->Check(now)) {
      SML_VLOG(3) << "worker thread " << tid_ << ": timeout on slot " << s << " pkt "
                  << slots[s].pkt_id << ", retransmitting";
      Send(slots[s], true);  // re-arms the timer
      fired++;
      now = std::chrono::steady_clock::now();
    }
    return fired;
  }

 private:
  bool answered(int s) const { return answered_[s] != 0; }
  void mark_answered(int s) { answered_[s] = 1; }

  const Config& cfg_;
  WorkerTid tid_;
  int fd_;
  uint64_t session_id_;
  int window_;
  int pkts_per_msg_, packet_numel_;
  uint64_t all_packets_;
  int batch_ = 0;
  int shift_ = 0;
  uint8_t job_tag_ = 0;
  uint64_t foreign_tags_ = 0;  // results that matched a waiting packet in everything but the job tag
  std::vector<uint8_t> set_bits_;
  std::vector<uint8_t> answered_;
  std::vector<uint64_t> missing_;  // per slot: packets of the current message without a result yet
  // Bursts of up to kBurst datagrams per system call in both directions (the reference's
  // burst_rx / burst_tx of 64, config.cc:86-88).
  static const int kBurst = 64;
  static const size_t kRxStride = (kWireMaxBytes + 63) / 64 * 64;
  std::vector<WireHeader> tx_headers_;
  std::vector<iovec> tx_iov_;
  std::vector<mmsghdr> tx_msgs_;
  int tx_count_ = 0;
  std::vector<uint8_t> rx_buf_;
  std::vector<iovec> rx_iov_;
  std::vector<mmsghdr> rx_msgs_;
  std::unique_ptr<TimeoutQueue> timers_;
};

}  // namespace

bool EchoSwitch(int fd, uint16_t worker, uint8_t thread, uint64_t session, int timeout_ms) {
  uint8_t pkt[sizeof(WireHeader) + 8];
  WireHeader h;
  memset(&h, 0, sizeof(h));
  h.magic = htonl(kWireMagic);
  h.type = WIRE_ECHO_REQUEST;
  h.worker_id = htons(worker);
  h.thread_id = thread;
  h.session_lo = htons(static_cast<uint16_t>(session));
  const uint64_t cookie = session ^ (static_cast<uint64_t>(worker) << 48) ^ (static_cast<uint64_t>(thread) << 40);
  h.pkt_id = htonl(static_cast<uint32_t>(cookie));
  memcpy(pkt, &h, sizeof(h));
  memcpy(pkt + sizeof(h), &cookie, 8);
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  while (std::chrono::steady_clock::now() < deadline) {
    if (send(fd, pkt, sizeof(pkt), 0) < 0 && errno != ECONNREFUSED) return false;
    struct pollfd p = {fd, POLLIN, 0};
    if (poll(&p, 1, 100) <= 0) continue;
    uint8_t in[kWireMaxBytes];
    ssize_t n = recv(fd, in, sizeof(in), MSG_DONTWAIT);
    if (n != static_cast<ssize_t>(sizeof(pkt))) continue;  // ECONNREFUSED or something else: ask again
    WireHeader r;
    memcpy(&r, in, sizeof(r));
    if (ntohl(r.magic) == kWireMagic && r.type == WIRE_ECHO_REPLY && memcmp(in + sizeof(r), &cookie, 8) == 0)
      return true;
  }
  return false;
}

UdpBackend::UdpBackend(Context& context, Config& config) : Backend(context, config) {}
UdpBackend::~UdpBackend() { CleanupWorker(); }

void UdpBackend::SetupWorker() {
  const GeneralConfig& g = config_.general_;
  const UdpBackendConfig& u = config_.backend_.udp;
  if (g.rank == 0 && u.spawn_switch) {
    server_.reset(new ControlServer());
    // One pipe per worker thread unless told otherwise: a pipe then serves the same thread of
    // every worker and never shares a slot stripe's lock with another pipe for long.
    int pipes = u.switch_pipes ? static_cast<int>(u.switch_pipes) : std::min<int>(g.num_worker_threads, 8);
    SML_CHECK(server_->Start(g.controller_ip_str, g.controller_port, u.switch_port, pipes))
        << "cannot start the in-process controller/software switch";
  }
  SML_CHECK(client_.Connect(g.controller_ip_str, g.controller_port)) << "controller unreachable";

  // Session id: rank 0's clock, shared through the controller (reference
  // dpdk_backend.cc:78-93).
  session_id_ = static_cast<uint64_t>(
      std::chrono::duration_cast<std::chrono::nanoseconds>(
          std::chrono::system_clock::now().time_since_epoch()).count());
  SML_CHECK(client_.Broadcast(g.num_workers, g.rank, 0, &session_id_)) << "session broadcast failed";

  // One socket per worker thread.
  for (int t = 0; t < g.num_worker_threads; t++) {
    int fd = socket(AF_INET, SOCK_DGRAM, 0);
    SML_CHECK(fd >= 0) << "socket(): " << strerror(errno);
    int big = 4 << 20;
    setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &big, sizeof(big));
    sockaddr_in me;
    memset(&me, 0, sizeof(me));
    me.sin_family = AF_INET;
    inet_pton(AF_INET, u.worker_ip_str.c_str(), &me.sin_addr);
    me.sin_port = htons(u.worker_port ? static_cast<uint16_t>(u.worker_port + t) : 0);
    SML_CHECK(bind(fd, reinterpret_cast<sockaddr*>(&me), sizeof(me)) == 0)
        << "cannot bind worker UDP port " << u.worker_port + t << ": " << strerror(errno);
    fds_.push_back(fd);
  }

  // Rank 0 opens the session (which clears the switch) before anybody else joins.
  std::string sw_ip;
  if (g.rank == 0) {
    SML_CHECK(client_.CreateUdpSession(session_id_, g.rank, g.num_workers, g.packet_numel,
                                       u.worker_ip_str, u.worker_port, g.num_worker_threads,
                                       &sw_ip, &switch_udp_ports_)) << "session setup failed";
    SML_CHECK(client_.Barrier(g.num_workers)) << "barrier failed";
  } else {
    SML_CHECK(client_.Barrier(g.num_workers)) << "barrier failed";
    SML_CHECK(client_.CreateUdpSession(session_id_, g.rank, g.num_workers, g.packet_numel,
                                       u.worker_ip_str, u.worker_port, g.num_worker_threads,
                                       &sw_ip, &switch_udp_ports_)) << "session setup failed";
  }
  // Worker thread t talks to pipe t mod pipes: its slots are then always served by the
  // same pipe of the switch.
  for (size_t t = 0; t < fds_.size(); t++) {
    sockaddr_in sw;
    memset(&sw, 0, sizeof(sw));
    sw.sin_family = AF_INET;
    inet_pton(AF_INET, u.switch_ip_str.c_str(), &sw.sin_addr);
    sw.sin_port = htons(switch_udp_ports_[t % switch_udp_ports_.size()]);
    SML_CHECK(connect(fds_[t], reinterpret_cast<sockaddr*>(&sw), sizeof(sw)) == 0)
        << "connect to switch: " << strerror(errno);
  }
  // Make sure the data plane answers before any job depends on it: one echo request per
  // socket (the switch answers these itself, like the reference switch answers ARP and
  // ping for its own address, p4/arp_icmp_responder.p4:40-84). The drop simulator does not
  // touch echo traffic, so a missing answer means a wrong address or a closed port.
  for (int t = 0; t < g.num_worker_threads; t++) {
    SML_CHECK(EchoSwitch(fds_[t], static_cast<uint16_t>(g.rank), static_cast<uint8_t>(t), session_id_, 2000))
        << "the software switch does not answer on UDP " << u.switch_ip_str << ":"
        << switch_udp_ports_[t % switch_udp_ports_.size()];
  }
  SML_CHECK(client_.Barrier(g.num_workers)) << "barrier failed";

  for (int t = 0; t < g.num_worker_threads; t++) {
    threads_.emplace_back(&UdpBackend::WorkerLoop, this, static_cast<WorkerTid>(t), fds_[t]);
  }
}

void UdpBackend::CleanupWorker() {
  for (auto& t : threads_) {
    if (t.joinable()) t.join();
  }
  threads_.clear();
  if (server_) server_->StopAccepting();
  if (client_.connected()) client_.Barrier(config_.general_.num_workers, 5000);
  for (int fd : fds_) close(fd);
  fds_.clear();
  client_.Close();
  if (server_) {
    server_->Stop();
    server_.reset();
  }
}

void UdpBackend::WorkerLoop(WorkerTid tid, int fd) {
  const GeneralConfig& g = config_.general_;
  // The unit of the window, of the timers and of the exponent is the message ([backend.udp]
  // msg_numel, one packet unless configured otherwise).
  const int msg_numel = static_cast<int>(config_.backend_.udp.msg_numel ? config_.backend_.udp.msg_numel : g.packet_numel);
  const int pkts_per_msg = msg_numel / static_cast<int>(g.packet_numel);
  int window = static_cast<int>(g.max_outstanding_packets / g.num_worker_threads) / pkts_per_msg;
  if (window < 1) window = 1;
  auto ppp = PrePostProcessor::CreateInstance(config_, tid, static_cast<Numel>(msg_numel) * 4, window);
  if (!config_.backend_.udp.cores.empty()) {
    int ids[256], count = 0;
    std::string err;
    if (ParseCoreList(config_.backend_.udp.cores, &err, ids, 256, &count) && tid < count && !BindToCore(ids[tid])) {
      SML_LOG(WARNING) << "worker thread " << tid << ": cannot bind to core " << ids[tid];
    }
  }
  UdpTransport transport(config_, tid, fd, session_id_, window, pkts_per_msg);
  std::vector<int32_t> pool;
  Stats& stats = context_.GetStats();
  auto running = [this] { return context_.GetContextState() == Context::RUNNING; };
  JobSlice js;
  while (running() && context_.GetJobSlice(tid, js)) {
    if (js.slice.numel > 0 && !g.instant_job_completion) {
      SlotWindowResult r = RunSlotWindow(js, *ppp, transport, window, msg_numel, pool, running);
      // the statistics count packets, as the reference's do (rdma_worker_thread.cc:187,283-292)
      stats.AddTotalPktsSent(tid, r.sent * pkts_per_msg);
      stats.AddCorrectPktsReceived(tid, r.received * pkts_per_msg);
      stats.AddWrongPktsReceived(tid, r.wrong);
      stats.AddTimeouts(tid, r.timeouts * pkts_per_msg);
      if (!r.ok) js.job->failure_reason_ = "context stopped during the job";
    }
    context_.NotifyJobSliceCompletion(tid, js);
  }
}

}  // namespace switchml
