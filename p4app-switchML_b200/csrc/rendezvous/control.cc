// See control.h.
#include "rendezvous/control.h"

#include <arpa/inet.h>
#include <errno.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <chrono>
#include <cstring>
#include <sstream>

#include "switchml/log.h"

namespace switchml {

std::string HexEncode(const std::string& raw) {
  static const char* d = "0123456789abcdef";
  std::string o;
  o.reserve(raw.size() * 2 + 1);
  for (unsigned char c : raw) {
    o.push_back(d[c >> 4]);
    o.push_back(d[c & 15]);
  }
  if (o.empty()) o = "-";
  return o;
}

std::string HexDecode(const std::string& hex) {
  std::string o;
  if (hex == "-") return o;
  auto v = [](char c) { return c <= '9' ? c - '0' : c - 'a' + 10; };
  for (size_t i = 0; i + 1 < hex.size(); i += 2) o.push_back(static_cast<char>(v(hex[i]) << 4 | v(hex[i + 1])));
  return o;
}

namespace {

bool WriteAll(int fd, const std::string& s) {
  size_t off = 0;
  while (off < s.size()) {
    ssize_t n = send(fd, s.data() + off, s.size() - off, MSG_NOSIGNAL);
    if (n <= 0) {
      if (n < 0 && errno == EINTR) continue;
      return false;
    }
    off += static_cast<size_t>(n);
  }
  return true;
}

// Reads up to and excluding '\n'. `buf` keeps bytes beyond the line for the next call.
bool ReadLine(int fd, std::string* buf, std::string* line, const std::atomic<bool>* stop,
              int timeout_ms = -1) {
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (;;) {
    if (timeout_ms >= 0 && std::chrono::steady_clock::now() > deadline) return false;
    size_t nl = buf->find('\n');
    if (nl != std::string::npos) {
      *line = buf->substr(0, nl);
      buf->erase(0, nl + 1);
      return true;
    }
    struct pollfd p = {fd, POLLIN, 0};
    int r = poll(&p, 1, 200);
    if (stop && stop->load()) return false;
    if (r < 0 && errno != EINTR) return false;
    if (r <= 0) continue;
    char tmp[4096];
    ssize_t n = recv(fd, tmp, sizeof(tmp), 0);
    if (n == 0) return false;
    if (n < 0) {
      if (errno == EINTR || errno == EAGAIN) continue;
      return false;
    }
    buf->append(tmp, static_cast<size_t>(n));
  }
}

}  // namespace

ControlServer::ControlServer() {
  memset(learned_, 0, sizeof(learned_));
  for (int i = 0; i < kMaxPipes; i++) {
    udp_fds_[i] = -1;
    pending_udp_fds_[i] = -1;
    udp_ports_[i] = 0;
    udp_rx_packets_[i] = udp_rx_bytes_[i] = udp_tx_packets_[i] = udp_tx_bytes_[i] = 0;
  }
}

// A bound, non-connected UDP socket with large buffers, or -1 with the reason in *err.
static int BindUdp(const std::string& ip, unsigned port, uint16_t* bound, std::string* err) {
  int fd = socket(AF_INET, SOCK_DGRAM, 0);
  if (fd < 0) {
    *err = strerror(errno);
    return -1;
  }
  sockaddr_in u;
  memset(&u, 0, sizeof(u));
  u.sin_family = AF_INET;
  u.sin_port = htons(static_cast<uint16_t>(port));
  if (inet_pton(AF_INET, ip.c_str(), &u.sin_addr) != 1) u.sin_addr.s_addr = htonl(INADDR_ANY);
  int big = 8 << 20;
  setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &big, sizeof(big));
  setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &big, sizeof(big));
  if (bind(fd, reinterpret_cast<sockaddr*>(&u), sizeof(u)) != 0) {
    *err = strerror(errno);
    close(fd);
    return -1;
  }
  socklen_t al = sizeof(u);
  getsockname(fd, reinterpret_cast<sockaddr*>(&u), &al);
  *bound = ntohs(u.sin_port);
  return fd;
}
ControlServer::~ControlServer() { Stop(); }

bool ControlServer::Start(const std::string& ip, uint16_t port, uint16_t udp_port, int pipes) {
  listen_fd_ = socket(AF_INET, SOCK_STREAM, 0);
  if (listen_fd_ < 0) return false;
  int one = 1;
  setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in a;
  memset(&a, 0, sizeof(a));
  a.sin_family = AF_INET;
  a.sin_port = htons(port);
  if (inet_pton(AF_INET, ip.c_str(), &a.sin_addr) != 1) a.sin_addr.s_addr = htonl(INADDR_ANY);
  if (bind(listen_fd_, reinterpret_cast<sockaddr*>(&a), sizeof(a)) != 0 ||
      listen(listen_fd_, 64) != 0) {
    SML_LOG(ERROR) << "control server: cannot listen on " << ip << ":" << port << ": "
                   << strerror(errno);
    close(listen_fd_);
    listen_fd_ = -1;
    return false;
  }
  socklen_t al = sizeof(a);
  getsockname(listen_fd_, reinterpret_cast<sockaddr*>(&a), &al);
  port_ = ntohs(a.sin_port);

  ip_ = ip;
  pipes_ = 0;
  if (udp_port) {
    if (pipes < 1) pipes = 1;
    if (pipes > kMaxPipes) pipes = kMaxPipes;
    for (int i = 0; i < pipes; i++) {
      uint16_t bound = 0;
      std::string err;
      int fd = BindUdp(ip, udp_port + i, &bound, &err);
      if (fd < 0 && i > 0) {
        // The neighbouring port is taken: any free port does, the workers are told the
        // actual port of every pipe when they open their session.
        SML_VLOG(1) << "software switch: UDP port " << udp_port + i << " is taken (" << err << "), pipe " << i
                    << " gets a port chosen by the kernel";
        fd = BindUdp(ip, 0, &bound, &err);
      }
      if (fd < 0) {
        SML_LOG(ERROR) << "software switch: cannot bind UDP port " << udp_port + i << ": " << err;
        for (int j = 0; j < i; j++) {
          close(udp_fds_[j]);
          udp_fds_[j] = -1;
        }
        close(listen_fd_);
        listen_fd_ = -1;
        return false;
      }
      udp_fds_[i] = fd;
      udp_ports_[i] = bound;
    }
    pipes_ = pipes;
    stopping_ = false;
    for (int i = 0; i < pipes; i++) data_threads_.emplace_back(&ControlServer::DataPlaneLoop, this, i);
  }
  stopping_ = false;
  accepting_ = true;
  accept_thread_ = std::thread(&ControlServer::AcceptLoop, this);
  SML_VLOG(1) << "control server listening on " << ip << ":" << port_
              << (pipes_ ? " (software switch on UDP " + std::to_string(udp_ports_[0].load()) + ", " +
                               std::to_string(pipes_) + " pipe(s))"
                         : "");
  return true;
}

void ControlServer::StopAccepting() {
  accepting_ = false;
  if (accept_thread_.joinable()) accept_thread_.join();
  if (listen_fd_ >= 0) close(listen_fd_);
  listen_fd_ = -1;
}

void ControlServer::Stop() {
  if (listen_fd_ < 0 && udp_fds_[0] < 0 && !accept_thread_.joinable() && conn_threads_.empty()) return;
  stopping_ = true;
  {
    // Release anybody blocked in a collective.
    std::lock_guard<std::mutex> lk(coll_mu_);
    for (auto& kv : collectives_) {
      std::lock_guard<std::mutex> cl(kv.second->mu);
      kv.second->cv.notify_all();
    }
  }
  if (accept_thread_.joinable()) accept_thread_.join();
  for (auto& t : data_threads_)
    if (t.joinable()) t.join();
  data_threads_.clear();
  std::vector<std::thread> threads;
  {
    std::lock_guard<std::mutex> lk(conn_mu_);
    for (int fd : conn_fds_) shutdown(fd, SHUT_RDWR);
    threads.swap(conn_threads_);
  }
  for (auto& t : threads) t.join();
  if (listen_fd_ >= 0) close(listen_fd_);
  for (int i = 0; i < kMaxPipes; i++) {
    if (udp_fds_[i] >= 0) close(udp_fds_[i]);
    udp_fds_[i] = -1;
    int pend = pending_udp_fds_[i].exchange(-1);
    if (pend >= 0) close(pend);
  }
  pipes_ = 0;
  listen_fd_ = -1;
}

void ControlServer::AcceptLoop() {
  while (!stopping_ && accepting_) {
    struct pollfd p = {listen_fd_, POLLIN, 0};
    int r = poll(&p, 1, 200);
    if (r <= 0) continue;
    int fd = accept(listen_fd_, nullptr, nullptr);
    if (fd < 0) continue;
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    std::lock_guard<std::mutex> lk(conn_mu_);
    conn_fds_.push_back(fd);
    conn_threads_.emplace_back(&ControlServer::Serve, this, fd);
  }
}

void ControlServer::Serve(int fd) {
  std::string buf, line;
  while (!stopping_ && ReadLine(fd, &buf, &line, &stopping_)) {
    std::string reply;
    try {
      reply = Handle(line);
    } catch (const std::exception& e) {
      reply = std::string("ERR ") + e.what();
    }
    if (!WriteAll(fd, reply + "\n")) break;
  }
  close(fd);
  std::lock_guard<std::mutex> lk(conn_mu_);
  for (int& f : conn_fds_) {
    if (f == fd) f = -1;
  }
}

bool ControlServer::Collect(const std::string& name, int n, int rank, const std::string& token,
                            std::vector<std::string>* all) {
  Collective* c;
  {
    std::lock_guard<std::mutex> lk(coll_mu_);
    auto& slot = collectives_[name + "/" + std::to_string(n)];
    if (!slot) slot.reset(new Collective());
    c = slot.get();
  }
  std::unique_lock<std::mutex> lk(c->mu);
  if (c->tokens.size() != static_cast<size_t>(n)) c->tokens.assign(n, "");
  if (rank < 0 || rank >= n) return false;
  c->tokens[rank] = token;
  uint64_t gen = c->generation;
  if (++c->arrived == n) {
    c->arrived = 0;
    c->last_tokens = c->tokens;
    c->tokens.assign(n, "");
    c->generation++;
    c->cv.notify_all();
  } else {
    c->cv.wait(lk, [&] { return c->generation != gen || stopping_.load(); });
    if (c->generation == gen) return false;
  }
  *all = c->last_tokens;
  return true;
}

std::string ControlServer::RebindDataPlane(const std::string& ip, unsigned port) {
  if (pipes_ == 0) return "ERR no software switch in this server";
  // All pipes move: to port, port + 1, ... First bind them all, then hand them over.
  int fds[kMaxPipes];
  uint16_t bound[kMaxPipes];
  for (int i = 0; i < pipes_; i++) {
    std::string err;
    fds[i] = BindUdp(ip, port ? port + i : 0, &bound[i], &err);
    if (fds[i] < 0 && i > 0) fds[i] = BindUdp(ip, 0, &bound[i], &err);
    if (fds[i] < 0) {
      for (int j = 0; j < i; j++) close(fds[j]);
      return "ERR cannot bind " + ip + ":" + std::to_string(port + i) + ": " + err;
    }
  }
  for (int i = 0; i < pipes_; i++) {
    int previous = pending_udp_fds_[i].exchange(fds[i]);
    if (previous >= 0) close(previous);
  }
  // The data-plane threads adopt the sockets between two bursts (they poll with 100 ms).
  for (int i = 0; i < pipes_; i++) {
    for (int tries = 0; tries < 200 && pending_udp_fds_[i].load() == fds[i] && !stopping_; tries++) usleep(5 * 1000);
    if (pending_udp_fds_[i].load() == fds[i]) return "ERR the data plane did not pick up the new socket";
  }
  {
    std::lock_guard<std::mutex> lk(learned_mu_);
    ip_ = ip;
  }
  for (int i = 0; i < pipes_; i++) udp_ports_[i] = bound[i];
  return "OK " + std::to_string(bound[0]);
}

static std::string AddrText(const sockaddr_in& a) {
  char ip[INET_ADDRSTRLEN] = "?";
  inet_ntop(AF_INET, &a.sin_addr, ip, sizeof(ip));
  return std::string(ip) + ":" + std::to_string(ntohs(a.sin_port));
}

std::string ControlServer::DescribePorts() {
  // The "front panel" of the software switch: its control socket, its data-plane socket and
  // one virtual port per worker (the set of that worker's learned return addresses).
  std::ostringstream o;
  std::string ip;
  {
    std::lock_guard<std::mutex> lk(learned_mu_);
    ip = ip_;
  }
  o << " port  address  state  rx_pkts  rx_bytes  tx_pkts  tx_bytes\n";
  o << " control  " << ip << ":" << port_ << "/tcp  " << (listen_fd_ >= 0 ? "up" : "closed") << "  "
    << ctl_requests_.load() << "  -  -  -\n";
  for (int i = 0; i < (pipes_ ? pipes_ : 1); i++) {
    o << " data" << (i ? std::to_string(i) : "") << "  " << ip << ":" << udp_ports_[i].load() << "/udp  "
      << (udp_fds_[i] >= 0 ? "up" : "absent") << "  " << udp_rx_packets_[i].load() << "  " << udp_rx_bytes_[i].load()
      << "  " << udp_tx_packets_[i].load() << "  " << udp_tx_bytes_[i].load() << "\n";
  }
  for (int w = 0; w < switch_.num_workers(); w++) {
    int endpoints = 0;
    {
      std::lock_guard<std::mutex> lk(learned_mu_);
      for (int t = 0; t < kMaxThreads; t++) endpoints += learned_[w][t].sin_port != 0;
    }
    WorkerCounters c = switch_.worker_counters(w);
    o << " worker" << w << "  " << endpoints << " endpoint(s)  " << (endpoints ? "up" : "down") << "  "
      << c.rx_packets << "  " << c.rx_bytes << "  " << c.tx_packets << "  " << c.tx_bytes << "\n";
  }
  return o.str();
}

std::string ControlServer::DescribeForwarding() {
  std::ostringstream o;
  o << " rank  thread  address\n";
  std::lock_guard<std::mutex> lk(learned_mu_);
  for (int w = 0; w < kMaxWorkers; w++)
    for (int t = 0; t < kMaxThreads; t++)
      if (learned_[w][t].sin_port != 0) o << " " << w << "  " << t << "  " << AddrText(learned_[w][t]) << "\n";
  return o.str();
}

std::string ControlServer::Handle(const std::string& line) {
  ctl_requests_++;
  std::istringstream in(line);
  std::string cmd;
  in >> cmd;
  if (cmd == "BARRIER") {
    int n = 0;
    in >> n;
    // Barrier callers are anonymous: only the number of arrivals counts.
    Collective* c;
    {
      std::lock_guard<std::mutex> lk(coll_mu_);
      auto& slot = collectives_["barrier/" + std::to_string(n)];
      if (!slot) slot.reset(new Collective());
      c = slot.get();
    }
    std::unique_lock<std::mutex> lk(c->mu);
    uint64_t gen = c->generation;
    if (++c->arrived >= n) {
      c->arrived = 0;
      c->generation++;
      c->cv.notify_all();
    } else {
      c->cv.wait(lk, [&] { return c->generation != gen || stopping_.load(); });
      if (c->generation == gen) return "ERR server stopping";
    }
    return "OK";
  }
  if (cmd == "BCAST") {
    int n = 0, rank = 0, root = 0;
    uint64_t v = 0;
    in >> n >> rank >> root >> v;
    std::vector<std::string> all;
    if (root < 0 || root >= n || !Collect("bcast", n, rank, std::to_string(v), &all))
      return "ERR broadcast failed";
    return "OK " + all[root];
  }
  if (cmd == "GATHER") {
    int n = 0, rank = 0;
    std::string tok;
    in >> n >> rank >> tok;
    std::vector<std::string> all;
    if (!Collect("gather", n, rank, tok, &all)) return "ERR gather failed";
    std::string r = "OK";
    for (auto& t : all) r += " " + t;
    return r;
  }
  if (cmd == "UDPSESSION") {
    uint64_t session = 0;
    int rank = 0, n = 0, packet_numel = 0, nthreads = 0;
    std::string ip;
    unsigned port0 = 0;
    in >> session >> rank >> n >> packet_numel >> ip >> port0 >> nthreads;
    if (pipes_ == 0) return "ERR no software switch in this server";
    if (n < 1 || n > kMaxWorkers || rank < 0 || rank >= n) return "ERR bad rank or num_workers";
    if (packet_numel < 1 || packet_numel > kMaxPacketNumel) return "ERR bad packet_numel";
    // Rank 0 opens the session and wipes the switch; the others join afterwards (the
    // caller orders this with barriers, like the reference dpdk_backend.cc:95-128).
    if (rank == 0) switch_.Reset(session, n, packet_numel);
    if (switch_.session_id() != session) return "ERR unknown session";
    if (!switch_.AddWorker(rank)) return "ERR cannot add worker";
    (void)ip; (void)port0; (void)nthreads;  // return addresses are learned from the data packets
    // One UDP port per pipe; worker thread t uses the (t mod pipes)-th.
    std::string reply = "OK";
    for (int i = 0; i < pipes_; i++) reply += " " + std::to_string(udp_ports_[i].load());
    return reply;
  }
  if (cmd == "SHOW") {
    std::string what;
    in >> what;
    std::string text;
    if (what == "workers") text = switch_.DescribeWorkers();
    else if (what == "statistics") text = switch_.DescribeStatistics();
    else if (what == "drop") {
      double i, e;
      switch_.GetDropProbabilities(&i, &e);
      text = "ingress " + std::to_string(i) + " egress " + std::to_string(e) + "\n";
    } else if (what == "bitmap") {
      uint32_t slot = 0;
      in >> slot;
      text = "slot " + std::to_string(slot) + " set0 " + std::to_string(switch_.Bitmap(slot, 0)) +
             " set1 " + std::to_string(switch_.Bitmap(slot, 1)) + "\n";
    } else if (what == "slot") {
      uint32_t slot = 0;
      in >> slot;
      text = switch_.DescribeSlot(slot);
    } else if (what == "dropped") text = switch_.DescribeDropped();
    else if (what == "qp") text = switch_.DescribeEndpoints();
    else if (what == "ports") text = DescribePorts();
    else if (what == "forwarding") text = DescribeForwarding();
    else if (what == "address") {
      std::string ip;
      {
        std::lock_guard<std::mutex> lk(learned_mu_);
        ip = ip_;
      }
      text = "ip " + ip + " control_port " + std::to_string(port_) + " udp_port " +
             std::to_string(udp_ports_[0].load()) + " pipes " + std::to_string(pipes_) + "\n";
    } else return "ERR unknown table";
    return "OK " + HexEncode(text);
  }
  if (cmd == "SET") {
    std::string what;
    in >> what;
    if (what == "address") {
      std::string ip;
      unsigned port = 0;
      in >> ip >> port;
      if (ip.empty() || port > 65535) return "ERR usage: SET address <ip> <udp port>";
      return RebindDataPlane(ip, port);
    }
    if (what != "drop") return "ERR unknown setting";
    double i = 0, e = 0;
    uint64_t seed = 0;
    in >> i >> e >> seed;
    switch_.SetDropProbabilities(i, e, seed);
    return "OK";
  }
  if (cmd == "RESET") {
    switch_.Reset(0, 0, 0);
    std::lock_guard<std::mutex> lk(learned_mu_);
    memset(learned_, 0, sizeof(learned_));
    return "OK";
  }
  if (cmd == "PING") return "OK";
  return "ERR unknown command '" + cmd + "'";
}

void ControlServer::DataPlaneLoop(int pipe) {
  // Datagrams are received and sent in bursts, one system call per burst (the reference's
  // workers use rx/tx bursts of 64, config.cc:86-88; the hardware switch needs none).
  const int kBurst = 64;
  const size_t kStride = (kWireMaxBytes + 63) / 64 * 64;
  std::vector<uint8_t> rx(static_cast<size_t>(kBurst) * kStride);
  std::vector<sockaddr_in> from(kBurst);
  std::vector<iovec> rx_iov(kBurst);
  std::vector<mmsghdr> rx_msgs(kBurst);
  for (int i = 0; i < kBurst; i++) {
    rx_iov[i].iov_base = rx.data() + static_cast<size_t>(i) * kStride;
    rx_iov[i].iov_len = kStride;
  }
  std::vector<SwitchOutput> out;
  std::vector<sockaddr_in> to;
  std::vector<iovec> tx_iov;
  std::vector<mmsghdr> tx_msgs;
  while (!stopping_) {
    int pend = pending_udp_fds_[pipe].exchange(-1);
    if (pend >= 0) {
      // "SET address": move the data plane to the new socket. Workers learn the port when
      // they open a session, so sessions that are running keep talking to a closed port
      // and must be restarted, as after a change of the reference switch's address.
      close(udp_fds_[pipe]);
      udp_fds_[pipe] = pend;
    }
    const int fd = udp_fds_[pipe];
    struct pollfd p = {fd, POLLIN, 0};
    int r = poll(&p, 1, 100);
    if (r <= 0) continue;
    for (int i = 0; i < kBurst; i++) {
      memset(&rx_msgs[i], 0, sizeof(mmsghdr));
      rx_msgs[i].msg_hdr.msg_iov = &rx_iov[i];
      rx_msgs[i].msg_hdr.msg_iovlen = 1;
      rx_msgs[i].msg_hdr.msg_name = &from[i];
      rx_msgs[i].msg_hdr.msg_namelen = sizeof(sockaddr_in);
    }
    int got = recvmmsg(fd, rx_msgs.data(), kBurst, MSG_DONTWAIT, nullptr);
    if (got <= 0) continue;
    out.clear();
    to.clear();
    for (int m = 0; m < got; m++) {
      const uint8_t* data = rx.data() + static_cast<size_t>(m) * kStride;
      const size_t n = rx_msgs[m].msg_len;
      const sockaddr_in& src = from[m];
      udp_rx_packets_[pipe]++;
      udp_rx_bytes_[pipe] += n;
      if (n >= sizeof(WireHeader)) {
        // Learn where this worker thread listens, like a switch learns a port. Echo
        // requests may come from anybody and teach nothing.
        WireHeader h;
        memcpy(&h, data, sizeof(h));
        int w = ntohs(h.worker_id);
        if (ntohl(h.magic) == kWireMagic && h.type != WIRE_ECHO_REQUEST && w < kMaxWorkers &&
            h.thread_id < kMaxThreads) {
          std::lock_guard<std::mutex> lk(learned_mu_);
          learned_[w][h.thread_id] = src;
        }
      }
      const size_t before = out.size();
      switch_.Process(data, n, &out);
      for (size_t o = before; o < out.size(); o++) {
        sockaddr_in d = src;
        if (!out[o].to_sender) {
          const int dw = out[o].dest_worker, dt = out[o].dest_thread;
          if (dw < 0 || dw >= kMaxWorkers || dt < 0 || dt >= kMaxThreads) {
            memset(&d, 0, sizeof(d));  // no such port: port 0 is skipped below
          } else {
            std::lock_guard<std::mutex> lk(learned_mu_);
            d = learned_[dw][dt];
          }
        }
        to.push_back(d);
      }
    }
    // One sendmmsg for everything this burst produced (destinations that were never learned
    // are skipped).
    tx_iov.resize(out.size());
    tx_msgs.resize(out.size());
    size_t count = 0;
    for (size_t o = 0; o < out.size(); o++) {
      if (to[o].sin_port == 0) continue;
      tx_iov[count].iov_base = out[o].bytes.data();
      tx_iov[count].iov_len = out[o].bytes.size();
      memset(&tx_msgs[count], 0, sizeof(mmsghdr));
      tx_msgs[count].msg_hdr.msg_iov = &tx_iov[count];
      tx_msgs[count].msg_hdr.msg_iovlen = 1;
      tx_msgs[count].msg_hdr.msg_name = &to[o];
      tx_msgs[count].msg_hdr.msg_namelen = sizeof(sockaddr_in);
      udp_tx_bytes_[pipe] += out[o].bytes.size();
      count++;
    }
    udp_tx_packets_[pipe] += count;
    size_t done = 0;
    while (done < count) {
      int sent = sendmmsg(fd, tx_msgs.data() + done, static_cast<unsigned>(count - done), 0);
      if (sent <= 0) {
        if (sent < 0 && errno == EINTR) continue;
        break;  // the workers' retransmission timers cover what was not sent
      }
      done += static_cast<size_t>(sent);
    }
  }
}

// ----------------------------------------------------------------------------------------

ControlClient::ControlClient() {}
ControlClient::~ControlClient() { Close(); }

bool ControlClient::Connect(const std::string& ip, uint16_t port, int timeout_ms) {
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (;;) {
    int fd = socket(AF_INET, SOCK_STREAM, 0);
    sockaddr_in a;
    memset(&a, 0, sizeof(a));
    a.sin_family = AF_INET;
    a.sin_port = htons(port);
    inet_pton(AF_INET, ip.c_str(), &a.sin_addr);
    if (fd >= 0 && connect(fd, reinterpret_cast<sockaddr*>(&a), sizeof(a)) == 0) {
      int one = 1;
      setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
      fd_ = fd;
      return true;
    }
    if (fd >= 0) close(fd);
    if (std::chrono::steady_clock::now() > deadline) {
      SML_LOG(ERROR) << "cannot reach the controller at " << ip << ":" << port;
      return false;
    }
    usleep(50 * 1000);
  }
}

void ControlClient::Close() {
  if (fd_ >= 0) close(fd_);
  fd_ = -1;
}

bool ControlClient::RoundTrip(const std::string& line, std::string* reply, int timeout_ms) {
  std::lock_guard<std::mutex> lk(mu_);
  if (fd_ < 0) return false;
  if (!WriteAll(fd_, line + "\n")) return false;
  std::string r;
  if (!ReadLine(fd_, &rbuf_, &r, nullptr, timeout_ms)) {
    // The reply may still arrive later and would be taken for the answer to the next
    // request: this connection is no longer usable.
    close(fd_);
    fd_ = -1;
    return false;
  }
  if (r.compare(0, 2, "OK") != 0) {
    SML_LOG(ERROR) << "controller replied: " << r << " (to '" << line.substr(0, 60) << "')";
    return false;
  }
  *reply = r.size() > 3 ? r.substr(3) : "";
  return true;
}

bool ControlClient::Barrier(int n, int timeout_ms) {
  std::string r;
  return RoundTrip("BARRIER " + std::to_string(n), &r, timeout_ms);
}

bool ControlClient::Broadcast(int n, int rank, int root, uint64_t* value) {
  std::string r;
  if (!RoundTrip("BCAST " + std::to_string(n) + " " + std::to_string(rank) + " " +
                     std::to_string(root) + " " + std::to_string(*value), &r))
    return false;
  *value = strtoull(r.c_str(), nullptr, 10);
  return true;
}

bool ControlClient::AllGather(int n, int rank, const std::string& token,
                              std::vector<std::string>* all) {
  std::string r;
  if (!RoundTrip("GATHER " + std::to_string(n) + " " + std::to_string(rank) + " " + token, &r))
    return false;
  std::istringstream in(r);
  all->clear();
  std::string t;
  while (in >> t) all->push_back(t);
  return all->size() == static_cast<size_t>(n);
}

bool ControlClient::CreateUdpSession(uint64_t session_id, int rank, int num_workers,
                                     int packet_numel, const std::string& my_ip, uint16_t port0,
                                     int nthreads, std::string* switch_ip,
                                     std::vector<uint16_t>* switch_udp_ports) {
  std::ostringstream o;
  o << "UDPSESSION " << session_id << " " << rank << " " << num_workers << " " << packet_numel
    << " " << my_ip << " " << port0 << " " << nthreads;
  std::string r;
  if (!RoundTrip(o.str(), &r)) return false;
  (void)switch_ip;
  switch_udp_ports->clear();
  std::istringstream ports(r);
  unsigned p;
  while (ports >> p) switch_udp_ports->push_back(static_cast<uint16_t>(p));
  return !switch_udp_ports->empty();
}

bool ControlClient::Command(const std::string& line, std::string* reply) {
  std::string r;
  if (!RoundTrip(line, &r)) return false;
  if (line.compare(0, 4, "SHOW") == 0) r = HexDecode(r);
  *reply = r;
  return true;
}

}  // namespace switchml
