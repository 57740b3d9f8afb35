// Control plane: the in-process replacement of the reference's controller.
//
// The reference runs a Python controller next to the switch that (a) serves a gRPC API
// to the workers — Session.{RdmaSession,UdpSession}, Sync.{Barrier,Broadcast}
// (protos/switchml.proto:21-91, controller/grpc_server.py:109-353, client side
// client_lib/src/grpc_client.{h,cc}) — and (b) offers an operator CLI
// (controller/cli.py). Here a ControlServer thread inside rank 0 (or the stand-alone
// switchml_switchd program) plays both roles over a line-based TCP protocol, and also
// hosts the UDP data plane of the software switch. ControlClient is what backends use.
//
// Requests are one text line each; the reply is one line starting with "OK" or "ERR".
//   BARRIER <n>                      wait until n callers arrived
//   BCAST <n> <rank> <root> <u64>    everyone receives root's value
//   GATHER <n> <rank> <token>        everyone receives all n tokens, ordered by rank
//   UDPSESSION <session> <rank> <n> <packet_numel> <ip> <port0> <nthreads>
//   SHOW workers|statistics|drop|dropped|qp|ports|forwarding|address|bitmap <s>|slot <s>   (CLI)
//   SET drop <ingress> <egress> [seed] | SET address <ip> <udp port>                 (CLI)
//   RESET | PING                                                                      (CLI)
// (docs/control_protocol.md is the full description, the counterpart of switchml.proto.)
// Collective requests are matched by arrival order, so all workers must issue them in
// the same sequence (they do: one per setup step).
#ifndef SWITCHML_RENDEZVOUS_CONTROL_H_
#define SWITCHML_RENDEZVOUS_CONTROL_H_

#include <netinet/in.h>

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "backends/softswitch/soft_switch.h"

namespace switchml {

class ControlServer {
 public:
  ControlServer();
  ~ControlServer();
  // Listen on ip:port (port 0 = pick one). `udp_port` > 0 also starts the software
  // switch data plane on that UDP port. With `pipes` > 1 the data plane runs that many
  // threads, each with a socket of its own on udp_port, udp_port + 1, ... (the switch ASIC
  // has four pipes, too); worker thread t talks to pipe t mod pipes, so a slot is always
  // served by the same pipe. Returns false if a socket cannot be bound.
  bool Start(const std::string& ip, uint16_t port, uint16_t udp_port = 0, int pipes = 1);
  void Stop();
  // Close the listening socket but keep serving the connections that exist. A rank that
  // restarts right after the final barrier of a shutdown then cannot reach the old server
  // by accident; it retries until the next one listens.
  void StopAccepting();
  uint16_t port() const { return port_; }
  uint16_t udp_port() const { return udp_ports_[0]; }
  int pipes() const { return pipes_; }
  static const int kMaxPipes = 8;
  SoftSwitch& soft_switch() { return switch_; }

 private:
  struct Collective {
    std::mutex mu;
    std::condition_variable cv;
    uint64_t generation = 0;
    int arrived = 0;
    std::vector<std::string> tokens;       // being collected
    std::vector<std::string> last_tokens;  // of the completed generation
  };
  void AcceptLoop();
  void Serve(int fd);
  void DataPlaneLoop(int pipe);
  std::string Handle(const std::string& line);
  // Blocks until `n` callers contributed; returns all tokens ordered by rank.
  bool Collect(const std::string& name, int n, int rank, const std::string& token,
               std::vector<std::string>* all);

  std::atomic<int> listen_fd_{-1};
  std::atomic<int> udp_fds_[kMaxPipes];
  int pipes_ = 0;  // 0: no data plane
  uint16_t port_ = 0;
  std::atomic<uint16_t> udp_ports_[kMaxPipes];
  std::atomic<bool> stopping_{false};
  std::atomic<bool> accepting_{false};
  std::thread accept_thread_;
  std::vector<std::thread> data_threads_;
  std::mutex conn_mu_;
  std::vector<std::thread> conn_threads_;
  std::vector<int> conn_fds_;
  std::mutex coll_mu_;
  std::map<std::string, std::unique_ptr<Collective>> collectives_;
  SoftSwitch switch_;
  // Return address of each worker thread, learned from its data packets (only the
  // data-plane thread touches this).
  // The forwarding table: return address of each worker thread, learned from its data
  // packets like a switch learns a port. Written by the data-plane thread, read by the
  // console commands.
  std::mutex learned_mu_;
  sockaddr_in learned_[kMaxWorkers][kMaxThreads];
  // Per data-plane socket ("port"): totals for the console's show_ports.
  std::atomic<uint64_t> udp_rx_packets_[kMaxPipes], udp_rx_bytes_[kMaxPipes], udp_tx_packets_[kMaxPipes],
      udp_tx_bytes_[kMaxPipes];
  std::atomic<uint64_t> ctl_requests_{0};
  std::string ip_;
  // A data-plane socket bound by "SET address", waiting to be adopted by the data-plane thread.
  std::atomic<int> pending_udp_fds_[kMaxPipes];
  std::string RebindDataPlane(const std::string& ip, unsigned port);
  std::string DescribePorts();
  std::string DescribeForwarding();
};

class ControlClient {
 public:
  ControlClient();
  ~ControlClient();
  // Retries for up to `timeout_ms` while the server is not up yet.
  bool Connect(const std::string& ip, uint16_t port, int timeout_ms = 30000);
  void Close();
  bool connected() const { return fd_ >= 0; }

  // Collective calls give up after `timeout_ms` (a peer that never arrives); the
  // connection is closed then, because a late reply would be misread.
  bool Barrier(int num_workers, int timeout_ms = 120000);
  bool Broadcast(int num_workers, int rank, int root, uint64_t* value);
  // `token` must not contain whitespace.
  bool AllGather(int num_workers, int rank, const std::string& token, std::vector<std::string>* all);
  bool CreateUdpSession(uint64_t session_id, int rank, int num_workers, int packet_numel,
                        const std::string& my_ip, uint16_t port0, int nthreads,
                        std::string* switch_ip, std::vector<uint16_t>* switch_udp_ports);  // one port per pipe
  // Send a raw command line (CLI); returns the reply without the leading "OK ".
  bool Command(const std::string& line, std::string* reply);

 private:
  bool RoundTrip(const std::string& line, std::string* reply, int timeout_ms = 120000);
  int fd_ = -1;
  std::string rbuf_;
  std::mutex mu_;
};

// Helpers shared with the fd-passing code.
std::string HexEncode(const std::string& raw);
std::string HexDecode(const std::string& hex);

}  // namespace switchml
#endif  // SWITCHML_RENDEZVOUS_CONTROL_H_
