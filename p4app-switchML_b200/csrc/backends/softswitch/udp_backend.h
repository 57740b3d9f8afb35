// UdpBackend: worker threads that stream packets to the software aggregation switch
// over UDP sockets, with per-slot retransmission timers.
//
// It takes the place of the reference's DPDK backend (backends/dpdk/dpdk_backend.cc:49-140
// session setup through the controller; dpdk_worker_thread.cc:199-402 hot loop; timers
// and back-off dpdk_worker_thread_utils.inc:225-265) with kernel sockets instead of a
// poll-mode driver: one socket per worker thread (the reference steers one NIC queue per
// thread by UDP port), slot addressing with a set bit that flips on every use, stale and
// duplicate results discarded by job tag and packet id, retransmission of the same slot
// and set after `timeout` ms. Rank 0 can host the switch and the controller in-process.
#ifndef SWITCHML_UDP_BACKEND_H_
#define SWITCHML_UDP_BACKEND_H_

#include <memory>
#include <thread>
#include <vector>

#include "rendezvous/control.h"
#include "switchml/backend.h"

namespace switchml {

// Sends echo requests from the connected socket `fd` until the software switch sends one
// back or `timeout_ms` passes. True if the data plane answered.
bool EchoSwitch(int fd, uint16_t worker, uint8_t thread, uint64_t session, int timeout_ms);

class UdpBackend : public Backend {
 public:
  UdpBackend(Context& context, Config& config);
  ~UdpBackend() override;
  void SetupWorker() override;
  void CleanupWorker() override;
  ControlServer* server() { return server_.get(); }

 private:
  void WorkerLoop(WorkerTid tid, int fd);
  std::unique_ptr<ControlServer> server_;
  ControlClient client_;
  std::vector<std::thread> threads_;
  std::vector<int> fds_;
  uint64_t session_id_ = 0;
  std::vector<uint16_t> switch_udp_ports_;  // one per pipe of the switch; thread t uses [t % size]
};

}  // namespace switchml
#endif  // SWITCHML_UDP_BACKEND_H_
