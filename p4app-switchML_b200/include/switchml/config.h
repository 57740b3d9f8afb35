// switchml.cfg: the INI configuration of a worker.
//
// Parity: reference client_lib/src/config.h:38-307 and config.cc:42-283 — same file
// grammar ([section], key = value, '#' comments), same key names and defaults for
// [general] and [backend.dummy], same search order (/etc/switchml.cfg, ./switchml.cfg,
// ./switchml-<hostname>.cfg), same Validate() rounding rules, same PrintConfig() dump.
// The parser is self-contained (the reference uses boost::program_options).
//
// The reference's NIC sections [backend.dpdk] / [backend.rdma] are accepted and ignored
// with a warning, so an existing file keeps loading; their role is taken by
//   [backend.udp]   software aggregation switch over UDP sockets (CPU, loss-tolerant)
//   [backend.cuda]  NVSwitch/NVLink aggregation on B200 (NVLS multimem or peer memory)
#ifndef SWITCHML_CONFIG_H_
#define SWITCHML_CONFIG_H_

#include <cstdint>
#include <map>
#include <string>

#include "switchml/common.h"

namespace switchml {

struct GeneralConfig {
  uint16_t rank = 0;                       // unique id in [0, num_workers)
  uint16_t num_workers = 1;                // at most 32 (aggregator bitmap width)
  uint16_t num_worker_threads = 4;         // CPU backends: threads; cuda: slices ("channels") per job
  uint32_t max_outstanding_packets = 256;  // slot window per worker, split over worker threads
  uint64_t packet_numel = 1024;            // elements per packet = quantisation block length
  std::string backend = "dummy";           // dummy | udp | cuda
  std::string scheduler = "fifo";
  std::string prepostprocessor = "cpu_exponent_quantizer";  // or bypass
  bool instant_job_completion = false;     // debug: finish every job without doing work
  std::string controller_ip_str = "127.0.0.1";  // rendezvous / software-switch control address
  uint16_t controller_port = 50099;
  double timeout = 10.0;                   // ms before a slot is retransmitted / a device wait gives up
  uint64_t timeout_threshold = 100;        // after this many timeouts double `timeout` ...
  uint64_t timeout_threshold_increment = 100;  // ... and raise the threshold by this much
};

struct DummyBackendConfig {
  float bandwidth = 1000.0f;    // Mbps modelled by sleeping; 0 = no sleep
  bool process_packets = true;  // multiply payloads by num_workers to fake an N-way sum
};

struct UdpBackendConfig {
  std::string switch_ip_str = "127.0.0.1";  // where the software aggregation switch listens
  uint16_t switch_port = 48864;             // 0xBEE0, the SwitchML UDP port
  std::string worker_ip_str = "127.0.0.1";
  uint16_t worker_port = 4000;              // thread t binds worker_port + t (0 = ephemeral)
  bool spawn_switch = true;                 // rank 0 hosts the switch in-process
  uint32_t pool_size = 8192;                // switch slots per worker thread (x2 sets)
  uint32_t switch_pipes = 0;                // data-plane threads of the in-process switch on ports switch_port, +1, ...;
                                            // 0 = one per worker thread, at most 8
  std::string cores = "";                   // e.g. "0-3" or "0,2,4,6": pin worker thread t to the t-th core
  uint32_t msg_numel = 0;                   // elements of a message: several packets that share one slot of the
                                            // window, one timer and ONE exponent (carried by the message's last
                                            // packet); 0 = one packet per message (= packet_numel)
};

struct CudaBackendConfig {
  int device = -1;                        // -1: LOCAL_RANK env or rank % visible devices
  std::string transport = "auto";         // auto | nvls | p2p
  std::string mode = "int32_quant";       // int32_quant | float_sum  (FLOAT32/BFLOAT16 jobs)
  uint32_t channels = 0;                  // CTAs per kernel; 0 = pick from message size
  uint64_t slot_bytes = 524288;           // staging bytes per slot per channel
  uint32_t slots_per_channel = 4;         // ring depth (the switch keeps 2 sets per slot; here the loader may run further ahead)
  uint64_t oneshot_max_bytes = 4194304;   // messages up to this size take the one-barrier kernel
  uint64_t symm_heap_mb = 0;              // user symmetric heap for zero-copy tensors
  bool average = false;                   // fold 1/num_workers into the result
  std::string launch = "worker";          // worker: launcher thread pulls the FIFO; inline: caller launches
  std::string rendezvous_dir = "";        // directory for unix sockets (default: abstract namespace)
  double wait_timeout_ms = 10000.0;       // budget of every device-side wait for a peer
  bool numa_bind = false;                 // keep the launcher and completion threads on the GPU's NUMA node
  std::string p2p_algo = "push";          // peer-memory transport, large messages: push (posted stores only) | staged
  uint32_t exponent_lookahead = 0;        // int32_quant: tiles by which the block exponents run ahead of their data (0..ring/2)
  std::string signal_fence = "release";   // sc: fence.sc.sys before every flag store | release: the flag's st.release.sys alone
  bool trace = false;                     // channel 0 timestamps every tile of its roles; GetStats shows the last job's timeline
};

class Config {
 public:
  Config() = default;

  // Search /etc/switchml.cfg, ./switchml.cfg, ./switchml-<hostname>.cfg (first hit wins)
  // unless `path` is given. $SWITCHML_CONFIG overrides the search. Returns false when no
  // file was found or it does not parse.
  bool LoadFromFile(std::string path = "");
  // Parse INI text directly (bindings and tests).
  bool LoadFromString(const std::string& text, const std::string& origin = "<string>");
  // Apply SWITCHML_RANK / SWITCHML_NUM_WORKERS / SWITCHML_BACKEND environment overrides.
  void ApplyEnvOverrides();
  // Check ranges and round dependent values; throws FatalError on an unusable config.
  void Validate();
  // Dump every option and the derived values at INFO level.
  void PrintConfig() const;
  std::string ToString() const;

  GeneralConfig general_;
  struct {
    DummyBackendConfig dummy;
    UdpBackendConfig udp;
    CudaBackendConfig cuda;
  } backend_;

  // Keys seen in [backend.dpdk] / [backend.rdma]; kept only for PrintConfig.
  std::map<std::string, std::string> ignored_;
  std::string loaded_from_;
};

}  // namespace switchml
#endif  // SWITCHML_CONFIG_H_
