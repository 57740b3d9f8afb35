// Small host-side helpers.
// Parity: reference client_lib/src/utils.h:38-101 (reusable thread Barrier with
// Destroy(), Execute(cmd) popen helper).
#ifndef SWITCHML_UTILS_H_
#define SWITCHML_UTILS_H_

#include <condition_variable>
#include <mutex>
#include <string>

namespace switchml {

// Reusable barrier for a fixed number of threads. Destroy() releases every waiter and
// makes all later Wait() calls return immediately (used to unblock workers at Stop()).
class Barrier {
 public:
  explicit Barrier(int num_participants);
  Barrier(const Barrier&) = delete;
  void operator=(const Barrier&) = delete;
  // Returns true for a normal release, false if the barrier was destroyed.
  bool Wait();
  void Destroy();

 private:
  const int num_participants_;
  int waiting_ = 0;
  unsigned long generation_ = 0;
  bool destroyed_ = false;
  std::mutex mu_;
  std::condition_variable cv_;
};

// Run a shell command and return its standard output.
std::string Execute(const char* cmd);

// Parse "a-b,c" style core lists ("0-3", "0,2,4-6") into ids; empty on syntax error.
bool ParseCoreList(const std::string& spec, std::string* error, int* out, int max_out, int* count);

// Pin the calling thread to one CPU core; false if the kernel refuses.
// (The reference pins its RDMA worker threads to cores on the NIC's NUMA node,
// backends/rdma/rdma_utils.h:135-204.)
bool BindToCore(int core);
// NUMA node of a PCI device given its sysfs bus id ("0000:1b:00.0"), -1 if unknown.
int GetDeviceNuma(const std::string& pci_bus_id);
// The CPU cores of a NUMA node (sysfs cpulist; the reference parses `lscpu` for the same,
// rdma_utils.h:135-170). False if the node is unknown.
bool GetCoresNuma(int node, int* out, int max_out, int* count);
// Restrict the calling thread to the cores of `node`; false if unknown or refused.
bool BindToNumaNode(int node);

}  // namespace switchml
#endif  // SWITCHML_UTILS_H_
