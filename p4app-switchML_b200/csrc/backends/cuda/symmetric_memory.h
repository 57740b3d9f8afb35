// SymmetricRegion: device memory that every rank of the job can address.
//
// Each rank allocates the same number of bytes with the virtual memory API, exports the
// allocation as a file descriptor, imports everybody else's and maps all of them, so a
// kernel can load/store any peer's copy over NVLink. When the machine supports NVLink
// SHARP, the allocations are also bound to one multicast object whose mapping gives the
// `multimem.*` instructions their address: a load-reduce through it returns the
// element-wise reduction of all ranks' copies computed in the NVSwitch, a store through
// it lands in all copies.
//
// In SwitchML terms this is the slot memory of the switch plus the session that the
// controller sets up (reference controller/grpc_server.py:198-353 hands out addresses
// and keys of the switch; backends/rdma/rdma_connection.cc:66-131 registers one buffer
// at the same address on every node).
#ifndef SWITCHML_CUDA_SYMMETRIC_MEMORY_H_
#define SWITCHML_CUDA_SYMMETRIC_MEMORY_H_

#include <cuda.h>

#include <cstdint>
#include <string>
#include <vector>

#include "backends/cuda/fd_channel.h"
#include "rendezvous/control.h"

namespace switchml {

struct SymmetricRegion {
  size_t bytes = 0;                 // usable size (same on all ranks)
  size_t mapped_bytes = 0;          // rounded to the allocation granularity
  void* local = nullptr;            // this rank's copy
  std::vector<void*> peers;         // [rank] -> mapping of that rank's copy (peers[me] == local)
  void* multicast = nullptr;        // multimem address, nullptr without NVLS
  // driver handles
  CUmemGenericAllocationHandle handle = 0;
  std::vector<CUmemGenericAllocationHandle> peer_handles;
  CUmemGenericAllocationHandle mc_handle = 0;
  bool mc_bound = false;
};

class SymmetricAllocator {
 public:
  SymmetricAllocator(int rank, int num_workers, int device, ControlClient* control,
                     FdChannel* fds);
  // True when this device reports multicast support.
  bool DeviceSupportsMulticast() const;
  // Collective: every rank calls it with the same arguments, in the same order.
  // `want_multicast` is honoured only if every rank can do it; on any rank's failure all
  // ranks fall back to peer mappings only. Returns false when even that fails.
  bool Create(size_t bytes, bool want_multicast, SymmetricRegion* out, std::string* error);
  // Collective teardown. Unbinds the multicast object on every rank before any rank frees
  // its memory. `peers_alive` = false skips the barriers (a peer is gone).
  void Destroy(SymmetricRegion* r, bool peers_alive);

 private:
  int rank_, n_, device_;
  ControlClient* control_;
  FdChannel* fds_;
  int next_tag_ = 1;
};

}  // namespace switchml
#endif  // SWITCHML_CUDA_SYMMETRIC_MEMORY_H_
