// CudaBackend: the B200 backend. The NVSwitch fabric does what the Tofino does for the
// reference: it adds the workers' tiles (multimem.ld_reduce) and multicasts the result
// (multimem.st); where NVLink SHARP is missing, the same kernels read and write the
// peers' staging memory directly.
//
// It replaces, at once, the reference's NIC backends (backends/dpdk, backends/rdma), the
// switch program (p4/) and the controller session setup (controller/grpc_server.py):
//  * SetupWorker(): choose the device, start/reach the in-process controller, allocate
//    the symmetric staging region (flags, exponent slots, one-shot buffers, data slots)
//    and, if asked, a symmetric heap for zero-copy tensors; start the launcher and the
//    completion threads.
//  * launch = worker: a launcher thread pulls jobs from the FIFO scheduler and enqueues
//    their kernels on an internal high-priority stream, ordered after the producer
//    stream by an event. launch = inline: the submitting thread enqueues the kernels on
//    the caller's own stream (stream-ordered like any other kernel).
//  * A completion thread waits for each job's event, reads the kernel's status word and
//    finishes or fails the job.
#ifndef SWITCHML_CUDA_BACKEND_H_
#define SWITCHML_CUDA_BACKEND_H_

#include <cstddef>
#include <string>

#include "switchml/backend.h"

namespace switchml {

class CudaBackendInterface : public Backend {
 public:
  using Backend::Backend;
  // Allocate from the symmetric heap ([backend.cuda] symm_heap_mb). Collective in the
  // sense that every rank must perform the same sequence of allocations. nullptr when the
  // heap is exhausted or absent. Alignment is 256 bytes.
  virtual void* SymmetricAlloc(size_t bytes) = 0;
  // Release everything allocated from the heap (again on every rank alike).
  virtual void SymmetricReset() = 0;
  virtual bool UsesMultimem() const = 0;
  // Mappings of the symmetric heap: this rank's base, every rank's base as mapped here
  // (`peers` has room for 8 entries), the multicast base (nullptr without NVLS), its size.
  virtual bool SymmetricHeapInfo(void** local, void** peers, void** multicast, size_t* bytes) = 0;
  virtual int Device() const = 0;
  // Enqueue a kernel that waits for a signal nobody sends and report how the wait ended
  // (kernels::Status). Used to check that bounded waits give up cleanly.
  virtual int RunWaitProbe(double budget_ms) = 0;
};

// Factory used by Backend::CreateInstance. Throws FatalError when no usable GPU exists.
Backend* CreateCudaBackend(Context& context, Config& config);

// Stand-alone multi-rank emulation on one GPU (no Context needed): `nranks` virtual
// ranks, all memory on the current device, one cooperative kernel. in/out are arrays of
// `nranks` device pointers. `exponent_lookahead` < 0 takes the default. Returns 0 or a negative error / positive kernels::Status.
int EmulatedAllReduce(int nranks, void* const* in_ptrs, void* const* out_ptrs,
                      unsigned long long numel, int elem_type, int mode, int algo, int block_numel,
                      size_t slot_bytes, int slots_per_channel, int channels, float post_scale,
                      int repeats, int exponent_lookahead, std::string* error);

// True if the kernels were compiled with -DSWITCHML_CHECKED (geometry checks before every
// tile; a violation sets STATUS_BOUNDS instead of touching memory).
bool KernelsCheckedBuild();

// The uint8 <-> int32 conversion kernels on their own (no Context needed), enqueued on
// `stream` (a cudaStream_t, nullptr = default stream) of the current device. `widen`
// zero-extends `numel` bytes into int32, otherwise the low byte of each int32 is kept.
// Returns 0 or the CUDA error code.
int ConvertU8OnDevice(bool widen, const void* in, void* out, unsigned long long numel, void* stream,
                      std::string* error);

}  // namespace switchml
#endif  // SWITCHML_CUDA_BACKEND_H_
