// Local global-to-global copies through the TMA unit (cp.async.bulk), driven by ONE thread.
//
// The copy-in and copy-out roles of the streaming kernels move whole tiles between a user
// tensor and a staging slot. Done with ordinary loads and stores, a role of a few warps keeps
// only (threads x unroll x 16) bytes in flight, far less than the ~35 KB per SM that HBM3e
// needs to run at speed. Here one thread streams the tile through a ring of shared-memory
// buffers: bulk loads global -> shared complete on an mbarrier, bulk stores shared -> global
// run as bulk groups, kBulkStages - 1 chunks of kBulkChunk bytes are in flight at any time,
// and the rest of the role's warps cost nothing.
//
// Rules that the callers keep: both addresses 16-byte aligned and the size a multiple of 16
// bytes (BulkCopyable); every call leaves the ring idle (all groups complete), so the data is
// in place before the role signals its peers. Every wait is bounded by the %globaltimer budget
// of the job; a wait that runs out marks the CTA as failed and the call drains what it can.
// No multicast, no tensor map: plain one-dimensional bulk copies of this GPU's own memory.
#ifndef SWITCHML_BULK_COPY_CUH_
#define SWITCHML_BULK_COPY_CUH_

#include <stdint.h>

#include "kernels/device_sync.cuh"

namespace switchml {
namespace kernels {

static const int kBulkStages = 4;
static const unsigned kBulkChunk = 16384;
static const size_t kBulkRingBytes = size_t(kBulkStages) * kBulkChunk;

struct BulkRing {
  unsigned long long full[kBulkStages];  // mbarriers: a chunk has landed in its stage
  unsigned long long chunks;             // chunks moved so far (stage and phase parity follow from it)
};

__device__ __forceinline__ uint32_t BulkSmemAddr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Once per kernel, by one thread, before anybody uses the ring (followed by a CTA barrier).
__device__ __forceinline__ void BulkRingInit(BulkRing* ring) {
  for (int s = 0; s < kBulkStages; s++)
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(BulkSmemAddr(&ring->full[s])));
  ring->chunks = 0;
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ bool BulkCopyable(const void* dst, const void* src, size_t bytes) {
  return ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src) | bytes) & 15) == 0 && bytes > 0;
}

// Called by ONE thread. Copies `bytes` from `src` to `dst` (both this GPU's global memory)
// through `buffers` (kBulkRingBytes of shared memory, 128-byte aligned). Returns false when a
// wait ran out (`*failed` is set then).
__device__ __forceinline__ bool BulkCopy(BulkRing* ring, char* buffers, char* dst, const char* src, size_t bytes,
                                         unsigned long long timeout_ns, volatile int* failed) {
  const unsigned long long n = (bytes + kBulkChunk - 1) / kBulkChunk;
  const unsigned long long first = ring->chunks;
  auto size_of = [&](unsigned long long j) {
    const size_t off = j * kBulkChunk;
    return static_cast<unsigned>(bytes - off < kBulkChunk ? bytes - off : kBulkChunk);
  };
  auto load = [&](unsigned long long j) {
    const int s = static_cast<int>((first + j) % kBulkStages);
    const unsigned sz = size_of(j);
    const uint32_t bar = BulkSmemAddr(&ring->full[s]);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(sz) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(BulkSmemAddr(buffers + static_cast<size_t>(s) * kBulkChunk)), "l"(src + j * kBulkChunk), "r"(sz), "r"(bar)
                 : "memory");
  };
  // The source may have been written by other GPUs or by this CTA's other warps with ordinary
  // stores (the caller has acquired their flag): order those against the async-proxy reads.
  asm volatile("fence.proxy.async.global;" ::: "memory");
  bool ok = true;
  for (unsigned long long j = 0; j < n && j < kBulkStages - 1; j++) load(j);
  for (unsigned long long j = 0; j < n; j++) {
    const int s = static_cast<int>((first + j) % kBulkStages);
    const uint32_t parity = static_cast<uint32_t>(((first + j) / kBulkStages) & 1);
    const uint32_t bar = BulkSmemAddr(&ring->full[s]);
    const unsigned long long start = GlobalTimerNs();
    unsigned spins = 0;
    for (;;) {
      uint32_t done;
      asm volatile(
          "{\n\t.reg .pred p;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(done) : "r"(bar), "r"(parity) : "memory");
      if (done) break;
      if ((++spins & 255) == 0 && (*failed || GlobalTimerNs() - start > timeout_ns)) {
        *failed = 1;
        ok = false;
        break;
      }
    }
    if (!ok) break;
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(dst + j * kBulkChunk), "r"(BulkSmemAddr(buffers + static_cast<size_t>(s) * kBulkChunk)), "r"(size_of(j))
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    if (j + kBulkStages - 1 < n) {
      // The stage of chunk j-1 is the one the next load goes to: its store must have read it.
      asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      load(j + kBulkStages - 1);
    }
  }
  // Everything written before the caller tells anybody. (After a failed wait the loads that
  // were issued still land in shared memory; the kernel is on its way out and never reads them.)
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  ring->chunks = first + n;
  return ok;
}

}  // namespace kernels
}  // namespace switchml
#endif  // SWITCHML_BULK_COPY_CUH_
