// WarpStream: a warp reads a run of global memory through its own ring of shared-memory
// chunks that the TMA unit fills (cp.async.bulk, one-dimensional, this GPU's memory only).
//
// The quantising loader of the streaming kernels has to look at every input element twice
// (block maxima, then quantisation) and do arithmetic on it, so it cannot hand the copy to
// the TMA unit wholesale like the plain copy roles (bulk_copy.cuh). Instead every loader
// warp prefetches: lane 0 keeps up to kWsStages chunks of kWsChunk bytes in flight into the
// warp's private ring, the warp waits on the chunk's mbarrier, works on it out of shared
// memory (conflict-free 16-byte reads) and passes the stage on. Six warps keep 96 KB in
// flight per SM where register-held loads managed 24 KB, and no warp ever waits for another.
//
// Waits are bounded by the job's %globaltimer budget; a wait that runs out marks the CTA as
// failed, and the stream drains the loads it still has in flight before it gives up.
#ifndef SWITCHML_WARP_STREAM_CUH_
#define SWITCHML_WARP_STREAM_CUH_

#include <stdint.h>

#include "kernels/bulk_copy.cuh"
#include "kernels/device_sync.cuh"

namespace switchml {
namespace kernels {

static const int kWsStages = 4;
static const unsigned kWsChunk = 4096;          // bytes: 1024 float32 = 8 rows of 128 elements
static const int kWsMaxWarps = 8;               // loader warps that may own a stream
static const size_t kWsRingBytes = size_t(kWsStages) * kWsChunk;  // per warp

struct WarpStreamBarriers {
  unsigned long long full[kWsMaxWarps][kWsStages];
};

// Once per kernel, by one thread, before anybody streams (followed by a CTA barrier).
__device__ __forceinline__ void WarpStreamInit(WarpStreamBarriers* b) {
  for (int w = 0; w < kWsMaxWarps; w++)
    for (int s = 0; s < kWsStages; s++)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(BulkSmemAddr(&b->full[w][s])));
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// State of one warp's stream; every lane holds the same values.
struct WarpStream {
  char* ring;                  // this warp's kWsRingBytes of shared memory
  unsigned long long* full;    // its kWsStages mbarriers
  unsigned long long used;     // chunks consumed so far, over the whole kernel: stage and parity follow from it
  unsigned long long timeout_ns;
  volatile int* failed;

  // Lane 0: start the load of `bytes` (a multiple of 16) at `src` (16-byte aligned) into the
  // stage that chunk number `seq` (counted like `used`) will be consumed from.
  __device__ __forceinline__ void Issue(unsigned long long seq, const char* src, unsigned bytes) const {
    const int s = static_cast<int>(seq % kWsStages);
    const uint32_t bar = BulkSmemAddr(&full[s]);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(BulkSmemAddr(ring + static_cast<size_t>(s) * kWsChunk)), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
  }

  // All lanes: wait for the chunk that is consumed next. Returns its shared-memory address,
  // or nullptr when the wait ran out (the same answer in every lane).
  __device__ __forceinline__ const char* Acquire() const {
    const int s = static_cast<int>(used % kWsStages);
    const uint32_t parity = static_cast<uint32_t>((used / kWsStages) & 1);
    const uint32_t bar = BulkSmemAddr(&full[s]);
    const unsigned long long start = GlobalTimerNs();
    unsigned spins = 0;
    bool ok = true;
    for (;;) {
      uint32_t done;
      asm volatile(
          "{\n\t.reg .pred p;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(done) : "r"(bar), "r"(parity) : "memory");
      if (done) break;
      if ((++spins & 255) == 0 && (*failed || GlobalTimerNs() - start > timeout_ns)) {
        ok = false;
        break;
      }
    }
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) {
      *failed = 1;
      return nullptr;
    }
    return ring + static_cast<size_t>(s) * kWsChunk;
  }

  // All lanes, after the last read of the acquired chunk.
  __device__ __forceinline__ void Release() {
    __syncwarp();
    ++used;
  }
};

// Runs `body(chunk_index, smem)` for the chunks w, w + W, w + 2W, ... < nchunks of a run of
// whole chunks starting at `src` (16-byte aligned), W = number of streaming warps, w = this
// warp's index among them. `source_of(chunk)` gives the global address of a chunk, so that
// a run may skip parts of the tile. Returns false if a wait ran out.
template <typename SourceOf, typename Body>
__device__ __forceinline__ bool WarpStreamRun(WarpStream& ws, int w, int W, int lane, size_t nchunks,
                                              SourceOf source_of, Body body) {
  const size_t mine = nchunks > static_cast<size_t>(w) ? (nchunks - w + W - 1) / W : 0;
  // Inputs may have been written by this stream's producers with ordinary stores.
  if (lane == 0) {
    asm volatile("fence.proxy.async.global;" ::: "memory");
    for (size_t i = 0; i < mine && i < kWsStages; i++) ws.Issue(ws.used + i, source_of(w + i * W), kWsChunk);
  }
  size_t issued = mine < kWsStages ? mine : kWsStages;
  for (size_t i = 0; i < mine; i++) {
    const char* smem = ws.Acquire();
    if (smem == nullptr) {
      // Drain what is still in flight (bounded), so that nothing lands in this shared
      // memory after the CTA has gone.
      for (size_t j = i + 1; j < issued; j++) {
        ++ws.used;
        const int s = static_cast<int>(ws.used % kWsStages);
        const uint32_t parity = static_cast<uint32_t>((ws.used / kWsStages) & 1);
        const uint32_t bar = BulkSmemAddr(&ws.full[s]);
        for (int spins = 0; spins < (1 << 16); spins++) {
          uint32_t done;
          asm volatile(
              "{\n\t.reg .pred p;\n\t"
              "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
              "selp.u32 %0, 1, 0, p;\n\t}"
              : "=r"(done) : "r"(bar), "r"(parity) : "memory");
          if (done) break;
        }
      }
      return false;
    }
    body(w + i * W, smem);
    ws.Release();
    if (i + kWsStages < mine) {
      // the stage just released is the one that chunk i + kWsStages will be consumed from
      if (lane == 0) ws.Issue(ws.used + kWsStages - 1, source_of(w + (i + kWsStages) * W), kWsChunk);
      ++issued;
    }
  }
  return true;
}

}  // namespace kernels
}  // namespace switchml
#endif  // SWITCHML_WARP_STREAM_CUH_
