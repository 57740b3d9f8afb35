// Cross-GPU synchronisation primitives for kernels that meet inside symmetric memory.
//
// Every rank owns a pad of 64-bit flags: flags[channel][phase][source rank]. To signal,
// a rank writes the current epoch into its own column of every peer's pad with a
// system-scope release store; to wait, it polls its local pad until every column has
// reached the epoch. Epochs only grow (the host hands every job a fresh range), so
// flags are never reset and a flag left behind by a failed job can never satisfy a
// later wait. These flags do the work of the per-slot worker bitmaps and counters of the
// reference switch (p4/bitmap_checker.p4:82-154, p4/workers_counter.p4:25-111).
//
// Waits are bounded: when the budget (ns on %globaltimer) runs out the waiter records
// STATUS_TIMEOUT with channel and phase in the status word and the kernel returns
// normally — the analogue of the reference's per-packet timers
// (dpdk_worker_thread_utils.inc:225-265), except that on a lossless fabric a timeout
// means a missing peer, so the job fails instead of retransmitting.
#ifndef SWITCHML_DEVICE_SYNC_CUH_
#define SWITCHML_DEVICE_SYNC_CUH_

#include "kernels/allreduce_kernels.h"

namespace switchml {
namespace kernels {

__device__ __forceinline__ unsigned long long GlobalTimerNs() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

typedef unsigned long long Epoch;

__device__ __forceinline__ void StoreReleaseSys(Epoch* p, Epoch v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ Epoch LoadAcquireSys(const Epoch* p) {
  Epoch v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ Epoch* FlagPtr(char* region, int channel, int phase, int src) {
  return reinterpret_cast<Epoch*>(region) +
         (static_cast<size_t>(channel) * kNumPhases + phase) * kMaxRanks + src;
}

// The status word may live in host memory mapped into the device (no atomics there): a
// plain store; when several waits fail at once any of their codes will do.
__device__ __forceinline__ void ReportStatus(const RankCtx& ctx, int code) {
  *reinterpret_cast<volatile int*>(ctx.status) = code;
  __threadfence_system();
}

// Barrier over all ranks for one channel. Must be called by every thread of the CTA.
// Returns false when the wait timed out (the whole CTA gets the same answer). With
// `signal` false the caller only waits (used to exercise the timeout path).
__device__ __forceinline__ bool ChannelBarrier(const RankCtx& ctx, int channel, int phase,
                                               Epoch epoch, int* s_failed, bool signal = true) {
  __syncthreads();  // everything this CTA wrote precedes the signal
  if (threadIdx.x < ctx.nranks) {
    int peer = threadIdx.x;
    if (ctx.sc_fence) __threadfence_system();
    if (signal) StoreReleaseSys(FlagPtr(ctx.stage_peer[peer], channel, phase, ctx.rank), epoch);
    const Epoch* mine = FlagPtr(ctx.stage_peer[ctx.rank], channel, phase, peer);
    unsigned long long start = GlobalTimerNs();
    unsigned long long spins = 0;
    while (LoadAcquireSys(mine) < epoch) {
      ++spins;
      if ((spins & 63) == 0 && GlobalTimerNs() - start > ctx.timeout_ns) {
        ReportStatus(ctx, STATUS_TIMEOUT | (phase << 4) | (channel << 8));
        atomicAdd(ctx.counters + 2, 1ull);
        *s_failed = 1;
        break;
      }
      __nanosleep(20);
    }
    if (spins) atomicAdd(ctx.counters + 1, spins);
  }
  __syncthreads();
  return *s_failed == 0;
}

}  // namespace kernels
}  // namespace switchml
#endif  // SWITCHML_DEVICE_SYNC_CUH_
