// Weight-gradient GEMM on the 5th-generation tensor cores (sm_100a):
//
//     dW[M, N] (fp32)  =  dY[K, M]^T  x  X[K, N]          dY, X: bf16, row-major
//
// which is what a Linear layer's backward computes with K = tokens (batch x sequence),
// M = out_features, N = in_features. Both operands have their non-reduction dimension
// contiguous ("MN-major"), so they are fed to tcgen05.mma without any transpose: TMA
// brings [K_TILE x 64] boxes with the 128-byte swizzle into shared memory, which is
// exactly the canonical MN-major operand layout of the instruction.
//
// One persistent CTA per SM, 128 x 256 output tiles, statically scheduled
// (tile = blockIdx.x, += gridDim.x). Warp roles:
//   warp 0      TMA producer: fills a ring of kStages operand stages
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (M128 N256 K16, fp32
//               accumulation in TMEM), commits stage-empty and accumulator-full barriers
//   warp 2      allocates / frees the 512 TMEM columns (two accumulators: the epilogue of
//               tile t overlaps the main loop of tile t+1)
//   warps 4-7   epilogue: tcgen05.ld 32 columns at a time, stage through swizzled shared
//               memory, TMA store to global
// The fused variant additionally reduces every finished tile across GPUs (see
// wgrad_gemm.h): warps 8-11 wait until all ranks have stored tile t, let the NVSwitch add
// the ranks' copies (multimem.ld_reduce) and broadcast the sum (multimem.st), while the
// tensor cores already work on later tiles; warps whose GEMM role is over join in.
//
// Every wait is bounded: an mbarrier or flag wait that runs out of budget raises an abort
// flag in shared memory, records an error code for the host, and all roles drain, free
// TMEM and return.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstring>
#include <mutex>

#include "kernels/wgrad_gemm.h"

namespace {

constexpr int kTileM = 128;
constexpr int kTileN = 256;
constexpr int kTileK = 64;    // rows of K per pipeline stage
constexpr int kMmaK = 16;     // K of one tcgen05.mma for 16-bit operands
constexpr int kStages = 4;
constexpr int kAtomMN = 64;   // bf16 elements in one 128-byte swizzle row
constexpr int kABytes = kTileK * kTileM * 2;  // 16 KiB
constexpr int kBBytes = kTileK * kTileN * 2;  // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kEpiCols = 32;  // fp32 columns per epilogue step = one 128-byte row
constexpr int kEpiBytes = kTileM * kEpiCols * 4;  // 16 KiB
constexpr int kEpiBufs = 2;
constexpr int kTmemCols = 512;
constexpr int kThreads = 384;  // 12 warps; warps 8-11 idle unless the reduce is fused
constexpr unsigned long long kMbarBudgetNs = 2000000000ull;  // an mbarrier wait gives up after two seconds

struct __align__(1024) SharedStorage {
  uint8_t stage[kStages][kStageBytes];
  uint8_t epi[kEpiBufs][kEpiBytes];
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  volatile int abort;
};

__device__ __forceinline__ uint32_t SmemAddr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void MbarInit(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(SmemAddr(bar)), "r"(count));
}

__device__ __forceinline__ void MbarArrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(SmemAddr(bar)) : "memory");
}

__device__ __forceinline__ void MbarExpectTx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(SmemAddr(bar)), "r"(bytes)
               : "memory");
}

// Bounded wait for the phase with the given parity: the budget is time on %globaltimer, not a
// number of polls. False = gave up or aborted.
__device__ __forceinline__ bool MbarWait(uint64_t* bar, uint32_t parity, volatile int* abort) {
  uint32_t addr = SmemAddr(bar);
  unsigned long long start = 0;
  for (uint32_t i = 0;; i++) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
    if ((i & 1023) == 1023) {
      if (*abort) return false;
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (start == 0) start = now;
      else if (now - start > kMbarBudgetNs) break;
    }
  }
  *abort = 1;
  return false;
}

__device__ __forceinline__ void TmaLoad2D(void* smem_dst, const CUtensorMap* map, int x, int y,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(SmemAddr(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(SmemAddr(bar)) : "memory");
}

__device__ __forceinline__ void TmaStore2D(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(SmemAddr(smem_src)), "r"(x), "r"(y) : "memory");
}

// Shared-memory matrix descriptor for an MN-major, 128-byte-swizzled bf16 operand:
// rows of 64 elements (128 bytes), 8 rows per swizzle atom (1024 bytes = stride between
// groups of 8 K-rows), `mn_atom_stride` bytes between blocks of 64 elements along M/N.
__device__ __forceinline__ uint64_t OperandDesc(uint32_t smem_addr, uint32_t mn_atom_stride) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);            // start address
  d |= static_cast<uint64_t>((mn_atom_stride >> 4) & 0x3fff) << 16;  // leading byte offset
  d |= static_cast<uint64_t>((1024 >> 4) & 0x3fff) << 32;            // stride byte offset
  d |= 1ull << 46;                                                   // descriptor version (sm100)
  d |= 2ull << 61;                                                   // SWIZZLE_128B
  return d;
}

// kind::f16 instruction descriptor: fp32 accumulate, bf16 x bf16, both MN-major, M128 N256.
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) |
                                (static_cast<uint32_t>(kTileN >> 3) << 17) |
                                (static_cast<uint32_t>(kTileM >> 4) << 24);

__device__ __forceinline__ void Mma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(kInstrDesc), "r"(accumulate) : "memory");
}

// Arrive on an mbarrier once every tcgen05 operation issued so far by this thread is done.
__device__ __forceinline__ void MmaCommit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(SmemAddr(bar)) : "memory");
}

__device__ __forceinline__ void TmemLoad32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}

__device__ __forceinline__ void NamedBarrier(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---- cross-GPU pieces of the fused variant ------------------------------------------
__device__ __forceinline__ void StoreReleaseSys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long LoadAcquireSys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long GlobalTimerNs() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ float4 MultimemLdReduceAddF32x4(const void* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void MultimemStoreF32x4(void* mc, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               ::"l"(mc), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// Wait until flags[0..n) (one per rank) reach `value`. One lane per rank polls.
__device__ __forceinline__ bool WaitFlags(const unsigned long long* flags, int nranks,
                                          unsigned long long value, unsigned long long budget_ns,
                                          volatile int* abort) {
  bool ok = true;
  int lane = threadIdx.x & 31;
  if (lane < nranks) {
    unsigned long long start = GlobalTimerNs();
    uint32_t spins = 0;
    while (LoadAcquireSys(flags + lane) < value) {
      if ((++spins & 63) == 0 && (*abort || GlobalTimerNs() - start > budget_ns)) {
        *abort = 1;
        ok = false;
        break;
      }
      __nanosleep(32);
    }
  }
  return __all_sync(0xffffffffu, ok);
}

// Cross-GPU reduction of the tiles this rank owns (tile index mod nranks == rank), shared
// by all warps of all CTAs through one work counter: an item is `rows_per_item` rows of a tile
// (a power of two between 2 and 32, chosen by the host so that every warp of the grid gets a
// few items: a small output is then spread over all SMs instead of a handful of warps that
// each walk thousands of vectors one switch round trip at a time).
// Called by whole warps. Items are handed out in tile order, the order in which the GEMM
// produces them, so a warp rarely waits long for the flags of its item.
__device__ __forceinline__ bool ReduceWork(const WgradFusedArgs& fused, int M, int N, int tiles_n,
                                           int num_tiles, int rows_per_item, volatile int* abort) {
  const int lane = threadIdx.x & 31;
  const int owned = (num_tiles - fused.rank + fused.nranks - 1) / fused.nranks;
  const int per_tile = kTileM / rows_per_item;
  const int items = owned * per_tile;
  char* mc = fused.out_mc;
  for (;;) {
    int item = 0;
    if (lane == 0) item = atomicAdd(fused.work_counter, 1);
    item = __shfl_sync(0xffffffffu, item, 0);
    if (item >= items) return true;
    const long long tile = static_cast<long long>(item / per_tile) * fused.nranks + fused.rank;
    if (!WaitFlags(fused.flags_peer[fused.rank] + static_cast<size_t>(tile) * 8, fused.nranks, fused.epoch,
                   fused.timeout_ns, abort))
      return false;
    const int m0 = static_cast<int>(tile / tiles_n) * kTileM + (item % per_tile) * rows_per_item;
    const int n0 = static_cast<int>(tile % tiles_n) * kTileN;
    const int rows = min(rows_per_item, M - m0), cols = min(kTileN, N - n0);
    if (rows <= 0) continue;
    const int vec_per_row = cols / 4;  // N is a multiple of 8: rows are whole float4s
    const int total = rows * vec_per_row;
    for (int idx = lane; idx < total; idx += 32 * 4) {
      float4 v[4];
      size_t off[4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        int id = idx + u * 32;
        if (id < total) {
          int r = id / vec_per_row, cv = id % vec_per_row;
          off[u] = (static_cast<size_t>(m0 + r) * N + n0 + cv * 4) * 4;
          v[u] = MultimemLdReduceAddF32x4(mc + off[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; u++) {
        int id = idx + u * 32;
        if (id < total) {
          if (fused.scale != 1.0f) { v[u].x *= fused.scale; v[u].y *= fused.scale; v[u].z *= fused.scale; v[u].w *= fused.scale; }
          MultimemStoreF32x4(mc + off[u], v[u]);
        }
      }
    }
  }
}

// Gather mode: the tiles this rank owns are complete sums already; hand them to every rank.
// Same work items as ReduceWork; an item waits for this rank's own flag of the tile only.
__device__ __forceinline__ bool BroadcastWork(const WgradFusedArgs& fused, const float* dw, int M, int N, int tiles_n,
                                              int num_tiles, int rows_per_item, volatile int* abort) {
  const int lane = threadIdx.x & 31;
  const int owned = (num_tiles - fused.rank + fused.nranks - 1) / fused.nranks;
  const int per_tile = kTileM / rows_per_item;
  const int items = owned * per_tile;
  char* mc = fused.out_mc;
  const char* local = reinterpret_cast<const char*>(dw);
  for (;;) {
    int item = 0;
    if (lane == 0) item = atomicAdd(fused.work_counter, 1);
    item = __shfl_sync(0xffffffffu, item, 0);
    if (item >= items) return true;
    const long long tile = static_cast<long long>(item / per_tile) * fused.nranks + fused.rank;
    if (!WaitFlags(fused.flags_peer[fused.rank] + static_cast<size_t>(tile) * 8 + fused.rank, 1, fused.epoch,
                   fused.timeout_ns, abort))
      return false;
    const int m0 = static_cast<int>(tile / tiles_n) * kTileM + (item % per_tile) * rows_per_item;
    const int n0 = static_cast<int>(tile % tiles_n) * kTileN;
    const int rows = min(rows_per_item, M - m0), cols = min(kTileN, N - n0);
    if (rows <= 0) continue;
    const int vec_per_row = cols / 4;
    const int total = rows * vec_per_row;
    for (int idx = lane; idx < total; idx += 32 * 8) {
      float4 v[8];
      size_t off[8];
#pragma unroll
      for (int u = 0; u < 8; u++) {
        int id = idx + u * 32;
        if (id < total) {
          int r = id / vec_per_row, cv = id % vec_per_row;
          off[u] = (static_cast<size_t>(m0 + r) * N + n0 + cv * 4) * 4;
          v[u] = __ldcg(reinterpret_cast<const float4*>(local + off[u]));
        }
      }
#pragma unroll
      for (int u = 0; u < 8; u++) {
        int id = idx + u * 32;
        if (id < total) {
          if (fused.scale != 1.0f) { v[u].x *= fused.scale; v[u].y *= fused.scale; v[u].z *= fused.scale; v[u].w *= fused.scale; }
          MultimemStoreF32x4(mc + off[u], v[u]);
        }
      }
    }
  }
}

// Gather mode, first step: this rank's dY (bytes_a) and X (bytes_b) into slab `rank` of the
// gather buffer of every rank; the last CTA to finish tells the peers (flag entry `flag_entry`).
__global__ void __launch_bounds__(512) WgradGatherKernel(const char* dy, const char* x, WgradFusedArgs fused,
                                                         size_t bytes_a, size_t bytes_b, size_t flag_entry) {
  const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t nthreads = static_cast<size_t>(gridDim.x) * blockDim.x;
  char* dst_a = fused.gather_mc + static_cast<size_t>(fused.rank) * bytes_a;
  char* dst_b = fused.gather_mc + static_cast<size_t>(fused.nranks) * bytes_a + static_cast<size_t>(fused.rank) * bytes_b;
  for (size_t v = tid; v < bytes_a / 16; v += nthreads) {
    float4 w = *reinterpret_cast<const float4*>(dy + v * 16);
    MultimemStoreF32x4(dst_a + v * 16, w);
  }
  for (size_t v = tid; v < bytes_b / 16; v += nthreads) {
    float4 w = *reinterpret_cast<const float4*>(x + v * 16);
    MultimemStoreF32x4(dst_b + v * 16, w);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int arrived = atomicAdd(fused.gather_counter, 1);
    if (arrived == static_cast<int>(gridDim.x) - 1) {
      *fused.gather_counter = 0;  // for the next call
      __threadfence_system();
      for (int p = 0; p < fused.nranks; p++)
        StoreReleaseSys(fused.flags_peer[p] + flag_entry * 8 + fused.rank, fused.epoch);
    }
  }
}

// kMode 0: plain GEMM; 1: every finished tile is reduced across the ranks; 2: gather mode (owned tiles over the
// gathered operands, broadcast).
template <int kMode>
__global__ void __launch_bounds__(kThreads, 1)
WgradGemmKernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ CUtensorMap map_d, const float* dw, int M, int N, int K, WgradFusedArgs fused,
                int rows_per_item, int* error_flag) {
  constexpr bool kFused = kMode != 0;
  extern __shared__ uint8_t smem_raw[];
  SharedStorage& sh = *reinterpret_cast<SharedStorage*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (M + kTileM - 1) / kTileM;
  const int tiles_n = (N + kTileN - 1) / kTileN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = (K + kTileK - 1) / kTileK;
  // The tiles this CTA walks: all of them in turn, or (gather mode) those this rank owns.
  const int my_tiles = kMode == 2 ? (num_tiles - fused.rank + fused.nranks - 1) / fused.nranks : num_tiles;
  auto tile_of = [&](int t) { return kMode == 2 ? t * fused.nranks + fused.rank : t; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; s++) {
      MbarInit(&sh.full[s], 1);
      MbarInit(&sh.empty[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      MbarInit(&sh.acc_full[b], 1);
      MbarInit(&sh.acc_empty[b], 128);
    }
    sh.abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(SmemAddr(&sh.tmem_base)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = sh.tmem_base;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    bool operands_in = true;
    if (kMode == 2) {
      // every rank's slab of the operands must have landed in this rank's gather buffer
      operands_in = WaitFlags(fused.flags_peer[fused.rank] + static_cast<size_t>(num_tiles + 148) * 8, fused.nranks, fused.epoch,
                              fused.timeout_ns, &sh.abort);
      asm volatile("fence.proxy.async.global;" ::: "memory");
    }
    if (lane == 0 && operands_in) {
      uint32_t it = 0;
      for (int t = blockIdx.x; t < my_tiles && !sh.abort; t += gridDim.x) {
        const int tile = tile_of(t);
        const int m0 = (tile / tiles_n) * kTileM, n0 = (tile % tiles_n) * kTileN;
        for (int kb = 0; kb < k_blocks; kb++, it++) {
          const int s = it % kStages;
          const uint32_t phase = (it / kStages) & 1;
          if (!MbarWait(&sh.empty[s], phase ^ 1, &sh.abort)) break;
          MbarExpectTx(&sh.full[s], kStageBytes);
          uint8_t* a = sh.stage[s];
          uint8_t* b = sh.stage[s] + kABytes;
          // Rows beyond K, and columns beyond M / N, are filled with zeros by the TMA unit.
          for (int j = 0; j < kTileM / kAtomMN; j++)
            TmaLoad2D(a + j * (kTileK * 128), &map_a, m0 + j * kAtomMN, kb * kTileK, &sh.full[s]);
          for (int j = 0; j < kTileN / kAtomMN; j++)
            TmaLoad2D(b + j * (kTileK * 128), &map_b, n0 + j * kAtomMN, kb * kTileK, &sh.full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      uint32_t it = 0, local_tile = 0;
      for (int t = blockIdx.x; t < my_tiles && !sh.abort; t += gridDim.x, local_tile++) {
        const int acc = local_tile & 1;
        const uint32_t acc_phase = (local_tile >> 1) & 1;
        if (!MbarWait(&sh.acc_empty[acc], acc_phase ^ 1, &sh.abort)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + acc * kTileN;
        bool ok = true;
        for (int kb = 0; kb < k_blocks && ok; kb++, it++) {
          const int s = it % kStages;
          const uint32_t phase = (it / kStages) & 1;
          ok = MbarWait(&sh.full[s], phase, &sh.abort);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = SmemAddr(sh.stage[s]);
          const uint32_t b_addr = a_addr + kABytes;
#pragma unroll
          for (int kk = 0; kk < kTileK / kMmaK; kk++) {
            // 16 K-rows further = 2048 bytes further in an MN-major operand
            uint64_t da = OperandDesc(a_addr + kk * kMmaK * 128, kTileK * 128);
            uint64_t db = OperandDesc(b_addr + kk * kMmaK * 128, kTileK * 128);
            Mma(tmem_d, da, db, (kb | kk) != 0);
          }
          MmaCommit(&sh.empty[s]);  // the stage may be refilled once these MMAs have read it
        }
        if (!ok) break;
        MmaCommit(&sh.acc_full[acc]);
      }
    }
  } else if (warp >= 4 && warp < 8) {
    // ------------------------------ epilogue ------------------------------
    const int q = warp - 4;               // TMEM lane quarter this warp may read
    const int row = q * 32 + lane;        // row of the tile held by this thread
    const int epi_tid = threadIdx.x - 128;
    uint32_t local_tile = 0, stores = 0;
    for (int t = blockIdx.x; t < my_tiles; t += gridDim.x, local_tile++) {
      const int tile = tile_of(t);
      const int m0 = (tile / tiles_n) * kTileM, n0 = (tile % tiles_n) * kTileN;
      const int acc = local_tile & 1;
      const uint32_t acc_phase = (local_tile >> 1) & 1;
      if (!MbarWait(&sh.acc_full[acc], acc_phase, &sh.abort)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      for (int c = 0; c < kTileN / kEpiCols; c++, stores++) {
        const int buf = stores % kEpiBufs;
        // The buffer is free once the TMA store that used it two steps ago has read it.
        if (epi_tid == 0 && stores >= kEpiBufs) asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kEpiBufs - 1) : "memory");
        NamedBarrier(1, 128);
        uint32_t v[32];
        TmemLoad32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * kTileN + c * kEpiCols, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        // Row `row` of the staging tile: 128 bytes = 8 chunks of 16 bytes, chunk index
        // XOR-ed with (row mod 8) as the 128-byte swizzle of the store's tensor map expects.
        uint8_t* dst_row = sh.epi[buf] + row * 128;
#pragma unroll
        for (int j = 0; j < 8; j++) {
          uint4 w = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          *reinterpret_cast<uint4*>(dst_row + ((j ^ (row & 7)) << 4)) = w;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        NamedBarrier(2, 128);
        if (epi_tid == 0) {
          TmaStore2D(&map_d, sh.epi[buf], n0 + c * kEpiCols, m0);  // out-of-range parts are clipped
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
      // All TMEM reads of this accumulator are done: hand it back to the MMA warp.
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      MbarArrive(&sh.acc_empty[acc]);
      if (kFused) {
        // Publish the tile: its stores must have landed before the peers may reduce it.
        if (epi_tid == 0) {
          asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
          asm volatile("fence.proxy.async.global;" ::: "memory");
          __threadfence_system();
          if (kMode == 2) {  // only this rank's broadcasting warps wait for it
            StoreReleaseSys(fused.flags_peer[fused.rank] + static_cast<size_t>(tile) * 8 + fused.rank, fused.epoch);
          } else {
            for (int p = 0; p < fused.nranks; p++)
              StoreReleaseSys(fused.flags_peer[p] + static_cast<size_t>(tile) * 8 + fused.rank, fused.epoch);
          }
        }
      }
    }
    if (epi_tid == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  if (kFused) {
    // Every warp that has nothing (more) to do for the GEMM helps with the cross-GPU
    // reduction: warps 8-11 and 3 from the start, the others when their role is finished.
    __syncwarp();
    if (kMode == 2) BroadcastWork(fused, dw, M, N, tiles_n, num_tiles, rows_per_item, &sh.abort);
    else ReduceWork(fused, M, N, tiles_n, num_tiles, rows_per_item, &sh.abort);
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
  if (kFused && warp == 0) {
    // No CTA leaves before the matching CTA of every rank has finished reducing, so when
    // the kernel has ended everywhere every tile holds the global sum on every rank.
    unsigned long long* done = fused.flags_peer[fused.rank] + static_cast<size_t>(num_tiles + blockIdx.x) * 8;
    if (lane < fused.nranks) {
      __threadfence_system();
      StoreReleaseSys(fused.flags_peer[lane] + static_cast<size_t>(num_tiles + blockIdx.x) * 8 + fused.rank,
                      fused.epoch);
    }
    __syncwarp();
    WaitFlags(done, fused.nranks, fused.epoch, fused.timeout_ns, &sh.abort);
  }
  if (threadIdx.x == 0 && sh.abort && error_flag) *reinterpret_cast<volatile int*>(error_flag) = 1;
}

// ---- 2-CTA variant ---------------------------------------------------------------------
// Two CTAs of a cluster share one 256 x 256 tile: each loads its own 128 rows of A and its
// own 128 columns of B, the leader issues tcgen05.mma.cta_group::2 (M256 N256 K16) which
// reads B from both CTAs' shared memory, and each CTA ends up with its 128 x 256 half of
// the accumulator in its own TMEM. Per SM this halves the shared-memory traffic for B, which
// is what bounds the 1-CTA kernel on large shapes. Plain GEMM only (no fused reduce).
constexpr int k2Stages = 6;
constexpr int k2ABytes = kTileK * 128 * 2;  // 128 rows of A   : 16 KiB
constexpr int k2BBytes = kTileK * 128 * 2;  // 128 columns of B: 16 KiB
constexpr int k2StageBytes = k2ABytes + k2BBytes;
constexpr int k2Threads = 256;
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;  // clears the CTA-rank bit of a shared::cluster address

struct __align__(1024) SharedStorage2 {
  uint8_t stage[k2Stages][k2StageBytes];
  uint8_t epi[kEpiBufs][kEpiBytes];
  uint64_t full[k2Stages];
  uint64_t empty[k2Stages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  volatile int abort;
};

constexpr uint32_t kInstrDesc2 = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) |
                                 (static_cast<uint32_t>(256 >> 3) << 17) | (static_cast<uint32_t>(256 >> 4) << 24);

__device__ __forceinline__ void ClusterSync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// TMA load issued by either CTA of the pair; the bytes are counted on the leader's barrier.
__device__ __forceinline__ void TmaLoad2D_2Cta(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(SmemAddr(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(SmemAddr(bar) & kPeerBitMask) : "memory");
}

__device__ __forceinline__ void Mma2(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(kInstrDesc2), "r"(accumulate) : "memory");
}

// Arrive, in both CTAs of the pair, on the barrier at this shared-memory offset once all
// MMAs issued so far are done.
__device__ __forceinline__ void MmaCommit2(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(SmemAddr(bar)), "h"(static_cast<uint16_t>(3)) : "memory");
}

__device__ __forceinline__ void MbarArriveOnLeader(uint64_t* bar) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(remote) : "r"(SmemAddr(bar)));
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(k2Threads, 1)
WgradGemm2CtaKernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_d, int M, int N, int K, int* error_flag) {
  extern __shared__ uint8_t smem_raw[];
  SharedStorage2& sh = *reinterpret_cast<SharedStorage2*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t cta_rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(cta_rank));
  const bool leader = cta_rank == 0;
  const int tiles_m = (M + 255) / 256, tiles_n = (N + 255) / 256;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = (K + kTileK - 1) / kTileK;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < k2Stages; s++) {
      MbarInit(&sh.full[s], 1);
      MbarInit(&sh.empty[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      MbarInit(&sh.acc_full[b], 1);
      MbarInit(&sh.acc_empty[b], 256);  // the epilogue threads of both CTAs
    }
    sh.abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(SmemAddr(&sh.tmem_base)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  ClusterSync();  // both CTAs' barriers exist before anybody signals across the pair
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = sh.tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = pair; tile < num_tiles && !sh.abort; tile += num_pairs) {
        const int m0 = (tile / tiles_n) * 256 + static_cast<int>(cta_rank) * 128;
        const int n0 = (tile % tiles_n) * 256 + static_cast<int>(cta_rank) * 128;
        for (int kb = 0; kb < k_blocks; kb++, it++) {
          const int s = it % k2Stages;
          const uint32_t phase = (it / k2Stages) & 1;
          if (!MbarWait(&sh.empty[s], phase ^ 1, &sh.abort)) break;
          if (leader) MbarExpectTx(&sh.full[s], 2 * k2StageBytes);  // both CTAs' loads
          uint8_t* a = sh.stage[s];
          uint8_t* b = sh.stage[s] + k2ABytes;
          for (int j = 0; j < 2; j++) TmaLoad2D_2Cta(a + j * (kTileK * 128), &map_a, m0 + j * kAtomMN, kb * kTileK, &sh.full[s]);
          for (int j = 0; j < 2; j++) TmaLoad2D_2Cta(b + j * (kTileK * 128), &map_b, n0 + j * kAtomMN, kb * kTileK, &sh.full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      uint32_t it = 0, local_tile = 0;
      for (int tile = pair; tile < num_tiles && !sh.abort; tile += num_pairs, local_tile++) {
        const int acc = local_tile & 1;
        const uint32_t acc_phase = (local_tile >> 1) & 1;
        if (!MbarWait(&sh.acc_empty[acc], acc_phase ^ 1, &sh.abort)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + acc * kTileN;
        bool ok = true;
        for (int kb = 0; kb < k_blocks && ok; kb++, it++) {
          const int s = it % k2Stages;
          const uint32_t phase = (it / k2Stages) & 1;
          ok = MbarWait(&sh.full[s], phase, &sh.abort);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = SmemAddr(sh.stage[s]);
          const uint32_t b_addr = a_addr + k2ABytes;
#pragma unroll
          for (int kk = 0; kk < kTileK / kMmaK; kk++) {
            uint64_t da = OperandDesc(a_addr + kk * kMmaK * 128, kTileK * 128);
            uint64_t db = OperandDesc(b_addr + kk * kMmaK * 128, kTileK * 128);
            Mma2(tmem_d, da, db, (kb | kk) != 0);
          }
          MmaCommit2(&sh.empty[s]);
        }
        if (!ok) break;
        MmaCommit2(&sh.acc_full[acc]);
      }
    }
  } else if (warp >= 4) {
    const int q = warp - 4;
    const int row = q * 32 + lane;
    const int epi_tid = threadIdx.x - 128;
    uint32_t local_tile = 0, stores = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs, local_tile++) {
      const int m0 = (tile / tiles_n) * 256 + static_cast<int>(cta_rank) * 128;
      const int n0 = (tile % tiles_n) * 256;
      const int acc = local_tile & 1;
      const uint32_t acc_phase = (local_tile >> 1) & 1;
      if (!MbarWait(&sh.acc_full[acc], acc_phase, &sh.abort)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      for (int c = 0; c < kTileN / kEpiCols; c++, stores++) {
        const int buf = stores % kEpiBufs;
        if (epi_tid == 0 && stores >= kEpiBufs) asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kEpiBufs - 1) : "memory");
        NamedBarrier(1, 128);
        uint32_t v[32];
        TmemLoad32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * kTileN + c * kEpiCols, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        uint8_t* dst_row = sh.epi[buf] + row * 128;
#pragma unroll
        for (int j = 0; j < 8; j++) {
          uint4 w = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          *reinterpret_cast<uint4*>(dst_row + ((j ^ (row & 7)) << 4)) = w;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        NamedBarrier(2, 128);
        if (epi_tid == 0) {
          TmaStore2D(&map_d, sh.epi[buf], n0 + c * kEpiCols, m0);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      if (leader) MbarArrive(&sh.acc_empty[acc]);
      else MbarArriveOnLeader(&sh.acc_empty[acc]);
    }
    if (epi_tid == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  ClusterSync();  // the peer may still be signalling into this CTA's shared memory
  if (warp == 2) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
  if (threadIdx.x == 0 && sh.abort && error_flag) *reinterpret_cast<volatile int*>(error_flag) = 1;
}

// ---- host side ------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn GetEncodeTiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 2-D row-major tensor [rows, cols]; box [box_rows, box_cols]; 128-byte swizzle.
bool MakeMap(CUtensorMap* map, CUtensorMapDataType type, int esz, const void* base, int rows, int cols,
             int box_rows, int box_cols) {
  EncodeTiledFn enc = GetEncodeTiled();
  if (!enc) return false;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * esz};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  return enc(map, type, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int g_sm_count[64] = {0};

}  // namespace

extern "C" int switchml_wgrad_gemm(const void* dy, const void* x, float* dw, int M, int N, int K,
                                   const WgradFusedArgs* fused, int* error_flag, void* stream_ptr) {
  if (!dy || !x || !dw || M <= 0 || N <= 0 || K <= 0) return -1;
  // TMA needs 16-byte aligned bases and row pitches that are multiples of 16 bytes.
  if ((M % 8) || (N % 8)) return -2;
  if ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dw)) & 15)
    return -2;
  const bool gather = fused && fused->nranks > 1 && fused->mode == 1;
  if (gather && (!fused->gather_local || !fused->gather_mc || !fused->gather_counter || !fused->out_mc || !fused->work_counter ||
                 fused->nranks > 8))
    return -1;
  // Gather mode multiplies the gathered operands: nranks * K rows, read from this rank's gather buffer.
  const int k_rows = gather ? fused->nranks * K : K;
  const void* a_base = gather ? static_cast<const void*>(fused->gather_local) : dy;
  const void* b_base = gather ? static_cast<const void*>(fused->gather_local + static_cast<size_t>(k_rows) * M * 2) : x;
  CUtensorMap map_a, map_b, map_d;
  if (!MakeMap(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a_base, k_rows, M, kTileK, kAtomMN) ||
      !MakeMap(&map_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, b_base, k_rows, N, kTileK, kAtomMN) ||
      !MakeMap(&map_d, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, dw, M, N, kTileM, kEpiCols))
    return -3;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && g_sm_count[dev] == 0)
    cudaDeviceGetAttribute(&g_sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
  int sms = (dev >= 0 && dev < 64 && g_sm_count[dev] > 0) ? g_sm_count[dev] : 148;
  if (sms > 148) sms = 148;  // the flag array has room for 148 closing flags
  int tiles = ((M + kTileM - 1) / kTileM) * ((N + kTileN - 1) / kTileN);
  int grid = tiles < sms ? tiles : sms;
  size_t smem = sizeof(SharedStorage) + 1024;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  WgradFusedArgs none;
  memset(&none, 0, sizeof(none));
  cudaError_t e;
  if (fused && fused->nranks > 1) {
    if (fused->nranks > 8 || !fused->out_mc || !fused->work_counter) return -1;
    // All CTAs take part in the closing cross-GPU barrier, so the grid must be the same on
    // every rank and fully resident: one CTA per SM at most.
    static bool attr_f = false;
    if (!attr_f) {
      cudaFuncSetAttribute(WgradGemmKernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      cudaFuncSetAttribute(WgradGemmKernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      attr_f = true;
    }
    // One CTA on every SM even when there are fewer tiles: the others only reduce (or broadcast).
    // Work items of that: a few per warp of the grid, between 2 and 32 rows of a tile each.
    grid = sms;
    const long long owned_rows = static_cast<long long>((tiles + fused->nranks - 1) / fused->nranks) * kTileM;
    const long long warps = static_cast<long long>(grid) * (kThreads / 32);
    int rows_per_item = 32;
    while (rows_per_item > 2 && owned_rows / rows_per_item < 2 * warps) rows_per_item >>= 1;
    if (gather) {
      const size_t bytes_a = static_cast<size_t>(K) * M * 2, bytes_b = static_cast<size_t>(K) * N * 2;
      size_t vecs = (bytes_a + bytes_b) / 16;
      int gblocks = static_cast<int>((vecs + 511) / 512);
      if (gblocks > sms) gblocks = sms;
      if (gblocks < 1) gblocks = 1;
      WgradGatherKernel<<<gblocks, 512, 0, stream>>>(static_cast<const char*>(dy), static_cast<const char*>(x), *fused,
                                                    bytes_a, bytes_b, static_cast<size_t>(tiles) + 148);
      if (cudaGetLastError() != cudaSuccess) return -4;
      WgradGemmKernel<2><<<grid, kThreads, smem, stream>>>(map_a, map_b, map_d, dw, M, N, k_rows, *fused, rows_per_item, error_flag);
    } else {
      WgradGemmKernel<1><<<grid, kThreads, smem, stream>>>(map_a, map_b, map_d, dw, M, N, K, *fused, rows_per_item, error_flag);
    }
    e = cudaGetLastError();
  } else {
    static bool attr_p = false;
    if (!attr_p) {
      cudaFuncSetAttribute(WgradGemmKernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      attr_p = true;
    }
    WgradGemmKernel<0><<<grid, kThreads, smem, stream>>>(map_a, map_b, map_d, dw, M, N, K, none, 32, error_flag);
    e = cudaGetLastError();
  }
  return e == cudaSuccess ? 0 : -4;
}

extern "C" int switchml_wgrad_gemm_2cta(const void* dy, const void* x, float* dw, int M, int N, int K,
                                        int* error_flag, void* stream_ptr) {
  if (!dy || !x || !dw || M <= 0 || N <= 0 || K <= 0) return -1;
  if ((M % 8) || (N % 8)) return -2;
  if ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dw)) & 15)
    return -2;
  CUtensorMap map_a, map_b, map_d;
  if (!MakeMap(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, dy, K, M, kTileK, kAtomMN) ||
      !MakeMap(&map_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, K, N, kTileK, kAtomMN) ||
      !MakeMap(&map_d, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, dw, M, N, kTileM, kEpiCols))
    return -3;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && g_sm_count[dev] == 0)
    cudaDeviceGetAttribute(&g_sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
  int sms = (dev >= 0 && dev < 64 && g_sm_count[dev] > 0) ? g_sm_count[dev] : 148;
  int tiles = ((M + 255) / 256) * ((N + 255) / 256);
  int pairs = tiles < sms / 2 ? tiles : sms / 2;
  size_t smem = sizeof(SharedStorage2) + 1024;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(WgradGemm2CtaKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    attr = true;
  }
  WgradGemm2CtaKernel<<<pairs * 2, k2Threads, smem, static_cast<cudaStream_t>(stream_ptr)>>>(
      map_a, map_b, map_d, M, N, K, error_flag);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int switchml_wgrad_flag_words(int M, int N) {
  int tiles = ((M + kTileM - 1) / kTileM) * ((N + kTileN - 1) / kTileN);
  return (tiles + 148 + 8) * 8;
}
