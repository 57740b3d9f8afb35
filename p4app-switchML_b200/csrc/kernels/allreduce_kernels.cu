// Aggregation kernels for sm_100a: see allreduce_kernels.h for the host interface.
//
// ALGO_STAGED — the streaming pipeline. A job is cut into contiguous per-channel ranges
// (the analogue of the reference scheduler's static per-thread slices,
// schedulers/fifo_scheduler.cc:92-109); a channel (one CTA on every rank) walks its range
// in tiles of at most one staging slot. Per tile:
//   MODE_QUANT   A  the block exponents were agreed one or two tiles earlier through tagged
//                   atomic maxima (quant_tile.cuh); quantise own tile into the slot  [phase 1]
//                B  owner of shard r: integer sum over ranks of its shard
//                   (multimem.ld_reduce.add.s32 / peer loads), dequantise, broadcast
//                   (multimem.st / peer stores) into the slot, or into the outputs
//                   themselves when they lie in symmetric memory                     [phase 2]
//                C  copy the finished tile from the slot to the output
//   MODE_SUM     copy-in [phase 1], B with a float/int add, [phase 2], copy-out.
// The signal after B is also the acknowledgement that lets the slot be reused, the role
// of the "other set" bitmap clear in the switch (p4/bitmap_checker.p4:82-123). Whole-tile
// copies go through the TMA unit (bulk_copy.cuh), the quantising loader reads through
// per-warp TMA streams (warp_stream.cuh), and a signaler warp tells the peers so that no
// role waits for its own system-scope fence.
//
// ALGO_PUSH — peer memory without multicast: see push_allreduce.cuh.
//
// ALGO_ONESHOT — for small messages: every rank pushes its input into a per-source buffer
// on every rank (one multimem.st, or n peer stores), one barrier, then each rank reduces
// the n copies locally (in QUANT mode with exactly the same integer arithmetic).
//
// ALGO_ZEROCOPY — tensors that live in symmetric memory are reduced in place: barrier,
// shard-wise reduce+broadcast, barrier. No staging traffic at all.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "kernels/allreduce_kernels.h"
#include "kernels/bulk_copy.cuh"
#include "kernels/device_sync.cuh"
#include "kernels/multimem.cuh"
#include "kernels/quant_tile.cuh"
#include "switchml/quant_math.h"

namespace switchml {
namespace kernels {

namespace {

static const int kMaxBlocksPerSlot = 8192;  // scale factors of all slots of a channel (shared memory)
static const int kUnroll = 8;        // 16-byte vectors in flight per thread, local copies
static const int kDefaultUnrollLink = 4;  // ... for staged loads that cross NVLink (8 measured slower)
static const int kZeroCopyUnrollLink = 2;  // in-switch reduction: few requests in flight are best (8 GPUs: 2.25 ms vs 2.38 ms with 8)
static const int kZeroCopyUnrollPeer = 16;  // plain peer loads want many (2 GPUs: 1.75 ms vs 1.91 ms with 2)


__device__ __forceinline__ bool Aligned16(const void* p) {
  return (reinterpret_cast<uintptr_t>(p) & 15) == 0;
}

__device__ __forceinline__ uint4 LoadCg16(const void* p) {
  return __ldcg(reinterpret_cast<const uint4*>(p));
}

// bf16 pair helpers -----------------------------------------------------------------
__device__ __forceinline__ float2 Bf16x2ToFloat2(unsigned u) {
  return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
}
__device__ __forceinline__ unsigned Float2ToBf16x2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<unsigned*>(&h);
}
__device__ __forceinline__ float Bf16ToFloat(unsigned short u) {
  return __uint_as_float(static_cast<unsigned>(u) << 16);
}
__device__ __forceinline__ unsigned short FloatToBf16(float f) {
  __nv_bfloat16 h = __float2bfloat16_rn(f);
  return *reinterpret_cast<unsigned short*>(&h);
}

// Element `i` of the input as float (QUANT mode reads f32 or bf16).
template <int ELEM>
__device__ __forceinline__ float LoadAsFloat(const void* in, size_t i) {
  if (ELEM == ELEM_BF16) return Bf16ToFloat(reinterpret_cast<const unsigned short*>(in)[i]);
  return reinterpret_cast<const float*>(in)[i];
}

// ------------------------------------------------------------------------------------
// Reduce one 16-byte vector at byte offset `off` of the staging/user regions over all
// ranks and return it post-scaled. `nvalid` is unused here; tails are handled by callers.
template <int ELEM>
__device__ __forceinline__ uint4 ReduceVec(const RankCtx& ctx, char* const* peers, char* mc,
                                           size_t off, float post_scale) {
  uint4 r;
  if (ELEM == ELEM_F32) {
    float4 a;
    if (ctx.use_multimem) {
      a = MultimemLdReduceAddF32x4(mc + off);
    } else {
      a = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int p = 0; p < ctx.nranks; p++) {
        uint4 v = LoadCg16(peers[p] + off);
        a.x += __uint_as_float(v.x);
        a.y += __uint_as_float(v.y);
        a.z += __uint_as_float(v.z);
        a.w += __uint_as_float(v.w);
      }
    }
    if (post_scale != 1.0f) { a.x *= post_scale; a.y *= post_scale; a.z *= post_scale; a.w *= post_scale; }
    r = make_uint4(__float_as_uint(a.x), __float_as_uint(a.y), __float_as_uint(a.z), __float_as_uint(a.w));
  } else if (ELEM == ELEM_I32) {
    if (ctx.use_multimem) {
      r.x = static_cast<unsigned>(MultimemLdReduceAddS32(mc + off));
      r.y = static_cast<unsigned>(MultimemLdReduceAddS32(mc + off + 4));
      r.z = static_cast<unsigned>(MultimemLdReduceAddS32(mc + off + 8));
      r.w = static_cast<unsigned>(MultimemLdReduceAddS32(mc + off + 12));
    } else {
      r = make_uint4(0, 0, 0, 0);
      for (int p = 0; p < ctx.nranks; p++) {
        uint4 v = LoadCg16(peers[p] + off);
        r.x += v.x; r.y += v.y; r.z += v.z; r.w += v.w;  // wrapping
      }
    }
  } else {  // bf16: 8 values, float32 accumulation
    float acc[8];
    if (ctx.use_multimem) {
      uint4 v = MultimemLdReduceAddBf16x8(mc + off);
      if (post_scale == 1.0f) return v;
      float2 t;
      t = Bf16x2ToFloat2(v.x); acc[0] = t.x; acc[1] = t.y;
      t = Bf16x2ToFloat2(v.y); acc[2] = t.x; acc[3] = t.y;
      t = Bf16x2ToFloat2(v.z); acc[4] = t.x; acc[5] = t.y;
      t = Bf16x2ToFloat2(v.w); acc[6] = t.x; acc[7] = t.y;
    } else {
#pragma unroll
      for (int j = 0; j < 8; j++) acc[j] = 0.f;
      for (int p = 0; p < ctx.nranks; p++) {
        uint4 v = LoadCg16(peers[p] + off);
        float2 t;
        t = Bf16x2ToFloat2(v.x); acc[0] += t.x; acc[1] += t.y;
        t = Bf16x2ToFloat2(v.y); acc[2] += t.x; acc[3] += t.y;
        t = Bf16x2ToFloat2(v.z); acc[4] += t.x; acc[5] += t.y;
        t = Bf16x2ToFloat2(v.w); acc[6] += t.x; acc[7] += t.y;
      }
    }
    if (post_scale != 1.0f) {
#pragma unroll
      for (int j = 0; j < 8; j++) acc[j] *= post_scale;
    }
    r.x = Float2ToBf16x2(acc[0], acc[1]);
    r.y = Float2ToBf16x2(acc[2], acc[3]);
    r.z = Float2ToBf16x2(acc[4], acc[5]);
    r.w = Float2ToBf16x2(acc[6], acc[7]);
  }
  return r;
}

// Write one 16-byte vector to every rank's copy.
__device__ __forceinline__ void BroadcastVec(const RankCtx& ctx, char* const* peers, char* mc,
                                             size_t off, uint4 v) {
  if (ctx.use_multimem) {
    MultimemStore16(mc + off, v);
  } else {
    for (int p = 0; p < ctx.nranks; p++) *reinterpret_cast<uint4*>(peers[p] + off) = v;
  }
}

// Shard [begin,end) (elements) of a tile that has `len` elements; units of `unit`.
__device__ __forceinline__ void ShardRange(size_t len, int nranks, int rank, size_t unit,
                                           size_t* begin, size_t* end) {
  size_t per = (len + nranks - 1) / nranks;
  per = (per + unit - 1) / unit * unit;
  size_t b = per * rank, e = b + per;
  *begin = b < len ? b : len;
  *end = e < len ? e : len;
}

// ------------------------------------------------------------------------------------
// Warp-specialised streaming pipeline. The 16 warps of a channel split into three roles
// that walk the channel's tiles independently, so that for different tiles the local
// HBM copies and the NVLink phase run at the same time:
//   loader   (warps 0-3; 0-5 when it quantises)  copy-in / quantise, exponents ahead -> phase 1
//   reducer  (the next 8 warps)   waits phase 1, reduces + broadcasts its shard    -> phase 2
//   storer   (all but the last of the rest)  waits phase 2, copies the tile out    -> frees the slot
//   signaler (the last warp)      fences and stores the flags for loader and reducer
// A role synchronises internally with its own named barrier; the loader may run ahead of
// the storer by the number of slots of the channel.
static const int kDefaultLoadWarps = 4, kDefaultReduceWarps = 8;  // of the 16 warps; one signals, the rest store

struct StagedShared {
  int failed;
  volatile unsigned long long stored;  // tiles copied out so far
  unsigned long long done[3];          // tiles that loader / reducer / storer have finished: the signaler warp tells the peers
  BulkRing ring[2];                    // TMA copy rings of the loader [0] and the storer [1]
  WarpStreamBarriers ws;               // mbarriers of the quantising loader's per-warp streams
  char* ring_buffers;                  // dynamic shared memory (nullptr: the job's tensors rule the TMA paths out):
                                       // [0, kBulkRingBytes) storer ring, then the loader's ring or its warps' rings
};
static const int kStreamWarps = 6;     // loader warps of the quantised mode; each owns kWsRingBytes
static const size_t kLoaderSmemOffset = kBulkRingBytes;
static const size_t kLoaderSmemBytes = kStreamWarps * kWsRingBytes > kBulkRingBytes ? kStreamWarps * kWsRingBytes : kBulkRingBytes;

struct Role {
  int tid;       // thread index inside the role
  int nthreads;  // threads of the role
  int bar_id;    // named barrier of the role
  __device__ __forceinline__ void Sync() const {
    asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(nthreads) : "memory");
  }
};

// All threads of the role call this after writing data the peers will read.
__device__ __forceinline__ void RoleSignal(const RankCtx& ctx, const Role& role, int channel,
                                           int phase, Epoch epoch) {
  role.Sync();
  if (role.tid < ctx.nranks) {
    if (ctx.sc_fence) __threadfence_system();
    StoreReleaseSys(FlagPtr(ctx.stage_peer[role.tid], channel, phase, ctx.rank), epoch);
  }
}

// All threads of the role call this before reading data the peers wrote. False = timed
// out or another role failed.
__device__ __forceinline__ bool RoleWait(const RankCtx& ctx, const Role& role, int channel,
                                         int phase, Epoch epoch, StagedShared* sh) {
  if (role.tid < ctx.nranks) {
    const Epoch* mine = FlagPtr(ctx.stage_peer[ctx.rank], channel, phase, role.tid);
    unsigned long long start = GlobalTimerNs();
    unsigned long long spins = 0;
    while (LoadAcquireSys(mine) < epoch) {
      ++spins;
      if ((spins & 63) == 0) {
        if (*reinterpret_cast<volatile int*>(&sh->failed)) break;
        if (GlobalTimerNs() - start > ctx.timeout_ns) {
          ReportStatus(ctx, STATUS_TIMEOUT | (phase << 4) | (channel << 8));
          atomicAdd(ctx.counters + 2, 1ull);
          *reinterpret_cast<volatile int*>(&sh->failed) = 1;
          break;
        }
      }
      __nanosleep(20);
    }
    if (spins) atomicAdd(ctx.counters + 1, spins);
  }
  role.Sync();
  return *reinterpret_cast<volatile int*>(&sh->failed) == 0;
}

// A role has finished tile number `tiles_done` (counted from 1): its data is where the peers
// will read it. Telling them takes a system-scope fence, which on a busy link waits tens of
// microseconds for the role's posted stores to be acknowledged; the role does not wait for
// that itself but leaves a note in shared memory for the signaler warp and goes on with the
// next tile. All threads of the role call this.
__device__ __forceinline__ void RoleDone(const Role& role, StagedShared* sh, int which, unsigned long long tiles_done) {
  role.Sync();
  if (role.tid == 0)
    asm volatile("st.release.cta.shared::cta.u64 [%0], %1;" ::"r"(BulkSmemAddr(&sh->done[which])), "l"(tiles_done) : "memory");
}

// The signaler warp: turns the roles' notes into flag stores. For every role whose count has
// grown it fences at system scope (everything the role wrote before its note, which this warp
// acquired, is ordered before the flag) and stores the epoch of the newest finished tile into
// the role's phase on every rank; waits are ">=", so the newest epoch answers for all. Ends
// when every signalling role has finished `ntiles` tiles or the CTA failed.
__device__ __forceinline__ void RunSignaler(const RankCtx& ctx, StagedShared* sh, int channel, Epoch base,
                                            unsigned long long ntiles, int nroles) {
  const int lane = threadIdx.x & 31;
  unsigned long long told[3] = {0, 0, 0};
  volatile int* failed = reinterpret_cast<volatile int*>(&sh->failed);
  for (;;) {
    // All notes first, then one fence for whatever is new: the fence is the expensive part
    // (it drains behind the SM's stores in flight) and covers every role's writes at once.
    unsigned long long d[3] = {0, 0, 0};
    bool news = false;
#pragma unroll
    for (int r = 0; r < 3; r++) {
      if (r >= nroles) continue;
      asm volatile("ld.acquire.cta.shared::cta.u64 %0, [%1];" : "=l"(d[r]) : "r"(BulkSmemAddr(&sh->done[r])) : "memory");
      news |= d[r] > told[r];
    }
    if (news && ctx.sc_fence) __threadfence_system();
    bool all = true;
#pragma unroll
    for (int r = 0; r < 3; r++) {
      if (r >= nroles) continue;
      if (d[r] > told[r]) {
        if (lane < ctx.nranks) StoreReleaseSys(FlagPtr(ctx.stage_peer[lane], channel, r + 1, ctx.rank), base + d[r]);
        told[r] = d[r];
      }
      if (told[r] < ntiles) all = false;
    }
    if (all || *failed) return;
    __nanosleep(40);
  }
}

// Byte-wise identical copy by the threads of one role.
__device__ __forceinline__ void RoleCopy(const Role& role, void* dst, const void* src, size_t bytes,
                                         int esz) {
  const int t = role.tid, n = role.nthreads;
  if (Aligned16(dst) && Aligned16(src)) {
    size_t nvec = bytes / 16;
    const uint4* s = reinterpret_cast<const uint4*>(src);
    uint4* d = reinterpret_cast<uint4*>(dst);
    size_t i = t;
    for (; i + (kUnroll - 1) * n < nvec; i += kUnroll * n) {
      uint4 v[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; u++) v[u] = s[i + u * n];
#pragma unroll
      for (int u = 0; u < kUnroll; u++) d[i + u * n] = v[u];
    }
    for (; i < nvec; i += n) d[i] = s[i];
    for (size_t b = nvec * 16 + static_cast<size_t>(t) * esz; b < bytes; b += static_cast<size_t>(n) * esz) {
      if (esz == 4) *reinterpret_cast<unsigned*>(static_cast<char*>(dst) + b) = *reinterpret_cast<const unsigned*>(static_cast<const char*>(src) + b);
      else *reinterpret_cast<unsigned short*>(static_cast<char*>(dst) + b) = *reinterpret_cast<const unsigned short*>(static_cast<const char*>(src) + b);
    }
  } else if (esz == 4) {
    const unsigned* s = reinterpret_cast<const unsigned*>(src);
    unsigned* d = reinterpret_cast<unsigned*>(dst);
    for (size_t i = t; i < bytes / 4; i += n) d[i] = s[i];
  } else {
    const unsigned short* s = reinterpret_cast<const unsigned short*>(src);
    unsigned short* d = reinterpret_cast<unsigned short*>(dst);
    for (size_t i = t; i < bytes / 2; i += n) d[i] = s[i];
  }
}

// A local copy by a role: through the TMA unit when the geometry allows it (one thread drives
// it, see bulk_copy.cuh), else with the role's own loads and stores. `which` picks the ring.
// The caller synchronises the role afterwards (RoleSignal / role.Sync) and checks `failed`.
__device__ __forceinline__ void RoleLocalCopy(const RankCtx& ctx, const Role& role, StagedShared* sh, int which,
                                              void* dst, const void* src, size_t bytes, int esz) {
  if (sh->ring_buffers != nullptr && BulkCopyable(dst, src, bytes)) {
    if (role.tid == 0)
      BulkCopy(&sh->ring[which], sh->ring_buffers + (which == 0 ? kLoaderSmemOffset : 0), static_cast<char*>(dst),
               static_cast<const char*>(src), bytes, ctx.timeout_ns, reinterpret_cast<volatile int*>(&sh->failed));
  } else {
    RoleCopy(role, dst, src, bytes, esz);
  }
}

// Checked build (-DSWITCHML_CHECKED): before a tile, a one-shot buffer or a symmetric tensor
// is touched, its geometry is verified against the sizes of the regions it indexes. A
// violation stores STATUS_BOUNDS with the channel in the status word, marks the CTA as
// failed and skips the work: nothing out of range is dereferenced and nothing traps. The
// condition depends only on launch arguments that are the same on every rank, so all
// threads of the CTA, and the same channel on the peers, take the same way out.
#ifdef SWITCHML_CHECKED
#define SML_GEOMETRY_CHECK(CTX, CHANNEL, FAILED, COND)                      \
  if (!(COND)) {                                                            \
    ReportStatus((CTX), STATUS_BOUNDS | ((CHANNEL) << 8));                  \
    *(FAILED) = 1;                                                          \
    return;                                                                 \
  }
#else
#define SML_GEOMETRY_CHECK(CTX, CHANNEL, FAILED, COND)
#endif

template <int ELEM, int MODE, int kLoadWarps = kDefaultLoadWarps, int kReduceWarps = kDefaultReduceWarps,
          int kUnrollLink = kDefaultUnrollLink>
__device__ void RunStaged(const RankCtx& ctx, const JobArgs& job, int channel,
                          unsigned long long elems_per_channel, Epoch base, StagedShared* sh, float* s_sf) {
  constexpr int kStoreWarps = kThreads / 32 - kLoadWarps - kReduceWarps - 1;  // the last warp tells the peers
  static_assert(kStoreWarps >= 1, "the storer needs a warp");
  constexpr int kUnrollInt = 4 * kUnrollLink;  // 4-byte integer lanes in flight per thread
  const int in_esz = ELEM == ELEM_BF16 ? 2 : 4;
  const int st_esz = MODE == MODE_QUANT ? 4 : in_esz;
  const size_t slot_elems = ctx.slot_bytes / st_esz;  // what the checked build verifies tiles against
  (void)slot_elems;
  const size_t vec_elems = 16 / st_esz;
  const size_t unit = MODE == MODE_QUANT ? static_cast<size_t>(ctx.block_numel) : 128;
  const int S = ctx.slots_per_channel;

  unsigned long long c0 = static_cast<unsigned long long>(channel) * elems_per_channel;
  if (c0 >= job.numel) return;
  unsigned long long c1 = c0 + elems_per_channel;
  if (c1 > job.numel) c1 = job.numel;
  const size_t tile_elems = job.tile_elems;  // <= slot_elems; small jobs use small tiles
  const unsigned long long ntiles = (c1 - c0 + tile_elems - 1) / tile_elems;
  char* my_stage = ctx.stage_peer[ctx.rank];
  const size_t blocks_per_slot = ctx.slot_bytes / 4 / ctx.block_numel;
  const int shift = 31 - __clz(ctx.block_numel);  // block_numel is a power of two
  // The exponents of tile k+A travel while tile k is quantised, so the agreement never costs a
  // wait of its own: what tile k needs was signalled A tiles ago, with the payload of tile k-A.
  // That signal is slow to arrive while a reducer saturates the link (its fence drains behind
  // the bulk stores), so A tiles have to cover it: with A = 2 the loaders of four GPUs waited
  // 300 us per pair of tiles for it. The exponent words have a ring of E slots of their own. The
  // words of tile k+A were last used by tile k+A-E, which every rank consumed before it signalled
  // that tile's payload (phase 1); the loader has awaited phase 1 of tile k-A by then, and
  // E >= 2A. A single data slot leaves no room to run ahead (A = 0).
  const unsigned long long A = static_cast<unsigned long long>(ctx.exp_lookahead);
  const int E = ctx.exp_ring;
  // The output lies in symmetric memory: the owner of a shard broadcasts the finished values
  // straight into every rank's output and nothing is copied out of the slot.
  const bool direct_out = job.out_zero_copy != 0;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  Role role;
  int which;
  if (warp < kLoadWarps) {
    which = 0; role.tid = threadIdx.x; role.nthreads = kLoadWarps * 32; role.bar_id = 1;
  } else if (warp < kLoadWarps + kReduceWarps) {
    which = 1; role.tid = threadIdx.x - kLoadWarps * 32; role.nthreads = kReduceWarps * 32; role.bar_id = 2;
  } else if (warp < kLoadWarps + kReduceWarps + kStoreWarps) {
    which = 2; role.tid = threadIdx.x - (kLoadWarps + kReduceWarps) * 32; role.nthreads = kStoreWarps * 32; role.bar_id = 3;
  } else {
    RunSignaler(ctx, sh, channel, base, ntiles, 2);  // loader (phase 1) and reducer (phase 2)
    return;
  }
  volatile int* failed = reinterpret_cast<volatile int*>(&sh->failed);
  // Channel 0 keeps a coarse time budget of its roles (ns waiting for others / ns doing
  // its own work) in counters[3 + 2*role], [4 + 2*role]: a built-in pipeline profile.
  const bool timed = channel == 0 && role.tid == 0;
  unsigned long long t_mark = timed ? GlobalTimerNs() : 0;
  unsigned long long cur_tile = 0;  // for the trace
  if (timed && which == 0 && ctx.trace) ctx.trace[6 * kTraceTiles] = t_mark;
  auto lap = [&](int idx) {
    if (timed) {
      unsigned long long now = GlobalTimerNs();
      atomicAdd(ctx.counters + idx, now - t_mark);
      t_mark = now;
      // idx 3/5/7: the role's waits for this tile are over; 4/6/8: the tile is finished
      if (ctx.trace && idx >= 3 && idx <= 8 && cur_tile < kTraceTiles)
        ctx.trace[(which * 2 + ((idx - 3) & 1)) * kTraceTiles + cur_tile] = now;
    }
  };
  auto tile_len = [&](unsigned long long k) {
    const unsigned long long pos = c0 + k * tile_elems;
    return static_cast<size_t>(c1 - pos < tile_elems ? c1 - pos : tile_elems);
  };
  auto exp_offset_of = [&](unsigned long long k) {
    const size_t ring_index = static_cast<size_t>(channel) * E + static_cast<size_t>(k % E);
    return ctx.exp_offset + ring_index * blocks_per_slot * kExpWordBytes;
  };
  // The quantising loader reads float32 device memory through per-warp TMA streams.
  static_assert(MODE != MODE_QUANT || kLoadWarps <= kStreamWarps, "every loader warp needs a ring");
  const bool stream = MODE == MODE_QUANT && ELEM == ELEM_F32 && sh->ring_buffers != nullptr &&
                      (reinterpret_cast<uintptr_t>(job.in) & 15) == 0;
  WarpStream ws;
  if (MODE == MODE_QUANT && warp < kLoadWarps) {
    ws.ring = stream ? sh->ring_buffers + kLoaderSmemOffset + static_cast<size_t>(warp) * kWsRingBytes : nullptr;
    ws.full = sh->ws.full[warp];
    ws.used = 0;
    ws.timeout_ns = ctx.timeout_ns;
    ws.failed = failed;
  }
  auto publish = [&](const char* tile_in, size_t tile_len_, size_t tile_exp_off, Epoch tag) {
    if (stream) return StreamTileExponents(ctx, ws, warp, kLoadWarps, lane, tile_in, tile_len_, tile_exp_off, tag);
    PublishTileExponents<ELEM>(ctx, warp, kLoadWarps, lane, tile_in, tile_len_, tile_exp_off, tag);
    return true;
  };

  for (unsigned long long k = 0; k < ntiles; ++k) {
    cur_tile = k;
    const unsigned long long pos = c0 + k * tile_elems;
    const Epoch epoch = base + k + 1;
    const size_t len = tile_len(k);
    const int slot = static_cast<int>(k % S);
    const size_t slot_index = static_cast<size_t>(channel) * S + slot;
    const size_t slot_off = ctx.data_offset + slot_index * ctx.slot_bytes;  // same on all ranks
    const size_t exp_off = exp_offset_of(k);
    SML_GEOMETRY_CHECK(ctx, channel, failed,
                       len > 0 && len <= slot_elems && pos + len <= job.numel &&
                       slot_off >= ctx.data_offset && slot_off + ctx.slot_bytes <= ctx.stage_bytes &&
                       (MODE != MODE_QUANT ||
                        (blocks_per_slot * S <= static_cast<size_t>(kMaxBlocksPerSlot) &&
                         E >= 1 && 2 * A <= static_cast<unsigned long long>(E) &&
                         exp_off + blocks_per_slot * kExpWordBytes <= ctx.oneshot_offset)) &&
                       (!direct_out || job.out_offset + (pos + len) * in_esz <= job.user_bytes));
    float* sf = s_sf + static_cast<size_t>(slot) * blocks_per_slot;

    if (which == 0) {
      // ------------------------------ loader ------------------------------
      const char* in = static_cast<const char*>(job.in) + pos * in_esz;
      // The slot is free once the tile that used it last has been copied out here; by
      // then every peer has finished reading it as well (their phase-2 signals came
      // before that copy-out).
      if (k >= static_cast<unsigned long long>(S)) {
        if (role.tid == 0) {
          unsigned long long start = GlobalTimerNs(), spins = 0;
          while (sh->stored + S < k + 1) {
            if ((++spins & 63) == 0 && (*failed || GlobalTimerNs() - start > ctx.timeout_ns)) {
              if (!*failed) ReportStatus(ctx, STATUS_TIMEOUT | (3 << 4) | (channel << 8));
              *failed = 1;
              break;
            }
            __nanosleep(20);
          }
        }
        role.Sync();
        if (*failed) return;
      }
      if (MODE == MODE_QUANT) {
        if (k == 0 || A == 0) {
          // Nobody has published the exponents of this tile (of the first A tiles, at the start
          // of a job) yet: do it now and meet (phase 0). Without lookahead the words are free
          // by now: their last user is E tiles back, and every rank consumed that tile before it
          // signalled its payload, which the meeting of the tile before this one came after.
          bool published = publish(in, len, exp_off, epoch);
          for (unsigned long long t = 1; published && t < A && t < ntiles; t++)
            published = publish(in + t * tile_elems * in_esz, tile_len(t), exp_offset_of(t), epoch + t);
          RoleSignal(ctx, role, channel, 0, epoch);
          const bool met = RoleWait(ctx, role, channel, 0, epoch, sh);  // every warp takes part, whatever happened
          if (!published || !met) return;
        } else if (k >= A) {
          // They came with the payload signal of tile k-A.
          if (!RoleWait(ctx, role, channel, 1, epoch - A, sh)) return;
        }
      }
      lap(3);
      if (MODE == MODE_QUANT) {
        const size_t nblocks = (len + ctx.block_numel - 1) / ctx.block_numel;
        TileScaleFactors(ctx, role.tid, role.nthreads, exp_off, nblocks, epoch, sf, channel, failed);
        role.Sync();
        if (*failed) return;
        lap(9);
        int* q = reinterpret_cast<int*>(my_stage + slot_off);
        bool streamed = true;
        size_t done = 0;
        if (stream) {
          const size_t nchunks = len / (kWsChunk / 4);
          streamed = StreamQuantize(ws, warp, kLoadWarps, lane, in, 0, nchunks, sf, shift,
                                    [&](size_t e, int4 r) { *reinterpret_cast<int4*>(q + e) = r; });
          done = nchunks * (kWsChunk / 4);
        }
        QuantizeRange<ELEM, 8>(role.tid, role.nthreads, in, q + done, done, len, sf, shift);
        lap(10);
        // Exponents of tile k+A, ahead of its data.
        if (streamed && A > 0 && k + A < ntiles)
          streamed = publish(in + A * tile_elems * in_esz, tile_len(k + A), exp_offset_of(k + A), epoch + A);
        if (!streamed) {
          role.Sync();  // the other warps are on their way to the signal's barrier: meet them, then leave together
          return;
        }
        lap(11);
      } else {
        RoleLocalCopy(ctx, role, sh, 0, my_stage + slot_off, in, len * in_esz, in_esz);
      }
      RoleDone(role, sh, 0, k + 1);
      if (*failed) return;
      lap(4);
    } else if (which == 1) {
      // ------------------------------ reducer ------------------------------
      if (!RoleWait(ctx, role, channel, 1, epoch, sh)) return;
      lap(5);
      size_t sb, se;
      ShardRange(len, ctx.nranks, ctx.rank, unit, &sb, &se);
      const int t = role.tid, n = role.nthreads;
      // Where finished values go: this tile's place in the slot, or in the output itself.
      char* const* dst_peer = direct_out ? job.user_peer : ctx.stage_peer;
      char* dst_mc = direct_out ? job.user_mc : ctx.stage_mc;
      // bf16 jobs of the exact mode get their results as bf16: into the output itself, or into
      // the second part of the slot, behind the int32 payload of a full tile.
      const size_t narrow_area = job.tile_elems * 4;
      const bool narrow = MODE == MODE_QUANT && ELEM == ELEM_BF16 && (direct_out || job.tile_elems * 6 <= ctx.slot_bytes);
      const size_t dst_off = direct_out ? job.out_offset + pos * in_esz : (narrow ? slot_off + narrow_area : slot_off);
      // An empty shard (short last tile) must not touch anything: rounding its bounds to
      // whole vectors would make it overlap the last vector of the previous rank's shard.
      if (sb >= se) {
      } else if (narrow) {
        // Two neighbouring lanes pair their results into one 32-bit store.
        char* mc = ctx.stage_mc + slot_off;
        for (size_t i0 = sb + (t & ~31); i0 < se; i0 += n) {
          const size_t i = i0 + lane;
          int v = 0;
          if (i < se) {
            if (ctx.use_multimem) {
              v = MultimemLdReduceAddS32(mc + i * 4);
            } else {
              for (int p = 0; p < ctx.nranks; p++) v += __ldcg(reinterpret_cast<const int*>(ctx.stage_peer[p] + slot_off) + i);
            }
          }
          float y = i < se ? quant::Dequantize(v, sf[i >> shift]) : 0.f;
          if (job.post_scale != 1.0f) y *= job.post_scale;
          const float hi = __shfl_down_sync(0xffffffffu, y, 1);
          if ((lane & 1) == 0 && i < se) {
            if (i + 1 < se) {
              const unsigned pair = Float2ToBf16x2(y, hi);
              if (ctx.use_multimem) MultimemStore4(dst_mc + dst_off + i * 2, pair);
              else for (int p = 0; p < ctx.nranks; p++) *reinterpret_cast<unsigned*>(dst_peer[p] + dst_off + i * 2) = pair;
            } else {
              const unsigned short h = FloatToBf16(y);  // odd tail of the job's last tile
              for (int p = 0; p < ctx.nranks; p++) *reinterpret_cast<unsigned short*>(dst_peer[p] + dst_off + i * 2) = h;
            }
          }
        }
      } else if (MODE == MODE_QUANT || ELEM == ELEM_I32) {
        if (ctx.use_multimem) {
          // Integer in-switch adds are one 32-bit lane per instruction: let consecutive
          // lanes take consecutive words so that a warp moves one full 128-byte line.
          char* mc = ctx.stage_mc + slot_off;
          char* out_mc = dst_mc + dst_off;
          size_t i = sb + t;
          for (; i + (kUnrollInt - 1) * n < se; i += kUnrollInt * n) {
            int v[kUnrollInt];
#pragma unroll
            for (int u = 0; u < kUnrollInt; u++) v[u] = MultimemLdReduceAddS32(mc + (i + u * n) * 4);
#pragma unroll
            for (int u = 0; u < kUnrollInt; u++) {
              unsigned bits = static_cast<unsigned>(v[u]);
              if (MODE == MODE_QUANT) {
                float y = quant::Dequantize(v[u], sf[(i + u * n) >> shift]);
                if (job.post_scale != 1.0f) y *= job.post_scale;
                bits = __float_as_uint(y);
              }
              MultimemStore4(out_mc + (i + u * n) * 4, bits);
            }
          }
          if (i < se) {
            // The remainder, fewer than kUnrollInt * n words: all of them in flight at once (one
            // trip through the switch instead of one per word and thread).
            int v[kUnrollInt];
#pragma unroll
            for (int u = 0; u < kUnrollInt; u++)
              if (i + u * n < se) v[u] = MultimemLdReduceAddS32(mc + (i + u * n) * 4);
#pragma unroll
            for (int u = 0; u < kUnrollInt; u++) {
              if (i + u * n < se) {
                unsigned bits = static_cast<unsigned>(v[u]);
                if (MODE == MODE_QUANT) {
                  float y = quant::Dequantize(v[u], sf[(i + u * n) >> shift]);
                  if (job.post_scale != 1.0f) y *= job.post_scale;
                  bits = __float_as_uint(y);
                }
                MultimemStore4(out_mc + (i + u * n) * 4, bits);
              }
            }
          }
        } else {
          size_t v0 = sb / 4, v1 = (se + 3) / 4;
          auto finish = [&](size_t v, uint4 sum) {
            if (MODE == MODE_QUANT) {
              float f = sf[(v * 4) >> shift];
              float4 y;
              y.x = quant::Dequantize(static_cast<int>(sum.x), f);
              y.y = quant::Dequantize(static_cast<int>(sum.y), f);
              y.z = quant::Dequantize(static_cast<int>(sum.z), f);
              y.w = quant::Dequantize(static_cast<int>(sum.w), f);
              if (job.post_scale != 1.0f) { y.x *= job.post_scale; y.y *= job.post_scale; y.z *= job.post_scale; y.w *= job.post_scale; }
              sum = make_uint4(__float_as_uint(y.x), __float_as_uint(y.y), __float_as_uint(y.z), __float_as_uint(y.w));
            }
            if (direct_out && v * 4 + 4 > len) {
              // the job's ragged end must not spill past the output tensor
              const unsigned w[4] = {sum.x, sum.y, sum.z, sum.w};
              for (size_t j = 0; v * 4 + j < len; j++)
                for (int p = 0; p < ctx.nranks; p++) *reinterpret_cast<unsigned*>(dst_peer[p] + dst_off + (v * 4 + j) * 4) = w[j];
            } else {
              BroadcastVec(ctx, dst_peer, dst_mc, dst_off + v * 16, sum);
            }
          };
          size_t v = v0 + t;
          for (; v + (kUnrollLink - 1) * n < v1; v += kUnrollLink * n) {
            uint4 r[kUnrollLink];
#pragma unroll
            for (int u = 0; u < kUnrollLink; u++)
              r[u] = ReduceVec<ELEM_I32>(ctx, ctx.stage_peer, ctx.stage_mc, slot_off + (v + u * n) * 16, 1.0f);
#pragma unroll
            for (int u = 0; u < kUnrollLink; u++) finish(v + u * n, r[u]);
          }
          if (v < v1) {  // the remainder in one go, see above
            uint4 r[kUnrollLink];
#pragma unroll
            for (int u = 0; u < kUnrollLink; u++)
              if (v + u * n < v1) r[u] = ReduceVec<ELEM_I32>(ctx, ctx.stage_peer, ctx.stage_mc, slot_off + (v + u * n) * 16, 1.0f);
#pragma unroll
            for (int u = 0; u < kUnrollLink; u++)
              if (v + u * n < v1) finish(v + u * n, r[u]);
          }
        }
      } else {
        size_t v0 = sb / vec_elems, v1 = (se + vec_elems - 1) / vec_elems;
        size_t v = v0 + t;
        for (; v + (kUnrollLink - 1) * n < v1; v += kUnrollLink * n) {
          uint4 r[kUnrollLink];
#pragma unroll
          for (int u = 0; u < kUnrollLink; u++)
            r[u] = ReduceVec<ELEM>(ctx, ctx.stage_peer, ctx.stage_mc, slot_off + (v + u * n) * 16, job.post_scale);
#pragma unroll
          for (int u = 0; u < kUnrollLink; u++)
            BroadcastVec(ctx, ctx.stage_peer, ctx.stage_mc, slot_off + (v + u * n) * 16, r[u]);
        }
        if (v < v1) {  // the remainder in one go, see above
          uint4 r[kUnrollLink];
#pragma unroll
          for (int u = 0; u < kUnrollLink; u++)
            if (v + u * n < v1) r[u] = ReduceVec<ELEM>(ctx, ctx.stage_peer, ctx.stage_mc, slot_off + (v + u * n) * 16, job.post_scale);
#pragma unroll
          for (int u = 0; u < kUnrollLink; u++)
            if (v + u * n < v1) BroadcastVec(ctx, ctx.stage_peer, ctx.stage_mc, slot_off + (v + u * n) * 16, r[u]);
        }
      }
      RoleDone(role, sh, 1, k + 1);
      lap(6);
    } else {
      // ------------------------------ storer ------------------------------
      if (!RoleWait(ctx, role, channel, 2, epoch, sh)) return;
      lap(7);
      if (!direct_out) {
        char* out = static_cast<char*>(job.out) + pos * in_esz;
        if (MODE == MODE_QUANT && ELEM == ELEM_BF16 && job.tile_elems * 6 <= ctx.slot_bytes) {
          RoleLocalCopy(ctx, role, sh, 1, out, my_stage + slot_off + job.tile_elems * 4, len * 2, 2);  // bf16 results
        } else if (MODE == MODE_QUANT && ELEM == ELEM_BF16) {
          const float* y = reinterpret_cast<const float*>(my_stage + slot_off);
          unsigned short* o = reinterpret_cast<unsigned short*>(out);
          for (size_t i = role.tid; i < len; i += role.nthreads) o[i] = FloatToBf16(y[i]);
        } else {
          RoleLocalCopy(ctx, role, sh, 1, out, my_stage + slot_off, len * in_esz, in_esz);
        }
      }
      role.Sync();
      if (*failed) return;
      if (role.tid == 0) {
        __threadfence_block();
        sh->stored = k + 1;
        atomicAdd(ctx.counters, 1ull);
      }
      lap(8);
    }
  }
}

}  // namespace
}  // namespace kernels
}  // namespace switchml
#include "kernels/push_allreduce.cuh"
namespace switchml {
namespace kernels {
namespace {

// ------------------------------------------------------------------------------------
template <int ELEM, int MODE>
__device__ void RunOneShot(const RankCtx& ctx, const JobArgs& job, int channel,
                           unsigned long long elems_per_channel, Epoch base, int* s_failed) {
  const int esz = ELEM == ELEM_BF16 ? 2 : 4;
  unsigned long long c0 = static_cast<unsigned long long>(channel) * elems_per_channel;
  if (c0 >= job.numel) return;
  unsigned long long c1 = c0 + elems_per_channel;
  if (c1 > job.numel) c1 = job.numel;
  const size_t len = static_cast<size_t>(c1 - c0);
  const unsigned long long epoch = base + 1;

  // Buffer of source rank s (same offset on every rank).
  auto buf_off = [&](int s) {
    return ctx.oneshot_offset +
           (static_cast<size_t>(job.oneshot_parity) * ctx.nranks + s) * ctx.oneshot_bytes + c0 * esz;
  };
  const char* in = static_cast<const char*>(job.in) + c0 * esz;
  const size_t bytes = len * esz;
  SML_GEOMETRY_CHECK(ctx, channel, s_failed,
                     c0 * esz + bytes <= ctx.oneshot_bytes && job.oneshot_parity >= 0 && job.oneshot_parity < 3 &&
                     buf_off(ctx.nranks - 1) + bytes <= ctx.data_offset && ctx.data_offset <= ctx.stage_bytes);

  if (MODE == MODE_SUM && ctx.use_multimem) {
    // Pull variant: every rank parks its input at the same offset of its own buffer, and
    // after one barrier each rank lets the switch reduce the whole range straight into its
    // output. No broadcast, no second barrier; costs n times the outbound traffic, which
    // small messages do not notice.
    const size_t off = buf_off(0);
    char* mine = ctx.stage_peer[ctx.rank] + off;
    Role all = {static_cast<int>(threadIdx.x), static_cast<int>(blockDim.x), 0};
    RoleCopy(all, mine, in, bytes, esz);
    if (!ChannelBarrier(ctx, channel, 3, epoch, s_failed)) return;
    char* mc = ctx.stage_mc + off;
    char* out = static_cast<char*>(job.out) + c0 * esz;
    if (ELEM == ELEM_I32) {
      // one 32-bit lane per instruction: keep eight of them in flight per thread
      constexpr int kInts = 8;
      size_t i = threadIdx.x;
      for (; i + (kInts - 1) * blockDim.x < len; i += kInts * blockDim.x) {
        int v[kInts];
#pragma unroll
        for (int u = 0; u < kInts; u++) v[u] = MultimemLdReduceAddS32(mc + (i + u * blockDim.x) * 4);
#pragma unroll
        for (int u = 0; u < kInts; u++) reinterpret_cast<int*>(out)[i + u * blockDim.x] = v[u];
      }
      for (; i < len; i += blockDim.x) reinterpret_cast<int*>(out)[i] = MultimemLdReduceAddS32(mc + i * 4);
    } else {
      const size_t vec_elems = 16 / esz;
      const size_t nfull = len / vec_elems;
      const bool aligned = Aligned16(out);
      for (size_t v = threadIdx.x; v * vec_elems < len; v += blockDim.x) {
        uint4 r = ReduceVec<ELEM>(ctx, ctx.stage_peer, ctx.stage_mc, off + v * 16, job.post_scale);
        if (aligned && v < nfull) {
          reinterpret_cast<uint4*>(out)[v] = r;
        } else {
          // unaligned output or the ragged last vector: element by element
          const unsigned w[4] = {r.x, r.y, r.z, r.w};
          for (size_t j = 0; j < vec_elems && v * vec_elems + j < len; j++) {
            if (esz == 4) reinterpret_cast<unsigned*>(out)[v * vec_elems + j] = w[j];
            else reinterpret_cast<unsigned short*>(out)[v * vec_elems + j] =
                     static_cast<unsigned short>(w[j >> 1] >> ((j & 1) * 16));
          }
        }
      }
    }
    if (threadIdx.x == 0) atomicAdd(ctx.counters, 1ull);
    // Replayable launches reuse one buffer: nobody may refill it before all have read it.
    if (job.trailing_barrier) ChannelBarrier(ctx, channel, 3, epoch + 1, s_failed);
    return;
  }

  const size_t my_off = buf_off(ctx.rank);
  // ---- push my range to everybody ----
  if (Aligned16(in)) {
    size_t nvec = bytes / 16;
    for (size_t i = threadIdx.x; i < nvec; i += blockDim.x) {
      uint4 v = reinterpret_cast<const uint4*>(in)[i];
      BroadcastVec(ctx, ctx.stage_peer, ctx.stage_mc, my_off + i * 16, v);
    }
    for (size_t b = nvec * 16 + threadIdx.x * esz; b < bytes; b += blockDim.x * esz) {
      for (int p = 0; p < ctx.nranks; p++) {
        if (esz == 4) *reinterpret_cast<unsigned*>(ctx.stage_peer[p] + my_off + b) = *reinterpret_cast<const unsigned*>(in + b);
        else *reinterpret_cast<unsigned short*>(ctx.stage_peer[p] + my_off + b) = *reinterpret_cast<const unsigned short*>(in + b);
      }
    }
  } else {
    for (size_t b = threadIdx.x * esz; b < bytes; b += blockDim.x * esz) {
      for (int p = 0; p < ctx.nranks; p++) {
        if (esz == 4) *reinterpret_cast<unsigned*>(ctx.stage_peer[p] + my_off + b) = *reinterpret_cast<const unsigned*>(in + b);
        else *reinterpret_cast<unsigned short*>(ctx.stage_peer[p] + my_off + b) = *reinterpret_cast<const unsigned short*>(in + b);
      }
    }
  }
  if (!ChannelBarrier(ctx, channel, 3, epoch, s_failed)) return;

  // ---- reduce the n local copies ----
  char* mine = ctx.stage_peer[ctx.rank];
  char* out = static_cast<char*>(job.out) + c0 * esz;
  if (MODE == MODE_QUANT) {
    // One warp per block: exponent over all ranks' copies, then quantise, add, dequantise.
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const size_t B = ctx.block_numel;
    const size_t nblocks = (len + B - 1) / B;
    for (size_t b = warp; b < nblocks; b += nwarps) {
      size_t base = b * B;
      size_t n = len - base < B ? len - base : B;
      float m = 0.f;
      int e = quant::kZeroExponent;
      for (int s = 0; s < ctx.nranks; s++) {
        const char* src = mine + buf_off(s);
        m = 0.f;
        for (size_t i = lane; i < n; i += 32) {
          float v = fabsf(LoadAsFloat<ELEM>(src, base + i));
          if (v > m) m = v;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          float t = __shfl_xor_sync(0xffffffffu, m, o);
          if (t > m) m = t;
        }
        int le = quant::LocalExponent(m);
        if (le > e) e = le;
      }
      float sf = quant::ScaleFactorFromBase(e, ctx.quant_base);
      for (size_t i = lane; i < n; i += 32) {
        unsigned acc = 0;
        for (int s = 0; s < ctx.nranks; s++)
          acc += static_cast<unsigned>(quant::Quantize(LoadAsFloat<ELEM>(mine + buf_off(s), base + i), sf));
        float y = quant::Dequantize(static_cast<int>(acc), sf);
        if (job.post_scale != 1.0f) y *= job.post_scale;
        if (ELEM == ELEM_BF16) reinterpret_cast<unsigned short*>(out)[base + i] = FloatToBf16(y);
        else reinterpret_cast<float*>(out)[base + i] = y;
      }
    }
  } else {
    // Whole 16-byte vectors first, four in flight per thread and source (the buffers are
    // vector aligned; the output may not be), then what is left element by element.
    size_t first = 0;
    if (Aligned16(out)) {
      const size_t vec_elems = 16 / esz, nvec = len / vec_elems;
      constexpr int U = 4;
      const size_t stride = blockDim.x;
      size_t v = threadIdx.x;
      for (; v + (U - 1) * stride < nvec; v += U * stride) {
        VecAcc<ELEM> acc[U];
#pragma unroll
        for (int u = 0; u < U; u++) acc[u].Init(*reinterpret_cast<const uint4*>(mine + buf_off(0) + (v + u * stride) * 16));
        for (int s = 1; s < ctx.nranks; s++) {
          const char* src = mine + buf_off(s);
          uint4 t[U];
#pragma unroll
          for (int u = 0; u < U; u++) t[u] = *reinterpret_cast<const uint4*>(src + (v + u * stride) * 16);
#pragma unroll
          for (int u = 0; u < U; u++) acc[u].Add(t[u]);
        }
#pragma unroll
        for (int u = 0; u < U; u++) *reinterpret_cast<uint4*>(out + (v + u * stride) * 16) = acc[u].Finish(job.post_scale);
      }
      for (; v < nvec; v += stride) {
        VecAcc<ELEM> acc;
        acc.Init(*reinterpret_cast<const uint4*>(mine + buf_off(0) + v * 16));
        for (int s = 1; s < ctx.nranks; s++) acc.Add(*reinterpret_cast<const uint4*>(mine + buf_off(s) + v * 16));
        *reinterpret_cast<uint4*>(out + v * 16) = acc.Finish(job.post_scale);
      }
      first = nvec * vec_elems;
    }
    for (size_t i = first + threadIdx.x; i < len; i += blockDim.x) {
      if (ELEM == ELEM_I32) {
        unsigned acc = 0;
        for (int s = 0; s < ctx.nranks; s++) acc += reinterpret_cast<const unsigned*>(mine + buf_off(s))[i];
        reinterpret_cast<unsigned*>(out)[i] = acc;
      } else {
        float acc = 0.f;
        for (int s = 0; s < ctx.nranks; s++) acc += LoadAsFloat<ELEM>(mine + buf_off(s), i);
        if (job.post_scale != 1.0f) acc *= job.post_scale;
        if (ELEM == ELEM_BF16) reinterpret_cast<unsigned short*>(out)[i] = FloatToBf16(acc);
        else reinterpret_cast<float*>(out)[i] = acc;
      }
    }
  }
  if (threadIdx.x == 0) atomicAdd(ctx.counters, 1ull);
  if (job.trailing_barrier) ChannelBarrier(ctx, channel, 3, epoch + 1, s_failed);
}

// ------------------------------------------------------------------------------------
template <int ELEM, int kUnrollLink = kZeroCopyUnrollLink>
__device__ void RunZeroCopy(const RankCtx& ctx, const JobArgs& job, int channel,
                            unsigned long long elems_per_channel, Epoch base, int* s_failed) {
  const int esz = ELEM == ELEM_BF16 ? 2 : 4;
  const size_t vec_elems = 16 / esz;
  const unsigned long long epoch = base + 1;
  SML_GEOMETRY_CHECK(ctx, channel, s_failed,
                     job.in_offset + job.numel * esz <= job.user_bytes &&
                     job.out_offset + job.numel * esz <= job.user_bytes);
  // Everybody's input must be complete before anybody reads it.
  if (!ChannelBarrier(ctx, channel, 0, epoch, s_failed)) return;

  unsigned long long c0 = static_cast<unsigned long long>(channel) * elems_per_channel;
  unsigned long long c1 = c0 + elems_per_channel;
  if (c1 > job.numel) c1 = job.numel;
  if (c0 < job.numel) {
    const size_t len = static_cast<size_t>(c1 - c0);
    size_t sb, se;
    ShardRange(len, ctx.nranks, ctx.rank, 128, &sb, &se);
    if (sb >= se) sb = se = 0;  // empty shard: nothing to do, and no unsigned wrap below
    // Whole vectors of my shard; the ragged end of the range (fewer than one vector, only
    // in the last channel) is done element-wise by the rank that owns the last shard.
    size_t full_end = se / vec_elems * vec_elems;
    if (se < len) full_end = se;  // interior shard boundaries are multiples of 128 elements
    if (full_end < sb) full_end = sb;
    const bool inplace = job.in_offset == job.out_offset;
    size_t in_base = job.in_offset + (c0 + sb) * esz;
    size_t out_base = job.out_offset + (c0 + sb) * esz;
    size_t nvec = (full_end - sb) / vec_elems;
    char* const* peers = job.user_peer;
    size_t v = threadIdx.x;
    for (; v + (kUnrollLink - 1) * blockDim.x < nvec; v += kUnrollLink * blockDim.x) {
      uint4 r[kUnrollLink];
#pragma unroll
      for (int u = 0; u < kUnrollLink; u++)
        r[u] = ReduceVec<ELEM>(ctx, peers, job.user_mc, in_base + (v + u * blockDim.x) * 16, job.post_scale);
#pragma unroll
      for (int u = 0; u < kUnrollLink; u++)
        BroadcastVec(ctx, peers, job.user_mc, out_base + (v + u * blockDim.x) * 16, r[u]);
    }
    if (v < nvec) {
      // The remainder, fewer than kUnrollLink * blockDim.x vectors: all in flight at once.
      uint4 r[kUnrollLink];
#pragma unroll
      for (int u = 0; u < kUnrollLink; u++)
        if (v + u * blockDim.x < nvec)
          r[u] = ReduceVec<ELEM>(ctx, peers, job.user_mc, in_base + (v + u * blockDim.x) * 16, job.post_scale);
#pragma unroll
      for (int u = 0; u < kUnrollLink; u++)
        if (v + u * blockDim.x < nvec)
          BroadcastVec(ctx, peers, job.user_mc, out_base + (v + u * blockDim.x) * 16, r[u]);
    }
    (void)inplace;
    // Ragged end: plain peer loads and stores, element by element.
    for (size_t i = full_end + threadIdx.x; i < se; i += blockDim.x) {
      size_t io = job.in_offset + (c0 + i) * esz, oo = job.out_offset + (c0 + i) * esz;
      if (ELEM == ELEM_I32) {
        unsigned acc = 0;
        for (int p = 0; p < ctx.nranks; p++) acc += __ldcg(reinterpret_cast<const unsigned*>(peers[p] + io));
        for (int p = 0; p < ctx.nranks; p++) *reinterpret_cast<unsigned*>(peers[p] + oo) = acc;
      } else if (ELEM == ELEM_F32) {
        float acc = 0.f;
        for (int p = 0; p < ctx.nranks; p++) acc += __ldcg(reinterpret_cast<const float*>(peers[p] + io));
        acc *= job.post_scale;
        for (int p = 0; p < ctx.nranks; p++) *reinterpret_cast<float*>(peers[p] + oo) = acc;
      } else {
        float acc = 0.f;
        for (int p = 0; p < ctx.nranks; p++) acc += Bf16ToFloat(__ldcg(reinterpret_cast<const unsigned short*>(peers[p] + io)));
        acc *= job.post_scale;
        unsigned short h = FloatToBf16(acc);
        for (int p = 0; p < ctx.nranks; p++) *reinterpret_cast<unsigned short*>(peers[p] + oo) = h;
      }
    }
    if (threadIdx.x == 0) atomicAdd(ctx.counters, 1ull);
  }
  // Nobody may return (and let its stream touch the output) before all shards landed.
  ChannelBarrier(ctx, channel, 1, epoch, s_failed);
}

// ------------------------------------------------------------------------------------
template <int ELEM, int MODE, int ALGO>
__device__ __forceinline__ void RunJob(const RankCtx& ctx, const JobArgs& job, int channel,
                                       unsigned long long epc, Epoch base, int* s_failed, float* s_sf) {
  // The quantising loader reads its input twice and meets its peers once more per tile,
  // so it gets more warps than the plain copy-in of the SUM modes (8-GPU measurements with
  // 1 GiB: 4/8/4 3.72 ms, 6/8/2 3.30 ms, 8/6/2 3.07 ms before the loader was vectorised).
  if (ALGO == ALGO_STAGED && MODE == MODE_QUANT)
    RunStaged<ELEM, MODE, 6, 8>(ctx, job, channel, epc, base, reinterpret_cast<StagedShared*>(s_failed), s_sf);
  else if (ALGO == ALGO_STAGED)
    RunStaged<ELEM, MODE>(ctx, job, channel, epc, base, reinterpret_cast<StagedShared*>(s_failed), s_sf);
  else if (ALGO == ALGO_PUSH)
    RunPush<ELEM, MODE>(ctx, job, channel, epc, base, reinterpret_cast<StagedShared*>(s_failed), s_sf);
  else if (ALGO == ALGO_ONESHOT) RunOneShot<ELEM, MODE>(ctx, job, channel, epc, base, s_failed);
  else if (ctx.use_multimem) RunZeroCopy<ELEM, kZeroCopyUnrollLink>(ctx, job, channel, epc, base, s_failed);
  else RunZeroCopy<ELEM, kZeroCopyUnrollPeer>(ctx, job, channel, epc, base, s_failed);
}

// Every channel keeps the epoch it has reached in device memory: read it when the kernel
// starts, advance it by the job's count when the kernel ends (on every path, also after a
// timeout, so that the ranks stay in step). Nothing about epochs is baked into the launch,
// which is what lets a captured launch be replayed.
#define SML_EPOCH_PROLOGUE(CTX, JOB, CHANNEL, ALGO)                       \
  __shared__ Epoch s_base;                                                \
  if (threadIdx.x == 0) {                                                 \
    s_state.failed = 0;                                                   \
    s_state.stored = 0;                                                   \
    s_state.done[0] = s_state.done[1] = s_state.done[2] = 0;              \
    s_state.ring_buffers = nullptr;                                       \
    if (((ALGO) == ALGO_STAGED || (ALGO) == ALGO_PUSH) && (JOB).bulk_copy) { \
      BulkRingInit(&s_state.ring[0]);                                     \
      BulkRingInit(&s_state.ring[1]);                                     \
      WarpStreamInit(&s_state.ws);                                        \
      s_state.ring_buffers = reinterpret_cast<char*>(s_dyn);              \
    }                                                                     \
    s_base = (CTX).epoch_words[CHANNEL];                                  \
  }                                                                       \
  __syncthreads();
#define SML_EPOCH_EPILOGUE(CTX, JOB, CHANNEL)                             \
  __syncthreads();                                                        \
  if (threadIdx.x == 0) (CTX).epoch_words[CHANNEL] = s_base + (JOB).epochs;

// Dynamic shared memory of the streaming kernels: the two TMA copy rings.
extern __shared__ __align__(128) unsigned char s_dyn[];

template <int ALGO>
constexpr size_t DynamicSmemBytes() {
  return (ALGO == ALGO_STAGED || ALGO == ALGO_PUSH) ? kLoaderSmemOffset + kLoaderSmemBytes : 0;
}

template <int ELEM, int MODE, int ALGO>
__global__ void __launch_bounds__(kThreads, 1)
AllReduceKernel(const RankCtx ctx, const JobArgs job, unsigned long long epc) {
  __shared__ StagedShared s_state;
  __shared__ float s_sf[(MODE == MODE_QUANT && (ALGO == ALGO_STAGED || ALGO == ALGO_PUSH)) ? kMaxBlocksPerSlot : 1];
  SML_EPOCH_PROLOGUE(ctx, job, blockIdx.x, ALGO)
  RunJob<ELEM, MODE, ALGO>(ctx, job, blockIdx.x, epc, s_base, &s_state.failed, s_sf);
  SML_EPOCH_EPILOGUE(ctx, job, blockIdx.x)
}

// All ranks in one grid: blockIdx.y selects the rank whose role this CTA plays.
template <int ELEM, int MODE, int ALGO>
__global__ void __launch_bounds__(kThreads, 1)
AllReduceEmuKernel(const RankCtx* ctxs, const JobArgs* jobs, unsigned long long epc) {
  __shared__ StagedShared s_state;
  __shared__ float s_sf[(MODE == MODE_QUANT && (ALGO == ALGO_STAGED || ALGO == ALGO_PUSH)) ? kMaxBlocksPerSlot : 1];
  __shared__ RankCtx s_ctx;
  __shared__ JobArgs s_job;
  if (threadIdx.x == 0) {
    s_ctx = ctxs[blockIdx.y];
    s_job = jobs[blockIdx.y];
  }
  __syncthreads();
  SML_EPOCH_PROLOGUE(s_ctx, s_job, blockIdx.x, ALGO)
  RunJob<ELEM, MODE, ALGO>(s_ctx, s_job, blockIdx.x, epc, s_base, &s_state.failed, s_sf);
  SML_EPOCH_EPILOGUE(s_ctx, s_job, blockIdx.x)
}

// The sum over a single worker, out of place: one pass over the data, no staging.
__global__ void __launch_bounds__(kThreads) LocalCopyKernel(const char* in, char* out, size_t bytes) {
  const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t nthreads = static_cast<size_t>(gridDim.x) * blockDim.x;
  if (Aligned16(in) && Aligned16(out)) {
    const size_t nvec = bytes / 16;
    const uint4* s = reinterpret_cast<const uint4*>(in);
    uint4* d = reinterpret_cast<uint4*>(out);
    size_t i = tid;
    for (; i + (kUnroll - 1) * nthreads < nvec; i += kUnroll * nthreads) {
      uint4 v[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; u++) v[u] = s[i + u * nthreads];
#pragma unroll
      for (int u = 0; u < kUnroll; u++) d[i + u * nthreads] = v[u];
    }
    for (; i < nvec; i += nthreads) d[i] = s[i];
    for (size_t b = nvec * 16 + tid; b < bytes; b += nthreads) out[b] = in[b];
  } else {
    for (size_t b = tid; b < bytes; b += nthreads) out[b] = in[b];
  }
}

// The exact mode with a single worker: nothing to exchange, so the round trip through the
// fixed-point grid (block maximum -> exponent -> int32 -> float32, exactly what one worker
// contributes and receives) is one pass over the data: every warp takes chunks of 1024
// elements, 8 float4 per lane, finds its blocks' maxima with shuffles and writes the result.
// Bit-identical to the streaming kernels and to the CPU oracle.
__global__ void __launch_bounds__(kThreads)
LocalQuantKernel(const float* in, float* out, size_t numel, int block_numel, float quant_base, float post_scale) {
  const int lane = threadIdx.x & 31;
  const size_t warp = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const size_t nwarps = (static_cast<size_t>(gridDim.x) * blockDim.x) >> 5;
  const size_t B = block_numel;
  const size_t whole = numel / B * B;     // elements in blocks without a ragged end
  const size_t nchunks = whole / 1024;    // 1024 is a multiple of every block size
  const float4* in4 = reinterpret_cast<const float4*>(in);
  float4* out4 = reinterpret_cast<float4*>(out);
  for (size_t c = warp; c < nchunks; c += nwarps) {
    float4 x[8];
    float m[8];
#pragma unroll
    for (int u = 0; u < 8; u++) x[u] = in4[c * 256 + u * 32 + lane];
#pragma unroll
    for (int u = 0; u < 8; u++) m[u] = fmaxf(fmaxf(fabsf(x[u].x), fabsf(x[u].y)), fmaxf(fabsf(x[u].z), fabsf(x[u].w)));
    if (B < 128) {
      const int g = static_cast<int>(B / 4);  // lanes per block
#pragma unroll
      for (int u = 0; u < 8; u++)
        for (int o = g >> 1; o > 0; o >>= 1) m[u] = fmaxf(m[u], __shfl_xor_sync(0xffffffffu, m[u], o));
    } else {
      const int rows = static_cast<int>(B / 128);  // rows of 128 elements per block: 1, 2, 4 or 8
#pragma unroll
      for (int span = 1; span < 8; span <<= 1) {
        if (span < rows) {
#pragma unroll
          for (int u = 0; u + span < 8; u += 2 * span) m[u] = fmaxf(m[u], m[u + span]);
        }
      }
#pragma unroll
      for (int u = 0; u < 8; u++) {
        if ((u % rows) != 0) continue;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m[u] = fmaxf(m[u], __shfl_xor_sync(0xffffffffu, m[u], o));
      }
      // hand every block's maximum back to all of its rows
#pragma unroll
      for (int span = 4; span >= 1; span >>= 1) {
        if (span < rows) {
#pragma unroll
          for (int u = 0; u + span < 8; u += 2 * span) m[u + span] = m[u];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 8; u++) {
      const float f = quant::ScaleFactorFromBase(quant::LocalExponent(m[u]), quant_base);
      float4 y;
      y.x = quant::Dequantize(quant::Quantize(x[u].x, f), f) * post_scale;
      y.y = quant::Dequantize(quant::Quantize(x[u].y, f), f) * post_scale;
      y.z = quant::Dequantize(quant::Quantize(x[u].z, f), f) * post_scale;
      y.w = quant::Dequantize(quant::Quantize(x[u].w, f), f) * post_scale;
      out4[c * 256 + u * 32 + lane] = y;
    }
  }
  // What is left: fewer than 1024 elements of whole blocks and a ragged last block, one
  // block per warp.
  const size_t nblocks = (numel + B - 1) / B;
  for (size_t b = nchunks * (1024 / B) + warp; b < nblocks; b += nwarps) {
    const size_t base = b * B, n = numel - base < B ? numel - base : B;
    float mx = 0.f;
    for (size_t i = lane; i < n; i += 32) mx = fmaxf(mx, fabsf(in[base + i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float f = quant::ScaleFactorFromBase(quant::LocalExponent(mx), quant_base);
    for (size_t i = lane; i < n; i += 32) out[base + i] = quant::Dequantize(quant::Quantize(in[base + i], f), f) * post_scale;
  }
}

// uint8 -> int32 (zero extended) and back (low byte kept, i.e. the sum modulo 256): uint8
// tensors make the trip as int32. 16 elements per thread and step when the byte side is
// 16-byte aligned (the int32 side is scratch memory and always is), else one by one.
__global__ void __launch_bounds__(kThreads) WidenU8Kernel(const unsigned char* in, int* out, size_t n) {
  const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t nthreads = static_cast<size_t>(gridDim.x) * blockDim.x;
  size_t done = 0;
  if (Aligned16(in) && Aligned16(out)) {
    const size_t nvec = n / 16;
    const uint4* s = reinterpret_cast<const uint4*>(in);
    int4* d = reinterpret_cast<int4*>(out);
    for (size_t i = tid; i < nvec; i += nthreads) {
      const uint4 v = s[i];
      const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int k = 0; k < 4; k++)
        d[4 * i + k] = make_int4(w[k] & 0xff, (w[k] >> 8) & 0xff, (w[k] >> 16) & 0xff, w[k] >> 24);
    }
    done = nvec * 16;
  }
  for (size_t i = done + tid; i < n; i += nthreads) out[i] = in[i];
}

__global__ void __launch_bounds__(kThreads) NarrowI32Kernel(const int* in, unsigned char* out, size_t n) {
  const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t nthreads = static_cast<size_t>(gridDim.x) * blockDim.x;
  size_t done = 0;
  if (Aligned16(in) && Aligned16(out)) {
    const size_t nvec = n / 16;
    const int4* s = reinterpret_cast<const int4*>(in);
    uint4* d = reinterpret_cast<uint4*>(out);
    for (size_t i = tid; i < nvec; i += nthreads) {
      unsigned w[4];
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const int4 v = s[4 * i + k];
        w[k] = (v.x & 0xff) | ((v.y & 0xff) << 8) | ((v.z & 0xff) << 16) | (static_cast<unsigned>(v.w) << 24);
      }
      d[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    done = nvec * 16;
  }
  for (size_t i = done + tid; i < n; i += nthreads) out[i] = static_cast<unsigned char>(in[i]);
}

__global__ void WaitProbeKernel(const RankCtx ctx) {
  __shared__ int s_failed;
  if (threadIdx.x == 0) s_failed = 0;
  __syncthreads();
  // Waits, without signalling, for an epoch that no job ever reaches.
  ChannelBarrier(ctx, kMaxChannels - 1, kNumPhases - 1, ~0ull, &s_failed, false);
}

template <int ELEM, int MODE, int ALGO>
cudaError_t LaunchOne(const RankCtx& ctx, const JobArgs& job, const LaunchPlan& plan,
                      cudaStream_t stream) {
  constexpr size_t dyn = DynamicSmemBytes<ALGO>();
  if (dyn > 0) {
    cudaError_t e = cudaFuncSetAttribute(AllReduceKernel<ELEM, MODE, ALGO>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(dyn));
    if (e != cudaSuccess) return e;
  }
  AllReduceKernel<ELEM, MODE, ALGO><<<plan.channels, kThreads, dyn, stream>>>(ctx, job, plan.elems_per_channel);
  return cudaGetLastError();
}

template <int ELEM, int MODE, int ALGO>
cudaError_t LaunchOneEmu(const RankCtx* ctxs, const JobArgs* jobs, int nranks,
                         const LaunchPlan& plan, cudaStream_t stream) {
  unsigned long long epc = plan.elems_per_channel;
  void* args[] = {&ctxs, &jobs, &epc};
  dim3 grid(plan.channels, nranks);
  // Cooperative launch: the runtime refuses the launch unless all CTAs can be resident
  // together, which the cross-"rank" barriers need.
  constexpr size_t dyn = DynamicSmemBytes<ALGO>();
  if (dyn > 0) {
    cudaError_t e = cudaFuncSetAttribute(AllReduceEmuKernel<ELEM, MODE, ALGO>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(dyn));
    if (e != cudaSuccess) return e;
  }
  return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(AllReduceEmuKernel<ELEM, MODE, ALGO>),
                                     grid, dim3(kThreads), args, dyn, stream);
}

#define SML_DISPATCH(FN, elem, mode, algo, ...)                                             \
  do {                                                                                      \
    if ((algo) == ALGO_ZEROCOPY) {                                                          \
      if ((mode) != MODE_SUM) return cudaErrorInvalidValue;                                 \
      if ((elem) == ELEM_F32) return FN<ELEM_F32, MODE_SUM, ALGO_ZEROCOPY>(__VA_ARGS__);    \
      if ((elem) == ELEM_I32) return FN<ELEM_I32, MODE_SUM, ALGO_ZEROCOPY>(__VA_ARGS__);    \
      return FN<ELEM_BF16, MODE_SUM, ALGO_ZEROCOPY>(__VA_ARGS__);                           \
    }                                                                                       \
    if ((algo) == ALGO_PUSH) {                                                              \
      if ((elem) == ELEM_I32) return FN<ELEM_I32, MODE_SUM, ALGO_PUSH>(__VA_ARGS__);        \
      if ((elem) == ELEM_F32 && (mode) == MODE_QUANT) return FN<ELEM_F32, MODE_QUANT, ALGO_PUSH>(__VA_ARGS__); \
      if ((elem) == ELEM_F32) return FN<ELEM_F32, MODE_SUM, ALGO_PUSH>(__VA_ARGS__);        \
      if ((mode) == MODE_QUANT) return FN<ELEM_BF16, MODE_QUANT, ALGO_PUSH>(__VA_ARGS__);   \
      return FN<ELEM_BF16, MODE_SUM, ALGO_PUSH>(__VA_ARGS__);                               \
    }                                                                                       \
    if ((elem) == ELEM_I32) {                                                               \
      if ((algo) == ALGO_STAGED) return FN<ELEM_I32, MODE_SUM, ALGO_STAGED>(__VA_ARGS__);   \
      return FN<ELEM_I32, MODE_SUM, ALGO_ONESHOT>(__VA_ARGS__);                             \
    }                                                                                       \
    if ((elem) == ELEM_F32) {                                                               \
      if ((mode) == MODE_QUANT) {                                                           \
        if ((algo) == ALGO_STAGED) return FN<ELEM_F32, MODE_QUANT, ALGO_STAGED>(__VA_ARGS__); \
        return FN<ELEM_F32, MODE_QUANT, ALGO_ONESHOT>(__VA_ARGS__);                         \
      }                                                                                     \
      if ((algo) == ALGO_STAGED) return FN<ELEM_F32, MODE_SUM, ALGO_STAGED>(__VA_ARGS__);   \
      return FN<ELEM_F32, MODE_SUM, ALGO_ONESHOT>(__VA_ARGS__);                             \
    }                                                                                       \
    if ((mode) == MODE_QUANT) {                                                             \
      if ((algo) == ALGO_STAGED) return FN<ELEM_BF16, MODE_QUANT, ALGO_STAGED>(__VA_ARGS__); \
      return FN<ELEM_BF16, MODE_QUANT, ALGO_ONESHOT>(__VA_ARGS__);                          \
    }                                                                                       \
    if ((algo) == ALGO_STAGED) return FN<ELEM_BF16, MODE_SUM, ALGO_STAGED>(__VA_ARGS__);    \
    return FN<ELEM_BF16, MODE_SUM, ALGO_ONESHOT>(__VA_ARGS__);                              \
  } while (0)

}  // namespace

bool DeviceMemory(const void* p) {
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return at.type == cudaMemoryTypeDevice;
}

size_t SlotElems(const RankCtx& ctx, int elem_type, int mode) {
  if (mode == MODE_QUANT && elem_type == ELEM_BF16) {
    // int32 payload and, behind it, the bf16 results (they travel as bf16: half the return leg)
    const size_t unit = static_cast<size_t>(ctx.nranks) * (ctx.block_numel > 128 ? ctx.block_numel : 128);
    const size_t cap = ctx.slot_bytes / 6 / unit * unit;
    return cap > 0 ? cap : unit;  // a slot of one unit (the configured minimum) keeps float32 results instead
  }
  int st_esz = mode == MODE_QUANT ? 4 : (elem_type == ELEM_BF16 ? 2 : 4);
  return ctx.slot_bytes / st_esz;
}

size_t PushTileCapacity(const RankCtx& ctx, int elem_type, int mode) {
  const size_t n = ctx.nranks;
  if (n < 2) return 0;
  const size_t in_esz = elem_type == ELEM_BF16 ? 2 : 4;
  const size_t leg_in = mode == MODE_QUANT ? 4 : in_esz;                                // reduce leg
  const size_t leg_out = mode == MODE_QUANT ? (elem_type == ELEM_BF16 ? 2 : 4) : in_esz;  // result leg
  // (n-1) receive areas + (n-1) result areas of tile/n elements each
  size_t cap = ctx.slot_bytes * n / ((n - 1) * (leg_in + leg_out));
  if (mode == MODE_QUANT) {
    const size_t by_words = ctx.slot_bytes / 4;  // one exponent word per block of the slot
    if (cap > by_words) cap = by_words;
  }
  const size_t unit = n * (ctx.block_numel > 128 ? ctx.block_numel : 128);
  const size_t stream_unit = n * (kWsChunk / 4);  // shards of whole TMA chunks where the slot allows it
  if (cap >= stream_unit) return cap / stream_unit * stream_unit;
  return cap / unit * unit;
}

size_t StagingBytes(size_t slot_bytes, int slots_per_channel, int block_numel, int max_channels,
                    size_t oneshot_bytes, int nranks, size_t* data_offset, size_t* exp_offset,
                    size_t* oneshot_offset) {
  auto align = [](size_t x) { return (x + 4095) / 4096 * 4096; };
  size_t flags = size_t(kMaxChannels) * kFlagWordsPerChannel * 8;
  size_t off = align(flags);
  *exp_offset = off;
  size_t blocks_per_slot = slot_bytes / 4 / block_numel;
  off = align(off + size_t(max_channels) * ExpRingDepth(slots_per_channel) * blocks_per_slot * kExpWordBytes);
  *oneshot_offset = off;
  off = align(off + 3 * size_t(nranks) * oneshot_bytes);  // two alternating sets + one for captured launches
  *data_offset = off;
  off = align(off + size_t(max_channels) * slots_per_channel * slot_bytes);
  return off;
}

bool CheckedBuild() {
#ifdef SWITCHML_CHECKED
  return true;
#else
  return false;
#endif
}

size_t ReportedStageBytes(size_t actual) {
#ifdef SWITCHML_CHECKED
  const char* e = getenv("SWITCHML_CHECKED_PRETEND_STAGE_BYTES");
  if (e && *e) return static_cast<size_t>(strtoull(e, nullptr, 0));
#endif
  return actual;
}

LaunchPlan PlanLaunch(const RankCtx& ctx, const JobArgs& job, int requested_channels,
                      int max_channels) {
  LaunchPlan p;
  const unsigned long long numel = job.numel ? job.numel : 1;
  if (max_channels > kMaxChannels) max_channels = kMaxChannels;
  p.tile_elems = 0;
  if (job.algo == ALGO_STAGED || job.algo == ALGO_PUSH) {
    size_t slot_elems = job.algo == ALGO_PUSH ? PushTileCapacity(ctx, job.elem_type, job.mode)
                                              : SlotElems(ctx, job.elem_type, job.mode);
    int ch = requested_channels > 0 ? requested_channels : max_channels;
    if (ch > max_channels) ch = max_channels;
    // Tile: a slot for big jobs; for smaller ones shrink it so that the job still spreads
    // over all channels and every channel has about four tiles to pipeline (loader, reducer
    // and storer then work on different tiles at the same time), but not below 16 Ki elements
    // (the cost of meeting the peers would dominate).
    unsigned long long unit = static_cast<unsigned long long>(ctx.nranks) *
                              (ctx.block_numel > 128 ? ctx.block_numel : 128);
    unsigned long long tile = (numel + 4ull * ch - 1) / (4ull * ch);
    if (tile < 16384) tile = 16384;
    tile = (tile + unit - 1) / unit * unit;
    if (tile > slot_elems) tile = slot_elems;
    p.tile_elems = tile;
    unsigned long long tiles = (numel + tile - 1) / tile;
    if (static_cast<unsigned long long>(ch) > tiles) ch = static_cast<int>(tiles);
    unsigned long long tiles_per_channel = (tiles + ch - 1) / ch;
    p.elems_per_channel = tiles_per_channel * tile;
    p.channels = static_cast<int>((numel + p.elems_per_channel - 1) / p.elems_per_channel);
    p.epochs = static_cast<unsigned>(tiles_per_channel);
    p.tiles = tiles;
  } else if (job.algo == ALGO_ONESHOT) {
    // Whole quantisation blocks per channel; a few CTAs are enough for small messages.
    unsigned long long unit = ctx.block_numel > 128 ? ctx.block_numel : 128;
    unsigned long long units = (numel + unit - 1) / unit;
    // A few CTAs are enough for small messages; from 256 Ki elements on every SM takes part.
    int ch = requested_channels > 0 ? requested_channels : (numel >= (256u << 10) ? max_channels : 64);
    if (ch > max_channels) ch = max_channels;
    unsigned long long per = (units + ch - 1) / ch;
    unsigned long long min_per = (4096 + unit - 1) / unit;  // at least 4 Ki elements per CTA
    if (per < min_per) per = min_per;
    p.elems_per_channel = per * unit;
    p.channels = static_cast<int>((numel + p.elems_per_channel - 1) / p.elems_per_channel);
    p.epochs = 1;
    p.tiles = p.channels;
  } else {
    // Ranges are multiples of nranks*128 elements so that interior shard boundaries stay
    // vector aligned.
    unsigned long long unit = 128ull * ctx.nranks;
    unsigned long long units = (numel + unit - 1) / unit;
    int ch = requested_channels > 0 ? requested_channels : max_channels;
    if (ch > max_channels) ch = max_channels;
    unsigned long long per = (units + ch - 1) / ch;
    unsigned long long min_per = (64 * 1024) / (128 * 4);  // >= 64 KiB per shard-range
    if (per < min_per) per = min_per;
    p.elems_per_channel = per * unit;
    p.channels = static_cast<int>((numel + p.elems_per_channel - 1) / p.elems_per_channel);
    p.epochs = 1;
    p.tiles = p.channels;
  }
  if (p.channels < 1) p.channels = 1;
  return p;
}

cudaError_t LaunchAllReduce(const RankCtx& ctx, const JobArgs& job, const LaunchPlan& plan,
                            cudaStream_t stream) {
  if (ctx.nranks < 1 || ctx.nranks > kMaxRanks || plan.channels > kMaxChannels)
    return cudaErrorInvalidValue;
  SML_DISPATCH(LaunchOne, job.elem_type, job.mode, job.algo, ctx, job, plan, stream);
}

cudaError_t LaunchAllReduceEmulated(const RankCtx* ctxs_dev, const JobArgs* jobs_dev,
                                    const JobArgs& job0, int nranks, const LaunchPlan& plan,
                                    cudaStream_t stream) {
  if (nranks < 1 || nranks > kMaxRanks || plan.channels > kMaxChannels) return cudaErrorInvalidValue;
  SML_DISPATCH(LaunchOneEmu, job0.elem_type, job0.mode, job0.algo, ctxs_dev, jobs_dev, nranks, plan, stream);
}

cudaError_t LaunchLocalCopy(const void* in, void* out, size_t bytes, cudaStream_t stream) {
  if (bytes == 0 || in == out) return cudaSuccess;
  int blocks = 148 * 4;
  LocalCopyKernel<<<blocks, kThreads, 0, stream>>>(static_cast<const char*>(in), static_cast<char*>(out), bytes);
  return cudaGetLastError();
}

cudaError_t LaunchLocalQuant(const void* in, void* out, size_t numel, int block_numel, float quant_base,
                             float post_scale, cudaStream_t stream) {
  if (numel == 0) return cudaSuccess;
  if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) return cudaErrorInvalidValue;
  size_t want = (numel / 1024 + kThreads / 32 - 1) / (kThreads / 32);  // one chunk per warp and turn
  if (want < 1) want = 1;
  const int blocks = static_cast<int>(want < 148 * 4 ? want : 148 * 4);
  LocalQuantKernel<<<blocks, kThreads, 0, stream>>>(static_cast<const float*>(in), static_cast<float*>(out), numel,
                                                   block_numel, quant_base, post_scale);
  return cudaGetLastError();
}

static int ElementwiseBlocks(size_t n) {
  size_t want = (n / 16 + kThreads - 1) / kThreads;
  if (want < 1) want = 1;
  return static_cast<int>(want < 148 * 8 ? want : 148 * 8);
}

cudaError_t LaunchWidenU8(const void* in, void* out, size_t numel, cudaStream_t stream) {
  if (numel == 0) return cudaSuccess;
  WidenU8Kernel<<<ElementwiseBlocks(numel), kThreads, 0, stream>>>(static_cast<const unsigned char*>(in),
                                                                  static_cast<int*>(out), numel);
  return cudaGetLastError();
}

cudaError_t LaunchNarrowI32(const void* in, void* out, size_t numel, cudaStream_t stream) {
  if (numel == 0) return cudaSuccess;
  NarrowI32Kernel<<<ElementwiseBlocks(numel), kThreads, 0, stream>>>(static_cast<const int*>(in),
                                                                    static_cast<unsigned char*>(out), numel);
  return cudaGetLastError();
}

cudaError_t LaunchWaitProbe(const RankCtx& ctx, cudaStream_t stream) {
  WaitProbeKernel<<<1, 32, 0, stream>>>(ctx);
  return cudaGetLastError();
}

}  // namespace kernels
}  // namespace switchml

// ---------------------------------------------------------------------------------------
// Allocation-free single-worker entry point; see kernels/local_noalloc.h for the contract.
#include <mutex>

#include "kernels/local_noalloc.h"

namespace {

// Geometry small enough for a static array: 8 channels x 2 slots x 32 KiB.
const int kNoAllocChannels = 8;
const int kNoAllocSlots = 2;
const size_t kNoAllocSlotBytes = 32768;
const size_t kNoAllocAuxOffset = 896u << 10;  // counters and status word behind the staging (at most 772 KiB, with blocks of 32)

// Scratch of the allocation-free entry point. In host code this name is only a handle for
// cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[SWITCHML_NOALLOC_SCRATCH_BYTES];

std::mutex g_noalloc_mu;
void* g_noalloc_ptr[64] = {nullptr};  // per device: device address of g_noalloc_scratch

}  // namespace

// Device address of the scratch array on `dev` (the current device). Once per device, with
// that device current: ask the runtime where the array lives. Caller holds g_noalloc_mu.
static char* NoAllocScratch(int dev) {
  if (!g_noalloc_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) return nullptr;
    g_noalloc_ptr[dev] = p;
  }
  return static_cast<char*>(g_noalloc_ptr[dev]);
}

extern "C" int switchml_noalloc_last_status(void* stream_ptr, int* status) {
  if (!status) return SWITCHML_NOALLOC_BAD_ARGUMENT;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return SWITCHML_NOALLOC_CUDA_ERROR;
  char* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    scratch = NoAllocScratch(dev);
  }
  if (!scratch) return SWITCHML_NOALLOC_CUDA_ERROR;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  int word = 0;
  if (cudaMemcpyAsync(&word, scratch + kNoAllocAuxOffset + 256, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
      cudaStreamSynchronize(stream) != cudaSuccess)
    return SWITCHML_NOALLOC_CUDA_ERROR;
  *status = word;
  return SWITCHML_NOALLOC_OK;
}

extern "C" const char* switchml_noalloc_strerror(int code) {
  switch (code) {
    case SWITCHML_NOALLOC_OK: return "ok";
    case SWITCHML_NOALLOC_BAD_ARGUMENT:
      return "bad argument: null pointer, unknown elem_type/mode, int32 with quantised mode, or "
             "block_numel not a power of two in [32,1024]";
    case SWITCHML_NOALLOC_TOO_LARGE:
      return "numel exceeds SWITCHML_NOALLOC_MAX_NUMEL (2^26 elements)";
    case SWITCHML_NOALLOC_CUDA_ERROR: return "a CUDA call failed (see cudaGetLastError)";
  }
  return "unknown code";
}

extern "C" int switchml_local_allreduce_noalloc(const void* in, void* out,
                                                unsigned long long numel, int elem_type, int mode,
                                                int block_numel, void* stream_ptr) {
  using namespace switchml::kernels;
  if (!in || !out) return SWITCHML_NOALLOC_BAD_ARGUMENT;
  if (elem_type < ELEM_F32 || elem_type > ELEM_BF16) return SWITCHML_NOALLOC_BAD_ARGUMENT;
  if (mode != MODE_SUM && mode != MODE_QUANT) return SWITCHML_NOALLOC_BAD_ARGUMENT;
  if (elem_type == ELEM_I32 && mode == MODE_QUANT) return SWITCHML_NOALLOC_BAD_ARGUMENT;
  if (block_numel < 32 || block_numel > 1024 || (block_numel & (block_numel - 1)))
    return SWITCHML_NOALLOC_BAD_ARGUMENT;
  if (numel > SWITCHML_NOALLOC_MAX_NUMEL) return SWITCHML_NOALLOC_TOO_LARGE;
  if (numel == 0) return SWITCHML_NOALLOC_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);

  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return SWITCHML_NOALLOC_CUDA_ERROR;
  // Held until the call's three enqueues (two clears and the kernel) are on the stream, so
  // that host threads calling at the same time cannot interleave them.
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  char* scratch = NoAllocScratch(dev);
  if (!scratch) return SWITCHML_NOALLOC_CUDA_ERROR;

  RankCtx ctx;
  memset(&ctx, 0, sizeof(ctx));
  ctx.rank = 0;
  ctx.nranks = 1;
  ctx.use_multimem = 0;
  ctx.stage_peer[0] = scratch;
  ctx.slot_bytes = kNoAllocSlotBytes;
  ctx.slots_per_channel = kNoAllocSlots;
  ctx.sc_fence = 1;
  ctx.exp_ring = ExpRingDepth(kNoAllocSlots);
  ctx.exp_lookahead = ExpLookahead(kNoAllocSlots, kDefaultExpLookahead);
  ctx.block_numel = block_numel;
  ctx.oneshot_bytes = 256;
  ctx.timeout_ns = 1000000000ull;
  ctx.quant_base = switchml::quant::QuantBase(1);
  size_t staging = StagingBytes(ctx.slot_bytes, ctx.slots_per_channel, ctx.block_numel,
                                kNoAllocChannels, ctx.oneshot_bytes, 1, &ctx.data_offset,
                                &ctx.exp_offset, &ctx.oneshot_offset);
  if (staging > kNoAllocAuxOffset) return SWITCHML_NOALLOC_BAD_ARGUMENT;  // cannot happen for the limits above
  ctx.stage_bytes = staging;
  ctx.counters = reinterpret_cast<unsigned long long*>(scratch + kNoAllocAuxOffset);
  ctx.status = reinterpret_cast<int*>(scratch + kNoAllocAuxOffset + 256);
  ctx.epoch_words = reinterpret_cast<unsigned long long*>(scratch + kNoAllocAuxOffset + 320);  // 8 channels

  JobArgs job;
  memset(&job, 0, sizeof(job));
  job.in = in;
  job.out = out;
  job.numel = numel;
  job.elem_type = elem_type;
  job.mode = mode;
  job.algo = ALGO_STAGED;
  job.post_scale = 1.0f;
  job.bulk_copy = DeviceMemory(in) && DeviceMemory(out);
  LaunchPlan plan = PlanLaunch(ctx, job, 0, kNoAllocChannels);
  job.tile_elems = plan.tile_elems;
  job.epochs = plan.epochs;

  // The array keeps the previous call's flags (epochs), exponent words (tagged with epochs)
  // and counters; this call counts its epochs from zero again, so all three have to be
  // cleared first, in stream order. Flags and exponent words are neighbours.
  if (cudaMemsetAsync(scratch, 0, ctx.oneshot_offset, stream) != cudaSuccess) return SWITCHML_NOALLOC_CUDA_ERROR;
  if (cudaMemsetAsync(scratch + kNoAllocAuxOffset, 0, 512, stream) != cudaSuccess)
    return SWITCHML_NOALLOC_CUDA_ERROR;
  if (LaunchAllReduce(ctx, job, plan, stream) != cudaSuccess) return SWITCHML_NOALLOC_CUDA_ERROR;
  return SWITCHML_NOALLOC_OK;
}
