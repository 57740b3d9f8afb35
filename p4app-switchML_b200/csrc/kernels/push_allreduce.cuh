// ALGO_PUSH — the streaming pipeline for peer-memory transport (no in-switch reduction),
// built from posted stores only: nothing on the critical path waits for a load to come back
// over NVLink.
//
// Per tile, with n ranks and the tile cut into n shards (rank r owns shard r):
//   loader   pushes shard p of its own input straight from the user's tensor into the
//            receive area of owner p's slot (quantised to int32 on the way in MODE_QUANT);
//            its own shard is not copied anywhere                              [phase 1]
//   reducer  adds its own shard (read from the user's tensor) and the n-1 received copies,
//            all local reads; writes the result into its own output and pushes it into the
//            result area of every peer's slot, or, when the output lies in symmetric
//            memory, into every peer's output itself                            [phase 2]
//   storer   copies the n-1 received result shards from the slot to the output   [phase 3]
// Compared with copying whole tiles into and out of the slot (ALGO_STAGED without
// multicast) every element makes one trip less through local memory on the way in, the
// owner's 1/n never touches the slot, and NVLink carries stores only: (n-1)/n of the
// message out for the reduce leg and the same for the result leg, the traffic of a
// reduce-scatter + all-gather.
//
// Flow control (epochs only grow; e(k) = base + k + 1 for tile k, S slots per channel):
//   * a loader may overwrite a peer's receive area of slot k % S once that peer's reducer is
//     done with tile k - S: phase 2 >= e(k - S) from everybody;
//   * a reducer may overwrite a peer's result area once that peer's storer is done with
//     tile k - S: phase 3 >= e(k - S) from everybody;
//   * MODE_QUANT: the exponent words of tile k+A (slot (k+A) % E of a ring of E exponent slots;
//     A tiles of lookahead, none with a single data slot) are published while tile k is pushed;
//     their previous user is tile k+A-E, consumed by every loader before its phase-1 signal of
//     that tile; the publishing loader has awaited phase 1 >= e(k - A) by then, and E >= 2A.
// Between jobs nothing extra is needed: a rank's kernel ends after its storer has seen
// every peer's phase 2 for every tile (their reducers are done with all receive areas), and
// a result is pushed only after the peer's loader of the new job has signalled, i.e. after
// the peer's previous kernel (storer included) has ended.
#ifndef SWITCHML_PUSH_ALLREDUCE_CUH_
#define SWITCHML_PUSH_ALLREDUCE_CUH_

namespace switchml {
namespace kernels {
namespace {

static const int kPushUnroll = 8;  // 16-byte vectors in flight per thread

// Index of source rank `s` among the n-1 areas that destination `d` keeps (s != d).
__device__ __forceinline__ int PushAreaIndex(int s, int d) { return s < d ? s : s - 1; }

// Four consecutive elements of the input as floats (f32: one 16-byte load, bf16: 8 bytes).
template <int ELEM>
__device__ __forceinline__ float4 LoadGroupAsFloat(const char* in, size_t group) {
  if (ELEM == ELEM_BF16) {
    uint2 u = *reinterpret_cast<const uint2*>(in + group * 8);
    float2 a = Bf16x2ToFloat2(u.x), b = Bf16x2ToFloat2(u.y);
    return make_float4(a.x, a.y, b.x, b.y);
  }
  return *reinterpret_cast<const float4*>(in + group * 16);
}

// 16-byte vector accumulators of the plain-sum mode.
template <int ELEM> struct VecAcc;
template <> struct VecAcc<ELEM_F32> {
  float4 a;
  __device__ __forceinline__ void Init(uint4 v) { a = make_float4(__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w)); }
  __device__ __forceinline__ void Add(uint4 v) { a.x += __uint_as_float(v.x); a.y += __uint_as_float(v.y); a.z += __uint_as_float(v.z); a.w += __uint_as_float(v.w); }
  __device__ __forceinline__ uint4 Finish(float s) {
    if (s != 1.0f) { a.x *= s; a.y *= s; a.z *= s; a.w *= s; }
    return make_uint4(__float_as_uint(a.x), __float_as_uint(a.y), __float_as_uint(a.z), __float_as_uint(a.w));
  }
};
template <> struct VecAcc<ELEM_I32> {
  uint4 a;
  __device__ __forceinline__ void Init(uint4 v) { a = v; }
  __device__ __forceinline__ void Add(uint4 v) { a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w; }  // wrapping
  __device__ __forceinline__ uint4 Finish(float) { return a; }
};
template <> struct VecAcc<ELEM_BF16> {
  float a[8];
  __device__ __forceinline__ void Init(uint4 v) {
    float2 q;
    q = Bf16x2ToFloat2(v.x); a[0] = q.x; a[1] = q.y;
    q = Bf16x2ToFloat2(v.y); a[2] = q.x; a[3] = q.y;
    q = Bf16x2ToFloat2(v.z); a[4] = q.x; a[5] = q.y;
    q = Bf16x2ToFloat2(v.w); a[6] = q.x; a[7] = q.y;
  }
  __device__ __forceinline__ void Add(uint4 v) {
    float2 q;
    q = Bf16x2ToFloat2(v.x); a[0] += q.x; a[1] += q.y;
    q = Bf16x2ToFloat2(v.y); a[2] += q.x; a[3] += q.y;
    q = Bf16x2ToFloat2(v.z); a[4] += q.x; a[5] += q.y;
    q = Bf16x2ToFloat2(v.w); a[6] += q.x; a[7] += q.y;
  }
  __device__ __forceinline__ uint4 Finish(float s) {
    if (s != 1.0f) {
#pragma unroll
      for (int j = 0; j < 8; j++) a[j] *= s;
    }
    return make_uint4(Float2ToBf16x2(a[0], a[1]), Float2ToBf16x2(a[2], a[3]), Float2ToBf16x2(a[4], a[5]),
                      Float2ToBf16x2(a[6], a[7]));
  }
};

// Where the owner `me` writes its results on the n ranks: the output itself when it lies in
// symmetric memory, else the result area that each peer's slot keeps for `me`.
struct PushTargets {
  char* const* bases;   // per-rank base pointers (symmetric user region or staging region)
  size_t direct_off;    // direct: offset of the shard inside the user region
  size_t result_off;    // staged: offset of the slot's result areas
  size_t res_bytes;     // staged: bytes of one result area
  int direct, me;
  __device__ __forceinline__ char* Of(int p) const {
    return bases[p] + (direct ? direct_off : result_off + static_cast<size_t>(PushAreaIndex(me, p)) * res_bytes);
  }
};

// U vectors (v, v+stride, ...) of the owner's shard: own input + the n-1 received copies, all
// local reads with U loads in flight per source; result to the own output and to every peer.
template <int ELEM, int U>
__device__ __forceinline__ void PushSumStep(size_t v, size_t stride, const char* own, const char* recv,
                                            size_t recv_bytes, int n, int me, char* out,
                                            const PushTargets& tg, float post_scale) {
  VecAcc<ELEM> acc[U];
#pragma unroll
  for (int u = 0; u < U; u++) acc[u].Init(*reinterpret_cast<const uint4*>(own + (v + u * stride) * 16));
  for (int j = 0; j < n - 1; j++) {
    const char* src = recv + static_cast<size_t>(j) * recv_bytes;
    uint4 tmp[U];
#pragma unroll
    for (int u = 0; u < U; u++) tmp[u] = *reinterpret_cast<const uint4*>(src + (v + u * stride) * 16);
#pragma unroll
    for (int u = 0; u < U; u++) acc[u].Add(tmp[u]);
  }
  uint4 r[U];
#pragma unroll
  for (int u = 0; u < U; u++) {
    r[u] = acc[u].Finish(post_scale);
    *reinterpret_cast<uint4*>(out + (v + u * stride) * 16) = r[u];
  }
  for (int d = 1; d < n; d++) {
    char* dst = tg.Of((me + d) % n);
#pragma unroll
    for (int u = 0; u < U; u++) *reinterpret_cast<uint4*>(dst + (v + u * stride) * 16) = r[u];
  }
}

// The same for the quantised mode, in groups of four elements: the own input is quantised
// here, the peers' contributions arrive as int32; the sum is dequantised once. NARROW:
// the results leave as bf16 (8 bytes per group) instead of float32.
template <int ELEM, int U, bool NARROW>
__device__ __forceinline__ void PushQuantStep(size_t g, size_t stride, size_t first_elem, const char* own,
                                              const char* recv, size_t recv_bytes, int n, int me, char* out,
                                              const PushTargets& tg, float post_scale, const float* sf, int shift) {
  uint4 acc[U];
  float f[U];
#pragma unroll
  for (int u = 0; u < U; u++) {
    const float4 x = LoadGroupAsFloat<ELEM>(own, g + u * stride);
    f[u] = sf[(first_elem + (g + u * stride) * 4) >> shift];
    acc[u] = make_uint4(static_cast<unsigned>(quant::Quantize(x.x, f[u])), static_cast<unsigned>(quant::Quantize(x.y, f[u])),
                        static_cast<unsigned>(quant::Quantize(x.z, f[u])), static_cast<unsigned>(quant::Quantize(x.w, f[u])));
  }
  for (int j = 0; j < n - 1; j++) {
    const char* src = recv + static_cast<size_t>(j) * recv_bytes;
    uint4 tmp[U];
#pragma unroll
    for (int u = 0; u < U; u++) tmp[u] = *reinterpret_cast<const uint4*>(src + (g + u * stride) * 16);
#pragma unroll
    for (int u = 0; u < U; u++) { acc[u].x += tmp[u].x; acc[u].y += tmp[u].y; acc[u].z += tmp[u].z; acc[u].w += tmp[u].w; }
  }
  uint4 w[U];
  uint2 h[U];
#pragma unroll
  for (int u = 0; u < U; u++) {
    float4 y;
    y.x = quant::Dequantize(static_cast<int>(acc[u].x), f[u]);
    y.y = quant::Dequantize(static_cast<int>(acc[u].y), f[u]);
    y.z = quant::Dequantize(static_cast<int>(acc[u].z), f[u]);
    y.w = quant::Dequantize(static_cast<int>(acc[u].w), f[u]);
    if (post_scale != 1.0f) { y.x *= post_scale; y.y *= post_scale; y.z *= post_scale; y.w *= post_scale; }
    w[u] = make_uint4(__float_as_uint(y.x), __float_as_uint(y.y), __float_as_uint(y.z), __float_as_uint(y.w));
    h[u] = make_uint2(Float2ToBf16x2(y.x, y.y), Float2ToBf16x2(y.z, y.w));
    if (ELEM == ELEM_BF16) *reinterpret_cast<uint2*>(out + (g + u * stride) * 8) = h[u];
    else *reinterpret_cast<uint4*>(out + (g + u * stride) * 16) = w[u];
  }
  for (int d = 1; d < n; d++) {
    char* dst = tg.Of((me + d) % n);
#pragma unroll
    for (int u = 0; u < U; u++) {
      if (NARROW) *reinterpret_cast<uint2*>(dst + (g + u * stride) * 8) = h[u];
      else *reinterpret_cast<uint4*>(dst + (g + u * stride) * 16) = w[u];
    }
  }
}

template <int ELEM, int MODE>
__device__ void RunPush(const RankCtx& ctx, const JobArgs& job, int channel,
                        unsigned long long elems_per_channel, Epoch base, StagedShared* sh, float* s_sf) {
  constexpr int kLoadWarps = MODE == MODE_QUANT ? 6 : 5;
  constexpr int kReduceWarps = MODE == MODE_QUANT ? 7 : 7;
  constexpr int kStoreWarps = kThreads / 32 - kLoadWarps - kReduceWarps - 1;  // the last warp tells the peers
  static_assert(kStoreWarps >= 1, "the storer needs a warp");
  const int in_esz = ELEM == ELEM_BF16 ? 2 : 4;
  const int st_esz = MODE == MODE_QUANT ? 4 : in_esz;   // what travels on the reduce leg
  const int res_esz = MODE == MODE_QUANT ? (ELEM == ELEM_BF16 ? 2 : 4) : in_esz;  // what travels on the result leg (bf16 jobs: bf16)
  const size_t unit = MODE == MODE_QUANT ? static_cast<size_t>(ctx.block_numel) : 128;
  const int S = ctx.slots_per_channel;
  const int n = ctx.nranks, me = ctx.rank;

  unsigned long long c0 = static_cast<unsigned long long>(channel) * elems_per_channel;
  if (c0 >= job.numel) return;
  unsigned long long c1 = c0 + elems_per_channel;
  if (c1 > job.numel) c1 = job.numel;
  const size_t tile_elems = job.tile_elems;
  const unsigned long long ntiles = (c1 - c0 + tile_elems - 1) / tile_elems;
  const size_t shard_cap = tile_elems / n;  // elements of the largest shard (tiles are multiples of n * unit)
  const size_t recv_bytes = shard_cap * st_esz, res_bytes = shard_cap * res_esz;
  char* my_stage = ctx.stage_peer[me];
  const size_t blocks_per_slot = ctx.slot_bytes / 4 / ctx.block_numel;
  const int shift = 31 - __clz(ctx.block_numel);
  const unsigned long long A = static_cast<unsigned long long>(ctx.exp_lookahead);  // exponents travel A tiles ahead of the data (see RunStaged)
  const int E = ctx.exp_ring;
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
    // loader (phase 1), reducer (phase 2) and, unless results go straight into the outputs, storer (phase 3)
    RunSignaler(ctx, sh, channel, base, ntiles, direct_out ? 2 : 3);
    return;
  }
  volatile int* failed = reinterpret_cast<volatile int*>(&sh->failed);
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
  auto slot_offset_of = [&](unsigned long long k) {
    return ctx.data_offset + (static_cast<size_t>(channel) * S + static_cast<size_t>(k % S)) * ctx.slot_bytes;
  };
  auto exp_offset_of = [&](unsigned long long k) {
    return ctx.exp_offset + (static_cast<size_t>(channel) * E + static_cast<size_t>(k % E)) * blocks_per_slot * kExpWordBytes;
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
    const size_t slot_off = slot_offset_of(k);
    const size_t result_off = slot_off + static_cast<size_t>(n - 1) * recv_bytes;
    const size_t exp_off = exp_offset_of(k);
    SML_GEOMETRY_CHECK(ctx, channel, failed,
                       len > 0 && len <= tile_elems && pos + len <= job.numel && tile_elems % (n * unit) == 0 &&
                       slot_off >= ctx.data_offset && result_off + static_cast<size_t>(n - 1) * res_bytes <= slot_off + ctx.slot_bytes &&
                       slot_off + ctx.slot_bytes <= ctx.stage_bytes &&
                       (MODE != MODE_QUANT ||
                        (blocks_per_slot * S <= static_cast<size_t>(kMaxBlocksPerSlot) &&
                         tile_elems / ctx.block_numel <= blocks_per_slot &&
                         E >= 1 && 2 * A <= static_cast<unsigned long long>(E) &&
                         exp_off + blocks_per_slot * kExpWordBytes <= ctx.oneshot_offset)) &&
                       (!direct_out || job.out_offset + (pos + len) * in_esz <= job.user_bytes));
    float* sf = s_sf + static_cast<size_t>(slot) * blocks_per_slot;
    const char* in = static_cast<const char*>(job.in) + pos * in_esz;

    if (which == 0) {
      // ------------------------------ loader ------------------------------
      // Room in the peers' slots (see the flow-control notes above).
      if (k >= static_cast<unsigned long long>(S)) {
        if (!RoleWait(ctx, role, channel, 2, epoch - S, sh)) return;
      }
      if (MODE == MODE_QUANT) {
        if (k == 0 || A == 0) {
          bool published = publish(in, len, exp_off, epoch);
          for (unsigned long long t = 1; published && t < A && t < ntiles; t++)
            published = publish(in + t * tile_elems * in_esz, tile_len(t), exp_offset_of(t), epoch + t);
          RoleSignal(ctx, role, channel, 0, epoch);
          const bool met = RoleWait(ctx, role, channel, 0, epoch, sh);  // every warp takes part, whatever happened
          if (!published || !met) return;
        } else if (k >= A) {
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
      }
      bool streamed = true;
      const size_t per = len / n;  // a full tile: n shards of whole chunks
      if (MODE == MODE_QUANT && stream && len == tile_elems && per % (kWsChunk / 4) == 0) {
        // All n-1 foreign shards as one run of chunks, the right-hand neighbour's first.
        const size_t cps = per / (kWsChunk / 4);  // chunks per shard
        char* const* peers = ctx.stage_peer;
        streamed = WarpStreamRun(
            ws, warp, kLoadWarps, lane, cps * (n - 1),
            [&](size_t c) {
              const int p = (me + 1 + static_cast<int>(c / cps)) % n;
              return in + (static_cast<size_t>(p) * per + (c % cps) * (kWsChunk / 4)) * 4;
            },
            [&](size_t c, const char* smem) {
              const int p = (me + 1 + static_cast<int>(c / cps)) % n;
              const size_t off = (c % cps) * (kWsChunk / 4);  // first element of the chunk inside its shard
              int4* dst = reinterpret_cast<int4*>(peers[p] + slot_off + static_cast<size_t>(PushAreaIndex(me, p)) * recv_bytes) + off / 4;
              const float* sfp = sf;
              float4 x[8];
#pragma unroll
              for (int u = 0; u < 8; u++) x[u] = reinterpret_cast<const float4*>(smem)[u * 32 + lane];
#pragma unroll
              for (int u = 0; u < 8; u++) {
                const size_t e = static_cast<size_t>(p) * per + off + static_cast<size_t>(u * 32 + lane) * 4;
                const float f = sfp[e >> shift];
                int4 r;
                r.x = quant::Quantize(x[u].x, f);
                r.y = quant::Quantize(x[u].y, f);
                r.z = quant::Quantize(x[u].z, f);
                r.w = quant::Quantize(x[u].w, f);
                dst[u * 32 + lane] = r;
              }
            });
      } else {
        for (int d = 1; d < n; d++) {
          const int p = (me + d) % n;  // start with the right-hand neighbour: spreads the traffic
          size_t sb, se;
          ShardRange(len, n, p, unit, &sb, &se);
          if (sb >= se) continue;
          char* dst = ctx.stage_peer[p] + slot_off + static_cast<size_t>(PushAreaIndex(me, p)) * recv_bytes;
          if (MODE == MODE_QUANT) {
            QuantizeRange<ELEM, kPushUnroll>(role.tid, role.nthreads, in, reinterpret_cast<int*>(dst), sb, se, sf, shift);
          } else {
            RoleCopy(role, dst, in + sb * in_esz, (se - sb) * in_esz, in_esz);
          }
        }
      }
      lap(10);
      if (MODE == MODE_QUANT && streamed && A > 0 && k + A < ntiles)
        streamed = publish(in + A * tile_elems * in_esz, tile_len(k + A), exp_offset_of(k + A), epoch + A);
      if (!streamed) {
        role.Sync();  // the other warps are on their way to the signal's barrier: meet them, then leave together
        return;
      }
      lap(11);
      RoleDone(role, sh, 0, k + 1);
      if (*failed) return;
      lap(4);
    } else if (which == 1) {
      // ------------------------------ reducer ------------------------------
      if (!RoleWait(ctx, role, channel, 1, epoch, sh)) return;
      if (!direct_out && k >= static_cast<unsigned long long>(S)) {
        if (!RoleWait(ctx, role, channel, 3, epoch - S, sh)) return;
      }
      lap(5);
      size_t sb, se;
      ShardRange(len, n, me, unit, &sb, &se);
      if (sb < se) {
        const size_t cnt = se - sb;
        const char* own = in + sb * in_esz;
        char* out = static_cast<char*>(job.out) + (pos + sb) * in_esz;
        PushTargets tg;
        tg.bases = direct_out ? job.user_peer : ctx.stage_peer;
        tg.direct_off = job.out_offset + (pos + sb) * in_esz;
        tg.result_off = result_off;
        tg.res_bytes = res_bytes;
        tg.direct = direct_out ? 1 : 0;
        tg.me = me;
        const char* recv = my_stage + slot_off;
        const size_t t = role.tid, nt = role.nthreads;
        const uintptr_t both = reinterpret_cast<uintptr_t>(own) | reinterpret_cast<uintptr_t>(out);
        if (MODE == MODE_QUANT) {
          const bool narrow = ELEM == ELEM_BF16;  // bf16 jobs receive bf16: in their output, or in the result areas
          const size_t ngroups = (both & (ELEM == ELEM_BF16 ? 7 : 15)) == 0 ? cnt / 4 : 0;
          constexpr int U = 4;
          size_t g = t;
          if (narrow) {
            for (; g + (U - 1) * nt < ngroups; g += U * nt)
              PushQuantStep<ELEM, U, true>(g, nt, sb, own, recv, recv_bytes, n, me, out, tg, job.post_scale, sf, shift);
            for (; g < ngroups; g += nt)
              PushQuantStep<ELEM, 1, true>(g, nt, sb, own, recv, recv_bytes, n, me, out, tg, job.post_scale, sf, shift);
          } else {
            for (; g + (U - 1) * nt < ngroups; g += U * nt)
              PushQuantStep<ELEM, U, false>(g, nt, sb, own, recv, recv_bytes, n, me, out, tg, job.post_scale, sf, shift);
            for (; g < ngroups; g += nt)
              PushQuantStep<ELEM, 1, false>(g, nt, sb, own, recv, recv_bytes, n, me, out, tg, job.post_scale, sf, shift);
          }
          // Ragged end, or pointers that are not vector aligned: element by element.
          for (size_t i = ngroups * 4 + t; i < cnt; i += nt) {
            const float f = sf[(sb + i) >> shift];
            unsigned a = static_cast<unsigned>(quant::Quantize(TileLoadAsFloat(own, i, ELEM), f));
            for (int j = 0; j < n - 1; j++)
              a += reinterpret_cast<const unsigned*>(recv + static_cast<size_t>(j) * recv_bytes)[i];
            float y = quant::Dequantize(static_cast<int>(a), f);
            if (job.post_scale != 1.0f) y *= job.post_scale;
            if (ELEM == ELEM_BF16) reinterpret_cast<unsigned short*>(out)[i] = FloatToBf16(y);
            else reinterpret_cast<float*>(out)[i] = y;
            for (int d = 1; d < n; d++) {
              char* dst = tg.Of((me + d) % n);
              if (narrow) reinterpret_cast<unsigned short*>(dst)[i] = FloatToBf16(y);
              else reinterpret_cast<float*>(dst)[i] = y;
            }
          }
        } else {
          const size_t vec_elems = 16 / in_esz;
          const size_t nvec = (both & 15) == 0 ? cnt / vec_elems : 0;
          size_t v = t;
          for (; v + (kPushUnroll - 1) * nt < nvec; v += kPushUnroll * nt)
            PushSumStep<ELEM, kPushUnroll>(v, nt, own, recv, recv_bytes, n, me, out, tg, job.post_scale);
          for (; v < nvec; v += nt)
            PushSumStep<ELEM, 1>(v, nt, own, recv, recv_bytes, n, me, out, tg, job.post_scale);
          for (size_t i = nvec * vec_elems + t; i < cnt; i += nt) {
            if (ELEM == ELEM_I32) {
              unsigned a = reinterpret_cast<const unsigned*>(own)[i];
              for (int j = 0; j < n - 1; j++) a += reinterpret_cast<const unsigned*>(recv + static_cast<size_t>(j) * recv_bytes)[i];
              reinterpret_cast<unsigned*>(out)[i] = a;
              for (int d = 1; d < n; d++) reinterpret_cast<unsigned*>(tg.Of((me + d) % n))[i] = a;
            } else if (ELEM == ELEM_F32) {
              float a = reinterpret_cast<const float*>(own)[i];
              for (int j = 0; j < n - 1; j++) a += reinterpret_cast<const float*>(recv + static_cast<size_t>(j) * recv_bytes)[i];
              if (job.post_scale != 1.0f) a *= job.post_scale;
              reinterpret_cast<float*>(out)[i] = a;
              for (int d = 1; d < n; d++) reinterpret_cast<float*>(tg.Of((me + d) % n))[i] = a;
            } else {
              float a = Bf16ToFloat(reinterpret_cast<const unsigned short*>(own)[i]);
              for (int j = 0; j < n - 1; j++)
                a += Bf16ToFloat(reinterpret_cast<const unsigned short*>(recv + static_cast<size_t>(j) * recv_bytes)[i]);
              if (job.post_scale != 1.0f) a *= job.post_scale;
              const unsigned short h = FloatToBf16(a);
              reinterpret_cast<unsigned short*>(out)[i] = h;
              for (int d = 1; d < n; d++) reinterpret_cast<unsigned short*>(tg.Of((me + d) % n))[i] = h;
            }
          }
        }
      }
      RoleDone(role, sh, 1, k + 1);
      lap(6);
    } else {
      // ------------------------------ storer ------------------------------
      if (!RoleWait(ctx, role, channel, 2, epoch, sh)) return;
      lap(7);
      if (!direct_out) {
        for (int d = 1; d < n; d++) {
          const int p = (me + d) % n;
          size_t sb, se;
          ShardRange(len, n, p, unit, &sb, &se);
          if (sb >= se) continue;
          const char* src = my_stage + result_off + static_cast<size_t>(PushAreaIndex(p, me)) * res_bytes;
          char* out = static_cast<char*>(job.out) + (pos + sb) * in_esz;
          {
            RoleLocalCopy(ctx, role, sh, 1, out, src, (se - sb) * in_esz, in_esz);
          }
        }
        RoleDone(role, sh, 2, k + 1);  // my result areas of this slot may be refilled
        if (*failed) return;
      }
      if (role.tid == 0) {
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
#endif  // SWITCHML_PUSH_ALLREDUCE_CUH_
