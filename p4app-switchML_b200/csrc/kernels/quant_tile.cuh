// Per-tile pieces of the block fixed-point pipeline that the streaming kernels share:
// publishing a tile's block exponents to every rank, turning the agreed exponents into
// scale factors, and quantising a range of a tile.
//
// Exponent exchange. Every slot has one 64-bit word per quantisation block in the symmetric
// staging region of every rank. A rank publishes its local exponent of block b of the tile
// with epoch E as  word = (E << 8) | (exponent + 128)  through an atomic MAX into the word
// of ALL ranks: one multimem.red through the switch, or one red per peer over NVLink. After
// everybody has published, every rank's own copy of the word holds the largest exponent
// tagged with E: the agreement costs no load that crosses the fabric and no reset, because
// a tag from an older tile is always smaller and a newer one never arrives before the word
// was consumed (see the flow-control notes at the callers). It is the switch's exponent
// register (p4/exponents.p4:48-54) turned into a posted write, and since the words of
// tile k+1 travel while the payload of tile k is quantised, the exchange rides one tile
// ahead of the data like the reference's exponents ride one packet batch ahead
// (prepostprocessors/cpu_exponent_quantizer_ppp.cc:115-156).
#ifndef SWITCHML_QUANT_TILE_CUH_
#define SWITCHML_QUANT_TILE_CUH_

#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels/allreduce_kernels.h"
#include "kernels/device_sync.cuh"
#include "kernels/warp_stream.cuh"
#include "switchml/quant_math.h"

namespace switchml {
namespace kernels {

static const int kExpWordBytes = 8;

__device__ __forceinline__ unsigned long long ExpWord(Epoch tag, int exponent) {
  return (tag << 8) | static_cast<unsigned long long>(exponent + 128);
}

// MAX `word` into the exponent word at byte offset `off` of every rank's staging region.
__device__ __forceinline__ void ExpPublish(const RankCtx& ctx, size_t off, unsigned long long word) {
  if (ctx.use_multimem) {
    asm volatile("multimem.red.relaxed.sys.global.max.u64 [%0], %1;" ::"l"(ctx.stage_mc + off), "l"(word) : "memory");
  } else {
    for (int p = 0; p < ctx.nranks; p++)
      asm volatile("red.relaxed.sys.global.max.u64 [%0], %1;" ::"l"(ctx.stage_peer[p] + off), "l"(word) : "memory");
  }
}

__device__ __forceinline__ float TileLoadAsFloat(const void* in, size_t i, int elem) {
  if (elem == ELEM_BF16) return __uint_as_float(static_cast<unsigned>(reinterpret_cast<const unsigned short*>(in)[i]) << 16);
  return reinterpret_cast<const float*>(in)[i];
}

// Local exponents of the `len` elements at `in` (one tile), published under `tag` into the
// exponent words starting at byte offset `exp_off`. Called by all threads of a role of
// `nwarps` warps; `warp` is the caller's warp index inside the role.
// One step of the exponent pass: 8 consecutive rows of 128 float32 elements starting at row
// `row0` of the tile, one float4 per lane and row in `x` (from global or shared memory).
// Blocks of 32 or 64 elements are groups of 8 or 16 neighbouring lanes of one row; larger
// blocks are 1, 2, 4 or 8 whole rows, which a step always holds completely because steps
// start at multiples of 8 rows.
__device__ __forceinline__ void PublishRows8(const RankCtx& ctx, int lane, const float4* x, size_t row0,
                                             size_t exp_off, Epoch tag) {
  constexpr int kRows = 8;
  const size_t B = ctx.block_numel;
  float m[kRows];
#pragma unroll
  for (int u = 0; u < kRows; u++)
    m[u] = fmaxf(fmaxf(fabsf(x[u].x), fabsf(x[u].y)), fmaxf(fabsf(x[u].z), fabsf(x[u].w)));
  if (B < 128) {
    const int g = static_cast<int>(B / 4);  // lanes per block: 8 or 16
    const size_t per_row = 128 / B;         // blocks per row: 4 or 2
#pragma unroll
    for (int u = 0; u < kRows; u++) {
      float mm = m[u];
      for (int o = g >> 1; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
      if ((lane % g) == 0)
        ExpPublish(ctx, exp_off + ((row0 + u) * per_row + lane / g) * kExpWordBytes,
                   ExpWord(tag, quant::LocalExponent(mm)));
    }
  } else {
    const int rows_per_block = static_cast<int>(B / 128);  // 1, 2, 4 or 8
    // fold the rows of one block into the first of them, then one butterfly per block
#pragma unroll
    for (int span = 1; span < kRows; span <<= 1) {
      if (span < rows_per_block) {
#pragma unroll
        for (int u = 0; u + span < kRows; u += 2 * span) m[u] = fmaxf(m[u], m[u + span]);
      }
    }
#pragma unroll
    for (int u = 0; u < kRows; u++) {
      if ((u % rows_per_block) != 0) continue;  // warp-uniform
      float mm = m[u];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
      if (lane == 0)
        ExpPublish(ctx, exp_off + ((row0 + u) / rows_per_block) * kExpWordBytes,
                   ExpWord(tag, quant::LocalExponent(mm)));
    }
  }
}

// The blocks [first_block, nblocks) of a tile, one block per warp and step, any element type
// and alignment: what the row-wise passes leave over (last rows, a ragged last block).
template <int ELEM>
__device__ __forceinline__ void PublishBlocksSlow(const RankCtx& ctx, int warp, int nwarps, int lane, const char* in,
                                                  size_t len, size_t first_block, size_t exp_off, Epoch tag) {
  const size_t B = ctx.block_numel;
  const size_t nblocks = (len + B - 1) / B;
  for (size_t b = first_block + warp; b < nblocks; b += nwarps) {
    const size_t base = b * B;
    const size_t n = len - base < B ? len - base : B;
    float m = 0.f;
    for (size_t i = lane; i < n; i += 32) {
      float v = fabsf(TileLoadAsFloat(in, base + i, ELEM));
      if (v > m) m = v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float t = __shfl_xor_sync(0xffffffffu, m, o);
      if (t > m) m = t;
    }
    if (lane == 0) ExpPublish(ctx, exp_off + b * kExpWordBytes, ExpWord(tag, quant::LocalExponent(m)));
  }
}

template <int ELEM>
__device__ __forceinline__ void PublishTileExponents(const RankCtx& ctx, int warp, int nwarps, int lane,
                                                     const char* in, size_t len, size_t exp_off, Epoch tag) {
  const size_t B = ctx.block_numel;
  size_t first_block = 0;
  if (ELEM == ELEM_F32 && (reinterpret_cast<uintptr_t>(in) & 15) == 0) {
    // The tile as rows of 128 elements, one float4 per lane. A warp takes 8 consecutive rows
    // per step and issues all their loads before it looks at any value.
    constexpr int kRows = 8;
    const size_t whole_blocks = len / B;                          // blocks without a ragged end
    const size_t nrows = whole_blocks * B / 128 / kRows * kRows;  // rows handled here, in whole steps
    const float4* p4 = reinterpret_cast<const float4*>(in);
    for (size_t r0 = static_cast<size_t>(warp) * kRows; r0 < nrows; r0 += static_cast<size_t>(nwarps) * kRows) {
      float4 x[kRows];
#pragma unroll
      for (int u = 0; u < kRows; u++) x[u] = p4[(r0 + u) * 32 + lane];
      PublishRows8(ctx, lane, x, r0, exp_off, tag);
    }
    first_block = nrows * 128 / B;
  }
  PublishBlocksSlow<ELEM>(ctx, warp, nwarps, lane, in, len, first_block, exp_off, tag);
}

// Scale factors of the tile's blocks from this rank's own copy of the exponent words, which
// by now hold the maximum over all ranks. A word with a foreign tag means the protocol was
// violated (a peer ran another job, or ran ahead): reported, never silently used.
__device__ __forceinline__ void TileScaleFactors(const RankCtx& ctx, int tid, int nthreads, size_t exp_off,
                                                 size_t nblocks, Epoch tag, float* sf, int channel,
                                                 volatile int* failed) {
  const unsigned long long* words =
      reinterpret_cast<const unsigned long long*>(ctx.stage_peer[ctx.rank] + exp_off);
  for (size_t b = tid; b < nblocks; b += nthreads) {
    unsigned long long w = __ldcg(words + b);
    if ((w >> 8) != tag) {
      ReportStatus(ctx, STATUS_PROTOCOL | (channel << 8));
      *failed = 1;
    }
    sf[b] = quant::ScaleFactorFromBase(static_cast<int>(w & 0xff) - 128, ctx.quant_base);
  }
}

// q[i - begin] = Quantize(in[i], sf[i >> shift]) for i in [begin, end), elements of one tile.
// `begin` is a multiple of the block size, so a 4-element vector never straddles a block.
template <int ELEM, int UNROLL>
__device__ __forceinline__ void QuantizeRange(int tid, int nthreads, const char* in, int* q, size_t begin,
                                              size_t end, const float* sf, int shift) {
  if (begin >= end) return;
  const size_t n = end - begin;
  if (ELEM == ELEM_F32 && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(q)) & 15) == 0) {
    const float4* in4 = reinterpret_cast<const float4*>(in) + begin / 4;
    int4* q4 = reinterpret_cast<int4*>(q);
    const size_t nvec = n / 4;
    const size_t nt = nthreads;
    size_t i = tid;
    for (; i + (UNROLL - 1) * nt < nvec; i += UNROLL * nt) {
      float4 x[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; u++) x[u] = in4[i + u * nt];
#pragma unroll
      for (int u = 0; u < UNROLL; u++) {
        const float f = sf[(begin + (i + u * nt) * 4) >> shift];
        int4 r;
        r.x = quant::Quantize(x[u].x, f);
        r.y = quant::Quantize(x[u].y, f);
        r.z = quant::Quantize(x[u].z, f);
        r.w = quant::Quantize(x[u].w, f);
        q4[i + u * nt] = r;
      }
    }
    for (; i < nvec; i += nt) {
      float4 x = in4[i];
      const float f = sf[(begin + i * 4) >> shift];
      int4 r;
      r.x = quant::Quantize(x.x, f);
      r.y = quant::Quantize(x.y, f);
      r.z = quant::Quantize(x.z, f);
      r.w = quant::Quantize(x.w, f);
      q4[i] = r;
    }
    for (size_t j = nvec * 4 + tid; j < n; j += nthreads)
      q[j] = quant::Quantize(reinterpret_cast<const float*>(in)[begin + j], sf[(begin + j) >> shift]);
  } else {
    for (size_t j = tid; j < n; j += nthreads)
      q[j] = quant::Quantize(TileLoadAsFloat(in, begin + j, ELEM), sf[(begin + j) >> shift]);
  }
}

// ---- the same two passes fed by the TMA unit (float32 input, 16-byte aligned, device memory) ----

// A tile's exponent pass: whole chunks of 1024 elements stream through the warps' rings, the
// rest goes the slow way. False if a wait ran out.
__device__ __forceinline__ bool StreamTileExponents(const RankCtx& ctx, WarpStream& ws, int warp, int nwarps, int lane,
                                                    const char* in, size_t len, size_t exp_off, Epoch tag) {
  const size_t nchunks = len / (kWsChunk / 4);
  const bool ok = WarpStreamRun(
      ws, warp, nwarps, lane, nchunks, [&](size_t c) { return in + c * kWsChunk; },
      [&](size_t c, const char* smem) {
        float4 x[8];
#pragma unroll
        for (int u = 0; u < 8; u++) x[u] = reinterpret_cast<const float4*>(smem)[u * 32 + lane];
        PublishRows8(ctx, lane, x, c * 8, exp_off, tag);
      });
  if (!ok) return false;
  PublishBlocksSlow<ELEM_F32>(ctx, warp, nwarps, lane, in, len, nchunks * (kWsChunk / 4) / ctx.block_numel, exp_off, tag);
  return true;
}

// Quantise the elements [begin, end) of a tile (both multiples of 1024 apart from the tile's
// ragged end): whole chunks stream through the warps' rings; `store(e, q)` receives the four
// quantised values of elements e..e+3 (tile-relative). The ragged end is left to the caller
// (QuantizeRange on [begin + whole chunks, end)). False if a wait ran out.
template <typename Store>
__device__ __forceinline__ bool StreamQuantize(WarpStream& ws, int warp, int nwarps, int lane, const char* in,
                                               size_t begin, size_t nchunks, const float* sf, int shift, Store store) {
  return WarpStreamRun(
      ws, warp, nwarps, lane, nchunks, [&](size_t c) { return in + begin * 4 + c * kWsChunk; },
      [&](size_t c, const char* smem) {
        float4 x[8];
#pragma unroll
        for (int u = 0; u < 8; u++) x[u] = reinterpret_cast<const float4*>(smem)[u * 32 + lane];
#pragma unroll
        for (int u = 0; u < 8; u++) {
          const size_t e = begin + c * (kWsChunk / 4) + static_cast<size_t>(u * 32 + lane) * 4;
          const float f = sf[e >> shift];
          int4 r;
          r.x = quant::Quantize(x[u].x, f);
          r.y = quant::Quantize(x[u].y, f);
          r.z = quant::Quantize(x[u].z, f);
          r.w = quant::Quantize(x[u].w, f);
          store(e, r);
        }
      });
}

}  // namespace kernels
}  // namespace switchml
#endif  // SWITCHML_QUANT_TILE_CUH_
