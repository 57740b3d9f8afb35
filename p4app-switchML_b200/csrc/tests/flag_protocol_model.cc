// A host model of the flag protocol the aggregation kernels use between GPUs, run with real
// threads so that ThreadSanitizer can judge it.
//
// The device code (kernels/allreduce_kernels.cu, RunStaged, and kernels/device_sync.cuh) cannot
// run under a race detector on this project's machines. What can be checked on the host is the
// protocol itself: which memory is written and read between which release stores and acquire
// loads. This model keeps that structure and nothing else:
//   * every rank owns a staging region (data slots, exponent slots) and a pad of 64-bit flags
//     flags[channel][phase][source rank] that only ever grow (epochs);
//   * a channel of a rank is three roles - loader, reducer, storer - here one thread each
//     (on the GPU: groups of warps), walking the tiles of the channel independently;
//   * tile k of a job uses epoch base + k + 1 and slot k mod S; a signal is a release store of
//     the epoch into the sender's column of every peer's pad, a wait polls the local pad with
//     acquire loads and a time budget;
//   * loader: waits until its own storer has emptied the slot, publishes block exponents
//     (phase 0), waits for everybody's, quantises its tile into its own slot (phase 1);
//     reducer: waits for phase 1, sums its shard over all ranks' slots, dequantises and writes
//     the result into the slot of every rank (phase 2); storer: waits for phase 2, copies the
//     tile to the output, which frees the slot;
//   * each channel keeps the epoch it has reached in a word of its own and advances it when a
//     job ends, so consecutive jobs need no host-side epoch bookkeeping.
// A second variant, not yet in the kernels, is modelled as well ("piggyback"): the exponents of
// tile k+1 travel with the payload of tile k - the reference sends the exponent of a block one
// batch ahead of its payload for the same reason (cpu_exponent_quantizer_ppp.cc:115-156) - so
// that only the first tile of a job needs the exponent barrier (phase 0) and every other tile
// gets by with two all-to-all waits instead of three. It needs one exponent slot more than data
// slots. The model shows that this ordering is race-free and gives the same bits.
// The arithmetic is switchml/quant_math.h, so the result must equal the CPU oracle bit for bit.
// The model has teeth: letting the reducer wait for phase 0 instead of phase 1 makes
// ThreadSanitizer report data races on the slots and the results differ from the oracle.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <thread>
#include <vector>

#include "ppp/cpu_exponent_quantizer_ppp.h"
#include "switchml/quant_math.h"

namespace switchml {
namespace {

const int kPhases = 3;

struct Geometry {
  int ranks, channels, slots, block, tile;  // tile: elements, a multiple of ranks * block
  bool piggyback;                           // exponents of tile k+1 ride with the payload of tile k
  int exp_slots() const { return slots + 1; }
};

struct RankMemory {
  std::vector<std::atomic<uint64_t>> flags;  // [channel][phase][src]
  std::vector<int32_t> data;                 // [channel][slot][tile]: quantised values, then results (as bits)
  std::vector<int32_t> exps;                 // [channel][slot][blocks per tile]
  std::vector<uint64_t> epoch_words;         // [channel], touched by the loader only between jobs
  std::vector<std::atomic<uint64_t>> stored;  // [channel]: tiles the storer has copied out in this job
  std::atomic<int> failed{0};
  RankMemory(const Geometry& g)
      : flags(static_cast<size_t>(g.channels) * kPhases * g.ranks), data(static_cast<size_t>(g.channels) * g.slots * g.tile),
        exps(static_cast<size_t>(g.channels) * g.exp_slots() * (g.tile / g.block)), epoch_words(g.channels, 0),
        stored(g.channels) {
    for (auto& f : flags) f.store(0);
    for (auto& s : stored) s.store(0);
  }
};

struct Model {
  Geometry g;
  std::vector<std::unique_ptr<RankMemory>> mem;
  std::atomic<uint64_t>& Flag(int rank, int channel, int phase, int src) {
    return mem[rank]->flags[(static_cast<size_t>(channel) * kPhases + phase) * g.ranks + src];
  }
  int32_t* Data(int rank, int channel, int slot) {
    return mem[rank]->data.data() + (static_cast<size_t>(channel) * g.slots + slot) * g.tile;
  }
  // exponent slot of tile k: a ring one deeper than the data slots
  int32_t* Exps(int rank, int channel, size_t k) {
    return mem[rank]->exps.data() +
           (static_cast<size_t>(channel) * g.exp_slots() + k % g.exp_slots()) * (g.tile / g.block);
  }
  void Signal(int me, int channel, int phase, uint64_t epoch) {
    for (int p = 0; p < g.ranks; p++) Flag(p, channel, phase, me).store(epoch, std::memory_order_release);
  }
  // False when the budget ran out or somebody on this rank already failed.
  bool Wait(int me, int channel, int phase, uint64_t epoch) {
    const auto t0 = std::chrono::steady_clock::now();
    for (int src = 0; src < g.ranks; src++) {
      while (Flag(me, channel, phase, src).load(std::memory_order_acquire) < epoch) {
        if (mem[me]->failed.load() || std::chrono::steady_clock::now() - t0 > std::chrono::seconds(20)) {
          mem[me]->failed.store(1);
          return false;
        }
        std::this_thread::yield();
      }
    }
    return true;
  }
};

struct ChannelRange {
  size_t begin, end;
};

ChannelRange RangeOf(const Geometry& g, size_t numel, int channel) {
  size_t per = (numel + g.channels - 1) / g.channels;
  per = (per + g.tile - 1) / g.tile * g.tile;
  size_t b = per * channel, e = b + per;
  return {b < numel ? b : numel, e < numel ? e : numel};
}

void ShardOf(const Geometry& g, size_t len, int rank, size_t* begin, size_t* end) {
  size_t per = (len + g.ranks - 1) / g.ranks;
  per = (per + g.block - 1) / g.block * g.block;
  size_t b = per * rank, e = b + per;
  *begin = b < len ? b : len;
  *end = e < len ? e : len;
}

void Loader(Model& m, int me, int c, const float* in, size_t numel) {
  const Geometry& g = m.g;
  ChannelRange r = RangeOf(g, numel, c);
  const uint64_t base = m.mem[me]->epoch_words[c];
  const size_t ntiles = (r.end - r.begin + g.tile - 1) / g.tile;
  for (size_t k = 0; k < ntiles; k++) {
    const uint64_t epoch = base + k + 1;
    const int slot = static_cast<int>(k % g.slots);
    const size_t pos = r.begin + k * g.tile, len = std::min<size_t>(g.tile, r.end - pos);
    // the slot is free once this rank's storer has copied out the tile that used it last
    const auto t0 = std::chrono::steady_clock::now();
    while (m.mem[me]->stored[c].load(std::memory_order_acquire) + g.slots < k + 1) {
      if (m.mem[me]->failed.load() || std::chrono::steady_clock::now() - t0 > std::chrono::seconds(20)) {
        m.mem[me]->failed.store(1);
        return;
      }
      std::this_thread::yield();
    }
    const size_t nblocks = (len + g.block - 1) / g.block;
    auto publish_exponents = [&](size_t tile) {
      const size_t tpos = r.begin + tile * g.tile, tlen = std::min<size_t>(g.tile, r.end - tpos);
      int32_t* my_exp = m.Exps(me, c, tile);
      for (size_t b = 0; b * g.block < tlen; b++) {
        float mx = 0.f;
        for (size_t i = b * g.block; i < std::min<size_t>(tlen, (b + 1) * g.block); i++) {
          float v = fabsf(in[tpos + i]);
          if (v > mx) mx = v;
        }
        my_exp[b] = quant::LocalExponent(mx);
      }
    };
    if (!g.piggyback || k == 0) {
      publish_exponents(k);
      m.Signal(me, c, 0, epoch);
      if (!m.Wait(me, c, 0, epoch)) return;
    } else {
      // everybody's exponents of this tile came with their payload of the previous one
      if (!m.Wait(me, c, 1, epoch - 1)) return;
    }
    int32_t* mine = m.Data(me, c, slot);
    for (size_t b = 0; b < nblocks; b++) {
      int e = quant::kZeroExponent;
      for (int p = 0; p < g.ranks; p++) e = std::max(e, static_cast<int>(m.Exps(p, c, k)[b]));
      const float sf = quant::ScaleFactor(e, g.ranks);
      for (size_t i = b * g.block; i < std::min<size_t>(len, (b + 1) * g.block); i++)
        mine[i] = quant::Quantize(in[pos + i], sf);
    }
    // The exponent slot of tile k+1 was last used by tile k-S, which this rank's storer has
    // copied out (checked above), so every rank is done reading it.
    if (g.piggyback && k + 1 < ntiles) publish_exponents(k + 1);
    m.Signal(me, c, 1, epoch);
  }
}

void Reducer(Model& m, int me, int c, size_t numel) {
  const Geometry& g = m.g;
  ChannelRange r = RangeOf(g, numel, c);
  const uint64_t base = m.mem[me]->epoch_words[c];
  const size_t ntiles = (r.end - r.begin + g.tile - 1) / g.tile;
  for (size_t k = 0; k < ntiles; k++) {
    const uint64_t epoch = base + k + 1;
    const int slot = static_cast<int>(k % g.slots);
    const size_t pos = r.begin + k * g.tile, len = std::min<size_t>(g.tile, r.end - pos);
    if (!m.Wait(me, c, 1, epoch)) return;
    size_t sb, se;
    ShardOf(g, len, me, &sb, &se);
    for (size_t i = sb; i < se; i++) {
      uint32_t acc = 0;
      for (int p = 0; p < g.ranks; p++) acc += static_cast<uint32_t>(m.Data(p, c, slot)[i]);
      int e = quant::kZeroExponent;
      for (int p = 0; p < g.ranks; p++) e = std::max(e, static_cast<int>(m.Exps(p, c, k)[i / g.block]));
      const float y = quant::Dequantize(static_cast<int32_t>(acc), quant::ScaleFactor(e, g.ranks));
      int32_t bits;
      memcpy(&bits, &y, 4);
      for (int p = 0; p < g.ranks; p++) m.Data(p, c, slot)[i] = bits;  // the broadcast
    }
    m.Signal(me, c, 2, epoch);
  }
}

void Storer(Model& m, int me, int c, float* out, size_t numel) {
  const Geometry& g = m.g;
  ChannelRange r = RangeOf(g, numel, c);
  const uint64_t base = m.mem[me]->epoch_words[c];
  const size_t ntiles = (r.end - r.begin + g.tile - 1) / g.tile;
  for (size_t k = 0; k < ntiles; k++) {
    const uint64_t epoch = base + k + 1;
    const int slot = static_cast<int>(k % g.slots);
    const size_t pos = r.begin + k * g.tile, len = std::min<size_t>(g.tile, r.end - pos);
    if (!m.Wait(me, c, 2, epoch)) return;
    memcpy(out + pos, m.Data(me, c, slot), len * 4);
    m.mem[me]->stored[c].store(k + 1, std::memory_order_release);
  }
}

// One job on every rank; returns the number of ranks that failed.
int RunJob(Model& m, const std::vector<std::vector<float>>& in, std::vector<std::vector<float>>* out) {
  const Geometry& g = m.g;
  const size_t numel = in[0].size();
  std::vector<std::thread> threads;
  for (int r = 0; r < g.ranks; r++) {
    for (int c = 0; c < g.channels; c++) {
      m.mem[r]->stored[c].store(0);
      threads.emplace_back(Loader, std::ref(m), r, c, in[r].data(), numel);
      threads.emplace_back(Reducer, std::ref(m), r, c, numel);
      threads.emplace_back(Storer, std::ref(m), r, c, (*out)[r].data(), numel);
    }
  }
  for (auto& t : threads) t.join();
  int failed = 0;
  for (int r = 0; r < g.ranks; r++) {
    failed += m.mem[r]->failed.load();
    // every exit path advances the channel's epoch by the job's tile count, as the kernels do
    for (int c = 0; c < g.channels; c++) {
      ChannelRange range = RangeOf(g, numel, c);
      m.mem[r]->epoch_words[c] += (range.end - range.begin + g.tile - 1) / g.tile;
    }
  }
  return failed;
}

}  // namespace

// Returns the number of failed expectations; prints what went wrong.
int RunFlagProtocolModel() {
  int failures = 0;
  uint32_t seed = 99;
  auto next = [&] { seed = seed * 1664525u + 1013904223u; return seed; };
  const Geometry geometries[] = {{2, 2, 2, 64, 256, false}, {3, 2, 2, 64, 384, false}, {4, 3, 3, 32, 256, false},
                                 {2, 2, 2, 64, 256, true},  {3, 1, 2, 64, 384, true},  {4, 3, 3, 32, 256, true}};
  for (const Geometry& g : geometries) {
    Model m;
    m.g = g;
    for (int r = 0; r < g.ranks; r++) m.mem.emplace_back(new RankMemory(g));
    // several jobs back to back over the same flags and slots: epochs only grow
    for (size_t numel : {size_t(1), size_t(g.tile), size_t(5 * g.tile + 77), size_t(13 * g.tile - 1)}) {
      std::vector<std::vector<float>> in(g.ranks, std::vector<float>(numel)), out(g.ranks, std::vector<float>(numel, -1.f));
      for (int r = 0; r < g.ranks; r++)
        for (size_t i = 0; i < numel; i++)
          in[r][i] = (static_cast<int>(next() >> 8) % 2001 - 1000) * 0.001f * static_cast<float>(1 << (next() % 12));
      if (RunJob(m, in, &out) != 0) {
        printf("  FAILED flag protocol model: a wait ran out (%d ranks, %zu elements)\n", g.ranks, numel);
        return failures + 1;
      }
      std::vector<const float*> ptrs;
      for (int r = 0; r < g.ranks; r++) ptrs.push_back(in[r].data());
      std::vector<float> want(numel);
      OracleQuantAllReduce(ptrs.data(), g.ranks, numel, g.block, want.data());
      for (int r = 0; r < g.ranks; r++) {
        if (memcmp(out[r].data(), want.data(), numel * 4) != 0) {
          printf("  FAILED flag protocol model: rank %d of %d differs from the oracle (%zu elements)\n", r, g.ranks, numel);
          failures++;
        }
      }
    }
  }
  return failures;
}

}  // namespace switchml
