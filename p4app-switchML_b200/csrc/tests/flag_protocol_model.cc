// A host model of the flag protocols the aggregation kernels use between GPUs, run with real
// threads so that ThreadSanitizer can judge them.
//
// The device code (kernels/allreduce_kernels.cu RunStaged, kernels/push_allreduce.cuh RunPush,
// kernels/quant_tile.cuh, kernels/device_sync.cuh) cannot run under a race detector on this
// project's machines. What can be checked on the host is the protocol itself: which memory is
// written and read between which release stores and acquire loads. This model keeps that
// structure and nothing else:
//   * every rank owns a staging region (data slots, exponent words) and a pad of 64-bit flags
//     flags[channel][phase][source rank] that only ever grow (epochs);
//   * a channel of a rank is three roles - loader, reducer, storer - here one thread each
//     (on the GPU: groups of warps), walking the tiles of the channel independently;
//   * tile k of a job uses epoch e(k) = base + k + 1 and slot k mod S; a signal is a release
//     store of the epoch into the sender's column of every peer's pad, a wait polls the local
//     pad with acquire loads and a time budget;
//   * exponents: one 64-bit word per block on every rank, in a ring of E >= 8 exponent slots per
//     channel that is independent of the data slots (tile k uses exponent slot k mod E); a
//     rank publishes (epoch << 8 | exponent + 128) with an atomic MAX into the word of ALL
//     ranks, for tile k+A while it handles the payload of tile k (A <= E/2 tiles of lookahead;
//     with a single data slot or A = 0 every tile meets in phase 0). After the awaited signal each rank reads only its OWN word; a foreign tag is a
//     protocol violation. The loader hands the scale factors to its reducer through a per-slot
//     array that the phase-1 signal (which the reducer awaits from its own rank too) covers;
//   * "staged" (with NVLink multicast): the loader quantises its tile into its own slot
//     (phase 1); the reducer sums its shard over all ranks' slots, dequantises and writes the
//     result into the slot of every rank (phase 2); the storer copies the tile out, which frees
//     the slot for the loader;
//   * "push" (peer memory): the loader pushes the quantised shard p of its input into the
//     receive area that rank p's slot keeps for it (phase 1), after phase 2 >= e(k+1-S) from
//     everybody; the reducer adds its own shard (quantised from the input) and the received
//     ones, writes its output and pushes the result into the result areas of its peers (phase
//     2), after phase 3 >= e(k-S) from everybody; the storer copies the received results out
//     (phase 3);
//   * on the GPU a role leaves a note in shared memory and a signaler warp fences and stores the
//     flags for it; the note is released and acquired at CTA scope, so for the ordering of
//     memory it is as if the role signalled itself, which is what the model does;
//   * each channel keeps the epoch it has reached in a word of its own and advances it when a
//     job ends, so consecutive jobs need no host-side epoch bookkeeping.
// The arithmetic is switchml/quant_math.h, so the result must equal the CPU oracle bit for bit.
// The model has teeth: letting the reducer wait for phase 0 instead of phase 1, or dropping
// the flow-control wait of the pushing loader, makes ThreadSanitizer report data races on the
// slots and the results differ from the oracle.
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

const int kPhases = 4;

struct Geometry {
  int ranks, channels, slots, block, tile;  // tile: elements, a multiple of ranks * block
  bool push;                                // false: staged through whole-tile slots, true: shards pushed to owners
  int lookahead;                            // tiles by which exponents run ahead of their data, as configured
  int blocks() const { return tile / block; }
  int ring() const { return slots > 8 ? slots : 8; }  // exponent slots per channel (kernels::ExpRingDepth)
  size_t A() const {                                  // kernels::ExpLookahead
    if (slots < 2 || lookahead < 0) return 0;
    return static_cast<size_t>(std::min(lookahead, ring() / 2));
  }
  int shard() const { return tile / ranks; }  // elements of the largest shard
};

struct RankMemory {
  std::vector<std::atomic<uint64_t>> flags;      // [channel][phase][src]
  std::vector<int32_t> data;                     // staged: [channel][slot][tile]: quantised values, then results (as bits)
                                                 // push:   [channel][slot][2 * (ranks-1) * shard]: receive areas, result areas
  std::vector<std::atomic<uint64_t>> exp_words;  // [channel][exponent slot][blocks]: tagged exponents, atomic MAX from every rank
  std::vector<float> scale;                      // [channel][slot][blocks]: loader -> reducer of the same rank
  std::vector<uint64_t> epoch_words;             // [channel], touched only between jobs
  std::vector<std::atomic<uint64_t>> stored;     // [channel]: tiles the storer has copied out in this job
  std::atomic<int> failed{0};
  std::atomic<int> protocol_errors{0};
  RankMemory(const Geometry& g)
      : flags(static_cast<size_t>(g.channels) * kPhases * g.ranks),
        data(static_cast<size_t>(g.channels) * g.slots * (g.push ? 2 * (g.ranks - 1) * g.shard() : g.tile)),
        exp_words(static_cast<size_t>(g.channels) * g.ring() * g.blocks()),
        scale(static_cast<size_t>(g.channels) * g.slots * g.blocks()), epoch_words(g.channels, 0), stored(g.channels) {
    for (auto& f : flags) f.store(0);
    for (auto& w : exp_words) w.store(0);
    for (auto& s : stored) s.store(0);
  }
};

struct Model {
  Geometry g;
  std::vector<std::unique_ptr<RankMemory>> mem;
  std::atomic<uint64_t>& Flag(int rank, int channel, int phase, int src) {
    return mem[rank]->flags[(static_cast<size_t>(channel) * kPhases + phase) * g.ranks + src];
  }
  size_t SlotIndex(int channel, size_t k) const { return static_cast<size_t>(channel) * g.slots + k % g.slots; }
  int32_t* Data(int rank, int channel, size_t k) {
    return mem[rank]->data.data() + SlotIndex(channel, k) * (g.push ? 2 * (g.ranks - 1) * g.shard() : g.tile);
  }
  // push: where `src` writes shard data on rank `dst` (src != dst)
  int32_t* Recv(int dst, int channel, size_t k, int src) { return Data(dst, channel, k) + (src < dst ? src : src - 1) * g.shard(); }
  int32_t* Result(int dst, int channel, size_t k, int src) {
    return Data(dst, channel, k) + (g.ranks - 1 + (src < dst ? src : src - 1)) * g.shard();
  }
  std::atomic<uint64_t>* ExpWords(int rank, int channel, size_t k) {
    return mem[rank]->exp_words.data() + (static_cast<size_t>(channel) * g.ring() + k % g.ring()) * g.blocks();
  }
  float* Scale(int rank, int channel, size_t k) { return mem[rank]->scale.data() + SlotIndex(channel, k) * g.blocks(); }
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
  // The atomic MAX of a tagged exponent into the word of every rank (multimem.red.max.u64 /
  // red.max.u64 on the device: relaxed, ordered by the signal that follows).
  void Publish(int channel, size_t k, size_t block, uint64_t tag, int exponent) {
    const uint64_t word = (tag << 8) | static_cast<uint64_t>(exponent + 128);
    for (int p = 0; p < g.ranks; p++) {
      std::atomic<uint64_t>& w = ExpWords(p, channel, k)[block];
      uint64_t seen = w.load(std::memory_order_relaxed);
      while (seen < word && !w.compare_exchange_weak(seen, word, std::memory_order_relaxed)) {
      }
    }
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

// Local exponents of tile `tile`, published under its tag into everybody's words.
void PublishTile(Model& m, int c, const ChannelRange& r, size_t tile, uint64_t base, const float* in) {
  const Geometry& g = m.g;
  const size_t tpos = r.begin + tile * g.tile, tlen = std::min<size_t>(g.tile, r.end - tpos);
  for (size_t b = 0; b * g.block < tlen; b++) {
    float mx = 0.f;
    for (size_t i = b * g.block; i < std::min<size_t>(tlen, (b + 1) * g.block); i++) {
      float v = fabsf(in[tpos + i]);
      if (v > mx) mx = v;
    }
    m.Publish(c, tile, b, base + tile + 1, quant::LocalExponent(mx));
  }
}

void Loader(Model& m, int me, int c, const float* in, size_t numel) {
  const Geometry& g = m.g;
  ChannelRange r = RangeOf(g, numel, c);
  const uint64_t base = m.mem[me]->epoch_words[c];
  const size_t ntiles = (r.end - r.begin + g.tile - 1) / g.tile;
  const size_t A = g.A();  // exponents travel A tiles ahead of the data
  const size_t S = g.slots;
  for (size_t k = 0; k < ntiles; k++) {
    const uint64_t epoch = base + k + 1;
    const size_t pos = r.begin + k * g.tile, len = std::min<size_t>(g.tile, r.end - pos);
    if (g.push) {
      // room in the peers' receive areas and exponent words (flow control of RunPush)
      if (k >= S && !m.Wait(me, c, 2, epoch - S)) return;
    } else {
      // the slot is free once this rank's storer has copied out the tile that used it last
      const auto t0 = std::chrono::steady_clock::now();
      while (m.mem[me]->stored[c].load(std::memory_order_acquire) + S < k + 1) {
        if (m.mem[me]->failed.load() || std::chrono::steady_clock::now() - t0 > std::chrono::seconds(20)) {
          m.mem[me]->failed.store(1);
          return;
        }
        std::this_thread::yield();
      }
    }
    if (k == 0 || A == 0) {
      for (size_t t = k; t < k + std::max<size_t>(A, 1) && t < ntiles; t++) PublishTile(m, c, r, t, base, in);
      m.Signal(me, c, 0, epoch);
      if (!m.Wait(me, c, 0, epoch)) return;
    } else if (k >= A) {
      // everybody's exponents of this tile came with their payload of tile k-A
      if (!m.Wait(me, c, 1, epoch - A)) return;
    }
    const size_t nblocks = (len + g.block - 1) / g.block;
    float* sf = m.Scale(me, c, k);
    for (size_t b = 0; b < nblocks; b++) {
      const uint64_t w = m.ExpWords(me, c, k)[b].load(std::memory_order_relaxed);
      if ((w >> 8) != epoch) m.mem[me]->protocol_errors++;
      sf[b] = quant::ScaleFactor(static_cast<int>(w & 0xff) - 128, g.ranks);
    }
    if (g.push) {
      for (int p = 0; p < g.ranks; p++) {
        if (p == me) continue;
        size_t sb, se;
        ShardOf(g, len, p, &sb, &se);
        int32_t* dst = m.Recv(p, c, k, me);
        for (size_t i = sb; i < se; i++) dst[i - sb] = quant::Quantize(in[pos + i], sf[i / g.block]);
      }
    } else {
      int32_t* mine = m.Data(me, c, k);
      for (size_t i = 0; i < len; i++) mine[i] = quant::Quantize(in[pos + i], sf[i / g.block]);
    }
    // Exponents of tile k+A, ahead of its data: its words were last used by tile k+A-S, which
    // every rank consumed before the signals awaited above (S >= 2A).
    if (A > 0 && k + A < ntiles) PublishTile(m, c, r, k + A, base, in);
    m.Signal(me, c, 1, epoch);
  }
}

void Reducer(Model& m, int me, int c, const float* in, float* out, size_t numel) {
  const Geometry& g = m.g;
  ChannelRange r = RangeOf(g, numel, c);
  const uint64_t base = m.mem[me]->epoch_words[c];
  const size_t ntiles = (r.end - r.begin + g.tile - 1) / g.tile;
  for (size_t k = 0; k < ntiles; k++) {
    const uint64_t epoch = base + k + 1;
    const size_t pos = r.begin + k * g.tile, len = std::min<size_t>(g.tile, r.end - pos);
    if (!m.Wait(me, c, 1, epoch)) return;
    if (g.push && k >= static_cast<size_t>(g.slots) && !m.Wait(me, c, 3, epoch - g.slots)) return;
    size_t sb, se;
    ShardOf(g, len, me, &sb, &se);
    const float* sf = m.Scale(me, c, k);
    for (size_t i = sb; i < se; i++) {
      uint32_t acc = 0;
      if (g.push) {
        acc = static_cast<uint32_t>(quant::Quantize(in[pos + i], sf[i / g.block]));
        for (int p = 0; p < g.ranks; p++)
          if (p != me) acc += static_cast<uint32_t>(m.Recv(me, c, k, p)[i - sb]);
      } else {
        for (int p = 0; p < g.ranks; p++) acc += static_cast<uint32_t>(m.Data(p, c, k)[i]);
      }
      const float y = quant::Dequantize(static_cast<int32_t>(acc), sf[i / g.block]);
      int32_t bits;
      memcpy(&bits, &y, 4);
      if (g.push) {
        out[pos + i] = y;
        for (int p = 0; p < g.ranks; p++)
          if (p != me) m.Result(p, c, k, me)[i - sb] = bits;
      } else {
        for (int p = 0; p < g.ranks; p++) m.Data(p, c, k)[i] = bits;  // the broadcast
      }
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
    const size_t pos = r.begin + k * g.tile, len = std::min<size_t>(g.tile, r.end - pos);
    if (!m.Wait(me, c, 2, epoch)) return;
    if (g.push) {
      for (int p = 0; p < g.ranks; p++) {
        if (p == me) continue;
        size_t sb, se;
        ShardOf(g, len, p, &sb, &se);
        if (se > sb) memcpy(out + pos + sb, m.Result(me, c, k, p), (se - sb) * 4);
      }
      m.Signal(me, c, 3, epoch);
    } else {
      memcpy(out + pos, m.Data(me, c, k), len * 4);
    }
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
      threads.emplace_back(Reducer, std::ref(m), r, c, in[r].data(), (*out)[r].data(), numel);
      threads.emplace_back(Storer, std::ref(m), r, c, (*out)[r].data(), numel);
    }
  }
  for (auto& t : threads) t.join();
  int failed = 0;
  for (int r = 0; r < g.ranks; r++) {
    failed += m.mem[r]->failed.load() + m.mem[r]->protocol_errors.load();
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
  const Geometry geometries[] = {{2, 2, 2, 64, 256, false, 4}, {3, 2, 1, 64, 384, false, 4}, {4, 3, 4, 32, 256, false, 4},
                                 {2, 2, 2, 64, 256, true, 4},  {3, 1, 1, 64, 384, true, 4},  {4, 3, 4, 32, 256, true, 4},
                                 {2, 1, 5, 64, 256, true, 3},  {2, 2, 3, 64, 256, false, 1}, {3, 2, 4, 64, 384, false, 2},
                                 {2, 2, 8, 64, 256, true, 2},  {2, 2, 2, 64, 256, false, 0}, {2, 1, 3, 64, 256, true, 0}};
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
        printf("  FAILED flag protocol model: a wait ran out or an exponent word had a foreign tag (%d ranks, %zu elements, %s)\n",
               g.ranks, numel, g.push ? "push" : "staged");
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
