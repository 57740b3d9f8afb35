// Host-side interface of the aggregation kernels (sm_100a).
//
// One launch = one allreduce job on one rank. All ranks launch the same kernel with the
// same geometry; the kernels meet through flags in symmetric memory (device_sync.cuh).
// The kernels stand in for the reference's worker hot loops + prepostprocessor + switch
// pipeline: quantise (cpu_exponent_quantizer_ppp.cc:88-156), exponent max
// (p4/exponents.p4:48-54), integer add (p4/processor.p4:48-54), multicast of the result
// (p4/next_step_selector.p4:118-129), dequantise (cpu_exponent_quantizer_ppp.cc:200-260),
// streamed through a ring of staging slots like the switch's slot pool.
#ifndef SWITCHML_ALLREDUCE_KERNELS_H_
#define SWITCHML_ALLREDUCE_KERNELS_H_

#include <cuda_runtime.h>
#include <stdint.h>

namespace switchml {
namespace kernels {

static const int kMaxRanks = 8;
static const int kMaxChannels = 512;
static const int kNumPhases = 4;
static const int kThreads = 512;            // threads per CTA of every aggregation kernel
static const int kExpRing = 8;              // exponent slots per channel, at least (a slot per data slot if those are more)
static const int kTraceTiles = 64;          // tiles per job that the per-tile trace remembers
static const int kTraceWords = 6 * kTraceTiles + 1;  // [role][began, finished][tile] in ns of %globaltimer, then the job's start
static const int kFlagWordsPerChannel = kNumPhases * kMaxRanks;
// Layout of a rank's symmetric staging region (byte offsets from its base).
static const size_t kFlagBytes = size_t(kMaxChannels) * kFlagWordsPerChannel * 8;  // 128 KiB of 64-bit epochs

enum ElemType : int { ELEM_F32 = 0, ELEM_I32 = 1, ELEM_BF16 = 2 };
enum ReduceMode : int {
  MODE_SUM = 0,    // float add in f32 (bf16 inputs accumulate in f32) / wrapping int add
  MODE_QUANT = 1,  // per-block exponent fixed point: exact, order-independent integer sum
};
enum Algo : int {
  ALGO_STAGED = 0,    // copy-in, shard reduce, copy-out through the slot ring (any pointers)
  ALGO_ONESHOT = 1,   // push inputs to every rank, one barrier, reduce locally (small messages)
  ALGO_ZEROCOPY = 2,  // tensors live in symmetric memory: reduce in place, no staging (SUM only)
  ALGO_PUSH = 3,      // peer-memory transport: shards pushed to their owners and results pushed back,
                      // posted stores only (push_allreduce.cuh); needs at least two ranks
};
enum Status : int {
  STATUS_OK = 0,
  STATUS_TIMEOUT = 1,  // a bounded wait ran out; bits 8.. hold the channel, 4..7 the phase
  STATUS_BAD_ARGS = 2,
  STATUS_BOUNDS = 3,   // checked build only: a tile or buffer would reach outside its region (bits 8.. = channel)
  STATUS_PROTOCOL = 4, // an exponent word carried the tag of another tile: the ranks are not running the same job
};

// What a rank's kernel needs to reach its peers. Passed by value.
struct RankCtx {
  int rank;
  int nranks;
  int use_multimem;              // 1: reduce/broadcast through the multicast mapping
  char* stage_peer[kMaxRanks];   // every rank's staging region as mapped here ([rank] = own)
  char* stage_mc;                // multicast mapping of the staging regions (or nullptr)
  size_t data_offset;            // start of the data slots inside the region
  size_t exp_offset;             // start of the exponent slots
  size_t oneshot_offset;         // start of the one-shot buffers
  size_t slot_bytes;             // bytes of one data slot
  int slots_per_channel;
  int sc_fence;                  // 1: a sequentially consistent system fence before every flag store (signal_fence = sc);
                                 // 0: the flag's release store alone orders the data before it
  int exp_ring;                  // exponent slots per channel: a ring of its own, ExpRingDepth(slots_per_channel)
  int exp_lookahead;             // how many tiles the exponents travel ahead of their data (2 * lookahead <= ring)
  int block_numel;               // quantisation block (= packet_numel)
  float quant_base;              // quant::QuantBase(nranks): scale factor at exponent 0
  size_t oneshot_bytes;          // capacity of one rank's one-shot buffer (per parity)
  size_t stage_bytes;            // size of one rank's staging region (what the checked build verifies against)
  unsigned long long timeout_ns; // budget of every wait
  int* status;                   // device-visible status word (0 = ok)
  unsigned long long* counters;  // [0] tiles processed, [1] wait iterations, [2] timeouts
  unsigned long long* trace;     // nullptr, or kTraceWords words in this rank's device memory: when channel 0's roles
                                 // began and finished each of a job's first kTraceTiles tiles ([backend.cuda] trace)
  unsigned long long* epoch_words;  // [kMaxChannels] in this rank's device memory: the epoch each channel has
                                 // reached. Kept on the device so that a captured launch can be replayed.
};

struct JobArgs {
  const void* in;
  void* out;
  unsigned long long numel;
  int elem_type;     // ElemType
  int mode;          // ReduceMode
  int algo;          // Algo
  float post_scale;  // multiplied into the result (1/num_workers for averaging)
  unsigned epochs;      // how far the job advances the epoch counter of each channel it uses
  int trailing_barrier; // ALGO_ONESHOT: meet once more after reading, so the buffer needs no parity (graph replays)
  int oneshot_parity;
  int bulk_copy;     // `in` and `out` are ordinary device memory of this GPU: whole-tile copies may go through the
                     // TMA unit (never set for pinned host or managed memory)
  int out_zero_copy; // ALGO_STAGED / ALGO_PUSH: `out` lies in the symmetric user region (user_* and out_offset are
                     // set): finished shards are broadcast straight into every rank's output, no copy-out
  unsigned long long tile_elems;  // ALGO_STAGED: elements per tile (<= elements of a slot)
  // ALGO_ZEROCOPY (and out_zero_copy): offsets of in/out inside the symmetric user region and its mappings
  char* user_peer[kMaxRanks];
  char* user_mc;
  size_t in_offset, out_offset;
  size_t user_bytes;  // size of the symmetric user region (checked build)
};

// Geometry chosen on the host; identical on every rank for the same job.
struct LaunchPlan {
  int channels;            // CTAs
  unsigned epochs;         // how far the job advances the epoch counter
  unsigned long long elems_per_channel;  // contiguous range of each channel (last may be short)
  unsigned long long tiles;              // staged tiles summed over channels (stats)
  unsigned long long tile_elems;         // ALGO_STAGED: copy into JobArgs::tile_elems
};

// The exponent words of a channel form a ring of their own: they are 1/128 of the data, so
// the ring can be deeper than the data slots and the exponents can run further ahead.
inline int ExpRingDepth(int slots_per_channel) { return slots_per_channel > kExpRing ? slots_per_channel : kExpRing; }
// Tiles by which exponents run ahead of their data: `wanted` clamped to half the ring; none
// with a single data slot (every tile then meets over its own exponents first).
inline int ExpLookahead(int slots_per_channel, int wanted) {
  if (slots_per_channel < 2 || wanted < 0) return 0;
  const int most = ExpRingDepth(slots_per_channel) / 2;
  return wanted > most ? most : wanted;
}
// Default: none. Every tile's exponents are published right before it is quantised, so the
// quantising pass finds the tile in L2 (with lookahead the exponent pass runs A tiles ahead and
// its data is evicted again: all channels together touch 74 MB per tile step), and the loaders
// have time for the extra meeting: they are several times faster than the reducers.
static const int kDefaultExpLookahead = 0;

// True if `p` is device memory (cudaMalloc or the virtual-memory API), not pinned host or managed memory.
bool DeviceMemory(const void* p);
// Number of elements of a slot for this element type / mode.
size_t SlotElems(const RankCtx& ctx, int elem_type, int mode);
// Largest tile of ALGO_PUSH that fits a slot (a multiple of nranks * max(block, 128)
// elements), or 0 when the slots are too small for that algorithm (use ALGO_STAGED then).
size_t PushTileCapacity(const RankCtx& ctx, int elem_type, int mode);
// Bytes a staging region must have for `channels` channels.
size_t StagingBytes(size_t slot_bytes, int slots_per_channel, int block_numel, int max_channels,
                    size_t oneshot_bytes, int nranks, size_t* data_offset, size_t* exp_offset,
                    size_t* oneshot_offset);
// The value for RankCtx::stage_bytes: `actual`, the size of the region. In a checked build
// the environment variable SWITCHML_CHECKED_PRETEND_STAGE_BYTES replaces it, so that a test
// can watch the geometry checks refuse every tile (the memory itself stays as large as it
// was, and a refused tile is not touched anyway).
size_t ReportedStageBytes(size_t actual);
// True if the library was compiled with -DSWITCHML_CHECKED.
bool CheckedBuild();

LaunchPlan PlanLaunch(const RankCtx& ctx, const JobArgs& job, int requested_channels,
                      int max_channels);
// Enqueue the job on `stream`. Returns cudaSuccess or the launch error.
cudaError_t LaunchAllReduce(const RankCtx& ctx, const JobArgs& job, const LaunchPlan& plan,
                            cudaStream_t stream);
// Single-GPU emulation of `nranks` ranks: one cooperative launch whose blockIdx.y is the
// rank, every "peer" region living on the same device. `ctxs`/`jobs` are device arrays
// of length nranks. Exercises the peer-memory code path bit for bit.
// `job0` is the host copy of jobs_dev[0] (selects the instantiation).
cudaError_t LaunchAllReduceEmulated(const RankCtx* ctxs_dev, const JobArgs* jobs_dev,
                                    const JobArgs& job0, int nranks, const LaunchPlan& plan,
                                    cudaStream_t stream);
// Single worker, plain sum, out of place: copy `bytes` bytes with one kernel.
cudaError_t LaunchLocalCopy(const void* in, void* out, size_t bytes, cudaStream_t stream);
// Single worker, exact mode, float32, both pointers 16-byte aligned: the quantise / dequantise round
// trip in one pass (bit-identical to what the streaming kernels give one worker).
cudaError_t LaunchLocalQuant(const void* in, void* out, size_t numel, int block_numel, float quant_base,
                             float post_scale, cudaStream_t stream);
// uint8 tensors travel as int32: zero-extend `numel` bytes into int32 scratch, and keep the
// low byte of every int32 on the way back (the sum modulo 256).
cudaError_t LaunchWidenU8(const void* in, void* out, size_t numel, cudaStream_t stream);
cudaError_t LaunchNarrowI32(const void* in, void* out, size_t numel, cudaStream_t stream);
// A kernel whose only job is to wait for a flag nobody sets: checks that a bounded wait
// gives up, reports STATUS_TIMEOUT and leaves the context usable.
cudaError_t LaunchWaitProbe(const RankCtx& ctx, cudaStream_t stream);

}  // namespace kernels
}  // namespace switchml
#endif  // SWITCHML_ALLREDUCE_KERNELS_H_
