// Native unit tests of the host-side building blocks. Prints one line per test and exits
// non-zero on the first failure; run by tests/test_native_core.py.
#include <arpa/inet.h>

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstddef>
#include <cstring>
#include <thread>
#include <vector>

#include "backends/softswitch/soft_switch.h"
#include "backends/timeout_queue.h"
#include "ppp/cpu_exponent_quantizer_ppp.h"
#include "rendezvous/control.h"
#include "simd/simd_kernels.h"
#include "switchml/context.h"
#include "switchml/log.h"
#include "switchml/quant_math.h"
#include "switchml/scheduler.h"
#include "switchml/utils.h"

using namespace switchml;

namespace switchml {
int RunFlagProtocolModel();  // flag_protocol_model.cc
}

static int g_failures = 0;
#define EXPECT(cond)                                                         \
  do {                                                                       \
    if (!(cond)) {                                                           \
      printf("  FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);             \
      g_failures++;                                                          \
    }                                                                        \
  } while (0)

static int g_sink_lines = 0;
static void CountingSink(int, const char*) { g_sink_lines++; }

static void TestLogging() {
  const int before = GetVerbosity();
  SetLogSink(CountingSink);
  SetVerbosity(1);
  g_sink_lines = 0;
  SML_VLOG(1) << "printed";
  SML_VLOG(2) << "not printed";
  SML_VLOG_IF(1, false) << "not printed";
  EXPECT(g_sink_lines == 1);
  // Per-module level: this file may speak up to 3, everything else keeps level 1.
  SetVModule("core_tests=3,control=0");
  EXPECT(SML_VLOG_IS_ON(3) && !SML_VLOG_IS_ON(4));
  EXPECT(VlogIsOn("/somewhere/csrc/rendezvous/control.cc", 0) && !VlogIsOn("csrc/rendezvous/control.cc", 1));
  EXPECT(VlogIsOn("udp_backend.cc", 1) && !VlogIsOn("udp_backend.cc", 2));
  EXPECT(!VlogIsOn("core_tests_more.cc", 3));  // whole names only
  SML_VLOG(3) << "printed";
  EXPECT(g_sink_lines == 2);
  SetVModule("");
  EXPECT(!SML_VLOG_IS_ON(2));
  SML_DVLOG(0) << "only in debug builds";
#ifdef SWITCHML_DEBUG
  EXPECT(g_sink_lines == 3);
#else
  EXPECT(g_sink_lines == 2);
#endif
  bool threw = false;
  try {
    SML_CHECK(1 + 1 == 3) << "arithmetic";
  } catch (const FatalError& e) {
    threw = std::string(e.what()).find("arithmetic") != std::string::npos;
  }
  EXPECT(threw);
  SetLogSink(nullptr);
  SetVerbosity(before);
}

static void TestSimdMatchesScalar() {
  // Whatever the AVX-512 loops compute must be what the scalar loops compute, bit for bit,
  // including NaN, infinities, denormals, values that saturate and every tail length.
  simd::Enable(true);
  if (!simd::Enabled()) {
    printf("  (no avx512f+avx512bw on this CPU: scalar loops only)\n");
    return;
  }
  std::vector<float> x(1000);
  uint32_t seed = 12345;
  auto next = [&] { seed = seed * 1664525u + 1013904223u; return seed; };
  for (size_t i = 0; i < x.size(); i++) {
    uint32_t bits = next();
    memcpy(&x[i], &bits, 4);  // random bit patterns: all exponents, NaNs, infinities, denormals
  }
  x[3] = 0.0f; x[4] = -0.0f; x[5] = 1e30f; x[6] = -1e30f; x[7] = 0.5f; x[8] = 1.5f; x[9] = 2.5f; x[10] = -2.5f;
  const float sfs[] = {1.0f, 1073741823.5f, 3.0e-30f, 2.5e9f, quant::ScaleFactor(-3, 8), quant::ScaleFactor(127, 3)};
  for (size_t n : {size_t(0), size_t(1), size_t(15), size_t(16), size_t(17), size_t(64), size_t(255), size_t(1000)}) {
    for (float sf : sfs) {
      std::vector<int32_t> a(n + 1, 0x5a5a5a5a), b(n + 1, 0x5a5a5a5a);
      std::vector<float> ya(n + 1, -1.0f), yb(n + 1, -1.0f);
      simd::Enable(true);
      float ma = simd::BlockMaxAbs(x.data(), n);
      simd::QuantizeToWire(x.data(), n, sf, a.data());
      simd::DequantizeFromWire(a.data(), n, sf, ya.data());
      simd::Enable(false);
      float mb = simd::BlockMaxAbs(x.data(), n);
      simd::QuantizeToWire(x.data(), n, sf, b.data());
      simd::DequantizeFromWire(b.data(), n, sf, yb.data());
      EXPECT(memcmp(&ma, &mb, 4) == 0);
      EXPECT(memcmp(a.data(), b.data(), (n + 1) * 4) == 0);   // n + 1: nothing written past the end
      EXPECT(memcmp(ya.data(), yb.data(), (n + 1) * 4) == 0);
    }
    std::vector<int32_t> in(n), s1(n + 1, 7), s2(n + 1, 7), acc1(n + 1, 1000), acc2(n + 1, 1000);
    for (size_t i = 0; i < n; i++) in[i] = static_cast<int32_t>(next());
    std::vector<uint8_t> wire(4 * n + 3);
    if (n) memcpy(wire.data() + 1, in.data(), 4 * n);   // odd address on purpose
    simd::Enable(true);
    simd::Swap32(in.data(), n, s1.data());
    simd::AddWire(wire.data() + 1, n, acc1.data());
    simd::Enable(false);
    simd::Swap32(in.data(), n, s2.data());
    simd::AddWire(wire.data() + 1, n, acc2.data());
    EXPECT(s1 == s2 && acc1 == acc2);
    if (n) EXPECT(static_cast<uint32_t>(s1[0]) == htonl(static_cast<uint32_t>(in[0])));
  }
  simd::Enable(true);
}

static void TestNumaHelpers() {
  int ids[1024], count = 0;
  // Node 0 exists on every Linux machine with NUMA information; without it the helpers say no.
  if (GetCoresNuma(0, ids, 1024, &count)) {
    EXPECT(count > 0 && ids[0] >= 0);
    std::thread t([] { EXPECT(BindToNumaNode(0)); });
    t.join();
  } else {
    EXPECT(count == 0 && !BindToNumaNode(0));
  }
  EXPECT(!GetCoresNuma(-1, ids, 1024, &count) && !GetCoresNuma(4095, ids, 1024, &count));
  EXPECT(GetDeviceNuma("ffff:ff:1f.7") == -1);
}

static void TestStaticSlice() {
  // 10 elements over 4 threads: 3,3,2,2 at offsets 0,3,6,8 (remainder to the first threads)
  Numel off, len;
  Numel want_off[] = {0, 3, 6, 8}, want_len[] = {3, 3, 2, 2};
  for (int i = 0; i < 4; i++) {
    StaticSlice(10, 4, i, &off, &len);
    EXPECT(off == want_off[i] && len == want_len[i]);
  }
  Numel total = 0;
  for (int i = 0; i < 7; i++) {
    StaticSlice(1000003, 7, i, &off, &len);
    EXPECT(off == total);
    total += len;
  }
  EXPECT(total == 1000003);
  StaticSlice(2, 4, 3, &off, &len);
  EXPECT(len == 0);
}

static void TestBarrier() {
  const int n = 4, rounds = 50;
  Barrier b(n);
  std::atomic<int> counter{0};
  std::atomic<int> errors{0};
  std::vector<std::thread> th;
  for (int t = 0; t < n; t++) {
    th.emplace_back([&] {
      for (int r = 0; r < rounds; r++) {
        counter++;
        if (!b.Wait()) errors++;
        if (counter.load() < (r + 1) * n) errors++;
        if (!b.Wait()) errors++;
      }
    });
  }
  for (auto& t : th) t.join();
  EXPECT(errors == 0);
  // Destroy releases waiters and poisons the barrier.
  Barrier d(2);
  std::thread w([&] { EXPECT(!d.Wait()); });
  std::this_thread::sleep_for(std::chrono::milliseconds(20));
  d.Destroy();
  w.join();
  EXPECT(!d.Wait());
}

static void TestJobFsm() {
  Tensor t;
  ExtraJobInfo x;
  x.allreduce_operation = SUM;
  Job j(t, ALLREDUCE, x);
  Job j2(t, ALLREDUCE, x);
  EXPECT(j2.id_ == j.id_ + 1);
  EXPECT(j.GetJobStatus() == INIT);
  j.SetJobStatus(QUEUED);
  j.SetJobStatus(RUNNING);
  bool threw = false;
  try { j.SetJobStatus(QUEUED); } catch (const FatalError&) { threw = true; }
  EXPECT(threw);
  EXPECT(!j.WaitToCompleteFor(5));
  std::thread fin([&] { j.SetJobStatus(FINISHED); });
  j.WaitToComplete();
  fin.join();
  threw = false;
  try { j.SetJobStatus(FAILED); } catch (const FatalError&) { threw = true; }
  EXPECT(threw);
}

static void TestTimeoutQueue() {
  typedef TimeoutQueue::TimePoint TP;
  TP t0 = std::chrono::steady_clock::now();
  auto at = [&](int ms) { return t0 + std::chrono::milliseconds(ms); };
  TimeoutQueue q(4, 10.0, 2, 2);
  EXPECT(q.Check(at(100)) == -1);
  q.Push(0, at(0));
  q.Push(1, at(1));
  q.Push(2, at(2));
  EXPECT(q.Check(at(5)) == -1);
  EXPECT(q.Check(at(10)) == 0);      // oldest first
  q.Push(0, at(10));                  // retransmitted: becomes the youngest
  EXPECT(q.Check(at(11)) == 1);      // second timeout: threshold reached, timeout doubles
  EXPECT(std::fabs(q.timeout_ms() - 20.0) < 1e-9);
  q.Remove(1);
  EXPECT(q.Check(at(12)) == -1);     // entry 2 is 10 ms old, budget is now 20
  EXPECT(q.Check(at(22)) == 2);
  q.Remove(2);
  q.Remove(0);
  EXPECT(q.Empty());
  EXPECT(q.timeouts() == 3);
}

static std::vector<uint8_t> MakePacket(int worker, uint16_t pool_index, uint32_t pkt_id, int8_t exp,
                                       const std::vector<int32_t>& v, uint64_t session) {
  std::vector<uint8_t> b(sizeof(WireHeader) + v.size() * 4);
  WireHeader h;
  h.magic = htonl(kWireMagic);
  h.type = WIRE_DATA;
  h.job_tag = 7;
  h.worker_id = htons(static_cast<uint16_t>(worker));
  h.pkt_id = htonl(pkt_id);
  h.pool_index = htons(pool_index);
  h.numel = htons(static_cast<uint16_t>(v.size()));
  h.exponent = exp;
  h.thread_id = 0;
  h.session_lo = htons(static_cast<uint16_t>(session));
  memcpy(b.data(), &h, sizeof(h));
  for (size_t i = 0; i < v.size(); i++) {
    uint32_t be = htonl(static_cast<uint32_t>(v[i]));
    memcpy(b.data() + sizeof(h) + 4 * i, &be, 4);
  }
  return b;
}

static int32_t PayloadAt(const SwitchOutput& o, int i) {
  uint32_t be;
  memcpy(&be, o.bytes.data() + sizeof(WireHeader) + 4 * i, 4);
  return static_cast<int32_t>(ntohl(be));
}

static void TestSoftSwitch() {
  SoftSwitch sw(64);
  sw.Reset(42, 3, 4);
  for (int w = 0; w < 3; w++) EXPECT(sw.AddWorker(w));
  EXPECT(!sw.AddWorker(3));
  std::vector<SwitchOutput> out;
  auto send = [&](int w, uint16_t idx, uint32_t id, int8_t e, std::vector<int32_t> v) {
    auto p = MakePacket(w, idx, id, e, v, 42);
    sw.Process(p.data(), p.size(), &out);
  };
  // Two of three workers: nothing comes out yet.
  send(0, 5, 100, -3, {1, 2, 3, 4});
  send(1, 5, 100, 2, {10, 20, 30, 2147483647});
  EXPECT(out.empty());
  EXPECT(sw.Bitmap(5, 0) == 0x3);
  // A duplicate of worker 0 while the slot is still open is ignored.
  send(0, 5, 100, -3, {1, 2, 3, 4});
  EXPECT(out.empty());
  // Third worker completes the slot: multicast to all three, exponent = max, wrapping add.
  send(2, 5, 100, 0, {100, 200, 300, 1});
  EXPECT(out.size() == 3);
  if (out.size() == 3) {
    WireHeader h;
    memcpy(&h, out[1].bytes.data(), sizeof(h));
    EXPECT(h.type == WIRE_RESULT && h.exponent == 2 && ntohl(h.pkt_id) == 100 && h.job_tag == 7);
    EXPECT(out[1].dest_worker == 1);
    EXPECT(PayloadAt(out[0], 0) == 111 && PayloadAt(out[0], 2) == 333);
    EXPECT(PayloadAt(out[0], 3) == static_cast<int32_t>(2147483647u + 4u + 1u));  // wrapped
  }
  // A retransmission to the finished slot is answered to that worker only.
  out.clear();
  send(1, 5, 100, 2, {10, 20, 30, 40});
  EXPECT(out.size() == 1 && out[0].dest_worker == 1);
  if (!out.empty()) {
    WireHeader h;
    memcpy(&h, out[0].bytes.data(), sizeof(h));
    EXPECT(h.type == WIRE_RESULT_RETX);
    EXPECT(PayloadAt(out[0], 0) == 111);
  }
  // Using the other set acknowledges this one (bits cleared one worker at a time).
  out.clear();
  send(0, 5 | kSetBit, 164, 0, {1, 1, 1, 1});
  EXPECT(sw.Bitmap(5, 0) == 0x6 && sw.Bitmap(5, 1) == 0x1);
  send(1, 5 | kSetBit, 164, 0, {1, 1, 1, 1});
  send(2, 5 | kSetBit, 164, 0, {1, 1, 1, 1});
  EXPECT(out.size() == 3 && sw.Bitmap(5, 0) == 0);
  // Set 0 is free again: a new first packet overwrites instead of adding.
  out.clear();
  send(2, 5, 228, 1, {7, 7, 7, 7});
  send(0, 5, 228, 1, {1, 1, 1, 1});
  send(1, 5, 228, 1, {1, 1, 1, 1});
  EXPECT(out.size() == 3 && PayloadAt(out[0], 0) == 9);
  // Per-slot counters of slot 5 so far: set 0 finished twice (one retransmission answered, one
  // duplicate ignored), set 1 once.
  EXPECT(sw.DescribeSlot(5).find(" 0  7  0  yes  2  1  4  1") != std::string::npos);
  EXPECT(sw.DescribeSlot(5).find(" 1  0  0  yes  1  0  2  0") != std::string::npos);
  // Wrong session, unknown worker, short packet: counted as malformed, no output.
  out.clear();
  auto bad = MakePacket(0, 5, 1, 0, {1}, 43);
  sw.Process(bad.data(), bad.size(), &out);
  bad = MakePacket(9, 5, 1, 0, {1}, 42);
  sw.Process(bad.data(), bad.size(), &out);
  sw.Process(bad.data(), 3, &out);
  EXPECT(out.empty() && sw.counters().malformed == 3);
  // A valid session and worker, but a thread id beyond the return-port table: refused
  // before any slot state is touched (slot 11 stays empty).
  bad = MakePacket(0, 11, 1, 0, {1}, 42);
  bad[offsetof(WireHeader, thread_id)] = 200;
  sw.Process(bad.data(), bad.size(), &out);
  EXPECT(out.empty() && sw.counters().malformed == 4 && sw.Bitmap(11, 0) == 0);
  // Drop simulator: everything dropped on ingress.
  sw.SetDropProbabilities(1.0, 0.0, 1);
  send(0, 9, 1, 0, {1, 1, 1, 1});
  EXPECT(sw.counters().ingress_dropped == 1 && sw.Bitmap(9, 0) == 0);
  sw.SetDropProbabilities(0.0, 1.0, 1);
  send(0, 9, 1, 0, {1, 1, 1, 1});
  send(1, 9, 1, 0, {1, 1, 1, 1});
  send(2, 9, 1, 0, {1, 1, 1, 1});
  EXPECT(out.empty() && sw.counters().egress_dropped == 3);
  // The drops are also counted per worker, the traffic per worker thread.
  EXPECT(sw.worker_counters(0).ingress_dropped == 1 && sw.worker_counters(1).ingress_dropped == 0);
  EXPECT(sw.worker_counters(0).egress_dropped + sw.worker_counters(1).egress_dropped +
         sw.worker_counters(2).egress_dropped == 3);
  EXPECT(sw.endpoint_counters(1, 0).out_of_order == 1);          // its retransmission above
  EXPECT(sw.endpoint_counters(1, 0).retransmitted_results == 1);
  EXPECT(sw.endpoint_counters(0, 0).out_of_order == 1);          // the duplicate while the slot was open
  EXPECT(sw.endpoint_counters(2, 0).results == 3 && sw.endpoint_counters(2, 0).out_of_order == 0);
  EXPECT(sw.DescribeDropped().find(" total  1  3") != std::string::npos);
  EXPECT(sw.DescribeEndpoints().find(" 1  0  ") != std::string::npos);
  // Echo: answered to the sender whoever it is, payload unchanged; the drop simulator does
  // not apply.
  sw.SetDropProbabilities(1.0, 1.0, 1);
  out.clear();
  auto echo = MakePacket(17, 0, 77, 0, {123, 456}, 9999);
  echo[offsetof(WireHeader, type)] = WIRE_ECHO_REQUEST;
  sw.Process(echo.data(), echo.size(), &out);
  EXPECT(out.size() == 1 && out[0].to_sender && out[0].bytes.size() == echo.size());
  if (!out.empty()) {
    EXPECT(out[0].bytes[offsetof(WireHeader, type)] == WIRE_ECHO_REPLY && PayloadAt(out[0], 1) == 456);
  }
  EXPECT(sw.counters().echo_replies == 1);
  // Forwarding between registered workers: unicast by (worker, thread), flood to all others.
  out.clear();
  auto fwd = MakePacket(0, static_cast<uint16_t>(2 << 8 | 3), 5, 0, {42}, 42);
  fwd[offsetof(WireHeader, type)] = WIRE_FORWARD;
  sw.Process(fwd.data(), fwd.size(), &out);
  EXPECT(out.size() == 1 && out[0].dest_worker == 2 && out[0].dest_thread == 3 && !out[0].to_sender);
  EXPECT(!out.empty() && PayloadAt(out[0], 0) == 42);
  out.clear();
  fwd = MakePacket(1, static_cast<uint16_t>(kFloodWorker << 8 | 0), 5, 0, {43}, 42);
  fwd[offsetof(WireHeader, type)] = WIRE_FORWARD;
  sw.Process(fwd.data(), fwd.size(), &out);
  EXPECT(out.size() == 2 && out[0].dest_worker == 0 && out[1].dest_worker == 2);
  out.clear();
  uint64_t malformed = sw.counters().malformed;
  fwd = MakePacket(0, static_cast<uint16_t>(7 << 8), 5, 0, {44}, 42);  // worker 7 does not exist
  fwd[offsetof(WireHeader, type)] = WIRE_FORWARD;
  sw.Process(fwd.data(), fwd.size(), &out);
  fwd = MakePacket(0, static_cast<uint16_t>(1 << 8), 5, 0, {44}, 41);  // another session
  fwd[offsetof(WireHeader, type)] = WIRE_FORWARD;
  sw.Process(fwd.data(), fwd.size(), &out);
  EXPECT(out.empty() && sw.counters().malformed == malformed + 2);
  EXPECT(sw.counters().forwarded == 1 && sw.counters().flooded == 1);
  // A message of two packets on slots 12 and 13: the first says "more follow" and leaves the
  // exponent register alone whatever its header holds; the last carries the exponents.
  sw.SetDropProbabilities(0, 0);
  out.clear();
  for (int w = 0; w < 3; w++) {
    auto more = MakePacket(w, 12, 24, 99, {1, 2, 3, 4}, 42);
    more[offsetof(WireHeader, type)] = WIRE_DATA_MORE;
    sw.Process(more.data(), more.size(), &out);
  }
  EXPECT(out.size() == 3 && PayloadAt(out[0], 3) == 12);
  if (out.size() == 3) EXPECT(static_cast<int8_t>(out[0].bytes[offsetof(WireHeader, exponent)]) == -128);
  out.clear();
  send(0, 13, 25, 3, {1, 1, 1, 1});
  send(1, 13, 25, 9, {1, 1, 1, 1});
  send(2, 13, 25, 5, {1, 1, 1, 1});
  EXPECT(out.size() == 3);
  if (out.size() == 3) EXPECT(static_cast<int8_t>(out[0].bytes[offsetof(WireHeader, exponent)]) == 9);
  // Single worker: every packet completes its slot at once.
  sw.SetDropProbabilities(0, 0);
  sw.Reset(1, 1, 4);
  sw.AddWorker(0);
  out.clear();
  auto p1 = MakePacket(0, 0, 0, 0, {5, 6, 7, 8}, 1);
  sw.Process(p1.data(), p1.size(), &out);
  EXPECT(out.size() == 1 && PayloadAt(out[0], 3) == 8);
}

static void TestSoftSwitchConcurrentPipes() {
  // Four threads feed the switch at once, each playing all three workers of "its" slots
  // (what a pipe of the data plane does), while a fifth reads tables: every slot must
  // complete exactly once with the right sum, and the counters must add up.
  const int kPipes = 4, kSlotsPerPipe = 16, kRounds = 200, kWorkers = 3;
  SoftSwitch sw(256);
  sw.Reset(77, kWorkers, 4);
  for (int w = 0; w < kWorkers; w++) EXPECT(sw.AddWorker(w));
  std::atomic<int> wrong{0};
  std::atomic<bool> reading{true};
  std::thread reader([&] {
    while (reading) {
      (void)sw.DescribeStatistics();
      (void)sw.DescribeWorkers();
      (void)sw.Bitmap(3, 0);
      (void)sw.counters();
    }
  });
  std::vector<std::thread> pipes;
  for (int p = 0; p < kPipes; p++) {
    pipes.emplace_back([&, p] {
      std::vector<SwitchOutput> out;
      for (int round = 0; round < kRounds; round++) {
        for (int s = 0; s < kSlotsPerPipe; s++) {
          uint16_t idx = static_cast<uint16_t>(p * kSlotsPerPipe + s) | ((round & 1) ? kSetBit : 0);
          out.clear();
          for (int w = 0; w < kWorkers; w++) {
            auto pkt = MakePacket(w, idx, static_cast<uint32_t>(round), static_cast<int8_t>(w),
                                  {w + 1, round, p, s}, 77);
            pkt[offsetof(WireHeader, thread_id)] = static_cast<uint8_t>(p);
            sw.Process(pkt.data(), pkt.size(), &out);
          }
          if (out.size() != static_cast<size_t>(kWorkers) || PayloadAt(out[0], 0) != 6 ||
              PayloadAt(out[0], 1) != 3 * round || PayloadAt(out[2], 3) != 3 * s) wrong++;
        }
      }
    });
  }
  for (auto& t : pipes) t.join();
  reading = false;
  reader.join();
  EXPECT(wrong == 0);
  const uint64_t slots_done = static_cast<uint64_t>(kPipes) * kSlotsPerPipe * kRounds;
  EXPECT(sw.counters().broadcast == slots_done && sw.counters().consumed == slots_done * (kWorkers - 1));
  EXPECT(sw.worker_counters(1).rx_packets == slots_done && sw.worker_counters(2).tx_packets == slots_done);
  EXPECT(sw.endpoint_counters(0, 3).rx_packets == static_cast<uint64_t>(kSlotsPerPipe) * kRounds);
}

static void TestFlagProtocolModel() {
  // The cross-GPU flag protocol of the aggregation kernels as a host model with real threads
  // (three roles per channel and rank): bit-exact against the oracle, and race-free when this
  // binary is built with -fsanitize=thread.
  EXPECT(RunFlagProtocolModel() == 0);
}

static void TestQuantMath() {
  using namespace quant;
  EXPECT(LocalExponent(0.0f) == -126);
  EXPECT(LocalExponent(1.0f) == 1);      // 2^1 > 1
  EXPECT(LocalExponent(0.75f) == 0);     // 2^0 > 0.75
  EXPECT(LocalExponent(3.0f) == 2);
  EXPECT(LocalExponent(INFINITY) == 127);
  EXPECT(ScaleFactor(1, 2) == 536870912.0f);  // (2^31-1)/(2*2) rounds to 2^29 in float
  EXPECT(std::isfinite(ScaleFactor(-126, 8)));
  EXPECT(Quantize(0.5f, 4.0f) == 2 && Quantize(0.625f, 4.0f) == 2 && Quantize(0.875f, 4.0f) == 4);
  EXPECT(Quantize(NAN, 1.0f) == 0 && Quantize(1e30f, 1e30f) == INT32_MAX);
  // The float-only scale factor used on the GPU equals the double-precision definition.
  for (int n = 1; n <= 32; n++)
    for (int e = -130; e <= 130; e++) EXPECT(ScaleFactorFromBase(e, QuantBase(n)) == ScaleFactor(e, n));
  // Oracle: exact for values that are representable at the block scale.
  std::vector<float> a = {1.0f, -2.0f, 0.5f, 0.0f}, b = {0.25f, 4.0f, -0.5f, 0.0f}, out(4);
  const float* in[2] = {a.data(), b.data()};
  OracleQuantAllReduce(in, 2, 4, 4, out.data());
  EXPECT(out[0] == 1.25f && out[1] == 2.0f && out[2] == 0.0f && out[3] == 0.0f);
  // All-zero block stays zero (no NaN from an infinite scale).
  std::vector<float> z(8, 0.0f);
  const float* zin[2] = {z.data(), z.data()};
  std::vector<float> zo(8, 1.0f);
  OracleQuantAllReduce(zin, 2, 8, 4, zo.data());
  for (float v : zo) EXPECT(v == 0.0f);
}

static void TestControlPlane() {
  ControlServer s;
  EXPECT(s.Start("127.0.0.1", 0, 0));
  const int n = 3;
  std::vector<std::thread> th;
  std::atomic<int> errors{0};
  for (int r = 0; r < n; r++) {
    th.emplace_back([&, r] {
      ControlClient c;
      if (!c.Connect("127.0.0.1", s.port(), 2000)) { errors++; return; }
      for (int round = 0; round < 3; round++) {
        uint64_t v = r == 1 ? 1000 + round : 0;
        if (!c.Broadcast(n, r, 1, &v) || v != static_cast<uint64_t>(1000 + round)) errors++;
        std::vector<std::string> all;
        if (!c.AllGather(n, r, "tok" + std::to_string(r * 10 + round), &all)) errors++;
        for (int k = 0; k < n && all.size() == static_cast<size_t>(n); k++)
          if (all[k] != "tok" + std::to_string(k * 10 + round)) errors++;
        if (!c.Barrier(n)) errors++;
      }
    });
  }
  for (auto& t : th) t.join();
  EXPECT(errors == 0);
  ControlClient cli;
  EXPECT(cli.Connect("127.0.0.1", s.port(), 2000));
  std::string reply;
  EXPECT(cli.Command("SET drop 0.25 0.5 7", &reply));
  EXPECT(cli.Command("SHOW drop", &reply) && reply.find("0.25") != std::string::npos);
  EXPECT(!cli.Command("BOGUS", &reply));
  s.Stop();
}

static void TestContextDummy() {
  Config cfg;
  EXPECT(cfg.LoadFromString("[general]\nbackend = dummy\nnum_workers = 3\nnum_worker_threads = 3\n"
                            "max_outstanding_packets = 10\npacket_numel = 64\n"
                            "[backend.dummy]\nbandwidth = 0\n"));
  Context& ctx = Context::GetInstance();
  EXPECT(ctx.Start(&cfg));
  EXPECT(ctx.GetConfig().general_.max_outstanding_packets == 9);  // rounded to a multiple of 3
  const int numel = 100003;
  std::vector<float> in(numel), out(numel);
  for (int i = 0; i < numel; i++) in[i] = std::sin(i * 0.37f) * (i % 97);
  std::vector<std::shared_ptr<Job>> jobs;
  for (int k = 0; k < 4; k++) jobs.push_back(ctx.AllReduceAsync(in.data(), out.data(), numel, FLOAT32, SUM));
  ctx.WaitForAllJobs();
  for (auto& j : jobs) EXPECT(j->GetJobStatus() == FINISHED);
  double worst = 0;
  for (int i = 0; i < numel; i++) worst = std::max(worst, std::fabs(out[i] - 3.0 * in[i]));
  EXPECT(worst < 1e-4);
  std::vector<int32_t> iin(1000), iout(1000);
  for (int i = 0; i < 1000; i++) iin[i] = i - 500;
  auto j = ctx.AllReduce(iin.data(), iout.data(), 1000, INT32, SUM);
  EXPECT(j->GetJobStatus() == FINISHED && iout[0] == -1500 && iout[999] == 1497);
  EXPECT(ctx.GetStats().jobs_finished_num() == 5);
  ctx.Stop();
  EXPECT(ctx.GetContextState() == Context::STOPPED);
  bool threw = false;
  try { ctx.AllReduce(iin.data(), iout.data(), 10, INT32, SUM); } catch (const FatalError&) { threw = true; }
  EXPECT(threw);
  // Restart with instant completion: plumbing only, data untouched.
  Config c2;
  c2.LoadFromString("[general]\nbackend = dummy\ninstant_job_completion = true\n");
  EXPECT(ctx.Start(&c2));
  iout.assign(1000, -7);
  ctx.AllReduce(iin.data(), iout.data(), 1000, INT32, SUM);
  EXPECT(iout[10] == -7);
  ctx.Stop();
}

int main() {
  SetVerbosity(0);
  struct { const char* name; void (*fn)(); } tests[] = {
      {"logging", TestLogging}, {"numa_helpers", TestNumaHelpers}, {"simd_matches_scalar", TestSimdMatchesScalar}, {"static_slice", TestStaticSlice}, {"barrier", TestBarrier}, {"job_fsm", TestJobFsm},
      {"timeout_queue", TestTimeoutQueue}, {"soft_switch", TestSoftSwitch}, {"soft_switch_concurrent_pipes", TestSoftSwitchConcurrentPipes},
      {"quant_math", TestQuantMath}, {"flag_protocol_model", TestFlagProtocolModel}, {"control_plane", TestControlPlane},
      {"context_dummy", TestContextDummy},
  };
  for (auto& t : tests) {
    int before = g_failures;
    t.fn();
    printf("%s %s\n", g_failures == before ? "ok  " : "FAIL", t.name);
    fflush(stdout);
  }
  return g_failures ? 1 : 0;
}
