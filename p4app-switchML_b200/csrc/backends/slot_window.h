// SlotWindow: the self-clocked streaming loop every packet backend runs per job slice.
//
// A worker thread owns `window` slots. It fills the window with the first packets of the
// slice, then for every result that comes back it post-processes it and immediately
// sends the packet `window` ids later into the same slot, until all packets are
// answered. Slot s therefore only ever carries packet ids congruent to s modulo the
// window, identically on every worker. Float slices send one extra leading batch (see
// CpuExponentQuantizerPPP). This is the common core of the reference's three hot loops
// (dummy_worker_thread.cc:90-184, dpdk_worker_thread.cc:199-402,
// rdma_worker_thread.cc:169-300); the transports differ only in Send/Poll.
#ifndef SWITCHML_SLOT_WINDOW_H_
#define SWITCHML_SLOT_WINDOW_H_

#include <cstdint>
#include <vector>

#include "switchml/common.h"
#include "switchml/job.h"
#include "switchml/prepostprocessor.h"

namespace switchml {

struct SlotPacket {
  uint32_t pkt_id = 0;
  int slot = 0;            // local slot index in [0, window)
  uint16_t numel = 0;      // payload elements
  int8_t exponent = 0;
  int32_t* payload = nullptr;  // network byte order, packet_numel entries
};

// What a transport must provide to SlotWindow::Run.
class SlotTransport {
 public:
  virtual ~SlotTransport() {}
  // Hand one filled packet to the wire. The transport may hold it back until Flush(); the
  // packet's payload stays untouched until the slot has been answered.
  virtual void Send(const SlotPacket& p, bool retransmission) = 0;
  // Put everything handed to Send() on the wire now (transports that send in bursts, like
  // the reference's tx buffer with its drain timer, dpdk_worker_thread.cc:121-133,282-288).
  virtual void Flush() {}
  // Collect results that arrived; for each, copy payload/exponent into the matching
  // slot's SlotPacket (found through `slots`) and append the slot index to `ready`.
  // May block briefly. Returns false when the transport was shut down.
  virtual bool Poll(std::vector<SlotPacket>& slots, std::vector<int>* ready) = 0;
  // Called on every turn of the loop; gives the transport a chance to retransmit what has
  // waited too long. Returns the number of timeouts that fired.
  virtual uint64_t OnIdle(std::vector<SlotPacket>& slots) { (void)slots; return 0; }
  // A slot received its answer (stop its timer).
  virtual void OnAnswered(int slot) { (void)slot; }
  // A new job slice begins / ended.
  virtual void BeginSlice(const JobSlice& js, uint64_t total_packets, int batch) { (void)js; (void)total_packets; (void)batch; }
  virtual void EndSlice() {}
};

struct SlotWindowResult {
  uint64_t sent = 0, received = 0, wrong = 0, timeouts = 0;
  bool ok = true;
};

// Runs one job slice to completion. `keep_running` is polled so Stop() can interrupt.
template <typename KeepRunning>
SlotWindowResult RunSlotWindow(const JobSlice& js, PrePostProcessor& ppp, SlotTransport& tr,
                               int window, int packet_numel, std::vector<int32_t>& payload_pool,
                               KeepRunning keep_running) {
  SlotWindowResult res;
  JobSlice slice = js;
  uint64_t main_packets = ppp.SetupJobSlice(&slice);
  uint64_t batch = main_packets < static_cast<uint64_t>(window) ? main_packets : window;
  uint64_t total = main_packets + (ppp.NeedsExtraBatch() ? batch : 0);
  payload_pool.resize(static_cast<size_t>(window) * packet_numel);
  std::vector<SlotPacket> slots(batch);
  tr.BeginSlice(js, total, static_cast<int>(batch));

  auto fill = [&](int s, uint64_t id) {
    SlotPacket& p = slots[s];
    p.pkt_id = static_cast<uint32_t>(id);
    p.slot = s;
    p.payload = payload_pool.data() + static_cast<size_t>(s) * packet_numel;
    p.numel = static_cast<uint16_t>(packet_numel);
    p.exponent = 0;
    ppp.PreprocessSingle(id, p.payload, &p.exponent);
  };

  for (uint64_t i = 0; i < batch; i++) {
    fill(static_cast<int>(i), i);
    tr.Send(slots[i], false);
    res.sent++;
  }
  tr.Flush();
  uint64_t answered = 0;
  std::vector<int> ready;
  while (answered < total) {
    if (!keep_running()) { res.ok = false; break; }
    ready.clear();
    if (!tr.Poll(slots, &ready)) { res.ok = false; break; }
    // Timers are looked at on every turn, not only when nothing arrived: while results for
    // other slots keep coming, a slot whose packet or result was lost must not wait for the
    // traffic to go quiet (the reference checks its timers in every loop iteration,
    // rdma_worker_thread.cc:283-292).
    {
      uint64_t t = tr.OnIdle(slots);
      if (t) tr.Flush();
      res.timeouts += t;
      res.sent += t;
    }
    if (ready.empty()) continue;
    for (int s : ready) {
      if (s < 0) { res.wrong++; continue; }  // duplicate or stale packet, already discarded
      SlotPacket& p = slots[s];
      tr.OnAnswered(s);
      ppp.PostprocessSingle(p.pkt_id, p.payload, &p.exponent);
      res.received++;
      answered++;
      uint64_t next = static_cast<uint64_t>(p.pkt_id) + batch;
      if (next < total) {
        fill(s, next);
        tr.Send(p, false);
        res.sent++;
      }
    }
    tr.Flush();
  }
  tr.EndSlice();
  ppp.CleanupJobSlice();
  return res;
}

}  // namespace switchml
#endif  // SWITCHML_SLOT_WINDOW_H_
