// Datagram format between a worker thread and the software aggregation switch.
//
// It carries the same information as the SwitchML header + exponent header + payload of
// the reference (p4/headers.p4:72-79,118-157; client side dpdk_backend.h:56-84): job
// tag, packet id echoed back by the switch ("tsi"), pool index with the set bit in the
// MSB, element count, one exponent byte, then int32 payload in network byte order. The
// Ethernet/IP/UDP layers are left to the kernel socket.
#ifndef SWITCHML_SOFTSWITCH_WIRE_H_
#define SWITCHML_SOFTSWITCH_WIRE_H_

#include <stdint.h>

namespace switchml {

static const uint32_t kWireMagic = 0x534d4c31;  // "SML1"
static const uint16_t kSetBit = 0x8000;         // pool_index MSB selects the slot set
static const int kMaxPacketNumel = 256;         // 1024-byte payload, the largest SwitchML packet
static const int kMaxWorkers = 32;              // width of the per-slot worker bitmap
static const int kMaxThreads = 64;              // worker threads (return ports) per worker
static const uint8_t kFloodWorker = 0xff;       // WIRE_FORWARD destination: every other worker

enum WireType : uint8_t {
  WIRE_DATA = 0,        // worker -> switch
  WIRE_RESULT = 1,      // switch -> every worker (multicast of a completed slot)
  WIRE_RESULT_RETX = 2, // switch -> one worker (answer to a retransmission)
  // Traffic that is not aggregation (the reference switch answers ARP and ICMP echo for its
  // own address, p4/arp_icmp_responder.p4:40-84, and forwards everything else by destination
  // or floods it, p4/forwarder.p4:31-64):
  WIRE_ECHO_REQUEST = 3,  // anyone -> switch: "are you there"; payload comes back unchanged
  WIRE_ECHO_REPLY = 4,    // switch -> the sender of the request
  WIRE_FORWARD = 5,       // worker -> worker through the switch; pool_index = dest worker << 8 |
                          // dest thread, dest worker kFloodWorker = all other workers
  // A message of several packets ([backend.udp] msg_numel) occupies consecutive pool indices and
  // has ONE exponent, which only its last packet carries (that one is a WIRE_DATA packet); the
  // packets in front of it say so and are aggregated without touching the exponent register,
  // like packets whose last_packet flag is off in the reference (p4/rdma_receiver.p4:203-266,
  // p4/switchml.p4:141-146).
  WIRE_DATA_MORE = 6      // worker -> switch: payload only, more packets of this message follow
};

#pragma pack(push, 1)
struct WireHeader {
  uint32_t magic;
  uint8_t type;
  uint8_t job_tag;      // low 8 bits of the job id; stale results are discarded
  uint16_t worker_id;   // sender rank (DATA) / destination rank (RESULT)
  uint32_t pkt_id;      // echoed unchanged by the switch
  uint16_t pool_index;  // slot | set bit
  uint16_t numel;       // payload elements
  int8_t exponent;
  uint8_t thread_id;    // worker thread, selects the return port
  uint16_t session_lo;  // low 16 bits of the session id
};
#pragma pack(pop)

static const int kWireMaxBytes = sizeof(WireHeader) + kMaxPacketNumel * 4;

}  // namespace switchml
#endif  // SWITCHML_SOFTSWITCH_WIRE_H_
