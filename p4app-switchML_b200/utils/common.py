"""Constants of the wire format and small validators shared by the console and the tests.

The reference keeps the Python mirror of its P4 enums in controller/common.py:19-82
(WorkerType, PacketSize, PacketType, address validation). Here the single source of truth
is csrc/backends/softswitch/wire.h; this module restates the values for Python code that
builds or reads datagrams of the software switch (console, tests, packet tools).
"""
import ipaddress
import struct
from enum import IntEnum

WIRE_MAGIC = 0x534D4C31      # "SML1"
SET_BIT = 0x8000             # pool_index MSB: which of the two sets of a slot
MAX_PACKET_NUMEL = 256       # 1024-byte payload
MAX_WORKERS = 32             # width of the worker bitmap
MAX_THREADS = 64             # worker threads (return ports) per worker
FLOOD_WORKER = 0xFF          # WIRE_FORWARD destination: every other worker
SWITCH_UDP_PORT = 0xBEE0     # 48864, the SwitchML UDP port

# magic u32, type u8, job tag u8, worker u16, packet id u32, pool index u16, numel u16,
# exponent i8, thread u8, low half of the session id u16 - network byte order, 20 bytes
HEADER = struct.Struct("!IBBHIHHbBH")


class WireType(IntEnum):
    DATA = 0            # worker -> switch
    RESULT = 1          # switch -> every worker
    RESULT_RETX = 2     # switch -> one worker, answer to a retransmission
    ECHO_REQUEST = 3    # anyone -> switch
    ECHO_REPLY = 4      # switch -> the sender
    FORWARD = 5         # worker -> worker(s) through the switch
    DATA_MORE = 6       # worker -> switch: a packet of a message whose last packet (DATA) carries the exponent


class WorkerType(IntEnum):
    """Kinds of workers a controller can serve (the reference: forward-only, UDP, RoCEv2)."""
    FORWARD_ONLY = 0    # only echo / forwarding traffic
    SWITCHML_UDP = 1    # aggregates through the software switch
    NVLINK = 2          # backend = cuda: meets through the controller, aggregates over NVSwitch


class PacketSize(IntEnum):
    """Payload bytes per packet, as the reference's protobuf enum names them."""
    MTU_128 = 0
    MTU_256 = 1
    MTU_512 = 2
    MTU_1024 = 3

    @property
    def numel(self):
        return 32 << int(self)

    @classmethod
    def from_numel(cls, packet_numel):
        for size in cls:
            if size.numel == packet_numel:
                return size
        raise ValueError("packet_numel must be 32, 64, 128 or 256, not %r" % (packet_numel,))


def validate_ip(value):
    """True for a dotted IPv4 address."""
    try:
        ipaddress.IPv4Address(value)
        return True
    except (ipaddress.AddressValueError, ValueError):
        return False


def validate_port(value):
    try:
        return 0 <= int(value) <= 65535
    except (TypeError, ValueError):
        return False


def validate_probability(value):
    try:
        return 0.0 <= float(value) <= 1.0
    except (TypeError, ValueError):
        return False


def pack_header(wire_type, worker, thread=0, pkt_id=0, pool_index=0, numel=0, exponent=0, job_tag=0, session=0):
    return HEADER.pack(WIRE_MAGIC, int(wire_type), job_tag & 0xFF, worker, pkt_id & 0xFFFFFFFF, pool_index, numel,
                       exponent, thread, session & 0xFFFF)


def unpack_header(data):
    """dict of the header fields of a datagram, or None if it is not one of ours."""
    if len(data) < HEADER.size:
        return None
    magic, wire_type, job_tag, worker, pkt_id, pool_index, numel, exponent, thread, session = HEADER.unpack_from(data)
    if magic != WIRE_MAGIC:
        return None
    return {"type": wire_type, "job_tag": job_tag, "worker": worker, "pkt_id": pkt_id, "slot": pool_index & ~SET_BIT,
            "set": 1 if pool_index & SET_BIT else 0, "numel": numel, "exponent": exponent, "thread": thread,
            "session_lo": session}
