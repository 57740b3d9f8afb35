"""Configuration grammar, defaults, validation and rounding rules
(reference client_lib/src/config.cc:46-211)."""
import pytest

import switchml_b200 as sml
from switchml_b200.utils.config import check_config
from switchml_b200 import NativeError


def test_defaults_match_reference():
    dump = check_config("[general]\n")
    for line in ("rank = 0", "num_workers = 1", "num_worker_threads = 4", "max_outstanding_packets = 256",
                 "packet_numel = 1024", "backend = dummy", "scheduler = fifo",
                 "prepostprocessor = cpu_exponent_quantizer", "instant_job_completion = false",
                 "controller_ip = 127.0.0.1", "controller_port = 50099", "timeout = 10",
                 "timeout_threshold = 100", "timeout_threshold_increment = 100", "bandwidth = 1000",
                 "process_packets = true"):
        assert line in dump, line


def test_comments_and_whitespace():
    dump = check_config("# a comment\n[general]\n  rank=1 # trailing\nnum_workers =   2\n\n[backend.dummy]\nbandwidth = 0\n")
    assert "rank = 1" in dump and "num_workers = 2" in dump and "bandwidth = 0" in dump


def test_window_is_rounded_to_thread_multiple():
    dump = check_config("[general]\nnum_worker_threads = 3\nmax_outstanding_packets = 10\n")
    assert "max_outstanding_packets = 9" in dump
    dump = check_config("[general]\nnum_worker_threads = 3\nmax_outstanding_packets = 11\n")
    assert "max_outstanding_packets = 12" in dump


@pytest.mark.parametrize("text", [
    "[general]\nmax_outstanding_packets = 2\nnum_worker_threads = 4\n",   # fewer slots than threads
    "[general]\nrank = 2\nnum_workers = 2\n",                               # rank out of range
    "[general]\nnum_workers = 33\n",                                        # more than the bitmap holds
    "[general]\nbackend = rdma\n",                                          # NIC backends do not exist here
    "[general]\nbackend = udp\npacket_numel = 128\n",                       # udp wants 64 or 256
    "[general]\nbackend = cuda\npacket_numel = 100\n",                      # cuda wants a power of two
    "[general]\nbackend = cuda\npacket_numel = 256\n[backend.cuda]\nexponent_lookahead = 5\n",   # ring of 8: at most 4
    "[general]\nbackend = cuda\npacket_numel = 256\n[backend.cuda]\nsignal_fence = none\n",     # sc | release
    "[general]\nbogus_key = 1\n",
    "[general]\nrank = minus one\n",
    "[general\nrank = 1\n",
])
def test_rejected(text):
    with pytest.raises(NativeError):
        check_config(text)


def test_nic_sections_are_tolerated():
    dump = check_config("[general]\nbackend = dummy\n[backend.rdma]\nmsg_numel = 1024\ndevice_name = mlx5_0\n"
                        "[backend.dpdk]\ncores = 0-3\n")
    assert "(ignored) backend.rdma.msg_numel = 1024" in dump


def test_cuda_section_and_slot_rounding():
    dump = check_config(sml.make_config("cuda", rank=1, num_workers=4, packet_numel=256, mode="float_sum",
                                        slot_bytes=100000, transport="p2p"))
    assert "mode = float_sum" in dump and "transport = p2p" in dump
    # multiple of num_workers * max(packet_numel,128) * 4 = 4096
    assert "slot_bytes = 98304" in dump


def test_cuda_signalling_keys():
    """Defaults: flags are announced by their release store alone, exponents are agreed right
    before their tile; both can be set back, and the trace is off unless asked for."""
    dump = check_config(sml.make_config("cuda", packet_numel=256))
    assert "signal_fence = release" in dump and "exponent_lookahead = 0" in dump and "trace = false" in dump
    dump = check_config(sml.make_config("cuda", packet_numel=256, signal_fence="sc", exponent_lookahead=4, trace=True))
    assert "signal_fence = sc" in dump and "exponent_lookahead = 4" in dump and "trace = true" in dump


def test_make_config_routes_keys():
    text = sml.make_config("dummy", rank=0, num_workers=2, packet_numel=64, bandwidth=0)
    assert "[general]" in text and "packet_numel = 64" in text.split("[backend.dummy]")[0]
    assert "bandwidth = 0" in text.split("[backend.dummy]")[1]


def test_wire_constants_and_validators():
    from switchml_b200.utils.common import (HEADER, PacketSize, WireType, pack_header, unpack_header, validate_ip,
                                            validate_port, validate_probability)
    assert HEADER.size == 20
    assert [s.numel for s in PacketSize] == [32, 64, 128, 256] and PacketSize.from_numel(256) is PacketSize.MTU_1024
    with pytest.raises(ValueError):
        PacketSize.from_numel(100)
    raw = pack_header(WireType.DATA, worker=3, thread=2, pkt_id=77, pool_index=0x8005, numel=64, exponent=-4,
                      job_tag=300, session=0x12345)
    h = unpack_header(raw + b"\0" * 256)
    assert h == {"type": 0, "job_tag": 300 & 0xFF, "worker": 3, "pkt_id": 77, "slot": 5, "set": 1, "numel": 64,
                 "exponent": -4, "thread": 2, "session_lo": 0x2345}
    assert unpack_header(b"short") is None and unpack_header(b"\0" * 20) is None
    assert validate_ip("10.0.0.1") and not validate_ip("10.0.0.256") and not validate_ip("ten")
    assert validate_port("48864") and not validate_port("70000") and not validate_port("x")
    assert validate_probability("0.5") and not validate_probability("-0.1") and not validate_probability("2")


def test_api_reference_is_up_to_date():
    """docs/api.md is generated from the public headers; regenerate it after editing them."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = os.path.join(root, "p4app-switchML_b200", "docs", "make_api_reference.py")
    r = subprocess.run([sys.executable, script, "--check"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr


def test_udp_message_size_is_validated_and_rounded():
    """[backend.udp] msg_numel follows the rules of the reference's backend.rdma.msg_numel
    (client_lib/src/config.cc:185-211): not below a packet, rounded down to whole packets, and
    max_outstanding_packets moved to the nearest whole number of messages per worker thread."""
    from switchml_b200.utils.config import make_config, check_config
    base = dict(packet_numel=64, num_worker_threads=2, max_outstanding_packets=64)
    assert "msg_numel = 64" in check_config(make_config("udp", **base))          # default: one packet
    dump = check_config(make_config("udp", msg_numel=300, **base))
    assert "msg_numel = 256" in dump and "max_outstanding_packets = 64" in dump  # 4 packets, 8 messages a thread
    dump = check_config(make_config("udp", msg_numel=192, **base))               # 3 packets: 64 is not a multiple of 6
    assert "max_outstanding_packets = 66" in dump
    with pytest.raises(Exception):
        check_config(make_config("udp", msg_numel=32, **base))
    with pytest.raises(Exception):
        check_config(make_config("udp", msg_numel=64 * 65, **base))
