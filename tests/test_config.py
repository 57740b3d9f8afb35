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


def test_make_config_routes_keys():
    text = sml.make_config("dummy", rank=0, num_workers=2, packet_numel=64, bandwidth=0)
    assert "[general]" in text and "packet_numel = 64" in text.split("[backend.dummy]")[0]
    assert "bandwidth = 0" in text.split("[backend.dummy]")[1]
