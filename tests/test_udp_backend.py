"""Several worker processes aggregating through the software switch over UDP: real
multi-rank sums, bit-exact against the oracle, retransmission under injected packet loss
(the reference tests this with the switch's drop simulator, controller/cli.py:291-366),
and the controller console."""
import io
import multiprocessing as mp

import numpy as np
import pytest

import switchml_b200 as sml
from _workers import udp_worker, rank_data
from switchml_b200.ops.oracle import quant_allreduce_oracle


def _run(n, ports, numel, dtype="float32", threads=1, packet_numel=64, drop=0.0, jobs=2):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=udp_worker,
                         args=(r, n, ports[0], ports[1], numel, dtype, threads, packet_numel, drop, q, jobs))
             for r in range(n)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(n):
            rank, status, outs, stats, sw = q.get(timeout=120)
            assert status == "ok", outs
            results[rank] = (outs, stats, sw)
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    return results


def test_two_workers_bit_exact_vs_oracle(ports):
    numel = (1 << 16) + 37
    res = _run(2, ports, numel, threads=1, packet_numel=64)
    for j in range(2):
        inputs = [rank_data(r, numel, seed=j) for r in range(2)]
        want = quant_allreduce_oracle(inputs, block_numel=64)
        for r in range(2):
            assert np.array_equal(res[r][0][j], want), "rank %d job %d" % (r, j)
        exact = inputs[0].astype(np.float64) + inputs[1].astype(np.float64)
        assert np.max(np.abs(want - exact)) < 1e-6


def test_three_workers_four_threads_float64_check(ports):
    numel = 50000
    res = _run(3, ports, numel, threads=4, packet_numel=256, jobs=1)
    inputs = [rank_data(r, numel, seed=0) for r in range(3)]
    exact = sum(x.astype(np.float64) for x in inputs)
    for r in range(3):
        assert np.max(np.abs(res[r][0][0] - exact)) < 1e-5
    assert np.array_equal(res[0][0][0], res[1][0][0]) and np.array_equal(res[1][0][0], res[2][0][0])


def test_int32_exact(ports):
    numel = 12345
    res = _run(2, ports, numel, dtype="int32", threads=2, jobs=1)
    want = rank_data(0, numel, "int32") + rank_data(1, numel, "int32")
    assert np.array_equal(res[0][0][0], want) and np.array_equal(res[1][0][0], want)


def test_packet_loss_is_recovered_by_retransmission(ports):
    numel = 1 << 14
    res = _run(2, ports, numel, threads=2, packet_numel=64, drop=0.03, jobs=2)
    for j in range(2):
        inputs = [rank_data(r, numel, seed=j) for r in range(2)]
        exact = inputs[0].astype(np.float64) + inputs[1].astype(np.float64)
        for r in range(2):
            assert np.max(np.abs(res[r][0][j] - exact)) < 1e-5
    timeouts = sum(sum(res[r][1]["timeouts"]) for r in range(2))
    assert timeouts > 0, "with 3% loss each way some slot must have timed out"
    sw = res[0][2]
    assert "retransmit" in sw and "ingress_dropped" in sw
    dropped = sum(int(line.split()[1]) for line in sw.splitlines() if "dropped" in line)
    assert dropped > 0


def test_console_against_standalone_controller(ports):
    from switchml_b200._native import lib
    from switchml_b200.utils.cli import Cli
    srv = lib().sml_controller_start(b"127.0.0.1", ports[0], ports[1])
    assert srv
    try:
        out = io.StringIO()
        cli = Cli("127.0.0.1", ports[0], stdout=out)
        for c in ("ping", "set_drop_probabilities 0.5 0.25 3", "show_drop_probabilities", "show_statistics",
                  "show_bitmap 3", "show_workers", "reset_workers", "bogus", "history"):
            cli.onecmd(cli.precmd(c))
        text = out.getvalue()
        assert "ingress 0.5" in text and "egress 0.25" in text
        assert "broadcast 0" in text and "slot 3 set0 0 set1 0" in text
        assert "Unknown syntax: bogus" in text and "set_drop_probabilities" in text
    finally:
        lib().sml_controller_stop(srv)
