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


def _run(n, ports, numel, dtype="float32", threads=1, packet_numel=64, drop=0.0, jobs=2, msg_numel=0):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=udp_worker,
                         args=(r, n, ports[0], ports[1], numel, dtype, threads, packet_numel, drop, q, jobs, 10.0,
                               msg_numel))
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


def _oracle_per_thread_slice(inputs, threads, block):
    """Worker threads take contiguous slices (numel / threads, the first numel % threads one
    longer, reference schedulers/fifo_scheduler.cc:92-109) and cut THEIR slice into blocks."""
    numel = inputs[0].size
    base, rem = divmod(numel, threads)
    out, lo = [], 0
    for t in range(threads):
        hi = lo + base + (1 if t < rem else 0)
        out.append(quant_allreduce_oracle([x[lo:hi] for x in inputs], block_numel=block))
        lo = hi
    return np.concatenate(out)


def test_messages_of_several_packets_share_one_exponent(ports):
    """[backend.udp] msg_numel = 4 packets: the window, the timers and the exponent work per
    message (the reference's backend.rdma.msg_numel), so the result equals the oracle with a
    quantisation block of msg_numel elements, and the switch counts one message per four packets."""
    numel = 40000 + 13
    res = _run(2, ports, numel, threads=2, packet_numel=64, msg_numel=256, jobs=2)
    for j in range(2):
        inputs = [rank_data(r, numel, seed=j) for r in range(2)]
        want = _oracle_per_thread_slice(inputs, 2, 256)
        for r in range(2):
            assert np.array_equal(res[r][0][j], want), "rank %d job %d" % (r, j)
    rows = [l.split() for l in res[0][1]["switch_tables"]["qp"].splitlines()[1:]]
    assert rows and all(int(r[2]) == 4 * int(r[3]) for r in rows if int(r[3]) > 100), rows  # rx_pkts = 4 x rx_msgs
    sent = sum(res[0][1]["total_pkts_sent"])
    assert sent % 4 == 0 and sent >= 4 * 2 * (numel // 256), "statistics count packets, four per message"


def test_message_loss_is_recovered_packet_by_packet(ports):
    numel = 1 << 15
    res = _run(3, ports, numel, threads=2, packet_numel=64, msg_numel=512, drop=0.02, jobs=2)
    for j in range(2):
        inputs = [rank_data(r, numel, seed=j) for r in range(3)]
        want = _oracle_per_thread_slice(inputs, 2, 512)
        for r in range(3):
            assert np.array_equal(res[r][0][j], want), "rank %d job %d" % (r, j)
    assert sum(sum(res[r][1]["timeouts"]) for r in range(3)) > 0


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
    # the same loss, per worker and per worker thread (show_dropped_packets, show_queue_pairs_counters)
    tables = res[0][1]["switch_tables"]
    rows = [l.split() for l in tables["dropped"].splitlines()[1:]]
    assert [r[0] for r in rows] == ["0", "1", "total"]
    assert sum(int(r[1]) + int(r[2]) for r in rows[:2]) == int(rows[2][1]) + int(rows[2][2]) == dropped
    qp = [l.split() for l in tables["qp"].splitlines()[1:]]
    assert len(qp) == 4, tables["qp"]                      # 2 workers x 2 threads
    assert sum(int(r[3]) for r in qp) > 0                  # retransmissions arrive outside the expected order
    assert sum(int(r[5]) for r in qp) > 0                  # and some are answered from the retained copy


def test_stop_fails_a_job_that_total_loss_keeps_from_finishing(ports):
    from _workers import stop_during_loss_worker
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=stop_during_loss_worker, args=(r, 2, ports[0], ports[1], q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        for _ in range(2):
            rank, status, info = q.get(timeout=120)
            assert status == "ok", info
            assert info["early"] == int(sml.JobStatus.RUNNING)
            assert info["final"] == int(sml.JobStatus.FAILED) and info["error"], info
            assert info["stop_seconds"] < 10.0
            assert info["timeouts"] > 0, "the retransmission timers must have fired meanwhile"
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()


def test_switch_tables_of_a_live_session(ports):
    res = _run(2, ports, 20000, threads=2, packet_numel=64, jobs=1)
    t = res[0][1]["switch_tables"]
    fwd = [l.split() for l in t["forwarding"].splitlines()[1:]]
    assert sorted((r[0], r[1]) for r in fwd) == [("0", "0"), ("0", "1"), ("1", "0"), ("1", "1")]
    assert all(r[2].startswith("127.0.0.1:") for r in fwd)
    assert len({r[2] for r in fwd}) == 4                   # one return port per worker thread
    lines = {l.split()[0]: l.split() for l in t["ports"].splitlines()[1:]}
    assert lines["control"][1] == "127.0.0.1:%d/tcp" % ports[0] and lines["control"][2] == "up"
    assert lines["data"][1] == "127.0.0.1:%d/udp" % ports[1] and int(lines["data"][3]) > 0
    assert lines["worker0"][1:4] == ["2", "endpoint(s)", "up"] and lines["worker1"][3] == "up"
    packets = -(-20000 // 64)
    assert int(lines["worker1"][4]) >= packets             # rx packets of worker 1
    assert "udp_port %d" % ports[1] in t["address"]
    qp = [l.split() for l in t["qp"].splitlines()[1:]]
    assert sum(int(r[2]) for r in qp) >= 2 * packets and all(int(r[3]) == 0 or int(r[5]) >= 0 for r in qp)


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
        # every command of the reference's shell exists (controller/cli.py:136-660)
        for name in ("show_ports", "set_switch_address", "show_switch_address", "show_forwarding_table",
                     "set_drop_probabilities", "show_drop_probabilities", "show_dropped_packets",
                     "show_rdma_workers", "show_udp_workers", "show_queue_pairs_counters", "show_bitmap",
                     "show_statistics", "reset_workers", "history", "exit"):
            assert hasattr(cli, "do_" + name), name
        for c in ("show_ports", "show_forwarding_table", "show_dropped_packets", "show_queue_pairs_counters",
                  "show_rdma_workers", "show_switch_address", "show_statistics 3"):
            cli.onecmd(cli.precmd(c))
        text = out.getvalue()
        assert "127.0.0.1:%d/udp  up" % ports[1] in text and "udp_port %d" % ports[1] in text
        assert " total  0  0" in text
        assert " set  bitmap  missing  complete  broadcast  retransmit  consumed  ignored" in text
        assert "ingress 0.5" in text and "egress 0.25" in text
        assert "broadcast 0" in text and "slot 3 set0 0 set1 0" in text
        assert "Unknown syntax: bogus" in text and "set_drop_probabilities" in text

        # The data plane answers echo requests (the switch's ping), also after it has moved.
        from switchml_b200.utils.common import WireType, pack_header, unpack_header

        def echo(port):
            import socket
            pkt = pack_header(WireType.ECHO_REQUEST, worker=5, thread=1, pkt_id=1234, numel=2) + b"switchml"
            with socket.socket(socket.AF_INET, socket.SOCK_DGRAM) as so:
                so.settimeout(2.0)
                so.sendto(pkt, ("127.0.0.1", port))
                try:
                    data, _ = so.recvfrom(2048)
                except (socket.timeout, ConnectionError):
                    return None
            return data

        reply = echo(ports[1])
        assert reply is not None and reply[5:] == struct_tail(reply)
        head = unpack_header(reply)
        assert head["type"] == WireType.ECHO_REPLY and head["worker"] == 5 and head["thread"] == 1
        assert head["pkt_id"] == 1234 and head["numel"] == 2
        from conftest import free_port
        moved = free_port()
        out.truncate(0)
        cli.onecmd("set_switch_address 127.0.0.1 %d" % moved)
        cli.onecmd("show_switch_address")
        assert "udp_port %d" % moved in out.getvalue()
        assert echo(moved) is not None and echo(ports[1]) is None
        cli.onecmd("ping_switch 2")
        assert "2 of 2 echo requests answered" in out.getvalue()
        cli.onecmd("set_switch_address 127.0.0.1")
        cli.onecmd("set_switch_address 300.1.1.1 5000")
        assert out.getvalue().count("usage: set_switch_address") == 2
        cli.onecmd("set_drop_probabilities 1.5 0")
        assert "probabilities in [0, 1]" in out.getvalue()
    finally:
        lib().sml_controller_stop(srv)


def struct_tail(reply):
    """Everything after the type byte of an echo reply must be what was sent."""
    import struct
    return struct.pack("!BHIHHbBH", 0, 5, 1234, 0, 2, 0, 1, 0) + b"switchml"


def test_switch_survives_malformed_and_hostile_datagrams(ports):
    """The data plane parses bytes from the network: random garbage, truncated packets,
    lengths that do not match, slots and workers out of range, foreign sessions and
    forwarding to nowhere must all be counted and dropped, and service must go on."""
    import random
    import socket
    from switchml_b200._native import lib
    from switchml_b200.utils.cli import controller_command
    from switchml_b200.utils.common import HEADER, WIRE_MAGIC, WireType, pack_header, unpack_header
    srv = lib().sml_controller_start(b"127.0.0.1", ports[0], ports[1])
    assert srv
    try:
        session = 0xABCD1234
        for rank in range(2):
            controller_command("127.0.0.1", ports[0], "UDPSESSION %d %d 2 64 127.0.0.1 0 1" % (session, rank))
        rng = random.Random(7)
        sent = 0
        with socket.socket(socket.AF_INET, socket.SOCK_DGRAM) as so:
            def send(b):
                nonlocal sent
                so.sendto(b, ("127.0.0.1", ports[1]))
                sent += 1
            for _ in range(300):                                   # pure noise of every length
                send(bytes(rng.getrandbits(8) for _ in range(rng.randrange(0, 1100))))
            good = pack_header(WireType.DATA, worker=0, pkt_id=1, pool_index=3, numel=64, session=session)
            for cut in range(0, HEADER.size + 8):                  # truncated
                send((good + b"\0" * 256)[:cut])
            send(good + b"\0" * 252)                               # payload shorter than numel says
            send(good + b"\0" * 260)                               # longer
            send(pack_header(WireType.DATA, worker=0, numel=60000, session=session) + b"\0" * 1024)
            send(pack_header(WireType.DATA, worker=31, numel=64, session=session) + b"\0" * 256)   # not registered
            send(pack_header(WireType.DATA, worker=0, pool_index=0x7FFF, numel=64, session=session) + b"\0" * 256)
            send(pack_header(WireType.DATA, worker=0, numel=64, session=session + 1) + b"\0" * 256)  # other session
            send(pack_header(WireType.RESULT, worker=0, numel=64, session=session) + b"\0" * 256)    # not for a switch
            for r in range(2):                                     # valid in every field but the thread id: the
                send(pack_header(WireType.DATA, worker=r, thread=200, pool_index=9, numel=64,  # return-port table
                                 session=session) + b"\0" * 256)                             # has no such row
            send(pack_header(9, worker=0, numel=0, session=session))                                  # unknown type
            send(pack_header(WireType.FORWARD, worker=0, pool_index=(7 << 8), session=session) + b"x")   # no such worker
            send(pack_header(WireType.FORWARD, worker=5, pool_index=(1 << 8), session=session) + b"x")   # sender unknown
            send(HEADER.pack(WIRE_MAGIC ^ 1, 0, 0, 0, 0, 0, 64, 0, 0, session & 0xFFFF) + b"\0" * 256)   # wrong magic
            for _ in range(300):                                   # valid header, every other field random
                numel = rng.randrange(0, 300)
                head = HEADER.pack(WIRE_MAGIC, rng.randrange(0, 8), rng.getrandbits(8), rng.getrandbits(16),
                                   rng.getrandbits(32), rng.getrandbits(16), numel, rng.randrange(-128, 128),
                                   rng.getrandbits(8), rng.getrandbits(16))
                send(head + bytes(4 * min(numel, 256)))
            # and it still answers
            so.settimeout(2.0)
            so.sendto(pack_header(WireType.ECHO_REQUEST, worker=1, pkt_id=99) + b"alive", ("127.0.0.1", ports[1]))
            deadline = 50
            while deadline:
                data, _ = so.recvfrom(2048)
                head = unpack_header(data)
                if head and head["type"] == WireType.ECHO_REPLY and head["pkt_id"] == 99:
                    break
                deadline -= 1                                      # replies to random echo requests come first
            assert deadline, "no echo reply after the flood"
        assert controller_command("127.0.0.1", ports[0], "PING") == ""
        stats = dict(l.split() for l in controller_command("127.0.0.1", ports[0], "SHOW statistics").splitlines())
        assert int(stats["malformed"]) >= 332, stats
        assert "set0 0 set1 0" in controller_command("127.0.0.1", ports[0], "SHOW bitmap 9"), "slot 9 was touched"
        assert int(stats["broadcast"]) == 0 and int(stats["forwarded"]) == 0, stats
        ports_table = controller_command("127.0.0.1", ports[0], "SHOW ports")
        assert int(ports_table.splitlines()[2].split()[3]) >= sent
    finally:
        lib().sml_controller_stop(srv)


def test_controller_with_two_pipes(ports):
    """Two data-plane threads with a socket each: both answer echo requests, both are listed
    as ports, a session request returns both ports, and moving the switch moves both."""
    import socket
    from conftest import free_port
    from switchml_b200._native import lib
    from switchml_b200.utils.cli import controller_command
    from switchml_b200.utils.common import WireType, pack_header, unpack_header
    srv = lib().sml_controller_start_pipes(b"127.0.0.1", ports[0], ports[1], 2)
    assert srv
    try:
        def table():
            rows = [l.split() for l in controller_command("127.0.0.1", ports[0], "SHOW ports").splitlines()[1:]]
            return {r[0]: r for r in rows}

        def echo(port):
            with socket.socket(socket.AF_INET, socket.SOCK_DGRAM) as so:
                so.settimeout(2.0)
                so.sendto(pack_header(WireType.ECHO_REQUEST, worker=0, pkt_id=port) + b"hi", ("127.0.0.1", port))
                try:
                    head = unpack_header(so.recvfrom(2048)[0])
                except (socket.timeout, ConnectionError):
                    return False
                return head["type"] == WireType.ECHO_REPLY and head["pkt_id"] == port & 0xFFFFFFFF

        rows = table()
        assert "data" in rows and "data1" in rows and rows["data"][2] == rows["data1"][2] == "up"
        pipe_ports = [int(rows[k][1].split(":")[1].split("/")[0]) for k in ("data", "data1")]
        assert pipe_ports[0] == ports[1] and pipe_ports[1] != pipe_ports[0]
        assert all(echo(p) for p in pipe_ports)
        rows = table()
        assert int(rows["data"][3]) == 1 and int(rows["data1"][3]) == 1          # one datagram each
        assert "pipes 2" in controller_command("127.0.0.1", ports[0], "SHOW address")
        from switchml_b200._native import lib as _lib  # the session reply carries one port per pipe
        import ctypes
        buf = ctypes.create_string_buffer(256)
        n = _lib().sml_controller_command(b"127.0.0.1", ports[0], b"UDPSESSION 5 0 1 64 127.0.0.1 0 2", buf, len(buf))
        assert n >= 0 and [int(x) for x in buf.value.decode().split()] == pipe_ports
        moved = free_port()
        assert controller_command("127.0.0.1", ports[0], "SET address 127.0.0.1 %d" % moved) == str(moved)
        rows = table()
        new_ports = [int(rows[k][1].split(":")[1].split("/")[0]) for k in ("data", "data1")]
        assert new_ports[0] == moved and all(echo(p) for p in new_ports) and not echo(pipe_ports[0])
    finally:
        lib().sml_controller_stop(srv)


def test_broadcast_between_real_workers(ports):
    from _workers import broadcast_udp_worker
    n = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=broadcast_udp_worker, args=(r, n, ports[0], ports[1], q)) for r in range(n)]
    for p in procs:
        p.start()
    got = {}
    try:
        for _ in range(n):
            rank, status, out = q.get(timeout=180)
            assert status == "ok", out
            got[rank] = out
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    for root in range(n):
        want_int = np.arange(5000, dtype=np.int32) * (root + 1) - 77 * root
        want_float = np.random.default_rng(100 + root).standard_normal(3333).astype(np.float32)
        for r in range(n):
            assert np.array_equal(got[r]["int%d" % root], want_int), (root, r)
            assert np.array_equal(got[r]["float%d" % root], got[0]["float%d" % root]), "ranks must agree bit for bit"
            assert np.max(np.abs(got[r]["float%d" % root] - want_float)) < 1e-6
