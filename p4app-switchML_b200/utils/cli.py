"""Operator console for the controller / software switch.

The reference ships a ``cmd``-based shell inside its Python controller
(controller/cli.py:136-660) to inspect and poke the Tofino: show_ports, show_bitmap,
show_statistics, set_drop_probabilities, reset_workers ... This is the same kind of
shell for the controller that rank 0 hosts in-process (or ``bin/switchml_switchd``):

    python -m switchml_b200.utils.cli --ip 127.0.0.1 --port 50099
    (switchml) show_workers
    (switchml) set_drop_probabilities 0.01 0.01
    (switchml) show_statistics

Every command of the reference shell has a counterpart. The "ports" of the software switch
are its two sockets and one virtual port per worker; its forwarding table is the set of
return addresses it learned from the workers' packets; a worker thread's endpoint takes the
place of a queue pair. GPU workers (backend = cuda) meet through the same controller but
move their data over NVLink, so the data-plane tables stay empty for them.
"""
import argparse
import cmd
import ctypes


def controller_command(ip, port, line):
    """One request/reply with a controller; raises on error."""
    from .._native import lib, last_error, NativeError
    buf = ctypes.create_string_buffer(1 << 16)
    n = lib().sml_controller_command(ip.encode(), int(port), line.encode(), buf, len(buf))
    if n < 0:
        raise NativeError(last_error())
    return buf.value.decode(errors="replace")


class Cli(cmd.Cmd):
    intro = "SwitchML controller console. Type help or ? to list commands."
    prompt = "(switchml) "

    def __init__(self, ip, port, stdout=None):
        super().__init__(stdout=stdout)
        self.ip, self.port = ip, port
        self._history = []

    def _send(self, line):
        try:
            out = controller_command(self.ip, self.port, line)
            if out:
                self.stdout.write(out if out.endswith("\n") else out + "\n")
        except Exception as e:  # keep the shell alive
            self.stdout.write("error: %s\n" % e)

    def precmd(self, line):
        if line.strip():
            self._history.append(line)
        return line

    def do_show_workers(self, arg):
        "Workers of the current session with their packet and byte counters."
        self._send("SHOW workers")

    do_show_udp_workers = do_show_workers

    def do_show_rdma_workers(self, arg):
        "Workers of the current session (this switch has one kind of worker; same table as show_udp_workers)."
        self._send("SHOW workers")

    def do_show_ports(self, arg):
        "Sockets of the switch and one virtual port per worker, with state and packet/byte counters."
        self._send("SHOW ports")

    def do_show_forwarding_table(self, arg):
        "Where results for each (worker, thread) are sent: addresses learned from the workers' packets."
        self._send("SHOW forwarding")

    def do_show_switch_address(self, arg):
        "Address of the controller and UDP port of the data plane."
        self._send("SHOW address")

    def do_set_switch_address(self, arg):
        "set_switch_address <ip> <udp port>: move the data plane; sessions started afterwards use it."
        from .common import validate_ip, validate_port
        parts = arg.split()
        if len(parts) != 2 or not validate_ip(parts[0]) or not validate_port(parts[1]):
            self.stdout.write("usage: set_switch_address <ip> <udp port>\n")
            return
        self._send("SET address %s %s" % (parts[0], parts[1]))

    def do_show_dropped_packets(self, arg):
        "Packets lost to the drop simulator, per worker, on ingress and egress."
        self._send("SHOW dropped")

    def do_show_queue_pairs_counters(self, arg):
        "Per worker thread: packets received, packets outside the expected order, results, retransmitted results."
        self._send("SHOW qp")

    def do_show_statistics(self, arg):
        "show_statistics [slot]: packet counters of the switch, or of both sets of one slot."
        if arg.strip():
            self._send("SHOW slot %s" % arg.split()[0])
        else:
            self._send("SHOW statistics")

    def do_show_bitmap(self, arg):
        "show_bitmap <slot>: the worker bitmaps of both sets of a slot."
        self._send("SHOW bitmap %s" % (arg.strip() or "0"))

    def do_show_drop_probabilities(self, arg):
        "Current ingress and egress drop probabilities."
        self._send("SHOW drop")

    def do_set_drop_probabilities(self, arg):
        "set_drop_probabilities <ingress> <egress> [seed]: lose packets on purpose (0..1)."
        from .common import validate_probability
        parts = arg.split()
        if len(parts) < 2 or not all(validate_probability(p) for p in parts[:2]):
            self.stdout.write("usage: set_drop_probabilities <ingress> <egress> [seed], probabilities in [0, 1]\n")
            return
        self._send("SET drop " + " ".join(parts[:3]))

    def do_reset_workers(self, arg):
        "Forget every worker and clear all switch state."
        self._send("RESET")

    def do_ping(self, arg):
        "Check that the controller answers."
        self._send("PING")

    def do_ping_switch(self, arg):
        "ping_switch [count]: echo requests to the UDP data plane, with round-trip times (the switch's ICMP echo)."
        import socket
        import time
        from .common import WireType, pack_header, unpack_header
        try:
            fields = controller_command(self.ip, self.port, "SHOW address").split()
            where = (fields[fields.index("ip") + 1], int(fields[fields.index("udp_port") + 1]))
            count = int(arg.strip() or 3)
        except Exception as e:
            self.stdout.write("error: %s\n" % e)
            return
        if where[0] == "0.0.0.0":
            where = (self.ip, where[1])
        if where[1] == 0:
            self.stdout.write("this controller has no data plane\n")
            return
        answered = 0
        with socket.socket(socket.AF_INET, socket.SOCK_DGRAM) as so:
            so.settimeout(1.0)
            for seq in range(count):
                payload = b"ping%04d" % seq
                t0 = time.perf_counter()
                try:
                    so.sendto(pack_header(WireType.ECHO_REQUEST, worker=0, pkt_id=seq, numel=2) + payload, where)
                    data, _ = so.recvfrom(2048)
                except (socket.timeout, OSError):
                    self.stdout.write("seq %d: no answer from %s:%d\n" % (seq, where[0], where[1]))
                    continue
                head = unpack_header(data)
                if head and head["type"] == WireType.ECHO_REPLY and data.endswith(payload):
                    answered += 1
                    self.stdout.write("seq %d: reply from %s:%d in %.3f ms\n"
                                      % (seq, where[0], where[1], (time.perf_counter() - t0) * 1e3))
        self.stdout.write("%d of %d echo requests answered\n" % (answered, count))

    def do_history(self, arg):
        "Commands entered so far."
        for i, h in enumerate(self._history):
            self.stdout.write("%3d  %s\n" % (i, h))

    def do_exit(self, arg):
        "Leave the console."
        return True

    do_EOF = do_exit


def main(argv=None):
    ap = argparse.ArgumentParser(description="SwitchML controller console")
    ap.add_argument("--ip", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=50099)
    ap.add_argument("-c", "--command", action="append", help="run one command and exit (repeatable)")
    a = ap.parse_args(argv)
    cli = Cli(a.ip, a.port)
    if a.command:
        for c in a.command:
            cli.onecmd(c)
        return
    cli.cmdloop()


if __name__ == "__main__":
    main()
