"""``torch.distributed`` backend "sml" on CPU ranks (udp transport underneath)."""
import multiprocessing as mp
import os

import pytest

from conftest import free_port
from _workers import pg_worker


def test_sml_backend_allreduce_fallback_and_ddp():
    n = 2
    port = free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=pg_worker, args=(r, n, port, q)) for r in range(n)]
    for p in procs:
        p.start()
    try:
        for _ in range(n):
            rank, status, info = q.get(timeout=180)
            assert status == "ok", info
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()


def test_native_cpp_backend(tmp_path):
    import importlib.util
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("_switchml_build", os.path.join(root, "p4app-switchML_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build(programs=False)
    assert mod.build_torch_extension() is not None
    from _workers import native_pg_worker
    n = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ports = [free_port(), free_port(), free_port()]
    procs = [ctx.Process(target=native_pg_worker, args=(r, n, *ports, str(tmp_path), q)) for r in range(n)]
    for p in procs:
        p.start()
    try:
        for _ in range(n):
            rank, status, info = q.get(timeout=180)
            assert status == "ok", info
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()


def test_pytorch_benchmark_script_one_worker(tmp_path):
    """benchmarks/allreduce_pytorch_benchmark.py (the reference's tool of the same name) with
    the "sml" backend, verified."""
    import subprocess
    import sys
    from conftest import free_port
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = os.path.join(root, "p4app-switchML_b200", "benchmarks", "allreduce_pytorch_benchmark.py")
    env = dict(os.environ, MASTER_PORT=str(free_port()), MASTER_ADDR="127.0.0.1")
    for extra in (["-tt", "float", "--random", "--seed", "3"], ["-tt", "int32", "-sv", "0"]):
        r = subprocess.run([sys.executable, script, "-n", "1", "-r", "0", "-bk", "sml", "-d", "cpu", "-tn", "50000",
                            "-nj", "3", "-nw", "1", "-v"] + extra, capture_output=True, text=True, timeout=180,
                           env=env, cwd=tmp_path)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
        assert "Results verified successfully." in r.stdout and "median: Duration: #" in r.stdout


def test_pytorch_benchmark_script_two_workers_native_backend(tmp_path):
    """The same tool on the C++ c10d backend, two processes over the UDP backend."""
    import subprocess
    import sys
    from conftest import free_port
    import switchml_b200 as sml
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if not os.path.exists(os.path.join(root, "p4app-switchML_b200", "lib", "torch_switchml.so")):
        pytest.skip("native torch extension not built")
    script = os.path.join(root, "p4app-switchML_b200", "benchmarks", "allreduce_pytorch_benchmark.py")
    port, ctl, udp = free_port(), free_port(), free_port()
    procs = []
    for rank in range(2):
        cfg = tmp_path / ("switchml-rank%d.cfg" % rank)
        cfg.write_text(sml.make_config("udp", rank=rank, num_workers=2, packet_numel=64, num_worker_threads=2,
                                       max_outstanding_packets=64, controller_port=ctl, switch_port=udp,
                                       worker_port=0))
        env = dict(os.environ, MASTER_PORT=str(port), MASTER_ADDR="127.0.0.1", SWITCHML_CONFIG=str(cfg))
        procs.append(subprocess.Popen([sys.executable, script, "-n", "2", "-r", str(rank), "-bk", "sml_native", "-d",
                                       "cpu", "-tn", "30000", "-nj", "3", "-nw", "1", "-v", "-tt", "int32"],
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env, cwd=tmp_path))
    for p in procs:
        out, err = p.communicate(timeout=240)
        assert p.returncode == 0, out[-2000:] + err[-2000:]
        assert "Results verified successfully." in out
