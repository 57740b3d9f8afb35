"""``torch.distributed`` backend "sml" on CPU ranks (udp transport underneath)."""
import multiprocessing as mp

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
