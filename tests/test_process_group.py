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
