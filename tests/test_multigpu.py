"""The cuda backend on several GPUs of one box, one process per GPU: NVLink SHARP
(multimem) and peer-memory transports, quantised and float modes, all element types,
staged / one-shot / zero-copy algorithms. Every rank checks its own results against the
CPU oracle."""
import multiprocessing as mp

import pytest
import torch

from conftest import free_port
from _workers import cuda_worker

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _world():
    n = torch.cuda.device_count()
    return 8 if n >= 8 else (4 if n >= 4 else 2)


def _run(transport, mode, launch="inline"):
    n = _world()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=cuda_worker, args=(r, n, port, transport, mode, q, 64, launch)) for r in range(n)]
    for p in procs:
        p.start()
    reports = {}
    try:
        for _ in range(n):
            rank, status, rep = q.get(timeout=300)
            assert status == "ok", "rank %d:\n%s" % (rank, rep)
            reports[rank] = rep
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    return reports


@pytest.mark.parametrize("mode", ["int32_quant", "float_sum"])
def test_peer_memory_transport(mode):
    reps = _run("p2p", mode)
    assert all(not r["multimem"] for r in reps.values())
    assert all(r["stats"]["jobs_failed"] == 0 for r in reps.values())


@pytest.mark.parametrize("mode", ["int32_quant", "float_sum"])
def test_multimem_transport(mode):
    reps = _run("nvls", mode, launch="worker")
    assert all(r["multimem"] for r in reps.values())
    assert all(r["stats"]["jobs_failed"] == 0 for r in reps.values())


def test_auto_transport_agrees_on_all_ranks():
    reps = _run("auto", "float_sum")
    # Whatever the fabric offers, all ranks must agree and every case must pass.
    assert len({r["multimem"] for r in reps.values()}) == 1
    assert all(r["stats"]["jobs_failed"] == 0 for r in reps.values())


def _spawn(target, n, extra_ports=1):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ports = [free_port() for _ in range(extra_ports)]
    procs = [ctx.Process(target=target, args=(r, n, *ports, q)) for r in range(n)]
    for p in procs:
        p.start()
    out = {}
    try:
        for _ in range(n):
            rank, status, info = q.get(timeout=300)
            assert status == "ok", "rank %d:\n%s" % (rank, info)
            out[rank] = info
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    return out


def test_torch_ddp_with_switchml_comm_hook():
    from _workers import ddp_hook_worker
    _spawn(ddp_hook_worker, min(_world(), 4), extra_ports=2)


def test_absent_peer_is_detected_by_bounded_wait():
    from _workers import absent_peer_worker
    n = 2
    infos = _spawn(absent_peer_worker, n)
    waiting = infos[0]
    assert waiting["status"] == "FAILED" and "did not arrive" in waiting["error"]
    assert waiting["jobs_failed"] == 1 and waiting["device_timeouts"] >= 1
    assert waiting["seconds"] < 10 and waiting["alive"]


def test_native_c10d_backend_on_gpus(tmp_path):
    import os
    from _workers import native_pg_cuda_worker
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if not os.path.exists(os.path.join(root, "p4app-switchML_b200", "lib", "torch_switchml.so")):
        pytest.skip("torch_switchml.so not built")
    n = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ports = [free_port(), free_port()]
    procs = [ctx.Process(target=native_pg_cuda_worker, args=(r, n, *ports, str(tmp_path), q)) for r in range(n)]
    for p in procs:
        p.start()
    try:
        for _ in range(n):
            rank, status, info = q.get(timeout=300)
            assert status == "ok", "rank %d:\n%s" % (rank, info)
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
