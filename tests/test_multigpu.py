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
