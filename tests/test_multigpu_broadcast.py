"""Context.broadcast on several GPUs (a job type the reference declares but does not
implement): every rank checks that it received the root's tensor."""
import multiprocessing as mp

import pytest
import torch

from conftest import free_port
from _workers import broadcast_cuda_worker

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


@pytest.mark.parametrize("mode", ["float_sum", "int32_quant"])
def test_broadcast_reaches_every_gpu(mode):
    n = min(torch.cuda.device_count(), 4)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=broadcast_cuda_worker, args=(r, n, port, mode, q)) for r in range(n)]
    for p in procs:
        p.start()
    try:
        for _ in range(n):
            rank, status, info = q.get(timeout=240)
            assert status == "ok", "rank %d:\n%s" % (rank, info)
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
