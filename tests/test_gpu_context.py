"""The cuda backend through the public Context API on a single GPU (num_workers = 1):
lifecycle, both launch modes, stream ordering, statistics, and the bounded device wait
that reports a timeout instead of hanging."""
import numpy as np
import pytest
import torch

import switchml_b200 as sml
from switchml_b200.ops.oracle import quant_allreduce_oracle

pytestmark = pytest.mark.gpu


@pytest.fixture
def ctx():
    c = sml.Context.get_instance()
    yield c
    if c.state() == sml.ContextState.RUNNING:
        c.stop()


@pytest.mark.parametrize("launch", ["worker", "inline"])
@pytest.mark.parametrize("mode", ["int32_quant", "float_sum"])
def test_single_rank_roundtrip(ctx, launch, mode):
    assert ctx.start(sml.make_config("cuda", packet_numel=256, mode=mode, launch=launch))
    for numel in (1, 255, 70000, (1 << 22) + 5):
        x = torch.randn(numel, device="cuda")
        y = torch.empty_like(x)
        job = ctx.all_reduce_async(x, y)
        assert job.wait() == sml.JobStatus.FINISHED, job.error()
        if mode == "int32_quant":
            want = quant_allreduce_oracle([x.cpu().numpy()], 256)
            assert np.array_equal(y.cpu().numpy(), want)
        else:
            assert torch.equal(x, y)
    xi = torch.arange(100000, dtype=torch.int32, device="cuda")
    ctx.all_reduce(xi)
    assert torch.equal(xi, torch.arange(100000, dtype=torch.int32, device="cuda"))
    st = ctx.get_stats()
    assert st["jobs_finished"] == 5 and st["jobs_failed"] == 0
    if mode == "int32_quant":
        assert st["backend"]["tiles"] > 0   # a single worker still goes through the slot pipeline
    # (float_sum with one worker is a plain copy kernel, or nothing at all in place)


def test_stream_ordering_without_host_sync(ctx):
    assert ctx.start(sml.make_config("cuda", packet_numel=256, mode="float_sum", launch="worker"))
    side = torch.cuda.Stream()
    x = torch.zeros(1 << 22, device="cuda")
    with torch.cuda.stream(side):
        # The producer writes on `side`; the job is ordered after it by an event.
        for _ in range(20):
            x.add_(1.0)
        job = ctx.all_reduce_async(x)
        job.stream_wait(side)
        y = x * 2
    side.synchronize()
    assert job.wait() == sml.JobStatus.FINISHED
    assert float(y[0]) == 40.0 and float(y[-1]) == 40.0


def test_average_and_bf16(ctx):
    assert ctx.start(sml.make_config("cuda", packet_numel=256, mode="float_sum", average=True, launch="inline"))
    x = torch.randn(300000, device="cuda").bfloat16()
    keep = x.clone()
    ctx.all_reduce(x)
    assert torch.equal(x, keep)  # one worker: mean == value


def test_bounded_wait_reports_timeout_and_context_survives(ctx):
    assert ctx.start(sml.make_config("cuda", packet_numel=256, mode="float_sum"))
    status = ctx.wait_probe(budget_ms=30.0)
    assert status & 0xF == 1, "the wait must give up with STATUS_TIMEOUT"
    assert ctx.get_stats()["backend"]["device_timeouts"] >= 1
    x = torch.ones(1000, device="cuda")
    ctx.all_reduce(x)  # the context is still usable
    assert float(x.sum()) == 1000.0


def test_bfloat16_needs_cuda_backend():
    c = sml.Context.get_instance()
    assert c.start(sml.make_config("dummy", bandwidth=0))
    try:
        x = torch.ones(10, dtype=torch.bfloat16)
        job = c.all_reduce_async(x)
        assert job.wait() == sml.JobStatus.FAILED and "cuda" in job.error()
    finally:
        c.stop()


def test_host_pipeline_roundtrip(ctx):
    """Pinned host -> device -> allreduce -> pinned host, chunked over three streams."""
    from switchml_b200.parallel.host_pipeline import HostAllReduce
    assert ctx.start(sml.make_config("cuda", packet_numel=256, mode="float_sum", launch="inline"))
    n = (1 << 20) + 123
    hx = torch.randn(n).pin_memory()
    hy = torch.zeros(n).pin_memory()
    pipe = HostAllReduce(ctx, n, torch.float32, chunk_numel=1 << 18)
    assert pipe.launches_per_run == 5
    for _ in range(2):
        pipe.run(hx, hy)
        assert torch.equal(hx, hy)
        hy.zero_()
    pipe.close()
