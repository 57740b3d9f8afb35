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
        assert st["backend"]["kernel_launches"] >= 4   # a single worker still runs a kernel per float job: the round trip
                                                       # through the fixed-point grid changes the values
    # (float_sum with one worker is a plain copy kernel, or nothing at all in place)


@pytest.mark.parametrize("block", [32, 64, 128, 512, 1024])
def test_single_worker_exact_mode_is_one_pass_and_bit_exact(ctx, block):
    """One worker in int32_quant mode takes the single-pass kernel (aligned float32) or the
    streaming kernel (anything else); both must give the oracle's bits, in and out of place."""
    assert ctx.start(sml.make_config("cuda", packet_numel=block, mode="int32_quant", launch="inline"))
    g = torch.Generator(device="cuda").manual_seed(block)
    numel = 21 * 1024 + 3 * block + 17
    base = torch.randn(numel + 4, device="cuda", generator=g) * torch.logspace(-20, 20, numel + 4, device="cuda")
    base[5 * block:7 * block] = 0.0
    for x in (base[:numel], base[1:1 + numel]):            # 16-byte aligned, and 4-byte aligned only
        want = quant_allreduce_oracle([x.cpu().numpy()], block)
        y = torch.empty(numel + 4, device="cuda")[x.storage_offset():x.storage_offset() + numel]
        job = ctx.all_reduce_async(x.contiguous() if x.storage_offset() == 0 else x, y)
        assert job.wait() == sml.JobStatus.FINISHED, job.error()
        assert np.array_equal(y.cpu().numpy().view(np.uint32), want.view(np.uint32)), (block, x.storage_offset())
    z = base[:numel].clone()
    want = quant_allreduce_oracle([z.cpu().numpy()], block)
    ctx.all_reduce(z)
    assert np.array_equal(z.cpu().numpy().view(np.uint32), want.view(np.uint32))


def test_inline_jobs_on_unordered_streams_do_not_overlap(ctx):
    """launch = inline enqueues every job on its caller's stream, but all jobs of a context share
    the staging slots, the flags and the per-channel epochs: a job submitted on another stream
    than its predecessor must be ordered after it by the backend itself. Many quantised jobs on
    two streams that nothing else orders, each checked against the oracle."""
    assert ctx.start(sml.make_config("cuda", packet_numel=256, mode="int32_quant", launch="inline"))
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    numel = (1 << 21) + 77
    xs = [torch.randn(numel, device="cuda") * (3.0 ** i) for i in range(6)]
    ys = [torch.empty_like(x) for x in xs]
    torch.cuda.synchronize()
    jobs = []
    for rounds in range(3):
        for i, (x, y) in enumerate(zip(xs, ys)):
            jobs.append(ctx.all_reduce_async(x, y, stream=streams[i % 2]))
    for j in jobs:
        assert j.wait() == sml.JobStatus.FINISHED, j.error()
    torch.cuda.synchronize()
    for x, y in zip(xs, ys):
        want = quant_allreduce_oracle([x.cpu().numpy()], 256)
        assert np.array_equal(y.cpu().numpy(), want)
    assert ctx.get_stats()["jobs_failed"] == 0


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


def test_jobs_can_be_captured_in_a_cuda_graph_and_replayed(ctx):
    """Epochs live on the device, so a captured launch carries nothing that goes stale:
    replaying the graph runs the same jobs again on whatever the buffers hold then."""
    assert ctx.start(sml.make_config("cuda", packet_numel=256, mode="int32_quant", launch="inline"))
    small = torch.randn(10_000, device="cuda")          # one-barrier kernel
    large = torch.randn(3_000_001, device="cuda")       # streamed through the slot ring
    out_s, out_l = torch.empty_like(small), torch.empty_like(large)
    warm = ctx.all_reduce_async(large, out_l)            # ordinary job first: epochs are not zero
    assert warm.wait() == sml.JobStatus.FINISHED
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.graph(graph, stream=side):
        j1 = ctx.all_reduce_async(small, out_s)
        j2 = ctx.all_reduce_async(large, out_l)
        j1.stream_wait()
        j2.stream_wait()
    assert j1.status() == sml.JobStatus.FINISHED and j2.status() == sml.JobStatus.FINISHED
    for it in range(3):
        small.normal_()
        large.normal_()
        out_s.zero_()
        out_l.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert np.array_equal(out_s.cpu().numpy(), quant_allreduce_oracle([small.cpu().numpy()], 256))
        assert np.array_equal(out_l.cpu().numpy(), quant_allreduce_oracle([large.cpu().numpy()], 256))
    # ordinary jobs keep working after replays
    ctx.all_reduce(large, out_l)
    assert np.array_equal(out_l.cpu().numpy(), quant_allreduce_oracle([large.cpu().numpy()], 256))
    assert ctx.get_stats()["backend"]["device_timeouts"] == 0


@pytest.mark.parametrize("launch", ["worker", "inline"])
def test_ordinary_host_memory_is_refused_not_dereferenced(ctx, launch):
    """The kernels read their operands on the GPU. A pointer to pageable host memory fails
    the job on the host, before anything is launched; pinned memory is accepted."""
    assert ctx.start(sml.make_config("cuda", packet_numel=256, mode="float_sum", launch=launch))
    x = np.ones(1000, dtype=np.float32)
    job = ctx.all_reduce_async(x)
    assert job.wait(10000) == sml.JobStatus.FAILED
    assert "pageable" in job.error()
    d = torch.ones(1000, device="cuda")
    job = ctx.all_reduce_async(d, x)  # good input, bad output
    assert job.wait(10000) == sml.JobStatus.FAILED and "pageable" in job.error()
    assert float(x.sum()) == 1000.0
    p = torch.arange(1000, dtype=torch.float32).pin_memory()
    q = torch.zeros(1000, dtype=torch.float32).pin_memory()
    job = ctx.all_reduce_async(p.numpy(), q.numpy())
    assert job.wait(10000) == sml.JobStatus.FINISHED, job.error()
    torch.cuda.synchronize()
    assert torch.equal(p, q)
    y = torch.empty_like(d)
    assert ctx.all_reduce_async(d, y).wait(10000) == sml.JobStatus.FINISHED  # the context still works
    assert torch.equal(y.cpu(), d.cpu())


@pytest.mark.parametrize("numel,offset", [(1, 0), (15, 0), (16, 0), (4099, 0), (4099, 3), ((1 << 22) + 7, 0),
                                          ((1 << 22) + 7, 5), (1 << 24, 16)])
def test_uint8_widen_and_narrow_kernels(numel, offset):
    from switchml_b200.ops.elementwise import widen_u8, narrow_i32
    g = torch.Generator(device="cuda").manual_seed(numel)
    base = torch.randint(0, 256, (numel + offset + 9,), device="cuda", dtype=torch.uint8, generator=g)
    src = base[offset:offset + numel]
    wide = widen_u8(src)
    assert wide.dtype == torch.int32 and torch.equal(wide.cpu(), src.cpu().to(torch.int32))
    sums = wide * 5 - 300  # what an aggregate may look like: beyond a byte, also negative
    out = torch.full((numel + offset + 9,), 201, dtype=torch.uint8, device="cuda")
    narrow_i32(sums, out[offset:offset + numel])
    want = (sums.cpu().to(torch.int64) & 0xff).to(torch.uint8)
    assert torch.equal(out[offset:offset + numel].cpu(), want)
    assert bool((out[:offset] == 201).all()) and bool((out[offset + numel:] == 201).all())


def test_uint8_allreduce_single_rank(ctx):
    assert ctx.start(sml.make_config("cuda", packet_numel=256, mode="int32_quant", launch="inline"))
    x = torch.randint(0, 256, (100003,), device="cuda", dtype=torch.uint8)
    y = torch.zeros_like(x)
    ctx.all_reduce(x, y)
    torch.cuda.synchronize()
    assert torch.equal(x, y)


def test_service_threads_can_be_bound_to_the_gpus_numa_node(ctx):
    """numa_bind = true only narrows the CPU affinity of the launcher and completion threads
    (or does nothing where the machine has no NUMA information); jobs run as before."""
    assert ctx.start(sml.make_config("cuda", packet_numel=256, mode="float_sum", launch="worker", numa_bind=True))
    assert "numa_bind = true" in ctx.config_dump()
    x = torch.randn(1 << 20, device="cuda")
    y = torch.empty_like(x)
    for _ in range(3):
        assert ctx.all_reduce_async(x, y).wait(20000) == sml.JobStatus.FINISHED
    assert torch.equal(x, y)


def test_broadcast_single_rank(ctx):
    assert ctx.start(sml.make_config("cuda", packet_numel=256, mode="int32_quant", launch="inline"))
    x = torch.randn(100003, device="cuda")
    keep = x.clone()
    ctx.broadcast(x, 0)
    torch.cuda.synchronize()
    assert torch.equal(x, keep)
    job = ctx.broadcast_async(x, root=1)
    assert job.wait(5000) == sml.JobStatus.FAILED and "not a rank" in job.error()
