"""The software stack on the dummy backend (reference backends/dummy): every process
sees its own data multiplied by num_workers, packets complete out of order, float jobs go
through the block-exponent quantiser. Includes the plumbing configuration of the benchmark plan: 2 workers,
2^20 float32 ~N(0,1), packet_numel 64, 256 slots, checked against a float64 sum."""
import numpy as np
import pytest

import switchml_b200 as sml


@pytest.fixture
def ctx():
    c = sml.Context.get_instance()
    yield c
    if c.state() == sml.ContextState.RUNNING:
        c.stop()


def test_baseline_plumbing_config(ctx):
    assert ctx.start(sml.make_config("dummy", rank=0, num_workers=2, packet_numel=64,
                                     max_outstanding_packets=256, bandwidth=0))
    rng = np.random.default_rng(1234)
    x = rng.standard_normal(1 << 20).astype(np.float32)
    keep = x.copy()
    y = np.empty_like(x)
    job = ctx.all_reduce(x, y)
    assert job.status() == sml.JobStatus.FINISHED
    assert np.array_equal(x, keep), "the input buffer must stay untouched"
    want = 2.0 * x.astype(np.float64)
    # per block: n^2 * 2^(E-32) with 2^E < 2*max|x|
    assert np.max(np.abs(y - want)) < 4 * 2.0 ** -32 * 2 * np.abs(x).max() * 4
    stats = ctx.get_stats()
    assert stats["jobs_submitted"] == 1 and stats["jobs_finished"] == 1
    pkts = (1 << 20) // 64
    # one extra leading batch per worker thread carries only exponents
    assert sum(stats["total_pkts_sent"]) == pkts + 256
    assert sum(stats["correct_pkts_received"]) == pkts + 256


@pytest.mark.parametrize("numel", [1, 63, 64, 65, 255, 1000, 4097, (1 << 16) + 1])
@pytest.mark.parametrize("ppp", ["cpu_exponent_quantizer", "bypass"])
def test_odd_sizes_inplace_int(ctx, numel, ppp):
    assert ctx.start(sml.make_config("dummy", num_workers=3, packet_numel=64, num_worker_threads=4,
                                     max_outstanding_packets=32, prepostprocessor=ppp, bandwidth=0))
    x = (np.arange(numel, dtype=np.int32) * 7919) % 1000 - 500
    want = x * 3
    ctx.all_reduce(x)
    if ppp == "bypass":
        assert np.array_equal(x, want // 3)  # bypass never touches user data
    else:
        assert np.array_equal(x, want)


def test_uint8_is_summed_as_int32_and_narrowed(ctx):
    """uint8 tensors make the trip as int32 and come back modulo 256 (the dummy backend
    multiplies by the number of workers)."""
    assert ctx.start(sml.make_config("dummy", rank=0, num_workers=3, packet_numel=64, bandwidth=0))
    x = (np.arange(700) % 256).astype(np.uint8)
    y = np.zeros_like(x)
    job = ctx.all_reduce_async(x, y)
    assert job.wait(10000) == sml.JobStatus.FINISHED
    assert np.array_equal(y, ((np.arange(700) % 256) * 3 % 256).astype(np.uint8))
    assert np.array_equal(x, (np.arange(700) % 256).astype(np.uint8)), "the input must stay untouched"
    ctx.all_reduce(x)  # in place
    assert np.array_equal(x, y)


def test_async_jobs_and_stats(ctx):
    assert ctx.start(sml.make_config("dummy", num_workers=4, packet_numel=256, bandwidth=0))
    xs = [np.full(1 << 15, float(i + 1), dtype=np.float32) for i in range(8)]
    outs = [np.empty_like(x) for x in xs]
    jobs = [ctx.all_reduce_async(x, o) for x, o in zip(xs, outs)]
    ctx.wait_for_all_jobs()
    for i, (j, o) in enumerate(zip(jobs, outs)):
        assert j.status() == sml.JobStatus.FINISHED
        assert np.allclose(o, 4.0 * (i + 1), rtol=1e-6)
    rep = ctx.stats_report()
    assert "Submitted jobs: #8#" in rep and "Finished jobs: #8#" in rep


def test_zero_and_extreme_blocks(ctx):
    assert ctx.start(sml.make_config("dummy", num_workers=2, packet_numel=64, bandwidth=0))
    x = np.zeros(64 * 6, dtype=np.float32)
    x[64:128] = 1e-30          # tiny block
    x[128:192] = 3e37          # close to the top of the range
    x[192:256] = np.float32(1e-45)  # denormals
    x[256] = -1.5              # rest of the block zero
    y = np.empty_like(x)
    ctx.all_reduce(x, y)
    assert np.all(np.isfinite(y))
    assert np.all(y[:64] == 0)
    assert np.allclose(y[64:128], 2e-30, rtol=1e-6)
    assert np.allclose(y[128:192], 6e37, rtol=1e-6)
    assert y[256] == -3.0 and np.all(y[257:320] == 0)


def test_instant_job_completion(ctx):
    assert ctx.start(sml.make_config("dummy", num_workers=2, instant_job_completion=True))
    x = np.ones(1000, dtype=np.float32)
    ctx.all_reduce(x)
    assert np.all(x == 1.0)


def test_bandwidth_model_sleeps(ctx):
    import time
    # 100 Mbps: 2^16 floats (plus the exponent batch) take at least ~20 ms
    assert ctx.start(sml.make_config("dummy", num_workers=2, packet_numel=256, bandwidth=100.0))
    x = np.ones(1 << 16, dtype=np.float32)
    t0 = time.time()
    ctx.all_reduce(x)
    assert time.time() - t0 > 0.015


def test_api_misuse(ctx):
    with pytest.raises(sml.NativeError):
        ctx.all_reduce(np.ones(4, dtype=np.float32))  # not started
    assert ctx.start(sml.make_config("dummy", bandwidth=0))
    with pytest.raises(TypeError):
        ctx.all_reduce(np.ones(4, dtype=np.float64))
    with pytest.raises(ValueError):
        ctx.all_reduce(np.ones(4, dtype=np.float32), np.ones(5, dtype=np.float32))
    ctx.stop()
    assert ctx.state() == sml.ContextState.STOPPED
    assert ctx.start(sml.make_config("dummy", bandwidth=0))  # restart works


def test_broadcast_on_the_dummy_backend(ctx):
    """One worker: trivially done. Several "workers" of the dummy backend never meet, so only
    the root can be served."""
    assert ctx.start(sml.make_config("dummy", rank=0, num_workers=1, bandwidth=0))
    x = np.arange(10, dtype=np.float32)
    ctx.broadcast(x, 0)
    assert np.array_equal(x, np.arange(10, dtype=np.float32))
    ctx.stop()
    assert ctx.start(sml.make_config("dummy", rank=1, num_workers=2, bandwidth=0))
    assert ctx.broadcast_async(x, root=1).wait(5000) == sml.JobStatus.FINISHED
    job = ctx.broadcast_async(x, root=0)
    assert job.wait(5000) == sml.JobStatus.FAILED and "no peers" in job.error()
    assert np.array_equal(x, np.arange(10, dtype=np.float32))
    stats = ctx.get_stats()
    assert stats["jobs_submitted"] == 2 and stats["jobs_finished"] == 1 and stats["jobs_failed"] == 1


def test_running_context_manager_and_job_repr():
    c = sml.Context.get_instance()
    with c.running(sml.make_config("dummy", num_workers=2, bandwidth=0)) as ctx:
        x = np.ones(100, dtype=np.float32)
        job = ctx.all_reduce_async(x)
        job.wait()
        assert "FINISHED" in repr(job)
        job.release()
        assert "released" in repr(job)
        assert float(x[0]) == 2.0
    assert c.state() == sml.ContextState.STOPPED
    with pytest.raises(ZeroDivisionError):
        with c.running(sml.make_config("dummy", bandwidth=0)):
            1 / 0
    assert c.state() == sml.ContextState.STOPPED
