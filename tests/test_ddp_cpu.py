"""Gradient bucketing and the DDP wrapper on CPU tensors (dummy backend: every job
multiplies by num_workers, which stands in for a sum over identical workers)."""
import pytest
import torch

import switchml_b200 as sml
from switchml_b200.parallel.ddp import GradientBuckets, DistributedDataParallel


@pytest.fixture
def ctx():
    c = sml.Context.get_instance()
    assert c.start(sml.make_config("dummy", num_workers=2, packet_numel=64, bandwidth=0))
    yield c
    if c.state() == sml.ContextState.RUNNING:
        c.stop()


def _model():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(20, 64), torch.nn.Tanh(), torch.nn.Linear(64, 64), torch.nn.Tanh(),
                               torch.nn.Linear(64, 3))


def test_buckets_cover_all_parameters_in_reverse_order(ctx):
    m = _model()
    b = GradientBuckets(m.parameters(), ctx, bucket_mb=0.01)     # ~10 KB buckets -> several of them
    assert len(b.buckets) > 1
    assert sum(len(g) for g in b.bucket_params) == len(list(m.parameters()))
    assert b.bucket_params[0][0] is list(m.parameters())[-1]     # last parameter first
    for p in m.parameters():
        assert p.grad is not None and p.grad.shape == p.shape and float(p.grad.abs().sum()) == 0.0
        bucket = b.buckets[b.param_bucket[id(p)]]
        lo, hi = bucket.data_ptr(), bucket.data_ptr() + bucket.numel() * 4
        assert lo <= p.grad.data_ptr() < hi, "grad must be a view into its bucket"


def test_wrapper_reduces_every_gradient_once(ctx):
    m, ref = _model(), _model()
    ddp = DistributedDataParallel(m, ctx, bucket_mb=0.01, overlap=True)
    x = torch.randn(8, 20)
    for _ in range(2):
        ddp.zero_grad()
        ref.zero_grad()
        ddp(x).square().mean().backward()
        ref(x).square().mean().backward()
        for p, rp in zip(m.parameters(), ref.parameters()):
            assert torch.allclose(p.grad, 2.0 * rp.grad, rtol=1e-5, atol=1e-7)   # "sum" over 2 identical workers
    assert ctx.get_stats()["jobs_failed"] == 0


def test_unused_parameters_are_still_reduced(ctx):
    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.used = torch.nn.Linear(4, 4)
            self.unused = torch.nn.Linear(4, 4)

        def forward(self, x):
            return self.used(x)

    net = Net()
    ddp = DistributedDataParallel(net, ctx, bucket_mb=0.0001, overlap=True)
    before = ctx.get_stats()["jobs_submitted"]
    ddp(torch.randn(2, 4)).sum().backward()
    # every bucket is submitted, so all workers issue the same jobs in the same order
    assert ctx.get_stats()["jobs_submitted"] - before == len(ddp.buckets.buckets)
    assert float(net.unused.weight.grad.abs().sum()) == 0.0


def test_no_sync_accumulates_locally(ctx):
    m, ref = _model(), _model()
    ddp = DistributedDataParallel(m, ctx, bucket_mb=0.01)
    x = torch.randn(8, 20)
    ddp.zero_grad()
    before = ctx.get_stats()["jobs_submitted"]
    with ddp.no_sync():
        ddp(x).square().mean().backward()
        ddp(x).square().mean().backward()
    assert ctx.get_stats()["jobs_submitted"] == before, "no job may be submitted inside no_sync()"
    ref(x).square().mean().backward()
    for p, rp in zip(m.parameters(), ref.parameters()):
        assert torch.allclose(p.grad, 2.0 * rp.grad, rtol=1e-5, atol=1e-7)      # two local passes
    ddp(x).square().mean().backward()                                           # third pass, reduced with the rest
    for p, rp in zip(m.parameters(), ref.parameters()):
        assert torch.allclose(p.grad, 2.0 * 3.0 * rp.grad, rtol=1e-5, atol=1e-7)  # x2: the dummy "sum" of 2 workers


def test_parameters_are_broadcast_and_gradients_summed_across_real_workers():
    """Two processes over the UDP backend and the software switch."""
    import multiprocessing as mp
    from conftest import free_port
    from _workers import ddp_broadcast_worker
    ports = (free_port(), free_port())
    mpc = mp.get_context("spawn")
    q = mpc.Queue()
    procs = [mpc.Process(target=ddp_broadcast_worker, args=(r, 2, ports[0], ports[1], q)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    try:
        for _ in range(2):
            rank, status, payload = q.get(timeout=180)
            assert status == "ok", payload
            got[rank] = {"state": {k: torch.from_numpy(v) for k, v in payload["state"].items()},
                         **{k: [torch.from_numpy(g) for g in payload[k]] for k in ("g1", "g2", "local")}}
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    # same state everywhere, and it is rank 0's initial one (up to the fixed-point grid of the quantised trip)
    torch.manual_seed(100)
    want = torch.nn.Sequential(torch.nn.Linear(12, 32), torch.nn.BatchNorm1d(32), torch.nn.Tanh(),
                               torch.nn.Linear(32, 4)).state_dict()
    for k, v in got[0]["state"].items():
        assert torch.equal(v, got[1]["state"][k]), k
        if k.endswith("num_batches_tracked"):
            assert int(v) == 100
        else:
            assert torch.allclose(v, want[k], rtol=0, atol=1e-6), k
    # gradients: identical on both ranks and equal to the sum of the local ones
    model = torch.nn.Sequential(torch.nn.Linear(12, 32), torch.nn.BatchNorm1d(32), torch.nn.Tanh(),
                                torch.nn.Linear(32, 4))
    model.load_state_dict(got[0]["state"])
    xs = [torch.randn(6, 12, generator=torch.Generator().manual_seed(50 + r)) for r in range(2)]
    total = None
    for r in range(2):
        model.zero_grad()
        model.train()
        model(xs[r]).square().mean().backward()
        grads = [p.grad.clone() for p in model.parameters()]
        total = grads if total is None else [a + b for a, b in zip(total, grads)]
    for a, b, t in zip(got[0]["g1"], got[1]["g1"], total):
        assert torch.equal(a, b)
        assert torch.allclose(a, t, rtol=1e-4, atol=1e-6)
    for a, b in zip(got[0]["g2"], got[1]["g2"]):
        assert torch.equal(a, b)
    assert not all(torch.equal(a, b) for a, b in zip(got[0]["local"], got[1]["local"])), \
        "inside no_sync() the gradients must stay local"


def test_torch_ddp_with_the_comm_hook_on_cpu():
    """torch's own DistributedDataParallel, two processes, gradients reduced by the SwitchML
    comm hook over the UDP backend."""
    import multiprocessing as mp
    from conftest import free_port
    from _workers import ddp_hook_cpu_worker
    ports = (free_port(), free_port(), free_port())
    mpc = mp.get_context("spawn")
    q = mpc.Queue()
    procs = [mpc.Process(target=ddp_hook_cpu_worker, args=(r, 2, ports[0], ports[1], ports[2], q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        for _ in range(2):
            rank, status, info = q.get(timeout=180)
            assert status == "ok", info
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
