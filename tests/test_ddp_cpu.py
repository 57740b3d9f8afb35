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
