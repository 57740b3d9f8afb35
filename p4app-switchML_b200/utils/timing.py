"""Device-side timing helpers used by the benchmarks: CUDA events on the launching stream,
warm-up first, synchronise on both sides, and for several ranks the slowest one counts."""
import torch


def time_cuda(fn, iters, warmup=3, group_world=1):
    """Average milliseconds per call of `fn` over `iters` calls (after `warmup` calls),
    maximum over the ranks of the default process group when `group_world` > 1."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if group_world > 1:
        import torch.distributed as dist
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    if group_world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def flush_l2(scratch=None):
    """Overwrite a buffer larger than the 126 MB L2 so that the next kernel starts cold."""
    if scratch is None:
        scratch = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    scratch.zero_()
    return scratch
