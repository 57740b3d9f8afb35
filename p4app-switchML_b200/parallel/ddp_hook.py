"""Communication hook for ``torch.nn.parallel.DistributedDataParallel``.

    ddp = torch.nn.parallel.DistributedDataParallel(model, bucket_cap_mb=25)
    ddp.register_comm_hook(SwitchMLHookState(ctx), switchml_allreduce_hook)

The reference's process group cannot serve a comm hook because its work objects have no
future (pytorch_plugin/ProcessGroupSML.cpp:191-193). This hook returns a CUDA-aware
future: the bucket is reduced on a side stream while backward continues, and DDP's
finalisation orders the compute stream after it.
"""
import torch


class SwitchMLHookState:
    """`average` = True (what DDP expects of a hook): the bucket ends up holding the mean over
    the workers. If the context already averages (``average = true`` in [backend.cuda]) nothing
    is added; otherwise the hook divides the sum by the number of workers."""

    def __init__(self, ctx, average=True):
        self.ctx = ctx
        self.average = average
        self.stream = None
        self.jobs = []
        dump = ctx.config_dump()
        self.num_workers = 1
        for line in dump.splitlines():
            parts = line.split("=")
            if len(parts) == 2 and parts[0].strip() == "num_workers":
                self.num_workers = int(parts[1].strip())
        self.context_averages = "backend = cuda" in dump and "average = true" in dump
        self.divide = bool(average) and not self.context_averages and self.num_workers > 1


def switchml_allreduce_hook(state, bucket):
    buf = bucket.buffer()
    if not buf.is_cuda:
        job = state.ctx.all_reduce_async(buf)
        job.wait()
        job.release()
        if state.divide:
            buf.div_(state.num_workers)
        fut = torch.futures.Future()
        fut.set_result(buf)
        return fut
    if state.stream is None:
        state.stream = torch.cuda.Stream(device=buf.device, priority=-1)
    # Jobs of earlier buckets that have certainly been consumed can be dropped.
    if len(state.jobs) > 64:
        for j in state.jobs[:-32]:
            j.release()
        state.jobs = state.jobs[-32:]
    state.stream.wait_stream(torch.cuda.current_stream(buf.device))
    fut = torch.futures.Future(devices=[buf.device])
    with torch.cuda.stream(state.stream):
        job = state.ctx.all_reduce_async(buf, stream=state.stream)
        job.stream_wait(state.stream)
        state.jobs.append(job)
        if state.divide:
            buf.div_(state.num_workers)
        # set_result records an event on the current (side) stream; whoever waits on the
        # future is ordered after the reduction.
        fut.set_result(buf)
    return fut
