"""Allreduce for callers whose tensors live in (pinned) host memory.

The reference's PyTorch integration always works this way: a CUDA tensor is copied to
pinned host memory, reduced by the CPU library and copied back, one step after the other
(pytorch_plugin/ProcessGroupSML.cpp:117-163). Here the direction is reversed — host data
is brought to the GPU, reduced over NVLink and returned — and the three stages are
pipelined over chunks on three streams, so that the PCIe copies in both directions and
the reduction overlap.
"""
import torch


class HostAllReduce:
    def __init__(self, ctx, numel, dtype, chunk_numel=1 << 24, device=None):
        self.ctx = ctx
        self.numel = numel
        self.chunk = max(1, min(chunk_numel, numel))
        dev = torch.device("cuda", torch.cuda.current_device() if device is None else device)
        self.dx = torch.empty(numel, dtype=dtype, device=dev)
        self.dy = torch.empty(numel, dtype=dtype, device=dev)
        self.s_in = torch.cuda.Stream(device=dev)
        self.s_comm = torch.cuda.Stream(device=dev)
        self.s_out = torch.cuda.Stream(device=dev)
        self.bounds = [(o, min(o + self.chunk, numel)) for o in range(0, numel, self.chunk)]
        self.launches_per_run = len(self.bounds)

    def run(self, host_in, host_out):
        """Reduce `host_in` across workers into `host_out` (both pinned, 1-D). Blocks
        until `host_out` is complete."""
        jobs = []
        for lo, hi in self.bounds:
            with torch.cuda.stream(self.s_in):
                self.dx[lo:hi].copy_(host_in[lo:hi], non_blocking=True)
            self.s_comm.wait_stream(self.s_in)
            job = self.ctx.all_reduce_async(self.dx[lo:hi], self.dy[lo:hi], stream=self.s_comm)
            job.stream_wait(self.s_out)
            jobs.append(job)
            with torch.cuda.stream(self.s_out):
                host_out[lo:hi].copy_(self.dy[lo:hi], non_blocking=True)
        self.s_out.synchronize()
        for j in jobs:
            j.release()
        return host_out

    def close(self):
        self.dx = self.dy = None
