"""Allreduce for callers whose tensors live in (pinned) host memory.

The reference's PyTorch integration always works this way: a CUDA tensor is copied to
pinned host memory, reduced by the CPU library and copied back, one step after the other
(pytorch_plugin/ProcessGroupSML.cpp:117-163). Here the direction is reversed — host data
is brought to the GPU, reduced over NVLink and returned. Three ways of doing it:

* pipelined copies (default): the tensor is cut into chunks; host→device copy, reduction and
  device→host copy of different chunks overlap on three streams.
* ``direct="out"``: chunks are copied host→device as above, but every chunk's reduction writes
  its result straight into the pinned output (the kernel's storer warps store over PCIe), so
  the device→host copy, its stream and the device copy of the result disappear.
* ``direct=True``: one job on the pinned buffers themselves. The aggregation kernel's loader
  warps read the input over PCIe while its storer warps write finished tiles back, so both
  directions and the NVLink phase overlap tile by tile inside a single launch, and no device
  copy of the tensor exists at all. (The cuda backend accepts any memory the GPU can reach:
  device, managed, or pinned host memory.)
"""
import torch


class HostAllReduce:
    def __init__(self, ctx, numel, dtype, chunk_numel=1 << 24, device=None, direct=False):
        self.ctx = ctx
        self.numel = numel
        self.direct = direct
        dev = torch.device("cuda", torch.cuda.current_device() if device is None else device)
        self.s_comm = torch.cuda.Stream(device=dev)
        if direct is True:
            self.launches_per_run = 1
            return
        self.chunk = max(1, min(chunk_numel, numel))
        self.dx = torch.empty(numel, dtype=dtype, device=dev)
        self.dy = None if direct == "out" else torch.empty(numel, dtype=dtype, device=dev)
        self.s_in = torch.cuda.Stream(device=dev)
        self.s_out = torch.cuda.Stream(device=dev)
        self.bounds = [(o, min(o + self.chunk, numel)) for o in range(0, numel, self.chunk)]
        self.launches_per_run = len(self.bounds)

    def run(self, host_in, host_out):
        """Reduce `host_in` across workers into `host_out` (both pinned, 1-D). Blocks
        until `host_out` is complete."""
        if self.direct is True:
            job = self.ctx.all_reduce_async(host_in, host_out, stream=self.s_comm)
            status = job.wait()
            if status != 3:
                raise RuntimeError("allreduce on pinned memory failed: " + job.error())
            job.release()
            return host_out
        jobs = []
        if self.direct == "out":
            for lo, hi in self.bounds:
                with torch.cuda.stream(self.s_in):
                    self.dx[lo:hi].copy_(host_in[lo:hi], non_blocking=True)
                self.s_comm.wait_stream(self.s_in)
                jobs.append(self.ctx.all_reduce_async(self.dx[lo:hi], host_out[lo:hi], stream=self.s_comm))
            for j in jobs:
                if j.wait() != 3:
                    raise RuntimeError("allreduce into pinned memory failed: " + j.error())
                j.release()
            return host_out
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
