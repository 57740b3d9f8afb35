"""Data-parallel training on top of the Context: gradient buckets and a DDP wrapper.

The reference leaves bucketing to PyTorch DDP / Horovod and plugs in underneath as a
process group whose allreduce blocks inside the call (pytorch_plugin/ProcessGroupSML.cpp:
113-163), so communication never overlaps the backward pass; its dnn_benchmark models
the overlap it would like to have (benchmarks/dnn_benchmark/main.cc:298-327). Here the
overlap is real: gradients live in flat buckets (optionally inside the symmetric heap, so
they are reduced in place over NVLink with no staging copy), a bucket is submitted on a
side stream the moment its last gradient is produced, and the compute stream only waits
at the end of backward.
"""
import torch


class GradientBuckets:
    """Flat gradient storage for a set of parameters, cut into buckets of ~`bucket_mb`.

    Parameters are taken in reverse order (gradients appear roughly in that order during
    backward). Each parameter's ``.grad`` becomes a view into its bucket; keep it that
    way by zeroing with :meth:`zero_` (or ``optimizer.zero_grad(set_to_none=False)``).
    """

    def __init__(self, params, ctx, bucket_mb=25, symmetric="auto"):
        self.ctx = ctx
        # Gradients that a fused kernel already reduces during backward stay out of the buckets.
        params = [p for p in params if p.requires_grad and not getattr(p, "_sml_reduced_in_backward", False)]
        self.params = list(reversed(params))
        cap = int(bucket_mb * (1 << 20))
        groups, cur, cur_bytes, cur_dtype = [], [], 0, None
        for p in self.params:
            nbytes = p.numel() * p.element_size()
            if cur and (p.dtype != cur_dtype or cur_bytes + nbytes > cap):
                groups.append(cur)
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_bytes += nbytes
            cur_dtype = p.dtype
        if cur:
            groups.append(cur)
        self.buckets = []        # flat tensors
        self.bucket_params = groups
        self.param_bucket = {}   # id(param) -> bucket index
        self.in_symmetric_heap = []
        for bi, group in enumerate(groups):
            # 64-element alignment keeps every view 256-byte aligned for fp32
            offs, total = [], 0
            for p in group:
                offs.append(total)
                total += (p.numel() + 63) // 64 * 64
            flat, symm = self._allocate(total, group[0].dtype, group[0].device, symmetric)
            flat.zero_()
            for p, off in zip(group, offs):
                p.grad = flat[off:off + p.numel()].view_as(p)
                self.param_bucket[id(p)] = bi
            self.buckets.append(flat)
            self.in_symmetric_heap.append(symm)
        self.jobs = []

    def _allocate(self, numel, dtype, device, symmetric):
        if symmetric in (True, "auto") and device.type == "cuda":
            try:
                return self.ctx.symmetric_empty(numel, dtype), True
            except (MemoryError, RuntimeError):
                if symmetric is True:
                    raise
        return torch.empty(numel, dtype=dtype, device=device), False

    def zero_(self):
        for b in self.buckets:
            b.zero_()

    def all_reduce_bucket(self, index, stream=None):
        job = self.ctx.all_reduce_async(self.buckets[index], stream=stream)
        self.jobs.append(job)
        return job

    def all_reduce(self, stream=None):
        """Submit every bucket (no overlap with backward)."""
        for i in range(len(self.buckets)):
            self.all_reduce_bucket(i, stream)

    def wait(self, stream=None):
        """Order `stream` (default: current) after all submitted buckets."""
        for j in self.jobs:
            if self.buckets[0].is_cuda:
                j.stream_wait(stream)
            else:
                j.wait()
            j.release()
        self.jobs = []


class DistributedDataParallel(torch.nn.Module):
    """Wraps a module: broadcasts nothing (ranks must start from the same weights, e.g.
    the same seed), averages gradients across workers during backward.

    Configure the context with ``average = true`` in [backend.cuda] to get the mean; with
    the default the gradients are summed, like a raw SwitchML allreduce.
    """

    def __init__(self, module, ctx, bucket_mb=25, overlap=True, symmetric="auto"):
        super().__init__()
        self.module = module
        self.ctx = ctx
        self.overlap = overlap
        self.buckets = GradientBuckets(module.parameters(), ctx, bucket_mb, symmetric)
        self._pending = [0] * len(self.buckets.buckets)
        self._armed = False
        self._comm_stream = None
        dev = next(module.parameters()).device
        if dev.type == "cuda":
            self._comm_stream = torch.cuda.Stream(device=dev, priority=-1)
        for p in self.buckets.params:
            p.register_post_accumulate_grad_hook(self._on_grad)
        self._callback_queued = False

    def forward(self, *args, **kwargs):
        if torch.is_grad_enabled():
            self._pending = [len(g) for g in self.buckets.bucket_params]
            self._armed = True
            self._callback_queued = False
        return self.module(*args, **kwargs)

    def _on_grad(self, param):
        if not self._armed:
            return
        if not self._callback_queued:
            # Runs when the whole backward pass is done: make the compute stream wait.
            torch.autograd.Variable._execution_engine.queue_callback(self._finish)
            self._callback_queued = True
        bi = self.buckets.param_bucket[id(param)]
        self._pending[bi] -= 1
        if self._pending[bi] == 0 and self.overlap:
            self._launch(bi)

    def _launch(self, bi):
        if self._comm_stream is None:
            self.buckets.all_reduce_bucket(bi)
            return
        self._comm_stream.wait_stream(torch.cuda.current_stream())
        self.buckets.all_reduce_bucket(bi, stream=self._comm_stream)

    def _finish(self):
        if not self._armed:
            return
        self._armed = False
        for bi, left in enumerate(self._pending):
            if not self.overlap or left > 0:
                # Parameters unused in this step never fire their hook: reduce anyway so
                # that all ranks submit the same jobs in the same order.
                self._launch(bi)
        self.buckets.wait()
        from ..ops import wgrad as _wgrad
        _wgrad.wait_pending()  # fused weight-gradient kernels running on their side stream

    def zero_grad(self, set_to_none=False):
        self.buckets.zero_()
