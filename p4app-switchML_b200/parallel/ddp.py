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


def broadcast_tensors(ctx, tensors, src=0, chunk_numel=1 << 24):
    """Give every worker rank `src`'s values of `tensors`, in place, through
    ``Context.broadcast`` (a sum to which everybody but `src` contributes zeros). Exact with
    ``mode = float_sum`` and for integers; with the quantised mode the values come back
    rounded to the block's fixed-point grid, the same on every rank (`src` included), which
    is what data-parallel training needs.

    Floating-point tensors travel as float32, integer tensors as int32 (values must fit),
    bool as int32 as well. Tensors are packed into flat messages of at most `chunk_numel`
    elements.
    """
    cfg = ctx.config_dump()
    rank, n = _config_int(cfg, "rank"), _config_int(cfg, "num_workers")
    if n <= 1:
        return
    groups = {}
    for t in tensors:
        if t.numel() == 0:
            continue
        wire = torch.float32 if t.is_floating_point() else torch.int32
        groups.setdefault((wire, t.device), []).append(t)
    for (wire, device), group in groups.items():
        batch, count = [], 0
        for t in group + [None]:
            if t is not None and (not batch or count + t.numel() <= chunk_numel):
                batch.append(t)
                count += t.numel()
                continue
            flat = torch.empty(count, dtype=wire, device=device)
            if rank == src:
                off = 0
                for b in batch:
                    flat[off:off + b.numel()].copy_(b.detach().reshape(-1))
                    off += b.numel()
            job = ctx.broadcast(flat, src)
            if flat.is_cuda:
                job.stream_wait(None)
            job.release()
            off = 0
            with torch.no_grad():
                for b in batch:
                    b.copy_(flat[off:off + b.numel()].view_as(b))
                    off += b.numel()
            batch, count = ([t], t.numel()) if t is not None else ([], 0)


def _config_int(dump, key):
    for line in dump.splitlines():
        parts = line.split("=")
        if len(parts) == 2 and parts[0].strip() == key:
            return int(parts[1].strip())
    raise KeyError(key)


class DistributedDataParallel(torch.nn.Module):
    """Wraps a module: gives every worker rank 0's parameters and buffers when it is built
    (``broadcast_parameters``), sums or averages gradients across workers during backward.

    Configure the context with ``average = true`` in [backend.cuda] to get the mean; with
    the default the gradients are summed, like a raw SwitchML allreduce. ``no_sync()``
    skips the reduction for the backward passes inside it (gradient accumulation); the
    accumulated gradients are reduced by the first backward pass outside.
    ``broadcast_parameters="auto"`` broadcasts unless the backend is the dummy one, which
    has no peers and multiplies every job by ``num_workers``.
    """

    def __init__(self, module, ctx, bucket_mb=25, overlap=True, symmetric="auto", broadcast_parameters="auto"):
        super().__init__()
        self.module = module
        self.ctx = ctx
        self.overlap = overlap
        self._sync = True
        if broadcast_parameters == "auto":
            broadcast_parameters = "backend = dummy" not in ctx.config_dump()
        if broadcast_parameters:
            self.sync_parameters()
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

    def sync_parameters(self, src=0):
        """Overwrite parameters and buffers with those of rank `src` (see broadcast_tensors)."""
        state = [p.data for p in self.module.parameters()] + [b.data for b in self.module.buffers()]
        broadcast_tensors(self.ctx, state, src)

    def no_sync(self):
        """Context manager: backward passes inside accumulate gradients locally."""
        ddp = self

        class _NoSync:
            def __enter__(self):
                self.previous = ddp._sync
                ddp._sync = False

            def __exit__(self, *exc):
                ddp._sync = self.previous
                return False

        return _NoSync()

    def forward(self, *args, **kwargs):
        if torch.is_grad_enabled() and self._sync:
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
