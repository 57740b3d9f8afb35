"""``torch.distributed`` backend ``"sml"``.

    import switchml_b200.parallel.process_group   # registers the backend
    dist.init_process_group("sml", rank=r, world_size=n)
    dist.all_reduce(t)                             # through switchml::Context
    ddp = torch.nn.parallel.DistributedDataParallel(model)   # buckets go through it too

Counterpart of the reference's ``torch_switchml`` plugin (pytorch_plugin/ProcessGroupSML.
{hpp,cpp}: backend name "sml", context started in the constructor, allreduce of exactly
one tensor with SUM) and of its Gloo patch (pytorch_patch/switchml_pytorch.patch: anything
SwitchML cannot do falls back to Gloo). Differences: CUDA tensors are reduced on the GPU
instead of being staged through pinned host memory, the work object is asynchronous and
has a future, so DDP communication hooks work.

Which library backend runs is taken from ``SWITCHML_CONFIG`` (a switchml.cfg) if set;
otherwise ``cuda`` when a GPU is visible, else ``udp`` (several workers) or ``dummy`` (one).
"""
import os
from datetime import timedelta

import torch
import torch.distributed as dist

from .context import Context, JobStatus
from ..utils.config import make_config, load_config_file

_SUPPORTED = (torch.float32, torch.int32, torch.bfloat16, torch.uint8)


class WorkSML(dist._Work):
    """Handle of one allreduce (the reference's WorkSML, ProcessGroupSML.cpp:92-197)."""

    def __init__(self, job, tensors):
        super().__init__()
        self._job = job
        self._tensors = tensors
        self._fut = None

    def wait(self, timeout=None):
        t = self._tensors[0]
        if t.is_cuda:
            self._job.stream_wait(torch.cuda.current_stream(t.device))
        else:
            st = self._job.wait()
            if st != JobStatus.FINISHED:
                raise RuntimeError("SwitchML allreduce failed: " + self._job.error())
        return True

    def is_completed(self):
        return self._job.status() in (JobStatus.FINISHED, JobStatus.FAILED)

    def is_success(self):
        return self._job.status() == JobStatus.FINISHED

    def result(self):
        return self._tensors

    def get_future(self):
        if self._fut is None:
            t = self._tensors[0]
            if t.is_cuda:
                self._fut = torch.futures.Future(devices=[t.device])
                self._job.stream_wait(torch.cuda.current_stream(t.device))
            else:
                self._fut = torch.futures.Future()
                self._job.wait()
            self._fut.set_result(self._tensors)
        return self._fut


class ProcessGroupSML(dist.ProcessGroup):
    def __init__(self, store, rank, size, timeout=timedelta(seconds=300)):
        super().__init__(rank, size)
        self._rank, self._size = rank, size
        # Everything that is not a single-tensor SUM allreduce goes to Gloo, like the
        # reference's patched ProcessGroupGloo does.
        self._fallback = dist.ProcessGroupGloo(dist.PrefixStore("sml_fallback", store), rank, size, timeout)
        self._ctx = Context.get_instance()
        self._started_here = False
        if self._ctx.state().name != "RUNNING":
            if not self._ctx.start(self._config(rank, size)):
                raise RuntimeError("cannot start the SwitchML context")
            self._started_here = True

    @staticmethod
    def _config(rank, size):
        if os.environ.get("SWITCHML_CONFIG"):
            text = load_config_file()
            import re
            text = re.sub(r"(?m)^\s*rank\s*=.*$", "rank = %d" % rank, text)
            return re.sub(r"(?m)^\s*num_workers\s*=.*$", "num_workers = %d" % size, text)
        port = int(os.environ.get("MASTER_PORT", "29500"))
        addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
        if torch.cuda.is_available():
            return make_config("cuda", rank=rank, num_workers=size, packet_numel=256, controller_ip=addr,
                               controller_port=port + 401, launch="inline",
                               mode=os.environ.get("SWITCHML_MODE", "float_sum"))
        if size > 1:
            return make_config("udp", rank=rank, num_workers=size, packet_numel=256, controller_ip=addr,
                               controller_port=port + 401, switch_port=port + 402, switch_ip=addr,
                               worker_port=0, num_worker_threads=2, max_outstanding_packets=128)
        return make_config("dummy", bandwidth=0)

    # -- the one collective SwitchML implements ----------------------------------------
    def allreduce(self, tensors, opts=None):
        op = getattr(opts, "reduceOp", dist.ReduceOp.SUM) if opts is not None else dist.ReduceOp.SUM
        t = tensors[0] if len(tensors) == 1 else None
        if (t is None or op != dist.ReduceOp.SUM or t.dtype not in _SUPPORTED or not t.is_contiguous()
                or (t.dtype == torch.bfloat16 and not t.is_cuda)):
            return self._fallback_allreduce(tensors, opts)
        job = self._ctx.all_reduce_async(t.view(-1))
        return WorkSML(job, tensors)

    def _fallback_allreduce(self, tensors, opts):
        if tensors[0].is_cuda:
            host = [x.cpu() for x in tensors]
            w = self._fallback.allreduce(host, opts) if opts is not None else self._fallback.allreduce(host)
            w.wait()
            for x, h in zip(tensors, host):
                x.copy_(h)
            fut_work = _DoneWork(tensors)
            return fut_work
        return self._fallback.allreduce(tensors, opts) if opts is not None else self._fallback.allreduce(tensors)

    def allreduce_coalesced(self, tensors, opts=None):
        works = [self.allreduce([t], None) for t in tensors]
        for w in works:
            w.wait()
        return _DoneWork(tensors)

    # -- everything else: Gloo -----------------------------------------------------------
    def _via_host(self, name, tensor_args, *rest):
        """Run a Gloo collective on host copies of CUDA tensors and copy the results back."""
        flat = []

        def to_host(x):
            if isinstance(x, torch.Tensor):
                h = x.cpu() if x.is_cuda else x
                flat.append((x, h))
                return h
            return [to_host(y) for y in x]

        host_args = [to_host(a) for a in tensor_args]
        work = getattr(self._fallback, name)(*host_args, *rest)
        work.wait()
        for dev_t, h in flat:
            if dev_t.is_cuda:
                dev_t.copy_(h)
        return _DoneWork([t for t, _ in flat])

    def broadcast(self, tensors, opts=None):
        return self._via_host("broadcast", [tensors], *( [opts] if opts is not None else []))

    def allgather(self, output_tensors, input_tensors, opts=None):
        return self._via_host("allgather", [output_tensors, input_tensors], *([opts] if opts is not None else []))

    def barrier(self, opts=None):
        return self._fallback.barrier(opts) if opts is not None else self._fallback.barrier()

    def reduce(self, tensors, opts=None):
        return self._via_host("reduce", [tensors], *([opts] if opts is not None else []))

    def gather(self, output_tensors, input_tensors, opts=None):
        return self._via_host("gather", [output_tensors, input_tensors], *([opts] if opts is not None else []))

    def scatter(self, output_tensors, input_tensors, opts=None):
        return self._via_host("scatter", [output_tensors, input_tensors], *([opts] if opts is not None else []))

    def getBackendName(self):
        return "sml"

    def size(self):
        return self._size

    def rank(self):
        return self._rank

    def shutdown(self):
        if self._started_here and self._ctx.state().name == "RUNNING":
            self._ctx.stop()
            self._started_here = False


class _DoneWork(dist._Work):
    def __init__(self, tensors):
        super().__init__()
        self._tensors = tensors

    def wait(self, timeout=None):
        return True

    def is_completed(self):
        return True

    def is_success(self):
        return True

    def result(self):
        return self._tensors

    def get_future(self):
        f = torch.futures.Future()
        f.set_result(self._tensors)
        return f


def _create(store, rank, size, timeout):
    return ProcessGroupSML(store, rank, size, timeout)


try:
    dist.Backend.register_backend("sml", _create, devices=["cpu", "cuda"])
except (RuntimeError, ValueError, AssertionError):
    pass  # already registered (module imported twice)
