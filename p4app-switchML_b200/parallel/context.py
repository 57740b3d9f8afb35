"""Python face of ``switchml::Context`` (reference client_lib/src/context.h:76-155):
a process singleton with start/stop, asynchronous and blocking allreduce on numpy arrays,
torch CPU tensors or torch CUDA tensors, job handles, and the statistics report."""
import ctypes
import enum
import json

from .._native import lib, last_error, read_string, NativeError


class DataType(enum.IntEnum):
    FLOAT32 = 0
    INT32 = 1
    BFLOAT16 = 2
    UINT8 = 3


class JobStatus(enum.IntEnum):
    INIT = 0
    QUEUED = 1
    RUNNING = 2
    FINISHED = 3
    FAILED = 4


class ContextState(enum.IntEnum):
    CREATED = 0
    STARTING = 1
    RUNNING = 2
    STOPPING = 3
    STOPPED = 4


def _describe(t):
    """(pointer, numel, dtype code, cuda stream or None) of a tensor-like object."""
    try:
        import torch
    except ImportError:  # numpy-only environments
        torch = None
    if torch is not None and isinstance(t, torch.Tensor):
        if not t.is_contiguous():
            raise ValueError("tensor must be contiguous")
        code = {torch.float32: 0, torch.int32: 1, torch.bfloat16: 2, torch.uint8: 3}.get(t.dtype)
        if code is None:
            raise TypeError("unsupported dtype %s (float32, int32, bfloat16, uint8)" % t.dtype)
        stream = None
        if t.is_cuda:
            stream = torch.cuda.current_stream(t.device).cuda_stream
        return t.data_ptr(), t.numel(), code, stream, t.is_cuda
    import numpy as np
    if isinstance(t, np.ndarray):
        if not t.flags["C_CONTIGUOUS"]:
            raise ValueError("array must be C-contiguous")
        code = {np.dtype("float32"): 0, np.dtype("int32"): 1, np.dtype("uint8"): 3}.get(t.dtype)
        if code is None:
            raise TypeError("unsupported dtype %s (float32, int32, uint8)" % t.dtype)
        return t.ctypes.data, t.size, code, None, False
    raise TypeError("expected a torch.Tensor or numpy.ndarray")


class Job:
    """Handle of a submitted allreduce (``switchml::Job``)."""

    def __init__(self, handle, keepalive):
        self._h = handle
        self._keep = keepalive  # the tensors must outlive the job

    def wait(self, timeout_ms=None):
        """Block until FINISHED or FAILED (``Job::WaitToComplete``); returns the status."""
        st = lib().sml_job_wait(self._h, -1.0 if timeout_ms is None else float(timeout_ms))
        return JobStatus(st)

    def status(self):
        return JobStatus(lib().sml_job_status(self._h))

    def stream_wait(self, stream=None):
        """Order a CUDA stream after the job without waiting on the host (cuda backend)."""
        if stream is None:
            import torch
            stream = torch.cuda.current_stream()
        ptr = getattr(stream, "cuda_stream", stream)
        if lib().sml_job_stream_wait(self._h, ctypes.c_void_p(ptr)) != 0:
            raise NativeError(last_error())

    def error(self):
        return read_string(lib().sml_job_error, self._h)

    def __repr__(self):
        if not self._h:
            return "<switchml Job released>"
        return "<switchml Job handle=%d %s>" % (self._h, self.status().name)

    def release(self):
        if self._h:
            lib().sml_job_release(self._h)
            self._h = 0
            self._keep = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class Context:
    """The library's singleton (``Context.get_instance()``)."""

    _instance = None

    @classmethod
    def get_instance(cls):
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    # -- lifecycle -------------------------------------------------------------------
    def start(self, config_text=None, apply_env=False):
        """Start with INI text (see ``make_config``) or, with None, from the default
        configuration files. Returns True on success like the C++ API."""
        text = (config_text or "").encode()
        return lib().sml_start(text, 1 if apply_env else 0) == 0

    def start_from_file(self, path=None):
        return lib().sml_start_file(path.encode() if path else None) == 0

    def stop(self):
        if lib().sml_stop() != 0:
            raise NativeError(last_error())

    def state(self):
        return ContextState(lib().sml_state())

    def running(self, config_text=None, apply_env=False):
        """``with ctx.running(config):`` starts the context and stops it when the block ends,
        also when the block raises."""
        ctx = self

        class _Running:
            def __enter__(self):
                if not ctx.start(config_text, apply_env):
                    raise NativeError("the context did not start: " + last_error())
                return ctx

            def __exit__(self, *exc):
                if ctx.state() == ContextState.RUNNING:
                    ctx.stop()
                return False

        return _Running()

    def config_dump(self):
        return read_string(lib().sml_config_dump)

    # -- jobs ------------------------------------------------------------------------
    def all_reduce_async(self, tensor, out=None, stream=None):
        """Submit a SUM allreduce of `tensor` (result in `out`, default in place)."""
        ptr, numel, code, cur_stream, is_cuda = _describe(tensor)
        optr = ptr
        if out is not None:
            optr, onumel, ocode, _, _ = _describe(out)
            if onumel != numel or ocode != code:
                raise ValueError("out must match the input's size and dtype")
        if stream is not None:
            cur_stream = getattr(stream, "cuda_stream", stream)
        h = lib().sml_allreduce_async(ctypes.c_void_p(ptr), ctypes.c_void_p(optr), numel, code,
                                      ctypes.c_void_p(cur_stream or 0))
        if h < 0:
            raise NativeError(last_error())
        return Job(h, (tensor, out))

    def all_reduce(self, tensor, out=None):
        job = self.all_reduce_async(tensor, out)
        st = job.wait()
        if st != JobStatus.FINISHED:
            raise NativeError("allreduce failed: " + job.error())
        return job

    def broadcast_async(self, tensor, root=0, stream=None):
        """Every worker's `tensor` receives rank `root`'s values, in place
        (``Context::BroadcastAsync``: a sum to which the other workers contribute zeros)."""
        ptr, numel, code, cur_stream, _ = _describe(tensor)
        if stream is not None:
            cur_stream = getattr(stream, "cuda_stream", stream)
        h = lib().sml_broadcast_async(ctypes.c_void_p(ptr), numel, code, int(root), ctypes.c_void_p(cur_stream or 0))
        if h < 0:
            raise NativeError(last_error())
        return Job(h, (tensor,))

    def broadcast(self, tensor, root=0):
        job = self.broadcast_async(tensor, root)
        st = job.wait()
        if st != JobStatus.FINISHED:
            raise NativeError("broadcast failed: " + job.error())
        return job

    def wait_for_all_jobs(self):
        lib().sml_wait_all()

    # -- introspection ---------------------------------------------------------------
    def get_stats(self):
        return json.loads(read_string(lib().sml_stats_json))

    def stats_report(self):
        return read_string(lib().sml_stats_report)

    def reset_stats(self):
        lib().sml_stats_reset()

    def uses_multimem(self):
        return bool(lib().sml_uses_multimem())

    def device(self):
        return lib().sml_device()

    def wait_probe(self, budget_ms=50.0):
        """Launch a kernel that waits for a signal nobody sends; returns its status word
        (1 = the wait timed out cleanly)."""
        return lib().sml_wait_probe(float(budget_ms))

    # -- symmetric memory --------------------------------------------------------------
    def symmetric_empty(self, numel, dtype, device=None):
        """A 1-D torch tensor inside the symmetric heap ([backend.cuda] symm_heap_mb).
        Every rank must allocate the same sequence of sizes. Tensors from here are reduced
        in place through NVLink without staging copies. They live until
        ``symmetric_reset`` or ``stop``."""
        import torch
        esz = torch.empty((), dtype=dtype).element_size()
        nbytes = numel * esz
        ptr = lib().sml_symm_alloc(nbytes)
        if not ptr:
            raise MemoryError("symmetric heap exhausted or not configured (symm_heap_mb)")
        dev = torch.device("cuda", self.device() if device is None else device)
        return _tensor_from_ptr(ptr, numel, dtype, dev)

    def symmetric_info(self):
        """(local base, [peer bases], multicast base or None, bytes) of the symmetric heap."""
        local = ctypes.c_void_p()
        peers = (ctypes.c_void_p * 8)()
        mc = ctypes.c_void_p()
        nbytes = ctypes.c_size_t()
        if lib().sml_symm_info(ctypes.byref(local), peers, ctypes.byref(mc), ctypes.byref(nbytes)) != 0:
            raise NativeError(last_error())
        return local.value, [p for p in peers], mc.value, nbytes.value

    def symmetric_reset(self):
        lib().sml_symm_reset()


def _tensor_from_ptr(ptr, numel, dtype, device):
    """Wrap raw device memory as a torch tensor through the CUDA array interface."""
    import torch
    typestr = {torch.float32: "<f4", torch.int32: "<i4", torch.bfloat16: "<u2",
               torch.uint8: "|u1", torch.float16: "<f2"}[dtype]

    class _Holder:
        pass

    h = _Holder()
    h.__cuda_array_interface__ = {"shape": (numel,), "typestr": typestr, "data": (int(ptr), False),
                                  "version": 3, "strides": None}
    t = torch.as_tensor(h, device=device)
    if dtype == torch.bfloat16:
        t = t.view(torch.bfloat16)
    return t
