"""switchml-b200: SwitchML-style in-network aggregation for one NVSwitch box of B200s.

Public surface (mirrors ``switchml::Context`` of the reference, client_lib/src/context.h):

    import switchml_b200 as sml
    ctx = sml.Context.get_instance()
    ctx.start(sml.make_config(backend="cuda", rank=r, num_workers=n))
    job = ctx.all_reduce_async(tensor)         # returns at once
    job.wait()                                 # or job.stream_wait(stream)
    ctx.wait_for_all_jobs(); ctx.get_stats(); ctx.stop()

Sub-packages: ``parallel`` (context, DDP hook, gradient bucketing, process group),
``ops`` (kernel wrappers: allreduce emulation, oracle, weight-gradient GEMM),
``models`` (ResNet-50, VGG-19, BERT-large), ``utils`` (config files, timing, clocks, CLI).
"""
from ._native import lib, library_path, NativeError  # noqa: F401
from .utils.config import make_config, load_config_file  # noqa: F401
from .parallel.context import Context, Job, DataType, JobStatus, ContextState  # noqa: F401

__version__ = lib().sml_version().decode()


def set_verbosity(level, vmodule=None):
    """Log verbosity 0..4 of the native library; `vmodule` ("udp_backend=3,control=2") gives
    single source files their own level (the reference exposes glog's --v / --vmodule)."""
    lib().sml_set_verbosity(int(level))
    if vmodule is not None:
        lib().sml_set_vmodule(str(vmodule).encode())
