"""Loads the native c10d backend (``lib/torch_switchml.so``, csrc/torch/process_group_sml.cc)
and registers it as ``"sml_native"``. It implements allreduce only, like the reference's
plugin; the Python backend ``"sml"`` (process_group.py) additionally falls back to Gloo for
the other collectives, which DistributedDataParallel needs at construction time."""
import importlib.util
import os

import torch.distributed as dist

from .._native import lib, library_path

_MODULE = None


def load():
    global _MODULE
    if _MODULE is None:
        lib()  # the extension links against libswitchml_b200.so: load it first
        path = library_path("torch_switchml.so")
        if not os.path.exists(path):
            raise ImportError("torch_switchml.so is not built (python build.py --torch)")
        spec = importlib.util.spec_from_file_location("torch_switchml", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _MODULE = mod
        try:
            dist.Backend.register_backend("sml_native", mod.create_backend, devices=["cpu", "cuda"])
        except (RuntimeError, ValueError, AssertionError):
            pass
    return _MODULE


load()
