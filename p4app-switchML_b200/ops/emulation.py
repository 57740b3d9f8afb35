"""Run the multi-rank aggregation kernels on ONE GPU.

Kernels of different ranks wait for each other, so they cannot be tested as separate
launches on a single device. Instead one cooperative launch plays all ranks: its
``blockIdx.y`` is the rank, every rank's staging memory lives on the same device and the
peer-memory code path runs unchanged (csrc/kernels/allreduce_kernels.cu,
``AllReduceEmuKernel``). Used by the GPU tests and for kernel profiling on one device.
"""
import ctypes

from .._native import lib, last_error, NativeError

ELEM = {"float32": 0, "int32": 1, "bfloat16": 2}
MODE = {"sum": 0, "quant": 1}
ALGO = {"staged": 0, "oneshot": 1, "push": 3}


def emulated_allreduce(inputs, mode="quant", algo="staged", block_numel=256, slot_bytes=131072,
                       slots_per_channel=2, channels=0, post_scale=1.0, repeats=1, outputs=None,
                       exponent_lookahead=-1):
    """Allreduce `inputs` (a list of equally sized 1-D CUDA tensors, one per virtual rank,
    all on the current device). Returns the list of per-rank outputs. `exponent_lookahead`:
    tiles by which the exact mode's exponents run ahead of their data (-1: the library's default)."""
    import torch
    n = len(inputs)
    x0 = inputs[0]
    elem = {torch.float32: 0, torch.int32: 1, torch.bfloat16: 2}[x0.dtype]
    for x in inputs:
        assert x.is_cuda and x.is_contiguous() and x.dtype == x0.dtype and x.numel() == x0.numel()
    if outputs is None:
        outputs = [torch.empty_like(x) for x in inputs]
    esz_unit = n * max(block_numel, 128) * 4
    slot_bytes = max(esz_unit, slot_bytes // esz_unit * esz_unit)
    if algo == "push":  # a slot holds n-1 receive areas and n-1 result areas of one shard each
        slot_bytes = max(slot_bytes, 2 * esz_unit)
    ins = (ctypes.c_void_p * n)(*[x.data_ptr() for x in inputs])
    outs = (ctypes.c_void_p * n)(*[o.data_ptr() for o in outputs])
    torch.cuda.synchronize()
    rc = lib().sml_emu_allreduce(n, ins, outs, x0.numel(), elem, MODE[mode], ALGO[algo], block_numel,
                                 slot_bytes, slots_per_channel, channels, float(post_scale), repeats,
                                 int(exponent_lookahead))
    if rc != 0:
        raise NativeError("emulated allreduce failed (%d): %s" % (rc, last_error()))
    return outputs
