"""The uint8 <-> int32 conversions of the aggregation path as stand-alone ops.

SwitchML sums 32-bit integers. The reference's NCCL plugin accepts uint8 tensors (PyTorch
reduces uint8 flags across workers) by widening them to int32 on the CPU and narrowing the
result (frameworks_integration/nccl_plugin/switchml_plugin.cc:328-337,371-377); the cuda
backend does the same with two kernels (csrc/kernels/allreduce_kernels.cu, ``WidenU8Kernel``
and ``NarrowI32Kernel``) around an int32 allreduce. These wrappers run the kernels on their
own, on the current stream.
"""
from .._native import lib, last_error, NativeError


def _convert(widen, src, dst):
    import torch
    assert src.is_cuda and dst.is_cuda and src.is_contiguous() and dst.is_contiguous()
    assert src.numel() == dst.numel()
    stream = torch.cuda.current_stream(src.device).cuda_stream
    with torch.cuda.device(src.device):
        rc = lib().sml_convert_u8(int(widen), src.data_ptr(), dst.data_ptr(), src.numel(), stream)
    if rc != 0:
        raise NativeError("uint8 conversion failed (%d): %s" % (rc, last_error()))
    return dst


def widen_u8(src, out=None):
    """int32 tensor with the values of the uint8 CUDA tensor `src` (zero extended)."""
    import torch
    assert src.dtype == torch.uint8
    if out is None:
        out = torch.empty(src.shape, dtype=torch.int32, device=src.device)
    assert out.dtype == torch.int32
    return _convert(True, src, out)


def narrow_i32(src, out=None):
    """uint8 tensor holding the low byte of every element of the int32 CUDA tensor `src`."""
    import torch
    assert src.dtype == torch.int32
    if out is None:
        out = torch.empty(src.shape, dtype=torch.uint8, device=src.device)
    assert out.dtype == torch.uint8
    return _convert(False, src, out)
