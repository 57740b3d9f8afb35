"""Weight-gradient GEMM on the tcgen05 tensor cores (csrc/kernels/wgrad_gemm.cu).

    dW = wgrad_gemm(dY, X)          # dY [tokens, out], X [tokens, in], bf16 -> dW [out, in] fp32

``FusedWgrad`` additionally sums dW over all workers inside the same kernel: the output
lives in the symmetric heap, every finished tile is reduced through the NVSwitch while
later tiles are still being computed.
"""
import ctypes
import os

import torch

from .._native import library_path, NativeError

_LIB = None


class _FusedArgs(ctypes.Structure):
    _fields_ = [("rank", ctypes.c_int), ("nranks", ctypes.c_int),
                ("flags_peer", ctypes.c_void_p * 8), ("out_mc", ctypes.c_void_p),
                ("epoch", ctypes.c_ulonglong), ("timeout_ns", ctypes.c_ulonglong),
                ("scale", ctypes.c_float)]


def _lib():
    global _LIB
    if _LIB is None:
        path = library_path("libswitchml_gemm.so")
        if not os.path.exists(path):
            raise ImportError("libswitchml_gemm.so is not built (run build.py)")
        l = ctypes.CDLL(path)
        l.switchml_wgrad_gemm.restype = ctypes.c_int
        l.switchml_wgrad_gemm.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                          ctypes.c_int, ctypes.c_int, ctypes.POINTER(_FusedArgs),
                                          ctypes.c_void_p, ctypes.c_void_p]
        l.switchml_wgrad_flag_words.restype = ctypes.c_int
        l.switchml_wgrad_flag_words.argtypes = [ctypes.c_int, ctypes.c_int]
        _LIB = l
    return _LIB


_ERRORS = {-1: "bad argument", -2: "M and N must be multiples of 8 and all tensors 16-byte aligned",
           -3: "cannot build the TMA tensor maps", -4: "kernel launch failed"}


def wgrad_gemm(dy, x, out=None, error_flag=None):
    """dW[out_features, in_features] (fp32) = dY^T @ X for bf16 dY [K, M] and X [K, N]."""
    assert dy.is_cuda and x.is_cuda and dy.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
    assert dy.dim() == 2 and x.dim() == 2 and dy.shape[0] == x.shape[0]
    dy = dy.contiguous()
    x = x.contiguous()
    K, M = dy.shape
    N = x.shape[1]
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32, device=dy.device)
    assert out.is_contiguous() and out.dtype == torch.float32 and out.numel() == M * N
    stream = torch.cuda.current_stream(dy.device).cuda_stream
    rc = _lib().switchml_wgrad_gemm(dy.data_ptr(), x.data_ptr(), out.data_ptr(), M, N, K, None,
                                    error_flag.data_ptr() if error_flag is not None else None,
                                    ctypes.c_void_p(stream))
    if rc != 0:
        raise NativeError("wgrad_gemm: " + _ERRORS.get(rc, str(rc)))
    return out.view(M, N)


def flag_words(M, N):
    return _lib().switchml_wgrad_flag_words(M, N)
