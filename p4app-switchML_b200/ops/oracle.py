"""CPU reference results for the aggregation arithmetic (native code, see
csrc/ppp/cpu_exponent_quantizer_ppp.cc): what every backend must reproduce bit for bit in
integer-quantised mode."""
import ctypes

import numpy as np

from .._native import lib


def _ptr_array(arrays):
    arr = (ctypes.c_void_p * len(arrays))()
    for i, a in enumerate(arrays):
        arr[i] = a.ctypes.data
    return arr


def quant_allreduce_oracle(inputs, block_numel):
    """Block-exponent quantised SUM of a list of float32 arrays of equal length."""
    inputs = [np.ascontiguousarray(x, dtype=np.float32) for x in inputs]
    out = np.empty_like(inputs[0])
    lib().sml_oracle_quant_allreduce(_ptr_array(inputs), len(inputs), inputs[0].size, block_numel,
                                     ctypes.c_void_p(out.ctypes.data))
    return out


def int_allreduce_oracle(inputs):
    """Wrapping int32 SUM."""
    inputs = [np.ascontiguousarray(x, dtype=np.int32) for x in inputs]
    out = np.empty_like(inputs[0])
    lib().sml_oracle_int_allreduce(_ptr_array(inputs), len(inputs), inputs[0].size,
                                   ctypes.c_void_p(out.ctypes.data))
    return out
