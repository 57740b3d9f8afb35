"""The allocation-free entry point (csrc/kernels/local_noalloc.h).

Some callers of this library cannot allocate device memory: a serving process whose own
pool owns all of HBM, a latency-critical loop that must not trigger the device-wide
synchronisation an allocation can imply, a callback running under somebody else's
allocator locks. For them ``switchml_local_allreduce_noalloc`` runs the single-worker
aggregation round trip with its staging in a static device array instead of cudaMalloc'ed
memory. This test calls it through its exported C symbol, twice in a row (the second call
finds the first call's leftovers in the shared scratch), and checks each result against
the ordinary entry point (``sml_emu_allreduce`` with one rank), which allocates its staging,
and against the CPU oracle, which shares no device code with either. After every call the
kernel's status word is read back through ``switchml_noalloc_last_status`` and must be 0.
The file sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import ctypes

import pytest
import torch

from switchml_b200._native import lib
from switchml_b200.ops.emulation import emulated_allreduce
from switchml_b200.ops.oracle import quant_allreduce_oracle

pytestmark = pytest.mark.gpu


def _entry():
    fn = lib().switchml_local_allreduce_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_ulonglong, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_void_p]
    err = lib().switchml_noalloc_strerror
    err.restype = ctypes.c_char_p
    err.argtypes = [ctypes.c_int]
    return fn, err


def _status():
    """The status word the kernel of the last call left behind (0 = completed normally)."""
    fn = lib().switchml_noalloc_last_status
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int)]
    word = ctypes.c_int(-1)
    rc = fn(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), ctypes.byref(word))
    assert rc == 0, rc
    return word.value


def _call(fn, x, out, mode, block):
    elem = {torch.float32: 0, torch.int32: 1, torch.bfloat16: 2}[x.dtype]
    stream = torch.cuda.current_stream().cuda_stream
    return fn(x.data_ptr(), out.data_ptr(), x.numel(), elem, mode, block, ctypes.c_void_p(stream))


def test_two_calls_in_a_row_match_the_allocating_entry_point():
    fn, err = _entry()
    torch.manual_seed(7)
    cases = [
        (torch.randn(1_000_003, device="cuda") * 3.0, 1, 256),                    # quantised float32
        (torch.randn(70_001, device="cuda") * 1e-3, 1, 64),                       # smaller, other block
        (torch.randn(300_000, device="cuda").bfloat16(), 1, 256),                 # quantised bfloat16
        (torch.randint(-2 ** 30, 2 ** 30, (123_457,), device="cuda", dtype=torch.int32), 0, 256),
        (torch.randn(555_555, device="cuda"), 0, 128),                            # plain sum = copy
    ]
    for x, mode, block in cases:
        want = emulated_allreduce([x], mode="quant" if mode == 1 else "sum", algo="staged",
                                  block_numel=block, slot_bytes=32768)[0]
        # two calls back to back on the same stream; the second reuses the dirty scratch
        first = torch.empty_like(x)
        second = torch.empty_like(x)
        rc1 = _call(fn, x, first, mode, block)
        rc2 = _call(fn, x, second, mode, block)
        assert rc1 == 0 and rc2 == 0, (err(rc1), err(rc2))
        assert _status() == 0, "the kernel reported a status"
        torch.cuda.synchronize()
        assert torch.equal(first, want), "first call differs from the allocating entry point"
        assert torch.equal(second, want), "second call differs from the allocating entry point"
        if mode == 1:  # the CPU oracle: one worker's quantise / dequantise round trip
            cpu = quant_allreduce_oracle([x.float().cpu().numpy()], block)
            cpu = torch.from_numpy(cpu).to(x.dtype)
            assert torch.equal(second.cpu(), cpu), "differs from the CPU oracle"
        else:
            assert torch.equal(second, x)
    # in place
    x = torch.randn(40_000, device="cuda")
    want = emulated_allreduce([x.clone()], mode="quant", block_numel=256, slot_bytes=32768)[0]
    assert _call(fn, x, x, 1, 256) == 0
    assert _status() == 0
    torch.cuda.synchronize()
    assert torch.equal(x, want)


def test_limits_are_refused_with_a_clear_error():
    fn, err = _entry()
    x = torch.zeros(16, device="cuda")
    too_many = (1 << 26) + 1
    rc = fn(x.data_ptr(), x.data_ptr(), too_many, 0, 1, 256, None)
    assert rc == -2 and b"SWITCHML_NOALLOC_MAX_NUMEL" in err(rc)
    assert fn(None, x.data_ptr(), 16, 0, 1, 256, None) == -1
    assert fn(x.data_ptr(), x.data_ptr(), 16, 0, 1, 100, None) == -1      # block not a power of two
    assert fn(x.data_ptr(), x.data_ptr(), 16, 1, 1, 256, None) == -1      # int32 cannot be quantised
    assert fn(x.data_ptr(), x.data_ptr(), 16, 7, 0, 256, None) == -1
    assert b"bad argument" in err(-1)
    assert fn(x.data_ptr(), x.data_ptr(), 0, 0, 1, 256, None) == 0        # nothing to do
    torch.cuda.synchronize()
    assert float(x.abs().max()) == 0.0
