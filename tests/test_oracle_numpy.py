"""The block fixed-point arithmetic restated in numpy, independently of the library.

Every "bit-exact" test of the kernels compares with the library's CPU oracle, and that
oracle shares ``include/switchml/quant_math.h`` with the device code: a wrong formula
there would pass all of them. This file pins the formulas with a second implementation
that includes nothing of the library. Per block of B elements shared by n workers
(reference: client_lib/src/prepostprocessors/cpu_exponent_quantizer_ppp.cc:88-156,200-260):

    e_w  = biased_exponent(max |x_w|) - 126, at most 127            (per worker)
    E    = clamp(max_w e_w, -90, 127)
    sf   = float32( K / n * 2^-E ),  K = 2^31-1 (n a power of two) or 2^31-1-256
    q_w  = saturate_int32(round_half_even(float32(x_w * sf))), NaN -> 0
    Q    = wrapping int32 sum of q_w
    y    = float32(Q) / sf                                          (float32 division)
"""
import numpy as np
import pytest

from switchml_b200.ops.oracle import quant_allreduce_oracle


def numpy_quant_allreduce(inputs, block):
    n = len(inputs)
    numel = inputs[0].size
    k = 2147483647.0 if (n & (n - 1)) == 0 else 2147483647.0 - 256.0
    out = np.empty(numel, dtype=np.float32)
    old = np.seterr(all="ignore")
    try:
        for lo in range(0, numel, block):
            hi = min(lo + block, numel)
            e_global = -126
            for x in inputs:
                m = np.float32(0.0)
                for v in np.abs(x[lo:hi]):
                    if v > m:  # NaN never wins
                        m = v
                bits = int(np.array([m], dtype=np.float32).view(np.uint32)[0])
                e = ((bits & 0x7F800000) >> 23) - 126
                e_global = max(e_global, min(e, 127))
            e_global = min(max(e_global, -90), 127)
            sf = np.float32(np.ldexp(k / n, -e_global))       # exact in double, one rounding to float32
            total = np.zeros(hi - lo, dtype=np.int64)
            for x in inputs:
                p = x[lo:hi].astype(np.float32) * sf          # float32 product
                q = np.rint(p.astype(np.float64))             # half to even; exact on float32 values
                q = np.where(np.isnan(p), 0.0, q)
                q = np.clip(q, -2147483648.0, 2147483647.0)
                total += q.astype(np.int64)
            wrapped = ((total + 2 ** 31) % 2 ** 32 - 2 ** 31).astype(np.int32)
            out[lo:hi] = wrapped.astype(np.float32) / sf
    finally:
        np.seterr(**old)
    return out


def _case(rng, n, numel, block):
    xs = []
    for r in range(n):
        x = rng.standard_normal(numel).astype(np.float32) * np.float32(2.0 ** int(rng.integers(-40, 40)))
        for z in rng.integers(0, max(1, numel // block), size=2) * block:
            x[z:z + block] = 0.0
        xs.append(x)
    return xs


@pytest.mark.parametrize("n", [1, 2, 3, 4, 5, 7, 8])
@pytest.mark.parametrize("block", [32, 64, 256])
def test_cpp_oracle_matches_numpy_restatement(n, block):
    rng = np.random.default_rng(1000 * n + block)
    for numel in (1, block - 1, block, block + 1, 5 * block + 17):
        xs = _case(rng, n, numel, block)
        got = quant_allreduce_oracle(xs, block)
        want = numpy_quant_allreduce(xs, block)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (n, block, numel)


def test_special_values():
    block = 64
    a = np.zeros(block * 10, dtype=np.float32)
    a[64:128] = 1e-30
    a[128:192] = 3e37                      # near the top of the float32 range
    a[192:256] = 1e-45                     # denormal
    a[256] = -1.5
    a[320:384] = 2.0 ** -100               # below the exponent clamp
    a[384] = np.inf
    a[448] = np.nan
    a[449] = 0.75
    a[512:576] = np.float32(3.4e38)
    b = a.copy()
    b[576:640] = 7.0
    b[513] = np.float32(-3.4e38)
    for xs in ([a], [a, b], [a, b, a]):
        got = quant_allreduce_oracle(xs, block)
        want = numpy_quant_allreduce(xs, block)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), len(xs)
    two = quant_allreduce_oracle([a, b], block)
    assert np.all(two[:64] == 0) and two[256] == -3.0 and np.all(two[576:640] == 7.0)


def test_sum_is_independent_of_worker_order():
    rng = np.random.default_rng(5)
    xs = _case(rng, 5, 3000, 256)
    first = numpy_quant_allreduce(xs, 256)
    second = numpy_quant_allreduce(xs[::-1], 256)
    assert np.array_equal(first.view(np.uint32), second.view(np.uint32))
    assert np.array_equal(quant_allreduce_oracle(xs[::-1], 256).view(np.uint32), first.view(np.uint32))
