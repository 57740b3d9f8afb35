"""Property tests of the aggregation arithmetic: an independent restatement in numpy of
the reference's quantiser (client_lib/src/prepostprocessors/cpu_exponent_quantizer_ppp.cc:
local exponent :150-154, scale factor :256-258, quantise :96-103, dequantise :224-241) must
agree bit for bit with the native oracle (which the GPU kernels are tested against), for
arbitrary worker counts, block sizes, lengths and values, special values included; and the
result must not depend on the order of the workers."""
import numpy as np
import pytest
from hypothesis import HealthCheck, given, settings, strategies as st

from switchml_b200.ops.oracle import int_allreduce_oracle, quant_allreduce_oracle


def numpy_quant_allreduce(inputs, block):
    n = len(inputs)
    numel = inputs[0].size
    out = np.empty(numel, dtype=np.float32)
    k = 2147483647.0 if n & (n - 1) == 0 else 2147483647.0 - 256.0
    for off in range(0, numel, block):
        blocks = [x[off:off + block] for x in inputs]
        exps = []
        for b in blocks:
            m = np.float32(np.fmax.reduce(np.abs(b), initial=np.float32(0)))   # fmax: a NaN never wins
            e = ((int(m.view(np.uint32)) & 0x7F800000) >> 23) - 126
            exps.append(min(e, 127))
        e = min(max(max(exps), -90), 127)
        sf = np.float32(np.ldexp(k / n, -e))                                    # double, rounded once to float
        acc = np.zeros(len(blocks[0]), dtype=np.int64)
        for b in blocks:
            with np.errstate(over="ignore", invalid="ignore"):
                p = b.astype(np.float32) * sf
                q = np.rint(p)                                                  # nearest-even
            q = np.where(np.isnan(p), 0.0, q)
            q = np.clip(q.astype(np.float64), -2147483648.0, 2147483647.0).astype(np.int64)
            acc += q
        total = ((acc + 2 ** 31) % 2 ** 32 - 2 ** 31).astype(np.int32)          # the adders wrap
        with np.errstate(over="ignore", divide="ignore", invalid="ignore"):
            out[off:off + block] = total.astype(np.float32) / sf
    return out


finite = st.floats(width=32, allow_nan=False, allow_infinity=False)
anything = st.floats(width=32, allow_nan=True, allow_infinity=True)


@settings(max_examples=150, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(n=st.integers(1, 9), block=st.sampled_from([32, 64, 256, 1024]), numel=st.integers(1, 700),
       seed=st.integers(0, 2 ** 31), scale_exp=st.integers(-40, 38), special=st.booleans())
def test_native_oracle_equals_numpy_restatement(n, block, numel, seed, scale_exp, special):
    rng = np.random.default_rng(seed)
    xs = [(rng.standard_normal(numel) * 2.0 ** (scale_exp + rng.integers(-3, 4))).astype(np.float32)
          for _ in range(n)]
    if special:
        for x in xs:
            idx = rng.integers(0, numel, size=max(1, numel // 8))
            x[idx] = rng.choice(np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 3.4e38, -3.4e38, 1e-45, 1.17e-38],
                                         dtype=np.float32), size=idx.size)
    got = quant_allreduce_oracle(xs, block)
    want = numpy_quant_allreduce(xs, block)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@settings(max_examples=60, deadline=None)
@given(data=st.lists(st.lists(finite, min_size=1, max_size=200), min_size=2, max_size=6), block=st.sampled_from([32, 64]))
def test_quantised_sum_is_independent_of_worker_order(data, block):
    numel = min(len(d) for d in data)
    xs = [np.array(d[:numel], dtype=np.float32) for d in data]
    a = quant_allreduce_oracle(xs, block)
    b = quant_allreduce_oracle(list(reversed(xs)), block)
    c = quant_allreduce_oracle(xs[1:] + xs[:1], block)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32)) and np.array_equal(a.view(np.uint32), c.view(np.uint32))


@settings(max_examples=60, deadline=None)
@given(n=st.integers(1, 8), numel=st.integers(1, 500), seed=st.integers(0, 2 ** 31), spread=st.integers(0, 12))
def test_error_bound_of_the_quantised_sum(n, numel, seed, spread):
    """|result - exact| <= n^2 * 2^(E-31) per block (each worker rounds by half a quantum) plus
    the final rounding to float32, with 2^E > max|x| of the block (the reference's accepted trade)."""
    rng = np.random.default_rng(seed)
    xs = [(rng.standard_normal(numel) * 2.0 ** rng.integers(-spread, spread + 1)).astype(np.float32) for _ in range(n)]
    got = quant_allreduce_oracle(xs, 64).astype(np.float64)
    exact = np.sum([x.astype(np.float64) for x in xs], axis=0)
    for off in range(0, numel, 64):
        m = max(float(np.max(np.abs(x[off:off + 64]))) for x in xs)
        if m == 0.0:
            assert np.all(got[off:off + 64] == 0.0)
            continue
        e = np.frexp(np.float32(m))[1]                     # 2^e > m >= 2^(e-1)
        bound = n * n * 2.0 ** (e - 31) * 1.01 + 2.0 ** -23 * n * m
        assert np.max(np.abs(got[off:off + 64] - exact[off:off + 64])) <= bound


@settings(max_examples=50, deadline=None)
@given(n=st.integers(1, 8), numel=st.integers(1, 300), seed=st.integers(0, 2 ** 31))
def test_integer_sum_wraps_like_the_switch_adders(n, numel, seed):
    rng = np.random.default_rng(seed)
    xs = [rng.integers(-2 ** 31, 2 ** 31, size=numel, dtype=np.int64).astype(np.int32) for _ in range(n)]
    want = ((np.sum([x.astype(np.int64) for x in xs], axis=0) + 2 ** 31) % 2 ** 32 - 2 ** 31).astype(np.int32)
    assert np.array_equal(int_allreduce_oracle(xs), want)
