"""The aggregation kernels on one GPU, all ranks emulated inside one cooperative launch
(peer-memory code path), checked against the CPU oracle (bit-exact in quantised mode)
and a float64 sum. Sizes follow the plan: 1, 63, 64, 65, 255, 2^20+1, zero blocks,
extreme exponents, denormals."""
import numpy as np
import pytest
import torch

from switchml_b200.ops.emulation import emulated_allreduce
from switchml_b200.ops.oracle import quant_allreduce_oracle, int_allreduce_oracle

pytestmark = pytest.mark.gpu

SIZES = [1, 63, 64, 65, 255, 4096, 40000, (1 << 20) + 1]


def _inputs(n, numel, dtype=torch.float32, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    xs = []
    for r in range(n):
        if dtype == torch.int32:
            x = torch.randint(-2 ** 30, 2 ** 30, (numel,), generator=g, dtype=torch.int32)
        else:
            x = (torch.rand(numel, generator=g) * 2 - 1) * (10.0 ** (r - 1))
            x = x.to(dtype)
        xs.append(x)
    return xs


@pytest.mark.parametrize("algo", ["staged", "oneshot", "push"])
@pytest.mark.parametrize("n", [1, 2, 4, 8])
@pytest.mark.parametrize("numel", SIZES)
def test_quant_bit_exact(n, numel, algo):
    if algo == "oneshot" and numel > (1 << 16):
        pytest.skip("one-shot is for small messages")
    if algo == "push" and n == 1:
        pytest.skip("pushing needs a peer")
    xs = _inputs(n, numel)
    outs = emulated_allreduce([x.cuda() for x in xs], mode="quant", algo=algo, block_numel=64,
                              slot_bytes=32768)
    want = quant_allreduce_oracle([x.numpy() for x in xs], 64)
    for o in outs:
        assert np.array_equal(o.cpu().numpy(), want)
    exact = sum(x.double() for x in xs).numpy()
    scale = max(float(x.abs().max()) for x in xs)
    # n rounded addends of half a quantum each, plus the final rounding to float32
    assert np.max(np.abs(want - exact)) <= n * n * 2.0 ** -30 * scale + 2.0 ** -23 * n * scale


@pytest.mark.parametrize("algo", ["staged", "push"])
@pytest.mark.parametrize("block", [32, 256, 1024])
def test_quant_block_sizes_and_reuse(block, algo):
    # Several jobs back to back over the same staging (epochs and slot reuse).
    xs = _inputs(4, 300001, seed=3)
    outs = emulated_allreduce([x.cuda() for x in xs], mode="quant", algo=algo, block_numel=block,
                              slot_bytes=16 * 4 * block, repeats=3, channels=3)
    want = quant_allreduce_oracle([x.numpy() for x in xs], block)
    for o in outs:
        assert np.array_equal(o.cpu().numpy(), want)


@pytest.mark.parametrize("algo", ["staged", "push"])
@pytest.mark.parametrize("slots", [2, 4])
@pytest.mark.parametrize("lookahead", [0, 1, 2, 3, 4])
def test_quant_exponent_lookahead(lookahead, slots, algo):
    """The exponents of a tile travel `lookahead` tiles ahead of its data through a ring of
    exponent slots of its own (8 deep, whatever the number of data slots): every setting gives
    the oracle's bits, over many tiles per channel and several jobs on the same staging."""
    xs = _inputs(3, 200003, seed=11 + lookahead)
    outs = emulated_allreduce([x.cuda() for x in xs], mode="quant", algo=algo, block_numel=64,
                              slot_bytes=3 * 4 * 128 * 4, slots_per_channel=slots, channels=2,
                              repeats=2, exponent_lookahead=lookahead)
    want = quant_allreduce_oracle([x.numpy() for x in xs], 64)
    for o in outs:
        assert np.array_equal(o.cpu().numpy(), want)


@pytest.mark.parametrize("algo", ["staged", "oneshot", "push"])
@pytest.mark.parametrize("n", [2, 8])
def test_int32_wrapping_sum(n, algo):
    numel = 50001 if algo == "oneshot" else 777777
    xs = _inputs(n, numel, torch.int32)
    outs = emulated_allreduce([x.cuda() for x in xs], mode="sum", algo=algo)
    want = int_allreduce_oracle([x.numpy() for x in xs])
    for o in outs:
        assert np.array_equal(o.cpu().numpy(), want)


@pytest.mark.parametrize("algo", ["staged", "oneshot", "push"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_float_sum(dtype, algo):
    n, numel = 4, 65537 if algo == "oneshot" else 999999
    xs = _inputs(n, numel, dtype)
    outs = emulated_allreduce([x.cuda() for x in xs], mode="sum", algo=algo, post_scale=0.25)
    exact = sum(x.double() for x in xs) * 0.25
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    for o in outs:
        assert torch.allclose(o.cpu().double(), exact, rtol=tol, atol=tol * 10)
    for o in outs[1:]:
        assert torch.equal(o, outs[0]), "all ranks must hold identical bits"


@pytest.mark.parametrize("algo", ["staged", "push"])
def test_quant_bf16_matches_oracle_after_rounding(algo):
    n, numel = 4, 100000
    xs = _inputs(n, numel, torch.bfloat16)
    outs = emulated_allreduce([x.cuda() for x in xs], mode="quant", algo=algo, block_numel=256)
    want = quant_allreduce_oracle([x.float().numpy() for x in xs], 256)
    want_bf16 = torch.from_numpy(want).to(torch.bfloat16)
    for o in outs:
        assert torch.equal(o.cpu(), want_bf16)


def test_special_blocks():
    numel = 64 * 8
    a = torch.zeros(numel)
    a[64:128] = 1e-30
    a[128:192] = 3e37
    a[192:256] = 1e-45       # denormal
    a[256] = -1.5
    a[320:384] = 2.0 ** -100
    b = a.clone()
    b[384:448] = 7.0         # only one rank is non-zero here
    want = quant_allreduce_oracle([a.numpy(), b.numpy()], 64)
    for algo in ("staged", "push"):
        outs = emulated_allreduce([a.cuda(), b.cuda()], mode="quant", algo=algo, block_numel=64, slot_bytes=8192)
        got = outs[0].cpu().numpy()
        assert np.all(np.isfinite(got)) and np.array_equal(got, want), algo
        assert np.all(got[:64] == 0) and got[256] == -3.0 and np.all(got[384:448] == 7.0), algo


def test_unaligned_views_and_out_of_place():
    n, numel = 2, 10007
    bases = [torch.randn(numel + 3).cuda() for _ in range(n)]
    xs = [b[1:1 + numel] for b in bases]            # 4-byte aligned only
    keep = [x.clone() for x in xs]
    for algo in ("staged", "push"):
        outs = emulated_allreduce(xs, mode="sum", algo=algo)
        for x, k in zip(xs, keep):
            assert torch.equal(x, k), "inputs must stay untouched"
        assert torch.allclose(outs[0], keep[0] + keep[1]) and torch.equal(outs[0], outs[1]), algo
    # in place, unaligned, quantised: the owner reads and overwrites its own shard
    want = quant_allreduce_oracle([k.cpu().numpy() for k in keep], 64)
    for algo in ("staged", "push"):
        ys = [b[1:1 + numel] for b in [k2.clone() for k2 in bases]]
        outs = emulated_allreduce(ys, mode="quant", algo=algo, block_numel=64, slot_bytes=8192, outputs=ys)
        assert np.array_equal(outs[0].cpu().numpy(), want) and np.array_equal(outs[1].cpu().numpy(), want), algo


def _random_quant_cases(worker_counts, cases, seed):
    rng = np.random.default_rng(seed)
    for case in range(cases):
        n = int(rng.choice(worker_counts))
        block = int(rng.choice([32, 64, 256, 1024]))
        algo = ("staged", "push", "staged", "oneshot", "push")[case % 5]
        numel = int(rng.integers(1, 40000 if algo == "oneshot" else 400000))
        slot_bytes = int(rng.choice([8, 16, 64])) * 4 * block
        slots = int(rng.choice([1, 2, 3, 4, 5]))
        channels = int(rng.choice([0, 1, 3, 7]))
        xs = []
        for r in range(n):
            x = rng.standard_normal(numel).astype(np.float32) * np.float32(2.0 ** int(rng.integers(-30, 30)))
            for z in rng.integers(0, max(1, numel // block), size=2) * block:   # some all-zero blocks
                x[z:z + block] = 0.0
            xs.append(x)
        outs = emulated_allreduce([torch.from_numpy(x).cuda() for x in xs], mode="quant", algo=algo,
                                  block_numel=block, slot_bytes=slot_bytes, slots_per_channel=slots,
                                  channels=channels)
        want = quant_allreduce_oracle(xs, block)
        for r, o in enumerate(outs):
            assert np.array_equal(o.cpu().numpy().view(np.uint32), want.view(np.uint32)), \
                "case %d: n=%d numel=%d block=%d algo=%s slot=%d x%d channels=%d rank %d" % (
                    case, n, numel, block, algo, slot_bytes, slots, channels, r)


def test_quant_random_shapes_against_oracle():
    """Randomly drawn lengths, block sizes, slot sizes, channel counts and value scales (fixed
    seed) for 2, 4 and 8 workers: every rank must hold the oracle's bits."""
    _random_quant_cases([2, 4, 8], 18, 20240607)


def test_quant_worker_counts_that_are_not_powers_of_two():
    """3, 5, 6 and 7 workers: the scale factor is not a power of two any more (K = 2^31-1-256
    keeps the sum inside int32) and shards do not divide tiles evenly."""
    _random_quant_cases([3, 5, 6, 7], 12, 977)
