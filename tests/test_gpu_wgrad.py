"""The tcgen05 weight-gradient GEMM against a float32 PyTorch reference of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(dy, x):
    return dy.float().t() @ x.float()


@pytest.mark.parametrize("K,M,N", [
    (64, 128, 256),        # exactly one tile, one k-block
    (16, 128, 256),        # K shorter than a stage: zero fill
    (32, 4096, 2048),      # VGG fc-like: tiny K, output bound
    (100, 136, 264),       # ragged in every dimension (M, N multiples of 8)
    (1000, 384, 1000),
    (4096, 1024, 512),     # long K: many pipeline wraps, both accumulators
    (257, 8, 8),
])
@pytest.mark.parametrize("two_cta", [False, True])
def test_matches_fp32_reference(K, M, N, two_cta):
    from switchml_b200.ops.wgrad import wgrad_gemm
    torch.manual_seed(K + M + N)
    dy = torch.randn(K, M, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = wgrad_gemm(dy, x, error_flag=err, two_cta=two_cta)
    torch.cuda.synchronize()
    assert int(err.item()) == 0, "a bounded wait inside the kernel gave up"
    ref = _ref(dy, x)
    # bf16 products are exact in fp32; only the summation order differs
    tol = 1e-3 * (K ** 0.5)
    assert torch.allclose(out, ref, rtol=1e-3, atol=tol), float((out - ref).abs().max())


@pytest.mark.parametrize("two_cta", [False, True])
def test_repeated_calls_and_structured_input(two_cta):
    from switchml_b200.ops.wgrad import wgrad_gemm
    # An operand with one non-zero per row/column makes any layout mistake visible.
    K, M, N = 128, 512, 768
    dy = torch.zeros(K, M, device="cuda", dtype=torch.bfloat16)
    x = torch.zeros(K, N, device="cuda", dtype=torch.bfloat16)
    for k in range(K):
        dy[k, (k * 7) % M] = 1.0 + k % 3
        x[k, (k * 13) % N] = 2.0 + k % 5
    ref = _ref(dy, x)
    for _ in range(3):
        out = wgrad_gemm(dy, x, two_cta=two_cta)
        assert torch.equal(out, ref)


def test_rejects_unaligned_shapes():
    from switchml_b200.ops.wgrad import wgrad_gemm
    from switchml_b200 import NativeError
    dy = torch.randn(64, 100, device="cuda", dtype=torch.bfloat16)   # M not a multiple of 8
    x = torch.randn(64, 256, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(NativeError):
        wgrad_gemm(dy, x)
