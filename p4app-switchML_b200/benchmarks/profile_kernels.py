"""Small, self-terminating workloads for profiling one kernel at a time on ONE GPU.

    python p4app-switchML_b200/benchmarks/profile_kernels.py --kernel allreduce_quant
    ncu --set full --clock-control none -k regex:AllReduceEmuKernel -c 1 -o prof \
        python p4app-switchML_b200/benchmarks/profile_kernels.py --kernel allreduce_quant

Kernels: allreduce_quant / allreduce_sum / allreduce_int (streamed aggregation, 4 ranks
emulated in one cooperative launch over peer memory, 2^24 elements per rank: inputs and
outputs of 512 MiB together exceed the 126 MB L2 while staying far below a few GB);
wgrad / wgrad_2cta (tcgen05 weight-gradient GEMM, one CTA per 128x256 tile / two CTAs per
256x256 tile, BERT FFN shape 8192 x 4096 x 1024);
wgrad_fc6 (VGG fc6 shape, K = 32: output-bandwidth bound);
local_copy (what `bench.py --gpus 1` times: a one-worker, out-of-place float_sum allreduce of
2^26 elements through the Context, i.e. LocalCopyKernel over 256 MiB in and 256 MiB out).
Prints CUDA-event timings.
"""
import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def timed(fn, iters):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="allreduce_quant")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--ranks", type=int, default=4)
    ap.add_argument("--log2-numel", type=int, default=24)
    ap.add_argument("--algo", default="staged", choices=["staged", "push"],
                    help="streamed aggregation: whole tiles through the slots, or shards pushed to their owners")
    a = ap.parse_args()
    if a.kernel == "local_copy":
        import switchml_b200 as sml
        ctx = sml.Context.get_instance()
        assert ctx.start(sml.make_config("cuda", packet_numel=256, mode="float_sum", launch="inline"))
        numel = 1 << 26
        x = torch.rand(numel, device="cuda")
        y = torch.empty_like(x)

        def one():
            job = ctx.all_reduce_async(x, y)
            job.stream_wait()
            job.release()
        ms = timed(one, a.iters)
        assert torch.equal(x, y)
        ctx.stop()
        print("local_copy: %d elements, %.4f ms, %.0f GB/s read+write" % (numel, ms, 2 * numel * 4 / ms / 1e6))
    elif a.kernel.startswith("allreduce"):
        from switchml_b200.ops.emulation import emulated_allreduce
        numel = 1 << a.log2_numel
        dtype = torch.int32 if a.kernel == "allreduce_int" else torch.float32
        if dtype == torch.int32:
            xs = [torch.randint(-1000, 1000, (numel,), device="cuda", dtype=dtype) for _ in range(a.ranks)]
        else:
            xs = [torch.rand(numel, device="cuda") * 2 - 1 for _ in range(a.ranks)]
        outs = [torch.empty_like(x) for x in xs]
        mode = "quant" if a.kernel == "allreduce_quant" else "sum"
        ms = timed(lambda: emulated_allreduce(xs, mode=mode, algo=a.algo, block_numel=256, slot_bytes=262144,
                                              slots_per_channel=4, outputs=outs), a.iters)
        # includes allocation of the staging regions; the kernel itself is what ncu captures
        print("%s (%s): %d ranks x %d elements, %.3f ms per call (with staging setup)" % (a.kernel, a.algo, a.ranks, numel, ms))
    else:
        from switchml_b200.ops.wgrad import wgrad_gemm
        K, M, N = (32, 4096, 25088) if a.kernel == "wgrad_fc6" else (8192, 4096, 1024)
        dy = torch.randn(K, M, device="cuda", dtype=torch.bfloat16)
        x = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda")
        two = a.kernel == "wgrad_2cta"
        ms = timed(lambda: wgrad_gemm(dy, x, out=out, two_cta=two), a.iters)
        print("%s: K=%d M=%d N=%d, %.3f ms, %.0f TFLOP/s, output %.0f GB/s" %
              (a.kernel, K, M, N, ms, 2.0 * K * M * N / ms / 1e9, M * N * 4 / ms / 1e6))


if __name__ == "__main__":
    main()
