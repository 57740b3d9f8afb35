"""Weight-gradient GEMM with the cross-GPU reduction fused into the kernel, against the
same GEMM followed by a separate allreduce of the gradient.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        p4app-switchML_b200/benchmarks/wgrad_fused_bench.py

Shapes: VGG-19 fc6 (K = 32 per GPU, 4096 x 25088), fc7, BERT-large FFN (K = 8192 tokens per
GPU, 4096 x 1024). For each it reports
    gemm          the tcgen05 GEMM alone (no communication)
    gemm+reduce   GEMM, then the in-place zero-copy allreduce of dW (two kernels)
    fused         one kernel: tiles are reduced through the NVSwitch as they are produced
    gather        (where the operands are small next to the gradient) the ranks exchange dY and
                  X, every rank computes the tiles it owns over all of them and broadcasts them
    cublas+nccl   torch.mm (fp32 output) followed by NCCL all_reduce, the library baseline
and the roofline of the fused kernel: the slower of FLOPs at the measured bf16 peak and
dW bytes x (1 + 1/n) at 770 GB/s per direction. CUDA-event times, maximum over ranks.
"""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PEAK_TFLOPS = 1662.6   # measured cuBLAS bf16 burst on this pool
LINK_GBS = 770.0       # measured peer copy per direction


def main():
    import switchml_b200 as sml
    from switchml_b200.ops.wgrad import FusedWgrad, wgrad_gemm
    from switchml_b200.utils.timing import time_cuda
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    port = int(os.environ.get("MASTER_PORT", 29500))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = sml.Context.get_instance()
    assert ctx.start(sml.make_config("cuda", rank=rank, num_workers=world, packet_numel=256, device=local,
                                     controller_port=port + 501, mode="float_sum", launch="inline",
                                     transport="nvls" if world > 1 else "auto", symm_heap_mb=1200,
                                     wait_timeout_ms=30000))
    shapes = [("vgg_fc6", 32, 4096, 25088), ("vgg_fc7", 32, 4096, 4096), ("bert_ffn", 8192, 4096, 1024)]
    for name, K, M, N in shapes:
        ctx.symmetric_reset()
        fw = FusedWgrad(ctx, M, N, scale=1.0 / world, policy="fused")
        fg = FusedWgrad(ctx, M, N, scale=1.0 / world, policy="gather") if K * (M + N) * 2 * world <= M * N * 4 else None
        dy = torch.randn(K, M, device="cuda", dtype=torch.bfloat16)
        x = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
        plain = torch.empty(M, N, device="cuda")
        dyt = dy.t()

        def gemm_then_reduce():
            wgrad_gemm(dy, x, out=fw.grad)
            job = ctx.all_reduce_async(fw.grad.view(-1))
            job.release()

        def cublas_nccl():
            g = torch.mm(dyt, x, out_dtype=torch.float32)
            if world > 1:
                dist.all_reduce(g)

        t_gemm = time_cuda(lambda: wgrad_gemm(dy, x, out=plain), 20, 3, world)
        t_two = time_cuda(gemm_then_reduce, 20, 3, world)
        t_fused = time_cuda(lambda: fw.run(dy, x), 20, 3, world)
        t_lib = time_cuda(cublas_nccl, 20, 3, world)
        t_gather = time_cuda(lambda: fg.run(dy, x), 20, 3, world) if fg is not None and fg.fused else None
        torch.cuda.synchronize()
        assert int(fw.error.item()) == 0 and (fg is None or int(fg.error.item()) == 0)
        flops = 2.0 * K * M * N
        link_bytes = M * N * 4 * (1 + 1.0 / world) if world > 1 else 0
        roof_ms = max(flops / (PEAK_TFLOPS * 1e12), link_bytes / (LINK_GBS * 1e9)) * 1e3
        if rank == 0:
            print(json.dumps({"shape": name, "K": K, "M": M, "N": N, "n_gpus": world, "fused_in_kernel": fw.fused,
                              "gemm_ms": t_gemm, "gemm_then_reduce_ms": t_two, "fused_ms": t_fused,
                              "gather_ms": t_gather, "gather_roofline_ms": M * N * 4 / (LINK_GBS * 1e9) * 1e3,
                              "cublas_nccl_ms": t_lib, "roofline_ms": roof_ms,
                              "fused_fraction_of_roofline": roof_ms / t_fused}), flush=True)
    ctx.stop()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
