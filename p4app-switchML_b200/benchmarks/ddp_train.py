"""Synthetic data-parallel training throughput: ResNet-50 (images/s), VGG-19 (images/s),
BERT-large MLM (tokens/s).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        p4app-switchML_b200/benchmarks/ddp_train.py --model vgg19 --ddp sml --steps 20

Configurations (per GPU): ResNet-50 batch 64 of 3x224x224, SGD momentum 0.9; VGG-19 batch
32, SGD momentum 0.9; BERT-large sequence 512, batch 16, 15 % of the positions masked,
AdamW. Weights and gradients are float32, the forward/backward math runs under bf16
autocast. ``--ddp sml`` uses this library (gradient buckets in the symmetric heap reduced
in place while backward continues; with ``--fused-wgrad 1`` the largest Linear layers
compute their weight gradients with the tcgen05 GEMM that reduces across GPUs in its own
epilogue). ``--ddp torch`` is PyTorch DDP over NCCL, the baseline. Times are CUDA-event
times, maximum over ranks; the end-to-end figure also counts the host→device copy of each
batch from pinned memory and the device→host read of the loss.
"""
import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

DEFAULT_BATCH = {"resnet50": 64, "vgg19": 32, "bert": 16}


def build(model_name, fused):
    from switchml_b200.models import resnet50, vgg19, bert_large
    if model_name == "resnet50":
        return resnet50()
    if model_name == "vgg19":
        return vgg19(fused_fc=fused)
    return bert_large(fused_ffn=fused)


def make_batch(model_name, batch, seq, gen):
    """Pinned host tensors of one synthetic batch."""
    if model_name == "bert":
        ids = torch.randint(0, 30522, (batch, seq), generator=gen)
        labels = torch.full((batch, seq), -100, dtype=torch.long)
        mask = torch.rand(batch, seq, generator=gen) < 0.15
        labels[mask] = ids[mask]
        ids = ids.clone()
        ids[mask] = 103  # [MASK]
        return ids.pin_memory(), labels.pin_memory()
    x = torch.randn(batch, 3, 224, 224, generator=gen)
    y = torch.randint(0, 1000, (batch,), generator=gen)
    return x.pin_memory(), y.pin_memory()


def bench_training(args):
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    port = int(os.environ.get("MASTER_PORT", 29500))
    addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
    model_name = getattr(args, "workload", None) or args.model
    if model_name == "allreduce":
        model_name = args.model
    ddp_kind = getattr(args, "ddp", "sml")
    fused = bool(getattr(args, "fused_wgrad", 0)) and ddp_kind == "sml"
    batch = args.batch or DEFAULT_BATCH[model_name]
    seq = 512
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    torch.manual_seed(0)  # identical initial weights on every rank
    model = build(model_name, fused).to(dev)
    nparams = sum(p.numel() for p in model.parameters())

    ctx = None
    launches_per_step = 0
    if ddp_kind == "sml":
        import switchml_b200 as sml
        from switchml_b200.parallel.ddp import DistributedDataParallel
        ctx = sml.Context.get_instance()
        heap_mb = int(nparams * 4 / (1 << 20) * 1.15) + 256
        assert ctx.start(sml.make_config("cuda", rank=rank, num_workers=world, packet_numel=256, device=local,
                                         controller_ip=addr, controller_port=port + 301, mode=args.mode,
                                         launch="inline", symm_heap_mb=heap_mb, average=True,
                                         channels=args.channels or 32, wait_timeout_ms=60000))
        if fused:
            for layer in model.fused_layers():
                layer.attach(ctx, scale=1.0 / world)
        net = DistributedDataParallel(model, ctx, bucket_mb=25, overlap=True)
        launches_per_step = len(net.buckets.buckets) + (len(model.fused_layers()) if fused else 0)
    elif world > 1:
        net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local], bucket_cap_mb=25,
                                                        gradient_as_bucket_view=True)
    else:
        net = model
    if model_name == "bert":
        opt = torch.optim.AdamW(model.parameters(), lr=1e-4, fused=True)
    else:
        opt = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9)

    gen = torch.Generator().manual_seed(100 + rank)
    host_batches = [make_batch(model_name, batch, seq, gen) for _ in range(2)]
    dev_batches = [(a.to(dev), b.to(dev)) for a, b in host_batches]

    def step(data):
        a, b = data
        with torch.autocast("cuda", dtype=torch.bfloat16):
            if model_name == "bert":
                loss = net(a, b)
            else:
                loss = F.cross_entropy(net(a).float(), b)
        loss.backward()
        opt.step()
        if ddp_kind == "sml":
            net.zero_grad()
            if fused:
                pass  # fused gradients are overwritten, not accumulated
        else:
            opt.zero_grad(set_to_none=False)
        return loss

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(dev_batches[i % 2])
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        loss = step(dev_batches[i % 2])
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    loss_val = float(loss.item())

    # end to end: batch from pinned host memory every step, loss read back every step
    sync()
    t0 = time.perf_counter()
    e2e_steps = max(3, args.steps // 2)
    for i in range(e2e_steps):
        a, b = host_batches[i % 2]
        data = (a.to(dev, non_blocking=True), b.to(dev, non_blocking=True))
        _ = float(step(data).item())
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) / e2e_steps * 1e3
    if world > 1:
        t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])
    if ctx is not None:
        ctx.stop()
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return None
    per_step = batch * world * (seq if model_name == "bert" else 1)
    h2d = sum(t.numel() * t.element_size() for t in host_batches[0])
    out = {
        "metric": "tokens_per_s" if model_name == "bert" else "images_per_s",
        "value": per_step / (ms * 1e-3), "unit": "tokens/s" if model_name == "bert" else "images/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "impl": "switchml_b200" if ddp_kind == "sml" else "torch_ddp_nccl",
        "config": {"model": {"resnet50": "ResNet-50", "vgg19": "VGG-19", "bert": "BERT-large MLM"}[model_name],
                   "global_batch": batch * world, "seq_len": seq if model_name == "bert" else None,
                   "parallelism": "dp%d" % world, "params_m": nparams / 1e6, "ddp": ddp_kind,
                   "fused_wgrad": fused, "optimizer": "AdamW" if model_name == "bert" else "SGD-m0.9",
                   "l2": "activations and gradients of a step exceed the 126 MB L2"},
        "e2e": {"value": per_step / (e2e_ms * 1e-3), "unit": "tokens/s" if model_name == "bert" else "images/s",
                "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
        "gpu_launches": launches_per_step * args.steps, "final_loss": loss_val,
    }
    print(json.dumps(out), flush=True)
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="resnet50", choices=["resnet50", "vgg19", "bert"])
    ap.add_argument("--ddp", default="sml", choices=["sml", "torch"])
    ap.add_argument("--fused-wgrad", type=int, default=0)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--mode", default="float_sum", choices=["float_sum", "int32_quant"])
    ap.add_argument("--channels", type=int, default=0)
    a = ap.parse_args()
    a.workload = a.model
    bench_training(a)
