#!/usr/bin/env python
"""Headline benchmark: allreduce rate in aggregated tensor elements per second (ATE/s).

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5
    python bench.py --impl reference ...        # the reference's own NCCL path

One step = one SUM allreduce of a float32 tensor of 2^28 elements (the default of the
reference's benchmark tools, benchmarks/allreduce_benchmark/main.cc:101) through the
public Context API. ATE/s = numel / time per step; bus GB/s = 4*numel/time * 2(n-1)/n.
The timed region is bracketed by a barrier and a device synchronisation, timed with CUDA
events on the launching stream, and the slowest rank counts. Rank 0 prints one JSON line.

The end-to-end figure ("e2e") times the same allreduce for a caller whose data lives in
pinned host memory: every step copies the input host→device, reduces it and reads the
result back device→host, through switchml_b200.parallel.host_pipeline.HostAllReduce.

Other workloads (same JSON shape): --workload resnet50 | vgg19 | bert (synthetic DDP
training, images/s or tokens/s).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PUBLISHED_ATE = 2.82e9  # SwitchML-RDMA, 8 workers, read off the reference's benchmark figure


from switchml_b200.utils.clocks import ClockSampler  # noqa: E402


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
    port = int(os.environ.get("MASTER_PORT", "29500"))
    return rank, world, local, addr, port


def max_over_ranks(value, world):
    import torch
    import torch.distributed as dist
    if world == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world):
    import torch
    import torch.distributed as dist
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def start_context(args, rank, world, local, addr, port, heap_mb=0):
    import switchml_b200 as sml
    ctx = sml.Context.get_instance()
    opts = dict(packet_numel=args.packet_numel, device=local, controller_ip=addr,
                controller_port=port + 101, mode=args.mode, transport=args.transport, launch="inline",
                symm_heap_mb=heap_mb, wait_timeout_ms=30000)
    if args.slot_bytes:
        opts["slot_bytes"] = args.slot_bytes
    if args.channels:
        opts["channels"] = args.channels
    if not ctx.start(sml.make_config("cuda", rank=rank, num_workers=world, **opts)):
        raise RuntimeError("Context.start failed")
    return ctx


# ------------------------------------------------------------------------------------------
def bench_allreduce(args):
    import torch
    import torch.distributed as dist
    rank, world, local, addr, port = dist_env()
    if world != args.gpus:
        raise SystemExit("--gpus %d but WORLD_SIZE is %d (launch with torch.distributed.run)" % (args.gpus, world))
    torch.cuda.set_device(local)
    from switchml_b200.utils.numa import bind_to_device_numa
    numa_node = bind_to_device_numa(local)  # pinned host buffers end up next to the GPU
    if world > 1:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    numel = args.numel
    dtype = {"float32": torch.float32, "int32": torch.int32, "bfloat16": torch.bfloat16}[args.dtype]
    esz = torch.empty((), dtype=dtype).element_size()
    heap_mb = 0
    if args.symmetric:
        heap_mb = (2 * numel * esz >> 20) + 64
    ctx = start_context(args, rank, world, local, addr, port, heap_mb)

    g = torch.Generator(device="cuda").manual_seed(1234 + rank)

    def make_tensors(symmetric):
        if symmetric:
            a, b = ctx.symmetric_empty(numel, dtype), ctx.symmetric_empty(numel, dtype)
        else:
            a = torch.empty(numel, dtype=dtype, device="cuda")
            b = torch.empty(numel, dtype=dtype, device="cuda")
        if dtype == torch.int32:
            a.copy_(torch.randint(-2 ** 20, 2 ** 20, (numel,), generator=g, device="cuda", dtype=torch.int32))
        else:
            a.copy_((torch.rand(numel, generator=g, device="cuda") * 2 - 1).to(dtype))
        return a, b

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()  # nvidia-smi needs a moment to start: launch it before the warm-up

    def measure(x, y, steps, want_clocks):
        """W warm-up jobs, a correctness check against NCCL, then `steps` timed jobs."""
        jobs = [ctx.all_reduce_async(x, y) for _ in range(args.warmup)]  # enqueued on the current stream
        barrier(world)
        for j in jobs:
            assert j.wait() == 3, j.error()
            j.release()
        check = None
        if world > 1 and dtype != torch.int32:
            ref = x.clone().float()
            dist.all_reduce(ref)
            err = (y.float() - ref).abs().max().item()
            scale = ref.abs().max().item()
            check = {"max_abs_err_vs_nccl": err, "max_abs": scale}
            assert err <= 1e-3 * max(scale, 1.0), "allreduce result is wrong: err %g" % err
            del ref
        barrier(world)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.time()
        start.record()
        jobs = [ctx.all_reduce_async(x, y) for _ in range(steps)]
        stop.record()
        torch.cuda.synchronize()
        w1 = time.time()
        barrier(world)
        clocks = sampler.stop((w0, w1)) if (rank == 0 and want_clocks) else None
        t = max_over_ranks(start.elapsed_time(stop), world) / steps
        for j in jobs:
            assert j.wait() == 3, j.error()
            j.release()
        return t, check, clocks

    # Secondary measurement first: ordinary device tensors, which go through the staging ring.
    plain_ms = None
    if args.symmetric and args.mode == "float_sum":
        px, py = make_tensors(False)
        plain_ms, _, _ = measure(px, py, max(3, args.steps // 2), False)
        del px, py
    x, y = make_tensors(bool(args.symmetric) and args.mode == "float_sum")
    ms, check, clocks = measure(x, y, args.steps, True)

    # ---- end to end: pinned host -> device -> allreduce -> pinned host ----
    hx = torch.empty(numel, dtype=dtype, pin_memory=True)
    hy = torch.empty(numel, dtype=dtype, pin_memory=True)
    hx.copy_(x)
    from switchml_b200.parallel.host_pipeline import HostAllReduce
    pipe = HostAllReduce(ctx, numel, dtype, chunk_numel=args.e2e_chunk)
    for _ in range(max(1, min(args.warmup, 3))):
        pipe.run(hx, hy)
    torch.cuda.synchronize()
    barrier(world)
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        pipe.run(hx, hy)  # returns when the result is in host memory
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / args.e2e_steps
    e2e_ms = max_over_ranks(e2e_s * 1e3, world)
    e2e_launches = pipe.launches_per_run
    pipe.close()

    stats = ctx.get_stats()
    multimem = ctx.uses_multimem()
    ctx.stop()
    # Secondary measurement: the exact, order-independent integer mode (SwitchML's block
    # fixed point), ordinary tensors, same size. It needs its own context (mode is a setting).
    quant = None
    if args.mode == "float_sum" and dtype == torch.float32 and args.quant_steps > 0:
        del x, y
        saved_mode, args.mode = args.mode, "int32_quant"
        ctx = start_context(args, rank, world, local, addr, port, 0)
        args.mode = saved_mode
        qx, qy = make_tensors(False)
        q_ms, _, _ = measure(qx, qy, args.quant_steps, False)
        quant = {"note": "int32_quant mode (per-block exponent fixed point, exact integer sum), ordinary tensors",
                 "ms_per_step": q_ms, "ate_per_worker": numel / (q_ms * 1e-3), "steps": args.quant_steps}
        del qx, qy
        ctx.stop()
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return
    ate = numel / (ms * 1e-3)  # per worker, the reference's definition
    bus = esz * numel / (ms * 1e-3) * (2.0 * (world - 1) / world) / 1e9
    out = {
        "metric": "allreduce_ate_per_s", "value": ate * world, "unit": "elements/s", "n_gpus": world,
        "value_definition": "whole-job aggregate: n_gpus x numel / time per allreduce; ate_per_worker = numel / time "
                            "is the reference's per-worker ATE/s, and vs_baseline = ate_per_worker / 2.82e9 "
                            "(SwitchML-RDMA, 8 workers, published figure)",
        "ate_per_worker": ate,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": ate / PUBLISHED_ATE, "dtype": "fp32" if args.dtype == "float32" else args.dtype,
        "data": "synthetic U(-1,1) seeded per rank",
        "impl": "switchml_b200",
        "config": {"model": "allreduce_microbenchmark", "numel": numel, "tensor_bytes": numel * esz,
                   "global_batch": None, "seq_len": None, "parallelism": "dp%d" % world,
                   "op": "SUM", "mode": args.mode, "transport": "nvls" if multimem else ("p2p" if world > 1 else "local"),
                   "symmetric_buffers": bool(args.symmetric) and args.mode == "float_sum", "packet_numel": args.packet_numel,
                   "l2": "input and output tensors (%d MiB each) are larger than the 126 MB L2" % (numel * esz >> 20),
                   "placement": "out of place (input -> output), so repeated steps keep their values bounded",
                   "single_gpu_note": None if world > 1 else
                   "with one worker the sum is a copy: one pass over input and output at HBM speed; NCCL's "
                   "in-place allreduce on a single rank returns without touching the data"},
        "bus_gbs": bus, "alg_gbs": esz * numel / (ms * 1e-3) / 1e9,
        "int32_quant": quant,
        "plain_tensors": None if plain_ms is None else {
            "note": "same allreduce on ordinary torch tensors (staged through the slot ring)",
            "ms_per_step": plain_ms, "ate_per_worker": numel / (plain_ms * 1e-3)},
        "e2e": {"value": world * numel / (e2e_ms * 1e-3), "unit": "elements/s", "ms_per_step": e2e_ms,
                "ate_per_worker": numel / (e2e_ms * 1e-3),
                "h2d_bytes_per_step": numel * esz, "d2h_bytes_per_step": numel * esz,
                "steps": args.e2e_steps, "gpu_launches_per_step": e2e_launches, "host_numa_node": numa_node},
        "gpu_launches": args.steps,
        "clocks": clocks, "check": check,
        "stats": {"jobs_finished": stats["jobs_finished"], "jobs_failed": stats["jobs_failed"],
                  "tiles": stats["backend"]["tiles"]},
    }
    print(json.dumps(out), flush=True)


# ------------------------------------------------------------------------------------------
def bench_reference(args):
    """Run the reference's own benchmark script, unmodified, on its NCCL backend.

    The script times with the host clock around ``work.wait()``, which for NCCL does not
    wait for the GPU, so the device time is taken here with CUDA events recorded around
    the script's own ``dist.all_reduce`` calls (the calls themselves are untouched)."""
    rank, world, local, addr, port = dist_env()
    script = os.path.join(ROOT, "baseline", "_ref", "benchmarks", "allreduce_pytorch_benchmark",
                          "allreduce_pytorch_benchmark.py")
    if not os.path.exists(script):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable":
                              "baseline/_ref has no copy of the reference benchmark script (pip cannot install the "
                              "reference: it has no setup.py/pyproject.toml at its root)"}))
        return
    import runpy
    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "no GPU"}))
        return
    torch.cuda.set_device(local)
    events = []
    real_all_reduce = dist.all_reduce

    def traced(*a, **kw):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        r = real_all_reduce(*a, **kw)
        if hasattr(r, "wait"):
            r.wait()  # stream-orders the collective before the end event (no host block)
        e1.record()
        events.append((e0, e1))
        return r

    dist.all_reduce = traced
    tt = "float" if args.dtype == "float32" else "int32"
    argv = [script, "-n", str(world), "-r", str(rank), "-ip", addr, "-bk", "nccl", "-tn", str(args.numel),
            "-tt", tt, "-d", "gpu", "-nj", str(args.steps), "-nw", str(args.warmup), "--random", "--seed",
            str(1234 + rank)]
    # torchrun tells c10d to reuse the launcher's store; the script brings its own
    # tcp://<ip>:23456 store, whose server rank 0 only starts when that variable is unset.
    os.environ.pop("TORCHELASTIC_USE_AGENT_STORE", None)
    old_argv, old_stdout = sys.argv, sys.stdout
    sys.argv = argv
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    log = open(os.devnull, "w")
    sys.stdout = log
    try:
        runpy.run_path(script, run_name="__main__")
    finally:
        sys.stdout = old_stdout
        sys.argv = old_argv
        dist.all_reduce = real_all_reduce
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    timed = events[args.warmup:]
    total_ms = timed[0][0].elapsed_time(timed[-1][1])
    ms = total_ms / len(timed)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        real_all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.destroy_process_group()
    if rank != 0:
        return
    numel = args.numel
    ate = numel / (ms * 1e-3)
    print(json.dumps({
        "impl": "reference", "metric": "allreduce_ate_per_s", "value": ate * world, "unit": "elements/s",
        "ate_per_worker": ate,
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": ate / PUBLISHED_ATE,
        "dtype": "fp32" if args.dtype == "float32" else args.dtype, "data": "synthetic (script's --random)",
        "config": {"model": "allreduce_microbenchmark", "numel": numel, "parallelism": "dp%d" % world,
                   "backend": "nccl via dev_root/benchmarks/allreduce_pytorch_benchmark (unmodified)",
                   "timing": "CUDA events around the script's dist.all_reduce calls"},
        "bus_gbs": 4 * numel / (ms * 1e-3) * (2.0 * (world - 1) / world) / 1e9,
        "clocks": clocks,
    }), flush=True)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="allreduce", choices=["allreduce", "resnet50", "vgg19", "bert"])
    ap.add_argument("--numel", type=int, default=1 << 28)
    ap.add_argument("--dtype", default="float32", choices=["float32", "int32", "bfloat16"])
    ap.add_argument("--mode", default=os.environ.get("SWITCHML_MODE", "float_sum"),
                    choices=["int32_quant", "float_sum"])
    ap.add_argument("--transport", default="auto", choices=["auto", "nvls", "p2p"])
    ap.add_argument("--symmetric", type=int, default=1,
                    help="1: the tensors are allocated with Context.symmetric_empty (reduced in place over NVLink, "
                         "float_sum mode); 0: ordinary torch tensors through the staging ring")
    ap.add_argument("--packet-numel", type=int, default=256)
    ap.add_argument("--slot-bytes", type=int, default=0, help="0 = library default")
    ap.add_argument("--channels", type=int, default=0)
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--quant-steps", type=int, default=5, help="steps of the secondary int32_quant measurement (0 = skip)")
    ap.add_argument("--e2e-chunk", type=int, default=1 << 24)
    ap.add_argument("--batch", type=int, default=0, help="per-GPU batch for the training workloads")
    ap.add_argument("--ddp", default="sml", choices=["sml", "torch"], help="training workloads: this library or PyTorch DDP/NCCL")
    ap.add_argument("--fused-wgrad", type=int, default=0, help="training workloads: tcgen05 wgrad GEMM with fused reduce")
    ap.add_argument("--model", default="resnet50")
    ap.add_argument("--watchdog", type=float, default=float(os.environ.get("SWITCHML_BENCH_WATCHDOG", "0")),
                    help="dump all Python stacks and exit if the run takes longer than this many seconds")
    args = ap.parse_args()
    if args.watchdog > 0:
        import faulthandler
        faulthandler.dump_traceback_later(args.watchdog, exit=True)
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return bench_reference(args)
    if args.workload == "allreduce":
        return bench_allreduce(args)
    from switchml_b200.benchmarks.ddp_train import bench_training
    return bench_training(args)


if __name__ == "__main__":
    main()
