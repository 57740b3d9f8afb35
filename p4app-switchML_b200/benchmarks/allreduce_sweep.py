"""Allreduce microbenchmark over message sizes, this library against NCCL on the same box.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        p4app-switchML_b200/benchmarks/allreduce_sweep.py --out sweep.jsonl

For float32 and int32 tensors of 2^10 .. 2^28 elements (values U(-1,1) seeded per rank),
SUM, 10 warm-up + 100 timed iterations, it reports ATE/s (= numel / time per job) and
bus GB/s (= bytes/time * 2(n-1)/n) for
    nccl            torch.distributed.all_reduce on the NCCL backend, float32, in place
    nccl-int32      the same on int32 tensors
    sml-float       this library, float_sum mode, ordinary device tensors
    sml-float-symm  same, tensors in the symmetric heap (reduced where they lie)
    sml-quant       this library, int32_quant mode (exact, order independent), float32 tensors
    sml-int32       int32 tensors
All times are CUDA-event times on the launching stream, maximum over ranks. `--markdown FILE`
writes the table (microseconds per allreduce, and this library's time relative to NCCL's).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def timed(fn, iters, warmup, world):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def markdown_table(results, world, iters, warmup):
    """Microseconds per allreduce by size and implementation; in brackets NCCL's time divided by
    this library's (above 1 = faster than NCCL), against NCCL on the same element type."""
    impls = []
    for r in results:
        if r["impl"] not in impls:
            impls.append(r["impl"])
    by = {(r["impl"], r["numel"]): r for r in results}
    sizes = sorted({r["numel"] for r in results})
    lines = ["%d GPUs, SUM, %d warm-up + %d timed iterations (a quarter of that above 2^26), device time, slowest rank"
             % (world, warmup, iters), "", "| elements | " + " | ".join(impls) + " |", "|---|" + "---|" * len(impls)]
    for n in sizes:
        cells = []
        for impl in impls:
            r = by.get((impl, n))
            if r is None:
                cells.append("")
                continue
            base = by.get(("nccl-int32" if r["dtype"] == "int32" else "nccl", n))
            ratio = "" if base is None or impl.startswith("nccl") else " (%.2fx)" % (base["us"] / r["us"])
            cells.append("%.1f%s" % (r["us"], ratio))
        lines.append("| 2^%d | " % (n.bit_length() - 1) + " | ".join(cells) + " |")
    big = [by.get((impl, sizes[-1])) for impl in impls]
    lines += ["", "Largest size: " + ", ".join("%s %.3g ATE/s, bus %.0f GB/s" % (r["impl"], r["ate_per_s"], r["bus_gbs"])
                                               for r in big if r)]
    return "\n".join(lines) + "\n"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-log2", type=int, default=10)
    ap.add_argument("--max-log2", type=int, default=28)
    ap.add_argument("--step-log2", type=int, default=2)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impls", default="nccl,nccl-int32,sml-float,sml-float-symm,sml-quant,sml-int32")
    ap.add_argument("--markdown", default="", help="write the results as a markdown table to this file")
    ap.add_argument("--transport", default="auto")
    ap.add_argument("--channels", type=int, default=0)
    ap.add_argument("--slot-bytes", type=int, default=0, help="0 = library default")
    ap.add_argument("--exponent-lookahead", type=int, default=-1, help="-1 = library default")
    ap.add_argument("--signal-fence", default="", help="sc | release; empty = library default")
    ap.add_argument("--out", default="")
    a = ap.parse_args()

    import switchml_b200 as sml
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    port = int(os.environ.get("MASTER_PORT", 29500))
    addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    sizes = [1 << k for k in range(a.min_log2, a.max_log2 + 1, a.step_log2)]
    max_bytes = sizes[-1] * 4
    results = []
    ctx = sml.Context.get_instance()
    for impl in a.impls.split(","):
        is_sml = impl.startswith("sml")
        if is_sml:
            mode = "int32_quant" if impl == "sml-quant" else "float_sum"
            heap = (2 * max_bytes >> 20) + 64 if impl == "sml-float-symm" else 0
            opts = dict(packet_numel=256, device=local, controller_ip=addr, controller_port=port + 201,
                        mode=mode, transport=a.transport, launch="inline", symm_heap_mb=heap,
                        wait_timeout_ms=30000)
            if a.slot_bytes:
                opts["slot_bytes"] = a.slot_bytes
            if a.channels:
                opts["channels"] = a.channels
            if a.exponent_lookahead >= 0:
                opts["exponent_lookahead"] = a.exponent_lookahead
            if a.signal_fence:
                opts["signal_fence"] = a.signal_fence
            assert ctx.start(sml.make_config("cuda", rank=rank, num_workers=world, **opts))
        for numel in sizes:
            dtype = torch.int32 if impl.endswith("int32") else torch.float32
            g = torch.Generator(device="cuda").manual_seed(99 + rank)
            if impl == "sml-float-symm":
                ctx.symmetric_reset()
                x = ctx.symmetric_empty(numel, dtype)
                y = ctx.symmetric_empty(numel, dtype)
            else:
                x = torch.empty(numel, dtype=dtype, device="cuda")
                y = torch.empty(numel, dtype=dtype, device="cuda")
            if dtype == torch.int32:
                x.copy_(torch.randint(-1000, 1000, (numel,), generator=g, device="cuda", dtype=torch.int32))
            else:
                x.copy_(torch.rand(numel, generator=g, device="cuda") * 2 - 1)
            jobs = []
            if not is_sml:
                y.copy_(x)

                def fn():
                    dist.all_reduce(y)    # in place, like the reference's benchmark script
            else:
                def fn():
                    jobs.append(ctx.all_reduce_async(x, y))
            iters = a.iters if numel <= (1 << 26) else max(20, a.iters // 4)
            ms = timed(fn, iters, a.warmup, world)
            for j in jobs:
                assert j.wait() == 3, j.error()
                j.release()
            rec = {"impl": impl, "n_gpus": world, "numel": numel, "dtype": str(dtype).split(".")[1],
                   "us": ms * 1e3, "ate_per_s": numel / (ms * 1e-3),
                   "bus_gbs": 4 * numel / (ms * 1e-3) * 2 * (world - 1) / max(world, 1) / 1e9,
                   "transport": ("nvls" if ctx.uses_multimem() else "p2p") if is_sml else "nccl"}
            results.append(rec)
            if rank == 0:
                print(json.dumps(rec), flush=True)
            del x, y
        if is_sml:
            ctx.stop()
    if rank == 0 and a.out:
        with open(a.out, "w") as f:
            for r in results:
                f.write(json.dumps(r) + "\n")
    if rank == 0 and a.markdown:
        with open(a.markdown, "w") as f:
            f.write(markdown_table(results, world, a.iters, a.warmup))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
