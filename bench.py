#!/usr/bin/env python
"""Headline benchmark: allreduce rate in aggregated tensor elements per second (ATE/s).

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5
    python bench.py --impl reference ...        # the reference's own NCCL path

One step = one SUM allreduce, in place, of an ordinary float32 device tensor of 2^28
elements: what the reference's benchmark script runs
(benchmarks/allreduce_pytorch_benchmark/allreduce_pytorch_benchmark.py:112-127, default size
from benchmarks/allreduce_benchmark/main.cc:101). ATE/s = numel / time per step; bus GB/s =
4*numel/time * 2(n-1)/n. The timed region is bracketed by a barrier and a device
synchronisation, timed with CUDA events on the launching stream, and the slowest rank
counts. Rank 0 prints one JSON line. Both arms print the same ``config``.

Named extras of this library's arm: the same allreduce on tensors of the symmetric heap
(reduced in place over NVLink without staging), and the exact integer mode (per-block
exponent fixed point) with a bit-for-bit check against the CPU oracle.

The end-to-end figure ("e2e") times the same allreduce for a caller whose data lives in
pinned host memory: every step brings the input host→device, reduces it and returns the
result device→host. This library's arm measures two ways of doing that through its public
API (copies and kernels pipelined over chunks; one kernel that reads and writes the pinned
buffers itself) and reports the faster; the reference arm copies, calls the script's
``dist.all_reduce`` and copies back, the staging pattern of the reference's PyTorch plugin
(frameworks_integration/pytorch_plugin/ProcessGroupSML.cpp:117-163).

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


class SmiSampler:
    """SM clocks and throttle reasons from ``nvidia-smi`` while a region runs (reads only).

    Standard library only, so that the reference arm imports nothing of this repository."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits", "-lms", "25",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, window=None):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        time.sleep(0.05)
        lines = self.lines
        if window and lines:
            inside = [l for l in lines if window[0] <= l[0] <= window[1] + 0.06]
            if len(inside) < 3:  # region shorter than the sampling period: the nearest samples
                mid = 0.5 * (window[0] + window[1])
                inside = sorted(lines, key=lambda l: abs(l[0] - mid))[:5]
            lines = inside
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for _, line in lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])), smax.append(float(f[2])), power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
    port = int(os.environ.get("MASTER_PORT", "29500"))
    return rank, world, local, addr, port


def workload_config(numel, esz, dtype_name, world):
    """The ``config`` entry, identical in both arms."""
    return {"model": "allreduce_microbenchmark", "numel": numel, "tensor_bytes": numel * esz,
            "dtype": dtype_name, "op": "SUM", "placement": "in place, ordinary device tensor",
            "global_batch": None, "seq_len": None, "parallelism": "dp%d" % world,
            "l2": "the tensor (%d MiB) is larger than the 126 MB L2" % (numel * esz >> 20),
            "e2e": "pinned host input -> device -> allreduce -> pinned host output, every step",
            "single_gpu_note": None if world > 1 else
            "with one worker an in-place SUM changes nothing: neither arm moves data in the device-timed "
            "region (NCCL returns at once, this library launches no kernel); the end-to-end figure and "
            "the named extras are the measurements that do work at n_gpus = 1"}


# ------------------------------------------------------------------------------------------
def bench_allreduce(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    rank, world, local, addr, port = dist_env()
    if world != args.gpus:
        raise SystemExit("--gpus %d but WORLD_SIZE is %d (launch with torch.distributed.run)" % (args.gpus, world))
    torch.cuda.set_device(local)
    import switchml_b200 as sml
    from switchml_b200.utils.numa import bind_to_device_numa
    numa_node = bind_to_device_numa(local)  # pinned host buffers allocated from here on sit next to the GPU
    if world > 1:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    numel = args.numel
    dtype = {"float32": torch.float32, "int32": torch.int32, "bfloat16": torch.bfloat16}[args.dtype]
    esz = torch.empty((), dtype=dtype).element_size()

    def max_over_ranks(value):
        if world == 1:
            return value
        t = torch.tensor([value], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def start_context(mode, heap_mb):
        ctx = sml.Context.get_instance()
        opts = dict(packet_numel=args.packet_numel, device=local, controller_ip=addr,
                    controller_port=port + 101, mode=mode, transport=args.transport, launch="inline",
                    symm_heap_mb=heap_mb, wait_timeout_ms=30000)
        if args.slot_bytes:
            opts["slot_bytes"] = args.slot_bytes
        if args.channels:
            opts["channels"] = args.channels
        if not ctx.start(sml.make_config("cuda", rank=rank, num_workers=world, **opts)):
            raise RuntimeError("Context.start failed")
        return ctx

    g = torch.Generator(device="cuda").manual_seed(1234 + rank)

    def fill(t):
        if dtype == torch.int32:
            t.copy_(torch.randint(-2 ** 20, 2 ** 20, (numel,), generator=g, device="cuda", dtype=torch.int32))
        else:
            t.copy_((torch.rand(numel, generator=g, device="cuda") * 2 - 1).to(dtype))
        return t

    def launches(ctx):
        return ctx.get_stats()["backend"].get("kernel_launches", 0)

    def role_budget(ctx):
        """ns that the roles of channel 0 spent waiting / working so far (device counters)."""
        return dict(ctx.get_stats()["backend"].get("channel0_ns") or {})

    sampler = SmiSampler(local)
    if rank == 0:
        sampler.start()  # nvidia-smi needs a moment to start: launch it before the warm-up

    def measure(ctx, x, y, steps, want_clocks=False):
        """W warm-up jobs, then `steps` timed jobs (y None = in place). Returns ms per step
        (device time, slowest rank), kernels launched in the timed region, clocks."""
        jobs = [ctx.all_reduce_async(x, y) for _ in range(args.warmup)]  # enqueued on the current stream
        barrier()
        for j in jobs:
            assert j.wait() == 3, j.error()
            j.release()
        barrier()
        k0 = launches(ctx)
        b0 = role_budget(ctx)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.time()
        start.record()
        jobs = [ctx.all_reduce_async(x, y) for _ in range(steps)]
        stop.record()
        torch.cuda.synchronize()
        w1 = time.time()
        barrier()
        clocks = sampler.stop((w0, w1)) if (rank == 0 and want_clocks) else None
        dev_ms = start.elapsed_time(stop)
        for j in jobs:
            assert j.wait() == 3, j.error()
            j.release()
        k1 = launches(ctx)
        if k1 == k0:
            dev_ms = max(dev_ms, (w1 - w0) * 1e3)  # nothing ran on the device: the host's time per call
        b1 = role_budget(ctx)
        measure.budget_us_per_step = {k: round((b1[k] - b0.get(k, 0)) / steps / 1e3, 1) for k in b1}
        return max_over_ranks(dev_ms) / steps, k1 - k0, clocks

    heap_mb = (2 * numel * esz >> 20) + 64 if args.symmetric else 0
    ctx = start_context("float_sum", heap_mb)
    multimem = ctx.uses_multimem()

    # ---- correctness of the headline path against NCCL, on values that are still small ----
    x = fill(torch.empty(numel, dtype=dtype, device="cuda"))
    check = None
    if world > 1:
        ref = x.clone()
        dist.all_reduce(ref)
        mine = x.clone()
        j = ctx.all_reduce_async(mine)
        assert j.wait() == 3, j.error()
        j.release()
        torch.cuda.synchronize()
        if dtype == torch.int32:
            bad = int((mine != ref).sum().item())
            check = {"int32_mismatches_vs_nccl": bad}
            assert bad == 0, "int32 allreduce differs from NCCL in %d elements" % bad
        else:
            err = (mine.float() - ref.float()).abs().max().item()
            scale = ref.float().abs().max().item()
            check = {"max_abs_err_vs_nccl": err, "max_abs": scale}
            assert err <= 1e-3 * max(scale, 1.0), "allreduce result is wrong: err %g" % err
        del ref, mine

    # ---- headline: ordinary tensor, in place (the reference script's call) ----
    ms, head_launches, clocks = measure(ctx, x, None, args.steps, True)
    head_budget = measure.budget_us_per_step
    total_launches = head_launches
    breakdown = {"headline_in_place": head_launches}

    # ---- extra: tensors of the symmetric heap, out of place ----
    symmetric = None
    if args.symmetric:
        sx, sy = fill(ctx.symmetric_empty(numel, dtype)), ctx.symmetric_empty(numel, dtype)
        s_ms, s_launches, _ = measure(ctx, sx, sy, max(3, args.steps // 2))
        symmetric = {"note": "tensors from Context.symmetric_empty, out of place; with several workers they are "
                             "reduced over NVLink where they lie, with one worker this is a device copy",
                     "ms_per_step": s_ms, "ate_per_worker": numel / (s_ms * 1e-3),
                     "bus_gbs": esz * numel / (s_ms * 1e-3) * (2.0 * (world - 1) / world) / 1e9}
        total_launches += s_launches
        breakdown["symmetric_tensors"] = s_launches
        del sx, sy
        ctx.symmetric_reset()

    # ---- end to end: pinned host -> device -> allreduce -> pinned host ----
    hx = torch.empty(numel, dtype=dtype, pin_memory=True)
    hy = torch.empty(numel, dtype=dtype, pin_memory=True)
    hx.copy_(fill(x))
    torch.cuda.synchronize()
    e2e_steps = args.e2e_steps

    def time_host(fn, steps):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        barrier()
        k0 = launches(ctx)
        t0 = time.perf_counter()
        for _ in range(steps):
            fn()  # returns when the result is in host memory
        torch.cuda.synchronize()
        t = (time.perf_counter() - t0) / steps
        return max_over_ranks(t * 1e3), launches(ctx) - k0

    # ceiling: nothing but the two copies, at the same time, on every GPU at once
    dx = torch.empty(numel, dtype=dtype, device="cuda")
    s_up, s_down = torch.cuda.Stream(), torch.cuda.Stream()

    def copies_only():
        with torch.cuda.stream(s_up):
            dx.copy_(hx, non_blocking=True)
        with torch.cuda.stream(s_down):
            hy.copy_(x, non_blocking=True)
        s_up.synchronize()
        s_down.synchronize()

    ceiling_ms, _ = time_host(copies_only, max(2, e2e_steps // 2))
    del dx

    from switchml_b200.parallel.host_pipeline import HostAllReduce
    variants = {}
    pipe = HostAllReduce(ctx, numel, dtype, chunk_numel=args.e2e_chunk)
    variants["pipelined_copies"] = time_host(lambda: pipe.run(hx, hy), e2e_steps)
    pipe.close()
    store_out = HostAllReduce(ctx, numel, dtype, chunk_numel=args.e2e_chunk, direct="out")
    variants["copy_in_kernel_stores_to_pinned"] = time_host(lambda: store_out.run(hx, hy), e2e_steps)
    store_out.close()
    direct = HostAllReduce(ctx, numel, dtype, direct=True)
    variants["kernel_on_pinned_memory"] = time_host(lambda: direct.run(hx, hy), e2e_steps)
    direct.close()
    e2e_check = None
    if world > 1 and dtype != torch.int32:
        ref = x.clone()
        dist.all_reduce(ref)
        e2e_check = (hy.cuda().float() - ref.float()).abs().max().item()
        assert e2e_check <= 1e-3 * max(ref.float().abs().max().item(), 1.0), "end-to-end result is wrong"
        del ref
    best = min(variants, key=lambda k: variants[k][0])
    e2e_ms, e2e_launches = variants[best]
    total_launches += e2e_launches
    breakdown["e2e"] = e2e_launches

    stats = ctx.get_stats()
    ctx.stop()

    # ---- extra: the exact, order-independent integer mode (SwitchML's block fixed point) ----
    quant = None
    if dtype == torch.float32 and args.quant_steps > 0:
        ctx = start_context("int32_quant", 0)
        # bit-for-bit against the CPU oracle on an odd-sized tensor with zero blocks
        from switchml_b200.ops.oracle import quant_allreduce_oracle
        small = (1 << 22) + 1  # above the one-barrier kernel's limit at every worker count: the streaming path
        rng = [np.random.RandomState(77 + r) for r in range(world)]
        ins = [(r_.rand(small).astype(np.float32) * 2 - 1) * np.float32(10.0 ** (i - 2)) for i, r_ in enumerate(rng)]
        for a in ins:
            a[4096:8192] = 0.0
            a[-257:-1] = 0.0
        want = quant_allreduce_oracle(ins, args.packet_numel)
        t_in = torch.from_numpy(ins[rank]).cuda()
        t_out = torch.empty_like(t_in)
        j = ctx.all_reduce_async(t_in, t_out)
        assert j.wait() == 3, j.error()
        j.release()
        torch.cuda.synchronize()
        mismatches = int((t_out.cpu().numpy().view(np.uint32) != want.view(np.uint32)).sum())
        mismatches = int(max_over_ranks(float(mismatches)))
        assert mismatches == 0, "int32_quant result differs from the oracle in %d elements" % mismatches
        y = torch.empty(numel, dtype=dtype, device="cuda")
        q_ms, q_launches, _ = measure(ctx, fill(x), y, args.quant_steps)
        quant = {"note": "int32_quant mode (per-block exponent fixed point, exact integer sum), ordinary tensors, "
                         "out of place", "ms_per_step": q_ms, "ate_per_worker": numel / (q_ms * 1e-3),
                 "steps": args.quant_steps, "oracle_check": {"numel": small, "mismatched_bits": mismatches},
                 "channel0_us_per_step": measure.budget_us_per_step}
        total_launches += q_launches
        breakdown["int32_quant"] = q_launches
        del y
        ctx.stop()
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return
    ate = numel / (ms * 1e-3)  # per worker, the reference's definition
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
        "config": workload_config(numel, esz, args.dtype, world),
        "impl_details": {"mode": "float_sum", "transport": "nvls" if multimem else ("p2p" if world > 1 else "local"),
                         "packet_numel": args.packet_numel,
                         "channel0_us_per_step": head_budget},
        "bus_gbs": esz * numel / (ms * 1e-3) * (2.0 * (world - 1) / world) / 1e9,
        "alg_gbs": esz * numel / (ms * 1e-3) / 1e9,
        "symmetric_tensors": symmetric,
        "int32_quant": quant,
        "e2e": {"value": world * numel / (e2e_ms * 1e-3), "unit": "elements/s", "ms_per_step": e2e_ms,
                "ate_per_worker": numel / (e2e_ms * 1e-3),
                "h2d_bytes_per_step": numel * esz, "d2h_bytes_per_step": numel * esz,
                "steps": e2e_steps, "gpu_launches_per_step": e2e_launches / e2e_steps, "path": best,
                "variants_ms": {k: v[0] for k, v in variants.items()},
                "copy_ceiling_ms": ceiling_ms, "host_numa_node": numa_node,
                "max_abs_err_vs_nccl": e2e_check},
        "gpu_launches": total_launches,
        "gpu_launches_by_region": breakdown,
        "clocks": clocks, "check": check,
        "stats": {"jobs_finished": stats["jobs_finished"], "jobs_failed": stats["jobs_failed"],
                  "tiles": stats["backend"]["tiles"]},
    }
    print(json.dumps(out), flush=True)


# ------------------------------------------------------------------------------------------
def bench_reference(args):
    """Run the reference's own benchmark script, unmodified, on its NCCL backend.

    Nothing of this repository's package is imported here. The script times with the host
    clock around ``work.wait()``, which for NCCL does not wait for the GPU, so the device
    time is taken with CUDA events recorded around the script's own ``dist.all_reduce``
    calls (the calls themselves are untouched). Afterwards, on the process group the script
    created, the end-to-end loop: pinned host -> device copy, ``dist.all_reduce``, device ->
    pinned host copy, one after the other as the reference's PyTorch plugin stages them."""
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
    sampler = SmiSampler(local)
    if rank == 0:
        sampler.start()
    log = open(os.devnull, "w")
    sys.stdout = log
    w0 = time.time()
    try:
        runpy.run_path(script, run_name="__main__")
    finally:
        sys.stdout = old_stdout
        sys.argv = old_argv
        dist.all_reduce = real_all_reduce
    torch.cuda.synchronize()
    w1 = time.time()
    clocks = sampler.stop((w0, w1)) if rank == 0 else None
    timed = events[args.warmup:]
    total_ms = timed[0][0].elapsed_time(timed[-1][1])
    ms = total_ms / len(timed)

    def max_over_ranks(value):
        if world == 1:
            return value
        t = torch.tensor([value], dtype=torch.float64, device="cuda")
        real_all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ms = max_over_ranks(ms)

    # ---- end to end on the script's process group ----
    numel = args.numel
    dtype = torch.float32 if args.dtype == "float32" else torch.int32
    hx = torch.rand(numel, dtype=torch.float32).to(dtype).pin_memory()
    hy = torch.empty(numel, dtype=dtype, pin_memory=True)
    d = torch.empty(numel, dtype=dtype, device="cuda")

    def step():
        d.copy_(hx, non_blocking=True)
        real_all_reduce(d, op=dist.ReduceOp.SUM)
        hy.copy_(d, non_blocking=True)
        torch.cuda.synchronize()  # the result is in host memory

    for _ in range(2):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        step()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) / args.e2e_steps * 1e3)
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return
    ate = numel / (ms * 1e-3)
    print(json.dumps({
        "impl": "reference", "metric": "allreduce_ate_per_s", "value": ate * world, "unit": "elements/s",
        "ate_per_worker": ate,
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": ate / PUBLISHED_ATE,
        "dtype": "fp32" if args.dtype == "float32" else args.dtype, "data": "synthetic (script's --random)",
        "config": workload_config(numel, 4, args.dtype, world),
        "impl_details": {"backend": "nccl via dev_root/benchmarks/allreduce_pytorch_benchmark (unmodified)",
                         "timing": "CUDA events around the script's dist.all_reduce calls"},
        "bus_gbs": 4 * numel / (ms * 1e-3) * (2.0 * (world - 1) / world) / 1e9,
        "e2e": {"value": world * numel / (e2e_ms * 1e-3), "unit": "elements/s", "ms_per_step": e2e_ms,
                "ate_per_worker": numel / (e2e_ms * 1e-3), "h2d_bytes_per_step": numel * 4,
                "d2h_bytes_per_step": numel * 4, "steps": args.e2e_steps,
                "path": "pinned host -> device copy, dist.all_reduce (NCCL), device -> pinned host copy"},
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
    ap.add_argument("--mode", default=os.environ.get("SWITCHML_MODE", "float_sum"), choices=["int32_quant", "float_sum"],
                    help="training workloads: aggregation mode of the gradient allreduce (the allreduce workload "
                         "measures float_sum as the headline and int32_quant as a named extra)")
    ap.add_argument("--transport", default="auto", choices=["auto", "nvls", "p2p"])
    ap.add_argument("--symmetric", type=int, default=1,
                    help="1: also measure tensors allocated with Context.symmetric_empty (reduced where they lie)")
    ap.add_argument("--packet-numel", type=int, default=256)
    ap.add_argument("--slot-bytes", type=int, default=0, help="0 = library default")
    ap.add_argument("--channels", type=int, default=0)
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--quant-steps", type=int, default=5, help="steps of the int32_quant measurement (0 = skip)")
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
