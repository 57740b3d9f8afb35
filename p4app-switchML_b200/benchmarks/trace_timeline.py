"""Per-tile timeline of one allreduce on channel 0 (`[backend.cuda] trace = true`).

    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 \
        p4app-switchML_b200/benchmarks/trace_timeline.py --mode int32_quant --log2-numel 28

After 3 warm-up and 10 timed jobs (CUDA events, slowest rank) one more job runs and rank 0 prints,
for each of the first tiles of channel 0, when loader, reducer and storer began the tile (their
waits were over) and finished it, in microseconds after the kernel's start, followed by the
derived columns
    Lwork Rwork Swork   time each role spent on the tile
    L>R                 loader finished -> reducer began (signal latency, or the reducer was busy)
    R>S                 reducer finished -> storer began (all ranks' reducers have to finish)
    S>L                 storer finished tile k -> loader began tile k + slots (near 0: the loader
                        waits for slots)
A role that is never idle between tiles is the bottleneck. `--json FILE` stores every rank's raw
timeline (nanoseconds) as FILE.rank<r>.json.
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

KEYS = ("loader_began", "loader_finished", "reducer_began", "reducer_finished", "storer_began", "storer_finished")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="int32_quant", choices=["int32_quant", "float_sum"])
    ap.add_argument("--log2-numel", type=int, default=28)
    ap.add_argument("--transport", default="auto")
    ap.add_argument("--slot-bytes", type=int, default=0, help="0 = library default")
    ap.add_argument("--slots", type=int, default=0, help="0 = library default")
    ap.add_argument("--channels", type=int, default=0)
    ap.add_argument("--exponent-lookahead", type=int, default=-1, help="-1 = library default")
    ap.add_argument("--signal-fence", default="", help="sc | release; empty = library default")
    ap.add_argument("--rows", type=int, default=14, help="tiles to print from the start (the last four are always printed)")
    ap.add_argument("--json", default="")
    a = ap.parse_args()

    import switchml_b200 as sml
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    port = int(os.environ.get("MASTER_PORT", 29500))
    torch.cuda.set_device(local)
    assert world > 1, "a single worker has no tiles to trace: run one process per GPU on two or more GPUs"
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    opts = dict(packet_numel=256, device=local, controller_ip=os.environ.get("MASTER_ADDR", "127.0.0.1"),
                controller_port=port + 211, mode=a.mode, transport=a.transport, launch="inline",
                wait_timeout_ms=20000, trace=True)
    if a.slot_bytes:
        opts["slot_bytes"] = a.slot_bytes
    if a.slots:
        opts["slots_per_channel"] = a.slots
    if a.channels:
        opts["channels"] = a.channels
    if a.exponent_lookahead >= 0:
        opts["exponent_lookahead"] = a.exponent_lookahead
    if a.signal_fence:
        opts["signal_fence"] = a.signal_fence
    ctx = sml.Context.get_instance()
    assert ctx.start(sml.make_config("cuda", rank=rank, num_workers=world, **opts))
    numel = 1 << a.log2_numel
    x = torch.rand(numel, device="cuda") * 2 - 1
    y = torch.empty_like(x)
    jobs = [ctx.all_reduce_async(x, y) for _ in range(3)]
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    jobs += [ctx.all_reduce_async(x, y) for _ in range(10)]
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / 10], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.barrier()
    torch.cuda.synchronize()
    jobs.append(ctx.all_reduce_async(x, y))
    torch.cuda.synchronize()
    for j in jobs:
        assert j.wait() == sml.JobStatus.FINISHED, j.error()
        j.release()
    stats = ctx.get_stats()["backend"]
    tr = stats["channel0_trace_ns"]
    if a.json:
        with open("%s.rank%d.json" % (a.json, rank), "w") as f:
            json.dump({"args": vars(a), "ms": float(t), "trace_ns": tr}, f)
    if rank == 0:
        slots = a.slots or 4
        n = sum(1 for v in tr["loader_finished"] if v)
        print("%s, 2^%d elements, %d GPUs, %s: %.3f ms per job; %d tiles of channel 0 traced" %
              (a.mode, a.log2_numel, world, "multimem" if stats["multimem"] else "peer memory", float(t), n))
        print("  k   L_beg   L_fin   R_beg   R_fin   S_beg   S_fin |  Lwork  Rwork  Swork    L>R    R>S    S>L")
        us = lambda v: "%7.1f" % (v / 1e3)
        for k in list(range(min(n, a.rows))) + list(range(max(a.rows, n - 4), n)):
            lb, lf, rb, rf, sb, sf = [tr[key][k] for key in KEYS]
            nxt = tr["loader_began"][k + slots] - sf if k + slots < n else 0
            print("%3d" % k, us(lb), us(lf), us(rb), us(rf), us(sb), us(sf), "|",
                  us(lf - lb)[1:], us(rf - rb)[1:], us(sf - sb)[1:], us(rb - lf)[1:], us(sb - rf)[1:], us(nxt)[1:])
    ctx.stop()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
