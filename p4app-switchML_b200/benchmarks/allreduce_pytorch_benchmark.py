"""Allreduce benchmark through ``torch.distributed`` with a selectable backend.

Counterpart of the reference's benchmarks/allreduce_pytorch_benchmark/
allreduce_pytorch_benchmark.py: same options (-n/-r/-ip, --backend gloo|sml|mpi|nccl,
--tensor-numel 2^28, --tensor-type, --device, --num-jobs 10, --num-warmup-jobs 5,
--verify, --sync-every, --err, --random, --seed) and the same "#value#" report lines.
Two differences: the process group is taken from the torchrun environment when -r is not
given, and every synchronisation point waits for the device, so GPU numbers are real
(``work.wait()`` alone only orders the stream for GPU backends).
"""
import argparse
import os
import sys
import time

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
import switchml_b200.parallel.process_group  # noqa: E402,F401  (registers "sml")


def main():
    backends = ["sml", "sml_native", "gloo"] + (["mpi"] if dist.is_mpi_available() else []) + (["nccl"] if dist.is_nccl_available() else [])
    ap = argparse.ArgumentParser("AllReduce PyTorch Benchmark")
    ap.add_argument("-n", "--num-workers", type=int, default=int(os.environ.get("WORLD_SIZE", 1)))
    ap.add_argument("-r", "--rank", type=int, default=int(os.environ.get("RANK", 0)))
    ap.add_argument("-ip", "--rank0-ip", default=os.environ.get("MASTER_ADDR", "127.0.0.1"))
    ap.add_argument("-bk", "--backend", choices=backends, default="sml")
    ap.add_argument("-tn", "--tensor-numel", type=int, default=268435456)
    ap.add_argument("-tt", "--tensor-type", choices=["float", "int32"], default="float")
    ap.add_argument("-d", "--device", choices=["cpu", "gpu"], default="gpu" if torch.cuda.is_available() else "cpu")
    ap.add_argument("-nj", "--num-jobs", type=int, default=10)
    ap.add_argument("-nw", "--num-warmup-jobs", type=int, default=5)
    ap.add_argument("-v", "--verify", action="store_true")
    ap.add_argument("-sv", "--sync-every", type=int, default=1)
    ap.add_argument("-e", "--err", type=float, default=1.0)
    ap.add_argument("--random", action="store_true")
    ap.add_argument("--seed", type=int, default=None)
    a = ap.parse_args()
    if a.seed:
        torch.manual_seed(a.seed)
    gpu = a.device == "gpu"
    if gpu:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", a.rank)) % torch.cuda.device_count())
    device = "cuda" if gpu else "cpu"
    dtype = torch.float if a.tensor_type == "float" else torch.int32
    print("Allocating and initializing data..")
    if a.random:
        data = (torch.rand(a.tensor_numel, device=device) * 2 - 1).to(dtype) if dtype == torch.float else \
            torch.randint(-1000, 1000, (a.tensor_numel,), dtype=dtype, device=device)
    else:
        data = (torch.arange(a.tensor_numel, device=device) % 1000).to(dtype)
        data = data * (1 - 2 * (torch.arange(a.tensor_numel, device=device) % 2)).to(dtype)
    original = data.clone() if a.verify else None
    print("Initializing process group..")
    port = int(os.environ.get("MASTER_PORT", 23456))
    os.environ.setdefault("MASTER_ADDR", a.rank0_ip)
    os.environ.setdefault("MASTER_PORT", str(port))
    if a.backend == "sml_native":
        # The C++ c10d backend (lib/torch_switchml.so); it takes its settings from switchml.cfg /
        # SWITCHML_CONFIG, SWITCHML_RANK and SWITCHML_NUM_WORKERS like any C++ program.
        os.environ.setdefault("SWITCHML_RANK", str(a.rank))
        os.environ.setdefault("SWITCHML_NUM_WORKERS", str(a.num_workers))
        import switchml_b200.parallel.native_process_group  # noqa: F401
    dist.init_process_group(a.backend, rank=a.rank, world_size=a.num_workers,
                            init_method="tcp://%s:%d" % (a.rank0_ip, port))

    def sync():
        if gpu:
            torch.cuda.synchronize()

    print("Submitting %d warmup jobs.." % a.num_warmup_jobs)
    handles = [dist.all_reduce(data, async_op=True) for _ in range(a.num_warmup_jobs)]
    for h in handles:
        h.wait()
    sync()
    print("Warmup finished.\nSubmitting %d jobs.." % a.num_jobs)
    durations, goodput, rounds, handles = [], [], [], []
    every = a.sync_every or a.num_jobs
    begin = time.time_ns()
    for i in range(a.num_jobs):
        handles.append(dist.all_reduce(data, async_op=True))
        if len(handles) == every or i + 1 == a.num_jobs:
            for h in handles:
                h.wait()
            sync()
            durations.append(time.time_ns() - begin)
            goodput.append(a.tensor_numel * 32 * len(handles) / durations[-1])
            rounds.append("%d-%d" % (i - len(handles) + 1, i))
            print("Job(s) #%s# finished. Duration: #%d# ns Goodput: #%.3f# Gbps." % (rounds[-1], durations[-1], goodput[-1]))
            handles = []
            begin = time.time_ns()
    print("All jobs finished")
    if a.verify:
        factor = float(a.num_workers) ** (a.num_jobs + a.num_warmup_jobs)
        want = original.double() * factor
        if dtype == torch.int32:
            bad = (data.double() != want) & (want.abs() < 2 ** 31)
        else:
            bad = (data.double() - want).abs() > want.abs() * a.err / 100 + 1e-30
        n_bad = int(bad.sum())
        print("Results verified successfully." if n_bad == 0 else "Failed to verify data. Found %d errors." % n_bad)
    for name, fn in (("min", np.min), ("max", np.max), ("median", np.median), ("mean", np.mean), ("std", np.std)):
        print("%6s: Duration: #%11.0f# ns Goodput: #%7.2f# Gbps." % (name, fn(durations), fn(goodput)))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
