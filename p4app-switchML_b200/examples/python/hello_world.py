"""The C++ hello_world (examples/hello_world/main.cc) through the Python binding: eight
asynchronous allreduces of 2^15 floats each, out of place, then a check that every output is
the sum over the workers and that the inputs were left alone.

    python examples/python/hello_world.py                      # dummy backend, one process
    SWITCHML_CONFIG=/path/to/switchml.cfg python examples/python/hello_world.py --from-file
    torchrun --nproc-per-node 2 examples/python/hello_world.py --backend cuda

With the dummy backend every process sees its own data multiplied by num_workers; with the
udp or cuda backend the processes (one per rank) really exchange data.
"""
import argparse
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))))
import switchml_b200 as sml  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="dummy", choices=["dummy", "udp", "cuda"])
    ap.add_argument("--from-file", action="store_true", help="load switchml.cfg (search order of the library)")
    ap.add_argument("--num-tensors", type=int, default=8)
    ap.add_argument("--numel", type=int, default=1 << 15)
    a = ap.parse_args(argv)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    ctx = sml.Context.get_instance()
    if a.from_file:
        ctx.start_from_file()
    else:
        extra = {"bandwidth": 0} if a.backend == "dummy" else {}
        if a.backend == "cuda":
            extra.update(mode="float_sum", device=int(os.environ.get("LOCAL_RANK", "0")))
        ctx.start(sml.make_config(a.backend, rank=rank, num_workers=max(world, 1 if a.backend != "dummy" else 2),
                                  **extra))
    workers = int([l for l in ctx.config_dump().splitlines() if l.strip().startswith("num_workers")][0].split("=")[1])
    on_gpu = "backend = cuda" in ctx.config_dump()

    ins = [np.full(a.numel, float(i + 1), dtype=np.float32) for i in range(a.num_tensors)]
    if on_gpu:
        import torch
        torch.cuda.set_device(ctx.device())
        src = [torch.from_numpy(x).cuda() for x in ins]
        dst = [torch.zeros_like(x) for x in src]
    else:
        src, dst = ins, [np.zeros_like(x) for x in ins]
    jobs = [ctx.all_reduce_async(s, d) for s, d in zip(src, dst)]   # all in flight at once
    ctx.wait_for_all_jobs()
    for i, (job, s, d) in enumerate(zip(jobs, src, dst)):
        assert job.status() == sml.JobStatus.FINISHED, job.error()
        out = d.cpu().numpy() if on_gpu else d
        keep = s.cpu().numpy() if on_gpu else s
        assert np.allclose(out, (i + 1.0) * workers, rtol=1e-2), "tensor %d: wrong sum" % i
        assert np.array_equal(keep, ins[i]), "tensor %d: the input was modified" % i
    print("Data verified successfully: %d tensors of %d elements, %d workers, backend %s"
          % (a.num_tensors, a.numel, workers, "cuda" if on_gpu else a.backend))
    print(ctx.stats_report())
    ctx.stop()


if __name__ == "__main__":
    main()
