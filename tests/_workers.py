"""Child-process entry points used by the multi-rank tests (spawned with
multiprocessing 'spawn', so this module must be importable on its own)."""
import os
import sys
import traceback

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def rank_data(rank, numel, dtype="float32", seed=0):
    import numpy as np
    rng = np.random.default_rng(seed * 1000 + rank)
    if dtype == "int32":
        return rng.integers(-2 ** 20, 2 ** 20, size=numel, dtype=np.int32)
    return rng.standard_normal(numel).astype(np.float32)


def udp_worker(rank, n, ctl_port, udp_port, numel, dtype, threads, packet_numel, drop, q, jobs=2,
               timeout_ms=10.0):
    """One SwitchML worker over the software switch; reports its result through `q`."""
    try:
        import numpy as np
        import switchml_b200 as sml
        ctx = sml.Context.get_instance()
        cfg = sml.make_config("udp", rank=rank, num_workers=n, packet_numel=packet_numel,
                              num_worker_threads=threads, max_outstanding_packets=32 * threads,
                              controller_port=ctl_port, switch_port=udp_port, worker_port=0,
                              timeout=timeout_ms)
        assert ctx.start(cfg), "start failed"
        if drop and rank == 0:
            # the operator CLI path: tell the switch to lose packets both ways
            from switchml_b200.utils.cli import controller_command
            controller_command("127.0.0.1", ctl_port, "SET drop %g %g 99" % (drop, drop))
        outs = []
        for j in range(jobs):
            x = rank_data(rank, numel, dtype, seed=j)
            y = np.empty_like(x)
            job = ctx.all_reduce_async(x, y)
            st = job.wait(timeout_ms=60000)
            assert st == sml.JobStatus.FINISHED, "job %d ended %s: %s" % (j, st, job.error())
            outs.append(y)
        stats = ctx.get_stats()
        switch_stats = None
        if rank == 0:
            from switchml_b200.utils.cli import controller_command
            switch_stats = controller_command("127.0.0.1", ctl_port, "SHOW statistics")
        ctx.stop()
        q.put((rank, "ok", outs, stats, switch_stats))
    except Exception:
        q.put((rank, "error", traceback.format_exc(), None, None))
