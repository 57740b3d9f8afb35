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
               timeout_ms=10.0, msg_numel=0):
    """One SwitchML worker over the software switch; reports its result through `q`."""
    try:
        import numpy as np
        import switchml_b200 as sml
        ctx = sml.Context.get_instance()
        cfg = sml.make_config("udp", rank=rank, num_workers=n, packet_numel=packet_numel,
                              num_worker_threads=threads, max_outstanding_packets=32 * threads,
                              controller_port=ctl_port, switch_port=udp_port, worker_port=0,
                              timeout=timeout_ms, msg_numel=msg_numel)
        assert ctx.start(cfg), "start failed"
        if drop and rank == 0:
            # the operator CLI path: tell the switch to lose packets both ways
            from switchml_b200.utils.cli import controller_command
            controller_command("127.0.0.1", ctl_port, "SET drop %g %g 99" % (drop, drop))
        # uint8 flags, the way PyTorch reduces them: summed as int32, low byte returned
        flags = ((np.arange(1000) * (rank + 3)) % 256).astype(np.uint8)
        summed = np.zeros_like(flags)
        ctx.all_reduce(flags, summed)
        want = (sum(((np.arange(1000) * (r + 3)) % 256) for r in range(n)) % 256).astype(np.uint8)
        assert np.array_equal(summed, want), "uint8 allreduce"
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
            stats["switch_tables"] = {t: controller_command("127.0.0.1", ctl_port, "SHOW " + t)
                                      for t in ("ports", "forwarding", "qp", "dropped", "address", "workers")}
        ctx.stop()
        q.put((rank, "ok", outs, stats, switch_stats))
    except Exception:
        q.put((rank, "error", traceback.format_exc(), None, None))


def cuda_worker(rank, n, ctl_port, transport, mode, q, heap_mb=64, launch="inline"):
    """One rank of the cuda backend on GPU `rank`; runs a fixed list of cases and checks
    every result locally against the CPU oracle / a float64 sum."""
    try:
        import numpy as np
        import torch
        import switchml_b200 as sml
        from switchml_b200.ops.oracle import quant_allreduce_oracle, int_allreduce_oracle
        torch.cuda.set_device(rank)
        ctx = sml.Context.get_instance()
        cfg = sml.make_config("cuda", rank=rank, num_workers=n, packet_numel=256, device=rank,
                              controller_port=ctl_port, transport=transport, mode=mode,
                              symm_heap_mb=heap_mb, launch=launch, wait_timeout_ms=20000,
                              slot_bytes=65536, trace=True)
        assert ctx.start(cfg), "start failed"
        report = {"multimem": ctx.uses_multimem(), "cases": 0}
        sizes = [1, 255, 4097, 65536, 70001, (1 << 20) + 3, 5 * (1 << 20)]
        for numel in sizes:
            xs = [rank_data(r, numel, "float32", seed=numel % 97) for r in range(n)]
            x = torch.from_numpy(xs[rank]).cuda()
            y = torch.empty_like(x)
            job = ctx.all_reduce_async(x, y)
            assert job.wait(60000) == sml.JobStatus.FINISHED, job.error()
            got = y.cpu().numpy()
            if mode == "int32_quant":
                want = quant_allreduce_oracle(xs, 256)
                assert np.array_equal(got, want), "quant mismatch at numel %d" % numel
            else:
                exact = sum(a.astype(np.float64) for a in xs)
                assert np.max(np.abs(got - exact)) < 1e-4, "float sum mismatch at numel %d" % numel
            report["cases"] += 1
            # int32
            xi = [rank_data(r, numel, "int32", seed=1) for r in range(n)]
            t = torch.from_numpy(xi[rank]).cuda()
            ctx.all_reduce(t)
            assert np.array_equal(t.cpu().numpy(), int_allreduce_oracle(xi)), "int mismatch at %d" % numel
            report["cases"] += 1
            # uint8: summed as int32, low byte returned; out of place from an odd offset
            xu = [np.random.default_rng(7 * numel + r).integers(0, 256, numel + 3, dtype=np.uint8) for r in range(n)]
            tu = torch.from_numpy(xu[rank]).cuda()
            ou = torch.full((numel + 5,), 77, dtype=torch.uint8, device="cuda")
            ctx.all_reduce(tu[3:], ou[1:1 + numel])
            want_u = (sum(a[3:].astype(np.int64) for a in xu) & 0xff).astype(np.uint8)
            assert np.array_equal(ou[1:1 + numel].cpu().numpy(), want_u), "uint8 mismatch at %d" % numel
            assert int(ou[0]) == 77 and bool((ou[1 + numel:] == 77).all()), "uint8 wrote outside its output"
            assert np.array_equal(tu.cpu().numpy(), xu[rank]), "uint8 touched its input"
            report["cases"] += 1
            # bf16 in place
            xb = [torch.from_numpy(a).bfloat16() for a in xs]
            tb = xb[rank].cuda()
            ctx.all_reduce(tb)
            if mode == "int32_quant":
                want = torch.from_numpy(quant_allreduce_oracle([a.float().numpy() for a in xb], 256)).bfloat16()
                assert torch.equal(tb.cpu(), want), "bf16 quant mismatch at %d" % numel
            else:
                exact = sum(a.double() for a in xb)
                assert torch.allclose(tb.cpu().double(), exact, rtol=2e-2, atol=2e-2), "bf16 sum mismatch"
            report["cases"] += 1
        # zero-copy path: tensors in the symmetric heap, reduced in place and out of place
        if mode == "float_sum":
            for numel in (1000, 300007, 4 * (1 << 20)):
                xs = [rank_data(r, numel, "float32", seed=5) for r in range(n)]
                a = ctx.symmetric_empty(numel, torch.float32)
                b = ctx.symmetric_empty(numel, torch.float32)
                guard = ctx.symmetric_empty(64, torch.float32)
                guard.fill_(123.0)
                a.copy_(torch.from_numpy(xs[rank]))
                ctx.all_reduce(a, b)
                exact = sum(v.astype(np.float64) for v in xs)
                assert np.max(np.abs(b.cpu().numpy() - exact)) < 1e-4, "zero-copy mismatch at %d" % numel
                assert np.array_equal(a.cpu().numpy(), xs[rank]), "zero-copy touched its input"
                ctx.all_reduce(a)
                assert np.max(np.abs(a.cpu().numpy() - exact)) < 1e-4, "in-place zero-copy mismatch"
                assert float(guard.min()) == 123.0 and float(guard.max()) == 123.0, "wrote past the tensor"
                report["cases"] += 2
            ctx.symmetric_reset()
        # tcgen05 weight-gradient GEMM with the cross-GPU reduce fused into the kernel
        if mode == "float_sum":
            from switchml_b200.ops.wgrad import FusedWgrad
            for (K, M, N, policy) in ((256, 384, 520, "fused"), (64, 1024, 2048, "fused"), (1024, 128, 256, "split"),
                                      (32, 1024, 2048, "gather"), (200, 384, 520, "gather"), (64, 2048, 4096, "auto")):
                fw = FusedWgrad(ctx, M, N, scale=1.0 / n, policy=policy)
                report["fused_in_kernel"] = fw.fused
                for it in range(3):
                    g = torch.Generator(device="cuda").manual_seed(1000 * rank + it)
                    dy = torch.randn(K, M, device="cuda", generator=g).bfloat16()
                    x = torch.randn(K, N, device="cuda", generator=g).bfloat16()
                    got = fw.run(dy, x).clone()
                    ref = (dy.float().t() @ x.float()).contiguous()
                    ctx.all_reduce(ref.view(-1))
                    ref /= n
                    torch.cuda.synchronize()
                    assert int(fw.error.item()) == 0, "fused wgrad: a wait gave up"
                    err = float((got - ref).abs().max())
                    assert err < 2e-2 * (K ** 0.5), "fused wgrad mismatch %g at %s it %d" % (err, (K, M, N), it)
                    report["cases"] += 1
            ctx.symmetric_reset()
        # CUDA graph: capture a small (one-barrier) and a large (streamed) job, replay with new data
        if launch == "inline":
            gs = torch.full((20_000,), 0.0, device="cuda")
            gl = torch.full((2_500_003,), 0.0, device="cuda")
            os_, ol_ = torch.empty_like(gs), torch.empty_like(gl)
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.graph(graph, stream=side):
                ctx.all_reduce_async(gs, os_)
                ctx.all_reduce_async(gl, ol_)
            for it in range(4):
                gs.fill_(rank + 1.0 + it)
                gl.fill_(0.5 * (rank + 1) + it)
                graph.replay()
                torch.cuda.synchronize()
                want_s = sum(r + 1.0 + it for r in range(n))
                want_l = sum(0.5 * (r + 1) + it for r in range(n))
                assert abs(float(os_.min()) - want_s) < 1e-4 and abs(float(os_.max()) - want_s) < 1e-4, "graph small"
                assert abs(float(ol_.min()) - want_l) < 1e-4 and abs(float(ol_.max()) - want_l) < 1e-4, "graph large"
                report["cases"] += 1
            t = torch.full((50_000,), float(rank), device="cuda")   # ordinary job after the replays
            ctx.all_reduce(t)
            assert float(t[0]) == float(sum(range(n))), "job after graph replays"
        # DDP wrapper: overlapped, bucketed reduction must equal the mean of the local gradients
        if mode == "float_sum":
            from switchml_b200.parallel.ddp import DistributedDataParallel
            def make(seed):
                torch.manual_seed(seed)
                return torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.ReLU(), torch.nn.Linear(512, 512),
                                           torch.nn.ReLU(), torch.nn.Linear(512, 16)).cuda()
            model = make(rank)          # every rank starts from other weights ...
            ddp = DistributedDataParallel(model, ctx, bucket_mb=0.5, overlap=True)
            ref_model = make(0)         # ... and the wrapper hands out rank 0's, exactly in float_sum mode
            for p, rp in zip(model.parameters(), ref_model.parameters()):
                assert torch.equal(p, rp), "parameters were not broadcast from rank 0"
            report["cases"] += 1
            for it in range(3):
                ddp.zero_grad()
                xs_all = [torch.randn(32, 256, generator=torch.Generator().manual_seed(10 * r + it)) for r in range(n)]
                ddp(xs_all[rank].cuda()).square().mean().backward()
                torch.cuda.synchronize()
                ref_model.zero_grad()
                for r in range(n):
                    (ref_model(xs_all[r].cuda()).square().mean()).backward()
                for p, rp in zip(model.parameters(), ref_model.parameters()):
                    assert torch.allclose(p.grad, rp.grad, rtol=1e-4, atol=1e-6), "DDP gradient != sum of local gradients"
                report["cases"] += 1
        # the per-tile trace of channel 0: one streamed job, then its timeline must be ordered
        x = torch.from_numpy(rank_data(rank, 6 << 20, "float32", seed=5)).cuda()
        job = ctx.all_reduce_async(x, torch.empty_like(x))
        assert job.wait(60000) == sml.JobStatus.FINISHED, job.error()
        report["stats"] = ctx.get_stats()
        tr = report["stats"]["backend"]["channel0_trace_ns"]
        tiles = sum(1 for v in tr["loader_finished"] if v)
        assert tiles >= 2, "a 24 MiB job has several tiles per channel"
        for role in ("loader", "reducer", "storer"):
            began, finished = tr[role + "_began"][:tiles], tr[role + "_finished"][:tiles]
            assert all(0 < b <= f for b, f in zip(began, finished)), role + ": a tile finished before it began"
            assert all(finished[k] <= began[k + 1] for k in range(tiles - 1)), role + ": tiles out of order"
        assert all(l <= r for l, r in zip(tr["loader_finished"][:tiles], tr["reducer_finished"][:tiles])), \
            "a tile was reduced before it was loaded"
        report["cases"] += 1
        ctx.stop()
        q.put((rank, "ok", report))
    except Exception:
        q.put((rank, "error", traceback.format_exc()))


def pg_worker(rank, n, port, q):
    """torch.distributed with backend "sml" on CPU (udp transport): plain all_reduce and a
    DistributedDataParallel step, compared with the sum computed locally."""
    try:
        import torch
        import torch.distributed as dist
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        import switchml_b200.parallel.process_group  # noqa: F401
        dist.init_process_group("sml", rank=rank, world_size=n, init_method="tcp://127.0.0.1:%d" % port)
        t = torch.arange(10000, dtype=torch.float32) * (rank + 1)
        dist.all_reduce(t)
        want = torch.arange(10000, dtype=torch.float32) * sum(r + 1 for r in range(n))
        assert torch.allclose(t, want, rtol=1e-6), "float allreduce"
        ti = torch.full((1000,), rank + 1, dtype=torch.int32)
        work = dist.all_reduce(ti, async_op=True)
        work.wait()
        assert int(ti[0]) == sum(r + 1 for r in range(n)), "int allreduce"
        tu = torch.full((77,), 250 + rank, dtype=torch.uint8)
        dist.all_reduce(tu)
        assert int(tu[0]) == sum(250 + r for r in range(n)) % 256, "uint8 allreduce"
        d = torch.ones(4, dtype=torch.float64) * rank          # unsupported dtype: Gloo fallback
        dist.all_reduce(d)
        assert float(d[0]) == sum(range(n)), "fallback"
        torch.manual_seed(0)
        model = torch.nn.Linear(32, 8)
        ddp = torch.nn.parallel.DistributedDataParallel(model)
        x = torch.randn(16, 32, generator=torch.Generator().manual_seed(rank))
        ddp(x).square().mean().backward()
        g = model.weight.grad.clone()
        gl = [torch.zeros_like(g) for _ in range(n)]
        dist.all_gather(gl, g)
        assert all(torch.allclose(gl[0], o, atol=1e-6) for o in gl), "DDP gradients differ across ranks"
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok", None))
    except Exception:
        q.put((rank, "error", traceback.format_exc()))


def ddp_hook_worker(rank, n, ctl_port, dist_port, q):
    """PyTorch DDP (NCCL process group for its own bookkeeping) with the SwitchML
    communication hook doing the gradient reduction; compared with gradients computed
    from all ranks' data on one device."""
    try:
        import torch
        import torch.distributed as dist
        import switchml_b200 as sml
        from switchml_b200.parallel.ddp_hook import SwitchMLHookState, switchml_allreduce_hook
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=n, init_method="tcp://127.0.0.1:%d" % dist_port,
                                device_id=torch.device("cuda", rank))
        ctx = sml.Context.get_instance()
        assert ctx.start(sml.make_config("cuda", rank=rank, num_workers=n, packet_numel=256, device=rank,
                                         controller_port=ctl_port, mode="float_sum", launch="inline",
                                         average=True, wait_timeout_ms=20000))
        torch.manual_seed(0)
        def make():
            return torch.nn.Sequential(torch.nn.Linear(128, 1024), torch.nn.ReLU(), torch.nn.Linear(1024, 1024),
                                       torch.nn.ReLU(), torch.nn.Linear(1024, 8)).cuda()
        model, ref = make(), make()
        ref.load_state_dict(model.state_dict())
        ddp = torch.nn.parallel.DistributedDataParallel(model, device_ids=[rank], bucket_cap_mb=1)
        ddp.register_comm_hook(SwitchMLHookState(ctx), switchml_allreduce_hook)
        for it in range(3):
            xs = [torch.randn(16, 128, generator=torch.Generator().manual_seed(7 * r + it)) for r in range(n)]
            ddp.zero_grad()
            ddp(xs[rank].cuda()).square().mean().backward()
            torch.cuda.synchronize()
            ref.zero_grad()
            for r in range(n):
                (ref(xs[r].cuda()).square().mean() / n).backward()
            for p, rp in zip(model.parameters(), ref.parameters()):
                assert torch.allclose(p.grad, rp.grad, rtol=1e-4, atol=1e-6), "hook gradient != mean of local gradients"
        ctx.stop()
        dist.destroy_process_group()
        q.put((rank, "ok", None))
    except Exception:
        q.put((rank, "error", traceback.format_exc()))


def absent_peer_worker(rank, n, ctl_port, q):
    """Failure detection without any GPU fault: after one common job, the last rank
    simply stops submitting. The others' next job runs into the bounded device wait, fails
    with a timeout status, and their context remains usable for reading statistics and for
    an orderly stop. Peer memory only (no multicast objects are bound while a rank is
    'gone')."""
    try:
        import time
        import torch
        import switchml_b200 as sml
        torch.cuda.set_device(rank)
        ctx = sml.Context.get_instance()
        assert ctx.start(sml.make_config("cuda", rank=rank, num_workers=n, packet_numel=256, device=rank,
                                         controller_port=ctl_port, transport="p2p", mode="float_sum",
                                         launch="worker", wait_timeout_ms=400))
        x = torch.ones(1 << 20, device="cuda")
        ctx.all_reduce(x)                       # everybody takes part: works
        assert float(x[0]) == float(n)
        info = {}
        if rank == n - 1:
            time.sleep(3.0)                     # "absent": submits nothing while the others wait
        else:
            t0 = time.time()
            job = ctx.all_reduce_async(x)
            st = job.wait(timeout_ms=20000)
            info["status"] = st.name
            info["error"] = job.error()
            info["seconds"] = time.time() - t0
            stats = ctx.get_stats()
            info["jobs_failed"] = stats["jobs_failed"]
            info["device_timeouts"] = stats["backend"]["device_timeouts"]
            torch.cuda.synchronize()            # the device still answers
            info["alive"] = float((x * 0 + 1).sum()) == float(x.numel())
        ctx.stop()
        q.put((rank, "ok", info))
    except Exception:
        q.put((rank, "error", traceback.format_exc()))


def native_pg_worker(rank, n, port, ctl_port, udp_port, cfg_dir, q):
    """The native c10d backend "sml_native" (C++ extension) on CPU ranks over udp."""
    try:
        import torch
        import torch.distributed as dist
        import switchml_b200 as sml
        path = os.path.join(cfg_dir, "switchml-rank%d.cfg" % rank)
        with open(path, "w") as f:
            f.write(sml.make_config("udp", rank=rank, num_workers=n, packet_numel=64, num_worker_threads=2,
                                    max_outstanding_packets=64, controller_port=ctl_port, switch_port=udp_port,
                                    worker_port=0))
        os.environ["SWITCHML_CONFIG"] = path
        import switchml_b200.parallel.native_process_group  # noqa: F401
        dist.init_process_group("sml_native", rank=rank, world_size=n, init_method="tcp://127.0.0.1:%d" % port)
        t = torch.arange(5000, dtype=torch.float32) * (rank + 1)
        dist.all_reduce(t)
        assert torch.allclose(t, torch.arange(5000, dtype=torch.float32) * sum(r + 1 for r in range(n)), rtol=1e-6)
        ti = torch.full((333,), rank + 5, dtype=torch.int32)
        w = dist.all_reduce(ti, async_op=True)
        fut = w.get_future()
        fut.wait()
        assert int(ti[7]) == sum(r + 5 for r in range(n))
        tu = torch.full((100,), 200 + rank, dtype=torch.uint8)    # flags as PyTorch reduces them: modulo 256
        dist.all_reduce(tu)
        assert int(tu[3]) == sum(200 + r for r in range(n)) % 256
        try:
            dist.all_reduce(torch.ones(4, dtype=torch.float64))
            raised = False
        except RuntimeError:
            raised = True
        assert raised, "float64 must be refused"
        try:
            dist.broadcast(t, 0)
            raised = False
        except RuntimeError:
            raised = True
        assert raised, "the native backend implements allreduce only"
        dist.destroy_process_group()
        q.put((rank, "ok", None))
    except Exception:
        q.put((rank, "error", traceback.format_exc()))


def native_pg_cuda_worker(rank, n, port, ctl_port, cfg_dir, q):
    """The native c10d backend on GPUs: CUDA tensors are reduced in place on the device."""
    try:
        import torch
        import torch.distributed as dist
        import switchml_b200 as sml
        torch.cuda.set_device(rank)
        path = os.path.join(cfg_dir, "switchml-rank%d.cfg" % rank)
        with open(path, "w") as f:
            f.write(sml.make_config("cuda", rank=rank, num_workers=n, packet_numel=256, device=rank,
                                    controller_port=ctl_port, mode="float_sum", launch="inline",
                                    wait_timeout_ms=20000))
        os.environ["SWITCHML_CONFIG"] = path
        import switchml_b200.parallel.native_process_group  # noqa: F401
        dist.init_process_group("sml_native", rank=rank, world_size=n, init_method="tcp://127.0.0.1:%d" % port)
        for numel in (1000, 300001, 1 << 22):
            t = torch.full((numel,), float(rank + 1), device="cuda")
            dist.all_reduce(t)
            torch.cuda.synchronize()
            assert float(t.min()) == float(t.max()) == float(sum(r + 1 for r in range(n))), numel
        tb = torch.ones(70000, device="cuda", dtype=torch.bfloat16)
        work = dist.all_reduce(tb, async_op=True)
        work.get_future().wait()
        torch.cuda.synchronize()
        assert float(tb.float().mean()) == float(n)
        dist.destroy_process_group()
        q.put((rank, "ok", None))
    except Exception:
        q.put((rank, "error", traceback.format_exc()))


def ddp_broadcast_worker(rank, n, ctl_port, udp_port, q):
    """DDP wrapper over the UDP backend on CPU tensors: ranks start from different weights,
    the wrapper gives everybody rank 0's; then one synchronised step and one accumulated
    (no_sync) step are compared with gradients computed from all ranks' data."""
    try:
        import torch
        import switchml_b200 as sml
        from switchml_b200.parallel.ddp import DistributedDataParallel
        ctx = sml.Context.get_instance()
        assert ctx.start(sml.make_config("udp", rank=rank, num_workers=n, packet_numel=64, num_worker_threads=2,
                                         max_outstanding_packets=64, controller_port=ctl_port, switch_port=udp_port,
                                         worker_port=0))

        def make(seed):
            torch.manual_seed(seed)
            m = torch.nn.Sequential(torch.nn.Linear(12, 32), torch.nn.BatchNorm1d(32), torch.nn.Tanh(),
                                    torch.nn.Linear(32, 4))
            m[1].num_batches_tracked.fill_(seed)
            return m
        model = make(100 + rank)                      # every rank starts somewhere else
        ddp = DistributedDataParallel(model, ctx, bucket_mb=0.001)
        state = {k: v.clone() for k, v in model.state_dict().items()}
        xs = [torch.randn(6, 12, generator=torch.Generator().manual_seed(50 + r)) for r in range(n)]
        # one synchronised step
        ddp.zero_grad()
        ddp(xs[rank]).square().mean().backward()
        g1 = [p.grad.clone() for p in model.parameters()]
        # accumulate one local pass, then a synchronised one: reduced gradient = sum over ranks of both passes
        ddp.zero_grad()
        with ddp.no_sync():
            ddp(xs[rank]).square().mean().backward()
        local_only = [p.grad.clone() for p in model.parameters()]
        submitted = ctx.get_stats()["jobs_submitted"]
        ddp(2 * xs[rank]).square().mean().backward()
        g2 = [p.grad.clone() for p in model.parameters()]
        assert ctx.get_stats()["jobs_submitted"] - submitted == len(ddp.buckets.buckets)
        ctx.stop()
        # numpy, not tensors: a tensor in a queue is a handle to shared memory of this process
        q.put((rank, "ok", {"state": {k: v.numpy() for k, v in state.items()}, "g1": [g.numpy() for g in g1],
                            "g2": [g.numpy() for g in g2], "local": [g.numpy() for g in local_only]}))
    except Exception:
        q.put((rank, "error", traceback.format_exc()))


def stop_during_loss_worker(rank, n, ctl_port, udp_port, q):
    """Total packet loss after one good job: the next job cannot finish, its retransmission
    timers keep firing, and Context.stop() fails it in bounded time instead of hanging."""
    try:
        import threading
        import time
        import numpy as np
        import switchml_b200 as sml
        from switchml_b200.utils.cli import controller_command
        ctx = sml.Context.get_instance()
        assert ctx.start(sml.make_config("udp", rank=rank, num_workers=n, packet_numel=64, num_worker_threads=2,
                                         max_outstanding_packets=64, controller_port=ctl_port, switch_port=udp_port,
                                         worker_port=0, timeout=5))
        x = np.ones(100000, dtype=np.float32)
        ctx.all_reduce(x)
        assert float(x[0]) == float(n)
        if rank == 0:
            controller_command("127.0.0.1", ctl_port, "SET drop 1.0 1.0 1")
        time.sleep(0.3)                       # both ranks submit after the switch went deaf
        job = ctx.all_reduce_async(x)
        early = job.wait(timeout_ms=800)      # still running: nothing comes back
        seen = {}
        waiter = threading.Thread(target=lambda: seen.update(status=job.wait()))
        waiter.start()
        t0 = time.time()
        ctx.stop()
        waiter.join(10)
        timeouts = sum(ctx.get_stats()["timeouts"])   # the worker threads report when their slice ends
        q.put((rank, "ok", {"early": int(early), "final": int(seen.get("status", -1)), "error": job.error(),
                            "stop_seconds": time.time() - t0, "timeouts": timeouts}))
    except Exception:
        q.put((rank, "error", traceback.format_exc()))


def broadcast_udp_worker(rank, n, ctl_port, udp_port, q):
    """Context.broadcast over the UDP backend: exact for int32, the same rounded values on
    every rank for float32; bad arguments fail the job without hurting the context."""
    try:
        import numpy as np
        import switchml_b200 as sml
        ctx = sml.Context.get_instance()
        assert ctx.start(sml.make_config("udp", rank=rank, num_workers=n, packet_numel=64, num_worker_threads=2,
                                         max_outstanding_packets=64, controller_port=ctl_port, switch_port=udp_port,
                                         worker_port=0))
        out = {}
        for root in range(n):
            xi = np.arange(5000, dtype=np.int32) * (rank + 1) - 77 * rank
            ctx.broadcast(xi, root)
            out["int%d" % root] = xi
            xf = np.random.default_rng(100 + rank).standard_normal(3333).astype(np.float32)
            ctx.broadcast(xf, root)
            out["float%d" % root] = xf
        bad = ctx.broadcast_async(np.zeros(4, dtype=np.float32), root=n)
        assert bad.wait(5000) == sml.JobStatus.FAILED and "not a rank" in bad.error()
        bad = ctx.broadcast_async(np.zeros(4, dtype=np.uint8), root=0)
        assert bad.wait(5000) == sml.JobStatus.FAILED
        x = np.full(100, rank + 1.0, dtype=np.float32)
        ctx.all_reduce(x)                                   # still in step with the others
        assert float(x[0]) == sum(r + 1.0 for r in range(n))
        ctx.stop()
        q.put((rank, "ok", out))
    except Exception:
        q.put((rank, "error", traceback.format_exc()))


def broadcast_cuda_worker(rank, n, ctl_port, mode, q):
    """Context.broadcast on GPUs: the root's tensor reaches every rank, also when the context
    averages its allreduces and also for tensors of the symmetric heap."""
    try:
        import torch
        import switchml_b200 as sml
        torch.cuda.set_device(rank)
        ctx = sml.Context.get_instance()
        assert ctx.start(sml.make_config("cuda", rank=rank, num_workers=n, packet_numel=256, device=rank,
                                         controller_port=ctl_port, mode=mode, launch="inline", average=True,
                                         symm_heap_mb=16, wait_timeout_ms=20000))
        for root in range(n):
            for numel in (1, 1000, 300007, (1 << 21) + 5):
                g = torch.Generator().manual_seed(1000 * root + numel)        # what the root holds
                want = torch.randn(numel, generator=g)
                x = want.cuda() if rank == root else torch.full((numel,), float(rank + 5), device="cuda")
                ctx.broadcast(x, root)
                torch.cuda.synchronize()
                if mode == "float_sum":
                    assert torch.equal(x.cpu(), want), "float broadcast root %d numel %d" % (root, numel)
                else:
                    assert torch.allclose(x.cpu(), want, rtol=0, atol=2.0 ** -20 * float(want.abs().max()) + 1e-30)
                if rank == root:
                    xi = (torch.arange(numel, dtype=torch.int32) * 7 - root).cuda()
                else:
                    xi = torch.zeros(numel, dtype=torch.int32, device="cuda") - 1
                ctx.broadcast(xi, root)
                torch.cuda.synchronize()
                assert torch.equal(xi.cpu(), torch.arange(numel, dtype=torch.int32) * 7 - root), "int broadcast"
            s = ctx.symmetric_empty(70001, torch.float32)
            s.copy_(torch.full((70001,), 3.25 if rank == root else -1.0))
            ctx.broadcast(s, root)
            torch.cuda.synchronize()
            assert float(s.min()) == 3.25 and float(s.max()) == 3.25, "symmetric broadcast"
            ctx.symmetric_reset()
        y = torch.full((1000,), float(rank + 1), device="cuda")
        ctx.all_reduce(y)                                   # allreduces still average
        torch.cuda.synchronize()
        assert abs(float(y[0]) - sum(r + 1.0 for r in range(n)) / n) < 1e-5
        ctx.stop()
        q.put((rank, "ok", None))
    except Exception:
        q.put((rank, "error", traceback.format_exc()))


def ddp_hook_cpu_worker(rank, n, ctl_port, udp_port, dist_port, q):
    """PyTorch DDP on CPU tensors (Gloo for its own bookkeeping) with the SwitchML comm hook
    over the UDP backend: the gradients must be the mean of the workers' local gradients."""
    try:
        import torch
        import torch.distributed as dist
        import switchml_b200 as sml
        from switchml_b200.parallel.ddp_hook import SwitchMLHookState, switchml_allreduce_hook
        dist.init_process_group("gloo", rank=rank, world_size=n, init_method="tcp://127.0.0.1:%d" % dist_port)
        ctx = sml.Context.get_instance()
        assert ctx.start(sml.make_config("udp", rank=rank, num_workers=n, packet_numel=64, num_worker_threads=2,
                                         max_outstanding_packets=64, controller_port=ctl_port, switch_port=udp_port,
                                         worker_port=0))

        def make():
            torch.manual_seed(0)
            return torch.nn.Sequential(torch.nn.Linear(16, 64), torch.nn.ReLU(), torch.nn.Linear(64, 4))
        model, ref = make(), make()
        ddp = torch.nn.parallel.DistributedDataParallel(model, bucket_cap_mb=0.005)
        state = SwitchMLHookState(ctx)
        assert state.divide and state.num_workers == n
        ddp.register_comm_hook(state, switchml_allreduce_hook)
        for it in range(2):
            xs = [torch.randn(8, 16, generator=torch.Generator().manual_seed(3 * r + it)) for r in range(n)]
            ddp.zero_grad()
            ddp(xs[rank]).square().mean().backward()
            ref.zero_grad()
            for r in range(n):
                (ref(xs[r]).square().mean() / n).backward()
            for p, rp in zip(model.parameters(), ref.parameters()):
                assert torch.allclose(p.grad, rp.grad, rtol=1e-4, atol=1e-6), "hook gradient != mean of local gradients"
        ctx.stop()
        dist.destroy_process_group()
        q.put((rank, "ok", None))
    except Exception:
        q.put((rank, "error", traceback.format_exc()))
