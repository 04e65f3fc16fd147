"""Worker entry points for the multi-process parameter-server tests (importable for spawn)."""
import os
import sys
import traceback

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def make_cfg(world, base_port, **kw):
    from geeps_b200.utils.config import GeePsConfig
    cfg = GeePsConfig(host_list=["127.0.0.1"] * world, port_list=[base_port + 10 * r for r in range(world)], **kw)
    return cfg


def helloworld_worker(rank, world, base_port, slack, clocks, q, kw):
    """Every clock: read all rows, add +1.0 to every element (config 'helloworld-shaped')."""
    try:
        import torch
        from geeps_b200.parallel.ps import GeePs
        cfg = make_cfg(world, base_port, **kw)
        g = GeePs(rank, cfg)
        rows = list(range(kw.get("_rows", 1000))) if False else list(range(1000))
        r = g.virtual_read(0, rows, slack)
        u = g.virtual_pre_update(0, rows)
        pr = g.virtual_post_read(r)
        up = g.virtual_update(u)
        g.virtual_clock()
        g.finish_virtual_iteration()
        b = g.pre_update(u)
        b.zero_()
        g.update(up)
        g.clock()
        g.start_iterations()
        seen = []
        extra = slack + 1
        for c in range(clocks + extra):
            x = g.read(r, asynchronous=False)
            lo, hi = float(x.min()), float(x.max())
            seen.append((g.clock_value, lo, hi))
            b = g.pre_update(u)
            g.post_read(pr)
            b.fill_(1.0 if c < clocks else 0.0)
            g.update(up)
            g.clock()
        x = g.read(r, asynchronous=False)
        final = (float(x.min()), float(x.max()))
        stats = g.get_stats()
        g.shutdown()
        g.close()
        q.put((rank, "ok", final, seen, stats["client"]["max_staleness"], stats))
    except Exception as e:  # pragma: no cover
        q.put((rank, "error", repr(e) + traceback.format_exc(), None, None, None))


def placement_worker(rank, world, base_port, policy, q, kw):
    """Exercises the shards' placement service (FIND_ROW / ADD_ACCESS_INFO) under one of the three policies."""
    try:
        import time
        from geeps_b200.parallel.ps import GeePs
        cfg = make_cfg(world, base_port, pp_policy=policy, **kw)
        g = GeePs(rank, cfg)
        rows = list(range(16))
        r = g.virtual_read(0, rows, 0)
        u = g.virtual_pre_update(0, rows)
        pr = g.virtual_post_read(r)
        up = g.virtual_update(u)
        g.virtual_clock()
        g.finish_virtual_iteration()
        b = g.pre_update(u)
        b.zero_()
        g.update(up)
        g.clock()
        g.start_iterations()
        def tick():
            g.read(r, asynchronous=False)
            bb = g.pre_update(u)
            g.post_read(pr)
            bb.zero_()
            g.update(up)
            g.clock()

        def barrier():
            # the read of the second clock (slack 0) returns only after every shard applied every worker's update
            # of the first, and a worker's earlier messages to a shard precede that update on the same connection
            tick(); tick(); g.read(r, asynchronous=False); bb = g.pre_update(u); g.post_read(pr); bb.zero_(); g.update(up); g.clock()

        out = {}
        if policy == 1:
            out["owners"] = [g.locate_row(0, row) for row in range(8)]
        elif policy == 2:
            # first toucher: rank 0 asks first for rows 0,1,4,5 and rank 1 for rows 2,3,6,7
            mine = [row for row in range(8) if (row // 2) % world == rank]
            out["first"] = {row: g.locate_row(0, row) for row in mine}
            barrier()
            out["owners"] = [g.locate_row(0, row) for row in range(8)]
        else:
            # most frequent accessor: rank 1 reports 10 accesses of every row, rank 0 one; the decision is taken
            # when a statistics request reaches the shard, queries before that are held back
            for row in range(4):
                g.report_access(0, row, nread=10 if rank == 1 else 1)
            barrier()
            if rank == 0:
                g.get_stats()
            out["owners"] = [g.locate_row(0, row, timeout_ms=20000) for row in range(4)]
        barrier()
        md = g.get_stats()["server"]["metadata"]
        g.shutdown()
        g.close()
        q.put((rank, "ok", out, md))
    except Exception as e:  # pragma: no cover
        q.put((rank, "error", repr(e) + traceback.format_exc(), None))


def nvlink_hello_worker(rank, world, base_port, slack, clocks, q, kw):
    """Same helloworld-shaped run on the NVLINK transport: one GPU per rank, device-side clocks."""
    try:
        import torch
        from geeps_b200.parallel.ps import GeePs
        from geeps_b200.utils.config import DEVICE_CUDA, TRANSPORT_NVLINK
        torch.cuda.set_device(rank)
        kw = dict(kw)
        if kw.get("use_multicast"):     # small tables and two ranks would otherwise stay on the peer-load path
            os.environ["GEEPS_MC_MIN_MB"], os.environ["GEEPS_MC_MIN_RANKS"] = "0", "2"
        nrows = kw.pop("_rows", 1000)
        cfg = make_cfg(world, base_port, device=DEVICE_CUDA, cuda_device=rank, transport=TRANSPORT_NVLINK, **kw)
        stream = torch.cuda.Stream(device=rank)
        with torch.cuda.stream(stream):
            g = GeePs(rank, cfg)
            rows = list(range(nrows))
            r = g.virtual_read(0, rows, slack)
            u = g.virtual_pre_update(0, rows)
            pr = g.virtual_post_read(r)
            up = g.virtual_update(u)
            g.virtual_clock()
            g.finish_virtual_iteration()
            b = g.pre_update(u)
            b.zero_()
            g.update(up)
            g.clock()
            g.start_iterations()
            mins, maxs = [], []
            extra = slack + 1
            for c in range(clocks + extra):
                x = g.read(r)
                mins.append(x.min().clone())
                maxs.append(x.max().clone())
                b = g.pre_update(u)
                g.post_read(pr)
                b.fill_(1.0 if c < clocks else 0.0)
                g.update(up)
                g.clock()
            x = g.read(r, asynchronous=False)
            final = (float(x.min()), float(x.max()))
            torch.cuda.synchronize()
            seen = [(i + 1, float(a), float(b)) for i, (a, b) in enumerate(zip(mins, maxs))]
            err = g.last_error()
            stats = g.get_stats()
            g.shutdown()
            g.close()
        q.put((rank, "ok" if err == 0 else "error", final if err == 0 else f"runtime error {err}", seen, 0, stats))
    except Exception as e:  # pragma: no cover
        q.put((rank, "error", repr(e) + traceback.format_exc(), None, None, None))


def nvlink_train_worker(rank, world, base_port, steps, q, kw):
    """Data-parallel training of the small Inception-BN through the NVLINK parameter server."""
    try:
        import torch
        from geeps_b200.models.inception_bn import inception_bn_small
        from geeps_b200.parallel.ps_module import PSModule
        from geeps_b200.utils.config import DEVICE_CUDA, TABLE_SGD_MOMENTUM, TRANSPORT_NVLINK
        torch.cuda.set_device(rank)
        kw = dict(kw)
        if kw.get("use_multicast"):
            os.environ["GEEPS_MC_MIN_MB"], os.environ["GEEPS_MC_MIN_RANKS"] = "0", "2"
        mod_kw = kw.pop("_module", {})
        cfg = make_cfg(world, base_port, device=DEVICE_CUDA, cuda_device=rank, transport=TRANSPORT_NVLINK,
                       table_mode=TABLE_SGD_MOMENTUM, learning_rate=0.02, momentum=0.9, grad_scale=1.0 / world,
                       bf16_compute_cache=1, **kw)
        dev = torch.device("cuda", rank)
        with torch.cuda.stream(torch.cuda.Stream(device=dev)):
            net_name = mod_kw.pop("net", "inception_bn_small")
            if net_name == "fc_net":
                # two fully-connected layers whose input widths are whole table rows (eligible for pulled tables)
                from geeps_b200.models.net import Net
                from geeps_b200.ops.layers import Conv2d, Input, Linear, Pool
                net = Net("fc_net", Input(cpad=8), [
                    Conv2d("c1", 16, 3, pad=1, relu=True, std=0.1, need_dx=False), Pool("max", 2, 2),
                    Conv2d("c2", 32, 3, pad=1, relu=True, std=0.1), Pool("max", 2, 2), Pool("max", 2, 2),
                    Linear("f1", 256, relu=True, std=0.05), Linear("f2", 10, std=0.05, fp32_out=True)])
            else:
                net = inception_bn_small()
            mod = PSModule(net, (50, 3, 32, 32), cfg, rank=rank, world=world, device=dev, seed=3, **mod_kw)
            gen = torch.Generator(device=dev).manual_seed(100 + rank)
            x = torch.randn(50, 3, 32, 32, device=dev, generator=gen)
            y = torch.randint(0, 10, (50,), device=dev, generator=gen)
            losses = [mod.step(x, y, capture=(i == steps - 1)).item() for i in range(steps)]
            torch.cuda.synchronize()
            digest = {k: float(v.double().sum()) for k, v in list(mod.captured.items())[:6]}
            err = mod.ps.last_error()
            mod.close()
        q.put((rank, "ok" if err == 0 else "error", losses, digest, err, None))
    except Exception as e:  # pragma: no cover
        q.put((rank, "error", repr(e) + traceback.format_exc(), None, None, None))


def fault_worker(rank, world, base_port, mode, q, kw):
    """Host-side fault injection (no GPU): mode 'exit' - rank 1 leaves after 3 clocks without shutdown;
    'mute' - rank 1 stops sending heartbeats; 'drop' - rank 0 drops an inbound row batch."""
    try:
        import time
        import torch
        from geeps_b200.parallel.ps import GeePs, GeePsError
        from geeps_b200.utils.config import DEVICE_CPU
        cfg = make_cfg(world, base_port, device=DEVICE_CPU, **kw)
        g = GeePs(rank, cfg)
        rows = list(range(64))
        r = g.virtual_read(0, rows, 0); u = g.virtual_pre_update(0, rows)
        pr = g.virtual_post_read(r); up = g.virtual_update(u); g.virtual_clock()
        g.finish_virtual_iteration()
        g.pre_update(u).zero_(); g.update(up); g.clock(); g.start_iterations()
        t0 = time.time()
        result = ("ok", 0, "")
        try:
            for c in range(40):
                if c == 3 and rank == 1 and mode == "exit":
                    q.put((rank, "left", 0, "", 0.0))
                    q.close(); q.join_thread()        # flush the message before dying
                    os._exit(0)                       # dies between steps, sockets close
                if c == 3 and rank == 1 and mode == "mute":
                    g.inject(0, 1)
                    time.sleep(kw.get("heartbeat_timeout_ms", 1000) / 1000.0 * 3)
                if c == 3 and rank == 0 and mode == "drop":
                    g.inject(2, 1)
                x = g.read(r, asynchronous=False)
                b = g.pre_update(u); g.post_read(pr); b.fill_(1.0); g.update(up); g.clock()
                if mode == "mute" and rank == 1 and c > 6:
                    break
        except GeePsError as e:
            result = ("error", e.code, str(e))
        dt = time.time() - t0
        q.put((rank, result[0], result[1], result[2], dt))
        q.close(); q.join_thread()
        os._exit(0)                                   # skip the coordinated shutdown: peers may be gone
    except Exception as e:  # pragma: no cover
        q.put((rank, "exception", -1, repr(e) + traceback.format_exc(), 0.0))


def nvlink_pull_gemm_worker(rank, world, base_port, M, N, K, q, kw):
    """Fused pull+GEMM with the weight shards on different GPUs (peer pointers from torch symmetric
    memory); returns the max error vs an fp32 reference and timings vs all_gather + matmul."""
    try:
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        from geeps_b200.ops import functional as F
        from geeps_b200.ops import _lib as L
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(base_port), RANK=str(rank), WORLD_SIZE=str(world))
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", device_id=dev)
        per = (N + world - 1) // world
        n_start = [min(s * per, N) for s in range(world)]
        rows = [(n_start[s + 1] if s + 1 < world else N) - n_start[s] for s in range(world)]
        shard = symm_mem.empty((per, K), dtype=torch.bfloat16, device=dev)
        hdl = symm_mem.rendezvous(shard, dist.group.WORLD.group_name)
        full = []
        for s in range(world):
            g = torch.Generator(device=dev).manual_seed(1000 + s)
            full.append((torch.randn(per, K, device=dev, generator=g) * 0.1).to(torch.bfloat16))
        shard.copy_(full[rank])
        w = torch.cat([full[s][:rows[s]] for s in range(world)], 0)
        x = (torch.randn(M, K, device=dev, generator=torch.Generator(device=dev).manual_seed(7)) * 0.3).to(torch.bfloat16)
        ready = torch.full((world,), 3, dtype=torch.int32, device=dev)
        out = torch.zeros(M, (N + 7) // 8 * 8, dtype=torch.float32, device=dev)[:, :N]
        w_local = torch.zeros(N, K, dtype=torch.bfloat16, device=dev)
        st = L.new_status(dev)
        torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()

        def fused():
            F.pull_gemm(x, [int(p) for p in hdl.buffer_ptrs], n_start, out, ldw=K,
                        ready_ptrs=[ready.data_ptr() + 4 * s for s in range(world)], needed_stamp=3, w_local=w_local,
                        status=st)

        gathered = torch.empty(world * per, K, dtype=torch.bfloat16, device=dev)
        out2 = torch.empty(M, world * per, dtype=torch.float32, device=dev)

        def baseline():
            dist.all_gather_into_tensor(gathered, shard)
            torch.matmul(x, gathered.t(), out=out2.to(torch.bfloat16))

        def timeit(fn):
            for _ in range(3):
                fn()
            torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                fn()
            e1.record(); e1.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / 10], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t.item()

        fused()
        torch.cuda.synchronize()
        err = (out - x.float() @ w.float().t()).abs().max().item()
        same = bool(torch.equal(w_local, w))
        code = L.read_status(st)["code"]
        t_fused = timeit(fused)
        t_base = timeit(baseline)
        link_ms = (world - 1) / world * N * K * 2 / 770e9 * 1e3
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok", dict(err=err, w_local_ok=same, status=code, fused_ms=t_fused, nccl_allgather_matmul_ms=t_base,
                                nvlink_roofline_ms=link_ms, frac_of_roofline=link_ms / t_fused), None, None, None))
    except Exception as e:  # pragma: no cover
        q.put((rank, "error", repr(e) + traceback.format_exc(), None, None, None))


def snapshot_worker(rank, world, base_port, phase, snap_dir, q, kw):
    """phase 'save': run 4 clocks of +1 updates, snapshot, run 2 more and report what the next read sees.
    phase 'resume': load the snapshot (possibly with another world size), run the same 2 clocks."""
    try:
        import torch
        from geeps_b200.parallel.ps import GeePs
        from geeps_b200.utils.config import DEVICE_CPU, PARTITION_ROUND_ROBIN
        cfg = make_cfg(world, base_port, device=DEVICE_CPU, partitioner=PARTITION_ROUND_ROBIN, **kw)
        g = GeePs(rank, cfg)
        rows = list(range(37))
        r = g.virtual_read(0, rows, 0); u = g.virtual_pre_update(0, rows)
        pr = g.virtual_post_read(r); up = g.virtual_update(u); g.virtual_clock()
        g.finish_virtual_iteration()

        def step(val):
            x = g.read(r, asynchronous=False).clone()
            b = g.pre_update(u); g.post_read(pr); b.fill_(val); g.update(up); g.clock()
            return x

        if phase == "save":
            init = torch.arange(37 * 128, dtype=torch.float32).view(37, 128) if rank == 0 else torch.zeros(37, 128)
            g.pre_update(u).copy_(init); g.update(up); g.clock(); g.start_iterations()
            for _ in range(4):
                step(1.0)
            assert g.save_snapshot(snap_dir)
        else:
            assert g.load_snapshot(snap_dir), g.last_error_string()
            g.start_iterations()
        step(2.0 / world)         # the same total update regardless of the world size
        step(0.0)
        final = g.read(r, asynchronous=False).clone()
        g.shutdown(); g.close()
        q.put((rank, "ok", final.flatten().tolist(), None, None, None))   # plain list: no shared-memory handles
    except Exception as e:  # pragma: no cover
        q.put((rank, "error", repr(e) + traceback.format_exc(), None, None, None))


def nvlink_leave_worker(rank, world, base_port, q, kw):
    """NVLINK transport, 2 ranks: rank 1 leaves between steps with nothing of its own in flight; rank 0
    must get an error code from the runtime (host-side detection or a bounded device wait), not hang."""
    try:
        import time
        import torch
        from geeps_b200.parallel.ps import GeePs, GeePsError
        from geeps_b200.utils.config import DEVICE_CUDA, TRANSPORT_NVLINK
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        torch.cuda.set_device(rank)
        cfg = make_cfg(world, base_port, device=DEVICE_CUDA, cuda_device=rank, transport=TRANSPORT_NVLINK,
                       device_wait_budget_us=500_000, heartbeat_timeout_ms=3000)
        with torch.cuda.stream(torch.cuda.Stream(device=rank)):
            g = GeePs(rank, cfg)
            rows = list(range(256))
            r = g.virtual_read(0, rows, 0); u = g.virtual_pre_update(0, rows)
            pr = g.virtual_post_read(r); up = g.virtual_update(u); g.virtual_clock()
            g.finish_virtual_iteration()
            g.pre_update(u).zero_(); g.update(up); g.clock(); g.start_iterations()
            t0 = time.time()
            result = ("ok", 0)
            try:
                for c in range(30):
                    if rank == 1 and c == 5:
                        torch.cuda.synchronize()          # nothing of this rank is in flight
                        time.sleep(0.5)                   # let the peer finish the clock that used our signals
                        q.put((rank, "left", 0, 0.0)); q.close(); q.join_thread()
                        os._exit(0)
                    x = g.read(r); b = g.pre_update(u); g.post_read(pr); b.fill_(1.0); g.update(up); g.clock()
                    torch.cuda.synchronize()
            except GeePsError as e:
                result = ("error", e.code)
            torch.cuda.synchronize()
            alive = float(torch.ones(8, device=f"cuda:{rank}").sum()) == 8.0
            q.put((rank, result[0], result[1], time.time() - t0, alive)); q.close(); q.join_thread()
            os._exit(0)
    except Exception as e:  # pragma: no cover
        q.put((rank, "exception", repr(e) + traceback.format_exc(), 0.0, False))


def rmw_worker(rank, world, base_port, mode, rmw, q, kw):
    """Read-my-updates at slack 1 with a lagging peer.  Rank 1 sleeps before its update of clock 1; rank 0 reads in
    clock 2 (admitted on the bootstrap data alone) and reports what it sees of its own clock-1 update.  Afterwards
    both ranks run to the end and return the fully applied table (a slack-0 read declared after the Clock)."""
    try:
        import time
        import torch
        from geeps_b200.parallel.ps import GeePs
        from geeps_b200.utils.config import DEVICE_CPU, TABLE_SGD_MOMENTUM
        kw = dict(kw)
        kw.setdefault("device", DEVICE_CPU)
        cfg = make_cfg(world, base_port, read_my_writes=rmw, table_mode=mode, learning_rate=0.1, momentum=0.9,
                       weight_decay=0.0, grad_scale=1.0, **kw)
        g = GeePs(rank, cfg)
        rows = list(range(48))
        r = g.virtual_read(0, rows, 1)
        u = g.virtual_pre_update(0, rows)
        pr = g.virtual_post_read(r)
        up = g.virtual_update(u)
        g.virtual_clock()
        r0 = g.virtual_read(0, rows, 0)        # after the Clock: a one-off read with slack 0 (everything applied)
        g.virtual_post_read(r0)
        g.finish_virtual_iteration()
        g.pre_update(u).fill_(0.5)             # initial value 0.5 per worker (bootstrap updates always add)
        g.update(up)
        g.clock()
        g.start_iterations()
        seen = []
        for c in range(1, 6):                  # clocks 1..5, every worker contributes 1.0 per element per clock
            if rank == 1 and c == 1:
                time.sleep(2.5)
            x = g.read(r, asynchronous=False)
            seen.append((g.clock_value, float(x.min()), float(x.max())))
            b = g.pre_update(u)
            g.post_read(pr)
            b.fill_(1.0)
            g.update(up)
            g.clock()
        final = g.read(r0, asynchronous=False)
        out = (float(final.min()), float(final.max()))
        stats = g.get_stats()
        g.shutdown()
        g.close()
        q.put((rank, "ok", out, seen, stats["bgthread"]["nr_rmw_replay"], None))
    except Exception as e:  # pragma: no cover
        q.put((rank, "error", repr(e) + traceback.format_exc(), None, None, None))


def multitable_worker(rank, world, base_port, clocks, q, kw):
    """Three tables of different sizes, every clock +1 (table 0), +2 (table 1), +3 (table 2) per worker."""
    try:
        import torch
        from geeps_b200.parallel.ps import GeePs
        from geeps_b200.utils.config import DEVICE_CPU
        kw = dict(kw)
        kw.setdefault("device", DEVICE_CPU)
        cfg = make_cfg(world, base_port, num_tables=3, **kw)
        g = GeePs(rank, cfg)
        sizes = [64, 200, 17]
        hs = [[g.virtual_read(t, list(range(n)), 0)] for t, n in enumerate(sizes)]
        for t, n in enumerate(sizes):
            hs[t].append(g.virtual_pre_update(t, list(range(n))))
        for h in hs:
            h.append(g.virtual_post_read(h[0]))
            h.append(g.virtual_update(h[1]))
        g.virtual_clock()
        g.finish_virtual_iteration()
        for r, u, pr, up in hs:
            g.pre_update(u).zero_()
        for r, u, pr, up in hs:
            g.update(up)
        g.clock()
        g.start_iterations()
        for c in range(clocks + 1):
            xs = [g.read(r, asynchronous=False) for r, u, pr, up in hs]
            vals = [(float(x.min()), float(x.max())) for x in xs]
            bufs = [g.pre_update(u) for r, u, pr, up in hs]
            for t, (r, u, pr, up) in enumerate(hs):
                g.post_read(pr)
                bufs[t].fill_(float(t + 1) if c < clocks else 0.0)
                g.update(up)
            g.clock()
        stats = g.get_stats()
        g.shutdown()
        g.close()
        q.put((rank, "ok", vals, stats["channels"], stats["comm_channels"], None))
    except Exception as e:  # pragma: no cover
        q.put((rank, "error", repr(e) + traceback.format_exc(), None, None, None))


def lr_schedule_worker(rank, world, base_port, slack, q, kw):
    """Momentum-SGD table whose learning rate, momentum and weight decay change while the run goes on: both workers
    make the same set_hyper_params call before the same clock (rank 1 lags behind by a sleep, so the shards see the
    calls at different wall-clock times) and return the fully applied table."""
    try:
        import time
        import torch
        from geeps_b200.parallel.ps import GeePs
        from geeps_b200.utils.config import DEVICE_CPU, TABLE_SGD_MOMENTUM
        kw = dict(kw)
        kw.setdefault("device", DEVICE_CPU)
        cfg = make_cfg(world, base_port, table_mode=TABLE_SGD_MOMENTUM, learning_rate=0.1, momentum=0.9,
                       weight_decay=0.0, grad_scale=1.0 / world, **kw)
        g = GeePs(rank, cfg)
        rows = list(range(40))
        r = g.virtual_read(0, rows, slack)
        u = g.virtual_pre_update(0, rows)
        pr = g.virtual_post_read(r)
        up = g.virtual_update(u)
        g.virtual_clock()
        r0 = g.virtual_read(0, rows, 0)
        g.virtual_post_read(r0)
        g.finish_virtual_iteration()
        g.pre_update(u).fill_(1.0 / world)          # initial value 1.0
        g.update(up)
        g.clock()
        g.start_iterations()
        seen_hyper = []
        for c in range(1, 9):
            if c == 3:
                g.set_hyper_params(learning_rate=0.05)
            if c == 6:
                g.set_hyper_params(learning_rate=0.01, momentum=0.5, weight_decay=0.1)
            if rank == 1 and c in (3, 6):
                time.sleep(0.7)
            seen_hyper.append(g.hyper_params())
            g.read(r, asynchronous=False)
            b = g.pre_update(u)
            g.post_read(pr)
            b.fill_(float(c))                       # gradient c from every worker: mean c
            g.update(up)
            g.clock()
        final = g.read(r0, asynchronous=False)
        out = (float(final.min()), float(final.max()))
        g.shutdown()
        g.close()
        q.put((rank, "ok", out, seen_hyper, None, None))
    except Exception as e:  # pragma: no cover
        q.put((rank, "error", repr(e) + traceback.format_exc(), None, None, None))
