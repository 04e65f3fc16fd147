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
