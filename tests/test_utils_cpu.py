"""Host-only tests of the utilities: trace writer, config mirror."""
import json

from geeps_b200.utils.config import GeePsConfig
from geeps_b200.utils.trace import ChromeTrace


def test_chrome_trace_roundtrip(tmp_path):
    tr = ChromeTrace("unit", nvtx=False)
    with tr.span("fwd:conv1", "fwd", rows=3):
        with tr.span("read:conv1", "ps"):
            pass
    tr.instant("clock", clock=1)
    tr.counter("staleness", value=0)
    path = tmp_path / "trace.json"
    tr.save(str(path))
    data = json.loads(path.read_text())
    names = [e["name"] for e in data["traceEvents"]]
    assert "fwd:conv1" in names and "read:conv1" in names and "clock" in names
    spans = [e for e in data["traceEvents"] if e.get("ph") == "X"]
    assert all(e["dur"] >= 0 for e in spans)


def test_config_mirror_covers_every_numeric_field():
    cfg = GeePsConfig()
    for k in GeePsConfig._NUMERIC + GeePsConfig._STRING:
        assert hasattr(cfg, k), k
    assert cfg.tcp_base_port == 9090 and cfg.mm_warning_level == 1 and cfg.read_my_writes == 0


def test_tape_records_and_replays_native_calls():
    import ctypes as C
    from geeps_b200.ops import _lib as L
    seen = []

    def fake_kernel(a, b):
        seen.append((a.value, b))
        return 0

    def fake_ps(a):
        seen.append(("ps", a))
        return 1

    tape = L.start_recording()
    seed = C.c_ulonglong(7)
    L.launch(fake_kernel, "dropout", seed, 3)
    assert L.record_call(fake_ps, "read", 5) == 1
    assert L.stop_recording() is tape
    L.launch(fake_kernel, "dropout", seed, 4)            # not recorded any more
    assert len(tape.ops) == 2 and tape.kernel_launches == 1
    assert tape.signature() == [("dropout", 7, 3), ("ps:read", 5)]
    seen.clear()
    seed.value = 8
    n0 = L.launch_count()
    tape.replay()
    assert seen == [(8, 3), ("ps", 5)]
    assert L.launch_count() - n0 == 1


def test_bind_to_gpu_cores_is_harmless_without_a_gpu():
    import os
    from geeps_b200.utils.affinity import bind_to_gpu_cores
    before = os.sched_getaffinity(0)
    cores = bind_to_gpu_cores(0)
    after = os.sched_getaffinity(0)
    if cores is None:
        assert after == before          # no NVML here: nothing changed
    else:
        assert set(cores) == after and after <= before
        os.sched_setaffinity(0, before)


def test_affinity_splits_a_mask_shared_by_all_gpus():
    """A fake NVML reports the same 32-core mask for eight GPUs (a one-node virtual machine): the eight ranks get
    disjoint slices; distinct masks are left alone."""
    import os
    from geeps_b200.utils import affinity

    class FakeNvml:
        def __init__(self, masks):
            self.masks = masks

        def nvmlInit(self): pass
        def nvmlShutdown(self): pass
        def nvmlDeviceGetHandleByIndex(self, i): return i
        def nvmlDeviceGetCpuAffinity(self, h, words):
            return [self.masks[h]] + [0] * (words - 1)

    assert affinity.split_shared_mask(list(range(32)), 8, 3) == [12, 13, 14, 15]
    assert affinity.split_shared_mask(list(range(3)), 8, 3) == [0, 1, 2]
    slices = [affinity.split_shared_mask(list(range(30)), 8, k) for k in range(8)]
    assert sorted(c for s in slices for c in s) == list(range(30))
    allowed = sorted(os.sched_getaffinity(0))
    before = os.sched_getaffinity(0)
    try:
        mask = sum(1 << c for c in allowed if c < 64)
        n = len([c for c in allowed if c < 64])
        world = 2 if n >= 2 else 1
        got = []
        for k in range(world):      # one process plays both ranks: undo the binding in between
            got.append(affinity.bind_to_gpu_cores(k, world, nvml=FakeNvml([mask] * 8)))
            os.sched_setaffinity(0, before)
        if world == 2:
            assert not set(got[0]) & set(got[1]) and sorted(got[0] + got[1]) == [c for c in allowed if c < 64]
        os.sched_setaffinity(0, before)
        # different masks per GPU: each rank keeps its own
        if n >= 2:
            a, b = allowed[0], allowed[1]
            got = affinity.bind_to_gpu_cores(1, 2, nvml=FakeNvml([1 << a, 1 << b] + [0] * 6))
            assert got == [b]
    finally:
        os.sched_setaffinity(0, before)


def test_input_layer_augmentation_buffer_bookkeeping():
    """The augmentation of uint8 batches lives in one buffer the layer owns: random windows stay inside the source
    image, explicit values land in the same storage (captured steps keep reading it), and None restores the centre
    crop once the source size is known."""
    import torch
    from geeps_b200.ops.layers import Input
    B, H, W, Hin, Win = 6, 16, 18, 24, 30
    inp = Input(cpad=8, mean=(1.0, 2.0, 3.0), scale=0.5)
    assert inp.setup((B, 3, H, W), "cpu") == (B, H, W, 8)
    inp.randomize((Hin, Win), generator=torch.Generator().manual_seed(0))
    a = inp.aug.clone()
    assert a.shape == (B, 3) and a.dtype == torch.int32
    assert int(a[:, 0].min()) >= 0 and int(a[:, 0].max()) <= Hin - H
    assert int(a[:, 1].min()) >= 0 and int(a[:, 1].max()) <= Win - W
    assert set(a[:, 2].tolist()) <= {0, 1}
    ptr = inp.aug.data_ptr()
    inp.set_augmentation(torch.tensor([[1, 2, 1]] * B))
    assert inp.aug.data_ptr() == ptr and inp.aug.tolist() == [[1, 2, 1]] * B
    inp._src_hw = (Hin, Win)                  # what a forward on a uint8 batch records
    inp.set_augmentation(None)
    assert inp.aug.data_ptr() == ptr and inp.aug.tolist() == [[(Hin - H) // 2, (Win - W) // 2, 0]] * B
    inp.randomize((Hin, Win), mirror=False)
    assert int(inp.aug[:, 2].max()) == 0
    inp.set_transform((9.0, 8.0, 7.0), 2.0)
    assert inp.mean == (9.0, 8.0, 7.0) and inp.scale == 2.0


def test_bench_clock_sampler_reads_a_fake_nvidia_smi(tmp_path, monkeypatch):
    """The benchmark's clock record: the sampler waits for the tool's first line (its start can outlast a short timed
    region), keeps the samples of the marked window and reports the median clock and the active throttle reasons."""
    import os
    import stat
    import sys
    import time
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench
    fake = tmp_path / "nvidia-smi"
    fake.write_text("#!/bin/sh\nsleep 0.4\nwhile true; do echo '1867, 1965, 930.5, Not Active, Not Active, Not Active, Active'; "
                    "sleep 0.05; done\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", str(tmp_path) + os.pathsep + os.environ["PATH"])
    s = bench.ClockSampler(0)
    s.start()
    t0 = time.time()
    s.wait_first_sample()
    assert 0.3 < time.time() - t0 < 5.0 and s.samples          # blocked until the first line arrived
    s.mark_begin()
    time.sleep(0.3)
    s.mark_end()
    rec = s.stop()
    assert rec["sm_mhz"] == 1867.0 and rec["sm_max_mhz"] == 1965.0 and rec["reasons"] == ["sw_power_cap"]
    assert rec["samples"] >= 3
    # without the tool the record says so instead of failing the run
    monkeypatch.setenv("PATH", str(tmp_path / "empty"))
    s2 = bench.ClockSampler(0)
    s2.start()
    s2.wait_first_sample(0.2)
    assert s2.stop()["sm_mhz"] is None
    assert bench.pcie_links() == []
