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
