"""The host runtime under ThreadSanitizer and AddressSanitizer: tests/native/ps_stress.cpp runs several workers
(each a GeePs instance with its server shard, TCP loopback, host memory, SSP) inside one process, so every
runtime thread - application, push workers, decoders, routers, servers, heartbeats - is visible to the tool."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NATIVE = os.path.join(ROOT, "tests", "native")


def _compiler_with(lib):
    """A g++ whose installation carries the sanitizer runtime `lib` (some toolchains ship without it)."""
    for cxx in ("g++", "/usr/bin/g++"):
        path = shutil.which(cxx)
        if not path:
            continue
        out = subprocess.run([path, f"-print-file-name={lib}"], capture_output=True, text=True).stdout.strip()
        if os.path.isabs(out) and os.path.exists(out):
            return path
    return None


@pytest.mark.parametrize("san,lib,world,slack,port,mode", [("thread", "libtsan.so", 3, 1, 23100, ""),
                                                           ("address", "libasan.so", 3, 0, 23300, ""),
                                                           # optimizer table whose hyper-parameters change while
                                                           # the shards apply earlier clocks
                                                           ("thread", "libtsan.so", 3, 0, 23500, "sgd")])
def test_runtime_is_clean_under_sanitizer(san, lib, world, slack, port, mode):
    cxx = _compiler_with(lib)
    if cxx is None:
        pytest.skip(f"no g++ with {lib} in this image")
    from geeps_b200 import _native
    _native.build()                      # the kernel objects the stress binary links against
    r = subprocess.run(["make", "-C", NATIVE, f"SAN={san}", f"CXX={cxx}"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=0 exitcode=66", ASAN_OPTIONS="detect_leaks=1 exitcode=67")
    run = subprocess.run([os.path.join(NATIVE, f"ps_stress_{san}"), str(world), str(slack), "25", str(port)] + ([mode] if mode else []),
                         capture_output=True, text=True, timeout=600, env=env)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-6000:]
    assert "failures 0" in run.stdout
    assert "Sanitizer" not in run.stderr, run.stderr[-6000:]
