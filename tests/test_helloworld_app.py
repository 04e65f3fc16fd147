"""Builds and runs the C++ demo against the public header and the in-tree shared library (host memory)."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_helloworld_builds_and_runs_on_cpu():
    from geeps_b200 import _native
    _native.build()
    app = os.path.join(ROOT, "apps", "helloworld")
    subprocess.run(["make", "-C", app, "clean"], check=True, capture_output=True)
    r = subprocess.run(["make", "-C", app], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    run = subprocess.run([os.path.join(app, "helloworld"), "cpu"], capture_output=True, text=True, timeout=60)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "hello world" in run.stdout
