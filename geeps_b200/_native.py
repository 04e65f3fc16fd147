"""Build and load the native library (C++ runtime + sm_100a kernels).

The library is built in-tree with nvcc/g++ through a generated ninja file and loaded
with ctypes; it has no dependency on torch's C++ ABI.  A content hash of the sources and
flags is stored beside the .so so that an unchanged tree is never rebuilt (in particular
not on a machine that received the prebuilt .so).
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import threading
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
LIB_DIR = Path(__file__).resolve().parent / "lib"
BUILD_DIR = ROOT / "build" / "native"
LIB_NAME = "libgeeps_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall",
    "-Xptxas", "-v",
]
CXX_FLAGS = ["-O2", "-g", "-std=c++17", "-fPIC", "-Wall", "-pthread"]

_lock = threading.Lock()
_lib = None


def _cuda_home() -> Path:
    for cand in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if cand and (Path(cand) / "bin" / "nvcc").exists():
            return Path(cand)
    nvcc = shutil.which("nvcc")
    if nvcc:
        return Path(nvcc).resolve().parent.parent
    raise RuntimeError("nvcc not found: cannot build the geeps_b200 native library")


def sources() -> list[Path]:
    out = sorted(CSRC.rglob("*.cu")) + sorted(CSRC.rglob("*.cpp"))
    return [p for p in out if "apps" not in p.parts]


def _headers() -> list[Path]:
    return sorted(list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.hpp")) + list(CSRC.rglob("*.cuh"))
                  + list((ROOT / "include").glob("*.hpp")))


def source_hash() -> str:
    h = hashlib.sha256()
    for p in sources() + _headers():
        h.update(str(p.relative_to(ROOT)).encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS + CXX_FLAGS).encode())
    return h.hexdigest()


def lib_path() -> Path:
    return LIB_DIR / LIB_NAME


def is_built() -> bool:
    stamp = LIB_DIR / (LIB_NAME + ".hash")
    return lib_path().exists() and stamp.exists() and stamp.read_text().strip() == source_hash()


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile every .cu/.cpp under csrc/ for sm_100a and link lib/libgeeps_b200.so.

    Several processes may get here at once (one rank per GPU, test workers): a file lock serialises them, the
    check is repeated under the lock, and the library and its stamp are moved into place atomically, so no
    process ever loads a half-written file."""
    with _lock:
        if is_built() and not force:
            return lib_path()
        BUILD_DIR.mkdir(parents=True, exist_ok=True)
        LIB_DIR.mkdir(parents=True, exist_ok=True)
        with open(BUILD_DIR / ".lock", "w") as lock_file:
            fcntl.flock(lock_file, fcntl.LOCK_EX)
            try:
                if is_built() and not force:
                    return lib_path()
                return _build_locked(verbose)
            finally:
                fcntl.flock(lock_file, fcntl.LOCK_UN)


def _build_locked(verbose: bool) -> Path:
    cuda = _cuda_home()
    inc = [f"-I{CSRC}", f"-I{ROOT / 'include'}", f"-I{cuda / 'include'}"]
    lines = [
        f"nvcc = {cuda / 'bin' / 'nvcc'}",
        "cxx = g++",
        f"nvflags = {' '.join(NVCC_FLAGS)} {' '.join(inc)}",
        f"cxxflags = {' '.join(CXX_FLAGS)} {' '.join(inc)}",
        "rule nvcc",
        "  command = $nvcc $nvflags -MD -MF $out.d -c $in -o $out > $out.log 2>&1 || (cat $out.log; false)",
        "  depfile = $out.d",
        "  deps = gcc",
        "rule cxx",
        "  command = $cxx $cxxflags -MD -MF $out.d -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "rule link",
        f"  command = $nvcc -shared -o $out $in -cudart static -lpthread -ldl -lrt",
    ]
    staged = BUILD_DIR / (LIB_NAME + ".new")
    objs = []
    for src in sources():
        obj = BUILD_DIR / (str(src.relative_to(CSRC)).replace("/", "_") + ".o")
        rule = "nvcc" if src.suffix == ".cu" else "cxx"
        lines.append(f"build {obj}: {rule} {src}")
        objs.append(str(obj))
    lines.append(f"build {staged}: link {' '.join(objs)}")
    lines.append(f"default {staged}")
    (BUILD_DIR / "build.ninja").write_text("\n".join(lines) + "\n")
    cmd = ["ninja", "-C", str(BUILD_DIR)] + (["-v"] if verbose else [])
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout[-8000:] + proc.stderr[-4000:])
        raise RuntimeError("native build failed")
    # ninja considers `staged` up to date next time only if it still exists: install a copy
    tmp_lib = LIB_DIR / (LIB_NAME + f".tmp{os.getpid()}")
    shutil.copy2(staged, tmp_lib)
    os.replace(tmp_lib, lib_path())
    tmp_hash = LIB_DIR / (LIB_NAME + f".hash.tmp{os.getpid()}")
    tmp_hash.write_text(source_hash())
    os.replace(tmp_hash, LIB_DIR / (LIB_NAME + ".hash"))
    return lib_path()


def ptxas_report() -> str:
    """Concatenated `-Xptxas -v` output of the last build (registers, spills, smem)."""
    out = []
    for log in sorted(BUILD_DIR.glob("*.o.log")):
        out.append(f"== {log.name}\n{log.read_text()}")
    return "\n".join(out)


def load() -> ctypes.CDLL:
    """Load (building first if the tree changed) the native library."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not is_built():
        if os.environ.get("GEEPS_B200_NO_BUILD") and path.exists():
            pass
        else:
            path = build()
    with _lock:
        if _lib is None:
            _lib = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
    return _lib
