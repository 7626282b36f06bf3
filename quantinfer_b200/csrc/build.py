"""Compiles the CUDA sources of this folder for sm_100a into one shared library.

The library is plain C ABI (`extern "C" int qi_*`), loaded with ctypes, so no
Python or torch headers are compiled and a full build takes seconds. It is
built in-tree (``csrc/_build/``) when that folder can be written, else in a
per-user temporary folder, the first time it is needed; a stamp of the sources
and flags decides whether a build is still current. While nvcc runs, a line is
printed now and then so that a first call does not look hung.
"""

from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
LIB_NAME = "libquantinfer_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def timeline() -> bool:
    """QUANTINFER_B200_TIMELINE=1: the kernels are built with their time stamps (-DQI_TIMELINE), into a
    folder of their own beside the ordinary build."""
    return os.environ.get("QUANTINFER_B200_TIMELINE") == "1"


def _flags() -> list[str]:
    return NVCC_FLAGS + (["-DQI_TIMELINE"] if timeline() else [])


def _say(msg: str) -> None:
    print(f"[quantinfer_b200] {msg}", file=sys.stderr, flush=True)


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def find_nvcc() -> str:
    candidates = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            candidates.append(Path(os.environ[var]) / "bin" / "nvcc")
    which = shutil.which("nvcc")
    if which:
        candidates.append(Path(which))
    candidates.append(Path("/usr/local/cuda/bin/nvcc"))
    for c in candidates:
        if c.is_file() and os.access(c, os.X_OK):
            return str(c)
    raise RuntimeError(
        "nvcc was not found (looked at $CUDA_HOME/bin, $PATH and /usr/local/cuda/bin); "
        "the sm_100a kernels cannot be built"
    )


def _stamp() -> str:
    h = hashlib.sha256()
    h.update(" ".join(_flags()).encode())
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _build_dir() -> Path:
    override = os.environ.get("QUANTINFER_B200_BUILD_DIR")
    if override:
        d = Path(override)
        d.mkdir(parents=True, exist_ok=True)
        return d
    d = CSRC / "_build" / "timeline" if timeline() else CSRC / "_build"
    try:
        d.mkdir(parents=True, exist_ok=True)
        probe = d / f".write_probe_{os.getpid()}"
        probe.write_text("x")
        probe.unlink()
        return d
    except OSError:
        d = Path(tempfile.gettempdir()) / (f"quantinfer_b200_build_{os.getuid()}" + ("_timeline" if timeline() else ""))
        d.mkdir(parents=True, exist_ok=True)
        return d


def library_path(build: bool = True) -> Path:
    """Path of the current library; builds it first when it is missing or stale."""
    d = _build_dir()
    lib, stamp_file = d / LIB_NAME, d / "stamp"
    stamp = _stamp()
    if lib.is_file() and stamp_file.is_file() and stamp_file.read_text() == stamp:
        return lib
    if not build:
        raise FileNotFoundError(f"{lib} is missing or out of date")
    with open(d / "lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if lib.is_file() and stamp_file.is_file() and stamp_file.read_text() == stamp:
                return lib
            _compile(d, lib)
            stamp_file.write_text(stamp)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return lib


def _compile(d: Path, lib: Path) -> None:
    nvcc = find_nvcc()
    srcs = sources()
    t0 = time.time()
    _say(f"compiling {len(srcs)} CUDA sources for sm_100a into {d} (first call only)")
    done = threading.Event()

    def heartbeat() -> None:
        while not done.wait(10.0):
            _say(f"still compiling ... {time.time() - t0:.0f} s")

    beat = threading.Thread(target=heartbeat, daemon=True)
    beat.start()
    objs = [d / (s.stem + ".o") for s in srcs]

    def one(pair):
        src, obj = pair
        cmd = [nvcc, *_flags(), "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
        _say(f"compiled {src.name} ({time.time() - t0:.0f} s)")

    try:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
            list(pool.map(one, zip(srcs, objs)))
        tmp = d / (LIB_NAME + f".tmp{os.getpid()}")
        cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, lib)
    finally:
        done.set()
    _say(f"built {lib.name} in {time.time() - t0:.0f} s")


if __name__ == "__main__":
    print(library_path())
