"""Compiles the CUDA sources under ``csrc/`` into one shared library for sm_100a.

The library is built with nvcc alone (no torch headers, so a file takes seconds) the first time
it is needed, and again when a source changes.  It is kept beside the sources in ``csrc/_build``
when that folder can be written, else in a per-user folder under the system's temporary
directory.  While nvcc runs, a line is printed every few seconds so that a first call in a fresh
checkout does not look hung.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path
from typing import List, Optional

CSRC = Path(__file__).resolve().parent.parent / "csrc"
LIB_NAME = "libptl_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
] + os.environ.get("PTL_NVCC_EXTRA", "").split()      # e.g. -DPTL_VECTOR_REDUCE_COLUMNS=32 for a measuring build (give it a PTL_BUILD_DIR of its own)


class BuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[pytriton_llama_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("PTL_NVCC"),
                 shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found: set CUDA_HOME or PTL_NVCC; the CUDA kernels cannot be compiled")


def sources() -> List[Path]:
    return sorted(CSRC.glob("*.cu"))


def _fingerprint() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _writable_dir(path: Path) -> bool:
    try:
        path.mkdir(parents=True, exist_ok=True)
        probe = path / f".probe_{os.getpid()}"
        probe.write_text("x")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    env = os.environ.get("PTL_BUILD_DIR")
    if env:
        p = Path(env)
        if not _writable_dir(p):
            raise BuildError(f"PTL_BUILD_DIR={env} cannot be written")
        return p
    local = CSRC / "_build"
    if _writable_dir(local):
        return local
    p = Path(tempfile.gettempdir()) / f"pytriton_llama_b200_build_{os.getuid()}"
    if not _writable_dir(p):
        raise BuildError(f"neither {local} nor {p} can be written")
    return p


def _run(cmd: List[str], what: str) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise BuildError(f"{what} failed ({' '.join(cmd)}):\n{proc.stdout}")


class _Ticker:
    """Prints a line every ``period`` seconds until stopped."""

    def __init__(self, what: str, period: float = 10.0):
        self._stop = threading.Event()
        self._t0 = time.time()
        self._what = what
        self._period = period
        self._thread = threading.Thread(target=self._loop, daemon=True)

    def _loop(self) -> None:
        while not self._stop.wait(self._period):
            _log(f"{self._what} ... {time.time() - self._t0:.0f} s")

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join()


def library_path(force: bool = False, verbose: Optional[bool] = None) -> Path:
    """Path of the built library, compiling it first if it is missing or stale."""
    out_dir = build_dir()
    lib = out_dir / LIB_NAME
    stamp = out_dir / "build.json"
    fp = _fingerprint()
    if not force and lib.exists() and stamp.exists():
        try:
            if json.loads(stamp.read_text()).get("fingerprint") == fp:
                return lib
        except (OSError, ValueError):
            pass
    import fcntl
    with open(out_dir / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and lib.exists() and stamp.exists():
                try:
                    if json.loads(stamp.read_text()).get("fingerprint") == fp:
                        return lib
                except (OSError, ValueError):
                    pass
            _compile(out_dir, lib)
            stamp.write_text(json.dumps({"fingerprint": fp, "flags": NVCC_FLAGS}))
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return lib


def _compile(out_dir: Path, lib: Path) -> None:
    nvcc = find_nvcc()
    srcs = sources()
    if not srcs:
        raise BuildError(f"no .cu sources under {CSRC}")
    _log(f"compiling {len(srcs)} CUDA files for sm_100a into {out_dir} (first call only)")
    t0 = time.time()
    objs = [out_dir / (s.stem + ".o") for s in srcs]

    def one(pair):
        src, obj = pair
        _run([nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)], f"nvcc {src.name}")
        _log(f"  {src.name} done ({time.time() - t0:.0f} s)")

    workers = max(1, min(len(srcs), os.cpu_count() or 1, 8))
    with _Ticker("still compiling"):
        with concurrent.futures.ThreadPoolExecutor(workers) as pool:
            list(pool.map(one, zip(srcs, objs)))
        tmp = out_dir / (LIB_NAME + f".tmp{os.getpid()}")
        _run([nvcc, "-shared", "-o", str(tmp), *[str(o) for o in objs], "-lcudart_static", "-ldl", "-lrt", "-lpthread"],
             "link")
        os.replace(tmp, lib)
    _log(f"built {lib.name} in {time.time() - t0:.0f} s")
