"""Builds and loads the CUDA library of the package.

The kernels under ``rosellm_b200/csrc`` are plain CUDA with a C interface, so
they compile with ``nvcc`` alone in seconds and load through ``ctypes``; no
part of torch's extension machinery (and no cache under the home folder) is
involved.  The library is built for ``sm_100a`` at the first call that needs
it, beside the sources when that folder can be written, else under the
system's temporary folder, and is rebuilt when a source changes.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))
LIB_NAME = "librosellm_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]

# Further flags for nvcc, e.g. ROSELLM_B200_NVCC_EXTRA="-DRL_PHASE_TIMING" to compile the clock
# stamps of the fused decode kernels in (read with ``python -m rosellm_b200.ops.microbench --phases``).
NVCC_FLAGS += [f for f in os.environ.get("ROSELLM_B200_NVCC_EXTRA", "").split() if f]

_lock = threading.Lock()
_lib: ctypes.CDLL | None = None


class BuildError(RuntimeError):
    pass


def _sources() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def source_hash() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for name in _sources() + _headers():
        h.update(name.encode())
        with open(os.path.join(CSRC, name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def _find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError(
        "the CUDA library of rosellm_b200 is not built and nvcc was not found "
        "(looked at $NVCC, PATH and /usr/local/cuda/bin/nvcc)"
    )


def _build_dir() -> str:
    in_tree = os.path.join(CSRC, "_build")
    try:
        os.makedirs(in_tree, exist_ok=True)
        probe = os.path.join(in_tree, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return in_tree
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"rosellm_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def lib_path() -> str:
    return os.path.join(_build_dir(), LIB_NAME)


def _say(msg: str) -> None:
    print(f"[rosellm_b200] {msg}", file=sys.stderr, flush=True)


def build(force: bool = False, verbose: bool = True) -> str:
    """Compile every ``.cu`` under ``csrc`` for sm_100a and link the library.  Returns its path."""
    out_dir = _build_dir()
    lib = os.path.join(out_dir, LIB_NAME)
    stamp = os.path.join(out_dir, LIB_NAME + ".hash")
    want = source_hash()

    def fresh() -> bool:
        if not (os.path.isfile(lib) and os.path.isfile(stamp)):
            return False
        with open(stamp) as f:
            return f.read().strip() == want

    if not force and fresh():
        return lib
    # one builder at a time per folder: processes started together (test workers, a server and
    # a tool) would otherwise write the same object files at once
    lock = open(os.path.join(out_dir, ".build.lock"), "w")
    fcntl.flock(lock, fcntl.LOCK_EX)
    try:
        if not force and fresh():
            return lib
        return _build_locked(out_dir, lib, stamp, want, verbose)
    finally:
        fcntl.flock(lock, fcntl.LOCK_UN)
        lock.close()


def _build_locked(out_dir: str, lib: str, stamp: str, want: str, verbose: bool) -> str:
    nvcc = _find_nvcc()
    sources = _sources()
    if verbose:
        _say(f"compiling {len(sources)} CUDA files for sm_100a into {out_dir} ...")
    t0 = time.time()
    procs = []
    for src in sources:
        obj = os.path.join(out_dir, src[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    objs = []
    pending = list(procs)
    last_note = time.time()
    while pending:
        for item in list(pending):
            src, obj, proc = item
            if proc.poll() is not None:
                out = proc.stdout.read().decode(errors="replace")
                if proc.returncode != 0:
                    for _, _, other in pending:
                        if other is not proc and other.poll() is None:
                            other.kill()
                    raise BuildError(f"nvcc failed on {src}:\n{out}")
                if verbose:
                    _say(f"  compiled {src} ({time.time() - t0:.0f} s)")
                pending.remove(item)
        if pending:
            time.sleep(0.2)
            if verbose and time.time() - last_note > 10:
                _say(f"  still compiling: {', '.join(s for s, _, _ in pending)} ({time.time() - t0:.0f} s)")
                last_note = time.time()
    objs = [obj for _, obj, _ in procs]
    tmp_lib = lib + f".tmp{os.getpid()}"
    cmd = [nvcc, "-shared", "-o", tmp_lib, *objs, "-lcudart"]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    if res.returncode != 0:
        raise BuildError(f"linking {LIB_NAME} failed:\n{res.stdout.decode(errors='replace')}")
    os.replace(tmp_lib, lib)
    with open(stamp, "w") as f:
        f.write(want)
    if verbose:
        _say(f"built {lib} in {time.time() - t0:.0f} s")
    return lib


def load() -> ctypes.CDLL:
    """The loaded library; builds it first if it is missing or stale.  Raises if it cannot."""
    global _lib
    with _lock:
        if _lib is None:
            _lib = ctypes.CDLL(build())
        return _lib
