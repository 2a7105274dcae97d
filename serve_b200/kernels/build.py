"""Compiling the CUDA sources of ``csrc/`` for sm_100a into shared libraries, on demand.

Each library is built by one ``nvcc`` call, named after a hash of its sources
and flags, and kept in ``csrc/_build`` (or, if the package folder cannot be
written, in a per-user folder under the system's temporary directory), so a
second call finds it. While a compile runs, a line is printed to stderr every
few seconds. Nothing here needs a GPU: nvcc cross-compiles.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Iterable, List, Sequence, Tuple

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (
        os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
        os.path.join(os.environ.get("CUDA_PATH", ""), "bin", "nvcc") if os.environ.get("CUDA_PATH") else None,
        shutil.which("nvcc"),
        "/usr/local/cuda/bin/nvcc",
    ):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at CUDA_HOME, CUDA_PATH, PATH and /usr/local/cuda); "
                     "the engine's kernels cannot be compiled")


def build_dir() -> str:
    """A folder this user can write: beside the sources if possible."""
    override = os.environ.get("SERVE_B200_BUILD_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(CSRC, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"serve_b200-build-{os.getuid()}"))
    for d in candidates:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}.{threading.get_ident()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return d
        except OSError:
            continue
    raise BuildError("no writable folder for compiled kernels: tried " + ", ".join(c for c in candidates if c))


def _hash(sources: Sequence[str], flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cuh", ".h")):
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(f.encode() + b"\0" + fh.read())
    for s in sources:
        with open(os.path.join(CSRC, s), "rb") as fh:
            h.update(s.encode() + b"\0" + fh.read())
    h.update("\0".join(flags).encode())
    return h.hexdigest()[:16]


def library_path(name: str, sources: Sequence[str], defines: Sequence[str] = (), libs: Sequence[str] = ()) -> Tuple[str, List[str]]:
    flags = ARCH_FLAGS + BASE_FLAGS + [f"-D{d}" for d in defines]
    tag = _hash(sources, flags + list(libs))
    # a library built earlier may lie in any of the candidate folders (e.g. shipped in-tree, read-only)
    fname = f"{name}-{tag}.so"
    in_tree = os.path.join(CSRC, "_build", fname)
    if os.path.isfile(in_tree):
        return in_tree, flags
    return os.path.join(build_dir(), fname), flags


def _say(msg: str) -> None:
    print(f"[serve_b200] {msg}", file=sys.stderr, flush=True)


def build_library(name: str, sources: Sequence[str], defines: Sequence[str] = (), libs: Sequence[str] = (),
                  verbose: bool = True) -> str:
    """Compile (if not yet there) and return the path of the shared library."""
    path, flags = library_path(name, sources, defines, libs)
    if os.path.isfile(path):
        return path
    nvcc = find_nvcc()
    tmp = f"{path}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [nvcc] + flags + ["-I", CSRC, "-o", tmp] + [os.path.join(CSRC, s) for s in sources]
    cuda_lib = os.path.join(os.path.dirname(os.path.dirname(nvcc)), "lib64")
    for lib in libs:
        cmd += ["-L", cuda_lib, f"-l{lib}", "-Xlinker", f"-rpath={cuda_lib}"]
    if verbose:
        _say(f"compiling {name} ({', '.join(sources)}) for sm_100a ...")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            _say(f"  still compiling {name} ({time.time() - t0:.0f} s)")

    hb = threading.Thread(target=heartbeat, daemon=True)
    if verbose:
        hb.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise BuildError(f"nvcc failed for {name} (exit {proc.returncode}):\n{' '.join(cmd)}\n{out}")
    os.replace(tmp, path)
    # libraries of the same name built from older sources are of no use any more
    folder = os.path.dirname(path)
    for f in os.listdir(folder):
        if f.startswith(name + "-") and f.endswith(".so") and os.path.join(folder, f) != path:
            try:
                os.remove(os.path.join(folder, f))
            except OSError:
                pass
    if verbose:
        _say(f"  {name} ready in {time.time() - t0:.1f} s")
    return path


def build_many(jobs: Iterable[Dict]) -> Dict[str, str]:
    """Build several libraries side by side; returns name -> path."""
    jobs = list(jobs)
    with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 2))) as ex:
        paths = list(ex.map(lambda j: build_library(**j), jobs))
    return {j["name"]: p for j, p in zip(jobs, paths)}
