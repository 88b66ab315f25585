"""Ahead-of-time build of the sm_100a kernel library with nvcc, one shared object per source.

The reference compiles CUDA C held in C# strings at run time with NVRTC and keeps the cubin
in a cache (src/SharpInference.Cuda/CudaBackend.cs:7157-7268).  Here the kernels are ``.cu``
files compiled by ``nvcc`` for ``sm_100a`` into ``lib<name>.so`` beside the sources
(``csrc/_build/``), each with a C ABI that :mod:`sharpinference_b200.kernels.library` binds
with ``ctypes``.  A library is built when it is first asked for and whenever its source, a
header or the flags change, so a model compiles only the kernels it uses.  While ``nvcc``
runs, a line is printed to stderr every few seconds.  If the package folder is read-only the
objects go to a per-user folder under the system's temporary directory.
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
from typing import Dict, Iterable, List, Optional

CSRC_DIR = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]

# Per-source additions (include paths, libraries).
EXTRA_FLAGS: Dict[str, List[str]] = {}


class KernelBuildError(RuntimeError):
    pass


def kernel_sources() -> List[str]:
    """Names (without extension) of every kernel source in ``csrc/``."""
    return sorted(os.path.splitext(f)[0] for f in os.listdir(CSRC_DIR) if f.endswith(".cu"))


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError(
        "nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin/nvcc); the sm_100a kernels "
        "are compiled at first use and there is no fallback without them")


def _included(path: str, seen: Optional[set] = None) -> List[str]:
    """``path`` and every file of ``csrc/`` it includes with quotes, directly or not."""
    seen = seen if seen is not None else set()
    if path in seen or not os.path.isfile(path):
        return []
    seen.add(path)
    out = [path]
    with open(path, "r", encoding="utf-8") as fh:
        for line in fh:
            line = line.strip()
            if line.startswith("#include \""):
                out.extend(_included(os.path.join(CSRC_DIR, line.split('"')[1]), seen))
    return out


def _fingerprint(name: str, nvcc: str) -> str:
    h = hashlib.sha256()
    for path in sorted(_included(os.path.join(CSRC_DIR, name + ".cu"))):
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(ARCH_FLAGS + BASE_FLAGS + EXTRA_FLAGS.get(name, [])).encode())
    return h.hexdigest()


_build_dir_cache: Optional[str] = None


def build_dir() -> str:
    """``csrc/_build`` when it can be written, else a per-user folder in the temp directory."""
    global _build_dir_cache
    if _build_dir_cache:
        return _build_dir_cache
    candidates = [os.path.join(CSRC_DIR, "_build"),
                  os.path.join(tempfile.gettempdir(), f"sharpinference_b200_build_{os.getuid()}")]
    for cand in candidates:
        try:
            os.makedirs(cand, exist_ok=True)
            probe = os.path.join(cand, f".write_probe_{os.getpid()}")
            with open(probe, "w") as fh:
                fh.write("x")
            os.remove(probe)
            _build_dir_cache = cand
            return cand
        except OSError:
            continue
    raise KernelBuildError(f"no writable folder for compiled kernels (tried {candidates})")


def library_path(name: str) -> str:
    return os.path.join(build_dir(), f"lib{name}.so")


def is_current(name: str) -> bool:
    so, stamp = library_path(name), library_path(name) + ".stamp"
    if not (os.path.isfile(so) and os.path.isfile(stamp)):
        return False
    try:
        with open(stamp) as fh:
            return fh.read().strip() == _fingerprint(name, find_nvcc())
    except (OSError, KernelBuildError):
        return False


_locks: Dict[str, threading.Lock] = {}
_locks_guard = threading.Lock()


def _log(text: str) -> None:
    print(f"[sharpinference_b200] {text}", file=sys.stderr, flush=True)


def build_library(name: str, *, ptxas_info: bool = False) -> str:
    """Compile ``csrc/<name>.cu`` if its shared object is missing or stale; return its path."""
    src = os.path.join(CSRC_DIR, name + ".cu")
    if not os.path.isfile(src):
        raise KernelBuildError(f"no kernel source {src}")
    with _locks_guard:
        lock = _locks.setdefault(name, threading.Lock())
    with lock:
        if is_current(name) and not ptxas_info:
            return library_path(name)
        nvcc = find_nvcc()
        out = library_path(name)
        tmp_out = f"{out}.{os.getpid()}.tmp"
        cmd = [nvcc, *ARCH_FLAGS, *BASE_FLAGS, *EXTRA_FLAGS.get(name, []), "-I", CSRC_DIR, "-o", tmp_out, src]
        if ptxas_info:
            cmd[1:1] = ["-Xptxas", "-v"]
        _log(f"compiling {name}.cu for sm_100a ...")
        t0 = time.time()
        proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        done = threading.Event()

        def ticker() -> None:
            while not done.wait(10.0):
                _log(f"  still compiling {name}.cu ({time.time() - t0:.0f} s)")

        threading.Thread(target=ticker, daemon=True).start()
        output, _ = proc.communicate()
        done.set()
        if proc.returncode != 0:
            if os.path.exists(tmp_out):
                os.remove(tmp_out)
            raise KernelBuildError(f"nvcc failed for {name}.cu (exit {proc.returncode}):\n{' '.join(cmd)}\n{output}")
        os.replace(tmp_out, out)
        with open(out + ".stamp", "w") as fh:
            fh.write(_fingerprint(name, nvcc))
        _log(f"compiled {name}.cu in {time.time() - t0:.1f} s")
        if ptxas_info:
            print(output, file=sys.stderr)
        return out


def build_all(names: Optional[Iterable[str]] = None, *, jobs: int = 4, ptxas_info: bool = False) -> List[str]:
    """Compile every kernel source (or the named ones), a few at a time."""
    names = list(names) if names is not None else kernel_sources()
    build_dir()
    results: Dict[str, str] = {}
    errors: List[str] = []
    sem = threading.Semaphore(max(1, jobs))

    def one(n: str) -> None:
        with sem:
            try:
                results[n] = build_library(n, ptxas_info=ptxas_info)
            except KernelBuildError as exc:
                errors.append(str(exc))

    threads = [threading.Thread(target=one, args=(n,)) for n in names]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise KernelBuildError("\n\n".join(errors))
    return [results[n] for n in names]


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser(description="compile the sm_100a kernel library")
    ap.add_argument("names", nargs="*", help="kernel sources to build (default: all)")
    ap.add_argument("--ptxas-info", action="store_true", help="print registers / spills / shared memory")
    ns = ap.parse_args()
    for p in build_all(ns.names or None, ptxas_info=ns.ptxas_info):
        print(p)
