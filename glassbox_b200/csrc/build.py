"""Compile the CUDA sources of this folder for sm_100a into one shared library, in-tree.

The library is built by plain ``nvcc`` (no torch headers, so each file takes seconds) into
``csrc/_build/libglassbox_b200.so`` the first time it is needed and again whenever a source
changes (the stamp is a hash of every source and of the flags). The build prints a line per
file to stderr so that a first call is visibly busy, writes only inside this folder, and needs
neither network nor a home directory.
"""
from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import time
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD_DIR = os.path.join(HERE, "_build")
LIB_NAME = "libglassbox_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin/nvcc); "
                     "the CUDA kernels cannot be built and there is no fallback")


def sources():
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _stamp() -> str:
    h = hashlib.sha256()
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    for f in sorted(os.listdir(HERE)):
        if f.endswith((".cu", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(HERE, f), "rb") as fh:
                h.update(fh.read())
    return h.hexdigest()


def _log(msg: str) -> None:
    print(f"[glassbox_b200 build] {msg}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: str, verbose_ptxas: bool) -> str:
    obj = os.path.join(BUILD_DIR, src[:-3] + ".o")
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", HERE, "-c",
           os.path.join(HERE, src), "-o", obj]
    if verbose_ptxas:
        cmd += ["-Xptxas", "-v"]
    t0 = time.time()
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {src}:\n{proc.stdout}\n{proc.stderr}")
    _log(f"compiled {src} in {time.time() - t0:.1f}s")
    if verbose_ptxas:
        sys.stderr.write(proc.stderr)
    return obj


def library_path() -> str:
    return os.path.join(BUILD_DIR, LIB_NAME)


def ensure_built(force: bool = False, verbose_ptxas: bool = False) -> str:
    """Build if needed; return the path of the shared library."""
    lib = library_path()
    stamp_file = os.path.join(BUILD_DIR, "stamp")
    want = _stamp()

    def fresh() -> bool:
        try:
            with open(stamp_file) as f:
                return f.read().strip() == want and os.path.exists(lib)
        except OSError:
            return False

    if not force and fresh():
        return lib
    try:
        os.makedirs(BUILD_DIR, exist_ok=True)
    except OSError as e:
        raise BuildError(f"cannot create {BUILD_DIR}: {e}") from None
    with open(os.path.join(BUILD_DIR, "lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and fresh():
                return lib
            nvcc = _nvcc()
            srcs = sources()
            _log(f"compiling {len(srcs)} CUDA sources for sm_100a with {nvcc} (first use or sources changed)")
            t0 = time.time()
            with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 2)) as pool:
                objs = list(pool.map(lambda s: _compile_one(nvcc, s, verbose_ptxas), srcs))
            tmp = lib + f".{os.getpid()}.tmp"
            cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *objs, "-lcudart_static", "-ldl", "-lpthread", "-lrt"]
            proc = subprocess.run(cmd, capture_output=True, text=True)
            if proc.returncode != 0:
                raise BuildError(f"linking {LIB_NAME} failed:\n{proc.stdout}\n{proc.stderr}")
            os.replace(tmp, lib)
            with open(stamp_file, "w") as f:
                f.write(want)
            _log(f"built {LIB_NAME} in {time.time() - t0:.1f}s")
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return lib


HOST_DIR = os.path.join(HERE, "host")
HOST_LIB_NAME = "libglassbox_host.so"
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall"]


def host_library_path() -> str:
    return os.path.join(BUILD_DIR, HOST_LIB_NAME)


def ensure_host_built(force: bool = False) -> str:
    """Build the C++ host library (``csrc/host/*.cpp``: cache bookkeeping, step layout) with the C++
    compiler; it has no CUDA in it and is needed on machines without a GPU too."""
    lib = host_library_path()
    stamp_file = os.path.join(BUILD_DIR, "host_stamp")
    srcs = sorted(f for f in os.listdir(HOST_DIR) if f.endswith((".cpp", ".h")))
    h = hashlib.sha256(" ".join(HOST_FLAGS).encode())
    for f in srcs:
        h.update(f.encode())
        with open(os.path.join(HOST_DIR, f), "rb") as fh:
            h.update(fh.read())
    want = h.hexdigest()

    def fresh() -> bool:
        try:
            with open(stamp_file) as f:
                return f.read().strip() == want and os.path.exists(lib)
        except OSError:
            return False

    if not force and fresh():
        return lib
    try:
        os.makedirs(BUILD_DIR, exist_ok=True)
    except OSError as e:
        raise BuildError(f"cannot create {BUILD_DIR}: {e}") from None
    with open(os.path.join(BUILD_DIR, "host_lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and fresh():
                return lib
            cxx = next((c for c in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++"))
                        if c), None)
            if cxx is None:
                raise BuildError("no C++ compiler found (looked at $CXX, g++, c++, clang++); the host library cannot be built")
            t0 = time.time()
            tmp = lib + f".{os.getpid()}.tmp"
            cmd = [cxx, *HOST_FLAGS, "-o", tmp, *[os.path.join(HOST_DIR, f) for f in srcs if f.endswith(".cpp")]]
            proc = subprocess.run(cmd, capture_output=True, text=True)
            if proc.returncode != 0:
                raise BuildError(f"compiling {HOST_LIB_NAME} failed:\n{proc.stdout}\n{proc.stderr}")
            os.replace(tmp, lib)
            with open(stamp_file, "w") as f:
                f.write(want)
            _log(f"built {HOST_LIB_NAME} in {time.time() - t0:.1f}s")
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return lib


if __name__ == "__main__":
    print(ensure_host_built(force="--force" in sys.argv))
    print(ensure_built(force="--force" in sys.argv, verbose_ptxas="-v" in sys.argv))
