"""Compiles the CUDA sources beside this file into one shared library for sm_100a,
and the host sources under `host/` (C++, no CUDA) into a second one.

`nvcc` is called directly, one object per source file in parallel, then one link;
no Python or torch header is included by the sources, so a full build takes well
under a minute.  The library is built in `_build/` beside the sources when that
folder can be written, else under the system's temporary folder.  A build is
skipped when the library is newer than every source.  Progress lines go to
stderr.
"""
from __future__ import annotations

import concurrent.futures
import fcntl
import glob
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libvelox_b200_kernels.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    sys.stderr.write("[velox_b200] %s\n" % msg)
    sys.stderr.flush()


def find_nvcc() -> str:
    for cand in (os.environ.get("VELOX_B200_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 shutil.which("nvcc")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $VELOX_B200_NVCC, $CUDA_HOME/bin, /usr/local/cuda/bin, PATH); "
                     "the kernels cannot be compiled")


def sources() -> List[str]:
    return sorted(glob.glob(os.path.join(HERE, "*.cu")))


def _headers() -> List[str]:
    return sorted(glob.glob(os.path.join(HERE, "*.cuh")) + glob.glob(os.path.join(HERE, "*.h")))


def build_dir() -> str:
    env = os.environ.get("VELOX_B200_BUILD_DIR")
    if env:
        os.makedirs(env, exist_ok=True)
        return env
    local = os.path.join(HERE, "_build")
    try:
        os.makedirs(local, exist_ok=True)
        probe = os.path.join(local, ".w%d" % os.getpid())
        with open(probe, "w"):
            pass
        os.remove(probe)
        return local
    except OSError:
        tag = hashlib.sha1(HERE.encode()).hexdigest()[:10]
        d = os.path.join(tempfile.gettempdir(), "velox_b200_build_%d_%s" % (os.getuid(), tag))
        os.makedirs(d, exist_ok=True)
        return d


def _stale(target: str, deps: List[str]) -> bool:
    if not os.path.isfile(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(nvcc: str, src: str, obj: str, extra: List[str]) -> str:
    cmd = [nvcc] + NVCC_FLAGS + extra + ["-I", HERE, "-c", src, "-o", obj]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise BuildError("nvcc failed on %s:\n%s\n%s" % (os.path.basename(src), " ".join(cmd), p.stdout))
    return p.stdout


def build(force: bool = False, verbose: bool = True, ptxas_info: bool = False) -> str:
    """Build the kernel library if it is out of date; returns its path."""
    out_dir = build_dir()
    lib = os.path.join(out_dir, LIB_NAME)
    srcs, hdrs = sources(), _headers()
    if not srcs:
        raise BuildError("no .cu sources in %s" % HERE)
    if not force and not _stale(lib, srcs + hdrs + [os.path.abspath(__file__)]):
        return lib
    with open(os.path.join(out_dir, ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not _stale(lib, srcs + hdrs + [os.path.abspath(__file__)]):
                return lib  # another process built it meanwhile
            nvcc = find_nvcc()
            extra = ["-Xptxas", "-v"] if ptxas_info else []
            todo = []
            for s in srcs:
                obj = os.path.join(out_dir, os.path.basename(s)[:-3] + ".o")
                if force or _stale(obj, [s] + hdrs + [os.path.abspath(__file__)]):
                    todo.append((s, obj))
            t0 = time.time()
            if verbose:
                _say("compiling %d CUDA source file(s) for sm_100a into %s" % (len(todo), out_dir))
            logs = []
            with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(todo)))) as ex:
                futs = {ex.submit(_compile, nvcc, s, o, extra): s for s, o in todo}
                pending = set(futs)
                while pending:
                    done, pending = concurrent.futures.wait(pending, timeout=10.0)
                    for f in done:
                        logs.append(f.result())
                        if verbose:
                            _say("  compiled %s (%.0f s)" % (os.path.basename(futs[f]), time.time() - t0))
                    if pending and verbose and not done:
                        _say("  still compiling: %s (%.0f s)" % (
                            ", ".join(sorted(os.path.basename(futs[f]) for f in pending)), time.time() - t0))
            objs = [os.path.join(out_dir, os.path.basename(s)[:-3] + ".o") for s in srcs]
            tmp = lib + ".tmp%d" % os.getpid()
            cmd = [nvcc, "-shared", "-o", tmp] + objs
            p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            if p.returncode != 0:
                raise BuildError("link failed:\n%s\n%s" % (" ".join(cmd), p.stdout))
            os.replace(tmp, lib)
            if verbose:
                _say("built %s in %.0f s" % (lib, time.time() - t0))
            if ptxas_info:
                sys.stderr.write("\n".join(logs))
            return lib
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


HOST_LIB_NAME = "libvelox_b200_host.so"
HOST_DIR = os.path.join(HERE, "host")


def find_cxx() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if cand and (os.path.isfile(cand) or shutil.which(cand)):
            return cand
    raise BuildError("no C++ compiler found (looked at $CXX, g++, c++, clang++); the host library cannot be compiled")


def build_host(force: bool = False, verbose: bool = True) -> str:
    """Build the host library (scheduler, cache books, step builders) if it is out
    of date; returns its path.  Needs a C++17 compiler and nothing else."""
    out_dir = build_dir()
    lib = os.path.join(out_dir, HOST_LIB_NAME)
    srcs = sorted(glob.glob(os.path.join(HOST_DIR, "*.cpp")))
    deps = srcs + sorted(glob.glob(os.path.join(HOST_DIR, "*.hpp"))) + [os.path.abspath(__file__)]
    if not srcs:
        raise BuildError("no .cpp sources in %s" % HOST_DIR)
    if not force and not _stale(lib, deps):
        return lib
    with open(os.path.join(out_dir, ".lock_host"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not _stale(lib, deps):
                return lib
            t0 = time.time()
            if verbose:
                _say("compiling the host library into %s" % out_dir)
            tmp = lib + ".tmp%d" % os.getpid()
            cmd = [find_cxx(), "-O2", "-std=c++17", "-Wall", "-shared", "-fPIC", "-I", HOST_DIR] + srcs + ["-o", tmp]
            p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            if p.returncode != 0:
                raise BuildError("the host library failed to compile:\n%s\n%s" % (" ".join(cmd), p.stdout))
            os.replace(tmp, lib)
            if verbose:
                _say("built %s in %.0f s" % (lib, time.time() - t0))
            return lib
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


if __name__ == "__main__":
    build(force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    build_host(force="--force" in sys.argv)
