"""Compiles the CUDA sources of this folder for sm_100a into one shared library, in the tree.

The library is built at first use (or by `python -m ember_cpp_b200.csrc.build`) with nvcc alone:
the kernels are plain CUDA with C entry points, so no Python or torch headers are compiled and a
cold build takes well under a minute.  It is rebuilt when a source or a flag changes.  Progress
goes to stderr, a line per file.  If the tree is read-only the library goes to a per-user folder
under the system's temporary directory instead.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libember_kernels.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH_FLAGS + ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
# EMBER_TIMELINE=1: the kernels of a decode step note when their blocks start, pass their wait for
# the kernel in front and end (`CudaOps.timeline`).  That library is built beside the ordinary one.
TIMELINE = os.environ.get("EMBER_TIMELINE", "0") == "1"
if TIMELINE:
    NVCC_FLAGS = NVCC_FLAGS + ["-DEMBER_TIMELINE"]


class BuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[ember.cpp_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("EMBER_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (PATH, CUDA_HOME, /usr/local/cuda): the CUDA kernels cannot be built, and "
                     "this library has no other way to run a model")


def sources() -> list[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for name in sorted(f for f in os.listdir(HERE) if f.endswith((".cu", ".cuh", ".h"))):
        h.update(name.encode())
        with open(os.path.join(HERE, name), "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dir() -> str:
    d = os.path.join(HERE, "_build_timeline" if TIMELINE else "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"ember_cpp_b200_build{'_timeline' if TIMELINE else ''}_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path(build_if_needed: bool = True) -> str:
    """Path of the built library; builds it first if it is missing or stale."""
    d = _build_dir()
    lib, stamp = os.path.join(d, LIB_NAME), os.path.join(d, "stamp.txt")
    want = _digest()
    if os.path.isfile(lib) and os.path.isfile(stamp):
        with open(stamp) as f:
            if f.read().strip() == want:
                return lib
    if not build_if_needed:
        raise BuildError(f"{lib} is missing or older than its sources")
    return build(d)


def _compile(nvcc: str, src: str, obj: str, verbose: bool) -> float:
    t0 = time.time()
    cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(HERE, src), "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    if verbose and r.stderr:
        sys.stderr.write(r.stderr)
    return time.time() - t0


def build(build_dir: str | None = None, verbose: bool = False) -> str:
    nvcc = find_nvcc()
    d = build_dir or _build_dir()
    srcs = sources()
    _log(f"building {len(srcs)} CUDA sources for sm_100a with {nvcc} into {d} (first use; about half a minute)")
    t0 = time.time()
    objs = []
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        futures = {}
        for src in srcs:
            obj = os.path.join(d, src[:-3] + ".o")
            objs.append(obj)
            futures[pool.submit(_compile, nvcc, src, obj, verbose)] = src
        for fut in concurrent.futures.as_completed(futures):
            _log(f"  compiled {futures[fut]} in {fut.result():.1f} s")
    lib = os.path.join(d, LIB_NAME)
    tmp = lib + f".tmp{os.getpid()}"
    link = [nvcc, *ARCH_FLAGS, "-shared", "-cudart", "shared", "-o", tmp, *objs, "-lcublasLt",
            "-Xlinker", "-rpath=/usr/local/cuda/lib64"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    with open(os.path.join(d, "stamp.txt"), "w") as f:
        f.write(_digest())
    _log(f"built {LIB_NAME} in {time.time() - t0:.1f} s")
    return lib


if __name__ == "__main__":
    print(library_path())
