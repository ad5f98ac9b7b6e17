"""Builds the CUDA library for sm_100a with nvcc, in-tree, at the first call.

Each ``csrc/*.cu`` becomes an object file (compiled in parallel), then one shared library
``kernels/libturingserve_b200.so``.  A hash of the sources and flags sits beside it; the build
is skipped when it matches.  Where the package folder is not writable the build goes to a
per-user folder under the system temp directory.  Progress lines go to stderr so a caller that
waits on the first call sees that work is going on.
"""

from __future__ import annotations

import concurrent.futures
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time

PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(PKG, "csrc")
LIB_NAME = "libturingserve_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
              "-Xcompiler", "-fvisibility=hidden"]


def _say(msg: str) -> None:
    print(f"[turingserve_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if cand and os.path.exists(os.path.join(cand, "bin", "nvcc")):
            return os.path.join(cand, "bin", "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    raise RuntimeError("nvcc not found: the CUDA kernels cannot be built (set CUDA_HOME)")


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _source_hash() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(fh.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()


def _writable(folder: str) -> bool:
    try:
        os.makedirs(folder, exist_ok=True)
        probe = os.path.join(folder, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def _build_dirs() -> tuple[str, str]:
    """(folder of the library, folder of the object files)."""
    lib_dir = os.path.join(PKG, "kernels")
    obj_dir = os.path.join(CSRC, "_build")
    if _writable(lib_dir) and _writable(obj_dir):
        return lib_dir, obj_dir
    base = os.path.join(tempfile.gettempdir(), f"turingserve_b200-{os.getuid()}")
    os.makedirs(os.path.join(base, "obj"), exist_ok=True)
    return base, os.path.join(base, "obj")


def library_path() -> str:
    return os.path.join(_build_dirs()[0], LIB_NAME)


def _compile_one(nvcc: str, src: str, obj: str) -> tuple[str, float]:
    t0 = time.time()
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", CSRC, "-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {os.path.basename(src)}:\n{r.stdout}\n{r.stderr}")
    return src, time.time() - t0


def build(force: bool = False, verbose: bool = True) -> str:
    """Compile what is stale and return the path of the shared library."""
    lib_dir, obj_dir = _build_dirs()
    lib = os.path.join(lib_dir, LIB_NAME)
    stamp = lib + ".hash"
    want = _source_hash()

    def fresh() -> bool:
        if force or not os.path.exists(lib) or not os.path.exists(stamp):
            return False
        with open(stamp) as f:
            return f.read().strip() == want

    if fresh():
        return lib
    with open(os.path.join(lib_dir, ".build.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if fresh():
            return lib
        nvcc = find_nvcc()
        srcs = sources()
        if verbose:
            _say(f"building {LIB_NAME} for sm_100a: {len(srcs)} files with {nvcc}")
        objs = [os.path.join(obj_dir, os.path.basename(s)[:-3] + ".o") for s in srcs]
        t0 = time.time()
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
            futs = [pool.submit(_compile_one, nvcc, s, o) for s, o in zip(srcs, objs)]
            pending = set(futs)
            done_n = 0
            while pending:
                done, pending = concurrent.futures.wait(pending, timeout=10.0)
                for f in done:
                    src, dt = f.result()
                    done_n += 1
                    if verbose:
                        _say(f"  compiled {os.path.basename(src)} ({done_n}/{len(srcs)}, {dt:.0f} s)")
                if pending and not done and verbose:
                    _say(f"  still compiling, {len(pending)} files to go ({time.time() - t0:.0f} s)")
        tmp = lib + f".tmp{os.getpid()}"
        r = subprocess.run([nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *objs, "-lcudart"],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, lib)
        with open(stamp, "w") as f:
            f.write(want)
        if verbose:
            _say(f"built {lib} in {time.time() - t0:.0f} s")
    return lib
