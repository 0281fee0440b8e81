"""Compile the CUDA sources of this folder into one shared library, in-tree.

The kernels are plain ``extern "C"`` entry points over raw pointers (no Python
or torch headers), so a build is a handful of ``nvcc`` calls of a few seconds
each, made at the first call that needs a kernel.  The library lands in
``csrc/_build/`` next to a digest of the sources; it is rebuilt when a source
changes.  If the package folder cannot be written, a per-user folder under the
system's temporary directory is used instead.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor

CSRC_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libqwen_engine_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC"]


def timeline_build() -> bool:
    """QE_TIMELINE=1 in the environment (looked at when the library is first needed) asks for the build
    whose kernels record when they start and when their predecessors end (common.cuh): a library of
    its own, in a folder of its own beside the plain one."""
    return os.environ.get("QE_TIMELINE") == "1"


def nvcc_flags() -> list[str]:
    return NVCC_FLAGS + (["-DQE_TIMELINE"] if timeline_build() else [])


def lib_name() -> str:
    return "libqwen_engine_b200_timeline.so" if timeline_build() else LIB_NAME


def build_folder() -> str:
    return "_build_timeline" if timeline_build() else "_build"


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[qwen_engine_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin/nvcc); "
                     "the CUDA kernels of qwen_engine_b200 cannot be built")


def sources() -> list[str]:
    return sorted(f for f in os.listdir(CSRC_DIR) if f.endswith(".cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for f in sorted(f for f in os.listdir(CSRC_DIR) if f.endswith((".cu", ".cuh", ".h"))):
        h.update(f.encode())
        with open(os.path.join(CSRC_DIR, f), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(ARCH_FLAGS + nvcc_flags()).encode())
    return h.hexdigest()


def _build_dir() -> str:
    in_tree = os.path.join(CSRC_DIR, build_folder())
    try:
        os.makedirs(in_tree, exist_ok=True)
        probe = os.path.join(in_tree, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return in_tree
    except OSError:
        alt = os.path.join(tempfile.gettempdir(), f"qwen_engine_b200{build_folder()}_{os.getuid()}")
        os.makedirs(alt, exist_ok=True)
        return alt


def library_path(build_if_needed: bool = True, verbose: bool = True) -> str:
    """Path of an up-to-date library, compiling it first if it is stale or absent."""
    bdir = _build_dir()
    lib = os.path.join(bdir, lib_name())
    stamp = os.path.join(bdir, "sources.sha256")
    digest = _digest()
    if os.path.isfile(lib) and os.path.isfile(stamp):
        with open(stamp) as f:
            if f.read().strip() == digest:
                return lib
    if not build_if_needed:
        raise BuildError(f"{lib} is absent or stale")
    import fcntl
    with open(os.path.join(bdir, ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if os.path.isfile(lib) and os.path.isfile(stamp):
            with open(stamp) as f:
                if f.read().strip() == digest:
                    return lib
        _compile(bdir, lib, verbose)
        with open(stamp, "w") as f:
            f.write(digest + "\n")
    return lib


def _compile(bdir: str, lib: str, verbose: bool) -> None:
    nvcc = find_nvcc()
    srcs = sources()
    t0 = time.time()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA sources for sm_100a into {bdir} (first call only)")

    def one(src: str) -> str:
        obj = os.path.join(bdir, src[:-3] + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *nvcc_flags(), "-I", CSRC_DIR, "-c", os.path.join(CSRC_DIR, src), "-o", obj]
        t1 = time.time()
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            _say(f"  {src} done in {time.time() - t1:.1f}s")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(one, srcs))
    tmp = lib + f".tmp{os.getpid()}"
    r = subprocess.run([nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *objs], capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"linking {lib} failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    if verbose:
        _say(f"built {os.path.basename(lib)} in {time.time() - t0:.1f}s")


if __name__ == "__main__":
    print(library_path())
