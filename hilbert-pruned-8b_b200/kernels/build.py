"""Builds the CUDA kernel library for sm_100a with nvcc and finds it again.

The library is built in-tree (``csrc/_build/libhilbert_b200.so``) the first time it is
needed and whenever a source changed since; a tree that cannot be written to falls back to
a per-user folder under the system's temporary directory (or ``HILBERT_B200_BUILD_DIR``).
Compilation prints a line per file to stderr so that a first call does not look hung.
There is no fallback when nvcc is missing: the error says so.
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
import time
from typing import List, Optional

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
LIB_NAME = "libhilbert_b200.so"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]


# HILBERT_B200_TIMELINE=1 builds a second library (own folder) whose kernels note the time at
# which each of them started and found its predecessors finished (kernels/ops.py:
# Ops.timeline_begin); =2 a third one that also records events inside the kernels that have
# some, which lengthens those kernels by a few microseconds.
TIMELINE = os.environ.get("HILBERT_B200_TIMELINE", "0")
TIMELINE = int(TIMELINE) if TIMELINE.isdigit() else 0
if TIMELINE:
    NVCC_FLAGS = NVCC_FLAGS + ["-DHB_TIMELINE"] + (["-DHB_TIMELINE_EVENTS"] if TIMELINE > 1 else [])


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[hilbert-b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("HILBERT_B200_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("the CUDA kernels are not built and nvcc was not found (set CUDA_HOME or HILBERT_B200_NVCC); "
                     "there is no CPU or library fallback")


def sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe_{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dirs() -> List[str]:
    dirs = []
    if os.environ.get("HILBERT_B200_BUILD_DIR"):
        dirs.append(os.environ["HILBERT_B200_BUILD_DIR"])
    tag = "_timeline" + (str(TIMELINE) if TIMELINE > 1 else "") if TIMELINE else ""
    dirs.append(os.path.join(CSRC, "_build" + tag))
    dirs.append(os.path.join(tempfile.gettempdir(), f"hilbert_b200_build{tag}_{os.getuid()}"))
    return dirs


def _is_current(d: str, digest: str) -> bool:
    try:
        with open(os.path.join(d, "stamp.json")) as f:
            return json.load(f).get("digest") == digest and os.path.isfile(os.path.join(d, LIB_NAME))
    except (OSError, ValueError):
        return False


def library_path(build_if_needed: bool = True, force: bool = False) -> str:
    """Path of an up-to-date library, building it first if it is missing or stale."""
    digest = _digest()
    if not force:
        for d in build_dirs():
            if _is_current(d, digest):
                return os.path.join(d, LIB_NAME)
    if not build_if_needed:
        raise BuildError("the CUDA kernel library is not built")
    for d in build_dirs():
        if _writable_dir(d):
            return _build(d, digest)
    raise BuildError("no writable folder to build the CUDA kernel library in")


def _compile_one(nvcc: str, src: str, obj: str) -> None:
    t0 = time.time()
    _say(f"compiling {src} for sm_100a ...")
    cmd = [nvcc] + NVCC_FLAGS + ["-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise BuildError(f"nvcc failed on {src}:\n{res.stdout}\n{res.stderr}")
    _say(f"compiled {src} in {time.time() - t0:.1f} s")


def _build(d: str, digest: str) -> str:
    nvcc = find_nvcc()
    srcs = sources()
    t0 = time.time()
    _say(f"building {LIB_NAME} from {len(srcs)} sources in {d}")
    objs = [os.path.join(d, s[:-3] + ".o") for s in srcs]
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        futs = [pool.submit(_compile_one, nvcc, s, o) for s, o in zip(srcs, objs)]
        for f in futs:
            f.result()
    tmp = os.path.join(d, f".{LIB_NAME}.{os.getpid()}")
    res = subprocess.run([nvcc, "-shared", "-o", tmp] + objs, capture_output=True, text=True)
    if res.returncode != 0:
        raise BuildError(f"linking {LIB_NAME} failed:\n{res.stdout}\n{res.stderr}")
    os.replace(tmp, os.path.join(d, LIB_NAME))
    with open(os.path.join(d, "stamp.json"), "w") as f:
        json.dump({"digest": digest, "flags": NVCC_FLAGS, "sources": srcs}, f)
    _say(f"built {LIB_NAME} in {time.time() - t0:.1f} s")
    return os.path.join(d, LIB_NAME)


def build_library(force: bool = False) -> str:
    return library_path(True, force)
