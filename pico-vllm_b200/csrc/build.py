"""Builds the CUDA kernels of this folder into one shared library, in-tree.

``library_path()`` returns ``csrc/_build/libpico_kernels.so``, compiling it first when it is
missing or older than its sources (a digest of every source file and of the compiler flags is
kept beside it).  Every ``.cu`` file is compiled by its own ``nvcc`` process for sm_100a only,
then linked; while that runs a line is printed every few seconds.  If the package folder cannot
be written, the build goes to a folder under the system's temporary directory.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time
from typing import List, Optional

from ..errors import KernelError

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libpico_kernels.so"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _sources() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _digest() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for f in sorted(os.listdir(HERE)):
        if f.endswith((".cu", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(HERE, f), "rb") as fh:
                h.update(fh.read())
    return h.hexdigest()


def find_nvcc() -> str:
    for env in ("CUDA_HOME", "CUDA_PATH"):
        root = os.environ.get(env)
        if root and os.path.isfile(os.path.join(root, "bin", "nvcc")):
            return os.path.join(root, "bin", "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    if os.path.isfile("/usr/local/cuda/bin/nvcc"):
        return "/usr/local/cuda/bin/nvcc"
    raise KernelError("the CUDA kernels are not built and no nvcc was found (set CUDA_HOME)")


def _build_dir() -> str:
    d = os.path.join(HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"pico_vllm_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _say(msg: str) -> None:
    print(f"[pico-vllm_b200] {msg}", file=sys.stderr, flush=True)


def library_path(build_if_needed: bool = True, verbose: bool = True) -> str:
    """Path of the built library; builds it when needed."""
    digest = _digest()
    for d in (os.path.join(HERE, "_build"),
              os.path.join(tempfile.gettempdir(), f"pico_vllm_b200_build_{os.getuid()}")):
        lib, stamp = os.path.join(d, LIB_NAME), os.path.join(d, "stamp.json")
        if os.path.isfile(lib) and os.path.isfile(stamp):
            try:
                with open(stamp) as f:
                    if json.load(f).get("digest") == digest:
                        return lib
            except (OSError, ValueError):
                pass
    if not build_if_needed:
        raise KernelError("the CUDA kernels are not built (call pico_vllm_b200.csrc.build())")
    return build(verbose=verbose)


def build(verbose: bool = True, jobs: Optional[int] = None) -> str:
    """Compiles every .cu of this folder for sm_100a and links the library."""
    nvcc = find_nvcc()
    d = _build_dir()
    srcs = _sources()
    t0 = time.time()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA source files for sm_100a into {d} (first use only)")
    jobs = jobs or max(1, min(len(srcs), os.cpu_count() or 1))
    pending = list(srcs)
    running = {}
    objs = []
    last = time.time()
    while pending or running:
        while pending and len(running) < jobs:
            src = pending.pop(0)
            obj = os.path.join(d, src[:-3] + ".o")
            objs.append(obj)
            cmd = [nvcc] + NVCC_FLAGS + ["-c", os.path.join(HERE, src), "-o", obj]
            running[src] = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        for src, proc in list(running.items()):
            rc = proc.poll()
            if rc is None:
                continue
            out = proc.stdout.read()
            del running[src]
            if rc != 0:
                for p in running.values():
                    p.kill()
                raise KernelError(f"nvcc failed on {src}:\n{out}")
        if running:
            time.sleep(0.2)
            if verbose and time.time() - last > 5.0:
                last = time.time()
                _say(f"  … still compiling ({', '.join(sorted(running))}), {time.time() - t0:.0f} s")
    lib = os.path.join(d, LIB_NAME)
    tmp = lib + f".tmp{os.getpid()}"
    link = subprocess.run([nvcc, "-shared", "-o", tmp] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"],
                          stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if link.returncode != 0:
        raise KernelError(f"linking {LIB_NAME} failed:\n{link.stdout}")
    os.replace(tmp, lib)
    with open(os.path.join(d, "stamp.json"), "w") as f:
        json.dump({"digest": _digest(), "sources": srcs}, f)
    if verbose:
        _say(f"built {lib} in {time.time() - t0:.0f} s")
    return lib
